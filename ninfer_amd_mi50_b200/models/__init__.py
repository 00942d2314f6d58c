from . import qwen2_moe, vekasun, difavik  # noqa: F401  (registration)
