from . import qwen2_moe, vekasun  # noqa: F401  (registration)
