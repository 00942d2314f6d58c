"""Small Vekasun configurations for the tests, and a writer of model folders whose tensors a
test may replace.  The sizes are awkward on purpose: widths that are no power of two, a state
size that is no multiple of 16, rotated dimensions fewer than the rotated slice, one norm part
and several, as many groups as heads and a single one, every expert chosen, no feed-forward."""

import json
import os

import torch


def attention(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, base, dims):
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
            "scale": scale, "rot": {"base": base, "dims": dims}}


def state_space(heads, vdim, state, groups, conv, norm_groups):
    return {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}


def moe(ff, experts, top):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


# a loop over the two middle layers, three passes; a layer without a feed-forward; two of six and
# all of three experts
LOOPED = {
    "architecture": "Vekasun", "vocab": 301, "width": 192, "norm": {"eps": 1e-5}, "logit_scale": 0.5,
    "loop": {"start": 1, "stop": 3, "times": 3},
    "layers": [
        {"type": "mamba2", "mixer": state_space(6, 20, 24, 3, 3, 1), "mlp": moe(72, 6, 2)},
        {"type": "latent_attention", "mixer": attention(3, 24, 16, 40, 40, 56, 0.2, 5000.0, 8), "mlp": None},
        {"type": "mamba2", "mixer": state_space(4, 32, 16, 1, 5, 4), "mlp": moe(40, 3, 3)},
        {"type": "latent_attention", "mixer": attention(5, 16, 8, 24, 48, 64, 0.3, 300.0, 8), "mlp": moe(56, 4, 1)},
    ],
}

# no loop at all, attention first, conv of two taps, groups == heads
STRAIGHT = {
    "architecture": "Vekasun", "vocab": 257, "width": 136, "norm": {"eps": 3e-6}, "logit_scale": 1.5,
    "layers": [
        {"type": "latent_attention", "mixer": attention(2, 40, 24, 16, 72, 48, 0.15, 12345.0, 24), "mlp": moe(88, 5, 2)},
        {"type": "mamba2", "mixer": state_space(5, 24, 40, 5, 2, 5), "mlp": None},
        {"type": "latent_attention", "mixer": attention(4, 8, 8, 8, 16, 24, 0.5, 50.0, 4), "mlp": moe(32, 2, 2)},
    ],
}

# the whole model is the loop, one pass (so the pass vector is added once), conv of one tap
ONE_PASS = {
    "architecture": "Vekasun", "vocab": 199, "width": 96, "norm": {"eps": 1e-4}, "logit_scale": 1.0,
    "loop": {"start": 0, "stop": 2, "times": 1},
    "layers": [
        {"type": "mamba2", "mixer": state_space(3, 16, 8, 1, 1, 3), "mlp": moe(24, 7, 3)},
        {"type": "latent_attention", "mixer": attention(1, 32, 16, 48, 24, 32, 0.25, 777.0, 16), "mlp": moe(48, 3, 1)},
    ],
}

# nothing a multiple of 8: the 16-byte-row kernels must step aside for the general ones
AWKWARD = {
    "architecture": "Vekasun", "vocab": 97, "width": 100, "norm": {"eps": 2e-5}, "logit_scale": 3.0,
    "loop": {"start": 1, "stop": 2, "times": 2},
    "layers": [
        {"type": "latent_attention", "mixer": attention(2, 12, 6, 10, 20, 28, 0.3, 100.0, 6), "mlp": moe(36, 3, 2)},
        {"type": "mamba2", "mixer": state_space(3, 10, 12, 3, 4, 3), "mlp": moe(20, 5, 1)},
    ],
}

CONFIGS = {"looped": (LOOPED, 21), "straight": (STRAIGHT, 22), "one_pass": (ONE_PASS, 23), "awkward": (AWKWARD, 24)}


def write_folder(config, seed, out_dir, replace=None, scale=None):
    """A model folder with the engine's seeded random tensors; `replace` maps tensor names to
    tensors that take the place of the random ones, `scale` maps name suffixes to factors
    (random weights of standard deviation 0.02 make every mechanism nearly linear; scaled up,
    softmax, gates and decays leave their linear range)."""
    from safetensors import safe_open
    from safetensors.torch import save_file
    from ninfer_amd_mi50_b200.weights import write_random_model
    write_random_model(config, seed, out_dir)
    path = os.path.join(out_dir, "model.safetensors")
    tensors = {}
    with safe_open(path, framework="pt") as f:
        for n in f.keys():
            tensors[n] = f.get_tensor(n)
    for n in list(tensors):
        for suffix, factor in (scale or {}).items():
            if n.endswith(suffix):
                tensors[n] = (tensors[n].float() * factor).to(torch.bfloat16)
    for n, t in (replace or {}).items():
        assert n in tensors and tuple(tensors[n].shape) == tuple(t.shape), n
        tensors[n] = t.to(torch.bfloat16).contiguous()
    save_file(tensors, path)
    return out_dir


# factors that take the random weights out of their nearly linear range
LIVELY = {".mix.uq": 6.0, ".mix.uk": 6.0, ".mix.dkv": 3.0, ".mix.in": 4.0, ".router": 20.0, ".mix.g": 10.0,
          ".mix.conv": 10.0, "loop.step": 20.0}


def read_folder(model_dir, dtype=torch.float64):
    from safetensors import safe_open
    with open(os.path.join(model_dir, "config.json")) as fh:
        cfg = json.load(fh)
    w = {}
    with safe_open(os.path.join(model_dir, "model.safetensors"), framework="pt") as f:
        for n in f.keys():
            w[n] = f.get_tensor(n).to(dtype)
    return cfg, w
