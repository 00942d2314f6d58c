"""Small Difavik configurations for the tests.  The sizes are awkward on purpose: widths that are
no power of two, head sizes that are no multiple of 16 (or of 8), windows shorter and longer than
a page, no kept tokens and many, as many key heads as query heads and a single one, rotated
dimensions fewer than the head, every expert chosen and one of many, layers that borrow another
layer's tensors, a layer without a feed-forward, a model without the pair table."""

import vekasun_configs as VC

write_folder = VC.write_folder
read_folder = VC.read_folder


def lightning(heads, dim, vdim, decay):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay}


def parallel(left, right):
    return {"left": left, "right": right}


def attention(heads, kv_heads, dim, scale, size, keep_first):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale,
            "mask": {"size": size, "keep_first": keep_first}}


def retention(heads, dim, vdim, decay, base, dims):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay, "rot": {"base": base, "dims": dims}}


def dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(ff, limit, experts, top):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}


# parallel first, a borrowed lightning layer, a window of 21 over pages of 16, three kept tokens
BORROWING = {
    "architecture": "Difavik", "vocab": 211, "width": 96, "norm": {"eps": 1e-5},
    "embedding": {"bigram": {"buckets": 89, "mul_prev": 31, "mul_cur": 5}},
    "layers": [
        {"type": "parallel", "mixer": parallel(attention(6, 2, 16, 0.3, 21, 3), retention(3, 16, 24, [0.9, 0.97, 0.995], 500.0, 8)),
         "mlp": moe(40, 1.5, 5, 2)},
        {"type": "lightning", "mixer": lightning(2, 24, 16, [0.7, 0.95]), "mlp": dense(72, 2.5)},
        {"type": "lightning", "mixer": lightning(2, 24, 16, [0.7, 0.95]), "mlp": dense(72, 2.5), "weights_of": 1},
        {"type": "parallel", "mixer": parallel(attention(6, 2, 16, 0.3, 21, 3), retention(3, 16, 24, [0.9, 0.97, 0.995], 500.0, 8)),
         "mlp": moe(40, 1.5, 5, 2), "weights_of": 0},
    ],
}

# no pair table; one key head; nothing kept; the window longer than most requests; every expert chosen;
# the whole head rotated; a layer without a feed-forward
PLAIN = {
    "architecture": "Difavik", "vocab": 157, "width": 80, "norm": {"eps": 3e-6},
    "layers": [
        {"type": "lightning", "mixer": lightning(5, 8, 16, [0.5, 0.8, 0.9, 0.99, 0.999]), "mlp": moe(24, 0.75, 3, 3)},
        {"type": "parallel", "mixer": parallel(attention(4, 1, 32, 0.18, 100, 0), retention(2, 32, 40, [0.98, 0.9], 10000.0, 32)),
         "mlp": None},
        {"type": "parallel", "mixer": parallel(attention(2, 2, 16, 0.25, 5, 9), retention(4, 8, 8, [0.6, 0.7, 0.8, 0.9], 77.0, 4)),
         "mlp": dense(56, 1.0)},
    ],
}

# nothing a multiple of 8 where it can be helped: head sizes 12 and 20, width 100, a window of one token
AWKWARD = {
    "architecture": "Difavik", "vocab": 97, "width": 100, "norm": {"eps": 2e-5},
    "embedding": {"bigram": {"buckets": 1, "mul_prev": 1, "mul_cur": 0}},
    "layers": [
        {"type": "parallel", "mixer": parallel(attention(3, 3, 12, 0.4, 1, 2), retention(5, 20, 12, [0.99, 0.9, 0.8, 0.95, 0.5], 300.0, 6)),
         "mlp": moe(20, 3.0, 7, 1)},
        {"type": "lightning", "mixer": lightning(1, 36, 28, [0.93]), "mlp": moe(36, 1.25, 2, 1)},
    ],
}

CONFIGS = {"borrowing": (BORROWING, 31), "plain": (PLAIN, 32), "awkward": (AWKWARD, 33)}

# factors that take the random weights (standard deviation 0.02) out of their nearly linear range
# (a router much livelier than this turns the 8-bit rounding of its input into several per cent of a score,
# which is the design's sensitivity and not the engine's)
LIVELY = {".q": 6.0, ".k": 6.0, ".v": 4.0, ".g": 12.0, ".router": 8.0, ".gate": 6.0, ".up": 6.0, ".q.b": 20.0,
          ".k.b": 20.0, ".gate.b": 20.0, ".up.b": 20.0, ".down.b": 10.0, "bigram": 3.0, ".norm1": 5.0, ".norm2": 5.0}
