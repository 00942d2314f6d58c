"""A plain, slow implementation of the Difavik design for whole sequences: the tests' oracle.

One request, all its tokens at once, no cache, no state carried, no batching: every mechanism is
one function of whole-sequence tensors, written from the design's equations and sharing no code
with the package under test.  config.json is read as a plain dictionary, the weights as a
dictionary of tensors by name.  Everything is evaluated in the dtype of the weights handed in
(the tests hand in float64 or float32).

Notation: T tokens, W width, rows are tokens; a linear weight is stored [out, in].
"""

from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


# (generator, relative size) or None: every projection's output is then disturbed by that much, as a
# rounding to few bits would.  The tests use it to find the rows whose logits hang on a rounding
# (a sum that nearly cancels in front of a norm that blows it up again): no arithmetic of 8 bits
# can be held to a per cent there.
NOISE = None


def lin(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor] = None) -> torch.Tensor:
    y = x @ w.T
    if b is not None:
        y = y + b
    if NOISE is not None:
        gen, size = NOISE
        y = y * (1.0 + size * torch.randn(y.shape, generator=gen, dtype=y.dtype))
    return y


def silu(x: torch.Tensor) -> torch.Tensor:
    return x * torch.sigmoid(x)


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x over its root mean square along the last axis, eps inside the root."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


# ---- embedding ------------------------------------------------------------------------------

def pair_rows(tokens: List[int], buckets: int, mul_prev: int, mul_cur: int) -> List[int]:
    """Row of the pair table for every token: a hash of (previous, current); the first token of a
    sequence has no previous one and takes the table's last row."""
    return [buckets if i == 0 else (tokens[i - 1] * mul_prev + t * mul_cur) % buckets
            for i, t in enumerate(tokens)]


def embed(tokens: List[int], w: Dict[str, torch.Tensor], cfg: dict) -> torch.Tensor:
    x = w["embed"][torch.tensor(tokens)]
    bg = (cfg.get("embedding") or {}).get("bigram")
    if bg:
        rows = pair_rows(tokens, int(bg["buckets"]), int(bg["mul_prev"]), int(bg["mul_cur"]))
        x = x + w["bigram"][torch.tensor(rows)]
    return x


# ---- rotation -------------------------------------------------------------------------------

def rotate_half_split(v: torch.Tensor, base: float, dims: int) -> torch.Tensor:
    """v [T, heads, D]: the first `dims` of the last axis are turned, pair (i, i + dims/2) by the
    angle p * base^(-2i/dims), p the row's position from 0; the rest pass."""
    T = v.shape[0]
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=v.dtype)
    ang = torch.arange(T, dtype=v.dtype)[:, None] * f[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = v[..., :half], v[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, v[..., dims:]], dim=-1)


# ---- softmax attention whose values are its keys --------------------------------------------

def visible(T: int, window: int, keep_first: int) -> torch.Tensor:
    """[T, T] bool: row i sees column j iff j <= i and (i - j < window or j < keep_first)."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    return (j <= i) & ((i - j < window) | (j < keep_first))


def distance_slopes(H: int, dtype) -> torch.Tensor:
    return torch.tensor([2.0 ** (-8.0 * (h + 1) / H) for h in range(H)], dtype=dtype)


def tied_value_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, G, D = int(m["heads"]), int(m["kv_heads"]), int(m["dim"])
    q = lin(h, w[p + "q"], w[p + "q.b"])
    k = lin(h, w[p + "k"], w[p + "k.b"])
    v = k.reshape(T, G, D)                                   # the values are the keys as projected
    qn = (rms_unit(q, eps) * w[p + "q.norm"]).reshape(T, H, D)        # one norm over all heads' rows
    kn = (rms_unit(k, eps) * w[p + "k.norm"]).reshape(T, G, D)
    rep = H // G
    kh = kn.repeat_interleave(rep, dim=1)
    vh = v.repeat_interleave(rep, dim=1)
    s = torch.einsum("ihd,jhd->hij", qn, kh) * float(m["scale"])
    dist = (torch.arange(T)[:, None] - torch.arange(T)[None, :]).to(h.dtype)
    s = s - distance_slopes(H, h.dtype)[:, None, None] * dist[None]
    see = visible(T, int(m["mask"]["size"]), int(m["mask"]["keep_first"]))
    s = s.masked_fill(~see[None], float("-inf"))
    a = torch.softmax(s, dim=-1)
    o = torch.einsum("hij,jhd->ihd", a, vh)
    gate = torch.sigmoid(lin(h, w[p + "g"]))                 # [T, H]: one number a head
    o = o * gate[:, :, None]
    return lin(o.reshape(T, H * D), w[p + "o"])


# ---- linear attention with a fixed decay a head ---------------------------------------------

def decay_recurrence(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: List[float]) -> torch.Tensor:
    """q, k [T, H, D], v [T, H, V]: S_t = decay_h S_{t-1} + k_t v_t^T (S starts at zero), o_t = S_t^T q_t."""
    T, H, D = q.shape
    V = v.shape[-1]
    S = torch.zeros((H, D, V), dtype=q.dtype)
    g = torch.tensor(decay, dtype=q.dtype)[:, None, None]
    out = []
    for t in range(T):
        S = g * S + k[t][:, :, None] * v[t][:, None, :]
        out.append(torch.einsum("hdv,hd->hv", S, q[t]))
    return torch.stack(out)                                   # [T, H, V]


def retention(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, D, V = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    base, dims = float(m["rot"]["base"]), int(m["rot"]["dims"])
    q = lin(h, w[p + "q"]).reshape(T, H, D)
    k = lin(h, w[p + "k"]).reshape(T, H, D)
    v = lin(h, w[p + "v"]).reshape(T, H, V)
    if dims:
        q, k = rotate_half_split(q, base, dims), rotate_half_split(k, base, dims)
    k = k * D ** -0.5
    o = rms_unit(decay_recurrence(q, k, v, [float(d) for d in m["decay"]]), eps)      # every head by itself
    o = o.reshape(T, H * V) * silu(lin(h, w[p + "g"]))
    return lin(o, w[p + "o"])


def lightning(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, D, V = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    q = silu(lin(h, w[p + "q"])).reshape(T, H, D)
    k = silu(lin(h, w[p + "k"])).reshape(T, H, D)
    v = silu(lin(h, w[p + "v"])).reshape(T, H, V)
    o = decay_recurrence(q, k, v, [float(d) for d in m["decay"]]).reshape(T, H * V)
    o = rms_unit(o, eps) * w[p + "norm"] * torch.sigmoid(lin(h, w[p + "g"]))          # all heads together
    return lin(o, w[p + "o"])


def parallel(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    a = tied_value_attention(h, w, p + "left.", m["left"], eps)
    b = retention(h, w, p + "right.", m["right"], eps)
    return 0.5 * (rms_unit(a, eps) * w[p + "left.out"] + rms_unit(b, eps) * w[p + "right.out"])


# ---- feed-forward ---------------------------------------------------------------------------

def capped_glu(g: torch.Tensor, u: torch.Tensor, limit: float) -> torch.Tensor:
    g = torch.clamp(g, max=limit)
    u = torch.clamp(u, min=-limit, max=limit)
    return g * torch.sigmoid(1.702 * g) * (u + 1.0)


def dense_ff(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, f: dict) -> torch.Tensor:
    y = capped_glu(lin(h, w[p + "gate"], w[p + "gate.b"]), lin(h, w[p + "up"], w[p + "up.b"]), float(f["limit"]))
    return lin(y, w[p + "down"], w[p + "down.b"])


def routed_ff(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, f: dict, chosen=None, record=None) -> torch.Tensor:
    """softmax over all experts, the `top` largest, their scores as weights (not renormalised).
    `chosen` [T, top] forces the selection (a test may hand in the engine's, for near-ties);
    `record` collects (scores, selection)."""
    E, top = int(f["router"]["experts"]), int(f["router"]["top"])
    limit = float(f["expert"]["limit"])
    s = torch.softmax(lin(h, w[p + "router"]), dim=-1)
    sel = torch.topk(s, top, dim=-1).indices if chosen is None else chosen
    if record is not None:
        record.append((s, sel))
    out = torch.zeros_like(h)
    for e in range(E):
        q = f"{p}e{e}."
        y = lin(capped_glu(lin(h, w[q + "gate"]), lin(h, w[q + "up"]), limit), w[q + "down"])
        weight = (s[:, e:e + 1] * (sel == e).any(dim=-1, keepdim=True).to(h.dtype))
        out = out + weight * y
    return out


# ---- the model ------------------------------------------------------------------------------

def weights_owner(layers: List[dict], i: int) -> int:
    while layers[i].get("weights_of") is not None:
        i = int(layers[i]["weights_of"])
    return i


def forward(tokens: List[int], w: Dict[str, torch.Tensor], cfg: dict, streams: Optional[list] = None,
            chosen: Optional[list] = None, record: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab].  `streams` collects the residual stream after every layer run."""
    eps = float(cfg["norm"]["eps"])
    x = embed(tokens, w, cfg)
    routed_seen = 0
    for i, L in enumerate(cfg["layers"]):
        p = f"l{weights_owner(cfg['layers'], i)}."
        mix = {"parallel": parallel, "lightning": lightning}[L["type"]](x, w, p + "mix.", L["mixer"], eps)
        x = x + rms_unit(mix, eps) * (1.0 + w[p + "norm1"]) * w[p + "ls1"]
        f = L.get("mlp")
        if f is not None:
            if f["kind"] == "dense":
                y = dense_ff(x, w, p + "mlp.", f)
            else:
                y = routed_ff(x, w, p + "mlp.", f, None if chosen is None else chosen[routed_seen], record)
                routed_seen += 1
            x = x + rms_unit(y, eps) * (1.0 + w[p + "norm2"]) * w[p + "ls2"]
        if streams is not None:
            streams.append(x.clone())
    x = rms_unit(x, eps) * (1.0 + w["final.norm"])
    return lin(x, w["embed"])
