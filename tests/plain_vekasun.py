"""A plain, slow implementation of the Vekasun design for whole sequences: the tests' oracle.

One request, all its tokens at once, no cache, no state carried, no batching: every mechanism
is one function of whole-sequence tensors, written from the design's equations and sharing no
code with the package under test.  config.json is read as a plain dictionary, the weights as a
dictionary of tensors by name.  Everything is evaluated in the dtype of the weights handed in
(the tests hand in float64 or float32).

Notation: T tokens, W width, rows are tokens.  A linear weight is stored [out, in]; ``lin``
applies it to rows.
"""

from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def lin(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    return x @ w.T


def silu(x: torch.Tensor) -> torch.Tensor:
    return x * torch.sigmoid(x)


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x over its root mean square along the last axis, eps inside the root."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def layer_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """(x - mean) / sqrt(var + eps) * w, var the mean squared deviation; no bias."""
    mu = x.mean(dim=-1, keepdim=True)
    d = x - mu
    return d / torch.sqrt((d * d).mean(dim=-1, keepdim=True) + eps) * w


# ---- rotation -------------------------------------------------------------------------------

def rotate_half_split(v: torch.Tensor, base: float, dims: int, first_position: int = 0) -> torch.Tensor:
    """v [T, ..., D]: the first `dims` of the last axis are turned, pair (i, i + dims/2) by the
    angle p * base^(-2i/dims), p the row's position; the rest pass."""
    T = v.shape[0]
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=v.dtype)
    p = torch.arange(first_position, first_position + T, dtype=v.dtype)
    ang = p[:, None] * f[None, :]
    shape = [T] + [1] * (v.dim() - 2) + [half]
    c, s = torch.cos(ang).reshape(shape), torch.sin(ang).reshape(shape)
    a, b = v[..., :half], v[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, v[..., dims:]], dim=-1)


# ---- latent attention -----------------------------------------------------------------------

def sink_softmax(scores: torch.Tensor, sink: torch.Tensor) -> torch.Tensor:
    """scores [H, T, T] already masked with -inf; the denominator holds exp(sink_h) once more."""
    m = torch.maximum(scores.max(dim=-1, keepdim=True).values, sink[:, None, None])
    e = torch.exp(scores - m)
    return e / (e.sum(dim=-1, keepdim=True) + torch.exp(sink[:, None, None] - m))


def latent_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, dn, dr, dv, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    base, dims = float(m["rot"]["base"]), int(m["rot"]["dims"])
    cq = rms_unit(lin(h, w[p + "dq"]), eps) * w[p + "dq.norm"]
    q = lin(cq, w[p + "uq"]).reshape(T, H, dn + dr)
    q_plain, q_rot = q[..., :dn], rotate_half_split(q[..., dn:], base, dims)
    kv = lin(h, w[p + "dkv"])
    c = rms_unit(kv[:, :r], eps) * w[p + "dkv.norm"]
    k_rot = rotate_half_split(kv[:, r:], base, dims)                       # [T, dr], one for all heads
    k_plain = lin(c, w[p + "uk"]).reshape(T, H, dn)
    v = lin(c, w[p + "uv"]).reshape(T, H, dv)
    s = torch.einsum("ihd,jhd->hij", q_plain, k_plain) + torch.einsum("ihd,jd->hij", q_rot, k_rot)
    s = s * float(m["scale"])
    seen = torch.arange(T)[None, :] <= torch.arange(T)[:, None]
    s = s.masked_fill(~seen[None], float("-inf"))
    a = sink_softmax(s, w[p + "sink"].to(h.dtype))
    o = torch.einsum("hij,jhd->ihd", a, v).reshape(T, H * dv)
    o = o * torch.sigmoid(lin(h, w[p + "g"]))
    return lin(o, w[p + "o"])


# ---- mamba2 ---------------------------------------------------------------------------------

def causal_conv(u: torch.Tensor, taps: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """u [T, C], taps [C, K] (last column is the current token's), zeros before the start."""
    T, C = u.shape
    K = taps.shape[1]
    pad = torch.cat([torch.zeros(K - 1, C, dtype=u.dtype), u], dim=0)
    out = bias[None, :].expand(T, C).clone()
    for j in range(K):
        out = out + pad[j:j + T] * taps[:, j][None, :]
    return out


def ssd_recurrence(x, B, C, dt, A_log, D, heads_per_group):
    """x [T, Hh, P], B and C [T, G, N], dt [T, Hh] (already positive).  Token by token:
    S <- exp(-exp(A_log) dt) S + dt B x^T;  y = S^T C + D x."""
    T, Hh, P = x.shape
    N = B.shape[-1]
    S = torch.zeros(Hh, N, P, dtype=x.dtype)
    y = torch.empty_like(x)
    g = torch.arange(Hh) // heads_per_group
    rate = torch.exp(A_log)
    for t in range(T):
        decay = torch.exp(-rate * dt[t])
        S = decay[:, None, None] * S + dt[t][:, None, None] * B[t][g][:, :, None] * x[t][:, None, :]
        y[t] = torch.einsum("hnp,hn->hp", S, C[t][g]) + D[:, None] * x[t]
    return y


def mamba2(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    Hh, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = Hh * P
    proj = lin(h, w[p + "in"])
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, w[p + "conv"], w[p + "conv.b"]))
    x = xbc[:, :inner].reshape(T, Hh, P)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = torch.nn.functional.softplus(dt + w[p + "dt_bias"], threshold=1e9)
    y = ssd_recurrence(x, B, C, dt, w[p + "A_log"], w[p + "D"], Hh // G).reshape(T, inner)
    y = y * silu(z)
    parts = int(m["norm_groups"])
    y = rms_unit(y.reshape(T, parts, inner // parts), eps).reshape(T, inner) * w[p + "norm"]
    return lin(y, w[p + "o"])


# ---- feed-forward ---------------------------------------------------------------------------

def route_sigmoid_top(h: torch.Tensor, w_router: torch.Tensor, top: int):
    """Scores sigmoid(W_r h); the `top` largest; their scores are the weights as they are."""
    s = torch.sigmoid(lin(h, w_router))
    wts, idx = torch.topk(s, top, dim=-1)
    return idx, wts


def moe_scaled_input(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict,
                     forced: Optional[torch.Tensor] = None) -> torch.Tensor:
    """sum over chosen experts e of expert_e(s_e h): the weight multiplies the expert's input."""
    E, top = int(m["router"]["experts"]), int(m["router"]["top"])
    idx, wts = route_sigmoid_top(h, w[p + "router"], top)
    if forced is not None:
        idx = forced
        wts = torch.gather(torch.sigmoid(lin(h, w[p + "router"])), 1, idx)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(top):
            e = int(idx[t, j])
            u = wts[t, j] * h[t]
            a = silu(w[f"{p}e{e}.gate"] @ u) * (w[f"{p}e{e}.up"] @ u)
            out[t] = out[t] + w[f"{p}e{e}.down"] @ a
    return out


# ---- the model ------------------------------------------------------------------------------

MIXERS = {"latent_attention": latent_attention, "mamba2": mamba2}


def layer_runs(cfg: dict) -> List[tuple]:
    """(layer, pass) in the order they run: layers start..stop-1 `times` times in a row."""
    n = len(cfg["layers"])
    loop = cfg.get("loop") or {"start": 0, "stop": 0, "times": 1}
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    runs = [(i, None) for i in range(a)]
    for t in range(times):
        runs += [(i, t) for i in range(a, b)]
    return runs + [(i, None) for i in range(b, n)]


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens, residuals: Optional[list] = None,
            forced: Optional[Dict[int, torch.Tensor]] = None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence; `residuals` collects x after every layer run;
    `forced` maps the number of a layer run to the experts [T, top] its feed-forward is to use
    instead of its own choice (their weights are still this model's own scores)."""
    eps = float(cfg["norm"]["eps"])
    x = w["embed"][torch.as_tensor(list(tokens), dtype=torch.long)]
    loop = cfg.get("loop")
    for run, (i, t) in enumerate(layer_runs(cfg)):
        if t is not None and i == int(loop["start"]):
            x = x + w["loop.step"][t][None, :]
        L, p = cfg["layers"][i], f"l{i}."
        x = x + MIXERS[L["type"]](layer_norm(x, w[p + "norm1"], eps), w, p + "mix.", L["mixer"], eps)
        if L.get("mlp") is not None:
            x = x + moe_scaled_input(layer_norm(x, w[p + "norm2"], eps), w, p + "mlp.", L["mlp"],
                                     None if forced is None else forced.get(run))
        if residuals is not None:
            residuals.append(x.clone())
    return lin(layer_norm(x, w["final.norm"], eps), w["head"]) * float(cfg["logit_scale"])
