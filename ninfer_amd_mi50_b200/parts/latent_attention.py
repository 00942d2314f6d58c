"""Attention through a latent: queries, keys and values are projected down to a narrow latent
first, and only the keys' and values' common latent is cached.

With H heads, per head ``dim`` unrotated and ``rot_dim`` rotated query/key dimensions, value size
``vdim`` and latent width ``kv_rank``:

    c_q = rms(W_dq h) * w_qn          q = W_uq c_q, head by head [dim | rot_dim]
    [c_raw | k_rot_raw] = W_dkv h     c = rms(c_raw) * w_kvn,  k_rot = rotate(k_rot_raw)   (one for all heads)
    k_h = W_uk[h] c,  v_h = W_uv[h] c
    s = (q_plain_h . k_h + rotate(q_rot_h) . k_rot) * scale      over positions j <= i
    p = softmax with exp(sink_h) added to the denominator (a learned number per head)
    out = W_o ( concat_h(sum_j p_j v_h,j) * sigmoid(W_g h) )

The cache keeps one row ``[c | k_rot]`` per token (`CacheSpec` with `row_width`).  The kernels
never materialise k_h or v_h: the key projection is folded into the query
(``q_abs_h = W_uk[h]^T q_plain_h``, so ``q_plain_h . k_h = q_abs_h . c``) and the value projection
is applied after the weighted sum (``sum_j p_j v_h,j = W_uv[h] sum_j p_j c_j``), which is the same
arithmetic regrouped.  Prompts, portions and decoded tokens all run this one form.
Norms, rotation angles, scores and softmax are 32-bit in both modes.

The three projections that read the layer's input (W_dq, W_dkv, W_g) are one matrix, fused at load.
"""

from __future__ import annotations

from typing import List, Optional

import torch

from .. import kernels
from ..config.model_config import PartSpec
from ..registry import build_part, register_part
from .base import CacheSpec, CacheView, Fetch, Mixer, StepContext, TensorSpec


@register_part("mixer", "latent_attention")
class LatentAttention(Mixer):
    graph_safe = True

    DEFAULT_NAMES = (("dq", "dq"), ("dq_norm", "dq.norm"), ("uq", "uq"), ("dkv", "dkv"), ("dkv_norm", "dkv.norm"),
                     ("uk", "uk"), ("uv", "uv"), ("sink", "sink"), ("gate", "g"), ("out", "o"))

    def __init__(self, hidden_size: int, heads: int, dim: int, rot_dim: int, value_dim: int, kv_rank: int,
                 q_rank: int, scale: float, eps: float, position: PartSpec, prefix: str, sink: bool = True,
                 output_gate: bool = True, window: Optional[int] = None, tensor_names=None):
        self.hidden_size, self.heads, self.dim, self.rot_dim = int(hidden_size), int(heads), int(dim), int(rot_dim)
        self.value_dim, self.kv_rank, self.q_rank = int(value_dim), int(kv_rank), int(q_rank)
        self.scale, self.eps, self.prefix = float(scale), float(eps), prefix
        self.has_sink, self.has_gate, self.window = bool(sink), bool(output_gate), window
        if not 1 <= self.kv_rank <= kernels.LATENT_MAX_RANK:
            raise ValueError(f"kv_rank {self.kv_rank} outside 1..{kernels.LATENT_MAX_RANK}")
        self.position = build_part("position", position)
        self.q_head = self.dim + self.rot_dim
        self.names = dict(self.DEFAULT_NAMES)
        self.names.update(dict(tensor_names or ()))
        self.w_in = self.w_uq = self.w_uk = self.w_uv = self.w_o = None
        self.q_norm = self.kv_norm = self.sink = None

    def _n(self, what: str) -> str:
        return self.prefix + self.names[what]

    # ---- weights ----------------------------------------------------------------------
    def tensor_specs(self) -> List[TensorSpec]:
        W, H = self.hidden_size, self.heads
        specs = [TensorSpec(self._n("dq"), (self.q_rank, W)),
                 TensorSpec(self._n("dq_norm"), (self.q_rank,), role="vector", init="norm"),
                 TensorSpec(self._n("uq"), (H * self.q_head, self.q_rank)),
                 TensorSpec(self._n("dkv"), (self.kv_rank + self.rot_dim, W)),
                 TensorSpec(self._n("dkv_norm"), (self.kv_rank,), role="vector", init="norm"),
                 TensorSpec(self._n("uk"), (H * self.dim, self.kv_rank)),
                 TensorSpec(self._n("uv"), (H * self.value_dim, self.kv_rank)),
                 TensorSpec(self._n("out"), (W, H * self.value_dim))]
        if self.has_sink:
            specs.append(TensorSpec(self._n("sink"), (H,), role="vector"))
        if self.has_gate:
            specs.append(TensorSpec(self._n("gate"), (H * self.value_dim, W)))
        return specs

    def load(self, fetch: Fetch) -> None:
        H = self.heads
        parts = [fetch(self._n("dq")), fetch(self._n("dkv"))]
        if self.has_gate:
            parts.append(fetch(self._n("gate")))
        self.w_in = torch.cat(parts, dim=0).contiguous()            # rows: [c_q | c, k_rot | gate]
        self.w_uq, self.w_o = fetch(self._n("uq")), fetch(self._n("out"))
        self.w_uk = fetch(self._n("uk")).view(H, self.dim, self.kv_rank)                       # q_plain_h @ W_uk[h]
        self.w_uv = fetch(self._n("uv")).view(H, self.value_dim, self.kv_rank).transpose(1, 2)  # o_h @ W_uv[h]^T
        self.q_norm, self.kv_norm = fetch(self._n("dq_norm")), fetch(self._n("dkv_norm"))
        self.sink = fetch(self._n("sink")) if self.has_sink else None

    def weight_bytes(self) -> int:
        el = self.w_in.element_size()
        n = sum(t.numel() for t in (self.w_in, self.w_uq, self.w_uk, self.w_uv, self.w_o)) * el
        return n + 4 * (self.q_rank + self.kv_rank + (self.heads if self.has_sink else 0))

    # ---- cache ------------------------------------------------------------------------
    def cache_spec(self) -> CacheSpec:
        return CacheSpec("window" if self.window else "full", window=self.window,
                         row_width=self.kv_rank + self.rot_dim)

    # ---- forward ----------------------------------------------------------------------
    def forward(self, x: torch.Tensor, ctx: StepContext, cache: Optional[CacheView],
                state: Optional[torch.Tensor]) -> torch.Tensor:
        assert cache is not None, "latent attention needs a cache slot"
        H, R, Dr, T = self.heads, self.kv_rank, self.rot_dim, x.shape[0]
        proj = kernels.linear(x, self.w_in)                                   # [T, q_rank | R + Dr | H * vdim]
        cq = kernels.rms_norm_slice(proj, 0, self.q_rank, self.q_norm, self.eps)
        q = kernels.linear(cq, self.w_uq)                                     # [T, H * (dim + rot_dim)]
        table = self.position.rotary_table(x.device)        # None: nothing is turned
        inv_freq, rot = table if table is not None else (None, 0)
        if rot:
            kernels.rope_head_slices(q, H, self.q_head, self.dim, rot, inv_freq, ctx.positions)
        if cache.append:
            kernels.latent_append(proj, self.q_rank, R, Dr, self.kv_norm, self.eps, inv_freq, rot, ctx,
                                  cache.pages, cache.block_table, cache.page_size)
        # the key projection folded into the query: [H, T, dim] x [H, dim, R]
        q_abs = kernels.heads_linear(q.view(T, H, self.q_head)[:, :, :self.dim].transpose(0, 1), self.w_uk)
        o_lat = kernels.latent_attention(q_abs, q, self.q_head, self.dim, Dr, cache.pages, cache.block_table,
                                         cache.page_size, ctx, self.sink, self.scale, self.window or 0)
        v = kernels.heads_linear(o_lat, self.w_uv)                            # [H, T, vdim]
        if self.has_gate:
            o = kernels.heads_sigmoid_gate(v, proj, self.q_rank + R + Dr)
        else:
            o = v.transpose(0, 1).reshape(T, H * self.value_dim)
        return kernels.linear(o, self.w_o)
