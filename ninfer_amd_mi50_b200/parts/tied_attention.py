"""Grouped-query softmax attention whose values are its keys.

With H query heads, G key heads of size D (query head h reads key head ``h // (H / G)``) and the
layer's input x:

    q = W_q x + b_q,   k = W_k x + b_k,   v = k                     (no value projection)
    q' = q / rms(q) * w_qn,   k' = k / rms(k) * w_kn                 (one norm over the WHOLE
                                                                     projection, all heads at once)
    s_ij = (q'_i . k'_j) * scale - slope_h * (i - j)                 slope_h = 2^(-slope_span (h+1) / H)
    j visible to i  iff  j <= i and (i - j < window or j < keep_first)
    o_h = softmax(s) v * sigmoid(W_g x)_h                            (one gate number a head)
    out = W_o concat_h(o_h)

Positions enter only through the distance term: nothing is rotated, and the kept first keys keep
their true positions.  The cache holds k' as keys and k (bias added, not normed) as values, in
the usual page layout, so the cache manager and the attention kernels see an ordinary
grouped-query cache; its window group keeps the pages of the first `keep_first` tokens for good.
The three projections that read x (q, k and the gate) are one matrix, fused at load; its product
is taken as float32 sums so that biases and norms see unrounded values.
"""

from __future__ import annotations

from typing import List, Optional

import torch

from .. import kernels
from ..registry import register_part
from .base import CacheSpec, CacheView, Fetch, Mixer, StepContext, TensorSpec


@register_part("mixer", "tied_value_attention")
class TiedValueAttention(Mixer):
    graph_safe = True

    DEFAULT_NAMES = (("q", "q"), ("k", "k"), ("q_bias", "q.b"), ("k_bias", "k.b"), ("q_norm", "q.norm"),
                     ("k_norm", "k.norm"), ("gate", "g"), ("out", "o"))

    def __init__(self, hidden_size: int, heads: int, kv_heads: int, head_dim: int, scale: float, eps: float,
                 prefix: str, window: Optional[int] = None, keep_first: int = 0, slope_span: Optional[float] = 8.0,
                 qk_bias: bool = True, head_gate: bool = True, tensor_names=None):
        if heads % kv_heads:
            raise ValueError(f"{heads} query heads do not divide into {kv_heads} groups")
        if not 1 <= int(head_dim) <= 256:
            raise ValueError(f"head_dim={head_dim} outside 1..256")
        self.hidden_size, self.heads, self.kv_heads, self.head_dim = int(hidden_size), int(heads), int(kv_heads), int(head_dim)
        self.scale, self.eps, self.prefix = float(scale), float(eps), prefix
        self.window = int(window) if window else None
        self.keep_first = int(keep_first) if self.window else 0
        self.slope_span = None if slope_span is None else float(slope_span)
        self.qk_bias, self.head_gate = bool(qk_bias), bool(head_gate)
        self.q_width, self.k_width = self.heads * self.head_dim, self.kv_heads * self.head_dim
        self.names = dict(self.DEFAULT_NAMES)
        self.names.update(dict(tensor_names or ()))
        self.w_in = self.w_o = self.b_q = self.b_k = self.q_norm = self.k_norm = None
        self._slopes = {}

    def _n(self, what: str) -> str:
        return self.prefix + self.names[what]

    # ---- weights ----------------------------------------------------------------------
    def tensor_specs(self) -> List[TensorSpec]:
        W = self.hidden_size
        specs = [TensorSpec(self._n("q"), (self.q_width, W)), TensorSpec(self._n("k"), (self.k_width, W)),
                 TensorSpec(self._n("q_norm"), (self.q_width,), role="vector", init="norm"),
                 TensorSpec(self._n("k_norm"), (self.k_width,), role="vector", init="norm"),
                 TensorSpec(self._n("out"), (W, self.q_width))]
        if self.qk_bias:
            specs += [TensorSpec(self._n("q_bias"), (self.q_width,), role="vector"),
                      TensorSpec(self._n("k_bias"), (self.k_width,), role="vector")]
        if self.head_gate:
            specs.append(TensorSpec(self._n("gate"), (self.heads, W)))
        return specs

    def load(self, fetch: Fetch) -> None:
        parts = [fetch(self._n("q")), fetch(self._n("k"))]
        if self.head_gate:
            parts.append(fetch(self._n("gate")))
        self.w_in = torch.cat(parts, dim=0).contiguous()                 # rows: [q | k | gate]
        self.w_o = fetch(self._n("out"))
        self.q_norm, self.k_norm = fetch(self._n("q_norm")), fetch(self._n("k_norm"))
        if self.qk_bias:
            self.b_q, self.b_k = fetch(self._n("q_bias")), fetch(self._n("k_bias"))

    def weight_bytes(self) -> int:
        n = (self.w_in.numel() + self.w_o.numel()) * self.w_in.element_size()
        return n + 4 * (self.q_width + self.k_width) * (2 if self.qk_bias else 1)

    def slopes(self, device: torch.device) -> Optional[torch.Tensor]:
        if self.slope_span is None:
            return None
        key = str(device)
        if key not in self._slopes:
            H = self.heads
            self._slopes[key] = torch.tensor([2.0 ** (-self.slope_span * (h + 1) / H) for h in range(H)],
                                             dtype=torch.float32, device=device)
        return self._slopes[key]

    # ---- cache ------------------------------------------------------------------------
    def cache_spec(self) -> CacheSpec:
        return CacheSpec("window" if self.window else "full", self.kv_heads, self.head_dim, self.window,
                         keep_first=self.keep_first)

    # ---- forward ----------------------------------------------------------------------
    def forward(self, x: torch.Tensor, ctx: StepContext, cache: Optional[CacheView],
                state: Optional[torch.Tensor]) -> torch.Tensor:
        assert cache is not None, "attention needs a cache slot"
        H, G, D = self.heads, self.kv_heads, self.head_dim
        proj = kernels.linear(x, self.w_in, out_dtype=torch.float32)           # [T, q | k | gate] float32 sums
        q = kernels.qk_whole_norm_append(proj, 0, self.q_width, self.b_q, self.b_k, self.q_norm, self.k_norm,
                                         self.eps, H, G, D, ctx, cache.pages, cache.block_table, cache.page_size,
                                         cache.append)
        o = kernels.biased_window_attention(q, H, G, D, cache.pages, cache.block_table, cache.page_size, ctx,
                                            self.window or 0, self.keep_first, self.scale, self.slopes(x.device),
                                            proj if self.head_gate else None, self.q_width + self.k_width)
        return kernels.linear(o, self.w_o)
