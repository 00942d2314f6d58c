"""Linear attention with a fixed decay per head, its state in the request's slot.

Per head h, with q_t, k_t of size D and v_t of size V:

    S_t = g_h S_{t-1} + k_t v_t^T          (S starts at zero)         o_t = S_t^T q_t

without softmax or denominator.  Two designs of it are served by parameters:

* *retention*: q, k, v plain projections; the first `rotary_dim` dimensions of every q and k head
  turned by the position (half-split pairs); k times ``D^-1/2`` after the turn; each head's o over
  its own root mean square (no weight); times ``silu(W_g x)``; out-projection.
* *lightning*: q, k, v through SiLU; no rotation, no scale; all heads' o over one root mean square,
  times a weight; times ``sigmoid(W_g x)``; out-projection.

What a request keeps between steps is S for every head, float32, of fixed size (`state_spec`), so
prompts cut into portions, decoded tokens and mixed batches all run the same kernel
(``csrc/linear_attention.cu``), which continues from the slot and leaves it updated.  Decays,
angles, the turned and scaled vectors, S and the sums are 32-bit in both modes; the projections
(and their SiLU's argument) are in the engine's type.  The projections that read x (q, k, v and
the gate) are one matrix, fused at load.
"""

from __future__ import annotations

import math
from typing import List, Optional, Sequence

import torch

from .. import kernels
from ..config.model_config import PartSpec
from ..registry import build_part, register_part
from .base import CacheView, Fetch, Mixer, StateSpec, StepContext, TensorSpec


@register_part("mixer", "decay_linear_attention")
class DecayLinearAttention(Mixer):
    graph_safe = True

    DEFAULT_NAMES = (("q", "q"), ("k", "k"), ("v", "v"), ("gate", "g"), ("out", "o"), ("norm", "norm"))

    def __init__(self, hidden_size: int, heads: int, dim: int, value_dim: int, decay: Sequence[float], eps: float,
                 prefix: str, qkv_activation: str = "none", position: Optional[PartSpec] = None,
                 key_scale: Optional[float] = None, norm_per_head: bool = True, norm_weight: bool = False,
                 gate: str = "silu", tensor_names=None):
        self.hidden_size, self.heads, self.dim, self.value_dim = int(hidden_size), int(heads), int(dim), int(value_dim)
        self.decay_values = tuple(float(d) for d in decay)
        if len(self.decay_values) != self.heads:
            raise ValueError(f"{len(self.decay_values)} decays for {self.heads} heads")
        if not 1 <= self.dim <= kernels.LINEAR_ATTENTION_MAX_DIM:
            raise ValueError(f"dim {self.dim} outside 1..{kernels.LINEAR_ATTENTION_MAX_DIM}")
        if qkv_activation not in ("none", "silu"):
            raise ValueError(f"qkv_activation {qkv_activation!r}: 'none' or 'silu'")
        if gate not in ("silu", "sigmoid"):
            raise ValueError(f"gate {gate!r}: 'silu' or 'sigmoid'")
        self.eps, self.prefix = float(eps), prefix
        self.silu_qkv = qkv_activation == "silu"
        self.position = build_part("position", position) if position is not None else None
        self.key_scale = 1.0 if key_scale is None else float(key_scale)
        self.norm_per_head, self.norm_weight = bool(norm_per_head), bool(norm_weight)
        if self.norm_weight and self.norm_per_head:
            raise ValueError("a norm weight goes with the norm over all heads")
        self.gate = kernels.GATE_SILU if gate == "silu" else kernels.GATE_SIGMOID
        self.qk_width, self.v_width = self.heads * self.dim, self.heads * self.value_dim
        self.names = dict(self.DEFAULT_NAMES)
        self.names.update(dict(tensor_names or ()))
        self.w_in = self.w_o = self.norm_w = None
        self._decay = {}

    def _n(self, what: str) -> str:
        return self.prefix + self.names[what]

    def tensor_specs(self) -> List[TensorSpec]:
        W = self.hidden_size
        specs = [TensorSpec(self._n("q"), (self.qk_width, W)), TensorSpec(self._n("k"), (self.qk_width, W)),
                 TensorSpec(self._n("v"), (self.v_width, W)), TensorSpec(self._n("gate"), (self.v_width, W)),
                 TensorSpec(self._n("out"), (W, self.v_width))]
        if self.norm_weight:
            specs.append(TensorSpec(self._n("norm"), (self.v_width,), role="vector", init="norm"))
        return specs

    def load(self, fetch: Fetch) -> None:
        self.w_in = torch.cat([fetch(self._n(n)) for n in ("q", "k", "v", "gate")], dim=0).contiguous()
        self.w_o = fetch(self._n("out"))
        self.norm_w = fetch(self._n("norm")) if self.norm_weight else None

    def weight_bytes(self) -> int:
        return (self.w_in.numel() + self.w_o.numel()) * self.w_in.element_size() + (4 * self.v_width if self.norm_weight else 0)

    def state_spec(self) -> StateSpec:
        """S of every head, [heads][value column][dim], float32."""
        return StateSpec((self.heads * self.value_dim * self.dim,), torch.float32)

    def decay(self, device: torch.device) -> torch.Tensor:
        key = str(device)
        if key not in self._decay:
            self._decay[key] = torch.tensor(self.decay_values, dtype=torch.float64).to(torch.float32).to(device)
        return self._decay[key]

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: Optional[CacheView],
                state: Optional[torch.Tensor]) -> torch.Tensor:
        assert state is not None, "linear attention needs a state slot"
        proj = kernels.linear(x, self.w_in)                                    # [T, q | k | v | gate]
        table = self.position.rotary_table(x.device) if self.position is not None else None
        inv_freq, rot = table if table is not None else (None, 0)
        o = kernels.decay_linear_attention(proj, 0, self.qk_width, 2 * self.qk_width, self.decay(x.device), inv_freq,
                                           rot, self.key_scale, self.silu_qkv, state, ctx, self.heads, self.dim,
                                           self.value_dim)
        g = kernels.group_rmsnorm_gate(o, proj, 2 * self.qk_width + self.v_width, self.norm_w, self.eps,
                                       self.heads if self.norm_per_head else 1, self.gate, x.dtype)
        return kernels.linear(g, self.w_o)
