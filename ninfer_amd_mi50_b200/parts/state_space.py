"""A state-space mixer in the dual (Mamba-2) form, with its state in the request's slot.

With ``inner = heads * head_dim``, N the state size and G groups, the input projection's rows are
``[z: inner | x: inner | B: G N | C: G N | dt: heads]``.  x, B and C pass a short causal
convolution per channel (bias, SiLU); ``dt = softplus(dt + dt_bias)`` without a clamp; per head h
(whose B and C are those of group ``h // (heads / G)``)

    S_t = exp(-exp(A_log_h) dt_t) S_{t-1} + dt_t B_t x_t^T          S is N x head_dim
    y_t = S_t^T C_t + D_h x_t

then ``y * silu(z)`` is normalised in ``norm_groups`` equal parts (each over its own root mean
square), multiplied by a weight, and projected out.  The gate comes before the norm.

What a request keeps between steps is of fixed size: the convolution's last ``taps - 1`` inputs
and S for every head, both float32, side by side in one slot (`state_spec`).  A step's rows of
one request continue from the slot and leave it updated, so prompts cut into portions, decoded
tokens and mixed batches all run the same two kernels (``csrc/ssm.cu``).  Decays, step sizes and
the state are 32-bit in both modes; the projections, the convolution's output and the gate are in
the engine's type.
"""

from __future__ import annotations

from typing import List, Optional

import torch

from .. import kernels
from ..registry import register_part
from .base import CacheView, Fetch, Mixer, StateSpec, StepContext, TensorSpec


@register_part("mixer", "state_space_dual")
class StateSpaceDual(Mixer):
    graph_safe = True

    DEFAULT_NAMES = (("in", "in"), ("conv", "conv"), ("conv_bias", "conv.b"), ("dt_bias", "dt_bias"),
                     ("A_log", "A_log"), ("D", "D"), ("norm", "norm"), ("out", "o"))

    def __init__(self, hidden_size: int, heads: int, head_dim: int, state_size: int, groups: int,
                 conv_taps: int, norm_groups: int, eps: float, prefix: str, tensor_names=None):
        self.hidden_size, self.heads, self.head_dim = int(hidden_size), int(heads), int(head_dim)
        self.state_size, self.groups, self.taps = int(state_size), int(groups), int(conv_taps)
        self.norm_groups, self.eps, self.prefix = int(norm_groups), float(eps), prefix
        if self.heads % self.groups:
            raise ValueError(f"{self.heads} heads do not split into {self.groups} groups")
        self.inner = self.heads * self.head_dim
        if self.inner % self.norm_groups:
            raise ValueError(f"inner width {self.inner} does not split into {self.norm_groups} norm parts")
        if not 1 <= self.taps <= kernels.CONV_MAX_TAPS:
            raise ValueError(f"conv taps {self.taps} outside 1..{kernels.CONV_MAX_TAPS}")
        if not 1 <= self.state_size <= kernels.SCAN_MAX_STATE:
            raise ValueError(f"state size {self.state_size} outside 1..{kernels.SCAN_MAX_STATE}")
        self.conv_channels = self.inner + 2 * self.groups * self.state_size
        self.proj_width = 2 * self.inner + 2 * self.groups * self.state_size + self.heads
        self.conv_state = (self.taps - 1) * self.conv_channels
        self.names = dict(self.DEFAULT_NAMES)
        self.names.update(dict(tensor_names or ()))
        self.w_in = self.w_out = self.conv_w = self.conv_b = None
        self.dt_bias = self.A_log = self.D = self.norm_w = None

    def _n(self, what: str) -> str:
        return self.prefix + self.names[what]

    def tensor_specs(self) -> List[TensorSpec]:
        return [TensorSpec(self._n("in"), (self.proj_width, self.hidden_size)),
                TensorSpec(self._n("conv"), (self.conv_channels, self.taps), role="vector"),
                TensorSpec(self._n("conv_bias"), (self.conv_channels,), role="vector"),
                TensorSpec(self._n("dt_bias"), (self.heads,), role="vector"),
                TensorSpec(self._n("A_log"), (self.heads,), role="vector"),
                TensorSpec(self._n("D"), (self.heads,), role="vector"),
                TensorSpec(self._n("norm"), (self.inner,), role="vector", init="norm"),
                TensorSpec(self._n("out"), (self.hidden_size, self.inner))]

    def load(self, fetch: Fetch) -> None:
        self.w_in, self.w_out = fetch(self._n("in")), fetch(self._n("out"))
        # the checkpoint's taps are [channels, taps]; the kernel reads them tap-major
        self.conv_w, self.conv_b = fetch(self._n("conv")).t().contiguous(), fetch(self._n("conv_bias"))
        self.dt_bias, self.A_log, self.D = fetch(self._n("dt_bias")), fetch(self._n("A_log")), fetch(self._n("D"))
        self.norm_w = fetch(self._n("norm"))

    def weight_bytes(self) -> int:
        n = (self.w_in.numel() + self.w_out.numel()) * self.w_in.element_size()
        return n + 4 * (self.conv_w.numel() + self.conv_b.numel() + 3 * self.heads + self.inner)

    def state_spec(self) -> StateSpec:
        """[conv inputs: (taps - 1) x channels | S: heads x head_dim x N], float32."""
        return StateSpec((self.conv_state + self.heads * self.head_dim * self.state_size,), torch.float32)

    def state_bytes(self) -> int:
        return 4 * self.state_spec().shape[0]

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: Optional[CacheView],
                state: Optional[torch.Tensor]) -> torch.Tensor:
        assert state is not None, "the state-space mixer needs a state slot"
        inner, GN = self.inner, self.groups * self.state_size
        proj = kernels.linear(x, self.w_in)                                     # [T, z | x | B | C | dt]
        xbc = kernels.causal_conv_silu(proj, inner, self.conv_channels, self.conv_w, self.conv_b, state, ctx)
        y = kernels.ssd_scan(xbc, 0, inner, inner + GN, proj, 2 * inner + 2 * GN, self.dt_bias, self.A_log, self.D,
                             state, self.conv_state, ctx, self.heads, self.head_dim, self.state_size, self.groups)
        g = kernels.gated_group_rmsnorm(y, proj, 0, self.norm_w, self.eps, self.norm_groups, x.dtype)
        return kernels.linear(g, self.w_out)
