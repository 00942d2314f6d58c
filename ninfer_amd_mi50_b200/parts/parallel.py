"""Several mixers side by side on the same input: the mean of their outputs, each first over its
own root mean square and times its own weight.

    out = (1 / n) * sum_m (y_m / rms(y_m)) * w_m,      y_m = mixer_m(x)

At most one of the mixers may keep pages and at most one a fixed-size state: the layer's cache
slot and state slot go to those.  The result is float32 (a norm reads it next).
"""

from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch

from .. import kernels
from ..config.model_config import PartSpec
from ..registry import build_part, register_part
from .base import CacheSpec, CacheView, Fetch, Mixer, StateSpec, StepContext, TensorSpec


@register_part("mixer", "parallel_mean")
class ParallelMean(Mixer):
    def __init__(self, hidden_size: int, eps: float, prefix: str, branches: Sequence[Tuple[str, PartSpec]],
                 weight_suffix: str = "out"):
        """`branches`: (name, mixer spec) pairs; branch `name`'s tensors lie below ``prefix + name + "."``
        and its weight is ``prefix + name + "." + weight_suffix``."""
        if not 1 <= len(branches) <= 4:
            raise ValueError("one to four mixers side by side")
        self.hidden_size, self.eps, self.prefix = int(hidden_size), float(eps), prefix
        self.branch_names = [n for n, _ in branches]
        self.mixers: List[Mixer] = [build_part("mixer", spec, prefix=f"{prefix}{n}.") for n, spec in branches]
        self.weight_names = [f"{prefix}{n}.{weight_suffix}" for n in self.branch_names]
        self.weights: List[torch.Tensor] = []
        if sum(m.cache_spec() is not None for m in self.mixers) > 1 or sum(m.state_spec() is not None for m in self.mixers) > 1:
            raise ValueError("at most one mixer with pages and one with a state may stand side by side")

    @property
    def graph_safe(self) -> bool:
        return all(m.graph_safe for m in self.mixers)

    def tensor_specs(self) -> List[TensorSpec]:
        specs = [s for m in self.mixers for s in m.tensor_specs()]
        return specs + [TensorSpec(n, (self.hidden_size,), role="vector", init="norm") for n in self.weight_names]

    def load(self, fetch: Fetch) -> None:
        for m in self.mixers:
            m.load(fetch)
        self.weights = [fetch(n) for n in self.weight_names]

    def weight_bytes(self) -> int:
        return sum(m.weight_bytes() for m in self.mixers) + 4 * self.hidden_size * len(self.mixers)

    def check_limits(self, dtype, max_context, page_size) -> None:
        for m in self.mixers:
            m.check_limits(dtype, max_context, page_size)

    def cache_spec(self) -> Optional[CacheSpec]:
        return next((s for s in (m.cache_spec() for m in self.mixers) if s is not None), None)

    def state_spec(self) -> Optional[StateSpec]:
        return next((s for s in (m.state_spec() for m in self.mixers) if s is not None), None)

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: Optional[CacheView],
                state: Optional[torch.Tensor]) -> torch.Tensor:
        outs = [m.forward(x, ctx, cache if m.cache_spec() is not None else None,
                          state if m.state_spec() is not None else None) for m in self.mixers]
        return kernels.mean_of_rmsnorms(outs, self.weights, self.eps)
