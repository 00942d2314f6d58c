"""Vekasun: its config.json keys, and configuration -> plan of parts.

A decoder-only model whose layers are listed one by one in config.json.  Every layer is
pre-norm (layer norm with a weight and no bias) around a *mixer* - latent attention or a
state-space mixer in the dual form - and, unless its ``mlp`` is null, a routed feed-forward
whose experts are scored by a sigmoid and weighted on their input.  A run of layers may be
repeated with the same weights (``loop``): each pass has cache and state of its own, and a
learned vector per pass is added to the stream right before the pass's first layer.  The logits
are the head's product times ``logit_scale``.

config.json (every size and constant comes from here or from a tensor's shape)::

    architecture   "Vekasun"
    vocab, width
    norm.eps
    logit_scale
    loop           {start, stop, times}: layers start .. stop-1 run `times` times in a row
    layers[i]      {type, mixer, mlp}
      type "latent_attention": mixer {heads, dim, rot_dim, vdim, kv_rank, q_rank, scale,
                                      rot: {base, dims}}
      type "mamba2":           mixer {heads, vdim, state, groups, conv, norm_groups}
      mlp            null, or {kind: "moe", expert: {ff}, router: {experts, top}}

Tensors: ``embed``, ``head``, ``final.norm``, ``loop.step`` [times, width], and per layer
``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*``, ``l<i>.mlp.router``, ``l<i>.mlp.e<j>.{gate,up,down}``.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

from ..config.model_config import (ConfigError, LayerCall, LayerSpec, ModelPlan, PartSpec, opt_float,
                                   req_int)
from ..registry import register_architecture

MIXER_TYPES = ("latent_attention", "mamba2")
_NAMES = (("norm1", "norm1"), ("mixer", "mix"), ("norm2", "norm2"), ("feed_forward", "mlp"))
LOOP_VECTORS = "loop.step"


def _obj(d: Dict[str, Any], key: str, where: str) -> Dict[str, Any]:
    v = d.get(key)
    if not isinstance(v, dict):
        raise ConfigError(f"config.json: {where}{key!r} must be an object")
    return v


def _req_float(d: Dict[str, Any], key: str, where: str) -> float:
    if key not in d or d[key] is None:
        raise ConfigError(f"config.json: required key {where}{key!r} is missing")
    return opt_float(d, key, 0.0)


def _int(d: Dict[str, Any], key: str, where: str, least: int = 1) -> int:
    try:
        v = req_int(d, key)
    except ConfigError as e:
        raise ConfigError(str(e).replace("config.json: ", f"config.json: {where}")) from None
    if v < least:
        raise ConfigError(f"config.json: {where}{key!r} must be at least {least}, got {v}")
    return v


@dataclass(frozen=True)
class LatentAttentionSizes:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    q_rank: int
    scale: float
    rot_base: float
    rot_dims: int


@dataclass(frozen=True)
class StateSpaceSizes:
    heads: int
    vdim: int
    state: int
    groups: int
    conv: int
    norm_groups: int


@dataclass(frozen=True)
class RoutedMlpSizes:
    ff: int
    experts: int
    top: int


@dataclass(frozen=True)
class VekasunLayer:
    type: str
    mixer: Any                              # LatentAttentionSizes | StateSpaceSizes
    mlp: Optional[RoutedMlpSizes]


@dataclass(frozen=True)
class VekasunConfig:
    vocab: int
    width: int
    eps: float
    logit_scale: float
    layers: Tuple[VekasunLayer, ...]
    loop_start: int
    loop_stop: int
    loop_times: int

    ARCHITECTURE = "Vekasun"

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "VekasunConfig":
        layers_raw = d.get("layers")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers: List[VekasunLayer] = []
        for i, L in enumerate(layers_raw):
            where = f"layers[{i}]."
            if not isinstance(L, dict):
                raise ConfigError(f"config.json: layers[{i}] must be an object")
            kind = L.get("type")
            if kind not in MIXER_TYPES:
                raise ConfigError(f"config.json: {where}type = {kind!r}; known: {list(MIXER_TYPES)}")
            m = _obj(L, "mixer", where)
            mw = where + "mixer."
            if kind == "latent_attention":
                rot_dim = _int(m, "rot_dim", mw, least=0)
                rot = m.get("rot") if rot_dim else (m.get("rot") or {"base": 10000.0, "dims": 0})
                if not isinstance(rot, dict):
                    raise ConfigError(f"config.json: {mw}'rot' must be an object")
                rot_dims = _int(rot, "dims", mw + "rot.", least=0)
                if rot_dims % 2 or rot_dims > rot_dim:
                    raise ConfigError(f"config.json: {mw}rot.dims={rot_dims} must be even and at most rot_dim={rot_dim}")
                base = _req_float(rot, "base", mw + "rot.")
                if base <= 0:
                    raise ConfigError(f"config.json: {mw}rot.base must be positive")
                mixer = LatentAttentionSizes(
                    heads=_int(m, "heads", mw), dim=_int(m, "dim", mw), rot_dim=rot_dim, vdim=_int(m, "vdim", mw),
                    kv_rank=_int(m, "kv_rank", mw), q_rank=_int(m, "q_rank", mw), scale=_req_float(m, "scale", mw),
                    rot_base=base, rot_dims=rot_dims)
            else:
                mixer = StateSpaceSizes(
                    heads=_int(m, "heads", mw), vdim=_int(m, "vdim", mw), state=_int(m, "state", mw),
                    groups=_int(m, "groups", mw), conv=_int(m, "conv", mw), norm_groups=_int(m, "norm_groups", mw))
                if mixer.heads % mixer.groups:
                    raise ConfigError(f"config.json: {mw}heads={mixer.heads} is not a multiple of groups={mixer.groups}")
                if (mixer.heads * mixer.vdim) % mixer.norm_groups:
                    raise ConfigError(f"config.json: {mw}heads * vdim does not split into norm_groups={mixer.norm_groups}")
            mlp = None
            if L.get("mlp") is not None:
                f = _obj(L, "mlp", where)
                fw = where + "mlp."
                if f.get("kind", "moe") != "moe":
                    raise ConfigError(f"config.json: {fw}kind = {f.get('kind')!r}; known: ['moe']")
                mlp = RoutedMlpSizes(ff=_int(_obj(f, "expert", fw), "ff", fw + "expert."),
                                     experts=_int(_obj(f, "router", fw), "experts", fw + "router."),
                                     top=_int(_obj(f, "router", fw), "top", fw + "router."))
                if mlp.top > mlp.experts:
                    raise ConfigError(f"config.json: {fw}router.top={mlp.top} exceeds experts={mlp.experts}")
            layers.append(VekasunLayer(kind, mixer, mlp))
        n = len(layers)
        loop = d.get("loop")
        if loop is None:
            start, stop, times = 0, 0, 1
        else:
            if not isinstance(loop, dict):
                raise ConfigError("config.json: 'loop' must be an object")
            start, stop = _int(loop, "start", "loop.", least=0), _int(loop, "stop", "loop.", least=0)
            times = _int(loop, "times", "loop.", least=1)
            if not start <= stop <= n:
                raise ConfigError(f"config.json: loop {start}..{stop} does not lie within the {n} layers")
        norm = _obj(d, "norm", "")
        eps = _req_float(norm, "eps", "norm.")
        if eps <= 0:
            raise ConfigError("config.json: norm.eps must be positive")
        return cls(vocab=_int(d, "vocab", ""), width=_int(d, "width", ""), eps=eps,
                   logit_scale=opt_float(d, "logit_scale", 1.0), layers=tuple(layers),
                   loop_start=start, loop_stop=stop, loop_times=times)

    @property
    def looped(self) -> bool:
        return self.loop_stop > self.loop_start

    def runs(self) -> List[Tuple[int, Optional[int]]]:
        """(layer, pass) in the order they run; pass is None outside the loop."""
        out: List[Tuple[int, Optional[int]]] = [(i, None) for i in range(self.loop_start)]
        if self.looped:
            for t in range(self.loop_times):
                out += [(i, t) for i in range(self.loop_start, self.loop_stop)]
        return out + [(i, None) for i in range(self.loop_stop, len(self.layers))]


def build_plan(cfg: VekasunConfig) -> ModelPlan:
    norm = PartSpec.make("layer_norm", size=cfg.width, eps=cfg.eps, weight_name="")
    layers = []
    for i, L in enumerate(cfg.layers):
        m = L.mixer
        if L.type == "latent_attention":
            if m.rot_dims:
                position = PartSpec.make("rotary_half_split", head_dim=m.rot_dim, theta=m.rot_base,
                                         rotary_dim=m.rot_dims)
            else:
                position = PartSpec.make("none", head_dim=m.rot_dim)
            mixer = PartSpec.make("latent_attention", hidden_size=cfg.width, heads=m.heads, dim=m.dim,
                                  rot_dim=m.rot_dim, value_dim=m.vdim, kv_rank=m.kv_rank, q_rank=m.q_rank,
                                  scale=m.scale, eps=cfg.eps, position=position)
        else:
            mixer = PartSpec.make("state_space_dual", hidden_size=cfg.width, heads=m.heads, head_dim=m.vdim,
                                  state_size=m.state, groups=m.groups, conv_taps=m.conv,
                                  norm_groups=m.norm_groups, eps=cfg.eps)
        if L.mlp is None:
            ffn = PartSpec.make("none")
        else:
            ffn = PartSpec.make(
                "sparse_moe_swiglu", hidden_size=cfg.width, num_experts=L.mlp.experts, top_k=L.mlp.top,
                norm_topk_prob=False, moe_intermediate_size=L.mlp.ff, shared_intermediate_size=0,
                scoring="sigmoid", weight_on="input",
                tensor_names=(("router", "router"), ("gate", "e{e}.gate"), ("up", "e{e}.up"), ("down", "e{e}.down")))
        layers.append(LayerSpec("pre_norm", norm, mixer, ffn, prefix=f"l{i}.", names=_NAMES))
    # every run of a layer has cache and state of its own: slot = the run's number
    order = []
    for slot, (i, t) in enumerate(cfg.runs()):
        add = (LOOP_VECTORS, t) if (t is not None and i == cfg.loop_start) else None
        order.append(LayerCall(i, slot, True, state=slot, add_vector=add))
    vectors = ((LOOP_VECTORS, cfg.loop_times),) if cfg.looped else ()
    return ModelPlan(vocab_size=cfg.vocab, hidden_size=cfg.width, layers=tuple(layers), order=tuple(order),
                     final_norm=norm, tie_word_embeddings=False, embedding_name="embed",
                     final_norm_name="final.norm.", head_name="head", logit_scale=cfg.logit_scale,
                     stream_vectors=vectors)


register_architecture(VekasunConfig.ARCHITECTURE, VekasunConfig.from_dict, build_plan)
