"""Difavik: its config.json keys, and configuration -> plan of parts.

A decoder-only model whose layers are listed one by one in config.json.  The token embedding has a
second table added to it, looked up by a hash of (previous token, token).  Every layer puts its
norm on the sublayer's OUTPUT and scales it per channel: ``x += ls1 * norm1(mixer(x))``, then
``x += ls2 * norm2(ff(x))``, with RMS norms whose stored weight lies around zero (``1 + w``
multiplies).  Two kinds of layer:

* ``lightning``: linear attention with a fixed decay per head over SiLU'd q, k, v; the heads normed
  together, a sigmoid gate.
* ``parallel``: two mixers side by side on the same input, their outputs RMS-normed (own weights)
  and averaged: on the left a grouped-query softmax attention whose values are its keys (whole-
  projection q/k norm, a linear distance penalty per head, a sliding window that keeps the first
  tokens, a sigmoid gate per head); on the right a retention (rotary q and k, k scaled, a fixed
  decay per head, per-head unit norm, a SiLU gate).

The feed-forward is dense (with biases) or a softmax-routed mixture of experts whose weights are
the chosen experts' scores as they are; both use the capped gated activation.  A layer may borrow
another layer's tensors (``weights_of``) while keeping cache and state of its own.  The head is
the embedding table.

config.json (every size and constant comes from here or from a tensor's shape)::

    architecture   "Difavik"
    vocab, width
    norm.eps
    embedding.bigram   {buckets, mul_prev, mul_cur}          (optional)
    layers[i]          {type, mixer, mlp, weights_of?}
      type "lightning": mixer {heads, dim, vdim, decay[heads]}
      type "parallel":  mixer {left:  {heads, kv_heads, dim, vdim, scale, mask: {size, keep_first}},
                               right: {heads, dim, vdim, decay[heads], rot: {base, dims}}}
      mlp   null, {kind: "dense", ff, limit}, or
            {kind: "moe", expert: {ff, limit}, router: {experts, top}}

Tensors: ``embed``, ``bigram`` [buckets + 1, width], ``final.norm``, and per layer with tensors of
its own ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.ls1``, ``l<i>.ls2``, ``l<i>.mix.*``, ``l<i>.mlp.*``.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

from ..config.model_config import (ConfigError, LayerCall, LayerSpec, ModelPlan, PartSpec, opt_float, req_int)
from ..registry import register_architecture

LAYER_TYPES = ("lightning", "parallel")
_NAMES = (("norm1", "norm1"), ("mixer", "mix"), ("norm2", "norm2"), ("feed_forward", "mlp"),
          ("scale1", "ls1"), ("scale2", "ls2"))
SLOPE_SPAN = 8.0            # head h's distance slope is 2^(-SLOPE_SPAN (h + 1) / heads)
GATE_ALPHA = 1.702          # the capped activation's sigmoid argument is GATE_ALPHA * gate


def _obj(d: Dict[str, Any], key: str, where: str) -> Dict[str, Any]:
    v = d.get(key)
    if not isinstance(v, dict):
        raise ConfigError(f"config.json: {where}{key!r} must be an object")
    return v


def _float(d: Dict[str, Any], key: str, where: str) -> float:
    if key not in d or d[key] is None:
        raise ConfigError(f"config.json: required key {where}{key!r} is missing")
    try:
        return opt_float(d, key, 0.0)
    except ConfigError as e:
        raise ConfigError(str(e).replace("config.json: ", f"config.json: {where}")) from None


def _int(d: Dict[str, Any], key: str, where: str, least: int = 1) -> int:
    try:
        v = req_int(d, key)
    except ConfigError as e:
        raise ConfigError(str(e).replace("config.json: ", f"config.json: {where}")) from None
    if v < least:
        raise ConfigError(f"config.json: {where}{key!r} must be at least {least}, got {v}")
    return v


def _decay(d: Dict[str, Any], heads: int, where: str) -> Tuple[float, ...]:
    v = d.get("decay")
    if not isinstance(v, list) or len(v) != heads or any(isinstance(x, bool) or not isinstance(x, (int, float)) for x in v):
        raise ConfigError(f"config.json: {where}'decay' must list one number per head ({heads})")
    return tuple(float(x) for x in v)


@dataclass(frozen=True)
class LinearAttentionSizes:
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]
    rot_base: float = 10000.0
    rot_dims: int = 0


@dataclass(frozen=True)
class TiedAttentionSizes:
    heads: int
    kv_heads: int
    dim: int
    scale: float
    window: int
    keep_first: int


@dataclass(frozen=True)
class MlpSizes:
    kind: str               # "dense" | "moe"
    ff: int
    limit: float
    experts: int = 0
    top: int = 0


@dataclass(frozen=True)
class DifavikLayer:
    type: str
    mixer: Any              # LinearAttentionSizes, or (TiedAttentionSizes, LinearAttentionSizes)
    mlp: Optional[MlpSizes]
    weights_of: Optional[int]


def _linear_attention(m: Dict[str, Any], where: str, rotary: bool) -> LinearAttentionSizes:
    heads = _int(m, "heads", where)
    base, dims = 10000.0, 0
    dim = _int(m, "dim", where)
    if rotary and m.get("rot") is not None:
        rot = _obj(m, "rot", where)
        dims = _int(rot, "dims", where + "rot.", least=0)
        base = _float(rot, "base", where + "rot.")
        if dims % 2 or dims > dim:
            raise ConfigError(f"config.json: {where}rot.dims={dims} must be even and at most dim={dim}")
        if base <= 0:
            raise ConfigError(f"config.json: {where}rot.base must be positive")
    return LinearAttentionSizes(heads=heads, dim=dim, vdim=_int(m, "vdim", where), decay=_decay(m, heads, where),
                                rot_base=base, rot_dims=dims)


def _tied_attention(m: Dict[str, Any], where: str) -> TiedAttentionSizes:
    heads, kv = _int(m, "heads", where), _int(m, "kv_heads", where)
    if heads % kv:
        raise ConfigError(f"config.json: {where}heads={heads} is not a multiple of kv_heads={kv}")
    dim = _int(m, "dim", where)
    if "vdim" in m and m["vdim"] is not None and _int(m, "vdim", where) != dim:
        raise ConfigError(f"config.json: {where}vdim must equal dim={dim}: the values are the keys")
    mask = _obj(m, "mask", where)
    return TiedAttentionSizes(heads=heads, kv_heads=kv, dim=dim, scale=_float(m, "scale", where),
                              window=_int(mask, "size", where + "mask."),
                              keep_first=_int(mask, "keep_first", where + "mask.", least=0))


def _mlp(f: Optional[Dict[str, Any]], where: str) -> Optional[MlpSizes]:
    if f is None:
        return None
    if not isinstance(f, dict):
        raise ConfigError(f"config.json: {where[:-1]} must be an object or null")
    kind = f.get("kind")
    if kind == "dense":
        out = MlpSizes("dense", ff=_int(f, "ff", where), limit=_float(f, "limit", where))
    elif kind == "moe":
        ex, ro = _obj(f, "expert", where), _obj(f, "router", where)
        out = MlpSizes("moe", ff=_int(ex, "ff", where + "expert."), limit=_float(ex, "limit", where + "expert."),
                       experts=_int(ro, "experts", where + "router."), top=_int(ro, "top", where + "router."))
        if out.top > out.experts:
            raise ConfigError(f"config.json: {where}router.top={out.top} exceeds experts={out.experts}")
    else:
        raise ConfigError(f"config.json: {where}kind = {kind!r}; known: ['dense', 'moe']")
    if out.limit <= 0:
        raise ConfigError(f"config.json: {where}limit must be positive")
    return out


@dataclass(frozen=True)
class DifavikConfig:
    vocab: int
    width: int
    eps: float
    bigram: Optional[Tuple[int, int, int]]          # (buckets, mul_prev, mul_cur)
    layers: Tuple[DifavikLayer, ...]

    ARCHITECTURE = "Difavik"

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "DifavikConfig":
        raw = d.get("layers")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers: List[DifavikLayer] = []
        for i, L in enumerate(raw):
            where = f"layers[{i}]."
            if not isinstance(L, dict):
                raise ConfigError(f"config.json: layers[{i}] must be an object")
            kind = L.get("type")
            if kind not in LAYER_TYPES:
                raise ConfigError(f"config.json: {where}type = {kind!r}; known: {list(LAYER_TYPES)}")
            m = _obj(L, "mixer", where)
            if kind == "lightning":
                mixer: Any = _linear_attention(m, where + "mixer.", rotary=False)
            else:
                mixer = (_tied_attention(_obj(m, "left", where + "mixer."), where + "mixer.left."),
                         _linear_attention(_obj(m, "right", where + "mixer."), where + "mixer.right.", rotary=True))
            owner = L.get("weights_of")
            if owner is not None:
                owner = _int(L, "weights_of", where, least=0)
                if owner >= len(raw) or owner == i:
                    raise ConfigError(f"config.json: {where}weights_of={owner} names no other layer")
            layers.append(DifavikLayer(kind, mixer, _mlp(L.get("mlp"), where + "mlp."), owner))
        for i, L in enumerate(layers):                   # a borrowed layer must be of the same make
            j = cls._owner(layers, i)
            if (layers[j].type, layers[j].mixer, layers[j].mlp) != (L.type, L.mixer, L.mlp):
                raise ConfigError(f"config.json: layers[{i}] uses the weights of layer {j} but differs from it")
        bigram = None
        emb = d.get("embedding")
        if isinstance(emb, dict) and emb.get("bigram") is not None:
            b = _obj(emb, "bigram", "embedding.")
            bigram = (_int(b, "buckets", "embedding.bigram."), _int(b, "mul_prev", "embedding.bigram.", least=0),
                      _int(b, "mul_cur", "embedding.bigram.", least=0))
        eps = _float(_obj(d, "norm", ""), "eps", "norm.")
        if eps <= 0:
            raise ConfigError("config.json: norm.eps must be positive")
        return cls(vocab=_int(d, "vocab", ""), width=_int(d, "width", ""), eps=eps, bigram=bigram, layers=tuple(layers))

    @staticmethod
    def _owner(layers, i: int) -> int:
        seen = set()
        while layers[i].weights_of is not None:
            if i in seen:
                raise ConfigError(f"config.json: layers[{i}].weights_of runs in a circle")
            seen.add(i)
            i = layers[i].weights_of
        return i

    def owner(self, i: int) -> int:
        """The layer whose tensors layer i uses (itself unless it borrows)."""
        return self._owner(self.layers, i)


_LINEAR_NAMES = (("q", "q"), ("k", "k"), ("v", "v"), ("gate", "g"), ("out", "o"), ("norm", "norm"))


def _mixer_spec(cfg: DifavikConfig, L: DifavikLayer) -> PartSpec:
    if L.type == "lightning":
        m = L.mixer
        return PartSpec.make("decay_linear_attention", hidden_size=cfg.width, heads=m.heads, dim=m.dim,
                             value_dim=m.vdim, decay=m.decay, eps=cfg.eps, qkv_activation="silu", position=None,
                             key_scale=None, norm_per_head=False, norm_weight=True, gate="sigmoid",
                             tensor_names=_LINEAR_NAMES)
    a, r = L.mixer
    left = PartSpec.make("tied_value_attention", hidden_size=cfg.width, heads=a.heads, kv_heads=a.kv_heads,
                         head_dim=a.dim, scale=a.scale, eps=cfg.eps, window=a.window, keep_first=a.keep_first,
                         slope_span=SLOPE_SPAN, qk_bias=True, head_gate=True)
    position = None
    if r.rot_dims:
        position = PartSpec.make("rotary_half_split", head_dim=r.dim, theta=r.rot_base, rotary_dim=r.rot_dims)
    right = PartSpec.make("decay_linear_attention", hidden_size=cfg.width, heads=r.heads, dim=r.dim, value_dim=r.vdim,
                          decay=r.decay, eps=cfg.eps, qkv_activation="none", position=position,
                          key_scale=float(r.dim) ** -0.5, norm_per_head=True, norm_weight=False, gate="silu",
                          tensor_names=_LINEAR_NAMES)
    return PartSpec.make("parallel_mean", hidden_size=cfg.width, eps=cfg.eps,
                         branches=(("left", left), ("right", right)), weight_suffix="out")


def _ff_spec(cfg: DifavikConfig, f: Optional[MlpSizes]) -> PartSpec:
    if f is None:
        return PartSpec.make("none")
    activation = ("capped", f.limit, GATE_ALPHA)
    if f.kind == "dense":
        return PartSpec.make("dense_swiglu", hidden_size=cfg.width, intermediate_size=f.ff, activation=activation,
                             bias=True, tensor_names=(("gate", "gate"), ("up", "up"), ("down", "down"),
                                                      ("gate_bias", "gate.b"), ("up_bias", "up.b"),
                                                      ("down_bias", "down.b")))
    return PartSpec.make("sparse_moe_swiglu", hidden_size=cfg.width, num_experts=f.experts, top_k=f.top,
                         norm_topk_prob=False, moe_intermediate_size=f.ff, shared_intermediate_size=0,
                         scoring="softmax", weight_on="output", activation=activation,
                         tensor_names=(("router", "router"), ("gate", "e{e}.gate"), ("up", "e{e}.up"),
                                       ("down", "e{e}.down")))


def build_plan(cfg: DifavikConfig) -> ModelPlan:
    norm = PartSpec.make("rms_norm", size=cfg.width, eps=cfg.eps, weight_name="", one_plus=True)
    # blocks exist for the layers that have tensors of their own; a borrowing layer is one more call of
    # its owner's block, with the cache slot and state slot of its own place in the list
    block_of: Dict[int, int] = {}
    layers = []
    for i, L in enumerate(cfg.layers):
        if L.weights_of is None:
            block_of[i] = len(layers)
            layers.append(LayerSpec("sublayer_norm_scaled", norm, _mixer_spec(cfg, L), _ff_spec(cfg, L.mlp),
                                    prefix=f"l{i}.", names=_NAMES))
    order = tuple(LayerCall(block_of[cfg.owner(i)], i, True, state=i) for i in range(len(cfg.layers)))
    extras = ()
    if cfg.bigram is not None:
        extras = (PartSpec.make("hashed_pair", hidden_size=cfg.width, buckets=cfg.bigram[0], mul_prev=cfg.bigram[1],
                                mul_cur=cfg.bigram[2], name="bigram"),)
    return ModelPlan(vocab_size=cfg.vocab, hidden_size=cfg.width, layers=tuple(layers), order=order,
                     final_norm=norm, tie_word_embeddings=True, embedding_name="embed",
                     final_norm_name="final.norm.", embedding_extras=extras)


register_architecture(DifavikConfig.ARCHITECTURE, DifavikConfig.from_dict, build_plan)
