"""Typed configuration of the Pamarax decoder.

Its config.json is nested: ``vocab``, ``width``, ``embedding.scale``, ``norm.eps`` and a list ``layers`` whose entries
give the mixer's kind (``type``: ``attention``, ``mlstm`` or ``parallel``), the mixer's sizes and constants (``mixer``)
and the feed-forward (``mlp``: dense with biases, or null).  Every size and every constant that can differ between two
models of the design is read here; nothing about a particular model stands in code.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from ..errors import ConfigError, UnsupportedModelError
from .schema import _take
from .surelorn import _obj, _positive


def _grouped(d: Mapping[str, Any]) -> Tuple[int, int]:
    heads, kv = _positive(d, "heads"), _positive(d, "kv_heads")
    if heads % kv:
        raise ConfigError(f"{heads} heads do not group over {kv} kv_heads")
    return heads, kv


@dataclass(frozen=True)
class GatedAttentionConfig:
    """Grouped-query attention whose keys double as values, normed over the whole projection, partly rotated, with an
    output gate."""

    heads: int
    kv_heads: int
    dim: int                   # query / key entries a head
    vdim: int                  # value entries a head (the keys are the values: equal to dim)
    scale: float               # multiplies q . k
    rot_dims: int              # leading entries of each head that are rotated; 0: none
    rot_base: float

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "GatedAttentionConfig":
        heads, kv = _grouped(d)
        dim, vdim = _positive(d, "dim"), _positive(d, "vdim")
        if vdim != dim:
            raise ConfigError(f"the keys are the values, so vdim {vdim} must equal dim {dim}")
        rot = _obj(d, "rot", optional=True)
        rot_dims, rot_base = (_take(rot, "dims", int), _take(rot, "base", float)) if rot is not None else (0, 10000.0)
        if rot_dims % 2 or not 0 <= rot_dims <= dim:
            raise ConfigError(f"rot.dims {rot_dims} must be even and at most dim {dim}")
        if rot_dims and rot_base <= 0:
            raise ConfigError("rot.base must be positive")
        return cls(heads, kv, dim, vdim, _take(d, "scale", float), rot_dims, rot_base)


@dataclass(frozen=True)
class SinkAttentionHalfConfig:
    """Grouped-query attention with a per-head q/k norm, a query temperature and one more in the softmax's denominator."""

    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    temp_coef: float           # q *= 1 + coef * ln(floor((p + 1) / every) + 1); every 0: no temperature
    temp_every: int

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "SinkAttentionHalfConfig":
        heads, kv = _grouped(d)
        qt = _obj(d, "q_temp", optional=True)
        coef, every = (_take(qt, "coef", float), _positive(qt, "every")) if qt is not None else (0.0, 0)
        return cls(heads, kv, _positive(d, "dim"), _positive(d, "vdim"), _take(d, "scale", float), coef, every)


@dataclass(frozen=True)
class DeltaRuleHalfConfig:
    """The gated delta rule: a matrix of state a head behind short convolutions."""

    heads: int
    kv_heads: int              # heads of q and k
    dim: int
    vdim: int
    conv: int                  # taps of the causal convolution

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "DeltaRuleHalfConfig":
        heads, kv = _grouped(d)
        return cls(heads, kv, _positive(d, "dim"), _positive(d, "vdim"), _positive(d, "conv"))


@dataclass(frozen=True)
class ParallelConfig:
    left: SinkAttentionHalfConfig
    right: DeltaRuleHalfConfig
    left_scale: float
    right_scale: float

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "ParallelConfig":
        return cls(SinkAttentionHalfConfig.from_dict(_obj(d, "left")), DeltaRuleHalfConfig.from_dict(_obj(d, "right")),
                   _take(d, "left_scale", float), _take(d, "right_scale", float))


@dataclass(frozen=True)
class MatrixLSTMConfig:
    heads: int
    dim: int
    vdim: int
    gate_cap: float            # log gates pass cap * tanh(. / cap)

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "MatrixLSTMConfig":
        cap = _take(d, "gate_cap", float)
        if not cap > 0:
            raise ConfigError(f"gate_cap must be positive, got {cap}")
        return cls(_positive(d, "heads"), _positive(d, "dim"), _positive(d, "vdim"), cap)


_MIXERS = {"attention": GatedAttentionConfig, "mlstm": MatrixLSTMConfig, "parallel": ParallelConfig}


@dataclass(frozen=True)
class PamaraxLayer:
    mixer_kind: str                       # "attention", "mlstm" or "parallel"
    mixer: object
    dense_ff: Optional[int]               # None: the layer has no feed-forward


@dataclass(frozen=True)
class PamaraxConfig:
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    layers: Tuple[PamaraxLayer, ...]
    architecture: str = "Pamarax"

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "PamaraxConfig":
        entries = d.get("layers")
        if not isinstance(entries, (list, tuple)) or not entries:
            raise ConfigError("`layers` must list at least one layer")
        layers = []
        for i, e in enumerate(entries):
            if not isinstance(e, Mapping):
                raise ConfigError(f"layers[{i}] must be an object")
            kind = _take(e, "type", str)
            if kind not in _MIXERS:
                raise UnsupportedModelError(f"layers[{i}]: mixer type {kind!r} is not implemented; known: {sorted(_MIXERS)}")
            try:
                mixer = _MIXERS[kind].from_dict(_obj(e, "mixer"))
                mlp = _obj(e, "mlp", optional=True)
                ff = None
                if mlp is not None:
                    mlp_kind = _take(mlp, "kind", str)
                    if mlp_kind != "dense":
                        raise UnsupportedModelError(f"feed-forward kind {mlp_kind!r} is not implemented")
                    ff = _positive(mlp, "ff")
            except ConfigError as err:
                raise ConfigError(f"layers[{i}]: {err}") from None
            layers.append(PamaraxLayer(kind, mixer, ff))
        eps = _take(_obj(d, "norm"), "eps", float)
        if eps <= 0:
            raise ConfigError(f"norm.eps must be positive, got {eps}")
        emb = _obj(d, "embedding", optional=True)
        return cls(vocab=_positive(d, "vocab"), width=_positive(d, "width"), norm_eps=eps,
                   embedding_scale=_take(emb, "scale", float, 1.0) if emb is not None else 1.0,
                   layers=tuple(layers), architecture=_take(d, "architecture", str, "Pamarax"))
