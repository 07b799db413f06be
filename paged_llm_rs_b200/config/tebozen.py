"""Typed configuration of the Tebozen decoder.

Its config.json is nested: ``vocab``, ``width``, ``embedding.scale``, ``norm.eps`` and a list ``layers`` whose entries give
the mixer's kind (``type``: ``attention``, ``mlstm`` or ``latent_attention``), the mixer's sizes and constants (``mixer``)
and the feed-forward (``mlp``: a mixture of experts, or null).  Every size and every constant that can differ between two
models of the design is read here; nothing about a particular model stands in code.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from ..errors import ConfigError, UnsupportedModelError
from .schema import _take
from .surelorn import _obj, _positive


def _rotation(d: Mapping[str, Any], most: int) -> Tuple[int, float]:
    rot = _obj(d, "rot", optional=True)
    if rot is None:
        return 0, 10000.0
    dims, base = _take(rot, "dims", int), _take(rot, "base", float)
    if dims % 2 or not 0 <= dims <= most:
        raise ConfigError(f"rot.dims {dims} must be even and at most {most}")
    if dims and base <= 0:
        raise ConfigError("rot.base must be positive")
    return dims, base


@dataclass(frozen=True)
class DifferentialAttentionConfig:
    """Grouped-query attention that takes two softmax maps a head over the same values and subtracts the second, behind
    short convolutions on q, k and v, within a sliding window."""

    heads: int
    kv_heads: int
    dim: int                   # query / key entries a map
    vdim: int
    scale: float               # multiplies q . k
    diff: float                # lambda's constant part; the head's output is also multiplied by 1 - diff
    conv: int                  # taps of the causal convolution on q, k and v; 0: none
    window: Optional[int]      # position i sees j with 0 <= i - j < window; None: every j <= i
    rot_dims: int              # leading entries of each map of each head that are rotated; 0: none
    rot_base: float

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "DifferentialAttentionConfig":
        heads, kv = _positive(d, "heads"), _positive(d, "kv_heads")
        if heads % kv:
            raise ConfigError(f"{heads} heads do not group over {kv} kv_heads")
        dim = _positive(d, "dim")
        mask = _obj(d, "mask", optional=True)
        window = _positive(mask, "size") if mask is not None else None
        rot_dims, rot_base = _rotation(d, dim)
        return cls(heads, kv, dim, _positive(d, "vdim"), _take(d, "scale", float), _take(d, "diff", float), _take(d, "conv", int, 0),
                   window, rot_dims, rot_base)


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


@dataclass(frozen=True)
class RotaryLatentAttentionConfig:
    """Attention whose keys and values are linear in one cached latent a token, with one rotated key part shared by the heads."""

    heads: int
    dim: int                   # unrotated query / key entries a head
    rot_dim: int               # rotated query / key entries a head (the key's are shared by the heads)
    vdim: int
    kv_rank: int
    scale: float
    rot_dims: int              # leading entries of the rotated part that are turned
    rot_base: float
    kv_from: Optional[int]     # the layer whose cached latent and key part this one attends over; None: its own

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "RotaryLatentAttentionConfig":
        rot_dim = _take(d, "rot_dim", int, 0)
        rot_dims, rot_base = _rotation(d, rot_dim)
        kv_from = _take(d, "kv_from", int, None)
        return cls(_positive(d, "heads"), _positive(d, "dim"), rot_dim, _positive(d, "vdim"), _positive(d, "kv_rank"),
                   _take(d, "scale", float), rot_dims, rot_base, kv_from)


@dataclass(frozen=True)
class ExpertsConfig:
    experts: int
    top: int
    expert_ff: int
    shared_ff: Optional[int]   # None: no shared expert

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "ExpertsConfig":
        kind = _take(d, "kind", str)
        if kind != "moe":
            raise UnsupportedModelError(f"feed-forward kind {kind!r} is not implemented")
        router = _obj(d, "router")
        experts, top = _positive(router, "experts"), _positive(router, "top")
        if top > experts:
            raise ConfigError(f"top {top} of {experts} experts")
        shared = _obj(d, "shared", optional=True)
        return cls(experts, top, _positive(_obj(d, "expert"), "ff"), _positive(shared, "ff") if shared is not None else None)


_MIXERS = {"attention": DifferentialAttentionConfig, "mlstm": MatrixLSTMConfig, "latent_attention": RotaryLatentAttentionConfig}


@dataclass(frozen=True)
class TebozenLayer:
    mixer_kind: str                       # "attention", "mlstm" or "latent_attention"
    mixer: object
    moe: Optional[ExpertsConfig]          # None: the layer has no feed-forward


@dataclass(frozen=True)
class TebozenConfig:
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    layers: Tuple[TebozenLayer, ...]
    architecture: str = "Tebozen"

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "TebozenConfig":
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
                moe = ExpertsConfig.from_dict(mlp) if mlp is not None else None
            except ConfigError as err:
                raise ConfigError(f"layers[{i}]: {err}") from None
            layers.append(TebozenLayer(kind, mixer, moe))
        for i, L in enumerate(layers):
            if L.mixer_kind != "latent_attention" or L.mixer.kv_from is None:
                continue
            m, j = L.mixer, L.mixer.kv_from
            if not 0 <= j < i or layers[j].mixer_kind != "latent_attention" or layers[j].mixer.kv_from is not None:
                raise ConfigError(f"layers[{i}]: kv_from {j} must name an earlier latent-attention layer that keeps its own latent")
            s = layers[j].mixer
            if (s.kv_rank, s.rot_dim, s.rot_dims, s.rot_base) != (m.kv_rank, m.rot_dim, m.rot_dims, m.rot_base):
                raise ConfigError(f"layers[{i}]: kv_rank, rot_dim and rotation must equal those of layer {j}, whose cache it reads")
        eps = _take(_obj(d, "norm"), "eps", float)
        if eps <= 0:
            raise ConfigError(f"norm.eps must be positive, got {eps}")
        emb = _obj(d, "embedding", optional=True)
        return cls(vocab=_positive(d, "vocab"), width=_positive(d, "width"), norm_eps=eps,
                   embedding_scale=_take(emb, "scale", float, 1.0) if emb is not None else 1.0,
                   layers=tuple(layers), architecture=_take(d, "architecture", str, "Tebozen"))
