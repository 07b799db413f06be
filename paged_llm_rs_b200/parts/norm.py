"""RMSNorm (crates/pagedllm/src/model/layers.rs:40-65): x / sqrt(mean(x^2) + eps)
times a gain, the statistic in float.  ``add_norm`` fuses the residual add that
precedes it (crates/pagedllm/src/model/mod.rs:131-132) into the same kernel."""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import Norm, register_norm
from .spec import TensorSpec


class RMSNorm(Norm):
    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.width = int(spec.params["width"])
        self.eps = float(spec.params["eps"])
        self.leaf = spec.params.get("leaf", "weight")       # the gain's name under the prefix ("": the prefix is its name)
        self.gain = None

    def _gain_name(self):
        return self._name(self.leaf) if self.leaf else self.prefix

    def tensors(self):
        return [TensorSpec(self._gain_name(), (self.width,), "gain")]

    def bind(self, tensors):
        self.gain = tensors[self._gain_name()]

    def forward(self, x, rows=None):
        n = rows.numel() if rows is not None else x.shape[0]
        out = torch.empty((n, self.width), dtype=x.dtype, device=x.device)
        ops.rmsnorm(x, self.gain, self.eps, out, rows=rows)
        self.rt.record(self._name("out"), out)
        return out

    def add_norm(self, residual, delta, rows=None):
        n = rows.numel() if rows is not None else residual.shape[0]
        out = torch.empty((n, self.width), dtype=residual.dtype, device=residual.device)
        # With rows the sum is formed for those rows only and not stored.
        ops.rmsnorm(residual, self.gain, self.eps, out, delta=delta,
                    residual_out=residual if (delta is not None and rows is None) else None, rows=rows)
        self.rt.record(self._name("out"), out)
        return out


class StreamRMSNorm(RMSNorm):
    """RMSNorm for a decoder whose residual stream stays float32.  Two uses: ``forward`` norms rows of
    the float32 stream into the compute dtype (the model's last norm); ``add_into`` is the norm on a
    sublayer's OUTPUT: stream += norm(a), with the stream's rounding to the compute dtype as a
    by-product for the next sublayer's products."""

    def forward(self, x, rows=None):
        if x.dtype != torch.float32:
            return super().forward(x, rows)
        n = rows.numel() if rows is not None else x.shape[0]
        out = torch.empty((n, self.width), dtype=self.rt.dtype, device=x.device)
        ops.rmsnorm_from32(x, self.gain, self.eps, out, rows=rows)
        self.rt.record(self._name("out"), out)
        return out

    def add_norm(self, residual, delta, rows=None):
        if delta is not None:
            raise ValueError("a float32 stream carries no pending addition: its blocks add their own outputs")
        return self.forward(residual, rows)

    def add_into(self, stream, a):
        """stream (float32, in place) += norm(a) * gain; returns what the next sublayer reads: the
        stream itself in a float32 engine, else its rounding to the compute dtype."""
        h = None if a.dtype == torch.float32 else torch.empty_like(a)
        ops.outnorm_add(stream, a, self.gain, self.eps, h)
        return stream if h is None else h


class ScaledStreamRMSNorm(RMSNorm):
    """RMSNorm in a pre-norm decoder whose residual stream stays float32 and whose sublayer outputs are multiplied by
    one constant ``mult`` as they are added: ``add_norm`` does stream += mult * delta (in place) and norms the sum into
    the compute dtype, in one kernel.  ``one_plus``: the file holds the gain's distance from one."""

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.mult = float(spec.params.get("mult", 1.0))
        self.one_plus = bool(spec.params.get("one_plus", False))     # the file holds gain - 1

    def bind(self, tensors):
        w = tensors[self._gain_name()]
        self.gain = (w + 1.0) if self.one_plus else w

    def forward(self, x, rows=None):
        return self.add_norm(x, None, rows)

    def add_norm(self, residual, delta, rows=None):
        if residual.dtype != torch.float32:
            raise ValueError("the residual stream of this norm is float32")
        n = rows.numel() if rows is not None else residual.shape[0]
        out = torch.empty((n, self.width), dtype=self.rt.dtype, device=residual.device)
        ops.add_scaled_norm32(residual, delta, self.mult, self.gain, self.eps, out, rows=rows)
        self.rt.record(self._name("out"), out)
        return out


class PendingNormed:
    """A sublayer's output that is still to be normed (by the norm that made this) and added to the stream: what a block
    that norms its sublayers' outputs hands on, so that the next norm's kernel does all three."""

    __slots__ = ("a", "gain", "bias", "eps")

    def __init__(self, a, gain, bias, eps):
        self.a, self.gain, self.bias, self.eps = a, gain, bias, eps


class SandwichStreamRMSNorm(RMSNorm):
    """RMSNorm in a decoder whose residual stream stays float32 and whose sublayers are normed on the way in AND on the way
    out: x <- x + norm_out(sublayer(norm_in(x))).  As the norm on a sublayer's output it only wraps that output
    (``pending``); as the norm on the next sublayer's input (or the model's last norm) ``add_norm`` takes the wrapped
    output, norms it with ITS gain, adds it to the stream (in place) and norms the sum into the compute dtype, in one
    kernel.  ``one_plus``: the file holds gain - 1."""

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.one_plus = bool(spec.params.get("one_plus", False))

    def bind(self, tensors):
        w = tensors[self._gain_name()]
        self.gain = (w + 1.0) if self.one_plus else w

    def pending(self, a, bias=None) -> PendingNormed:
        return PendingNormed(a, self.gain, bias, self.eps)

    def forward(self, x, rows=None):
        return self.add_norm(x, None, rows)

    def add_norm(self, residual, delta, rows=None):
        if residual.dtype != torch.float32:
            raise ValueError("the residual stream of this norm is float32")
        if delta is not None and not isinstance(delta, PendingNormed):
            raise ValueError("this norm adds a sublayer's output that another norm of its kind wrapped (pending)")
        if delta is not None and delta.eps != self.eps:
            raise ValueError("the norms of one stream share one eps")
        n = rows.numel() if rows is not None else residual.shape[0]
        out = torch.empty((n, self.width), dtype=self.rt.dtype, device=residual.device)
        if delta is None:
            ops.sandwich_norm32(residual, None, None, None, self.gain, out, self.eps, rows=rows)
        else:
            ops.sandwich_norm32(residual, delta.a, delta.bias, delta.gain, self.gain, out, self.eps, rows=rows)
        self.rt.record(self._name("out"), out)
        return out

    @staticmethod
    def settle(stream, delta: PendingNormed):
        """stream += norm(delta), with no norm behind it."""
        ops.sandwich_norm32(stream, delta.a, delta.bias, delta.gain, None, None, delta.eps)
        return stream


register_norm("rmsnorm", RMSNorm)
register_norm("rmsnorm_stream32", StreamRMSNorm)
register_norm("rmsnorm_scaled_stream32", ScaledStreamRMSNorm)
register_norm("rmsnorm_sandwich_stream32", SandwichStreamRMSNorm)
