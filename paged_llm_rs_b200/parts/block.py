"""The pre-norm residual block: x + mixer(norm(x)), then x + ff(norm(x))
(crates/pagedllm/src/model/mod.rs:117-135).  Each residual add is done by the
norm kernel that follows it: the block hands on the residual stream and the
addition that is still pending."""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import Block, register_block


class PreNormResidualBlock(Block):
    def pre_mixer(self, residual, delta):
        return self.norms["mixer"].add_norm(residual, delta)         # residual += delta, in place

    def post_mixer(self, residual, a, step):
        h = self.norms["feed_forward"].add_norm(residual, a)
        out = self.feed_forward.forward(h, step)
        rt = self.mixer.rt
        if rt.trace is not None and self.prefix:
            rt.record(f"{self.prefix}.out", residual + out)          # (otherwise formed by the next norm's kernel)
        return residual, out

    def forward(self, residual, delta, step, cache, writes_cache=True):
        h = self.pre_mixer(residual, delta)
        a = self.mixer.forward(h, step, cache, writes_cache)
        return self.post_mixer(residual, a, step)


class OutputNormResidualBlock(Block):
    """x + norm(mixer(x)), then x + norm(ff(x)): the norm sits on each sublayer's output and the
    sublayers read the stream itself.  The stream is float32 and is added to in place; what is
    handed on beside it is its rounding to the compute dtype (None before the first block, the
    stream itself in a float32 engine), not a pending addition.  A layer may have no feed-forward.
    Its norms are ``StreamRMSNorm``s."""

    def forward(self, stream, rounded, step, cache, writes_cache=True):
        rt = self.mixer.rt
        if rounded is None:
            rounded = stream if rt.dtype == torch.float32 else ops.round_rows(stream, rt.dtype)
        a = self.mixer.forward(rounded, step, cache, writes_cache)
        rounded = self.norms["mixer"].add_into(stream, a)
        if self.feed_forward is not None:
            f = self.feed_forward.forward(rounded, step)
            rounded = self.norms["feed_forward"].add_into(stream, f)
        if rt.trace is not None and self.prefix:
            rt.record(f"{self.prefix}.out", stream)
        return stream, rounded

    def settle(self, stream, rounded):
        return stream, None


class PreNormStreamBlock(Block):
    """x + m mixer(norm(x)), then x + m ff(norm(x)), on a float32 stream: the pre-norm block with its norms
    ``ScaledStreamRMSNorm``s, which add the pending sublayer output (times the model's constant m) into the stream
    and norm the sum into the compute dtype in one kernel.  A layer may have no feed-forward: the mixer's output is
    then what is handed on."""

    def pre_mixer(self, stream, delta):
        return self.norms["mixer"].add_norm(stream, delta)

    def post_mixer(self, stream, a, step):
        out = a
        if self.feed_forward is not None:
            out = self.feed_forward.forward(self.norms["feed_forward"].add_norm(stream, a), step)
        rt = self.mixer.rt
        if rt.trace is not None and self.prefix:
            rt.record(f"{self.prefix}.out", stream + self.norms["mixer"].mult * out.float())
        return stream, out

    def forward(self, stream, delta, step, cache, writes_cache=True):
        h = self.pre_mixer(stream, delta)
        a = self.mixer.forward(h, step, cache, writes_cache)
        return self.post_mixer(stream, a, step)


class SandwichStreamBlock(Block):
    """x + norm_b(mixer(norm_a(x))), then x + norm_d(ff(norm_c(x))), on a float32 stream: every sublayer is normed on the way
    in and on the way out.  Its norms are ``SandwichStreamRMSNorm``s named "mixer", "mixer_out", "feed_forward" and
    "feed_forward_out"; what is handed on beside the stream is the last sublayer's output wrapped by its output norm, so
    that ONE kernel norms it, adds it and norms the sum for the next sublayer.  A feed-forward with a bias on its last
    product leaves that bias to the same kernel.  A layer may have no feed-forward."""

    def pre_mixer(self, stream, pending):
        return self.norms["mixer"].add_norm(stream, pending)

    def post_mixer(self, stream, a, step):
        pending = self.norms["mixer_out"].pending(a)
        if self.feed_forward is not None:
            h = self.norms["feed_forward"].add_norm(stream, pending)
            if hasattr(self.feed_forward, "forward_deferred"):
                f, bias = self.feed_forward.forward_deferred(h, step)
            else:
                f, bias = self.feed_forward.forward(h, step), None
            pending = self.norms["feed_forward_out"].pending(f, bias)
        rt = self.mixer.rt
        if rt.trace is not None and self.prefix:
            x = stream.clone()
            self.norms["mixer_out"].settle(x, pending)
            rt.record(f"{self.prefix}.out", x)
        return stream, pending

    def forward(self, stream, pending, step, cache, writes_cache=True):
        h = self.pre_mixer(stream, pending)
        a = self.mixer.forward(h, step, cache, writes_cache)
        return self.post_mixer(stream, a, step)


register_block("prenorm_residual", PreNormResidualBlock)
register_block("prenorm_stream32", PreNormStreamBlock)
register_block("outnorm_residual", OutputNormResidualBlock)
register_block("sandwich_stream32", SandwichStreamBlock)
