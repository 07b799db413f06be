"""The gated feed-forward, down(act(gate(x), up(x))), act(g, u) = silu(g) * u
(crates/pagedllm/src/model/layers.rs:67-106) unless ``activation`` names another
gated activation of the kernels ("relu": max(g, 0) * u; "clamped", with ``limit``).
gate and up are one matrix product over the stacked weights, with the activation
in its epilogue for the few rows of a decode step and for the many of a prompt
portion, and as a kernel of its own otherwise."""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import FeedForward, register_feed_forward
from .spec import TensorSpec


class SwiGLUMLP(FeedForward):
    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.hidden = int(spec.params["hidden_size"])
        self.inter = int(spec.params["intermediate_size"])
        # the three tensors' leaves under the prefix (another checkpoint layout names them otherwise)
        self.names = dict(gate="gate_proj.weight", up="up_proj.weight", down="down_proj.weight")
        self.names.update(spec.params.get("names", {}))
        self.activation, self.limit = spec.params.get("activation", "silu"), float(spec.params.get("limit", 0.0))
        if self.activation not in ops.GLU_KINDS:
            raise ValueError(f"activation {self.activation!r} is not known; known: {sorted(ops.GLU_KINDS)}")
        # biases=True: every product has a bias, named by its matrix's leaf and ".b" (or names gate_b / up_b / down_b)
        self.biases = bool(spec.params.get("biases", False))
        if self.biases:
            for k in ("gate", "up", "down"):
                self.names.setdefault(f"{k}_b", self.names[k] + ".b")
        self.w_gate_up = self.w_down = self.b_gate_up = self.b_down = None

    def tensors(self):
        n = self.names
        return [TensorSpec(self._name(n["gate"]), (self.inter, self.hidden)),
                TensorSpec(self._name(n["up"]), (self.inter, self.hidden)),
                TensorSpec(self._name(n["down"]), (self.hidden, self.inter))] + ([
                    TensorSpec(self._name(n["gate_b"]), (self.inter,), "offset"), TensorSpec(self._name(n["up_b"]), (self.inter,), "offset"),
                    TensorSpec(self._name(n["down_b"]), (self.hidden,), "offset")] if self.biases else [])

    def bind(self, tensors):
        n = self.names
        self.w_gate_up = torch.cat([tensors[self._name(n["gate"])], tensors[self._name(n["up"])]], 0)
        self.w_down = tensors[self._name(n["down"])]
        if self.biases:
            self.b_gate_up = torch.cat([tensors[self._name(n["gate_b"])], tensors[self._name(n["up_b"])]], 0).contiguous()
            self.b_down = tensors[self._name(n["down_b"])]

    def forward_deferred(self, x, step):
        """(the last product's output without its bias, that bias or None): for a block whose next kernel adds it."""
        if not self.biases:
            return self.forward(x, step), None
        gu = ops.linear(x, self.w_gate_up, status=self.rt.status)
        act = ops.swiglu_bias(gu, self.b_gate_up, torch.empty((gu.shape[0], self.inter), dtype=gu.dtype, device=gu.device),
                              self.activation, self.limit)
        out = ops.linear(act, self.w_down, status=self.rt.status)
        if self.rt.trace is not None:
            self.rt.record(self._name("down.in"), act)
        return out, self.b_down

    def forward(self, x, step):
        if self.biases:
            out, bias = self.forward_deferred(x, step)
            return out.add_(bias.to(out.dtype))
        act = ops.linear_glu(x, self.w_gate_up, status=self.rt.status, act=self.activation, limit=self.limit)
        out = ops.linear(act, self.w_down, status=self.rt.status)
        if self.rt.trace is not None:
            self.rt.record(self._name("down_proj.in"), act)
            self.rt.record(self._name("down_proj.out"), out)
            self.rt.record(self._name("out"), out)
        return out


register_feed_forward("swiglu_mlp", SwiGLUMLP)
