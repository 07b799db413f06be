"""A mixture of gated feed-forward experts behind a softmax router.

Per token, with h the input (all router arithmetic in float32):

    s = softmax(W_r h)                       over every router output
    choice = s + correction                  the correction steers the choice only
    outputs form ``groups`` equal groups of neighbours; a group scores its largest choice;
    only outputs of the ``keep`` best groups can be chosen
    the ``top`` largest choices are taken; weight_k = s_k / (sum of the chosen s + 1e-20)
    out = sum_k weight_k * E_k(h)  (+ S(h))

E_k is expert k's down(act(gate h, up h)), act(g, u) = silu(g) * u unless ``activation`` (with
``limit``) names another gated activation; the LAST ``identity`` router outputs have no
tensors and return h itself; S is an optional expert of the same form (``shared_activation``,
``shared_limit``) that every token uses.

Options for routers of another make: ``router_bias`` adds a learned vector to W_r h before the
softmax; without a correction the choice is then by the largest logits and the weights are the
softmax over the chosen logits alone (s_k over the sum of the chosen s is exactly that).
``shared_gate`` multiplies S(h) by sigmoid(w_sg . h), one number a token; w_sg rides as one more
row of the router's float32 matrix.

Options for experts of another make: ``scoring`` "sigmoid" scores each router output by the sigmoid of its logit instead of
the softmax over all; ``renormalize`` False keeps the chosen scores themselves as weights; ``gated`` False makes every expert
(and the shared one) down(act(up h)) with a one-argument ``activation`` ("squared_relu": max(., 0)^2) and no gate tensors;
``weight_on`` "input" lets a chosen expert read the token TIMES its weight, out = sum_k E_k(weight_k h), instead of
weighting what it returns.  Counts, sizes and tensor leaves are parameters.  The router and the experts are kernels of
this library (csrc/moe.cu); the shared expert runs as the dense gated feed-forward does.
"""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import FeedForward, register_feed_forward
from .spec import TensorSpec


class RoutedExperts(FeedForward):
    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        p = spec.params
        self.hidden, self.ff = int(p["hidden_size"]), int(p["expert_size"])
        self.experts, self.identity, self.top = int(p["experts"]), int(p.get("identity", 0)), int(p["top"])
        self.groups, self.keep = int(p.get("groups", 1)), int(p.get("keep", 1))
        self.shared_ff = p.get("shared_size")
        self.corrected = bool(p.get("correction", True))
        self.router_bias, self.shared_gate = bool(p.get("router_bias", False)), bool(p.get("shared_gate", False))
        self.scoring, self.renormalize = p.get("scoring", "softmax"), bool(p.get("renormalize", True))
        self.gated, self.weight_input = bool(p.get("gated", True)), p.get("weight_on", "output") == "input"
        if self.scoring not in ops.ROUTER_SCORINGS or p.get("weight_on", "output") not in ("output", "input"):
            raise ValueError(f"scoring {self.scoring!r} / weight_on {p.get('weight_on')!r} are not known")
        self.activation, self.limit = p.get("activation", "silu"), float(p.get("limit", 0.0))
        self.shared_activation, self.shared_limit = p.get("shared_activation", self.activation), float(p.get("shared_limit", self.limit))
        if self.shared_gate and not self.shared_ff:
            raise ValueError("shared_gate without a shared expert")
        for a in (self.activation, self.shared_activation):
            if a not in (ops.GLU_KINDS if self.gated else ops.UNARY_KINDS):
                raise ValueError(f"activation {a!r} is not known for experts {'with' if self.gated else 'without'} a gate")
        outputs = self.experts + self.identity
        if outputs % self.groups or self.keep > self.groups or self.top > self.keep * (outputs // self.groups):
            raise ValueError(f"{outputs} router outputs, {self.groups} groups of which {self.keep} are kept, top {self.top}: "
                             "these do not fit together")
        self.names = dict(router="router", correction="correction", expert="e{}", gate="gate", up="up", down="down", shared="shared",
                          router_bias="router.b", shared_gate="sg")
        self.names.update(p.get("names", {}))
        self.w_router = self.correction = self.w_gu = self.w_d = self.ws_gu = self.ws_d = self.bias = None

    def _expert(self, e: int, leaf: str) -> str:
        return self._name(f"{self.names['expert'].format(e)}.{self.names[leaf]}")

    def _shared(self, leaf: str) -> str:
        return self._name(f"{self.names['shared']}.{self.names[leaf]}")

    def tensors(self):
        W, ff, outputs = self.hidden, self.ff, self.experts + self.identity
        t = [TensorSpec(self._name(self.names["router"]), (outputs, W), "matrix32")]
        if self.corrected:
            t.append(TensorSpec(self._name(self.names["correction"]), (outputs,), "offset"))
        if self.router_bias:
            t.append(TensorSpec(self._name(self.names["router_bias"]), (outputs,), "offset"))
        if self.shared_gate:
            t.append(TensorSpec(self._shared("shared_gate"), (1, W), "matrix32"))
        for e in range(self.experts):
            t += ([TensorSpec(self._expert(e, "gate"), (ff, W))] if self.gated else []) + [
                TensorSpec(self._expert(e, "up"), (ff, W)), TensorSpec(self._expert(e, "down"), (W, ff))]
        if self.shared_ff:
            sf = int(self.shared_ff)
            t += ([TensorSpec(self._shared("gate"), (sf, W))] if self.gated else []) + [
                TensorSpec(self._shared("up"), (sf, W)), TensorSpec(self._shared("down"), (W, sf))]
        return t

    def bind(self, tensors):
        self.w_router = tensors[self._name(self.names["router"])]
        self.correction = tensors[self._name(self.names["correction"])] if self.corrected else None
        self.bias = tensors[self._name(self.names["router_bias"])] if self.router_bias else None
        if self.shared_gate:      # one more row of the router's matrix: its product leaves the router kernel as it is
            self.w_router = torch.cat([self.w_router, tensors[self._shared("shared_gate")]], 0).contiguous()
        # experts stacked: [E, 2 ff, W] (an expert's gate rows, then its up rows; without gates [E, ff, W]) and [E, W, ff]
        halves = ("gate", "up") if self.gated else ("up",)
        self.w_gu = torch.stack([torch.cat([tensors[self._expert(e, k)] for k in halves], 0)
                                 for e in range(self.experts)], 0).contiguous()
        self.w_d = torch.stack([tensors[self._expert(e, "down")] for e in range(self.experts)], 0).contiguous()
        if self.shared_ff:
            self.ws_gu = torch.cat([tensors[self._shared(k)] for k in halves], 0)
            self.ws_d = tensors[self._shared("down")]

    def forward(self, x, step):
        st = self.rt.status
        routed = ops.moe_route(x, self.w_router, self.correction, self.top, self.groups, self.keep, bias=self.bias,
                               extra=1 if self.shared_gate else 0, scoring=self.scoring, renormalize=self.renormalize)
        ids, weights = routed[0], routed[1]
        gate = routed[2].view(-1) if self.shared_gate else None
        shared = None
        if self.shared_ff:
            first = ops.linear_glu(x, self.ws_gu, status=st, act=self.shared_activation, limit=self.shared_limit) if self.gated \
                else ops.linear_act(x, self.ws_gu, self.shared_activation, status=st)
            shared = ops.linear(first, self.ws_d, status=st)
        out = ops.moe_experts(x, ids, weights, self.w_gu, self.w_d, shared, st, act=self.activation, limit=self.limit,
                              shared_gate=gate, gated=self.gated, weight_input=self.weight_input)
        if self.rt.trace is not None:
            self.rt.record(self._name("router.ids"), ids)
            self.rt.record(self._name("router.weights"), weights)
            self.rt.record(self._name("out"), out)
        return out


register_feed_forward("routed_experts", RoutedExperts)
