"""Recurrent mixers whose state is one matrix a head, carried from token to token in float32 (a ``StateNeed`` slot a
request).  With h the mixer's input, S a head's matrix (key entries by value entries):

``matrix_lstm`` (the matrix memory of the xLSTM):

    q = W_q h * dim^(-1/2)    k = W_k h    v = W_v h                       (heads x dim, heads x dim, heads x vdim)
    i = cap tanh((W_i h + b_i) / cap)    f = logsigmoid(cap tanh((W_f h + b_f) / cap))     one of each a head, logarithms
    m' = max(f + m, i)                   a running maximum, zero at the start
    S' = exp(f + m - m') S + exp(i - m') k v^T        n' = exp(f + m - m') n + exp(i - m') k
    o  = S'^T q / (max(|n' . q|, exp(-m')) + 1e-6)
    out = W_o (o / rms(o) a head * gain * sigmoid(W_g h))                  gain: heads * vdim entries

``gated_delta_rule``:

    q = W_q h, k = W_k h (kv_heads x dim), v = W_v h (heads x vdim); head a uses q/k head a // (heads / kv_heads)
    q, k, v <- silu(conv(.))             a causal convolution of ``conv`` taps a channel, no bias, zeros before the start
    q <- q / sqrt(sum q^2 + 1e-6) * dim^(-1/2)        k <- k / sqrt(sum k^2 + 1e-6)       a head
    beta = sigmoid(W_b h)    g = exp(-exp(A_log) softplus(W_a h + dt_bias))                 one of each a head
    S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q          (o is read after the update)
    out = W_o (o / rms(o) a head * gain * silu(W_g h))                     gain: vdim entries, shared by the heads

The gates' and step sizes' projections leave in float32; everything from there to the output projection's input is
float32 whatever the compute dtype.  A step's requests are found through its segment list on the device, so a captured
step replays with any requests; the slot also keeps each convolution channel's last taps - 1 inputs.
"""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import Mixer, StateNeed, register_mixer
from .spec import TensorSpec


class MatrixLSTM(Mixer):
    graph_safe = True

    def __init__(self, spec, rt, position_encodings=None):
        super().__init__(spec, rt)
        p = spec.params
        self.hidden, self.heads, self.dim, self.vdim = int(p["hidden_size"]), int(p["heads"]), int(p["dim"]), int(p["vdim"])
        self.cap, self.eps = float(p["gate_cap"]), float(p["eps"])
        if not self.cap > 0:
            raise ValueError("gate_cap must be positive")
        self.names = dict(q="q", k="k", v="v", g="g", o="o", norm="norm", i="i", f="f", i_b="i.b", f_b="f.b")
        self.names.update(p.get("names", {}))
        self.w_in = self.w_gates = self.w_o = self.i_bias = self.f_bias = self.gain = None

    def tensors(self):
        n, W, H = self.names, self.hidden, self.heads
        return [TensorSpec(self._name(n["q"]), (H * self.dim, W)), TensorSpec(self._name(n["k"]), (H * self.dim, W)),
                TensorSpec(self._name(n["v"]), (H * self.vdim, W)), TensorSpec(self._name(n["g"]), (H * self.vdim, W)),
                TensorSpec(self._name(n["o"]), (W, H * self.vdim)), TensorSpec(self._name(n["norm"]), (H * self.vdim,), "gain"),
                TensorSpec(self._name(n["i"]), (H, W)), TensorSpec(self._name(n["f"]), (H, W)),
                TensorSpec(self._name(n["i_b"]), (H,), "offset"), TensorSpec(self._name(n["f_b"]), (H,), "offset")]

    def bind(self, tensors):
        t = lambda k: tensors[self._name(self.names[k])]
        self.w_in = torch.cat([t("q"), t("k"), t("v"), t("g")], 0).contiguous()
        self.w_gates = torch.cat([t("i"), t("f")], 0).contiguous()
        self.w_o, self.gain, self.i_bias, self.f_bias = t("o"), t("norm"), t("i_b"), t("f_b")

    def cache_need(self):
        return StateNeed((ops.mlstm_state_floats(self.heads, self.dim, self.vdim),), torch.float32)

    def forward(self, x, step, cache, writes_cache=True):
        st = self.rt.status
        u = ops.linear(x, self.w_in, status=st)
        gates = ops.linear(x, self.w_gates, out_dtype=torch.float32, status=st)
        y = torch.empty((x.shape[0], self.heads * self.vdim), dtype=x.dtype, device=x.device)
        ops.mlstm_mix(u, gates, self.i_bias, self.f_bias, self.cap, self.gain, step.segments, cache, y, self.heads, self.dim,
                      self.vdim, self.eps, max_segment_tokens=step.max_segment_tokens or 0)
        out = ops.linear(y, self.w_o, status=st)
        if self.rt.trace is not None:
            for leaf, t in (("in.out", u), ("gates", gates), ("o.in", y), ("out", out)):
                self.rt.record(self._name(leaf), t)
        return out


class GatedDeltaRule(Mixer):
    graph_safe = True

    def __init__(self, spec, rt, position_encodings=None):
        super().__init__(spec, rt)
        p = spec.params
        self.hidden, self.heads, self.kv_heads = int(p["hidden_size"]), int(p["heads"]), int(p["kv_heads"])
        self.dim, self.vdim, self.taps, self.eps = int(p["dim"]), int(p["vdim"]), int(p["conv"]), float(p["eps"])
        if self.heads % self.kv_heads:
            raise ValueError(f"{self.heads} heads do not group over {self.kv_heads} heads of q and k")
        if self.taps < 1:
            raise ValueError("the convolution has at least one tap")
        self.names = dict(q="q", k="k", v="v", g="g", o="o", norm="norm", b="b", a="a", a_log="A_log", dt_bias="dt_bias",
                          q_conv="q.conv", k_conv="k.conv", v_conv="v.conv")
        self.names.update(p.get("names", {}))
        self.w_in = self.w_ba = self.w_o = self.conv_w = self.a_log = self.dt_bias = self.gain = None

    def tensors(self):
        n, W, H, G = self.names, self.hidden, self.heads, self.kv_heads
        qk, v = G * self.dim, H * self.vdim
        return [TensorSpec(self._name(n["q"]), (qk, W)), TensorSpec(self._name(n["k"]), (qk, W)), TensorSpec(self._name(n["v"]), (v, W)),
                TensorSpec(self._name(n["g"]), (v, W)), TensorSpec(self._name(n["o"]), (W, v)),
                TensorSpec(self._name(n["q_conv"]), (qk, self.taps)), TensorSpec(self._name(n["k_conv"]), (qk, self.taps)),
                TensorSpec(self._name(n["v_conv"]), (v, self.taps)), TensorSpec(self._name(n["b"]), (H, W)),
                TensorSpec(self._name(n["a"]), (H, W)), TensorSpec(self._name(n["a_log"]), (H,), "offset"),
                TensorSpec(self._name(n["dt_bias"]), (H,), "offset"), TensorSpec(self._name(n["norm"]), (self.vdim,), "gain")]

    def bind(self, tensors):
        t = lambda k: tensors[self._name(self.names[k])]
        self.w_in = torch.cat([t("q"), t("k"), t("v"), t("g")], 0).contiguous()
        self.w_ba = torch.cat([t("b"), t("a")], 0).contiguous()
        self.conv_w = torch.cat([t("q_conv"), t("k_conv"), t("v_conv")], 0).contiguous()
        self.w_o, self.gain, self.a_log, self.dt_bias = t("o"), t("norm"), t("a_log"), t("dt_bias")

    def cache_need(self):
        return StateNeed((ops.delta_state_floats(self.heads, self.kv_heads, self.dim, self.vdim, self.taps),), torch.float32)

    def forward(self, x, step, cache, writes_cache=True):
        st = self.rt.status
        u = ops.linear(x, self.w_in, status=st)
        ba = ops.linear(x, self.w_ba, out_dtype=torch.float32, status=st)
        y = torch.empty((x.shape[0], self.heads * self.vdim), dtype=x.dtype, device=x.device)
        ops.delta_mix(u, self.conv_w, ba, self.a_log, self.dt_bias, self.gain, step.segments, step.max_segment_tokens or step.n_tokens,
                      cache, y, self.heads, self.kv_heads, self.dim, self.vdim, self.taps, self.eps)
        out = ops.linear(y, self.w_o, status=st)
        if self.rt.trace is not None:
            for leaf, t in (("in.out", u), ("ba", ba), ("o.in", y), ("out", out)):
                self.rt.record(self._name(leaf), t)
        return out


register_mixer("matrix_lstm", MatrixLSTM)
register_mixer("gated_delta_rule", GatedDeltaRule)
