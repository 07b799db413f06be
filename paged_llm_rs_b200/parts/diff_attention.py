"""Differential attention: every head takes TWO softmax maps over the same values and subtracts the second from the first.

With h the mixer's input, per token at position p, query head a (kv head a // (heads / kv_heads)) and map z in {1, 2}:

    q = W_q h + b_q    k = W_k h + b_k    v = W_v h + b_v          q: heads x 2 x key_dim, k: kv_heads x 2 x key_dim, laid out
                                                                   head by head as [map 1 | map 2]; v: kv_heads x value_dim
    q, k, v <- conv(.)                a causal convolution of ``conv`` taps a channel, no bias, zeros before the request's start
                                      (conv 0: none); the last conv - 1 inputs of a request are part of its state
    q, k <- rot_p(q), rot_p(k)        the first ``rot_dims`` entries of each map of each head, entry i with entry i + rot_dims / 2,
                                      by the angle p * rot_base^(-2i / rot_dims)
    A_z = softmax over the seen j of (scale q_z . k_z(j)) applied to v(j);   seen: 0 <= p - j < window (no window: j <= p)
    lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff                one number for the layer
    o = (A_1 - lambda A_2) over its root mean square, times (1 - diff), times sigmoid(W_g h)_a
    out = W_o [o]_a

The attention itself is the kernel of the windowed attention over joined key | value rows (``attention_sink``, without sink,
cap or kept tokens), run over 2 heads x 2 kv_heads: a map is a head of its own, and a kv head's row in the cache is doubled,
each copy a map's key followed by the same value.  For that the query heads are laid out [kv head][map][head of the group]
(W_q's rows are permuted once, when the weights are bound).  The convolution's state is a float32 slot a request
(``StateNeed``) beside the pages (``CompositeNeed``).  Biases, the convolution, angles, scores, weights, lambda, the
difference and its norm are float32 whatever the compute dtype.
"""

from __future__ import annotations

import math

import numpy as np
import torch

from ..errors import KernelError
from ..kernels import ops
from .base import CompositeNeed, JoinedKVNeed, Mixer, PlanWish, StateNeed, register_mixer
from .spec import TensorSpec

MAPS = 2


class DifferentialAttention(Mixer):
    graph_safe = True

    def __init__(self, spec, rt, position_encodings=None):
        super().__init__(spec, rt)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.nh, self.nkv = int(p["num_heads"]), int(p["num_kv_heads"])
        self.dk, self.dv = int(p["key_dim"]), int(p["value_dim"])
        self.scale, self.eps, self.diff = float(p["scale"]), float(p["eps"]), float(p["diff"])
        self.taps = int(p.get("conv") or 0)
        self.window = int(p.get("window") or 0)
        self.rot, self.rot_base = int(p.get("rot_dims") or 0), float(p.get("rot_base", 10000.0))
        self.biases = bool(p.get("biases", True))
        if self.nh % self.nkv:
            raise ValueError(f"{self.nh} heads do not group over {self.nkv} kv heads")
        if self.rot % 2 or self.rot > self.dk:
            raise ValueError(f"rot_dims {self.rot} must be even and at most key_dim {self.dk}")
        if max(self.dk, self.dv) > 256:
            raise KernelError(f"key_dim {self.dk} / value_dim {self.dv}: the attention kernel takes sizes up to 256")
        if self.taps > 16:
            raise KernelError(f"a convolution of {self.taps} taps: the kernel takes up to 16")
        self.group = self.nh // self.nkv
        self.cq, self.ck, self.cv = self.nh * MAPS * self.dk, self.nkv * MAPS * self.dk, self.nkv * self.dv
        self.channels = self.cq + self.ck + self.cv
        self.names = dict(q="q", k="k", v="v", o="o", g="g", q_b="q.b", k_b="k.b", v_b="v.b", q_conv="q.conv", k_conv="k.conv",
                          v_conv="v.conv", lq1="lq1", lk1="lk1", lq2="lq2", lk2="lk2")
        self.names.update(p.get("names", {}))
        self.w_in = self.w_o = self.bias = self.conv_w = self.inv_freq = None
        self.lam = 0.0
        # who owns each piece of the CompositeNeed: the pages' attention plan is this mixer's own wish
        self.parts = (self, self)
        self._need = None

    def tensors(self):
        n, W = self.names, self.hidden
        t = [TensorSpec(self._name(n["q"]), (self.cq, W)), TensorSpec(self._name(n["k"]), (self.ck, W)),
             TensorSpec(self._name(n["v"]), (self.cv, W)), TensorSpec(self._name(n["g"]), (self.nh, W)),
             TensorSpec(self._name(n["o"]), (W, self.nh * self.dv))]
        if self.biases:
            t += [TensorSpec(self._name(n["q_b"]), (self.cq,), "offset"), TensorSpec(self._name(n["k_b"]), (self.ck,), "offset"),
                  TensorSpec(self._name(n["v_b"]), (self.cv,), "offset")]
        if self.taps:
            t += [TensorSpec(self._name(n["q_conv"]), (self.cq, self.taps), "offset"),
                  TensorSpec(self._name(n["k_conv"]), (self.ck, self.taps), "offset"),
                  TensorSpec(self._name(n["v_conv"]), (self.cv, self.taps), "offset")]
        t += [TensorSpec(self._name(n[k]), (self.dk,), "offset") for k in ("lq1", "lk1", "lq2", "lk2")]
        return t

    def _query_order(self, device):
        """Row i of the permuted query projection is row order[i] of the stored one: stored head by head as [map 1 | map 2],
        wanted as [kv head][map][head of the group]."""
        g, z, a, e = np.meshgrid(np.arange(self.nkv), np.arange(MAPS), np.arange(self.group), np.arange(self.dk), indexing="ij")
        stored = ((g * self.group + a) * MAPS + z) * self.dk + e
        return torch.from_numpy(stored.reshape(-1).astype(np.int64)).to(device)

    def bind(self, tensors):
        n = self.names
        t = lambda k: tensors[self._name(n[k])]
        dev = t("o").device
        order = self._query_order(dev)
        self.w_in = torch.cat([t("q").index_select(0, order), t("k"), t("v"), t("g")], 0).contiguous()
        self.w_o = t("o")
        if self.biases:
            self.bias = torch.cat([t("q_b").index_select(0, order), t("k_b"), t("v_b")], 0).contiguous()
        if self.taps:
            self.conv_w = torch.cat([t("q_conv").index_select(0, order), t("k_conv"), t("v_conv")], 0).contiguous()
        else:
            self.conv_w = torch.ones((self.channels, 1), dtype=torch.float32, device=dev)
        d = lambda a, b: float((t(a).double() * t(b).double()).sum().item())
        self.lam = math.exp(d("lq1", "lk1")) - math.exp(d("lq2", "lk2")) + self.diff
        if self.rot:
            f = np.power(np.float64(self.rot_base), -2.0 * np.arange(self.rot // 2, dtype=np.float64) / self.rot)
            self.inv_freq = torch.from_numpy(f.astype(np.float32)).to(dev)

    def cache_need(self):
        if self._need is None:
            pages = JoinedKVNeed("window" if self.window else "full", self.nkv * MAPS, self.dk, self.dv, self.window or None, 0,
                                 group_size=self.group)
            self._need = CompositeNeed((pages, StateNeed((ops.conv_state_floats(self.channels, max(1, self.taps)),), torch.float32)))
        return self._need

    def plan_wish(self, page_size: int):
        a = (self.nh * MAPS, self.nkv * MAPS, self.rt.dtype, self.dk, self.dv)
        return PlanWish(ops.attention_sink_tile_tokens(*a), ops.attention_sink_ctas_per_item(*a), self.nh * MAPS, self.dv)

    def forward(self, x, step, cache, writes_cache=True):
        (kv_pool, gi), state = cache
        g = step.groups[gi]
        T, st = x.shape[0], self.rt.status
        proj = ops.linear(x, self.w_in, status=st)
        q = torch.empty((T, self.cq), dtype=x.dtype, device=x.device)
        ops.conv_rope_kv_write(proj, self.bias, self.conv_w, step.segments, step.max_segment_tokens or T, state, self.inv_freq, self.rot,
                               step.positions, g.slots, q, kv_pool if writes_cache else None, self.nh * MAPS, self.nkv * MAPS, MAPS,
                               self.dk, self.dv, st)
        a = torch.empty((T, self.nh * MAPS * self.dv), dtype=x.dtype, device=x.device)
        ops.attention_sink(q, kv_pool, g.block_tables, g.plan, a, None, self.nh * MAPS, self.nkv * MAPS, self.dk, self.dv, self.window, 0,
                           self.scale, 0.0, st)
        o = torch.empty((T, self.nh * self.dv), dtype=x.dtype, device=x.device)
        ops.diff_combine(a, proj[:, self.channels:self.channels + self.nh], o, self.nh, self.group, self.dv, self.lam, 1.0 - self.diff,
                         self.eps)
        out = ops.linear(o, self.w_o, status=st)
        if self.rt.trace is not None:
            for leaf, t in (("q.rotated", q), ("maps", a), ("o.in", o), ("out", out)):
                self.rt.record(self._name(leaf), t)
        return out


register_mixer("differential_attention", DifferentialAttention)
