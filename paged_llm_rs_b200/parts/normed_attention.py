"""Grouped-query attention whose queries and keys are normed before the scores, with the options that designs of this
family combine.

With h the mixer's input, per token at position p and query head a (kv head a // (heads / kv_heads)):

    q = W_q h     k = W_k h     v = W_v h, or (``values_are_keys``) no W_v: v is the raw W_k h
    q, k <- norm(q), norm(k)          ``qk_norm``: "head" (each head over its own root mean square, one gain of key_dim
                                      entries shared by the heads), "projection" (all heads of q at once, and all of k,
                                      a gain of the projection's size) or None
    q <- q * (1 + temp_coef * ln(floor((p + 1) / temp_every) + 1))          (``temp_every`` 0: no such factor)
    q, k <- rot_p(q), rot_p(k)        the first ``rot_dims`` entries of a head, entry i with entry i + rot_dims / 2, by
                                      the angle p * rot_base^(-2i / rot_dims); 0: no rotation
    weight(p, j) = exp(scale q . k_j) / (sink + sum over j' <= p of exp(scale q . k_j'))
                                      ``sink_one``: sink = 1 = exp(0), as if one more key scored zero and carried nothing; else 0
    out = W_o ([sum over j <= p of weight(p, j) v_j]_a * sigmoid(W_g h)_a)  (``gate`` None: no such factor)

A token's key and value lie side by side in one cache row (``JoinedKVNeed``); the attention itself is the kernel of the
windowed attention with sinks, run without window and cap.  Norms, the temperature, angles, scores and weights are
float32 whatever the compute dtype.
"""

from __future__ import annotations

import numpy as np
import torch

from ..errors import KernelError
from ..kernels import ops
from .base import JoinedKVNeed, Mixer, PlanWish, register_mixer
from .spec import TensorSpec


class NormedQKAttention(Mixer):
    graph_safe = True

    def __init__(self, spec, rt, position_encodings=None):
        super().__init__(spec, rt)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.nh, self.nkv = int(p["num_heads"]), int(p["num_kv_heads"])
        self.dk, self.dv = int(p["key_dim"]), int(p["value_dim"])
        self.scale, self.eps = float(p["scale"]), float(p["eps"])
        self.qk_norm = p.get("qk_norm")
        self.values_are_keys = bool(p.get("values_are_keys", False))
        self.rot, self.rot_base = int(p.get("rot_dims") or 0), float(p.get("rot_base", 10000.0))
        self.temp_coef, self.temp_every = float(p.get("temp_coef") or 0.0), int(p.get("temp_every") or 0)
        self.sink_one = bool(p.get("sink_one", False))
        self.gate = p.get("gate")
        if self.qk_norm not in ops.QK_NORMS:
            raise ValueError(f"qk_norm {self.qk_norm!r}: one of {list(ops.QK_NORMS)}")
        if self.gate not in (None,) + tuple(ops.GATE_KINDS):
            raise ValueError(f"gate {self.gate!r}: None or one of {sorted(ops.GATE_KINDS)}")
        if self.nh % self.nkv:
            raise ValueError(f"{self.nh} heads do not group over {self.nkv} kv heads")
        if self.rot % 2 or self.rot > self.dk:
            raise ValueError(f"rot_dims {self.rot} must be even and at most key_dim {self.dk}")
        if self.values_are_keys and self.dv != self.dk:
            raise ValueError(f"the keys are the values, so value_dim {self.dv} must equal key_dim {self.dk}")
        if max(self.dk, self.dv) > 256:
            raise KernelError(f"key_dim {self.dk} / value_dim {self.dv}: the attention kernel takes sizes up to 256")
        self.names = dict(q="q", k="k", v="v", o="o", g="g", q_norm="q.norm", k_norm="k.norm")
        self.names.update(p.get("names", {}))
        self.w_in = self.w_o = self.q_gain = self.k_gain = self.inv_freq = self.sinks = None
        self.k_off = self.nh * self.dk
        self.v_off = self.k_off + self.nkv * self.dk
        self.g_off = self.v_off + (0 if self.values_are_keys else self.nkv * self.dv)
        self._need = None

    def _stacked(self):
        return ["q", "k"] + ([] if self.values_are_keys else ["v"]) + (["g"] if self.gate else [])

    def tensors(self):
        n, W = self.names, self.hidden
        rows = dict(q=self.nh * self.dk, k=self.nkv * self.dk, v=self.nkv * self.dv, g=self.nh * self.dv)
        t = [TensorSpec(self._name(n[k]), (rows[k], W)) for k in self._stacked()]
        t.append(TensorSpec(self._name(n["o"]), (W, self.nh * self.dv)))
        if self.qk_norm is not None:
            sizes = (self.dk, self.dk) if self.qk_norm == "head" else (self.nh * self.dk, self.nkv * self.dk)
            t += [TensorSpec(self._name(n["q_norm"]), (sizes[0],), "gain"), TensorSpec(self._name(n["k_norm"]), (sizes[1],), "gain")]
        return t

    def bind(self, tensors):
        n = self.names
        self.w_in = torch.cat([tensors[self._name(n[k])] for k in self._stacked()], 0).contiguous()
        self.w_o = tensors[self._name(n["o"])]
        if self.qk_norm is not None:
            self.q_gain, self.k_gain = tensors[self._name(n["q_norm"])], tensors[self._name(n["k_norm"])]
        if self.rot:
            f = np.power(np.float64(self.rot_base), -2.0 * np.arange(self.rot // 2, dtype=np.float64) / self.rot)
            self.inv_freq = torch.from_numpy(f.astype(np.float32)).to(self.w_o.device)
        if self.sink_one:
            self.sinks = torch.zeros(self.nh, dtype=torch.float32, device=self.w_o.device)      # exp(0) in the denominator

    def cache_need(self):
        if self._need is None:
            self._need = JoinedKVNeed("full", self.nkv, self.dk, self.dv, None, 0, group_size=self.nh // self.nkv)
        return self._need

    def plan_wish(self, page_size: int):
        a = (self.nh, self.nkv, self.rt.dtype, self.dk, self.dv)
        return PlanWish(ops.attention_sink_tile_tokens(*a), ops.attention_sink_ctas_per_item(*a), self.nh, self.dv)

    def forward(self, x, step, cache, writes_cache=True):
        kv_pool, gi = cache
        g = step.groups[gi]
        T, st = x.shape[0], self.rt.status
        proj = ops.linear(x, self.w_in, status=st)
        q = torch.empty((T, self.nh * self.dk), dtype=x.dtype, device=x.device)
        ops.normed_qk_kv_write(proj, self.k_off, self.v_off, q, self.q_gain, self.k_gain, self.qk_norm, self.eps, self.temp_coef,
                               self.temp_every, self.inv_freq, self.rot, step.positions, g.slots, kv_pool if writes_cache else None,
                               self.nh, self.nkv, self.dk, self.dv, self.values_are_keys, st)
        o = torch.empty((T, self.nh * self.dv), dtype=x.dtype, device=x.device)
        ops.attention_sink(q, kv_pool, g.block_tables, g.plan, o, self.sinks, self.nh, self.nkv, self.dk, self.dv, 0, 0,
                           self.scale, 0.0, st)
        if self.gate:
            ops.gate_mul(o, proj[:, self.g_off:self.g_off + self.nh * self.dv], self.gate)
        out = ops.linear(o, self.w_o, status=st)
        if self.rt.trace is not None:
            for leaf, t in (("q.normed", q), ("o.in", o), ("out", out)):
                self.rt.record(self._name(leaf), t)
        return out


register_mixer("normed_qk_attention", NormedQKAttention)
