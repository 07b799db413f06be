"""Latent attention: keys and values of every head are linear in ONE cached row a token.

With h the mixer's input, per token

    c_q = norm(W_dq h) g_q          q_a = W_uq c_q  (head a: ``dim`` values)
    c   = norm(W_dkv h) g_kv        k_a = W_uk,a c     v_a = W_uv,a c
    score(i, j, a) = scale * q_a(i) . k_a(j),   causal softmax over j <= i,   out = W_o [sum_j p v_a(j)]_a

Only c (``kv_rank`` values a token) is kept between steps, as rows of a paged pool (``RowNeed``).
The products with W_uk and W_uv are moved across the sum over cached tokens, which changes no
value beyond rounding:

    q~_a(i) = W_uk,a^T q_a(i)              (kv_rank values a head)
    score   = scale * q~_a(i) . c(j)
    o~_a(i) = sum_j p(i, j, a) c(j)        (kv_rank values a head)
    out     = W_o [ W_uv,a o~_a(i) ]_a

so that every head attends over the same rows c(j): attention with one shared key/value head of
size kv_rank whose keys ARE its values, in prompt portions and in decoding alike, and a cached
token costs kv_rank values whatever the number of heads.  There is no position encoding inside
the mixer.  Sizes, the scale and the norms' eps are parameters.
"""

from __future__ import annotations

import os

import torch

from ..errors import KernelError
from ..kernels import ops
from .base import Mixer, PlanWish, RowNeed, register_mixer
from .spec import TensorSpec


# For the few rows of a decode step in bfloat16 the per-head products are folded into their neighbours ahead of time:
# q~ = (W_uk^T W_uq) c_q and out = (W_o W_uv) o~, each ONE weight-streaming product instead of a product and a batched
# product: two launches fewer a layer, at heads x kv_rank x (q_rank + width) further weights (formed in float32, rounded
# once).  Prompt portions keep the unfolded products, which cost fewer multiplications.  PAGED_LLM_LATENT_FOLD=0: never.
FOLD_FOR_FEW_ROWS = os.environ.get("PAGED_LLM_LATENT_FOLD", "1") != "0"


class LatentAttention(Mixer):
    graph_safe = True

    def __init__(self, spec, rt, position_encodings=None):
        super().__init__(spec, rt)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.heads, self.dim, self.vdim = int(p["heads"]), int(p["dim"]), int(p["vdim"])
        self.q_rank, self.kv_rank = int(p["q_rank"]), int(p["kv_rank"])
        self.scale, self.eps = float(p["scale"]), float(p["eps"])
        # tensor leaves under the prefix: down / up projections, their norms' gains, the output projection
        self.names = dict(dq="dq", dq_norm="dq.norm", uq="uq", dkv="dkv", dkv_norm="dkv.norm", uk="uk", uv="uv", o="o")
        self.names.update(p.get("names", {}))
        self.w_down = self.w_uq = self.w_uk = self.w_uv = self.w_o = self.g_q = self.g_kv = None
        self.w_quk = self.w_ov = None          # the folded weights of decode steps (bfloat16 only)
        self._need = None

    def tensors(self):
        n, H, W = self.names, self.heads, self.hidden
        return [TensorSpec(self._name(n["dq"]), (self.q_rank, W)), TensorSpec(self._name(n["dq_norm"]), (self.q_rank,), "gain"),
                TensorSpec(self._name(n["uq"]), (H * self.dim, self.q_rank)),
                TensorSpec(self._name(n["dkv"]), (self.kv_rank, W)), TensorSpec(self._name(n["dkv_norm"]), (self.kv_rank,), "gain"),
                TensorSpec(self._name(n["uk"]), (H * self.dim, self.kv_rank)),
                TensorSpec(self._name(n["uv"]), (H * self.vdim, self.kv_rank)),
                TensorSpec(self._name(n["o"]), (W, H * self.vdim))]

    def bind(self, tensors):
        n, H = self.names, self.heads
        t = lambda k: tensors[self._name(n[k])]
        self.w_down = torch.cat([t("dq"), t("dkv")], 0).contiguous()         # one product makes both latents
        self.w_uq, self.w_o = t("uq"), t("o")
        self.g_q, self.g_kv = t("dq_norm"), t("dkv_norm")
        self.w_uk = t("uk").view(H, self.dim, self.kv_rank)                   # q~_a = q_a W_uk,a       [dim] x [dim, kv_rank]
        self.w_uv = t("uv").view(H, self.vdim, self.kv_rank).transpose(1, 2).contiguous()   # o_a = o~_a W_uv,a^T  [kv_rank, vdim]
        if FOLD_FOR_FEW_ROWS and self.rt.dtype == torch.bfloat16:
            uk, uq = self.w_uk.float(), self.w_uq.view(H, self.dim, self.q_rank).float()
            self.w_quk = torch.einsum("hdr,hdq->hrq", uk, uq).reshape(H * self.kv_rank, self.q_rank).to(self.rt.dtype).contiguous()
            o, uv = self.w_o.view(self.hidden, H, self.vdim).float(), t("uv").view(H, self.vdim, self.kv_rank).float()
            self.w_ov = torch.einsum("whv,hvr->whr", o, uv).reshape(self.hidden, H * self.kv_rank).to(self.rt.dtype).contiguous()

    def cache_need(self):
        if self._need is None:
            self._need = RowNeed(self.kv_rank, plan_key=(self.heads,))      # (work items are cut by the number of heads)
        return self._need

    def plan_wish(self, page_size: int):
        tile = ops.latent_attention_tile_tokens(self.heads, self.kv_rank, self.rt.dtype)
        return PlanWish(tile, ops.latent_attention_ctas_per_item(self.heads, self.kv_rank, self.rt.dtype), self.heads, self.kv_rank)

    def forward(self, x, step, cache, writes_cache=True):
        rows, gi = cache
        g = step.groups[gi]
        T, H, R = x.shape[0], self.heads, self.kv_rank
        st = self.rt.status
        qa = ops.linear(x, self.w_down, status=st)
        cq = torch.empty((T, self.q_rank), dtype=x.dtype, device=x.device)
        ops.latent_norm_write(qa, self.g_q, self.g_kv, self.eps, cq, rows if writes_cache else None, g.slots,
                              self.q_rank, R, st)
        if self.w_quk is not None and T <= ops.SKINNY_MAX_M:
            q_lat = ops.linear(cq, self.w_quk, status=st).view(T, H, R)
            o_lat = torch.empty_like(q_lat)
            ops.latent_attention(q_lat, rows, g.block_tables, g.plan, o_lat, self.scale, st)
            return ops.linear(o_lat.view(T, H * R), self.w_ov, status=st)
        q = ops.linear(cq, self.w_uq, status=st)
        # per head, batched over views [H, T, .] of tensors laid out [T, H, .] (what the attention kernel reads and writes)
        q_lat = torch.empty((T, H, R), dtype=x.dtype, device=x.device)
        torch.bmm(q.view(T, H, self.dim).transpose(0, 1), self.w_uk, out=q_lat.transpose(0, 1))
        o_lat = torch.empty_like(q_lat)
        ops.latent_attention(q_lat, rows, g.block_tables, g.plan, o_lat, self.scale, st)
        o = torch.empty((T, H * self.vdim), dtype=x.dtype, device=x.device)
        torch.bmm(o_lat.transpose(0, 1), self.w_uv, out=o.view(T, H, self.vdim).transpose(0, 1))
        out = ops.linear(o, self.w_o, status=st)
        if self.rt.trace is not None:
            for leaf, t in (("q", q), ("q_latent", q_lat), ("o_latent", o_lat), ("o.in", o), ("out", out)):
                self.rt.record(self._name(leaf), t)
        return out


class RotaryLatentAttention(Mixer):
    """Latent attention whose heads also share ONE rotated key part a token, gated a head.

    With h the mixer's input, per token at position p and head a:

        q_a = (W_q h)_a = [q_a' (dim) | q_a'' (rot_dim)]                 the second part is rotated
        [d (kv_rank) | r (rot_dim)] = W_dkv h;   c = d over its root mean square times a gain;   k'' = rot_p(r)
        k_a'(j) = W_uk,a c(j)     v_a(j) = W_uv,a c(j)
        score(p, j, a) = scale * (q_a' . k_a'(j) + rot_p(q_a'') . k''(j)),   causal softmax over j <= p
        out = W_o [ sigmoid(W_g h)_a * sum_j weight_j v_a(j) ]_a

    rot_p turns the first ``rot_dims`` entries of the rotated part pairwise (entry 2i with 2i + 1) by the angle
    p * rot_base^(-2i / rot_dims).  Only the row [c | k''] (kv_rank + rot_dim values a token) is kept between steps
    (``RowNeed``).  As in ``latent_attention`` the products with W_uk and W_uv are moved across the sum over cached tokens:
    the query row of a head is [W_uk,a^T q_a' | rot_p(q_a'')], every head attends over the same cache rows with the kernels of
    ``latent_attention`` (rows as keys and values at once), and W_uv,a is applied to the first kv_rank entries of the result.

    ``keeps``: "own" (the layer has W_dkv and writes its rows; ``hands_on`` names them for later layers of the step),
    "nothing" (it attends over an earlier layer's pages, which the schedule hands it: no W_dkv) or "copy" (no W_dkv either:
    it stores the rows that the layer named by ``copies`` handed on in pages of its own, because its work items differ)."""

    graph_safe = True

    def __init__(self, spec, rt, position_encodings=None):
        super().__init__(spec, rt)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.heads, self.dim, self.rot_dim, self.vdim = int(p["heads"]), int(p["dim"]), int(p.get("rot_dim") or 0), int(p["vdim"])
        self.kv_rank, self.scale, self.eps = int(p["kv_rank"]), float(p["scale"]), float(p["eps"])
        self.rot, self.rot_base = int(p.get("rot_dims") or 0), float(p.get("rot_base", 10000.0))
        self.gate = p.get("gate")
        self.keeps = p.get("keeps", "own")
        self.hands_on, self.copies = p.get("hands_on"), p.get("copies")
        if self.keeps not in ("own", "nothing", "copy"):
            raise ValueError(f"keeps {self.keeps!r}: 'own', 'nothing' or 'copy'")
        if self.keeps == "copy" and not self.copies:
            raise ValueError("a layer that keeps a copy names whose rows it copies")
        if self.rot % 2 or self.rot > self.rot_dim:
            raise ValueError(f"rot_dims {self.rot} must be even and at most rot_dim {self.rot_dim}")
        if self.gate not in (None, "sigmoid"):
            raise ValueError(f"gate {self.gate!r}: None or 'sigmoid'")
        self.width = self.kv_rank + self.rot_dim
        self.names = dict(q="q", dkv="dkv", dkv_norm="dkv.norm", uk="uk", uv="uv", o="o", g="g")
        self.names.update(p.get("names", {}))
        self.w_in = self.w_uk = self.w_uv = self.w_o = self.g_kv = self.inv_freq = None
        self.cq = self.heads * (self.dim + self.rot_dim)
        self.down_off = self.cq + (self.heads if self.gate else 0)
        self._need = None

    def tensors(self):
        n, H, W = self.names, self.heads, self.hidden
        t = [TensorSpec(self._name(n["q"]), (self.cq, W)), TensorSpec(self._name(n["uk"]), (H * self.dim, self.kv_rank)),
             TensorSpec(self._name(n["uv"]), (H * self.vdim, self.kv_rank)), TensorSpec(self._name(n["o"]), (W, H * self.vdim))]
        if self.gate:
            t.append(TensorSpec(self._name(n["g"]), (H, W)))
        if self.keeps == "own":
            t += [TensorSpec(self._name(n["dkv"]), (self.width, W)), TensorSpec(self._name(n["dkv_norm"]), (self.kv_rank,), "gain")]
        return t

    def bind(self, tensors):
        import numpy as np
        n, H = self.names, self.heads
        t = lambda k: tensors[self._name(n[k])]
        stacked = [t("q")] + ([t("g")] if self.gate else []) + ([t("dkv")] if self.keeps == "own" else [])
        self.w_in = torch.cat(stacked, 0).contiguous()               # one product makes q, the gates and the down-projection
        self.w_o = t("o")
        self.g_kv = t("dkv_norm") if self.keeps == "own" else None
        self.w_uk = t("uk").view(H, self.dim, self.kv_rank)                                   # q~_a = q_a' W_uk,a
        self.w_uv = t("uv").view(H, self.vdim, self.kv_rank).transpose(1, 2).contiguous()   # o_a = o~_a W_uv,a^T
        if self.rot:
            f = np.power(np.float64(self.rot_base), -2.0 * np.arange(self.rot // 2, dtype=np.float64) / self.rot)
            self.inv_freq = torch.from_numpy(f.astype(np.float32)).to(self.w_o.device)

    def cache_need(self):
        if self._need is None:
            self._need = RowNeed(self.width, plan_key=("rotary", self.heads))      # (work items are cut by the number of heads)
        return self._need

    def plan_wish(self, page_size: int):
        tile = ops.latent_attention_tile_tokens(self.heads, self.width, self.rt.dtype)
        return PlanWish(tile, ops.latent_attention_ctas_per_item(self.heads, self.width, self.rt.dtype), self.heads, self.width)

    def forward(self, x, step, cache, writes_cache=True):
        rows, gi = cache
        g = step.groups[gi]
        T, H, R = x.shape[0], self.heads, self.kv_rank
        st = self.rt.status
        proj = ops.linear(x, self.w_in, status=st)
        q = proj[:, :self.cq]
        q_rows = torch.empty((T, H, self.width), dtype=x.dtype, device=x.device)
        # per head, batched over views [H, T, .] of tensors laid out [T, H, .]
        torch.bmm(q.view(T, H, self.dim + self.rot_dim)[:, :, :self.dim].transpose(0, 1), self.w_uk, out=q_rows[:, :, :R].transpose(0, 1))
        down = row_out = carried = None
        if self.keeps == "own":
            down = proj[:, self.down_off:self.down_off + self.width]
            if self.hands_on:
                row_out = step.carry[self.hands_on] = torch.empty((T, self.width), dtype=x.dtype, device=x.device)
        elif self.keeps == "copy":
            carried = step.carry.get(self.copies)
            if carried is None:
                raise KernelError(f"{self.prefix}: keeps a copy of {self.copies!r}, but no earlier layer of the step handed it on")
        ops.latent_rope_write(down, self.g_kv, self.eps, q, q_rows, rows if writes_cache else None, g.slots, step.positions,
                              self.inv_freq, H, self.dim, self.rot_dim, self.rot, R, st, row_out=row_out, carried=carried)
        o_rows = torch.empty_like(q_rows)
        ops.latent_attention(q_rows, rows, g.block_tables, g.plan, o_rows, self.scale, st)
        o = torch.empty((T, H * self.vdim), dtype=x.dtype, device=x.device)
        torch.bmm(o_rows[:, :, :R].transpose(0, 1), self.w_uv, out=o.view(T, H, self.vdim).transpose(0, 1))
        if self.gate:
            ops.gate_mul(o, proj[:, self.cq:self.cq + H], self.gate, per=self.vdim)
        out = ops.linear(o, self.w_o, status=st)
        if self.rt.trace is not None:
            for leaf, t in (("q_rows", q_rows), ("o_rows", o_rows), ("o.in", o), ("out", out)):
                self.rt.record(self._name(leaf), t)
        return out


register_mixer("latent_attention", LatentAttention)
register_mixer("rotary_latent_attention", RotaryLatentAttention)
