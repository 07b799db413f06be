"""Pamarax on the GPU against the plain implementation (tests/plain_pamarax.py): each kernel and each mixer alone (through
the cache manager and the step packer, with inputs made so that one far key, a missing extra one in the softmax, a
temperature that steps a token early or a lost state would show), then whole models through the engine's step function,
cache manager, state slots and scheduler."""

import os
import random
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_pamarax as P
from pamarax_models import (CONFIGS, attention, dense, draw, layer, left, mixer_shapes, mlstm, model, parallel, right,
                            write_model)

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]
NAMES = {torch.float32: "float32", torch.bfloat16: "bfloat16"}
EPS = 1e-5


def ops_():
    from paged_llm_rs_b200.kernels import ops
    return ops


def close(got, want, dtype, what="", f32=2e-5, bf16=2e-2):
    got, want = got.double().cpu(), want.double().cpu()
    err = float((got - want).abs().max()) / max(1e-9, float(want.abs().max()))
    assert err < (f32 if dtype == torch.float32 else bf16), f"{what}: relative error {err}"


def status():
    return torch.zeros(1, dtype=torch.int32, device=DEV)


def gen(seed):
    return torch.Generator().manual_seed(seed)


# ------------------------------------------------------------------------ each kernel alone

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,width", [(1, 64), (5, 90), (300, 1024), (3, 4100), (2, 9000)])
def test_output_norm_sum_and_input_norm_in_one_pass(dtype, rows, width):
    ops = ops_()
    g = gen(0)
    x0 = torch.randn(rows, width, generator=g)
    a = (torch.randn(rows, width, generator=g) * 3).to(dtype)
    bias = torch.randn(width, generator=g)
    ga, gb = 1 + 0.2 * torch.randn(width, generator=g), 1 + 0.2 * torch.randn(width, generator=g)
    for b in (None, bias):
        ad = a.double() + (b.double() if b is not None else 0)
        summed = x0.double() + P.unit_rms(ad, EPS) * ga.double()
        normed = P.unit_rms(summed, EPS) * gb.double()
        bd = b.to(DEV) if b is not None else None
        # every row: the stream takes the sum
        x = x0.clone().to(DEV)
        y = torch.empty(rows, width, dtype=dtype, device=DEV)
        ops.sandwich_norm32(x, a.to(DEV), bd, ga.to(DEV), gb.to(DEV), y, EPS)
        close(x, summed, torch.float32, "stream", f32=1e-5)
        close(y, normed, dtype, "norm", bf16=8e-3)
        # some rows only: the sum is formed for them and not stored
        idx = torch.tensor([rows - 1, 0], dtype=torch.int32, device=DEV)
        x = x0.clone().to(DEV)
        y2 = torch.empty(2, width, dtype=dtype, device=DEV)
        ops.sandwich_norm32(x, a.to(DEV), bd, ga.to(DEV), gb.to(DEV), y2, EPS, rows=idx)
        assert torch.equal(x.cpu(), x0)
        close(y2, normed[[rows - 1, 0]], dtype, "norm of gathered rows", bf16=8e-3)
        # the sum alone, with no norm behind it
        x = x0.clone().to(DEV)
        ops.sandwich_norm32(x, a.to(DEV), bd, ga.to(DEV), None, None, EPS)
        close(x, summed, torch.float32, "sum alone", f32=1e-5)
    # nothing pending: the norm of the stream as it is
    y = torch.empty(rows, width, dtype=dtype, device=DEV)
    ops.sandwich_norm32(x0.to(DEV), None, None, None, gb.to(DEV), y, EPS)
    close(y, P.unit_rms(x0.double(), EPS) * gb.double(), dtype, "norm alone", bf16=8e-3)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,inter", [(3, 64), (70, 128), (5, 37), (300, 256)])
def test_gated_activation_with_biases_and_the_weighted_sum(dtype, rows, inter):
    ops = ops_()
    g = gen(1)
    gu = torch.randn(rows, 2 * inter, generator=g).to(dtype)
    bias = torch.randn(2 * inter, generator=g)
    out = torch.empty(rows, inter, dtype=dtype, device=DEV)
    ops.swiglu_bias(gu.to(DEV), bias.to(DEV), out)
    z = gu.double() + bias.double()
    close(out, P.silu(z[:, :inter]) * z[:, inter:], dtype, "activation with biases", bf16=1e-2)
    x, y = torch.randn(rows, inter, generator=g).to(dtype), torch.randn(rows, inter, generator=g).to(dtype)
    s = ops.scaled_sum2(x.to(DEV), y.to(DEV), 1.25, -0.4)
    close(s, 1.25 * x.double() - 0.4 * y.double(), dtype, "weighted sum", bf16=8e-3)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,nh,nkv,dk,dv,norm,rot,every,keys_as_values,page", [
    (9, 4, 2, 16, 16, "projection", 8, 0, True, 16), (40, 5, 5, 12, 20, "head", 0, 1, False, 8), (3, 8, 2, 64, 64, "projection", 64, 0, True, 16),
    (17, 20, 1, 32, 64, "head", 0, 4, False, 4), (6, 3, 3, 24, 8, None, 6, 3, False, 8), (5, 2, 1, 128, 128, "projection", 2, 0, True, 16)])
def test_qk_norm_temperature_rotation_and_the_cache_write(dtype, T, nh, nkv, dk, dv, norm, rot, every, keys_as_values, page):
    ops = ops_()
    g = gen(2)
    k_off, v_off = nh * dk, nh * dk + nkv * dk
    extra = 7                                                    # columns behind q | k | v that the kernel must not touch
    width = v_off + (0 if keys_as_values else nkv * dv) + extra
    proj = torch.randn(T, width, generator=g).to(dtype)
    sizes = {"projection": (nh * dk, nkv * dk), "head": (dk, dk), None: (0, 0)}[norm]
    qg, kg = 1 + 0.3 * torch.randn(sizes[0], generator=g), 1 + 0.3 * torch.randn(sizes[1], generator=g)
    base, coef = 77.0, 0.8
    inv_freq = torch.tensor([base ** (-2.0 * i / rot) for i in range(rot // 2)], dtype=torch.float64).float() if rot else None
    pos = torch.arange(30, 30 + T, dtype=torch.int32)
    n_pages = 8 + T // page
    slots = torch.randperm(n_pages * page, generator=g)[:T].to(torch.int32)
    slots[0] = -1                                                # a token whose row is not written
    pool = torch.full((n_pages, nkv, page, dk + dv), 7.0, dtype=dtype, device=DEV)
    q = torch.empty(T, nh * dk, dtype=dtype, device=DEV)
    st = status()
    ops.normed_qk_kv_write(proj.to(DEV), k_off, v_off, q, qg.to(DEV) if norm else None, kg.to(DEV) if norm else None, norm, EPS, coef, every,
                           inv_freq.to(DEV) if rot else None, rot, pos.to(DEV), slots.to(DEV), pool, nh, nkv, dk, dv, keys_as_values, st)
    assert st.item() == 0
    pd = proj.double()
    qq, kk = pd[:, :k_off], pd[:, k_off:v_off]
    vv = kk.view(T, nkv, dk) if keys_as_values else pd[:, v_off:v_off + nkv * dv].view(T, nkv, dv)
    if norm == "projection":
        qq, kk = P.unit_rms(qq, EPS) * qg.double(), P.unit_rms(kk, EPS) * kg.double()
    qq, kk = qq.view(T, nh, dk), kk.view(T, nkv, dk)
    if norm == "head":
        qq, kk = P.unit_rms(qq, EPS) * qg.double(), P.unit_rms(kk, EPS) * kg.double()
    if every:
        qq = qq * torch.tensor([1.0 + coef * np.log((int(p) + 1) // every + 1) for p in pos], dtype=torch.float64)[:, None, None]
    qq, kk = P.rotate_half(qq, pos.tolist(), rot, base), P.rotate_half(kk, pos.tolist(), rot, base)
    # the angle is a float32 product: at position p its error is about p * 6e-8
    close(q.view(T, nh, dk), qq, dtype, "q", f32=1e-4, bf16=2e-2)
    rows = pool.double().cpu().permute(0, 2, 1, 3).reshape(n_pages * page, nkv, dk + dv)
    for t in range(1, T):
        close(rows[slots[t], :, :dk], kk[t], dtype, "cached key", f32=1e-4, bf16=2e-2)
        assert torch.equal(rows[slots[t], :, dk:], vv[t]), "a value is stored as it was projected"
    untouched = torch.ones(n_pages * page, dtype=torch.bool)
    untouched[slots[1:].long()] = False
    assert bool((rows[untouched] == 7.0).all())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("kind", ["sigmoid", "silu"])
def test_gate_on_a_strided_view(dtype, kind):
    ops = ops_()
    g = gen(3)
    wide = torch.randn(33, 200, generator=g).to(dtype)
    y = torch.randn(33, 90, generator=g).to(dtype)
    got = ops.gate_mul(y.clone().to(DEV), wide.to(DEV)[:, 50:140], kind)
    z = wide.double()[:, 50:140]
    close(got, y.double() * (torch.sigmoid(z) if kind == "sigmoid" else P.silu(z)), dtype, "gate", bf16=1e-2)


# ------------------------------------------------------------------------ each mixer alone, through the cache manager

class MixerRig:
    """One mixer of a registered kind with the cache manager and the step packer the engine gives it: steps of
    (request, input rows [n, width]), several requests side by side; returns each request's output rows."""

    def __init__(self, kind, params, tensors, dtype, page=16, pages=64, max_requests=4):
        from paged_llm_rs_b200.cache.manager import CacheManager
        from paged_llm_rs_b200.engine.runner import group_plans
        from paged_llm_rs_b200.engine.step import StepPacker
        from paged_llm_rs_b200.parts import base, decoder  # noqa: F401  (registers the parts)
        from paged_llm_rs_b200.parts.spec import PartSpec
        self.dtype = dtype
        self.rt = base.Runtime(torch.device(DEV), dtype)
        self.mixer = base.make(base.MIXERS, "mixer", PartSpec(kind, params, "m"), self.rt)
        bound = {}
        for s in self.mixer.tensors():
            t = tensors[s.name]
            assert tuple(t.shape) == tuple(s.shape), s.name
            bound[s.name] = (t.to(dtype) if s.role == "matrix" else t.float()).to(DEV)
        self.mixer.bind(bound)
        self.cache = CacheManager([self.mixer.cache_need()], page, pages, max_requests, dtype, DEV, prefix_cache=False)
        of = lambda cell: self.mixer if not isinstance(cell, tuple) else self.mixer.parts[cell[1]]
        self.packer = StepPacker(self.cache, group_plans(self.cache, of, page), 296, 1000, 1 << 24, DEV)

    def step(self, entries):
        from paged_llm_rs_b200.engine.step import StepEntry
        es = []
        for rid, x in entries:
            if not self.cache.has(rid):
                self.cache.open(rid)
            assert self.cache.reserve(rid, x.shape[0]), "no pages left"
            es.append(StepEntry(rid, [0] * x.shape[0], []))
        host, layout, sizes = self.packer.pack(es)
        state = self.packer.to_state(torch.from_numpy(host).to(DEV), layout, sizes)
        x = torch.cat([x for _, x in entries]).to(self.dtype).to(DEV).contiguous()
        out = self.mixer.forward(x, state, self.cache.layer_caches()[0]).double().cpu()
        assert self.rt.status.item() == 0
        res, at = [], 0
        for rid, xi in entries:
            self.cache.commit(rid, xi.shape[0], None)
            res.append(out[at:at + xi.shape[0]])
            at += xi.shape[0]
        return res

    def end(self, rid):
        self.cache.close(rid)

    def cut(self, rid, x, cuts):
        """One request alone, its rows in portions."""
        assert sum(cuts) == x.shape[0]
        outs, at = [], 0
        for c in cuts:
            outs.append(self.step([(rid, x[at:at + c])])[0])
            at += c
        return torch.cat(outs)


def rounded(t, dtype):
    """What the engine is given: the compute dtype's rounding of t, as float64."""
    return t.to(dtype).double()


def attention_rig(dtype, m, W, seed, page=16, pages=64, craft=None):
    w = draw(mixer_shapes("attention", m, W, "m"), seed)
    if craft:
        craft(w)
    rot = m.get("rot") or {}
    params = dict(hidden_size=W, num_heads=m["heads"], num_kv_heads=m["kv_heads"], key_dim=m["dim"], value_dim=m["dim"], scale=m["scale"],
                  eps=EPS, qk_norm="projection", values_are_keys=True, rot_dims=rot.get("dims", 0), rot_base=rot.get("base", 1.0), gate="sigmoid")
    plain = {k.replace("m.", "L.mix.", 1): v.double() for k, v in w.items()}
    return MixerRig("normed_qk_attention", params, w, dtype, page, pages), lambda h: P.gated_attention_mixer(h, plain, "L", m, EPS)


def left_rig(dtype, m, W, seed, page=16, pages=64, craft=None):
    w = draw(mixer_shapes("left", m, W, "m"), seed)
    if craft:
        craft(w)
    qt = m.get("q_temp") or {}
    params = dict(hidden_size=W, num_heads=m["heads"], num_kv_heads=m["kv_heads"], key_dim=m["dim"], value_dim=m["vdim"], scale=m["scale"],
                  eps=EPS, qk_norm="head", temp_coef=qt.get("coef", 0.0), temp_every=qt.get("every", 0), sink_one=True)
    plain = {k: v.double() for k, v in w.items()}
    return MixerRig("normed_qk_attention", params, w, dtype, page, pages), lambda h: P.sink_attention_mixer(h, plain, "m", m, EPS)


def mlstm_rig(dtype, m, W, seed, max_requests=4):
    w = draw(mixer_shapes("mlstm", m, W, "m"), seed)
    params = dict(hidden_size=W, heads=m["heads"], dim=m["dim"], vdim=m["vdim"], gate_cap=m["gate_cap"], eps=EPS)
    plain = {k.replace("m.", "L.mix.", 1): v.double() for k, v in w.items()}
    return MixerRig("matrix_lstm", params, w, dtype, max_requests=max_requests), lambda h: P.mlstm_mixer(h, plain, "L", m, EPS)


def delta_rig(dtype, m, W, seed, max_requests=4):
    w = draw(mixer_shapes("right", m, W, "m"), seed)
    params = dict(hidden_size=W, heads=m["heads"], kv_heads=m["kv_heads"], dim=m["dim"], vdim=m["vdim"], conv=m["conv"], eps=EPS)
    plain = {k: v.double() for k, v in w.items()}
    return MixerRig("gated_delta_rule", params, w, dtype, max_requests=max_requests), lambda h: P.delta_mixer(h, plain, "m", m, EPS)


CUTS = [[75], [2] * 5 + [1, 1, 3, 17, 16, 20, 1, 1, 1, 1, 1, 1], [1] * 75, [40, 35], [64, 2, 9]]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv,dim,rot,base,W,page", [(4, 2, 16, 8, 100.0, 64, 16), (6, 1, 24, 0, 1.0, 90, 8), (3, 3, 12, 12, 50.0, 40, 4),
                                                           (8, 2, 64, 32, 1e4, 128, 16), (2, 1, 128, 64, 5e5, 96, 16)])
def test_gated_attention_whole_in_portions_and_token_by_token(dtype, heads, kv, dim, rot, base, W, page):
    m = attention(heads, kv, dim, rot=rot, base=base)["mixer"]
    x = rounded(torch.randn(75, W, generator=gen(10)), dtype)
    for cuts in CUTS:
        rig, plain = attention_rig(dtype, m, W, 11, page=page)
        close(rig.cut("r", x, cuts), plain(x), dtype, f"{cuts}", f32=1e-4, bf16=3e-2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv,dim,vdim,coef,every,W,page", [(4, 2, 16, 8, 0.3, 7, 64, 16), (5, 5, 12, 20, 1.0, 1, 90, 8), (20, 1, 32, 64, 0.0, 0, 128, 16),
                                                                  (8, 2, 64, 32, 2.0, 16, 128, 16), (3, 1, 24, 24, 4.0, 5, 48, 4)])
def test_attention_with_one_more_in_the_softmax_and_a_temperature(dtype, heads, kv, dim, vdim, coef, every, W, page):
    """The temperature steps at positions every - 1, 2 every - 1, ...: with a large coefficient a step taken one token early
    or late moves the output far beyond rounding, in a prompt's portion and in a decoded token, also on a page's border."""
    m = left(heads, kv, dim, vdim, coef=coef, every=every)
    x = rounded(torch.randn(75, W, generator=gen(12)), dtype)
    for cuts in CUTS:
        rig, plain = left_rig(dtype, m, W, 13, page=page)
        close(rig.cut("r", x, cuts), plain(x), dtype, f"{cuts}", f32=1e-4, bf16=3e-2)


def same_direction(w, heads, kv, dim, sign=1.0):
    """W_q of every head becomes sign * W_k of its kv head (plain gains): a token's query then points along (or against)
    the key of any token with the same input."""
    k = w["m.k"].view(kv, dim, -1)
    w["m.q"] = (sign * k.repeat_interleave(heads // kv, 0)).reshape(heads * dim, -1).contiguous()
    w["m.q.norm"], w["m.k.norm"] = torch.ones_like(w["m.q.norm"]), torch.ones_like(w["m.k.norm"])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("kind", ["gated", "extra_one"])
def test_one_far_key_decides(dtype, kind):
    """The last token's input is a third of that of ONE earlier token, and queries point along keys: after the q/k norm that
    key scores like the token's own, and its value is three times as large, so it decides the output wherever it lies: the first token, a page's last and first row, hundreds of tokens back, the token before
    and the token itself; in a decoded token, at the end of a portion and beside other requests."""
    W, heads, kv, dim, ctx = 64, 4, 2, 32, 420
    g = gen(14)
    base_x = torch.randn(ctx + 1, W, generator=g)
    for at in (0, 15, 16, 255, 256, ctx - 1, ctx):
        x = base_x.clone()
        x[at] = 3.0 * x[ctx]
        x = rounded(x, dtype)
        if kind == "gated":
            m = attention(heads, kv, dim, rot=4, base=1e4, scale=1.0)["mixer"]
            make = lambda: attention_rig(dtype, m, W, 15, pages=90, craft=lambda w: same_direction(w, heads, kv, dim))
        else:
            m = left(heads, kv, dim, 24, every=0, scale=1.0)
            make = lambda: left_rig(dtype, m, W, 15, pages=90, craft=lambda w: same_direction(w, heads, kv, dim))
        rig, plain = make()
        want = plain(x)
        # the reference itself: leaving the key out would change the last row by far more than the tolerance
        without = plain(torch.cat([x[:at], x[at + 1:]]))[-1] if at < ctx else None
        if without is not None:
            assert float((without - want[-1]).abs().max()) > 0.2 * float(want[-1].abs().max())
        got = rig.cut("a", x, [ctx, 1])
        close(got[-1:], want[-1:], dtype, f"decoded, key {at}", f32=1e-4, bf16=3e-2)
        rig, _ = make()
        got = rig.cut("b", x, [ctx - 20, 21])
        close(got[-1:], want[-1:], dtype, f"portion, key {at}", f32=1e-4, bf16=3e-2)
        rig, _ = make()
        other = rounded(torch.randn(40, W, generator=g), dtype)
        rig.step([("c", x[:ctx - 2]), ("d", other[:5])])
        res = rig.step([("d", other[5:6]), ("c", x[ctx - 2:]), ("e", other[6:])])
        close(res[1][-1:], want[-1:], dtype, f"batch, key {at}", f32=1e-4, bf16=3e-2)


@pytest.mark.parametrize("dtype", DTYPES)
def test_the_extra_one_takes_the_weight_when_every_score_is_low(dtype):
    """Queries point against every key: all scores are far below zero, the one in the denominator takes the weight and the
    output vanishes.  Without it the softmax would hand out all the weight and the output would be of the values' size."""
    W, heads, kv, dim, vdim = 48, 4, 2, 16, 8
    m = left(heads, kv, dim, vdim, every=0, scale=2.0)
    x = rounded(torch.randn(1, W, generator=gen(16)).repeat(30, 1), dtype)
    rig, plain = left_rig(dtype, m, W, 17, craft=lambda w: same_direction(w, heads, kv, dim, sign=-1.0))
    got, want = rig.cut("r", x, [13, 2, 14, 1]), plain(x)
    assert float(want.abs().max()) < 1e-6 and float(got.abs().max()) < 1e-4
    rig, plain = left_rig(dtype, m, W, 17, craft=lambda w: same_direction(w, heads, kv, dim, sign=1.0))
    got, want = rig.cut("r", x, [13, 2, 14, 1]), plain(x)
    assert float(want.abs().max()) > 0.1
    close(got, want, dtype, "scores far above zero", f32=1e-4, bf16=3e-2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,dim,vdim,cap,W", [(2, 8, 16, 10.0, 64), (3, 20, 12, 5.0, 90), (4, 64, 64, 15.0, 128), (1, 96, 8, 20.0, 48),
                                                   (6, 8, 24, 15.0, 48), (1, 256, 40, 15.0, 64), (2, 48, 48, 2.0, 72)])
def test_matrix_lstm_whole_in_portions_and_token_by_token(dtype, heads, dim, vdim, cap, W):
    m = mlstm(heads, dim, vdim, cap)["mixer"]
    x = rounded(torch.randn(75, W, generator=gen(18)) * 1.5, dtype)
    for cuts in CUTS:
        rig, plain = mlstm_rig(dtype, m, W, 19)
        close(rig.cut("r", x, cuts), plain(x), dtype, f"{cuts}", f32=1e-4, bf16=3e-2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv,dim,vdim,conv,W", [(4, 2, 8, 16, 3, 64), (3, 3, 20, 12, 2, 90), (4, 2, 64, 32, 4, 128), (2, 1, 128, 64, 5, 96),
                                                       (6, 1, 16, 24, 1, 48), (2, 2, 256, 16, 4, 64), (2, 1, 48, 40, 4, 72)])
def test_gated_delta_rule_whole_in_portions_and_token_by_token(dtype, heads, kv, dim, vdim, conv, W):
    m = right(heads, kv, dim, vdim, conv)
    x = rounded(torch.randn(75, W, generator=gen(20)) * 1.5, dtype)
    for cuts in CUTS:
        rig, plain = delta_rig(dtype, m, W, 21)
        close(rig.cut("r", x, cuts), plain(x), dtype, f"{cuts}", f32=1e-4, bf16=3e-2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("kind", ["mlstm", "delta"])
def test_recurrent_mixers_in_batches_with_slots_used_again_and_long_decoding(dtype, kind):
    """Three slots for five requests: requests of unequal length side by side, a finished request's slot taken by the next
    (whose state must start at zero), a request left out of a step, and one request decoded for 300 tokens."""
    W = 64
    if kind == "mlstm":
        rig, plain = mlstm_rig(dtype, mlstm(3, 16, 24, 8.0)["mixer"], W, 23, max_requests=3)
    else:
        rig, plain = delta_rig(dtype, right(4, 2, 16, 8, 3), W, 23, max_requests=3)
    g = gen(22)
    lengths = dict(a=330, b=33, c=7, d=64, e=21)
    xs = {k: rounded(torch.randn(n, W, generator=g) * 1.5, dtype) for k, n in lengths.items()}
    want = {k: plain(x) for k, x in xs.items()}
    got, at = {k: [] for k in xs}, {k: 0 for k in xs}

    def run(step):
        res = rig.step([(k, xs[k][at[k]:at[k] + n]) for k, n in step])
        for (k, n), r in zip(step, res):
            got[k].append(r); at[k] += n
            if at[k] == lengths[k]:
                rig.end(k)
    run([("a", 20), ("b", 2), ("c", 1)])
    run([("a", 1), ("b", 31), ("c", 6)])              # b and c end: two slots are free again
    run([("d", 17), ("a", 1)])
    run([("e", 2), ("d", 47)])                        # a is left out of this step
    run([("a", 8), ("e", 19)])
    for _ in range(300):
        run([("a", 1)])
    for k in xs:
        assert at[k] == lengths[k]
        close(torch.cat(got[k]), want[k], dtype, k, f32=2e-4, bf16=3e-2)


@pytest.mark.parametrize("dtype", DTYPES)
def test_mixers_side_by_side_alone(dtype):
    """The two halves through one mixer: pages for the left, a slot for the right, the constants on the sum."""
    from paged_llm_rs_b200.parts import decoder  # noqa: F401
    W = 72
    l, r = left(6, 3, 16, 8, coef=0.7, every=9), right(4, 2, 8, 16, conv=3)
    w = dict(draw(mixer_shapes("left", l, W, "m.left"), 30), **draw(mixer_shapes("right", r, W, "m.right"), 31))
    lp = dict(hidden_size=W, num_heads=6, num_kv_heads=3, key_dim=16, value_dim=8, scale=l["scale"], eps=EPS, qk_norm="head",
              temp_coef=0.7, temp_every=9, sink_one=True)
    rp = dict(hidden_size=W, heads=4, kv_heads=2, dim=8, vdim=16, conv=3, eps=EPS)
    params = dict(parts=[dict(kind="normed_qk_attention", params=lp, under="left", scale=0.6),
                         dict(kind="gated_delta_rule", params=rp, under="right", scale=1.7)])
    plain = {k: v.double() for k, v in w.items()}
    x = rounded(torch.randn(75, W, generator=gen(32)), dtype)
    want = 0.6 * P.sink_attention_mixer(x, plain, "m.left", l, EPS) + 1.7 * P.delta_mixer(x, plain, "m.right", r, EPS)
    for cuts in CUTS:
        rig = MixerRig("parallel_mixers", params, w, dtype, page=8)
        close(rig.cut("r", x, cuts), want, dtype, f"{cuts}", f32=1e-4, bf16=3e-2)
