"""Tebozen on the GPU against the plain implementation (tests/plain_tebozen.py): each kernel and each mixer alone (through
the cache manager and the step packer, with inputs made so that a window that is one token off, a lost convolution state,
one far key or a score that is not squared would show), then whole models through the engine's step function, cache
manager, state slots and scheduler."""

import os
import random
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_tebozen as P
from tebozen_models import CONFIGS, attention, draw, latent, layer, mixer_shapes, mlp_shapes, mlstm, model, moe, write_model
from test_pamarax_gpu import MixerRig, Served, close, errors, gen, rounded

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]
NAMES = {torch.float32: "float32", torch.bfloat16: "bfloat16"}
EPS = 1e-5
F = P.F


def ops_():
    from paged_llm_rs_b200.kernels import ops
    return ops


# ------------------------------------------------------------------------ each kernel alone

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tokens,width,experts,top", [(1, 48, 6, 2), (7, 90, 5, 3), (300, 128, 16, 1), (33, 64, 9, 9)])
def test_router_scores_each_output_alone_and_keeps_the_scores(dtype, tokens, width, experts, top):
    ops = ops_()
    g = gen(1)
    h = rounded(torch.randn(tokens, width, generator=g), dtype)
    wr = rounded(2.5 * torch.randn(experts, width, generator=g) / width ** 0.5, torch.bfloat16)
    ids, weights = ops.moe_route(h.to(dtype).to(DEV), wr.float().to(DEV), None, top, 1, 1, scoring="sigmoid", renormalize=False)
    want_ids, want_w = P.route(h, wr, top)
    scores = torch.sigmoid(h @ wr.T)
    got_ids = ids.long().cpu()
    # a close call may fall either way: compare the chosen scores, and the ids where the choice was clear
    close(weights, want_w, torch.float32, "chosen scores", f32=1e-5)
    close(torch.gather(scores, 1, got_ids), want_w, torch.float32, "the chosen outputs' scores", f32=1e-5)
    assert float((got_ids == want_ids).double().mean()) > 0.98


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tokens,width,ff,experts,top,shared", [(1, 48, 40, 6, 2, 24), (5, 90, 50, 5, 3, 0), (64, 128, 128, 8, 2, 128),
                                                                 (200, 128, 128, 4, 1, 256), (9, 64, 20, 7, 7, 10)])
def test_experts_without_gates_read_the_token_times_its_score(dtype, tokens, width, ff, experts, top, shared):
    """Both forms of the experts (a pair a row; for many rows in bfloat16 the pairs sorted by expert and grouped tensor-core
    products) through the feed-forward part.  The score enters squared: weighting the output instead would show."""
    from paged_llm_rs_b200.parts import base, decoder  # noqa: F401
    from paged_llm_rs_b200.parts.spec import PartSpec
    mlp = moe(experts, top, ff, shared or None)
    w = draw(mlp_shapes(mlp, width, "m"), 2)
    rt = base.Runtime(torch.device(DEV), dtype)
    part = base.make(base.FEED_FORWARDS, "feed-forward", PartSpec("routed_experts", dict(
        hidden_size=width, expert_size=ff, experts=experts, top=top, correction=False, scoring="sigmoid", renormalize=False, gated=False,
        activation="squared_relu", weight_on="input", shared_size=shared or None), "m"), rt)
    part.bind({s.name: (w[s.name].to(dtype) if s.role == "matrix" else w[s.name].float()).to(DEV) for s in part.tensors()})
    h = rounded(torch.randn(tokens, width, generator=gen(3)), dtype)
    got = part.forward(h.to(dtype).to(DEV), None)
    want = P.routed_feed_forward(h, {k: v.double() for k, v in w.items()}, "m", mlp)
    if dtype == torch.float32:
        close(got, want, dtype, f32=2e-5)
    else:
        # (a router's close call moves a token's row by a whole expert: nine rows in ten within rounding)
        per_row = (got.double().cpu() - want).pow(2).mean(-1).sqrt() / want.pow(2).mean(-1).sqrt().clamp_min(1e-9)
        assert float(per_row.median()) < 2e-2 and float((per_row < 5e-2).double().mean()) >= 0.9, per_row
    _, sc = P.route(h, w["m.router"].double(), top)
    assert float(sc.min()) < 0.9      # scores far enough from one that score and score squared differ


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,n,k", [(3, 24, 48), (70, 128, 64), (300, 256, 128), (5, 77, 90)])
def test_product_with_a_one_argument_activation(dtype, rows, n, k):
    ops = ops_()
    g = gen(4)
    x, w = rounded(torch.randn(rows, k, generator=g), dtype), rounded(torch.randn(n, k, generator=g) / k ** 0.5, dtype)
    got = ops.linear_act(x.to(dtype).to(DEV), w.to(dtype).to(DEV), "squared_relu")
    close(got, torch.relu(x @ w.T) ** 2, dtype, f32=1e-5, bf16=1.5e-2)
    y = torch.randn(5, 7, generator=g)
    close(ops.unary_act(y.to(dtype).to(DEV).clone(), "squared_relu"), torch.relu(rounded(y, dtype)) ** 2, dtype, f32=1e-6, bf16=1e-2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,heads,group,dv,lam,post", [(1, 4, 2, 16, 0.37, 0.8), (9, 3, 3, 6, -0.2, 0.9), (40, 10, 10, 64, 1.1, 0.75), (5, 6, 1, 20, 0.5, 0.5)])
def test_difference_of_the_maps_norm_and_gate(dtype, T, heads, group, dv, lam, post):
    ops = ops_()
    g = gen(5)
    kv = heads // group
    a = rounded(torch.randn(T, kv, 2, group, dv, generator=g), dtype)
    wide = rounded(torch.randn(T, heads + 5, generator=g), dtype)
    out = torch.empty((T, heads * dv), dtype=dtype, device=DEV)
    ops.diff_combine(a.to(dtype).to(DEV).view(T, -1), wide.to(dtype).to(DEV)[:, 3:3 + heads], out, heads, group, dv, lam, post, EPS)
    o = (a[:, :, 0] - lam * a[:, :, 1]).reshape(T, heads, dv)
    want = P.rms_unit(o, EPS) * post * torch.sigmoid(wide[:, 3:3 + heads])[:, :, None]
    close(out, want.reshape(T, -1), dtype, f32=1e-5, bf16=1e-2)


@pytest.mark.parametrize("dtype", DTYPES)
def test_one_gate_a_head(dtype):
    ops = ops_()
    g = gen(6)
    y, wide = rounded(torch.randn(11, 5 * 12, generator=g), dtype), rounded(torch.randn(11, 9, generator=g), dtype)
    got = ops.gate_mul(y.to(dtype).to(DEV).clone(), wide.to(dtype).to(DEV)[:, 2:7], "sigmoid", per=12)
    close(got, (y.view(11, 5, 12) * torch.sigmoid(wide[:, 2:7])[:, :, None]).reshape(11, -1), dtype, f32=1e-6, bf16=1e-2)


# ------------------------------------------------------------------------ each mixer alone, through the cache manager

def diff_rig(dtype, m, W, seed, page=16, pages=64, craft=None):
    w = draw(mixer_shapes("attention", m, W, "m"), seed)
    if craft:
        craft(w)
    rot = m.get("rot") or {}
    params = dict(hidden_size=W, num_heads=m["heads"], num_kv_heads=m["kv_heads"], key_dim=m["dim"], value_dim=m["vdim"], scale=m["scale"],
                  diff=m["diff"], conv=m.get("conv", 0), window=(m.get("mask") or {}).get("size"), rot_dims=rot.get("dims", 0),
                  rot_base=rot.get("base", 1.0), eps=EPS, biases=True)
    plain = {k: v.double() for k, v in w.items()}
    return MixerRig("differential_attention", params, w, dtype, page, pages), lambda h: P.differential_attention(h, plain, "m", m, EPS)


def latent_rig(dtype, m, W, seed, page=16, pages=64, craft=None):
    w = draw(mixer_shapes("latent_attention", m, W, "m"), seed)
    if craft:
        craft(w)
    rot = m.get("rot") or {}
    params = dict(hidden_size=W, heads=m["heads"], dim=m["dim"], rot_dim=m["rot_dim"], vdim=m["vdim"], kv_rank=m["kv_rank"], scale=m["scale"],
                  rot_dims=rot.get("dims", 0), rot_base=rot.get("base", 1.0), eps=EPS, gate="sigmoid", keeps="own")
    plain = {k: v.double() for k, v in w.items()}
    mm = dict(m, rot=dict(dims=rot.get("dims", 0), base=rot.get("base", 1.0)))
    return MixerRig("rotary_latent_attention", params, w, dtype, page, pages), lambda h: P.latent_attention(h, plain, "m", mm, EPS)


CUTS = [[75], [2] * 5 + [1, 1, 3, 17, 16, 20, 2, 1, 1, 1, 1, 1], [1] * 75, [40, 35], [64, 2, 9]]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv,dim,vdim,conv,window,rot,base,W,page", [
    (4, 2, 8, 16, 3, 20, 4, 100.0, 48, 16), (3, 3, 10, 6, 1, 7, 10, 50.0, 90, 8), (6, 2, 12, 20, 5, 100, 0, 1.0, 40, 4),
    (8, 2, 64, 64, 4, 64, 32, 1e4, 128, 16), (10, 1, 32, 64, 2, 0, 32, 5e5, 96, 16), (2, 1, 16, 8, 0, 33, 16, 1e3, 64, 16)])
def test_differential_attention_whole_in_portions_and_token_by_token(dtype, heads, kv, dim, vdim, conv, window, rot, base, W, page):
    """A window inside a page and over several, a convolution of no, one and several taps whose state crosses every cut."""
    m = attention(heads, kv, dim, vdim, conv=conv, window=window or None, rot=rot, base=base)["mixer"]
    x = rounded(torch.randn(75, W, generator=gen(10)), dtype)
    for cuts in CUTS:
        rig, plain = diff_rig(dtype, m, W, 11, page=page)
        close(rig.cut("r", x, cuts), plain(x), dtype, f"{cuts}", f32=2e-4, bf16=5e-2)


def along_keys(w, heads, kv, dim):
    """Both maps' W_q of every head become W_k of its kv head's FIRST map, without biases, convolution taps on earlier tokens
    or lambda's exponents: a token's first-map query then points along the first-map key of any token with the same input."""
    k = w["m.k"].view(kv, 2, dim, -1)
    w["m.q"] = k[:, :1].repeat_interleave(heads // kv, 0).repeat(1, 2, 1, 1).reshape(heads * 2 * dim, -1).contiguous()
    for leaf in ("q", "k", "v"):
        w[f"m.{leaf}.b"].zero_()
        w[f"m.{leaf}.conv"].zero_()
        w[f"m.{leaf}.conv"][:, -1] = 1.0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window,page", [(24, 16), (16, 16), (33, 8), (1, 16), (17, 4)])
def test_one_key_just_inside_and_just_outside_the_window(dtype, window, page):
    """ONE earlier token has the last token's input three times over, and queries point along keys, so that its key takes the
    weight of the first map when the window still holds it and none when it has just left: the two cases differ by far more
    than rounding, in a decoded token, at the end of a portion and beside other requests; also where the window's edge is a
    page's edge and where the window holds the token alone."""
    W, heads, kv, dim, vdim, ctx = 64, 4, 2, 32, 16, 120
    g = gen(20)
    base_x = torch.randn(ctx + 1, W, generator=g)
    m = attention(heads, kv, dim, vdim, conv=3, window=window, scale=1.0)["mixer"]
    make = lambda: diff_rig(dtype, m, W, 21, page=page, pages=80, craft=lambda w: along_keys(w, heads, kv, dim))
    last = {}
    for back in sorted({window - 1, window, 0, 1} & set(range(0, ctx))):
        at = ctx - back
        x = base_x.clone()
        if back:
            x[at] = 3.0 * x[ctx]
        x = rounded(x, dtype)
        rig, plain = make()
        want = plain(x)
        last[back] = want[-1]
        got = rig.cut("a", x, [ctx, 1])
        close(got[-1:], want[-1:], dtype, f"decoded, key {back} back", f32=2e-4, bf16=5e-2)
        rig, _ = make()
        got = rig.cut("b", x, [ctx - 5, 6])
        close(got[-1:], want[-1:], dtype, f"portion, key {back} back", f32=2e-4, bf16=5e-2)
        rig, _ = make()
        other = rounded(torch.randn(40, W, generator=g), dtype)
        rig.step([("c", x[:ctx - 2]), ("d", other[:5])])
        res = rig.step([("d", other[5:6]), ("c", x[ctx - 2:]), ("e", other[6:])])
        close(res[1][-1:], want[-1:], dtype, f"batch, key {back} back", f32=2e-4, bf16=5e-2)
    if window > 1:
        # the plain implementation itself: the key just inside decides the output, the key just outside does not
        assert float((last[window - 1] - last[window]).abs().max()) > 0.2 * float(last[window].abs().max())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,dim,rot_dim,vdim,rank,rot,base,W,page", [
    (3, 8, 4, 12, 20, 4, 100.0, 48, 16), (5, 12, 6, 10, 30, 4, 50.0, 90, 8), (4, 32, 32, 64, 96, 32, 1e4, 128, 16), (2, 8, 2, 8, 40, 2, 7.0, 64, 4),
    (20, 16, 8, 16, 56, 8, 1e4, 64, 16)])
def test_latent_attention_whole_in_portions_and_token_by_token(dtype, heads, dim, rot_dim, vdim, rank, rot, base, W, page):
    m = latent(heads, dim, rot_dim, vdim, rank, rot=rot, base=base)["mixer"]
    x = rounded(torch.randn(75, W, generator=gen(30)), dtype)
    for cuts in CUTS:
        rig, plain = latent_rig(dtype, m, W, 31, page=page)
        close(rig.cut("r", x, cuts), plain(x), dtype, f"{cuts}", f32=2e-4, bf16=5e-2)


@pytest.mark.parametrize("dtype", DTYPES)
def test_one_far_latent_row_decides(dtype):
    """W_q is made so that the LAST token's unrotated query points along the unrotated keys of ONE earlier token (and its
    rotated part is zero): that token's row takes the weight wherever it lies, the first token, a page's last and first row,
    hundreds of tokens back, across split key ranges."""
    W, heads, dim, rot_dim, vdim, rank, ctx = 64, 4, 16, 8, 16, 32, 420
    m = latent(heads, dim, rot_dim, vdim, rank, rot=8, scale=1.0)["mixer"]
    mm = dict(m)
    g = gen(32)
    x = rounded(torch.randn(ctx + 1, W, generator=g), dtype)
    for at in (0, 15, 16, 255, 256, ctx - 1):
        def craft(w):
            plain = {k: v.double() for k, v in w.items()}
            c = P.latent_rows(x, plain, "m", mm, EPS)[0][at]
            along = plain["m.uk"].view(heads, dim, rank) @ c                        # the keys of token `at`, a head
            q = torch.zeros(heads, dim + rot_dim, W, dtype=F)
            q[:, :dim] = 2.0 * along[:, :, None] * x[ctx][None, None, :] / float(x[ctx] @ x[ctx])
            w["m.q"] = q.reshape(heads * (dim + rot_dim), W).to(torch.bfloat16)

        rig, plain = latent_rig(dtype, m, W, 33, pages=90, craft=craft)
        want = plain(x)
        without = plain(torch.cat([x[:at], x[at + 1:]]))[-1]
        assert float((without - want[-1]).abs().max()) > 0.1 * float(want[-1].abs().max())
        close(rig.cut("a", x, [ctx, 1])[-1:], want[-1:], dtype, f"decoded, row {at}", f32=2e-4, bf16=5e-2)
        rig, _ = latent_rig(dtype, m, W, 33, pages=90, craft=craft)
        close(rig.cut("b", x, [ctx - 20, 21])[-1:], want[-1:], dtype, f"portion, row {at}", f32=2e-4, bf16=5e-2)


@pytest.mark.parametrize("dtype", DTYPES)
def test_convolution_state_in_batches_with_slots_used_again(dtype):
    """Four live requests whose convolutions carry their last inputs from step to step; slots of finished requests are taken
    again and must start from zeros."""
    W = 48
    m = attention(4, 2, 8, 16, conv=4, window=20, rot=4, base=100.0)["mixer"]
    g = gen(40)
    xs = {k: rounded(torch.randn(n, W, generator=g), dtype) for k, n in dict(a=30, b=9, c=3, d=17, e=11, f=6).items()}
    rig, plain = diff_rig(dtype, m, W, 41, pages=24)
    want = {k: plain(x) for k, x in xs.items()}
    at, got = {k: 0 for k in xs}, {k: [] for k in xs}
    plan = [[("a", 10), ("b", 2), ("c", 1)], [("a", 1), ("b", 7), ("c", 2), ("d", 16)], [("a", 1), ("d", 1), ("e", 2)],
            [("a", 18), ("e", 9), ("f", 1)], [("f", 2)], [("f", 3)]]
    for step in plan:
        res = rig.step([(k, xs[k][at[k]:at[k] + n]) for k, n in step])
        for (k, n), r in zip(step, res):
            got[k].append(r); at[k] += n
            if at[k] == xs[k].shape[0]:
                rig.end(k)
    for k in xs:
        close(torch.cat(got[k]), want[k], dtype, k, f32=2e-4, bf16=5e-2)
    rig.cache.check_invariants()


# ------------------------------------------------------------------------ whole models through the engine

TOL = {torch.float32: 2e-4, torch.bfloat16: 6e-2}


def agrees(got, want, dtype):
    """float32: every position within rounding.  bfloat16: the typical position well within and nine in ten not far: a
    router's close call hands a token to another expert, and a recurrent head's read-out that nearly cancels is decided by
    rounding; such a position differs by a large part of its logits."""
    e = errors(got, want)
    ok = bool((e < TOL[dtype]).all()) if dtype == torch.float32 else (float(e.median()) < TOL[dtype] and float(e.quantile(0.9)) < 0.3)
    if not ok:
        print(f"errors: median {float(e.median()):.3g}, over {float((e > TOL[dtype]).double().mean()):.3g}, max {float(e.max()):.3g} at {int(e.argmax())}")
    return ok


_models = {}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = tmp_path_factory.mktemp("tebozen")

    def get(name):
        if name not in _models:
            _models[name] = write_model(root, name, seed=sorted(CONFIGS).index(name))
        return _models[name]
    return get


def tokens_for(cfg, n, seed):
    return np.random.default_rng(seed).integers(0, cfg["vocab"], n).tolist()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_whole_prompt_every_layer_and_the_first_tokens(models, dtype, name):
    folder, cfg, w = models(name)
    toks = tokens_for(cfg, 45, 1)
    streams = []
    want = P.forward(cfg, w, toks, streams)
    s = Served(folder, dtype)
    trace = {}
    got = s.step([("a", toks, list(range(len(toks))))], trace=trace)
    assert agrees(got, want, dtype)
    for i in range(len(cfg["layers"])):
        x = trace[f"l{i}.out"]
        assert x.dtype == torch.float32, "the stream between layers is float32 whatever the compute dtype"
        per_token = (x.double().cpu() - streams[i]).pow(2).mean(-1).sqrt() / streams[i].pow(2).mean(-1).sqrt()
        if dtype == torch.float32:
            assert float(per_token.max()) < 5e-5, f"stream after layer {i}: {per_token}"
        else:
            assert float(per_token.median()) < TOL[dtype] and float(per_token.quantile(0.9)) < 0.3, f"stream after layer {i}: {per_token}"
    s2 = Served(folder, dtype)
    first = torch.cat([s2.step([("b", toks[:1], [0])]), s2.step([("b", toks[1:2], [0])]), s2.step([("b", toks[2:4], [0, 1])])])
    if dtype == torch.float32:
        assert agrees(first, want[:4], dtype)
    else:
        assert float(errors(first, want[:4]).max()) < max(0.3, 1.5 * float(errors(got[:4], want[:4]).max()))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,page", [("small", 16), ("odd", 8), ("wide", 32), ("attention_only", 4), ("latent_only", 16)])
def test_prefill_against_token_by_token_decoding(models, dtype, name, page):
    folder, cfg, w = models(name)
    toks = tokens_for(cfg, 70, 2)
    want = P.forward(cfg, w, toks)
    s = Served(folder, dtype, page=page, pages=40)
    whole = s.step([("w", toks, list(range(70)))])
    one = torch.cat([s.step([("d", toks[i:i + 1], [0])]) for i in range(70)])
    assert agrees(whole, want, dtype) and agrees(one, want, dtype)
    if dtype == torch.float32:
        assert float(errors(one, whole).max()) < 5e-5          # cutting changes nothing beyond rounding


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["small", "odd", "wide"])
def test_portions_of_every_size(models, dtype, name):
    folder, cfg, w = models(name)
    toks = tokens_for(cfg, 150, 3)
    want = P.forward(cfg, w, toks)
    for cuts in ([2] * 10 + [3, 5, 16, 17, 31, 33, 25], [64, 64, 22], [1, 2, 13, 48, 1, 1, 84], [149, 1]):
        assert sum(cuts) == 150
        s = Served(folder, dtype, page=16, pages=12)
        at, outs = 0, []
        for c in cuts:
            outs.append(s.step([("p", toks[at:at + c], list(range(c)))]))
            at += c
        assert agrees(torch.cat(outs), want, dtype), cuts


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["small", "odd", "wide"])
def test_batches_of_unequal_requests_pages_and_slots_used_again(models, dtype, name):
    """Four live requests, portions beside single tokens, in a pool and with state slots that only hold them if those of
    finished requests are used again; every row against the plain implementation of its request alone."""
    folder, cfg, w = models(name)
    lengths = dict(a=90, b=33, c=7, d=64, e=50, f=21)
    toks = {k: tokens_for(cfg, n, 10 + i) for i, (k, n) in enumerate(lengths.items())}
    want = {k: P.forward(cfg, w, t) for k, t in toks.items()}
    s = Served(folder, dtype, page=16, pages=14, max_requests=4)
    at = {k: 0 for k in toks}
    got = {k: [] for k in toks}
    plan = [[("a", 40), ("b", 2), ("c", 1)], [("a", 1), ("b", 30), ("c", 3), ("d", 17)], [("a", 1), ("c", 3), ("d", 47), ("b", 1)],
            [("a", 48), ("e", 2)], [("e", 47), ("f", 1)], [("e", 1), ("f", 20)]]
    for step in plan:
        out = s.step([(k, toks[k][at[k]:at[k] + n], list(range(n))) for k, n in step])
        row = 0
        for k, n in step:
            got[k].append(out[row:row + n]); row += n; at[k] += n
            if at[k] == lengths[k]:
                s.end(k)
    for k in toks:
        assert at[k] == lengths[k]
        assert agrees(torch.cat(got[k]), want[k], dtype), k
    s.runner.cache.check_invariants()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,page", [("small", 8), ("odd", 4)])
def test_long_decoding_while_windows_pass_and_pages_go_back(models, dtype, name, page):
    """330 tokens, all but ten decoded one by one: every window passes over decoded tokens many times, the window groups give
    their pages back, the recurrent states run long and the latent layers read dozens of pages."""
    folder, cfg, w = models(name)
    toks = tokens_for(cfg, 330, 5)
    want = P.forward(cfg, w, toks)
    s = Served(folder, dtype, page=page, pages=-(-330 // page) + 1)
    s.step([("x", toks[:10], [])])
    outs = torch.cat([s.step([("x", toks[i:i + 1], [0])]) for i in range(10, 330)])
    assert agrees(outs, want[10:], dtype)
    windowed = [g for g in s.runner.cache.groups if g.window is not None]
    assert windowed and all(g.allocator.available() > g.allocator.total // 2 for g in windowed)


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_request_left_out_of_steps_goes_on_later(models, dtype):
    folder, cfg, w = models("small")
    ta, tb = tokens_for(cfg, 60, 8), tokens_for(cfg, 40, 9)
    wa, wb = P.forward(cfg, w, ta), P.forward(cfg, w, tb)
    s = Served(folder, dtype)
    a1 = s.step([("a", ta[:25], list(range(25)))])
    b1 = s.step([("b", tb[:39], list(range(39)))])
    both = s.step([("a", ta[25:], list(range(35))), ("b", tb[39:], [0])])
    assert agrees(torch.cat([a1, both[:35]]), wa, dtype) and agrees(torch.cat([b1, both[35:]]), wb, dtype)


# ------------------------------------------------------------------------ generation, replay, command line

def greedy(logits):
    return int(torch.argmax(logits))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["small", "wide"])
def test_greedy_generation_through_the_scheduler(models, dtype, name):
    """Engine.generate: chunked prompts, captured decode steps, several requests at once; every produced token against the
    plain implementation on the same history."""
    from paged_llm_rs_b200 import Engine
    folder, cfg, w = models(name)
    prompts = [tokens_for(cfg, n, 20 + n) for n in (3, 41, 18, 70, 1)]
    eng = Engine(folder, dtype=NAMES[dtype], block_size=16, blocks=64, max_batch=4, chunk=32, prefix_cache=False)
    outs = eng.generate(prompts, max_tokens=12)
    decided = total = out_of_noise = 0
    for p, o in zip(prompts, outs):
        assert len(o) == 12
        seq = list(p)
        for tok in o:
            logits = P.forward(cfg, w, seq)[-1]
            top2 = torch.topk(logits, 2).values
            noise = (1e-4 if dtype == torch.float32 else 0.05) * max(1.0, float(logits.abs().max()))
            out_of_noise += float(logits[greedy(logits)] - logits[tok]) >= noise
            decided += float(top2[0] - top2[1]) >= noise
            total += 1
            seq.append(tok)
    assert out_of_noise <= (0 if dtype == torch.float32 else 0.1 * total), (out_of_noise, total)
    assert decided >= 0.5 * total


def test_trace_replay_and_command_line(models, tmp_path):
    folder, cfg, w = models("small")
    from trace_tools import TraceBuilder, replay
    toks = tokens_for(cfg, 60, 7)
    tb = TraceBuilder()
    tb.step([("r", toks[:33], [0, 32])])
    tb.step([("r", toks[33:59], [25]), ("q", toks[:5], [4])], end=["q"])
    tb.step([("r", toks[59:], [0])], end=["r"])
    got = tb.collect(replay(folder, "float32", tb.steps, 128, cfg["vocab"]))
    want = P.forward(cfg, w, toks)
    for pos, row in got["r"].items():
        assert float(errors(torch.from_numpy(row).double()[None], want[pos:pos + 1]).max()) < 2e-4
    # the captured and replayed steps of generation give the same logits
    got2 = tb.collect(replay(folder, "float32", tb.steps, 128, cfg["vocab"], graphs=True, step_tokens=48))
    for pos, row in got2["r"].items():
        assert float(errors(torch.from_numpy(row).double()[None], want[pos:pos + 1]).max()) < 2e-4
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-m", "paged_llm_rs_b200", "generate", "--model", folder, "--dtype", "f32",
                        "--prompt-ids", ",".join(map(str, toks[:9])), "--max-tokens", "4", "--blocks", "32"],
                       cwd=root, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    out = [int(t) for t in r.stdout.strip().splitlines()[-1].split(",")]
    seq = toks[:9]
    for tok in out:
        assert tok == greedy(P.forward(cfg, w, seq)[-1])
        seq = seq + [tok]


# ------------------------------------------------------------------------ configurations drawn at random

def random_configuration(seed):
    """Sizes, counts, layer order, windows and constants drawn from a seed."""
    rnd = random.Random(seed)
    width = rnd.choice([48, 64, 96, 128, 160])

    def an_attention():
        kv = rnd.choice([1, 2, 3])
        dim = rnd.choice([8, 12, 16, 32, 64])
        return attention(kv * rnd.choice([1, 2, 4]), kv, dim, rnd.choice([8, 12, 24, 32, 64]), conv=rnd.choice([1, 2, 3, 4, 6]),
                         diff=rnd.choice([0.1, 0.3, 0.55]), window=rnd.choice([1, 5, 16, 31, 64, 200]), rot=rnd.choice([0, 2, dim // 2, dim]),
                         base=rnd.choice([10.0, 1e4, 5e5]))

    def an_mlstm():
        return mlstm(rnd.choice([1, 2, 3, 4]), rnd.choice([8, 16, 24, 32]), rnd.choice([8, 12, 32, 48]), cap=rnd.choice([5.0, 15.0, 30.0]))

    latents = []

    def a_latent(i):
        if latents and rnd.random() < 0.5:
            j, src = rnd.choice(latents)
            return latent(rnd.choice([src["heads"], 2, 6]), rnd.choice([8, 16, 32]), src["rot_dim"], rnd.choice([8, 16, 24]), src["kv_rank"],
                          rot=(src.get("rot") or {}).get("dims"), base=(src.get("rot") or {}).get("base", 1.0), kv_from=j)
        rot_dim = rnd.choice([2, 4, 8, 16, 32])
        L = latent(rnd.choice([1, 3, 4, 8]), rnd.choice([8, 16, 32, 64]), rot_dim, rnd.choice([8, 16, 48]), rnd.choice([16, 24, 40, 96]),
                   rot=rnd.choice([0, 2, rot_dim]), base=rnd.choice([10.0, 1e4]))
        latents.append((i, L["mixer"]))
        return L

    def a_mlp():
        if rnd.random() < 0.2:
            return None
        experts = rnd.choice([2, 4, 7, 16])
        return moe(experts, rnd.choice([t for t in (1, 2, 3, 4) if t <= experts]), rnd.choice([16, 40, 64, 128]), rnd.choice([None, 24, 128]))

    layers = []
    for i in range(rnd.choice([2, 3, 5])):
        kind = rnd.choice(["attention", "mlstm", "latent"])
        layers.append(layer(an_attention() if kind == "attention" else an_mlstm() if kind == "mlstm" else a_latent(i), a_mlp()))
    return model(rnd.choice([64, 200, 513]), width, layers, eps=rnd.choice([1e-6, 1e-5]), embedding_scale=rnd.choice([0.5, 1.0, 3.0]))


@pytest.mark.parametrize("seed", range(12))
def test_configurations_drawn_at_random(tmp_path, seed):
    """Whole against portions, token by token and a batch, float32 (where a failure is a fault and not a close call)."""
    cfg = random_configuration(seed)
    folder, cfg, w = write_model(tmp_path, f"random{seed}", seed=100 + seed, cfg=cfg)
    toks, other = tokens_for(cfg, 90, seed), tokens_for(cfg, 30, seed + 50)
    want, want_other = P.forward(cfg, w, toks), P.forward(cfg, w, other)
    s = Served(folder, torch.float32, page=rnd_page(seed), pages=48)
    assert agrees(s.step([("w", toks, list(range(90)))]), want, torch.float32), cfg
    s.end("w")
    outs = [s.step([("p", toks[:37], list(range(37)))])]
    mixed = s.step([("p", toks[37:39], [0, 1]), ("o", other, list(range(30)))])
    outs.append(mixed[:2])
    assert agrees(mixed[2:], want_other, torch.float32), cfg
    outs += [s.step([("p", toks[i:i + 1], [0])]) for i in range(39, 90)]
    assert agrees(torch.cat(outs), want, torch.float32), cfg
    b = Served(folder, torch.bfloat16, page=16, pages=40)
    e = errors(b.step([("w", toks, list(range(90)))]), want)
    assert float(e.median()) < 0.1, (cfg, e)


def rnd_page(seed):
    return [4, 8, 16, 32][seed % 4]
