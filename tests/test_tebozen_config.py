"""Tebozen without a GPU: the configuration reader, the description as parts, the tensors it asks for, what its mixers ask
of the cache manager (pages beside a state slot for the convolutions, shared pages, copied rows), and the plain
implementation's mechanisms against hand-made cases."""

import copy
import math

import pytest
import torch

import plain_tebozen as P
from tebozen_models import CONFIGS, ODD, SMALL, random_weights, tensor_shapes

from paged_llm_rs_b200.cache.manager import CacheManager
from paged_llm_rs_b200.config.registry import resolve_architecture
from paged_llm_rs_b200.errors import ConfigError, UnsupportedModelError
from paged_llm_rs_b200.parts.base import CompositeNeed, JoinedKVNeed, RowNeed, StateNeed
from paged_llm_rs_b200.parts.decoder import DecoderModel, Runtime, tensor_specs_of

F = P.F


def describe(cfg):
    arch = resolve_architecture(cfg)
    return arch, arch.describe(arch.parse(cfg))


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_the_parts_ask_for_exactly_the_files_tensors(name):
    cfg = CONFIGS[name]
    arch, spec = describe(cfg)
    assert arch.name == "Tebozen"
    asked = {s.name: tuple(s.shape) for s in tensor_specs_of(spec)}
    assert asked == {n: tuple(shape) for n, (shape, _) in tensor_shapes(cfg).items()}


def test_every_constant_comes_from_the_configuration():
    cfg = copy.deepcopy(SMALL)
    cfg["embedding"]["scale"], cfg["norm"]["eps"] = 0.3, 1e-3
    cfg["layers"][0]["mixer"].update(scale=0.7, diff=0.45, conv=5)
    cfg["layers"][0]["mixer"]["rot"] = dict(dims=6, base=77.0)
    cfg["layers"][0]["mixer"]["mask"] = dict(size=9)
    cfg["layers"][0]["mlp"]["router"].update(experts=9, top=4)
    cfg["layers"][1]["mixer"]["gate_cap"] = 3.5
    cfg["layers"][2]["mixer"].update(scale=0.21)
    _, spec = describe(cfg)
    a = spec.layers[0].mixer.params
    assert (a["scale"], a["diff"], a["conv"], a["window"], a["rot_dims"], a["rot_base"], a["eps"]) == (0.7, 0.45, 5, 9, 6, 77.0, 1e-3)
    f = spec.layers[0].feed_forward.params
    assert (f["experts"], f["top"], f["scoring"], f["renormalize"], f["gated"], f["activation"], f["weight_on"], f["shared_size"]) == \
        (9, 4, "sigmoid", False, False, "squared_relu", "input", 24)
    assert spec.layers[1].mixer.params["gate_cap"] == 3.5 and spec.layers[1].feed_forward is None
    assert set(spec.layers[1].norms) == {"mixer"} and set(spec.layers[0].norms) == {"mixer", "feed_forward"}
    l = spec.layers[2].mixer.params
    assert (l["scale"], l["keeps"], l["kv_rank"], l["rot_dim"], l["rot_dims"]) == (0.21, "own", 20, 4, 4)
    assert spec.embedding.params["scale"] == 0.3 and spec.final_norm.params["eps"] == 1e-3 and spec.final_norm.params["one_plus"]
    assert spec.layers[2].feed_forward.params["shared_size"] is None


def test_a_layer_that_attends_over_anothers_cache():
    # the same number of heads: the schedule hands it the other layer's pages
    _, spec = describe(SMALL)
    assert [e.reads_cache_of for e in spec.schedule] == [None, None, None, None, 2]
    assert spec.layers[4].mixer.params["keeps"] == "nothing" and spec.layers[2].mixer.params["hands_on"] is None
    # another number of heads: it keeps copies of the rows that the other layer hands on
    _, spec = describe(ODD)
    assert all(e.reads_cache_of is None for e in spec.schedule)
    assert spec.layers[0].mixer.params["hands_on"] == "latent.0"
    assert (spec.layers[2].mixer.params["keeps"], spec.layers[2].mixer.params["copies"]) == ("copy", "latent.0")


@pytest.mark.parametrize("change,error", [
    (lambda c: c["layers"][0].update(type="ring"), UnsupportedModelError),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), ConfigError),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=3), ConfigError),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=10), ConfigError),
    (lambda c: c["layers"][0]["mixer"].pop("scale"), ConfigError),
    (lambda c: c["layers"][0]["mixer"].pop("diff"), ConfigError),
    (lambda c: c["layers"][0]["mixer"]["mask"].update(size=0), ConfigError),
    (lambda c: c["layers"][1]["mixer"].update(gate_cap=0.0), ConfigError),
    (lambda c: c["layers"][2]["mixer"]["rot"].update(dims=6), ConfigError),
    (lambda c: c["layers"][4]["mixer"].update(kv_from=1), ConfigError),             # not a latent layer
    (lambda c: c["layers"][4]["mixer"].update(kv_from=4), ConfigError),             # not an earlier one
    (lambda c: c["layers"][4]["mixer"].update(kv_rank=24), ConfigError),            # rows of another width
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), UnsupportedModelError),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=7), ConfigError),
    (lambda c: c["norm"].update(eps=0.0), ConfigError),
    (lambda c: c.pop("layers"), ConfigError)])
def test_bad_configurations_are_refused(change, error):
    cfg = copy.deepcopy(SMALL)
    change(cfg)
    with pytest.raises(error):
        describe(cfg)


def test_cache_needs_groups_and_slots():
    _, spec = describe(SMALL)
    model = DecoderModel(spec, Runtime(torch.device("cpu"), torch.float32))
    needs = model.cache_needs()
    assert isinstance(needs[0], CompositeNeed)
    pages, slot = needs[0].parts
    # a map is a kv head of its own: 2 kv heads x 2 maps, a window of 20
    assert isinstance(pages, JoinedKVNeed) and (pages.kind, pages.window, pages.num_kv_heads, pages.key_dim, pages.value_dim, pages.group_size) == \
        ("window", 20, 4, 8, 16, 2)
    # the convolution's last two inputs of every q, k and v channel
    assert isinstance(slot, StateNeed) and slot.shape == (2 * (4 * 2 * 8 + 2 * 2 * 8 + 2 * 16),)
    assert isinstance(needs[1], StateNeed)
    assert isinstance(needs[2], RowNeed) and needs[2].width == 24
    assert needs[4] is None                               # attends over entry 2's pages
    cm = CacheManager(needs, 8, 16, 4, torch.float32, "cpu")
    assert [g.cells for g in cm.groups] == [[(0, 0)], [2], [(3, 0)]]
    assert cm.prefix_cache is False
    caches = cm.layer_caches()
    (pool, gi), state = caches[0]
    assert gi == 0 and tuple(pool.shape) == (16, 4, 8, 24) and tuple(state.shape) == (4, 2 * 128)
    # a window group gives back the pages the window has passed
    cm.open("a")
    assert cm.reserve("a", 64)
    cm.commit("a", 64)
    assert cm.get("a").tables[0].blocks[:5] == [-1] * 5 and all(b >= 0 for b in cm.get("a").tables[1].blocks)
    # in ODD the copying layer has pages of its own
    _, spec = describe(ODD)
    needs = DecoderModel(spec, Runtime(torch.device("cpu"), torch.float32)).cache_needs()
    cm = CacheManager(needs, 8, 4, 2, torch.float32, "cpu", allocate_device=False)
    assert isinstance(needs[2], RowNeed) and needs[2].group_key() != needs[0].group_key() and len(cm.groups) == 4


def test_plain_prefix_equals_whole():
    for cfg in (SMALL, ODD):
        w = {k: v.double() for k, v in random_weights(cfg, 3).items()}
        toks = torch.randint(0, cfg["vocab"], (40,), generator=torch.Generator().manual_seed(1)).tolist()
        whole = P.forward(cfg, w, toks)
        assert torch.allclose(P.forward(cfg, w, toks[:17]), whole[:17], atol=1e-9)


def test_plain_mechanisms_alone():
    # the norm whose file holds gain - 1
    x = torch.tensor([[3.0, 4.0]], dtype=F)
    assert torch.allclose(P.offset_norm(x, torch.tensor([0.0, 1.0], dtype=F), 0.0), torch.tensor([[3.0, 8.0]], dtype=F) / math.sqrt(12.5))
    # the convolution's last column meets the current token; zeros before the start
    u = torch.tensor([[1.0], [2.0], [3.0]], dtype=F)
    assert torch.allclose(P.causal_conv(u, torch.tensor([[100.0, 10.0, 1.0]], dtype=F)), torch.tensor([[1.0], [12.0], [123.0]], dtype=F))
    # halves: entry i with i + dims / 2; pairs: entry 2i with 2i + 1; the rest passes; position 0 turns nothing
    x = torch.arange(1, 9, dtype=F).view(1, 1, 8).repeat(4, 1, 1)
    h, p = P.rotate_halves(x, 4, 10.0), P.rotate_pairs(x, 4, 10.0)
    assert torch.equal(h[0], x[0]) and torch.equal(p[0], x[0]) and torch.equal(h[..., 4:], x[..., 4:]) and torch.equal(p[..., 4:], x[..., 4:])
    a0, a1 = 3.0, 3.0 * 10.0 ** -0.5
    assert abs(float(h[3, 0, 0]) - (1 * math.cos(a0) - 3 * math.sin(a0))) < 1e-12 and abs(float(h[3, 0, 2]) - (3 * math.cos(a0) + 1 * math.sin(a0))) < 1e-12
    assert abs(float(h[3, 0, 1]) - (2 * math.cos(a1) - 4 * math.sin(a1))) < 1e-12
    assert abs(float(p[3, 0, 0]) - (1 * math.cos(a0) - 2 * math.sin(a0))) < 1e-12 and abs(float(p[3, 0, 1]) - (2 * math.cos(a0) + 1 * math.sin(a0))) < 1e-12
    assert abs(float(p[3, 0, 3]) - (4 * math.cos(a1) + 3 * math.sin(a1))) < 1e-12
    # a window of 2: the third row sees the second and itself, not the first
    w = P.masked_softmax(torch.zeros(3, 3, dtype=F), 2)
    assert w.tolist() == [[1.0, 0.0, 0.0], [0.5, 0.5, 0.0], [0.0, 0.5, 0.5]]
    # the router keeps the chosen scores as they are, and the expert reads the token times its score
    h1 = torch.tensor([[1.0, 0.0]], dtype=F)
    ids, sc = P.route(h1, torch.tensor([[0.0, 0.0], [2.0, 0.0], [-1.0, 0.0]], dtype=F), 2)
    assert ids.tolist() == [[1, 0]] and torch.allclose(sc, torch.sigmoid(torch.tensor([[2.0, 0.0]], dtype=F)))
    wts = {"m.router": torch.tensor([[3.0, 0.0]], dtype=F), "m.e0.up": torch.tensor([[2.0, 0.0], [-1.0, 0.0]], dtype=F),
           "m.e0.down": torch.tensor([[1.0, 5.0], [0.0, 7.0]], dtype=F)}
    s = 1 / (1 + math.exp(-3.0))
    out = P.routed_feed_forward(h1, wts, "m", dict(router=dict(experts=1, top=1)))
    assert torch.allclose(out, torch.tensor([[(2 * s) ** 2, 0.0]], dtype=F))      # relu kills the second row; the score enters squared
    # the matrix memory's first token: m = max(f, i) with m starting at zero, not at minus infinity
    wm = {"x.q": torch.eye(2, dtype=F), "x.k": torch.eye(2, dtype=F), "x.v": torch.eye(2, dtype=F), "x.g": torch.zeros(2, 2, dtype=F),
          "x.o": torch.eye(2, dtype=F), "x.norm": torch.ones(2, dtype=F), "x.i": torch.zeros(1, 2, dtype=F), "x.i.b": torch.tensor([-2.0], dtype=F),
          "x.f": torch.zeros(1, 2, dtype=F), "x.f.b": torch.tensor([0.0], dtype=F)}
    _, (S, n, m) = P.matrix_lstm(torch.tensor([[1.0, 0.0]], dtype=F), wm, "x", dict(heads=1, dim=2, vdim=2, gate_cap=50.0), 0.0)
    f_log, i_log = math.log(0.5), 50.0 * math.tanh(-2.0 / 50.0)
    assert abs(float(m) - max(f_log, i_log)) < 1e-9 and abs(float(S[0, 0, 0]) - math.exp(i_log - f_log)) < 1e-9
    # two maps that agree cancel up to (1 - lambda); the head norm then brings the difference back to unit size
    wa = {"a.q": torch.zeros(4, 2, dtype=F), "a.k": torch.zeros(4, 2, dtype=F), "a.v": torch.eye(2, dtype=F), "a.q.b": torch.zeros(4, dtype=F),
          "a.k.b": torch.zeros(4, dtype=F), "a.v.b": torch.zeros(2, dtype=F), "a.g": torch.zeros(1, 2, dtype=F), "a.o": torch.eye(2, dtype=F),
          "a.lq1": torch.zeros(2, dtype=F), "a.lk1": torch.zeros(2, dtype=F), "a.lq2": torch.zeros(2, dtype=F), "a.lk2": torch.zeros(2, dtype=F)}
    o = P.differential_attention(torch.tensor([[3.0, 4.0]], dtype=F), wa, "a", dict(heads=1, kv_heads=1, dim=2, vdim=2, scale=1.0, diff=0.25), 0.0)
    # lambda = 1 - 1 + 0.25; o = 0.75 v over its root mean square, times 0.75, times sigmoid(0)
    assert torch.allclose(o, torch.tensor([[3.0, 4.0]], dtype=F) / math.sqrt(12.5) * 0.75 * 0.5)
