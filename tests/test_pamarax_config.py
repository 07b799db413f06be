"""Pamarax without a GPU: the configuration reader, the description as parts, the tensors it asks for, what its mixers ask
of the cache manager (pages, state slots, both for mixers side by side), and the plain implementation against itself."""

import copy
import math

import pytest
import torch

import plain_pamarax as P
from pamarax_models import CONFIGS, ODD, SMALL, WIDE, random_weights, tensor_shapes

from paged_llm_rs_b200.cache.manager import CacheManager
from paged_llm_rs_b200.config.registry import resolve_architecture
from paged_llm_rs_b200.errors import ConfigError, UnsupportedModelError
from paged_llm_rs_b200.parts.base import CompositeNeed, JoinedKVNeed, StateNeed
from paged_llm_rs_b200.parts.decoder import DecoderModel, Runtime, tensor_specs_of


def describe(cfg):
    arch = resolve_architecture(cfg)
    return arch, arch.describe(arch.parse(cfg))


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_the_parts_ask_for_exactly_the_files_tensors(name):
    cfg = CONFIGS[name]
    arch, spec = describe(cfg)
    assert arch.name == "Pamarax"
    asked = {s.name: tuple(s.shape) for s in tensor_specs_of(spec)}
    assert asked == {n: tuple(shape) for n, (shape, _) in tensor_shapes(cfg).items()}


def test_every_constant_comes_from_the_configuration():
    cfg = copy.deepcopy(SMALL)
    cfg["embedding"]["scale"], cfg["norm"]["eps"] = 0.3, 1e-3
    cfg["layers"][0]["mixer"].update(scale=0.7)
    cfg["layers"][0]["mixer"]["rot"] = dict(dims=4, base=77.0)
    cfg["layers"][1]["mixer"]["gate_cap"] = 3.5
    par = cfg["layers"][2]["mixer"]
    par.update(left_scale=0.11, right_scale=9.0)
    par["left"].update(scale=0.9)
    par["left"]["q_temp"] = dict(coef=0.01, every=33)
    par["right"]["conv"] = 5
    _, spec = describe(cfg)
    a = spec.layers[0].mixer.params
    assert (a["scale"], a["rot_dims"], a["rot_base"], a["eps"], a["qk_norm"], a["values_are_keys"], a["gate"]) == \
        (0.7, 4, 77.0, 1e-3, "projection", True, "sigmoid")
    assert spec.layers[1].mixer.params["gate_cap"] == 3.5 and spec.layers[1].mixer.params["eps"] == 1e-3
    l, r = spec.layers[2].mixer.params["parts"]
    assert (l["scale"], r["scale"], l["under"], r["under"]) == (0.11, 9.0, "left", "right")
    assert (l["params"]["scale"], l["params"]["temp_coef"], l["params"]["temp_every"], l["params"]["sink_one"], l["params"]["qk_norm"]) == \
        (0.9, 0.01, 33, True, "head")
    assert r["params"]["conv"] == 5 and r["params"]["eps"] == 1e-3
    assert spec.embedding.params["scale"] == 0.3 and spec.final_norm.params["eps"] == 1e-3 and spec.final_norm.params["one_plus"]
    assert spec.layers[1].feed_forward is None and set(spec.layers[1].norms) == {"mixer", "mixer_out"}
    assert spec.layers[0].feed_forward.params["biases"] and set(spec.layers[0].norms) == {"mixer", "mixer_out", "feed_forward", "feed_forward_out"}


@pytest.mark.parametrize("change,error", [
    (lambda c: c["layers"][0].update(type="ring"), UnsupportedModelError),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), ConfigError),
    (lambda c: c["layers"][0]["mixer"].update(vdim=8), ConfigError),                 # the keys are the values
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), ConfigError),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=18), ConfigError),
    (lambda c: c["layers"][0]["mixer"].pop("scale"), ConfigError),
    (lambda c: c["layers"][1]["mixer"].update(gate_cap=0.0), ConfigError),
    (lambda c: c["layers"][2]["mixer"]["right"].update(kv_heads=3), ConfigError),
    (lambda c: c["layers"][2]["mixer"]["right"].update(conv=0), ConfigError),
    (lambda c: c["layers"][2]["mixer"]["left"]["q_temp"].update(every=0), ConfigError),
    (lambda c: c["layers"][2]["mixer"].pop("left_scale"), ConfigError),
    (lambda c: c["layers"][0]["mlp"].update(kind="moe"), UnsupportedModelError),
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
    assert isinstance(needs[0], JoinedKVNeed) and (needs[0].kind, needs[0].key_dim, needs[0].value_dim) == ("full", 16, 16)
    assert isinstance(needs[1], StateNeed) and needs[1].shape == (2 * 8 * 16 + 2 * 8 + 2,)
    assert isinstance(needs[2], CompositeNeed)
    l, r = needs[2].parts
    assert isinstance(l, JoinedKVNeed) and (l.num_kv_heads, l.key_dim, l.value_dim, l.group_size) == (2, 16, 8, 2)
    assert isinstance(r, StateNeed) and r.shape == (4 * 8 * 16 + 2 * (2 * 2 * 8 + 4 * 16),)
    cm = CacheManager(needs, 8, 16, 4, torch.float32, "cpu", allocate_device=False)
    # the two attention layers share pages and tables; the attention beside the delta rule has pages of another shape
    assert [g.cells for g in cm.groups] == [[0, 3], [(2, 0)]]
    assert cm.prefix_cache is False                    # state of fixed size cannot be shared by prefix
    caches = cm.layer_caches()
    assert isinstance(caches[2], tuple) and len(caches[2]) == 2


def test_mixers_side_by_side_each_get_their_own(tmp_path):
    """On a CPU manager with tensors: the left part's pool view and group, the right part's slots."""
    _, spec = describe(SMALL)
    model = DecoderModel(spec, Runtime(torch.device("cpu"), torch.float32))
    cm = CacheManager(model.cache_needs(), 8, 6, 3, torch.float32, "cpu")
    caches = cm.layer_caches()
    (pool, gi), slots = caches[2]
    assert gi == 1 and tuple(pool.shape) == (6, 2, 8, 16 + 8) and tuple(slots.shape) == (3, 4 * 8 * 16 + 2 * (2 * 2 * 8 + 4 * 16))
    assert tuple(caches[1].shape) == (3, 2 * 8 * 16 + 2 * 8 + 2)
    # a slot is zeroed when it is taken again
    cm.open("a")
    s = cm.get("a").state_slot
    slots[s] = 3.0
    caches[1][s] = 2.0
    cm.close("a")
    cm.open("b")
    assert cm.get("b").state_slot == s and float(slots[s].abs().max()) == 0.0 and float(caches[1][s].abs().max()) == 0.0


def test_plain_token_by_token_equals_whole():
    """The plain implementation keeps nothing between calls: a prefix's logits are the whole's."""
    for cfg in (SMALL, ODD):
        w = {k: v.double() for k, v in random_weights(cfg, 3).items()}
        toks = torch.randint(0, cfg["vocab"], (40,), generator=torch.Generator().manual_seed(1)).tolist()
        whole = P.forward(cfg, w, toks)
        assert torch.allclose(P.forward(cfg, w, toks[:17]), whole[:17], atol=1e-9)


def test_plain_mechanisms_alone():
    F = P.F64
    # the norm whose file holds gain - 1
    x = torch.tensor([[3.0, 4.0]], dtype=F)
    assert torch.allclose(P.norm_one_plus(x, torch.tensor([0.0, 1.0], dtype=F), 0.0), torch.tensor([[3.0, 8.0]], dtype=F) / math.sqrt(12.5))
    # rotation turns pairs (i, i + dims / 2) and leaves the rest
    x = torch.arange(8, dtype=F).view(1, 1, 8)
    r = P.rotate_half(x, [3], 4, 10.0)
    assert torch.equal(r[..., 4:], x[..., 4:])
    assert abs(float(r[0, 0, 0]) - (0 * math.cos(3.0) - 2 * math.sin(3.0))) < 1e-12 and abs(float(r[0, 0, 2]) - (2 * math.cos(3.0) + 0 * math.sin(3.0))) < 1e-12
    a1 = 3 * 10.0 ** -0.5
    assert abs(float(r[0, 0, 1]) - (1 * math.cos(a1) - 3 * math.sin(a1))) < 1e-12
    # the temperature steps when (p + 1) reaches a multiple of ``every``
    t = P.query_temperature(9, 2.0, 4)
    assert t[:3].tolist() == [1.0] * 3 and abs(float(t[3]) - (1 + 2 * math.log(2))) < 1e-12 and float(t[6]) == float(t[3]) and abs(float(t[7]) - (1 + 2 * math.log(3))) < 1e-12
    # one more in the denominator: a lone key with score zero gets half the weight; without it, all
    q, k, v = torch.zeros(1, 1, 4, dtype=F), torch.ones(1, 1, 4, dtype=F), torch.full((1, 1, 2), 6.0, dtype=F)
    assert torch.allclose(P.causal_attention(q, k, v, 1.0, True), torch.full((1, 1, 2), 3.0, dtype=F))
    assert torch.allclose(P.causal_attention(q, k, v, 1.0, False), torch.full((1, 1, 2), 6.0, dtype=F))
    # very negative scores: the extra one takes everything
    assert float(P.causal_attention(torch.full((1, 1, 4), -9.0, dtype=F), k, v, 1.0, True).abs().max()) < 1e-12
    # the convolution's last column meets the current token; zeros before the start
    u = torch.tensor([[1.0], [2.0], [3.0]], dtype=F)
    c = P.causal_conv_silu(u, torch.tensor([[100.0, 10.0, 1.0]], dtype=F))
    assert torch.allclose(c, P.silu(torch.tensor([[1.0], [12.0], [123.0]], dtype=F)))
    # the delta rule with beta 1 and no decay stores v under a unit k and reads it back with the same k
    k1 = torch.tensor([[[1.0, 0.0]]], dtype=F)
    o = P.gated_delta_rule(k1, k1, torch.tensor([[[5.0, 7.0]]], dtype=F), torch.ones(1, 1, dtype=F), torch.ones(1, 1, dtype=F))
    assert torch.allclose(o, torch.tensor([[[5.0, 7.0]]], dtype=F))
    # the matrix memory's first token: m = max(f, i) with m starting at zero, not at minus infinity
    i_log, f_log = torch.tensor([[-2.0]], dtype=F), torch.tensor([[-0.5]], dtype=F)
    o = P.matrix_memory(k1, k1, torch.tensor([[[4.0, 8.0]]], dtype=F), i_log, f_log)
    b = math.exp(-2.0 + 0.5)
    assert torch.allclose(o, torch.tensor([[[4.0, 8.0]]], dtype=F) * b / (max(b, math.exp(0.5)) + 1e-6))
