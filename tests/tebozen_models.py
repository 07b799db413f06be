"""Small Tebozen configurations for the tests, and random weights for them.

Sizes differ between the configurations and between the layers of one: heads that share kv heads and heads that do not,
key and value sizes that differ, sizes that are no multiple of a 16-byte vector and sizes the tensor-core kernels take,
rotation of a whole map, of a part and of none, windows shorter than a page and longer than several, convolutions of one to
five taps, one expert a token and several, shared experts and none, layers without a feed-forward, latent layers that attend
over an earlier layer's cache with the same and with another number of heads, models of one mixer kind only.  Weights are
drawn so that attention, gates, routers and recurrences all decide something: matrices N(0, c / fan_in), gains near one (the
layer norms' files hold gain - 1), forget gates near one.
"""

import json
import os

import torch


def attention(heads, kv_heads, dim, vdim, conv=4, diff=0.3, window=None, rot=None, base=10000.0, scale=None):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, conv=conv, diff=diff, scale=scale if scale is not None else 1.5 / dim ** 0.5)
    if window:
        m["mask"] = dict(size=window)
    if rot:
        m["rot"] = dict(dims=rot, base=base)
    return dict(type="attention", mixer=m)


def mlstm(heads, dim, vdim, cap=15.0):
    return dict(type="mlstm", mixer=dict(heads=heads, dim=dim, vdim=vdim, gate_cap=cap))


def latent(heads, dim, rot_dim, vdim, kv_rank, rot=None, base=10000.0, kv_from=None, scale=None):
    m = dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=kv_rank,
             scale=scale if scale is not None else 1.5 / (dim + rot_dim) ** 0.5)
    if rot:
        m["rot"] = dict(dims=rot, base=base)
    if kv_from is not None:
        m["kv_from"] = kv_from
    return dict(type="latent_attention", mixer=m)


def moe(experts, top, ff, shared=None):
    m = dict(kind="moe", router=dict(experts=experts, top=top), expert=dict(ff=ff))
    if shared:
        m["shared"] = dict(ff=shared)
    return m


def layer(mix, mlp):
    return dict(mix, mlp=mlp)


def model(vocab, width, layers, eps=1e-6, embedding_scale=2.0):
    return dict(architecture="Tebozen", vocab=vocab, width=width, norm=dict(eps=eps), embedding=dict(scale=embedding_scale),
                layers=layers)


# S: every mixer, a layer with no feed-forward, part of a map rotated, a window of 20 (a page and a bit), two experts a token,
# a latent layer that attends over another's pages
SMALL = model(150, 48, [
    layer(attention(4, 2, 8, 16, conv=3, diff=0.2, window=20, rot=4, base=100.0), moe(6, 2, 40, shared=24)),
    layer(mlstm(2, 8, 12, cap=10.0), None),
    layer(latent(3, 8, 4, 12, 20, rot=4, base=100.0), moe(4, 1, 32)),
    layer(attention(2, 1, 16, 8, conv=2, diff=0.5, window=33, rot=16, base=1000.0), None),
    layer(latent(3, 16, 4, 8, 20, rot=4, base=100.0, kv_from=2), moe(6, 3, 24, shared=40))])

# O: sizes that are no multiple of eight, three heads each with its own kv head, a window of 7 (inside a page), a convolution of
# one tap and one of five, a latent layer that copies the rows of one with another number of heads, part of the rotated part
# turned, an embedding scale of one
ODD = model(333, 90, [
    layer(latent(5, 12, 6, 10, 30, rot=4, base=50.0), moe(5, 3, 50, shared=70)),
    layer(attention(3, 3, 10, 6, conv=1, diff=0.1, window=7, rot=10, base=50.0), moe(3, 1, 36)),
    layer(latent(2, 6, 6, 14, 30, rot=4, base=50.0, kv_from=0), None),
    layer(mlstm(3, 20, 12, cap=5.0), moe(7, 2, 20, shared=10)),
    layer(attention(6, 2, 12, 20, conv=5, diff=0.4, window=100), None)], eps=1e-5, embedding_scale=1.0)

# W: sizes the tensor-core kernels take (keys and values of 64 and 32, a cache row of 128, experts of 128), more query heads
# than one tile's rows, a window of 64
WIDE = model(512, 128, [
    layer(attention(8, 2, 64, 64, conv=4, diff=0.3, window=64, rot=32), moe(8, 2, 128, shared=128)),
    layer(latent(4, 32, 32, 64, 96, rot=32), moe(8, 1, 128)),
    layer(mlstm(4, 64, 32), moe(4, 2, 128, shared=256)),
    layer(attention(10, 1, 32, 64, conv=2, diff=0.25, window=300, rot=32, base=5e5), None),
    layer(latent(4, 64, 32, 32, 96, rot=32, kv_from=1), moe(8, 4, 128))], embedding_scale=0.5)

# one mixer kind only
ATTENTION_ONLY = model(128, 64, [layer(attention(4, 4, 16, 16, conv=3, window=12, rot=8), moe(4, 2, 32, shared=32)),
                                 layer(attention(8, 2, 8, 8, conv=4, diff=0.6, window=50, rot=2, base=3.0), moe(4, 1, 48))])
LATENT_ONLY = model(128, 64, [layer(latent(4, 16, 8, 16, 24, rot=8), moe(4, 2, 32)),
                              layer(latent(4, 8, 8, 8, 24, rot=8, kv_from=0), None),
                              layer(latent(2, 8, 2, 8, 40, rot=2, base=7.0), moe(2, 2, 16, shared=16))])

CONFIGS = dict(small=SMALL, odd=ODD, wide=WIDE, attention_only=ATTENTION_ONLY, latent_only=LATENT_ONLY)


def mixer_shapes(kind, m, D, p):
    """name -> (shape, kind) of one mixer's tensors under prefix p; D is the mixer's input width."""
    out = {}
    if kind == "attention":
        H, G, d, e, taps = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m.get("conv", 0)
        for leaf, rows in (("q", H * 2 * d), ("k", G * 2 * d), ("v", G * e)):
            out[f"{p}.{leaf}"], out[f"{p}.{leaf}.b"] = ((rows, D), "matrix"), ((rows,), "bias")
            if taps:
                out[f"{p}.{leaf}.conv"] = ((rows, taps), "conv")
        out.update({f"{p}.{k}": ((d,), "lambda") for k in ("lq1", "lk1", "lq2", "lk2")})
        out.update({f"{p}.g": ((H, D), "gate"), f"{p}.o": ((D, H * e), "matrix")})
    elif kind == "mlstm":
        H, d, e = m["heads"], m["dim"], m["vdim"]
        out.update({f"{p}.q": ((H * d, D), "matrix"), f"{p}.k": ((H * d, D), "matrix"), f"{p}.v": ((H * e, D), "matrix"),
                    f"{p}.g": ((H * e, D), "matrix"), f"{p}.o": ((D, H * e), "matrix"), f"{p}.norm": ((H * e,), "gain"),
                    f"{p}.i": ((H, D), "gate"), f"{p}.i.b": ((H,), "bias"), f"{p}.f": ((H, D), "gate"), f"{p}.f.b": ((H,), "forget_bias")})
    elif kind == "latent_attention":
        H, d, dr, e, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
        out.update({f"{p}.q": ((H * (d + dr), D), "matrix"), f"{p}.uk": ((H * d, r), "matrix"), f"{p}.uv": ((H * e, r), "matrix"),
                    f"{p}.g": ((H, D), "gate"), f"{p}.o": ((D, H * e), "matrix")})
        if m.get("kv_from") is None:
            out.update({f"{p}.dkv": ((r + dr, D), "matrix"), f"{p}.dkv.norm": ((r,), "gain")})
    else:
        raise ValueError(kind)
    return out


def mlp_shapes(mlp, D, q):
    out = {f"{q}.router": ((mlp["router"]["experts"], D), "router")}
    ff = mlp["expert"]["ff"]
    for e in range(mlp["router"]["experts"]):
        out[f"{q}.e{e}.up"], out[f"{q}.e{e}.down"] = ((ff, D), "matrix"), ((D, ff), "matrix")
    if mlp.get("shared"):
        sf = mlp["shared"]["ff"]
        out[f"{q}.shared.up"], out[f"{q}.shared.down"] = ((sf, D), "matrix"), ((D, sf), "matrix")
    return out


def tensor_shapes(cfg):
    """name -> (shape, kind)."""
    D = cfg["width"]
    out = {"embed": ((cfg["vocab"], D), "table"), "head": ((cfg["vocab"], D), "matrix"), "final.norm": ((D,), "offset_gain")}
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}"
        out[f"{p}.norm1"] = ((D,), "offset_gain")
        out.update(mixer_shapes(L["type"], L["mixer"], D, f"{p}.mix"))
        if L.get("mlp") is not None:
            out[f"{p}.norm2"] = ((D,), "offset_gain")
            out.update(mlp_shapes(L["mlp"], D, f"{p}.mlp"))
    return out


def draw(shapes, seed):
    """bfloat16 tensors (what a model file holds) for name -> (shape, kind)."""
    g = torch.Generator().manual_seed(seed)
    w = {}
    for name, (shape, kind) in shapes.items():
        r = lambda: torch.randn(shape, generator=g)
        if kind == "gain":
            t = 1.0 + 0.2 * r()
        elif kind == "offset_gain":
            t = 0.2 * r()
        elif kind == "bias":
            t = 0.5 * r()
        elif kind == "forget_bias":
            t = 2.5 + r()                         # forget gates from nearly one down to a half
        elif kind == "conv":
            t = 0.6 * r()
        elif kind == "lambda":
            t = 0.4 * r() / shape[-1] ** 0.25     # the two exponents of lambda of the order of a few tenths
        elif kind in ("gate", "router"):
            t = 2.5 * r() / shape[-1] ** 0.5
        elif kind == "table":
            t = r()
        else:
            t = 1.3 * r() / shape[-1] ** 0.5
        w[name] = t.to(torch.bfloat16)
    return w


def random_weights(cfg, seed):
    return draw(tensor_shapes(cfg), seed)


def write_model(folder, name, seed=0, cfg=None):
    """A model folder for configuration ``name``; returns (folder, config dict, float64 weights for the plain implementation)."""
    from paged_llm_rs_b200.weights.safetensors_io import write_safetensors

    cfg = cfg or CONFIGS[name]
    w = random_weights(cfg, seed)
    d = os.path.join(str(folder), f"tebozen_{name}_{seed}")
    os.makedirs(d, exist_ok=True)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(d, "model.safetensors"), w)
    return d, cfg, {k: v.double() for k, v in w.items()}
