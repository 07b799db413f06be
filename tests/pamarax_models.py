"""Small Pamarax configurations for the tests, and random weights for them.

Sizes differ between the configurations and between the layers of one: heads that share kv heads and heads that do
not, key and value sizes that differ, sizes that are no multiple of a 16-byte vector and sizes the tensor-core kernels
take, rotation of a whole head, of a part and of none, temperatures that step every few tokens (so that a short prompt
crosses several steps, also on a page's border), convolutions of one to five taps, several q/k heads in the delta rule,
layers without a feed-forward, models of one mixer kind only, an embedding scale of one.  Weights are drawn so that the
attention, the gates and the recurrences all decide something: matrices N(0, c / fan_in), gains near one (the layer
norms' files hold gain - 1), forget gates near one, decays from nearly one down to a fraction a token.
"""

import json
import os

import torch


def attention(heads, kv_heads, dim, rot=None, base=10000.0, scale=None):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=dim, scale=scale if scale is not None else 1.5 / dim ** 0.5)
    if rot:
        m["rot"] = dict(dims=rot, base=base)
    return dict(type="attention", mixer=m)


def mlstm(heads, dim, vdim, cap=15.0):
    return dict(type="mlstm", mixer=dict(heads=heads, dim=dim, vdim=vdim, gate_cap=cap))


def left(heads, kv_heads, dim, vdim, coef=0.5, every=16, scale=None):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale if scale is not None else 1.5 / dim ** 0.5)
    if every:
        m["q_temp"] = dict(coef=coef, every=every)
    return m


def right(heads, kv_heads, dim, vdim, conv=4):
    return dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, conv=conv)


def parallel(l, r, left_scale=1.0, right_scale=1.0):
    return dict(type="parallel", mixer=dict(left=l, right=r, left_scale=left_scale, right_scale=right_scale))


def dense(ff):
    return dict(kind="dense", ff=ff)


def layer(mix, mlp):
    return dict(mix, mlp=mlp)


def model(vocab, width, layers, eps=1e-6, embedding_scale=2.0):
    return dict(architecture="Pamarax", vocab=vocab, width=width, norm=dict(eps=eps), embedding=dict(scale=embedding_scale),
                layers=layers)


# S: every mixer, a layer with no feed-forward, part of a head rotated, a temperature that steps every 7 tokens
SMALL = model(200, 64, [
    layer(attention(4, 2, 16, rot=8, base=100.0), dense(96)),
    layer(mlstm(2, 8, 16, cap=10.0), None),
    layer(parallel(left(4, 2, 16, 8, coef=0.3, every=7), right(4, 2, 8, 16, conv=3), 0.7, 1.3), dense(80)),
    layer(attention(4, 2, 16, rot=8, base=100.0), dense(48))])

# O: sizes that are no multiple of eight, five heads each with its own kv head, no rotation, a temperature on every token,
# three q/k heads in the delta rule, a convolution of two taps, an embedding scale of one
ODD = model(333, 90, [
    layer(parallel(left(5, 5, 12, 20, coef=1.0, every=1), right(3, 3, 20, 12, conv=2), 1.5, 0.25), None),
    layer(attention(6, 1, 24), dense(50)),
    layer(mlstm(3, 20, 12, cap=5.0), dense(70)),
    layer(attention(3, 3, 12, rot=12, base=50.0, scale=0.5), None)], eps=1e-5, embedding_scale=1.0)

# W: sizes the tensor-core attention takes, more query heads than one tile's rows, wide states, no temperature
WIDE = model(512, 128, [
    layer(attention(8, 2, 64, rot=32), dense(256)),
    layer(parallel(left(20, 1, 32, 64, every=0), right(4, 2, 64, 32, conv=4), 1.0, 1.0), dense(192)),
    layer(mlstm(4, 64, 64), dense(128)),
    layer(attention(2, 1, 128, rot=64, base=5e5), None),
    layer(parallel(left(8, 2, 64, 32, coef=0.25, every=16), right(2, 1, 128, 64, conv=5), 0.5, 2.0), dense(64))], embedding_scale=0.5)

# only recurrent layers, and only attention layers
RECURRENT_ONLY = model(128, 48, [layer(mlstm(1, 96, 8, cap=20.0), dense(64)), layer(mlstm(6, 8, 24), None)])
ATTENTION_ONLY = model(128, 48, [layer(attention(3, 3, 16, rot=16), dense(64)), layer(attention(8, 2, 8, rot=2, base=3.0), dense(32))])

CONFIGS = dict(small=SMALL, odd=ODD, wide=WIDE, recurrent_only=RECURRENT_ONLY, attention_only=ATTENTION_ONLY)


def mixer_shapes(kind, m, D, p):
    """name -> (shape, kind) of one mixer's tensors under prefix p; D is the mixer's input width."""
    out = {}
    if kind == "attention":
        H, G, d = m["heads"], m["kv_heads"], m["dim"]
        out.update({f"{p}.q": ((H * d, D), "matrix"), f"{p}.k": ((G * d, D), "matrix"), f"{p}.q.norm": ((H * d,), "gain"),
                    f"{p}.k.norm": ((G * d,), "gain"), f"{p}.g": ((H * d, D), "matrix"), f"{p}.o": ((D, H * d), "matrix")})
    elif kind == "mlstm":
        H, d, e = m["heads"], m["dim"], m["vdim"]
        out.update({f"{p}.q": ((H * d, D), "matrix"), f"{p}.k": ((H * d, D), "matrix"), f"{p}.v": ((H * e, D), "matrix"),
                    f"{p}.g": ((H * e, D), "matrix"), f"{p}.o": ((D, H * e), "matrix"), f"{p}.norm": ((H * e,), "gain"),
                    f"{p}.i": ((H, D), "gate"), f"{p}.i.b": ((H,), "bias"), f"{p}.f": ((H, D), "gate"), f"{p}.f.b": ((H,), "forget_bias")})
    elif kind == "left":
        H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        out.update({f"{p}.q": ((H * d, D), "matrix"), f"{p}.k": ((G * d, D), "matrix"), f"{p}.v": ((G * e, D), "matrix"),
                    f"{p}.q.norm": ((d,), "gain"), f"{p}.k.norm": ((d,), "gain"), f"{p}.o": ((D, H * e), "matrix")})
    elif kind == "right":
        H, G, d, e, taps = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
        out.update({f"{p}.q": ((G * d, D), "matrix"), f"{p}.q.conv": ((G * d, taps), "conv"), f"{p}.k": ((G * d, D), "matrix"),
                    f"{p}.k.conv": ((G * d, taps), "conv"), f"{p}.v": ((H * e, D), "matrix"), f"{p}.v.conv": ((H * e, taps), "conv"),
                    f"{p}.b": ((H, D), "gate"), f"{p}.A_log": ((H,), "a_log"), f"{p}.norm": ((e,), "gain"), f"{p}.a": ((H, D), "gate"),
                    f"{p}.dt_bias": ((H,), "bias"), f"{p}.g": ((H * e, D), "matrix"), f"{p}.o": ((D, H * e), "matrix")})
    else:
        raise ValueError(kind)
    return out


def tensor_shapes(cfg):
    """name -> (shape, kind)."""
    D = cfg["width"]
    out = {"embed": ((cfg["vocab"], D), "table"), "head": ((cfg["vocab"], D), "matrix"), "final.norm": ((D,), "offset_gain")}
    for i, L in enumerate(cfg["layers"]):
        m, p = L["mixer"], f"l{i}"
        out[f"{p}.norm1"], out[f"{p}.norm1b"] = ((D,), "offset_gain"), ((D,), "offset_gain")
        if L["type"] == "parallel":
            out.update(mixer_shapes("left", m["left"], D, f"{p}.mix.left"))
            out.update(mixer_shapes("right", m["right"], D, f"{p}.mix.right"))
        else:
            out.update(mixer_shapes(L["type"], m, D, f"{p}.mix"))
        mlp = L.get("mlp")
        if mlp is None:
            continue
        out[f"{p}.norm2"], out[f"{p}.norm2b"] = ((D,), "offset_gain"), ((D,), "offset_gain")
        ff, q = mlp["ff"], f"{p}.mlp"
        out.update({f"{q}.gate": ((ff, D), "matrix"), f"{q}.gate.b": ((ff,), "bias"), f"{q}.up": ((ff, D), "matrix"),
                    f"{q}.up.b": ((ff,), "bias"), f"{q}.down": ((D, ff), "matrix"), f"{q}.down.b": ((D,), "bias")})
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
        elif kind == "a_log":
            t = -1.0 + r()                        # decays from nearly one down to a fraction a token
        elif kind == "conv":
            t = 0.6 * r()
        elif kind == "gate":
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
    d = os.path.join(str(folder), f"pamarax_{name}_{seed}")
    os.makedirs(d, exist_ok=True)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(d, "model.safetensors"), w)
    return d, cfg, {k: v.double() for k, v in w.items()}
