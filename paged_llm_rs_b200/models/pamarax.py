"""Pamarax, described as parts.

A decoder whose layers are listed in its configuration.  Each layer norms its sublayers on the way in and on the way out
(``sandwich_stream32``: x + norm(mixer(norm(x))), then x + norm(ff(norm(x))), each gain kept as its offset from one, the stream
float32) and has one of three mixers:

  attention   grouped-query attention whose keys are also its values, q and k normed over the whole projection, part of
              each head rotated, the heads' outputs gated by a sigmoid (``normed_qk_attention``)
  mlstm       the matrix memory of the xLSTM with capped log gates (``matrix_lstm``)
  parallel    two mixers on the same input, added with a constant each (``parallel_mixers``): attention with a q/k norm a
              head, a query temperature that grows with the position and a one in the softmax's denominator, beside a
              gated delta rule behind short convolutions (``gated_delta_rule``)

and a dense gated feed-forward with biases, or none.  The embedding is multiplied by a constant.  Nothing bounds a
request's length but float32 positions (exact up to 2^24).

Tensors: ``embed``, ``head``, ``final.norm``, and per layer i ``l<i>.norm1|norm1b|norm2|norm2b``, ``l<i>.mix.*`` and
``l<i>.mlp.*`` (see the parts for the leaves).
"""

from __future__ import annotations

from ..config.pamarax import PamaraxConfig
from ..config.registry import Architecture, register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

MAX_POSITIONS = 1 << 24      # positions enter the rotation as float32


def _attention(W, m, eps):
    return dict(hidden_size=W, num_heads=m.heads, num_kv_heads=m.kv_heads, key_dim=m.dim, value_dim=m.vdim, scale=m.scale, eps=eps,
                qk_norm="projection", values_are_keys=True, rot_dims=m.rot_dims, rot_base=m.rot_base, gate="sigmoid")


def _sink_attention(W, m, eps):
    return dict(hidden_size=W, num_heads=m.heads, num_kv_heads=m.kv_heads, key_dim=m.dim, value_dim=m.vdim, scale=m.scale, eps=eps,
                qk_norm="head", temp_coef=m.temp_coef, temp_every=m.temp_every, sink_one=True)


def _delta_rule(W, m, eps):
    return dict(hidden_size=W, heads=m.heads, kv_heads=m.kv_heads, dim=m.dim, vdim=m.vdim, conv=m.conv, eps=eps)


def describe_pamarax(cfg: PamaraxConfig) -> ModelSpec:
    W, eps = cfg.width, cfg.norm_eps
    norm = lambda name: PartSpec("rmsnorm_sandwich_stream32", dict(width=W, eps=eps, one_plus=True, leaf=""), name)
    layers = []
    for i, L in enumerate(cfg.layers):
        p, m = f"l{i}", L.mixer
        if L.mixer_kind == "attention":
            mixer = PartSpec("normed_qk_attention", _attention(W, m, eps), f"{p}.mix")
        elif L.mixer_kind == "mlstm":
            mixer = PartSpec("matrix_lstm", dict(hidden_size=W, heads=m.heads, dim=m.dim, vdim=m.vdim, gate_cap=m.gate_cap, eps=eps),
                             f"{p}.mix")
        else:
            mixer = PartSpec("parallel_mixers", dict(parts=[
                dict(kind="normed_qk_attention", params=_sink_attention(W, m.left, eps), under="left", scale=m.left_scale),
                dict(kind="gated_delta_rule", params=_delta_rule(W, m.right, eps), under="right", scale=m.right_scale)]), f"{p}.mix")
        norms = {"mixer": norm(f"{p}.norm1"), "mixer_out": norm(f"{p}.norm1b")}
        ff = None
        if L.dense_ff is not None:
            ff = PartSpec("swiglu_mlp", dict(hidden_size=W, intermediate_size=L.dense_ff, activation="silu", biases=True,
                                             names=dict(gate="gate", up="up", down="down")), f"{p}.mlp")
            norms["feed_forward"], norms["feed_forward_out"] = norm(f"{p}.norm2"), norm(f"{p}.norm2b")
        layers.append(LayerSpec(block="sandwich_stream32", mixer=mixer, feed_forward=ff, norms=norms, prefix=p))
    return ModelSpec(
        architecture=cfg.architecture,
        hidden_size=W,
        vocab_size=cfg.vocab,
        max_positions=MAX_POSITIONS,
        embedding=PartSpec("token_embedding", dict(vocab_size=cfg.vocab, hidden_size=W, leaf="", scale=cfg.embedding_scale,
                                                   stream="float32"), "embed"),
        layers=layers,
        schedule=[ScheduleEntry(i) for i in range(len(layers))],
        final_norm=norm("final.norm"),
        head=PartSpec("linear_head", dict(vocab_size=cfg.vocab, hidden_size=W, leaf=""), "head"),
    )


PAMARAX = Architecture(name="Pamarax", parse=PamaraxConfig.from_dict, describe=describe_pamarax, aliases=("pamarax",))
register_architecture(PAMARAX)
