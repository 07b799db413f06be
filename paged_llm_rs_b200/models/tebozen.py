"""Tebozen, described as parts.

A pre-norm decoder on a float32 stream (``prenorm_stream32``; the norms' gains are stored as their distance from one) whose
layers are listed in its configuration.  Each layer has one of three mixers:

  attention          differential attention: two softmax maps a head over the same values, the second subtracted lambda
                     times, behind short causal convolutions on q, k and v, inside a sliding window, each head over its
                     root mean square and gated by one sigmoid a head (``differential_attention``)
  mlstm              the matrix memory of the xLSTM with capped log gates (``matrix_lstm``)
  latent_attention   attention over one cached latent a token with one rotated key part shared by the heads, gated a head
                     (``rotary_latent_attention``); a layer may attend over an earlier layer's cache instead of keeping one

and a mixture of squared-relu experts without gates behind a sigmoid router whose scores multiply the experts' INPUT, with a
shared expert, or no feed-forward.  The embedding is multiplied by a constant.  Nothing bounds a request's length but
float32 positions (exact up to 2^24).

Tensors: ``embed``, ``head``, ``final.norm``, and per layer i ``l<i>.norm1|norm2``, ``l<i>.mix.*`` and ``l<i>.mlp.*`` (see the
parts for the leaves).
"""

from __future__ import annotations

from ..config.registry import Architecture, register_architecture
from ..config.tebozen import TebozenConfig
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

MAX_POSITIONS = 1 << 24      # positions enter the rotation as float32


def describe_tebozen(cfg: TebozenConfig) -> ModelSpec:
    W, eps = cfg.width, cfg.norm_eps
    norm = lambda name: PartSpec("rmsnorm_scaled_stream32", dict(width=W, eps=eps, mult=1.0, one_plus=True, leaf=""), name)
    layers, schedule = [], []
    for i, L in enumerate(cfg.layers):
        p, m = f"l{i}", L.mixer
        reads = None
        if L.mixer_kind == "attention":
            mixer = PartSpec("differential_attention",
                             dict(hidden_size=W, num_heads=m.heads, num_kv_heads=m.kv_heads, key_dim=m.dim, value_dim=m.vdim,
                                  scale=m.scale, diff=m.diff, conv=m.conv, window=m.window, rot_dims=m.rot_dims, rot_base=m.rot_base,
                                  eps=eps, biases=True), f"{p}.mix")
        elif L.mixer_kind == "mlstm":
            mixer = PartSpec("matrix_lstm", dict(hidden_size=W, heads=m.heads, dim=m.dim, vdim=m.vdim, gate_cap=m.gate_cap, eps=eps),
                             f"{p}.mix")
        else:
            params = dict(hidden_size=W, heads=m.heads, dim=m.dim, rot_dim=m.rot_dim, vdim=m.vdim, kv_rank=m.kv_rank, scale=m.scale,
                          rot_dims=m.rot_dims, rot_base=m.rot_base, eps=eps, gate="sigmoid")
            if m.kv_from is None:
                # (its rows are handed on to the layers of other head counts that attend over them: see below)
                params.update(keeps="own", hands_on=f"latent.{i}" if any(
                    o.mixer_kind == "latent_attention" and o.mixer.kv_from == i and o.mixer.heads != m.heads for o in cfg.layers) else None)
            elif cfg.layers[m.kv_from].mixer.heads == m.heads:
                # the same work items fit both layers: this one attends over the other's pages themselves
                params.update(keeps="nothing")
                reads = m.kv_from
            else:
                # another head count cuts a step into other work items: this layer keeps a copy of the other's rows in pages of
                # its own group
                params.update(keeps="copy", copies=f"latent.{m.kv_from}")
            mixer = PartSpec("rotary_latent_attention", params, f"{p}.mix")
        norms = {"mixer": norm(f"{p}.norm1")}
        ff = None
        if L.moe is not None:
            e = L.moe
            ff = PartSpec("routed_experts", dict(hidden_size=W, expert_size=e.expert_ff, experts=e.experts, top=e.top, correction=False,
                                                 scoring="sigmoid", renormalize=False, gated=False, activation="squared_relu",
                                                 weight_on="input", shared_size=e.shared_ff), f"{p}.mlp")
            norms["feed_forward"] = norm(f"{p}.norm2")
        layers.append(LayerSpec(block="prenorm_stream32", mixer=mixer, feed_forward=ff, norms=norms, prefix=p))
        schedule.append(ScheduleEntry(i, reads_cache_of=reads))
    return ModelSpec(
        architecture=cfg.architecture,
        hidden_size=W,
        vocab_size=cfg.vocab,
        max_positions=MAX_POSITIONS,
        embedding=PartSpec("token_embedding", dict(vocab_size=cfg.vocab, hidden_size=W, leaf="", scale=cfg.embedding_scale,
                                                   stream="float32"), "embed"),
        layers=layers,
        schedule=schedule,
        final_norm=norm("final.norm"),
        head=PartSpec("linear_head", dict(vocab_size=cfg.vocab, hidden_size=W, leaf=""), "head"),
    )


TEBOZEN = Architecture(name="Tebozen", parse=TebozenConfig.from_dict, describe=describe_tebozen, aliases=("tebozen",))
register_architecture(TEBOZEN)
