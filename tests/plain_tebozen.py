"""A plain, slow implementation of the Tebozen decoder in float64 on the CPU: one function per mechanism, whole
sequences at once (the matrix memory token by token), no cache, no batching.  It shares no code with the engine and is what
the engine's kernels, mixers and whole models are compared with.

``weights`` maps tensor names to tensors; ``cfg`` is the configuration as config.json spells it (a dict).
"""

from __future__ import annotations

import torch

F = torch.float64


def rms_unit(x, eps):
    """x over the root of (its mean square + eps), along the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def offset_norm(x, w, eps):
    """The block norm: the stored gain is the distance from one."""
    return rms_unit(x, eps) * (1.0 + w)


def embed(tokens, table, scale):
    return table[torch.as_tensor(tokens, dtype=torch.long)] * scale


def causal_conv(u, w):
    """u [T, C], w [C, taps]: y[t] = sum_j w[:, j] * u[t - taps + 1 + j], zeros before the first row."""
    T, C = u.shape
    taps = w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=u.dtype), u], 0)
    y = torch.zeros_like(u)
    for j in range(taps):
        y = y + padded[j:j + T] * w[:, j]
    return y


def _angles(T, dims, base, start=0):
    i = torch.arange(dims // 2, dtype=F)
    freq = base ** (-2.0 * i / dims)
    pos = torch.arange(start, start + T, dtype=F)
    return pos[:, None] * freq[None, :]            # [T, dims/2]


def rotate_halves(x, dims, base, start=0):
    """x [T, n, d]: entry i of the first ``dims`` is paired with entry i + dims/2."""
    if not dims:
        return x
    T = x.shape[0]
    a = _angles(T, dims, base, start)[:, None, :]
    c, s = torch.cos(a), torch.sin(a)
    u, v = x[..., :dims // 2], x[..., dims // 2:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], -1)


def rotate_pairs(x, dims, base, start=0):
    """x [T, n, d]: entry 2i of the first ``dims`` is paired with entry 2i + 1."""
    if not dims:
        return x
    T = x.shape[0]
    a = _angles(T, dims, base, start)[:, None, :]
    c, s = torch.cos(a), torch.sin(a)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def masked_softmax(scores, window=None):
    """scores [.., T, T]: row i sees column j when 0 <= i - j (< window, if one is given)."""
    T = scores.shape[-1]
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    seen = (j <= i) if window is None else ((j <= i) & (i - j < window))
    return torch.softmax(scores.masked_fill(~seen, float("-inf")), -1)


def differential_attention(h, w, p, m, eps):
    """Two softmax maps a head over the same values, the second taken off the first lambda times; q, k and v pass a short
    causal convolution before the rotation.  h [T, W]; p the tensors' prefix; m the mixer's configuration."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = h @ w[p + ".q"].T + w[p + ".q.b"]
    k = h @ w[p + ".k"].T + w[p + ".k.b"]
    v = h @ w[p + ".v"].T + w[p + ".v.b"]
    if m.get("conv"):
        q, k, v = causal_conv(q, w[p + ".q.conv"]), causal_conv(k, w[p + ".k.conv"]), causal_conv(v, w[p + ".v.conv"])
    rot = m.get("rot") or {"dims": 0, "base": 1.0}
    q = rotate_halves(q.view(T, H * 2, d), rot["dims"], rot["base"]).view(T, H, 2, d)
    k = rotate_halves(k.view(T, G * 2, d), rot["dims"], rot["base"]).view(T, G, 2, d)
    v = v.view(T, G, dv)
    lam = torch.exp((w[p + ".lq1"] * w[p + ".lk1"]).sum()) - torch.exp((w[p + ".lq2"] * w[p + ".lk2"]).sum()) + m["diff"]
    window = (m.get("mask") or {}).get("size")
    gate = torch.sigmoid(h @ w[p + ".g"].T)                       # [T, H]
    heads = []
    for a in range(H):
        g = a // (H // G)
        maps = []
        for z in range(2):
            s = (q[:, a, z] @ k[:, g, z].T) * m["scale"]
            maps.append(masked_softmax(s, window) @ v[:, g])
        o = maps[0] - lam * maps[1]
        o = rms_unit(o, eps) * (1.0 - m["diff"])
        heads.append(o * gate[:, a:a + 1])
    return torch.cat(heads, -1) @ w[p + ".o"].T


def latent_rows(h, w, p, m, eps):
    """What a latent-attention layer keeps of a token: the normed latent and the one rotated key part all heads share."""
    T = h.shape[0]
    r, dr = m["kv_rank"], m["rot_dim"]
    down = h @ w[p + ".dkv"].T
    c = rms_unit(down[:, :r], eps) * w[p + ".dkv.norm"]
    rot = m.get("rot") or {"dims": 0, "base": 1.0}
    kr = rotate_pairs(down[:, r:].view(T, 1, dr), rot["dims"], rot["base"]).view(T, dr)
    return c, kr


def latent_attention(h, w, p, m, eps, kept=None):
    """Causal attention whose keys and values are linear in the kept latent; ``kept`` (c, rotated key part) comes from another
    layer when this one keeps none of its own."""
    T = h.shape[0]
    H, d, dr, dv = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    c, kr = kept if kept is not None else latent_rows(h, w, p, m, eps)
    q = (h @ w[p + ".q"].T).view(T, H, d + dr)
    rot = m.get("rot") or {"dims": 0, "base": 1.0}
    qn, qr = q[..., :d], rotate_pairs(q[..., d:], rot["dims"], rot["base"])
    kn = (c @ w[p + ".uk"].T).view(T, H, d)
    v = (c @ w[p + ".uv"].T).view(T, H, dv)
    gate = torch.sigmoid(h @ w[p + ".g"].T)
    heads = []
    for a in range(H):
        s = (qn[:, a] @ kn[:, a].T + qr[:, a] @ kr.T) * m["scale"]
        heads.append((masked_softmax(s) @ v[:, a]) * gate[:, a:a + 1])
    return torch.cat(heads, -1) @ w[p + ".o"].T


def matrix_lstm(h, w, p, m, eps, state=None):
    """The matrix memory, token by token.  ``state`` (S [H, d, dv], n [H, d], m [H]) carries on from an earlier call."""
    T = h.shape[0]
    H, d, dv, cap = m["heads"], m["dim"], m["vdim"], m["gate_cap"]
    q = (h @ w[p + ".q"].T).view(T, H, d) * d ** -0.5
    k = (h @ w[p + ".k"].T).view(T, H, d)
    v = (h @ w[p + ".v"].T).view(T, H, dv)
    gi = cap * torch.tanh((h @ w[p + ".i"].T + w[p + ".i.b"]) / cap)
    gf = torch.nn.functional.logsigmoid(cap * torch.tanh((h @ w[p + ".f"].T + w[p + ".f.b"]) / cap))
    if state is None:
        state = (torch.zeros(H, d, dv, dtype=F), torch.zeros(H, d, dtype=F), torch.zeros(H, dtype=F))
    S, n, mx = (t.clone() for t in state)
    out = torch.zeros(T, H, dv, dtype=F)
    for t in range(T):
        new = torch.maximum(gf[t] + mx, gi[t])
        keep, take = torch.exp(gf[t] + mx - new), torch.exp(gi[t] - new)
        S = keep[:, None, None] * S + take[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = keep[:, None] * n + take[:, None] * k[t]
        mx = new
        num = torch.einsum("hde,hd->he", S, q[t])
        den = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-mx)) + 1e-6
        out[t] = num / den[:, None]
    o = rms_unit(out, eps).reshape(T, H * dv) * w[p + ".norm"] * torch.sigmoid(h @ w[p + ".g"].T)
    return o @ w[p + ".o"].T, (S, n, mx)


def squared_relu_expert(x, up, down):
    return torch.relu(x @ up.T) ** 2 @ down.T


def route(h, w_router, top):
    """Sigmoid scores; the ``top`` largest are chosen (the lower index on a tie) and keep their scores as weights."""
    s = torch.sigmoid(h @ w_router.T)
    order = torch.sort(s, dim=-1, descending=True, stable=True).indices[:, :top]
    return order, torch.gather(s, 1, order)


def routed_feed_forward(h, w, p, mlp):
    """Each token's chosen experts read the token TIMES its score; a shared expert reads every token as it is."""
    ids, weights = route(h, w[p + ".router"], mlp["router"]["top"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, s in zip(ids[t].tolist(), weights[t]):
            out[t] += squared_relu_expert(s * h[t], w[f"{p}.e{e}.up"], w[f"{p}.e{e}.down"])
    if mlp.get("shared"):
        out = out + squared_relu_expert(h, w[p + ".shared.up"], w[p + ".shared.down"])
    return out


def forward(cfg, weights, tokens, streams=None):
    """Logits [T, vocab] of a whole sequence.  ``streams`` (a list) receives the residual stream after every layer."""
    w = {k: v.to(F) for k, v in weights.items() if v.is_floating_point()}
    eps = cfg["norm"]["eps"]
    x = embed(tokens, w["embed"], (cfg.get("embedding") or {}).get("scale", 1.0))
    kept = {}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}", L["mixer"]
        h = offset_norm(x, w[p + ".norm1"], eps)
        if L["type"] == "attention":
            a = differential_attention(h, w, p + ".mix", m, eps)
        elif L["type"] == "mlstm":
            a, _ = matrix_lstm(h, w, p + ".mix", m, eps)
        elif L["type"] == "latent_attention":
            if m.get("kv_from") is None:
                kept[i] = latent_rows(h, w, p + ".mix", m, eps)
            a = latent_attention(h, w, p + ".mix", m, eps, kept[i if m.get("kv_from") is None else m["kv_from"]])
        else:
            raise ValueError(L["type"])
        x = x + a
        if L.get("mlp") is not None:
            x = x + routed_feed_forward(offset_norm(x, w[p + ".norm2"], eps), w, p + ".mlp", L["mlp"])
        if streams is not None:
            streams.append(x.clone())
    return offset_norm(x, w["final.norm"], eps) @ w["head"].T
