"""Pamarax in plain PyTorch on the CPU, float64, one function per mechanism, one token sequence at a time and
nothing kept between calls: what the engine's kernels, caches and state slots are compared with.

Notation: x is the residual stream [T, width]; positions count from 0; weights are stored [out, in];
w maps tensor names to float64 tensors; p is a layer's tensor prefix ("l3").
"""

import math

import torch

F64 = torch.float64


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_one_plus(x, weight, eps):
    """The layer norms: the file holds gain - 1."""
    return unit_rms(x, eps) * (1.0 + weight)


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


def logsigmoid(z):
    return -softplus(-z)


def capped(z, cap):
    return cap * torch.tanh(z / cap)


# ------------------------------------------------------------------------------------------ attention

def rotate_half(x, positions, dims, base):
    """x [T, heads, dim]: the first ``dims`` entries of each head turn by position * base^(-2i/dims), entry i
    paired with entry i + dims/2; the rest pass."""
    if not dims:
        return x
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F64)
    a = torch.as_tensor(positions, dtype=F64)[:, None] * f[None, :]
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], -1)


def causal_attention(q, k, v, scale, extra_one):
    """q [T, H, d], k [T, G, d], v [T, G, e], token t at position t.  One token and one head at a time.  With
    ``extra_one`` the softmax's denominator also holds a one: a sink with score zero that has no value."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[-1], dtype=F64)
    for t in range(T):
        for h in range(H):
            g = h // (H // G)
            s = (k[:t + 1, g] @ q[t, h]) * scale
            m = s.max()
            if extra_one:
                m = torch.clamp(m, min=0.0)
            e = torch.exp(s - m)
            den = e.sum() + (math.exp(-float(m)) if extra_one else 0.0)
            out[t, h] = (e / den) @ v[:t + 1, g]
    return out


def gated_attention_mixer(h, w, p, m, eps):
    """The value of a token is its raw key projection (taken ahead of the norm and the rotation); q and k are normed over the whole projection;
    part of each head is rotated; the heads' outputs are gated by sigmoid(W_g h)."""
    T = h.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    q, k = h @ w[f"{p}.mix.q"].T, h @ w[f"{p}.mix.k"].T
    v = k.view(T, G, d)
    q = (unit_rms(q, eps) * w[f"{p}.mix.q.norm"]).view(T, H, d)
    k = (unit_rms(k, eps) * w[f"{p}.mix.k.norm"]).view(T, G, d)
    rot = m.get("rot") or {}
    pos = list(range(T))
    q, k = rotate_half(q, pos, rot.get("dims", 0), rot.get("base", 1.0)), rotate_half(k, pos, rot.get("dims", 0), rot.get("base", 1.0))
    o = causal_attention(q, k, v, m["scale"], False).reshape(T, H * d)
    return (o * torch.sigmoid(h @ w[f"{p}.mix.g"].T)) @ w[f"{p}.mix.o"].T


def query_temperature(T, coef, every):
    return torch.tensor([1.0 + coef * math.log((t + 1) // every + 1) for t in range(T)], dtype=F64)


def sink_attention_mixer(h, w, p, m, eps):
    """The left half of a parallel mixer: per-head q/k norm with one weight for all heads, no rotation, a query
    temperature that grows with the position, a softmax whose denominator holds one more."""
    T = h.shape[0]
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[f"{p}.q"].T).view(T, H, d)
    k = (h @ w[f"{p}.k"].T).view(T, G, d)
    v = (h @ w[f"{p}.v"].T).view(T, G, e)
    q = unit_rms(q, eps) * w[f"{p}.q.norm"]
    k = unit_rms(k, eps) * w[f"{p}.k.norm"]
    qt = m.get("q_temp")
    if qt:
        q = q * query_temperature(T, qt["coef"], qt["every"])[:, None, None]
    o = causal_attention(q, k, v, m["scale"], True).reshape(T, H * e)
    return o @ w[f"{p}.o"].T


# ------------------------------------------------------------------------------------------ recurrences

def causal_conv_silu(u, taps_w):
    """u [T, C], taps_w [C, taps] (the last column meets the current token), zeros before the start, no bias."""
    T, C = u.shape
    taps = taps_w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=F64), u], 0)
    out = torch.zeros(T, C, dtype=F64)
    for j in range(taps):
        out += padded[j:j + T] * taps_w[:, j]
    return silu(out)


def unit_vector(x):
    return x / torch.sqrt((x * x).sum(-1, keepdim=True) + 1e-6)


def gated_delta_rule(q, k, v, beta, g):
    """q, k [T, G, d], v [T, H, e], beta and g [T, H].  Per head: S <- g S; u = beta (v - S^T k); S <- S + k u^T;
    o = S^T q."""
    T, H, e = v.shape
    G, d = q.shape[1], q.shape[2]
    out = torch.zeros(T, H, e, dtype=F64)
    for h in range(H):
        kh = h // (H // G)
        S = torch.zeros(d, e, dtype=F64)
        for t in range(T):
            S = g[t, h] * S
            u = beta[t, h] * (v[t, h] - S.T @ k[t, kh])
            S = S + torch.outer(k[t, kh], u)
            out[t, h] = S.T @ q[t, kh]
    return out


def delta_mixer(h, w, p, m, eps):
    """The right half of a parallel mixer."""
    T = h.shape[0]
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = causal_conv_silu(h @ w[f"{p}.q"].T, w[f"{p}.q.conv"]).view(T, G, d)
    k = causal_conv_silu(h @ w[f"{p}.k"].T, w[f"{p}.k.conv"]).view(T, G, d)
    v = causal_conv_silu(h @ w[f"{p}.v"].T, w[f"{p}.v.conv"]).view(T, H, e)
    q, k = unit_vector(q) * d ** -0.5, unit_vector(k)
    beta = torch.sigmoid(h @ w[f"{p}.b"].T)
    g = torch.exp(-torch.exp(w[f"{p}.A_log"]) * softplus(h @ w[f"{p}.a"].T + w[f"{p}.dt_bias"]))
    o = gated_delta_rule(q, k, v, beta, g)
    o = unit_rms(o, eps) * w[f"{p}.norm"]
    o = o.reshape(T, H * e) * silu(h @ w[f"{p}.g"].T)
    return o @ w[f"{p}.o"].T


def matrix_memory(q, k, v, i_log, f_log):
    """q, k [T, H, d], v [T, H, e], log gates [T, H].  Per head, with a running maximum m that starts at zero:
    m' = max(f + m, i); S' = exp(f + m - m') S + exp(i - m') k v^T; n' likewise with k alone;
    o = S'^T q / (max(|n' . q|, exp(-m')) + 1e-6)."""
    T, H, e = v.shape
    d = q.shape[2]
    out = torch.zeros(T, H, e, dtype=F64)
    for h in range(H):
        S, n, m = torch.zeros(d, e, dtype=F64), torch.zeros(d, dtype=F64), torch.zeros((), dtype=F64)
        for t in range(T):
            m_new = torch.maximum(f_log[t, h] + m, i_log[t, h])
            a, b = torch.exp(f_log[t, h] + m - m_new), torch.exp(i_log[t, h] - m_new)
            S = a * S + b * torch.outer(k[t, h], v[t, h])
            n = a * n + b * k[t, h]
            m = m_new
            den = torch.maximum(torch.abs(n @ q[t, h]), torch.exp(-m)) + 1e-6
            out[t, h] = (S.T @ q[t, h]) / den
    return out


def mlstm_mixer(h, w, p, m, eps):
    T = h.shape[0]
    H, d, e, cap = m["heads"], m["dim"], m["vdim"], m["gate_cap"]
    q = (h @ w[f"{p}.mix.q"].T).view(T, H, d) * d ** -0.5
    k = (h @ w[f"{p}.mix.k"].T).view(T, H, d)
    v = (h @ w[f"{p}.mix.v"].T).view(T, H, e)
    i_log = capped(h @ w[f"{p}.mix.i"].T + w[f"{p}.mix.i.b"], cap)
    f_log = logsigmoid(capped(h @ w[f"{p}.mix.f"].T + w[f"{p}.mix.f.b"], cap))
    o = unit_rms(matrix_memory(q, k, v, i_log, f_log), eps).reshape(T, H * e) * w[f"{p}.mix.norm"]
    return (o * torch.sigmoid(h @ w[f"{p}.mix.g"].T)) @ w[f"{p}.mix.o"].T


def parallel_mixer(h, w, p, m, eps):
    left = sink_attention_mixer(h, w, f"{p}.mix.left", m["left"], eps)
    right = delta_mixer(h, w, f"{p}.mix.right", m["right"], eps)
    return m["left_scale"] * left + m["right_scale"] * right


# ------------------------------------------------------------------------------------------ feed-forward, model

def dense_ff(h, w, p):
    g = h @ w[f"{p}.mlp.gate"].T + w[f"{p}.mlp.gate.b"]
    u = h @ w[f"{p}.mlp.up"].T + w[f"{p}.mlp.up.b"]
    return (silu(g) * u) @ w[f"{p}.mlp.down"].T + w[f"{p}.mlp.down.b"]


MIXERS = {"attention": gated_attention_mixer, "mlstm": mlstm_mixer, "parallel": parallel_mixer}


def forward(cfg, w, tokens, want_layers=False):
    """Logits [T, vocab] of one sequence; with ``want_layers`` also the stream after every layer."""
    w = {k: v.to(F64) for k, v in w.items()}
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)] * cfg["embedding"]["scale"]
    streams = []
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}"
        a = MIXERS[L["type"]](norm_one_plus(x, w[f"{p}.norm1"], eps), w, p, L["mixer"], eps)
        x = x + norm_one_plus(a, w[f"{p}.norm1b"], eps)
        if L.get("mlp") is not None:
            f = dense_ff(norm_one_plus(x, w[f"{p}.norm2"], eps), w, p)
            x = x + norm_one_plus(f, w[f"{p}.norm2b"], eps)
        streams.append(x)
    logits = norm_one_plus(x, w["final.norm"], eps) @ w["head"].T
    return (logits, streams) if want_layers else logits


def greedy(logits):
    return int(torch.argmax(logits))
