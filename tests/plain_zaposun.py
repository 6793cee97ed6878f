"""A plain, slow statement of the Zaposun architecture in float64, one function per mechanism.

It takes a configuration as the dictionary of ``config.json`` and the weights as a dictionary name -> tensor,
and runs one whole sequence at a time, token after token where the mechanism is a recurrence.  Nothing here is
shared with the engine: no part, no kernel, no configuration class.

Notation: ``T`` tokens, ``H`` the model width, ``S`` streams.  Linear weights are ``[out, in]`` and applied as
``x @ W.T``.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def group_norm(x, w, groups, eps):
    """The last axis in ``groups`` equal consecutive parts, each divided by its own root mean square; times w."""
    T, H = x.shape
    return (rms(x.reshape(T, groups, H // groups), eps).reshape(T, H)) * w


def previous_rows(h):
    """Row t holds h[t - 1]; row 0 holds zeros."""
    return torch.cat([torch.zeros_like(h[:1]), h[:-1]], dim=0)


def token_shift(h, mu):
    """h + (h' - h) * mu with h' the previous token's h (zeros before the first)."""
    return h + (previous_rows(h) - h) * mu


def embedding(tokens, embed, bigram, buckets, mul_prev, mul_cur):
    rows = []
    for t, tok in enumerate(tokens):
        rows.append(buckets if t == 0 else (tokens[t - 1] * mul_prev + tok * mul_cur) % buckets)
    return embed[torch.tensor(tokens)] + bigram[torch.tensor(rows)]


def rotate(x, positions, base, dims, layout, sign=1.0):
    """Turn the first ``dims`` elements of the last axis; x is [T, heads, d].  Pair i of ``dims / 2`` turns by
    ``sign * position * base^(-2 i / dims)``; layout 'halves' pairs i with i + dims/2, 'interleaved' 2i with 2i+1."""
    if dims == 0:
        return x
    half = dims // 2
    i = torch.arange(half, dtype=F64)
    freq = torch.pow(torch.tensor(float(base), dtype=F64), -2.0 * i / dims)
    ang = sign * positions.to(F64)[:, None] * freq[None, :]           # [T, half]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    out = x.clone()
    if layout == "halves":
        a, b = x[..., :half], x[..., half:dims]
        out[..., :half] = a * c - b * s
        out[..., half:dims] = b * c + a * s
    else:
        a, b = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = a * c - b * s
        out[..., 1:dims:2] = b * c + a * s
    return out


def chunk_attention(h, W, p, m, eps, layout="halves", chunk_delta=0):
    """The left branch of a 'parallel' mixer: grouped-query attention inside chunks of ``mask.size`` positions,
    q/k norm before a partial rotation, values rotated by their position and the head's sum turned back."""
    T = h.shape[0]
    nq, nkv, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = (h @ W[p + "q"].T).reshape(T, nq, d)
    k = (h @ W[p + "k"].T).reshape(T, nkv, d)
    v = (h @ W[p + "v"].T).reshape(T, nkv, dv)
    q = rms(q, eps) * W[p + "q.norm"]
    k = rms(k, eps) * W[p + "k.norm"]
    rot = m.get("rot") or {"dims": 0, "base": 10000.0}
    q = rotate(q, pos, rot["base"], rot["dims"], layout)
    k = rotate(k, pos, rot["base"], rot["dims"], layout)
    v = rotate(v, pos, rot["base"], dv, layout)
    size = (m.get("mask") or {}).get("size", 0)
    if size:
        size += chunk_delta                     # tests: what a chunk one position longer or shorter would give
    out = torch.zeros(T, nq, dv, dtype=F64)
    for i in range(T):
        lo = (i // size) * size if size else 0
        for hq in range(nq):
            g = hq // (nq // nkv)
            s = (k[lo:i + 1, g] @ q[i, hq]) * m["scale"]
            w = torch.softmax(s, dim=0)
            out[i, hq] = w @ v[lo:i + 1, g]
    out = rotate(out, pos, rot["base"], dv, layout, sign=-1.0)
    return out.reshape(T, nq * dv) @ W[p + "o"].T


def selective_scan(h, W, p, m):
    """The right branch of a 'parallel' mixer: Mamba."""
    T = h.shape[0]
    inner, N, R, taps = m["inner"], m["state"], m["dt_rank"], m["conv"]
    xz = h @ W[p + "in"].T
    x, z = xz[:, :inner], xz[:, inner:]
    conv, cb = W[p + "conv"], W[p + "conv.b"]
    xp = torch.cat([torch.zeros(taps - 1, inner, dtype=F64), x], dim=0)
    xc = torch.zeros_like(x)
    for j in range(taps):                       # the last column is the current token's
        xc += xp[j:j + T] * conv[:, j]
    x = silu(xc + cb)
    dbc = x @ W[p + "x"].T
    dt, B, C = dbc[:, :R], dbc[:, R:R + N], dbc[:, R + N:]
    dt = softplus(dt @ W[p + "dt"].T + W[p + "dt.b"])          # [T, inner]
    A = -torch.exp(W[p + "A_log"])                              # [inner, N]
    S = torch.zeros(inner, N, dtype=F64)
    y = torch.zeros(T, inner, dtype=F64)
    for t in range(T):
        S = torch.exp(dt[t][:, None] * A) * S + (dt[t] * x[t])[:, None] * B[t][None, :]
        y[t] = S @ C[t] + W[p + "D"] * x[t]
    return (y * silu(z)) @ W[p + "o"].T


def parallel_mixer(h, W, p, m, eps, layout="halves", chunk_delta=0):
    left = chunk_attention(h, W, p + "left.", m["left"], eps, layout, chunk_delta)
    right = selective_scan(h, W, p + "right.", m["right"])
    return 0.5 * (rms(left, eps) * W[p + "left.out"] + rms(right, eps) * W[p + "right.out"])


def wkv_mixer(h, W, p, m, eps):
    """RWKV-style time mixing with a decay that depends on the token."""
    T = h.shape[0]
    heads, d = m["heads"], m["dim"]
    prev = previous_rows(h)
    mix = {s: h + (prev - h) * W[p + "mu." + s] for s in "rkvgw"}
    r = (mix["r"] @ W[p + "r"].T).reshape(T, heads, d)
    k = (mix["k"] @ W[p + "k"].T).reshape(T, heads, d)
    v = (mix["v"] @ W[p + "v"].T).reshape(T, heads, d)
    gate = silu(mix["g"] @ W[p + "g"].T)
    w = torch.exp(-torch.exp(torch.tanh(mix["w"] @ W[p + "w1"].T) @ W[p + "w2"].T + W[p + "w0"])).reshape(T, heads, d)
    u = W[p + "u"]                                                  # [heads, d]
    S = torch.zeros(heads, d, d, dtype=F64)                         # [head, key channel, value channel]
    o = torch.zeros(T, heads, d, dtype=F64)
    for t in range(T):
        kv = k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hkv,hk->hv", S + u[:, :, None] * kv, r[t])
        S = w[t][:, :, None] * S + kv
    o = rms(o, eps).reshape(T, heads * d) * W[p + "norm"] * gate
    return o @ W[p + "o"].T


def gated_mlp(h, W, p):
    return (gelu_tanh(h @ W[p + "gate"].T) * (h @ W[p + "up"].T)) @ W[p + "down"].T


def load_folder(model_dir):
    import json
    import os

    from safetensors.torch import load_file
    with open(os.path.join(model_dir, "config.json")) as fh:
        cfg = json.load(fh)
    w = {k: (v.to(F64) if v.is_floating_point() else v) for k, v in
         load_file(os.path.join(model_dir, "model.safetensors")).items()}
    return cfg, w


def generate_greedy(config, W, prompt, n):
    toks, out = list(prompt), []
    for _ in range(n):
        nxt = int(torch.argmax(forward(config, W, toks)[-1]))
        out.append(nxt)
        toks.append(nxt)
    return out


def forward(config, W, tokens, *, want_layers=False, chunk_delta=0):
    """Logits [T, vocab] of one whole sequence (and the sum of the streams after every layer)."""
    W = {k: (v.to(F64) if v.is_floating_point() else v) for k, v in W.items()}
    eps, groups, S = config["norm"]["eps"], config["norm"].get("groups", 1), config.get("streams", 1)
    bg = config["embedding"]["bigram"]
    x0 = embedding(list(tokens), W["embed"], W["bigram"], bg["buckets"], bg["mul_prev"], bg["mul_cur"])
    xs = [x0.clone() for _ in range(S)]
    after = []
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        for q in (1, 2):
            if q == 2 and layer["mlp"] is None:
                continue
            hc = p + f"hc{q}."
            u = sum(W[hc + "in"][s] * xs[s] for s in range(S))
            h = group_norm(u, W[p + f"norm{q}"], groups, eps)
            if q == 1:
                h = token_shift(h, W[p + "shift"])
                if layer["type"] == "wkv":
                    y = wkv_mixer(h, W, p + "mix.", layer["mixer"], eps)
                else:
                    layout = (layer["mixer"]["left"].get("rot") or {}).get("layout", "halves")
                    y = parallel_mixer(h, W, p + "mix.", layer["mixer"], eps, layout, chunk_delta)
            else:
                y = gated_mlp(h, W, p + "mlp.")
            xs = [sum(W[hc + "mix"][s, t] * xs[s] for s in range(S)) + W[hc + "out"][t] * y for t in range(S)]
        after.append(sum(xs))
    x = group_norm(sum(xs), W["final.norm"], groups, eps)
    logits = (x @ W["head"].T) * config.get("logit_scale", 1.0)
    return (logits, after) if want_layers else logits
