"""A plain, slow statement of the Notedra architecture in float64, one function per mechanism, written from the
model's equations and sharing no code with the package.  Everything works on whole sequences except the
functions that carry state, which exist so that the statement itself can be run token by token.

Notation: x [S, W] the residual stream, h its normed copy, p positions 0 .. S-1.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence

import torch

DT = torch.float64


def load_folder(model_dir: str):
    from safetensors.torch import load_file
    with open(os.path.join(model_dir, "config.json")) as fh:
        cfg = json.load(fh)
    w = {k: (v.to(DT) if v.is_floating_point() else v) for k, v in
         load_file(os.path.join(model_dir, "model.safetensors")).items()}
    return cfg, w


# -- norms ---------------------------------------------------------------------------------
def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def offset_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """RMS norm whose weight is stored around zero."""
    return unit_rms(x, eps) * (1.0 + w)


# -- activations ---------------------------------------------------------------------------
def relu_squared(z: torch.Tensor) -> torch.Tensor:
    return torch.clamp(z, min=0.0) ** 2


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


# -- rotation ------------------------------------------------------------------------------
def rotate_pairs(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """x [S, heads, d]: neighbours (2i, 2i+1), i < dims/2, turn by p * base^(-2i/dims); the rest stays."""
    out = x.clone()
    for i in range(dims // 2):
        angle = positions.to(DT) * (base ** (-2.0 * i / dims))
        c, s = torch.cos(angle)[:, None], torch.sin(angle)[:, None]
        u, v = x[..., 2 * i], x[..., 2 * i + 1]
        out[..., 2 * i] = u * c - v * s
        out[..., 2 * i + 1] = v * c + u * s
    return out


# -- attention -----------------------------------------------------------------------------
def window_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float,
                     window_shift: int = 0) -> torch.Tensor:
    """Grouped-query attention of a whole sequence; ``window_shift`` widens or narrows the window (for
    showing that a comparison would notice a window that is one position off)."""
    S = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).view(S, H, d)
    k = (h @ w[p + "k"].T).view(S, G, d)
    v = (h @ w[p + "v"].T).view(S, G, dv)
    pos = torch.arange(S)
    if m.get("rot"):
        q = rotate_pairs(q, pos, m["rot"]["dims"], m["rot"]["base"])
        k = rotate_pairs(k, pos, m["rot"]["dims"], m["rot"]["base"])
    q, k = unit_rms(q, eps), unit_rms(k, eps)
    scale = m.get("scale", d ** -0.5)
    size = (m["mask"]["size"] + window_shift) if m.get("mask") else None
    out = torch.zeros(S, H, dv, dtype=DT)
    for head in range(H):
        g = head // (H // G)
        for i in range(S):
            lo = 0 if size is None else max(0, i - size + 1)
            scores = (k[lo:i + 1, g] @ q[i, head]) * scale
            weights = torch.softmax(scores, dim=0)
            out[i, head] = weights @ v[lo:i + 1, g]
    return out.reshape(S, H * dv) @ w[p + "o"].T


# -- matrix memory ---------------------------------------------------------------------------
def mlstm_gates(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, cap: float):
    """Capped log input gate and log forget gate, [S, heads] each."""
    i = cap * torch.tanh((h @ w[p + "i"].T + w[p + "i.b"]) / cap)
    f = torch.nn.functional.logsigmoid(cap * torch.tanh((h @ w[p + "f"].T + w[p + "f.b"]) / cap))
    return i, f


def mlstm_step(state, q, k, v, i, f):
    """One token of one head.  state = (S [d, dv], n [d], m scalar) or None for the start."""
    d, dv = k.shape[0], v.shape[0]
    if state is None:
        state = (torch.zeros(d, dv, dtype=DT), torch.zeros(d, dtype=DT), torch.zeros((), dtype=DT))
    S, n, m = state
    m_new = torch.maximum(f + m, i)
    keep, take = torch.exp(f + m - m_new), torch.exp(i - m_new)
    S = keep * S + take * torch.outer(k, v)
    n = keep * n + take * k
    o = (S.T @ q) / (torch.maximum((n @ q).abs(), torch.exp(-m_new)) + 1e-6)
    return (S, n, m_new), o


def mlstm_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float, states: Optional[list] = None):
    """The mixer over a sequence (or a further portion of one, when ``states`` carries a list per head)."""
    S = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).view(S, H, d) * d ** -0.5
    k = (h @ w[p + "k"].T).view(S, H, d)
    v = (h @ w[p + "v"].T).view(S, H, dv)
    ig, fg = mlstm_gates(h, w, p, m["gate_cap"])
    states = [None] * H if states is None else states
    o = torch.zeros(S, H, dv, dtype=DT)
    for head in range(H):
        for t in range(S):
            states[head], o[t, head] = mlstm_step(states[head], q[t, head], k[t, head], v[t, head], ig[t, head], fg[t, head])
    o = unit_rms(o, eps).reshape(S, H * dv) * w[p + "norm"]
    o = o * torch.sigmoid(h @ w[p + "g"].T)
    return o @ w[p + "o"].T, states


# -- feed-forward ----------------------------------------------------------------------------
def dense_ff(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    return relu_squared(h @ w[p + "up"].T + w[p + "up.b"]) @ w[p + "down"].T + w[p + "down.b"]


def router_scores(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str):
    """(s, choice scores): sigmoid of the router logits, and the same plus the correction."""
    s = torch.sigmoid(h @ w[p + "router"].T)
    return s, s + w[p + "correction"]


def mixture_ff(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, mlp: dict, forced: Optional[list] = None,
               margins: Optional[list] = None) -> torch.Tensor:
    """``forced[t]``: the experts to use for row t instead of the top ones (a list of ``top`` ids); ``margins``
    then receives, per row, how far the forced set's lowest choice score lies below the true top set's lowest."""
    top, scale = mlp["router"]["top"], mlp["router"].get("scale", 1.0)
    s, choice = router_scores(h, w, p)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        best = torch.topk(choice[t], top).indices.tolist()
        use = best if forced is None else list(forced[t])
        if margins is not None:
            margins.append(float(min(choice[t, e] for e in best) - min(choice[t, e] for e in use)))
        for e in use:
            y = relu_squared(h[t] @ w[f"{p}e{e}.up"].T) @ w[f"{p}e{e}.down"].T
            out[t] += scale * s[t, e] * y
    return out


# -- the model ---------------------------------------------------------------------------------
def layer_runs(cfg: dict) -> List[tuple]:
    """(layer, pass number or None) in running order."""
    n, loop = len(cfg["layers"]), cfg.get("loop")
    runs, i = [], 0
    while i < n:
        if loop and i == loop["start"]:
            for t in range(loop["times"]):
                runs += [(j, t) for j in range(loop["start"], loop["stop"])]
            i = loop["stop"]
        else:
            runs.append((i, None))
            i += 1
    return runs


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: Sequence[int], forced: Optional[list] = None,
            margins: Optional[list] = None, window_shift: int = 0, streams: Optional[list] = None) -> torch.Tensor:
    """Logits [S, vocab] of a whole sequence.  ``forced[r][t]``: experts of row t in the r-th routed layer run."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.tensor(list(tokens))]
    x0 = x.clone()
    loop = cfg.get("loop")
    routed = 0
    for layer, t in layer_runs(cfg):
        if t is not None and layer == loop["start"]:
            x = torch.cat([x, x0], dim=1) @ w["loop.in"].T + w["loop.step"][t]
        c, p = cfg["layers"][layer], f"l{layer}."
        h = offset_norm(x, w[p + "norm1"], eps)
        if c["type"] == "mlstm":
            mixed, _ = mlstm_mixer(h, w, p + "mix.", c["mixer"], eps)
        else:
            mixed = window_attention(h, w, p + "mix.", c["mixer"], eps, window_shift)
        mlp = c.get("mlp")
        if mlp is None:
            ff = torch.zeros_like(x)
        elif mlp["kind"] == "dense":
            ff = dense_ff(h, w, p + "mlp.")
        else:
            rows = [] if margins is not None else None
            ff = mixture_ff(h, w, p + "mlp.", mlp, None if forced is None else forced[routed], rows)
            if margins is not None:
                margins.append(rows)
            routed += 1
        x = x + (mixed + ff)
        if streams is not None:
            streams.append(x.clone())
    return offset_norm(x, w["final.norm"], eps) @ w["embed"].T


def generate_greedy(cfg: dict, w: Dict[str, torch.Tensor], prompt: Sequence[int], n: int) -> List[int]:
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(torch.argmax(forward(cfg, w, toks)[-1])))
    return toks[len(prompt):]
