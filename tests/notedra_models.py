"""Small Notedra configurations for the tests, and folders with random weights for them.

The configurations differ from each other in every size; between them they cover: value heads wider and narrower
than key heads, a rotation of part of a head, of all of it and none, windows shorter than a page, longer than a
page and absent, one expert a row and several, expert widths that are and are not multiples of 8, a width that is
no multiple of 8, layers without a feed-forward, loops from the first layer, of one pass, and none.

Random weights alone would hide some faults, so ``write`` edits a few tensors afterwards: forget-gate biases are
raised (a matrix memory that keeps what it saw hundreds of tokens ago: losing or mixing up a state shows), the
router corrections are spread (so that the correction, not the score, decides many choices), and the attention
score factor in the configurations is large (so that single keys carry a row's output and a window that is one
position off shows).
"""
from __future__ import annotations

import os

import torch


def _attn(heads, kv, dim, vdim, scale, window=None, rot=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if rot:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
    if window:
        m["mask"] = {"size": window}
    return m


def _moe(experts, top, ff, scale):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "scale": scale}}


# P: a loop from the first layer on, three passes; unequal key and value sizes both ways; window of 5.
CASE_P = {
    "architecture": "Notedra", "vocab": 97, "width": 64, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "attention", "mixer": _attn(4, 2, 16, 16, 0.6, window=5, rot=(8, 100.0)), "mlp": {"kind": "dense", "ff": 40}},
        {"type": "mlstm", "mixer": {"heads": 2, "dim": 16, "vdim": 32, "gate_cap": 8.0}, "mlp": _moe(4, 1, 24, 1.5)},
        {"type": "mlstm", "mixer": {"heads": 1, "dim": 32, "vdim": 24, "gate_cap": 15.0}, "mlp": None},
        {"type": "attention", "mixer": _attn(3, 3, 32, 48, 0.3, window=70, rot=(32, 10000.0)), "mlp": _moe(6, 3, 16, 0.8)},
    ],
    "loop": {"start": 0, "stop": 2, "times": 3},
}

# Q: no loop; head size 64 (the tensor-core attention kernels), a window longer than two pages, an attention
# layer that sees everything and is not rotated, expert width no multiple of 8, value heads narrower than keys.
CASE_Q = {
    "architecture": "Notedra", "vocab": 131, "width": 72, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "mlstm", "mixer": {"heads": 3, "dim": 24, "vdim": 40, "gate_cap": 10.0}, "mlp": _moe(5, 2, 20, 2.0)},
        {"type": "attention", "mixer": _attn(2, 1, 64, 64, 0.11, window=130, rot=(64, 5000.0)), "mlp": {"kind": "dense", "ff": 56}},
        {"type": "attention", "mixer": _attn(4, 2, 32, 16, 0.25), "mlp": None},
        {"type": "mlstm", "mixer": {"heads": 2, "dim": 64, "vdim": 64, "gate_cap": 12.0}, "mlp": _moe(3, 3, 32, 1.0)},
    ],
}

# R: a width that is no multiple of 8 (no library product, no tensor-core product anywhere), a loop of one pass
# over the last layers, head sizes that the tensor-core attention does not take.
CASE_R = {
    "architecture": "Notedra", "vocab": 61, "width": 52, "norm": {"eps": 1e-4},
    "layers": [
        {"type": "mlstm", "mixer": {"heads": 2, "dim": 8, "vdim": 8, "gate_cap": 6.0}, "mlp": {"kind": "dense", "ff": 30}},
        {"type": "attention", "mixer": _attn(2, 2, 24, 40, 0.35, window=33, rot=(12, 300.0)), "mlp": _moe(7, 2, 12, 1.2)},
        {"type": "mlstm", "mixer": {"heads": 4, "dim": 12, "vdim": 20, "gate_cap": 9.0}, "mlp": _moe(2, 1, 18, 3.0)},
    ],
    "loop": {"start": 1, "stop": 3, "times": 1},
}

# S: ones and twos wherever a size can be one or two: one head, one key/value head, a head of two elements, a window
# of one position (a token sees itself only) and of two, one expert, a loop of one layer run four times, a dense
# network one wide.
CASE_S = {
    "architecture": "Notedra", "vocab": 23, "width": 16, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "attention", "mixer": _attn(1, 1, 2, 6, 1.5, window=1, rot=(2, 10.0)), "mlp": _moe(1, 1, 8, 1.0)},
        {"type": "mlstm", "mixer": {"heads": 1, "dim": 2, "vdim": 1, "gate_cap": 5.0}, "mlp": {"kind": "dense", "ff": 1}},
        {"type": "attention", "mixer": _attn(2, 1, 4, 2, 0.9, window=2, rot=(2, 7.0)), "mlp": _moe(2, 2, 3, 0.5)},
    ],
    "loop": {"start": 1, "stop": 2, "times": 4},
}

# T: the largest heads: a matrix memory with keys of 256 and of 136 elements, attention heads of 128 (the tcgen05
# prompt kernel) under a window of exactly one page and of 256 (no tensor-core attention kernel takes them), rotated
# in part.
CASE_T = {
    "architecture": "Notedra", "vocab": 50, "width": 128, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "mlstm", "mixer": {"heads": 1, "dim": 256, "vdim": 24, "gate_cap": 20.0}, "mlp": None},
        {"type": "attention", "mixer": _attn(2, 1, 128, 128, 0.05, window=64, rot=(96, 10000.0)), "mlp": _moe(3, 2, 64, 1.0)},
        {"type": "mlstm", "mixer": {"heads": 2, "dim": 136, "vdim": 72, "gate_cap": 12.0}, "mlp": {"kind": "dense", "ff": 48}},
        {"type": "attention", "mixer": _attn(1, 1, 256, 32, 0.03, window=100, rot=(256, 1000.0)), "mlp": None},
    ],
    "loop": {"start": 0, "stop": 4, "times": 2},
}

# config, std of the weights, seed
CASES = {"P": (CASE_P, 0.12, 11), "Q": (CASE_Q, 0.1, 12), "R": (CASE_R, 0.15, 13), "S": (CASE_S, 0.4, 14),
         "T": (CASE_T, 0.08, 15)}


def write(name: str, out_dir: str) -> str:
    """``config.json`` and ``model.safetensors`` for a case: seeded random weights, then the edits named above."""
    from safetensors.torch import load_file

    from sharpinference_b200.weights import safetensors_io, write_random_model
    cfg, std, seed = CASES[name]
    write_random_model(dict(cfg), out_dir, seed, std=std, norm_std=0.1)
    path = os.path.join(out_dir, "model.safetensors")
    tensors = load_file(path)
    g = torch.Generator().manual_seed(seed + 1000)
    for key in list(tensors):
        t = tensors[key]
        if key.endswith(".mix.f.b"):
            tensors[key] = (3.0 + 1.5 * torch.rand(t.shape, generator=g)).to(t.dtype)
        elif key.endswith(".mix.i.b"):
            tensors[key] = (torch.rand(t.shape, generator=g) - 0.5).to(t.dtype)
        elif key.endswith(".mlp.correction"):
            tensors[key] = (0.5 * torch.randn(t.shape, generator=g)).to(t.dtype)
        elif key.endswith(".mlp.router"):
            tensors[key] = (t.float() * 4.0).to(t.dtype)
    safetensors_io.save_file(sorted(tensors.items()), path, metadata={"format": "pt"})
    return out_dir
