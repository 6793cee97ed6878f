"""Small Zaposun configurations for the tests, and folders with random weights for them.

The configurations differ from each other in every size; between them they cover: one, two, three and four
residual streams; one to four norm groups; value heads wider and narrower than key heads; a rotation of part of a
head, of all of it and none, in both pair layouts; chunks shorter than a page, of exactly a page and longer than two;
layers without a feed-forward; wkv first and parallel first; a width that is no multiple of 8; convolutions of one
to five taps; state counts from 1 to 200; heads from 2 to 160 elements.

Random weights alone would hide some faults, so ``write`` edits a few tensors afterwards: the decay offsets of the
wkv layers and ``A_log`` of the scans are lowered (memories that keep what they saw hundreds of tokens ago: losing or
mixing up a state shows), the stream coefficients are set near an identity (so that the streams neither vanish nor
explode), the mixing vectors lie in (0, 1), and the attention score factor in the configurations is large (so that
single keys carry a row's output and a chunk that is one position off shows).
"""
from __future__ import annotations

import os

import torch


def _left(heads, kv, dim, vdim, scale, chunk, rot=None, layout=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": chunk}}
    if rot:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
        if layout:
            m["rot"]["layout"] = layout
    return m


def _right(inner, state, dt_rank, conv):
    return {"inner": inner, "state": state, "dt_rank": dt_rank, "conv": conv}


def _par(left, right, ff):
    return {"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def _wkv(heads, dim, rank, ff):
    return {"type": "wkv", "mixer": {"heads": heads, "dim": dim, "decay_rank": rank},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def _top(vocab, width, streams, groups, eps, scale, bigram, layers):
    return {"architecture": "Zaposun", "vocab": vocab, "width": width, "streams": streams, "logit_scale": scale,
            "norm": {"eps": eps, "groups": groups},
            "embedding": {"bigram": {"buckets": bigram[0], "mul_prev": bigram[1], "mul_cur": bigram[2]}},
            "layers": layers}


# P: two streams; value heads wider than keys with a rotation of half a head and a chunk of 7, then narrower with a
# rotation of the whole head and a chunk longer than a page; a wkv layer without a feed-forward.
CASE_P = _top(97, 64, 2, 2, 1e-5, 1.5, (53, 31, 5), [
    _par(_left(4, 2, 16, 32, 0.9, 7, rot=(8, 100.0)), _right(40, 5, 3, 3), 40),
    _wkv(2, 24, 6, 0),
    _par(_left(2, 2, 32, 16, 0.5, 70, rot=(32, 10000.0)), _right(24, 16, 4, 2), 24),
])

# Q: three streams and groups; head size 64 (the tensor-core attention kernels) under a chunk longer than two pages,
# neighbours paired; a chunk of exactly one page with unequal sizes; wkv heads of 64.
CASE_Q = _top(131, 72, 3, 3, 1e-6, 0.7, (211, 3, 17), [
    _wkv(1, 64, 8, 56),
    _par(_left(2, 1, 64, 64, 0.3, 130, rot=(64, 5000.0), layout="interleaved"), _right(48, 20, 5, 5), 0),
    _par(_left(4, 2, 32, 64, 0.4, 64, rot=(16, 50.0), layout="interleaved"), _right(80, 9, 2, 4), 32),
    _wkv(3, 8, 3, 16),
])

# R: a width that is no multiple of 8 (no library product anywhere), one stream, one group, no rotation of q and k,
# a convolution of one tap, head sizes that the tensor-core attention does not take.
CASE_R = _top(61, 52, 1, 1, 1e-4, 1.0, (7, 2, 3), [
    _wkv(2, 12, 5, 30),
    _par(_left(2, 2, 24, 40, 0.6, 33), _right(30, 3, 7, 1), 18),
    _par(_left(3, 1, 20, 10, 0.8, 5, rot=(4, 300.0)), _right(12, 33, 1, 3), 0),
])

# S: ones and twos wherever a size can be one or two.
CASE_S = _top(23, 16, 1, 2, 1e-5, 2.5, (1, 1, 1), [
    _par(_left(1, 1, 2, 2, 1.5, 1, rot=(2, 10.0)), _right(2, 1, 1, 2), 1),
    _wkv(1, 2, 1, 0),
    _par(_left(2, 1, 4, 2, 0.9, 2, rot=(2, 7.0)), _right(1, 2, 2, 2), 2),
])

# T: the largest heads: wkv heads of 128 and of 160, attention heads of 128 (the tcgen05 prompt kernel) and of 256,
# 64 and 200 states.
CASE_T = _top(50, 128, 4, 4, 1e-5, 1.0, (301, 7, 11), [
    _wkv(1, 128, 4, 0),
    _par(_left(2, 1, 128, 128, 0.08, 64, rot=(96, 10000.0)), _right(16, 64, 3, 4), 48),
    _wkv(1, 160, 2, 24),
    _par(_left(1, 1, 256, 32, 0.05, 100, rot=(256, 1000.0)), _right(8, 200, 2, 3), 0),
])

# U: wkv layers only (no keys or values anywhere: a model without a cache group); V: parallel layers only, two of
# them with equal attention sizes (one cache group of two entries) and one that sees every earlier position.
CASE_U = _top(40, 32, 2, 1, 1e-5, 1.0, (11, 5, 3), [_wkv(2, 16, 4, 24), _wkv(1, 32, 2, 0)])
CASE_V = _top(45, 48, 2, 3, 1e-5, 0.5, (19, 2, 9), [
    _par(_left(2, 1, 16, 16, 0.7, 9, rot=(16, 30.0)), _right(24, 8, 2, 3), 32),
    _par(_left(2, 1, 16, 16, 0.7, 9, rot=(16, 30.0)), _right(16, 4, 3, 2), 0),
    _par({"heads": 3, "kv_heads": 3, "dim": 8, "vdim": 8, "scale": 0.9}, _right(16, 12, 2, 4), 16),
])

# config, std of the weights, seed
CASES = {"P": (CASE_P, 0.12, 21), "Q": (CASE_Q, 0.1, 22), "R": (CASE_R, 0.15, 23), "S": (CASE_S, 0.4, 24),
         "T": (CASE_T, 0.08, 25), "U": (CASE_U, 0.2, 26), "V": (CASE_V, 0.15, 27)}


def write(name: str, out_dir: str) -> str:
    """``config.json`` and ``model.safetensors`` for a case: seeded random weights, then the edits named above."""
    from safetensors.torch import load_file

    from sharpinference_b200.weights import safetensors_io, write_random_model
    cfg, std, seed = CASES[name]
    write_random_model(dict(cfg), out_dir, seed, std=std, norm_std=0.1)
    path = os.path.join(out_dir, "model.safetensors")
    tensors = load_file(path)
    g = torch.Generator().manual_seed(seed + 1000)
    S = cfg["streams"]
    for key in list(tensors):
        t = tensors[key]
        rnd = torch.rand(t.shape, generator=g)
        if key.endswith(".mix.w0"):
            new = -4.0 + 2.5 * rnd                       # decays of exp(-exp(-4)) = 0.98 to exp(-exp(-1.5)) = 0.8
        elif key.endswith(".A_log"):
            new = -5.0 + 4.0 * rnd
        elif key.endswith(".shift") or ".mix.mu." in key:
            new = 0.05 + 0.9 * rnd
        elif key.endswith(".in") and ".hc" in key:
            new = (1.0 + 0.6 * (rnd - 0.5)) / S
        elif key.endswith(".out") and ".hc" in key:
            new = 1.0 + 0.6 * (rnd - 0.5)
        elif key.endswith(".mix") and ".hc" in key:
            new = torch.eye(S) + 0.4 * (rnd - 0.5)
        elif key.endswith(".dt.b"):
            new = -1.0 + 2.0 * rnd
        else:
            continue
        tensors[key] = new.to(t.dtype)
    safetensors_io.save_file(sorted(tensors.items()), path, metadata={"format": "pt"})
    return out_dir
