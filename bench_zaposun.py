"""``bench.py --preset zaposun``: prefill and decode throughput of the Zaposun architecture at layer sizes that
resemble a real model's, beside Notedra (the framework's closest architecture: parallel layers, a recurrent mixer
with per-request state beside masked attention) at equal width and depth, both with random bfloat16 weights on one
B200.

Per width W, Zaposun has ten layers, parallel and wkv in turn, over four residual streams with norms in four groups:
the parallel mixer pairs chunked attention (W / 128 heads of size 128 for keys and values, a quarter as many key/value
heads, the leading 64 elements rotated, chunks of 1024 positions) with a selective scan (2 W channels, 16 states,
step-size rank W / 16, four taps); the wkv mixer has W / 64 heads of 64 and a decay rank of 64; every layer has a
dense gated feed-forward of 4 W.  Notedra is the configuration of ``--preset notedra`` (five layers that run twice).

Timing as in ``bench_notedra.py``: CUDA events after warm-up, a step's weights, state and cache exceed the L2 cache.
"""
from __future__ import annotations

import json
import time

from bench_notedra import _measure, notedra_config


def zaposun_config(W: int, vocab: int = 32768) -> dict:
    ah = max(1, W // 128)
    left = {"heads": ah, "kv_heads": max(1, ah // 4), "dim": 128, "vdim": 128, "scale": 128 ** -0.5,
            "rot": {"dims": 64, "base": 500000.0}, "mask": {"size": 1024}}
    right = {"inner": 2 * W, "state": 16, "dt_rank": max(1, W // 16), "conv": 4}
    wkv = {"heads": max(1, W // 64), "dim": 64, "decay_rank": 64}
    layers = []
    for i in range(10):
        mixer = {"left": dict(left), "right": dict(right)} if i % 2 == 0 else dict(wkv)
        layers.append({"type": "parallel" if i % 2 == 0 else "wkv", "mixer": mixer, "mlp": {"kind": "dense", "ff": 4 * W}})
    return {"architecture": "Zaposun", "vocab": vocab, "width": W, "streams": 4, "logit_scale": 1.0,
            "norm": {"eps": 1e-6, "groups": 4},
            "embedding": {"bigram": {"buckets": 65521, "mul_prev": 1000003, "mul_cur": 7919}}, "layers": layers}


def run(ns, pk, pk_kind) -> int:
    widths = [int(w) for w in ns.widths.split(",") if w.strip()]
    batches = [int(b) for b in ns.points.split(",") if b.strip()] or [8]
    t0 = time.time()
    sizes = {}
    for W in widths:
        sizes[str(W)] = {
            "zaposun": _measure("zaposun", zaposun_config(W), ns.prefill_tokens, batches, ns.context, ns.steps, max(ns.warmup, 3)),
            "notedra": _measure("notedra", notedra_config(W), ns.prefill_tokens, batches, ns.context, ns.steps, max(ns.warmup, 3)),
        }
    first = sizes[str(widths[0])]["zaposun"]["decode"][str(batches[0])]
    print(json.dumps({
        "metric": "decode tokens/s, Zaposun layer sizes beside Notedra at equal width (random bf16 weights)",
        "value": first["tokens_per_s"], "unit": "tokens/s", "n_gpus": 1, "steps": ns.steps, "warmup": max(ns.warmup, 3),
        "ms_per_step": first["ms_per_step"], "higher_is_better": True, "dtype": "bf16", "data": "synthetic",
        "config": {"preset": "zaposun", "widths": widths, "prefill_tokens": ns.prefill_tokens, "context": ns.context,
                   "batches": batches, "l2": "weights, state and cache of a step exceed the L2 cache"},
        "peaks": dict(pk, kind=pk_kind), "sizes": sizes, "seconds": round(time.time() - t0, 1)}))
    return 0
