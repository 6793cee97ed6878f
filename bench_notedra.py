"""``bench.py --preset notedra``: prefill and decode throughput of the Notedra architecture at layer sizes that
resemble a real model's, beside Llama 4 (the framework's other architecture) at equal width, depth and head sizes,
both with random bfloat16 weights on one B200.

Per width W: Notedra has five layers (attention, mlstm, mlstm, attention, mlstm) that all run twice (ten layer
runs); matrix-memory heads of key size 128 and value size 256 (W / 256 of them), attention heads of size 128 (W /
128, a quarter as many key/value heads) under a window of 1024 positions, a dense feed-forward of 4 W on the
second layer and 16 experts of W / 2 with two a row on the others.  Llama 4 has ten layers of the same
attention sizes under a chunk of 1024 positions, 16 experts of W / 2 with one a row plus the shared expert.

Timed with CUDA events after warm-up; every step's weights, state and cache exceed the L2 cache.  Prefill: one
request's whole prompt in one step.  Decode: `batch` requests at `context` positions, one token each a step, argmax
on the device, replayed as CUDA graphs where the engine does so.
"""
from __future__ import annotations

import json
import time


def notedra_config(W: int, vocab: int = 32768) -> dict:
    mh, ah = max(1, W // 256), max(1, W // 128)
    mlstm = {"heads": mh, "dim": 128, "vdim": 256, "gate_cap": 15.0}
    attn = {"heads": ah, "kv_heads": max(1, ah // 4), "dim": 128, "vdim": 128, "scale": 128 ** -0.5,
            "rot": {"dims": 64, "base": 500000.0}, "mask": {"size": 1024}}
    moe = {"kind": "moe", "expert": {"ff": W // 2}, "router": {"experts": 16, "top": 2, "scale": 2.0}}
    kinds = ["attention", "mlstm", "mlstm", "attention", "mlstm"]
    layers = [{"type": k, "mixer": dict(mlstm if k == "mlstm" else attn),
               "mlp": {"kind": "dense", "ff": 4 * W} if i == 1 else dict(moe)} for i, k in enumerate(kinds)]
    return {"architecture": "Notedra", "vocab": vocab, "width": W, "norm": {"eps": 1e-6}, "layers": layers,
            "loop": {"start": 0, "stop": 5, "times": 2}}


def llama4_config(W: int, vocab: int = 32768) -> dict:
    ah = max(1, W // 128)
    return dict(architectures=["Llama4ForCausalLM"], vocab_size=vocab, hidden_size=W, num_hidden_layers=10,
                num_attention_heads=ah, num_key_value_heads=max(1, ah // 4), head_dim=128, intermediate_size=W // 2,
                intermediate_size_mlp=4 * W, num_local_experts=16, num_experts_per_tok=1, interleave_moe_layer_step=1,
                rope_theta=10000.0, rope_scaling=None, no_rope_layers=[3, 7], attention_chunk_size=1024,
                use_qk_norm=True, attn_temperature_tuning=False, rms_norm_eps=1e-5, tie_word_embeddings=True)


def _measure(name: str, cfg_obj: dict, prompt: int, batches, context: int, steps: int, warmup: int) -> dict:
    import torch

    from sharpinference_b200 import Engine, EngineOptions, StepEntry, build_random_model
    from sharpinference_b200.kernels import library, ops
    from sharpinference_b200.registry import resolve
    dev = torch.device("cuda:0")
    _, cfg = resolve(cfg_obj, name)
    model = build_random_model(cfg, seed=0, dtype="bfloat16", device=dev, std=0.02, norm_std=0.0)
    page, max_b = 64, max(batches)
    engine = Engine(model, dtype="bfloat16", device=dev,
                    options=EngineOptions(page_size=page, max_batch=max_b + 1, max_tokens_per_step=max(prompt, max_b),
                                          max_cache_tokens=(max_b + 1) * (context + steps + warmup + 2 * page) + prompt))
    gen = torch.Generator().manual_seed(1)
    vocab = model.vocab_size

    def toks(n):
        return torch.randint(0, vocab, (n,), generator=gen).tolist()
    out = {"parameters_bytes": sum(t.numel() * t.element_size() for t in _tensors(model))}
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    # prefill: a fresh request's whole prompt, one step
    times = []
    for i in range(warmup + steps):
        engine.open_request("p")
        ids = toks(prompt)
        a.record()
        logits = engine.forward_step([StepEntry("p", ids, [prompt - 1])])
        ops.argmax_rows(logits)
        b.record()
        torch.cuda.synchronize()
        engine.close_request("p")
        if i >= warmup:
            times.append(a.elapsed_time(b))
    out["prefill"] = {"tokens": prompt, "ms": min(times), "tokens_per_s": prompt / min(times) * 1e3}
    # decode
    out["decode"] = {}
    for batch in batches:
        ids = [f"d{i}" for i in range(batch)]
        for rid in ids:
            engine.open_request(rid)
            done = 0
            while done < context:
                n = min(prompt, context - done)
                engine.forward_step([StepEntry(rid, toks(n), [])])
                done += n
        launches0 = None
        for i in range(warmup + steps):
            if i == warmup:
                torch.cuda.synchronize()
                launches0 = library.launch_count
                a.record()
            logits = engine.forward_step([StepEntry(rid, toks(1), [0]) for rid in ids])
            ops.argmax_rows(logits)
        b.record()
        torch.cuda.synchronize()
        engine.runner.flush_status()
        ms = a.elapsed_time(b) / steps
        out["decode"][str(batch)] = {"context": context, "ms_per_step": ms, "tokens_per_s": batch / ms * 1e3,
                                     "launches_per_step": (library.launch_count - launches0) / steps,
                                     "graph_replays": engine.runner.graph_replays}
        for rid in ids:
            engine.close_request(rid)
    del engine, model
    torch.cuda.empty_cache()
    return out


def _tensors(root, seen=None, depth=5):
    import torch
    seen = set() if seen is None else seen
    if id(root) in seen or depth < 0:
        return
    seen.add(id(root))
    if isinstance(root, torch.Tensor):
        yield root
    elif isinstance(root, (list, tuple)):
        for item in root:
            yield from _tensors(item, seen, depth)
    elif hasattr(root, "__dict__"):
        for v in vars(root).values():
            yield from _tensors(v, seen, depth - 1)


def run(ns, pk, pk_kind) -> int:
    widths = [int(w) for w in ns.widths.split(",") if w.strip()]
    batches = [int(b) for b in ns.points.split(",") if b.strip()] or [8]
    t0 = time.time()
    sizes = {}
    for W in widths:
        sizes[str(W)] = {
            "notedra": _measure("notedra", notedra_config(W), ns.prefill_tokens, batches, ns.context, ns.steps, max(ns.warmup, 3)),
            "llama4": _measure("llama4", llama4_config(W), ns.prefill_tokens, batches, ns.context, ns.steps, max(ns.warmup, 3)),
        }
    first = sizes[str(widths[0])]["notedra"]["decode"][str(batches[0])]
    print(json.dumps({
        "metric": "decode tokens/s, Notedra layer sizes beside Llama 4 at equal width (random bf16 weights)",
        "value": first["tokens_per_s"], "unit": "tokens/s", "n_gpus": 1, "steps": ns.steps, "warmup": max(ns.warmup, 3),
        "ms_per_step": first["ms_per_step"], "higher_is_better": True, "dtype": "bf16", "data": "synthetic",
        "config": {"preset": "notedra", "widths": widths, "prefill_tokens": ns.prefill_tokens, "context": ns.context,
                   "batches": batches, "l2": "weights, state and cache of a step exceed the L2 cache"},
        "peaks": dict(pk, kind=pk_kind), "sizes": sizes, "seconds": round(time.time() - t0, 1)}))
    return 0
