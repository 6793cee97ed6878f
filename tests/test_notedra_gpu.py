"""Notedra on the GPU: each new kernel against the plain statement of its mechanism, and whole models through the
engine (step function, cache manager, scheduler) under every way of cutting the work, in 32-bit and in bfloat16."""

import pytest
import torch

import plain_notedra as plain
import traces
from notedra_models import CASES, write

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

# Relative to the largest |logit| of a request.  float32: every product and sum is 32-bit.  bfloat16: operands of
# matrix products are rounded to 8 bits of mantissa, everything else stays 32-bit.
TOL = {"float32": 5e-5, "bfloat16": 3e-2}
# An expert choice that differs from the plain implementation's must be a near-tie of the choice scores.
MARGIN = 2e-2
LENGTHS = {"P": [1, 9, 40, 83, 150, 2], "Q": [150, 5, 67, 200, 31], "R": [3, 70, 12, 45, 100, 64, 65],
           "S": [1, 2, 30, 5], "T": [140, 66, 3, 129]}


def requests_for(name):
    vocab = CASES[name][0]["vocab"]
    return {f"r{i}": traces.random_tokens(vocab, n, seed=31 * i + n) for i, n in enumerate(LENGTHS[name])}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {name: write(name, str(tmp_path_factory.mktemp(f"notedra_{name}"))) for name in CASES}


@pytest.fixture(scope="module")
def expected(folders):
    out = {}
    for name, folder in folders.items():
        cfg, w = plain.load_folder(folder)
        out[name] = {rid: plain.forward(cfg, w, toks) for rid, toks in requests_for(name).items()}
    return out


def engine_for(folder, dtype, max_tokens, max_batch=4, page_size=None, graphs=True):
    from sharpinference_b200 import Engine, EngineOptions
    opts = EngineOptions()
    if page_size:
        opts.page_size = page_size
    opts.max_cache_tokens = max(max_tokens, opts.page_size)
    opts.max_batch = max_batch
    opts.cuda_graphs = graphs
    return Engine(folder, dtype=dtype, device=DEV, options=opts)


def reference_for(folder, reqs, routing, fallback, dtype):
    """float32 runs are held to the plain logits as they are; bfloat16 runs to the plain logits under the engine's
    own expert choices, each differing choice having to be a near-tie."""
    if dtype == "float32":
        return fallback
    cfg, w = plain.load_folder(folder)
    ref = {}
    for rid, toks in reqs.items():
        margins = []
        ref[rid] = plain.forward(cfg, w, toks, forced=routing[rid], margins=margins)
        worst = max((m for run in margins for m in run), default=0.0)
        assert worst < MARGIN, f"request {rid}: an expert choice differs beyond a near-tie ({worst})"
    return ref


# Case T has a position at which rounding alone is amplified beyond TOL (the matrix memory divides by a normaliser
# that passes close to its floor there): in bfloat16 a position's limit is the larger of TOL and three times the
# error that rounding the normed activations to bfloat16 causes in the plain model at that position.
_noise = {}


def rounding_noise(folder, name):
    if name not in _noise:
        cfg, w = plain.load_folder(folder)
        plain_norm = plain.offset_norm
        out = {}
        try:
            for rid, toks in requests_for(name).items():
                exact = plain.forward(cfg, w, toks)
                plain.offset_norm = lambda x, ww, eps: plain_norm(x, ww, eps).to(torch.bfloat16).to(plain.DT)
                rounded = plain.forward(cfg, w, toks)
                plain.offset_norm = plain_norm
                out[rid] = (rounded - exact).abs().max(dim=1).values / exact.abs().max()
        finally:
            plain.offset_norm = plain_norm
        _noise[name] = out
    return _noise[name]


def within_limits(got, ref, dtype, noise=None):
    """Every wanted row against the reference, relative to the largest |logit| of its request."""
    worst, where = 0.0, None
    for (rid, pos), row in got.items():
        scale = float(ref[rid].abs().max())
        err = float((row.double() - ref[rid][pos].double()).abs().max()) / scale
        limit = TOL[dtype] if noise is None else max(TOL[dtype], 3.0 * float(noise[rid][pos]))
        if not err / limit <= worst:
            worst, where = err / limit, (rid, pos, err)
    return worst, where


def run_and_compare(folder, name, dtype, steps, expected, page_size=None, max_batch=4):
    reqs = requests_for(name)
    eng = engine_for(folder, dtype, traces.max_tokens(steps, page_size or 64), max_batch=max_batch, page_size=page_size)
    routing = {} if dtype == "bfloat16" else None
    got = traces.replay(eng, steps, routing)
    eng.runner.flush_status()
    eng.cache.check_invariants()
    assert not eng.cache.requests and all(g.pages.held_count == 0 for g in eng.cache.groups)
    wanted = sum(len(e["want"]) for st in steps for e in st["entries"])
    assert len({rid for rid, _ in got}) == len(reqs) and len(got) == wanted
    ref = reference_for(folder, reqs, routing, expected[name], dtype)
    noise = rounding_noise(folder, name) if (dtype == "bfloat16" and name == "T") else None
    ratio, where = within_limits(got, ref, dtype, noise)
    assert ratio < 1.0, f"{name} {dtype}: error over its limit ({ratio:.2f} of it) at {where}"
    return eng


# ------------------------------------------------------------------------------------------
# kernels alone
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("act", ["relu2", "gelu_tanh", "silu"])
def test_bias_act(act):
    from sharpinference_b200.kernels import ops
    g = torch.Generator().manual_seed(1)
    y = (3 * torch.randn(7, 45, generator=g)).to(DEV)
    b = torch.randn(45, generator=g).to(DEV)
    z = (y + b).double().cpu()
    want = {"relu2": plain.relu_squared(z), "gelu_tanh": plain.gelu_tanh(z), "silu": z * torch.sigmoid(z)}[act]
    got = ops.bias_act(y, b, ops.ACTIVATIONS[act], torch.float32)
    assert torch.allclose(got.double().cpu(), want, rtol=2e-6, atol=2e-6)
    got16 = ops.bias_act(y, None, ops.ACTIVATIONS[act], torch.bfloat16)
    z0 = y.double().cpu()
    want0 = {"relu2": plain.relu_squared(z0), "gelu_tanh": plain.gelu_tanh(z0), "silu": z0 * torch.sigmoid(z0)}[act]
    assert torch.allclose(got16.double().cpu(), want0, rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("rows,E,N,K", [(5, 3, 24, 64), (300, 4, 136, 72), (2100, 6, 96, 192)])
def test_grouped_product_with_activation_in_the_epilogue(rows, E, N, K):
    """The tensor-core grouped product that stores act(a . w^T) in bfloat16, against float32 arithmetic on the same
    bfloat16 operands; few rows (K split over CTAs), a few hundred, and a few thousand."""
    from sharpinference_b200.kernels import ops
    g = torch.Generator().manual_seed(rows)
    a = torch.randn(rows, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(E, N, K, generator=g) * 0.2).to(torch.bfloat16)
    counts = torch.multinomial(torch.ones(E), rows, replacement=True, generator=g).bincount(minlength=E)
    offsets = torch.cat([torch.zeros(1, dtype=torch.int64), counts.cumsum(0)]).to(torch.int32)
    for act, fn in (("relu2", plain.relu_squared), ("gelu_tanh", plain.gelu_tanh)):
        got = ops.tc_grouped_gemm_act(a.to(DEV), w.to(DEV), offsets.to(DEV), ops.ACTIVATIONS[act])
        ops.check_status(DEV)
        want = torch.empty(rows, N, dtype=torch.float64)
        for e in range(E):
            lo, hi = int(offsets[e]), int(offsets[e + 1])
            want[lo:hi] = fn(a[lo:hi].double() @ w[e].double().T)
        assert got.dtype == torch.bfloat16
        assert torch.allclose(got.double().cpu(), want, rtol=1e-2, atol=1e-2 * float(want.abs().max()))


def test_concat2():
    from sharpinference_b200.kernels import ops
    g = torch.Generator().manual_seed(2)
    a, d, b = (torch.randn(5, 20, generator=g).to(DEV) for _ in range(3))
    assert torch.equal(ops.concat2(a, d, b, torch.float32), torch.cat([a + d, b], dim=1))
    assert torch.equal(ops.concat2(a, None, b, torch.bfloat16), torch.cat([a, b], dim=1).to(torch.bfloat16))


@pytest.mark.parametrize("E,k,H,renorm", [(4, 1, 40, False), (9, 3, 70, False), (64, 8, 33, True), (3, 3, 16, False)])
def test_router_topk(E, k, H, renorm):
    from sharpinference_b200.kernels import ops
    g = torch.Generator().manual_seed(E * 10 + k)
    T = 37
    h = torch.randn(T, H, generator=g)
    wr = torch.randn(E, H, generator=g) * 0.3
    corr = torch.randn(E, generator=g)
    expert, weight, scores = ops.router_topk(h.to(DEV), wr.to(DEV), k, correction=corr.to(DEV), scale=2.5,
                                             renormalize=renorm, want_scores=True)
    s = torch.sigmoid(h.double() @ wr.double().T)
    assert torch.allclose(scores.double().cpu(), s, atol=1e-6)
    choice = s + corr.double()
    for t in range(T):
        want = torch.topk(choice[t], k).indices.tolist()
        got = expert[t].tolist()
        assert got == want, (t, got, want)                     # in order of falling choice score
        w = s[t, got] * 2.5
        if renorm:
            w = w / s[t, got].sum()
        assert torch.allclose(weight[t].double().cpu(), w, atol=1e-6)
    # without a correction the scores choose; among equal scores the lowest index wins
    wr2 = wr.clone()
    wr2[E - 1] = wr2[0]
    e2, _, _ = ops.router_topk(h.to(DEV), wr2.to(DEV), 1)
    s2 = torch.sigmoid(h.double() @ wr2.double().T)
    for t in range(T):
        best = int(torch.argmax(s2[t]))
        assert e2[t, 0].item() == (0 if best in (0, E - 1) else best)


def test_pair_tokens_and_combine():
    from sharpinference_b200.kernels import ops
    g = torch.Generator().manual_seed(5)
    T, k, H, E = 11, 3, 50, 4
    expert = torch.randint(0, E, (T, k), generator=g, dtype=torch.int32).to(DEV)
    offsets, pairs = ops.moe_sort(expert.view(-1), E)
    rows = ops.moe_pair_tokens(pairs, k)
    assert torch.equal(rows.cpu(), pairs.cpu() // k)
    flat = expert.view(-1).cpu()
    assert torch.equal(flat[pairs.cpu().long()], torch.sort(flat, stable=True).values)
    y = torch.randn(T * k, H, generator=g).to(DEV)
    add = torch.randn(T, H, generator=g).to(DEV)
    want = add.double().cpu() + y.double().cpu().view(T, k, H).sum(1)
    assert torch.allclose(ops.moe_combine(y, k).double().cpu(), want - add.double().cpu(), atol=1e-5)
    out = ops.moe_combine(y, k, add=add, out=add)
    assert out.data_ptr() == add.data_ptr() and torch.allclose(add.double().cpu(), want, atol=1e-5)


@pytest.mark.parametrize("heads,d,dv", [(3, 24, 40), (1, 8, 8), (2, 64, 100), (2, 200, 33), (2, 16, 32), (1, 512, 40),
                                        (2, 2, 1)])
def test_mlstm_recurrence_kernel(heads, d, dv):
    """Three requests of unequal length in one step, then a second step that goes on from the state (one of the
    requests sits it out, one brings a single row), against the plain recurrence; gates over their whole range."""
    from sharpinference_b200.kernels import ops
    from sharpinference_b200.parts.mlstm import fused_mlstm_columns
    g = torch.Generator().manual_seed(heads * 1000 + d)
    cq, ck, cv, cg, ci, cf, width = fused_mlstm_columns(heads, d, dv)
    cap = 9.0
    # rows per request in step one and two; the first step has more than 256 rows (the gates' own kernel)
    lens = {0: [19, 1], 1: [2, 0], 2: [250, 23]}
    total = {b: sum(n) for b, n in lens.items()}
    proj = {b: torch.randn(total[b], width, generator=g) for b in lens}
    for b in lens:                                              # raw gates from very negative to very positive
        proj[b][:, ci:ci + heads] *= 6.0
        proj[b][:, cf:cf + heads] = proj[b][:, cf:cf + heads] * 6.0 + 2.0
    bias_i, bias_f = torch.randn(heads, generator=g), torch.randn(heads, generator=g)
    per_head, per_request = ops.mlstm_state_floats(heads, d, dv)
    slots = {0: 3, 1: 0, 2: 1}
    state = torch.zeros(5, per_request, device=DEV)
    state[2].fill_(7.0)                                         # a slot nobody uses stays as it is
    got = {b: [] for b in lens}
    for step in (0, 1):
        live = [b for b in lens if lens[b][step] > 0]
        starts = {b: sum(lens[b][:step]) for b in live}
        rows = torch.cat([proj[b][starts[b]:starts[b] + lens[b][step]] for b in live]).contiguous().to(DEV)
        offs = [0]
        for b in live:
            offs.append(offs[-1] + lens[b][step])
        num, nq, coef = ops.mlstm_recurrence(
            rows, col_q=cq, col_k=ck, col_v=cv, col_i=ci, col_f=cf, bias_i=bias_i.to(DEV), bias_f=bias_f.to(DEV),
            row_offsets=torch.tensor(offs, dtype=torch.int32, device=DEV),
            state_slots=torch.tensor([slots[b] for b in live], dtype=torch.int32, device=DEV),
            state=state, heads=heads, d=d, dv=dv, cap=cap, q_scale=d ** -0.5)
        for j, b in enumerate(live):
            rows_b = slice(offs[j], offs[j + 1])
            got[b].append((num[rows_b].double().cpu().view(-1, heads, dv), nq[rows_b].double().cpu(),
                           coef[rows_b, :, 2].double().cpu()))
    assert torch.all(state[2] == 7.0) and torch.all(state[4] == 0.0)
    for b in lens:
        p = proj[b].double()
        ig = cap * torch.tanh((p[:, ci:ci + heads] + bias_i.double()) / cap)
        fg = torch.nn.functional.logsigmoid(cap * torch.tanh((p[:, cf:cf + heads] + bias_f.double()) / cap))
        # what the kernels leave per row: the numerator S^T q, n . q and the running maximum (the quotient is formed
        # by the kernel that follows and has a test of its own: where n . q is a difference of near-equal numbers
        # it would magnify float32 rounding here)
        num_want = torch.zeros(total[b], heads, dv, dtype=plain.DT)
        nq_want = torch.zeros(total[b], heads, dtype=plain.DT)
        m_want = torch.zeros(total[b], heads, dtype=plain.DT)
        for hd in range(heads):
            st = None
            for t in range(total[b]):
                q_t = p[t, cq + hd * d:cq + (hd + 1) * d] * d ** -0.5
                st, _ = plain.mlstm_step(st, q_t, p[t, ck + hd * d:ck + (hd + 1) * d],
                                         p[t, cv + hd * dv:cv + (hd + 1) * dv], ig[t, hd], fg[t, hd])
                num_want[t, hd], nq_want[t, hd], m_want[t, hd] = st[0].T @ q_t, st[1] @ q_t, st[2]
            # the state that the kernels left: slices of 32 value columns [d, 32], then n [d], then m
            S, n, m = st
            flat = state[slots[b]].double().cpu()[hd * per_head:(hd + 1) * per_head]
            slices = (dv + 31) // 32
            S_got = flat[:slices * d * 32].view(slices, d, 32).permute(1, 0, 2).reshape(d, slices * 32)
            scale = max(1.0, float(S.abs().max()))
            assert torch.allclose(S_got[:, :dv], S, atol=2e-5 * scale), (b, hd)
            assert torch.all(S_got[:, dv:] == 0)
            assert torch.allclose(flat[slices * d * 32:slices * d * 32 + d], n, atol=2e-5 * max(1.0, float(n.abs().max())))
            assert flat[slices * d * 32 + d].item() == pytest.approx(float(m), abs=1e-5)
        num_got = torch.cat([g_[0] for g_ in got[b]])
        nq_got = torch.cat([g_[1] for g_ in got[b]])
        m_got = torch.cat([g_[2] for g_ in got[b]])
        assert torch.allclose(m_got, m_want, atol=1e-5), (b, (m_got - m_want).abs().max())
        assert torch.allclose(num_got, num_want, atol=3e-5 * max(1.0, float(num_want.abs().max()))), b
        assert torch.allclose(nq_got, nq_want, atol=3e-5 * max(1.0, float(nq_want.abs().max()))), b


def test_mlstm_out_kernel():
    from sharpinference_b200.kernels import ops
    g = torch.Generator().manual_seed(9)
    T, heads, dv, col_g, ld = 13, 3, 40, 17, 17 + 120 + 5
    num = torch.randn(T, heads * dv, generator=g) * 4
    nq = torch.randn(T, heads, generator=g) * 2          # some below exp(-m) in size, some above
    coef = torch.randn(T, heads, 4, generator=g)
    proj = torch.randn(T, ld, generator=g)
    w = torch.randn(heads * dv, generator=g)
    got = ops.mlstm_out(num.to(DEV), nq.to(DEV), coef.to(DEV), proj.to(DEV), col_g, w.to(DEV), 1e-4, heads, dv,
                        torch.float32)
    den = torch.maximum(nq.double().abs(), torch.exp(-coef.double()[:, :, 2])) + 1e-6
    o = num.double().view(T, heads, dv) / den[:, :, None]
    want = plain.unit_rms(o, 1e-4).reshape(T, -1) * w.double() \
        * torch.sigmoid(proj.double()[:, col_g:col_g + heads * dv])
    assert torch.allclose(got.double().cpu(), want, atol=1e-5)


# ------------------------------------------------------------------------------------------
# whole models through the engine
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CASES))
def test_whole_prompts(folders, expected, name, dtype):
    run_and_compare(folders[name], name, dtype, traces.whole(requests_for(name)), expected)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CASES))
def test_prompt_then_token_by_token(folders, expected, name, dtype):
    """The last 80 tokens one by one: a window of 5, of 33 and of 70 passes wholly over decoded tokens, and the
    matrix memory is carried through 80 single-row steps."""
    run_and_compare(folders[name], name, dtype, traces.tail_decode(requests_for(name), tail=80), expected)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CASES))
def test_portions_down_to_two_tokens(folders, expected, name, dtype):
    run_and_compare(folders[name], name, dtype, traces.portions(requests_for(name)), expected)
    run_and_compare(folders[name], name, dtype, traces.portions(requests_for(name), sizes=(2, 2, 3, 64, 1, 63, 2, 33)),
                    expected, page_size=16)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CASES))
def test_mixed_batches_reuse_pages_and_slots(folders, expected, name, dtype):
    """Up to three live requests for three state slots and a pool sized for the schedule's peak: every later
    request runs in a slot and on pages that an earlier one left behind."""
    steps = traces.mixed(requests_for(name), max_live=3)
    eng = run_and_compare(folders[name], name, dtype, steps, expected, max_batch=3)
    assert eng.cache.state_slots.free_count == 3
    run_and_compare(folders[name], name, dtype, traces.drawn(requests_for(name), seed=5, max_live=4), expected)


@pytest.mark.parametrize("name", sorted(CASES))
def test_one_slot_used_again_starts_from_zero(folders, expected, name):
    reqs = requests_for(name)
    eng = engine_for(folders[name], "float32", 256, max_batch=1)
    for rid, toks in reqs.items():
        got = traces.replay(eng, traces.whole({rid: toks}))
        err, where = traces.worst_error(got, expected[name])
        assert err < TOL["float32"], (rid, err, where)


@pytest.mark.parametrize("name", ["P", "R", "T"])
def test_a_window_one_position_off_would_show(folders, expected, name):
    """The comparison is sharp enough: the plain model with every window one position longer or shorter differs
    from the engine by far more than the tolerance once a sequence is longer than the window, in prompts and in
    decoded tokens, and not at all before."""
    cfg, w = plain.load_folder(folders[name])
    windows = [c["mixer"]["mask"]["size"] for c in cfg["layers"] if c["type"] == "attention" and c["mixer"].get("mask")]
    reqs = {"r": traces.random_tokens(cfg["vocab"], 120, seed=77)}
    eng = engine_for(folders[name], "float32", 256)
    got = traces.replay(eng, traces.tail_decode(reqs, tail=60))
    right = {"r": plain.forward(cfg, w, reqs["r"])}
    assert traces.worst_error(got, right)[0] < TOL["float32"]
    for shift in (-1, 1):
        wrong = plain.forward(cfg, w, reqs["r"], window_shift=shift)
        scale = float(right["r"].abs().max())
        early = min(windows) - 1
        assert float((wrong[:early] - right["r"][:early]).abs().max()) / scale < 1e-9
        cut = max(60, early + 10)                         # the last 60 tokens are decoded one by one
        late_prompt = float((wrong[early + 2:cut] - right["r"][early + 2:cut]).abs().max()) / scale
        late_decode = float((wrong[cut:] - right["r"][cut:]).abs().max()) / scale
        assert late_prompt > 100 * TOL["float32"] and late_decode > 100 * TOL["float32"], (shift, late_prompt, late_decode)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_through_graphs(folders, dtype):
    """Three requests decode 260 tokens each side by side, past every window and over several pages; decode-only
    steps are replayed as CUDA graphs."""
    name = "Q"
    cfg, w = plain.load_folder(folders[name])
    reqs = {f"d{i}": traces.random_tokens(cfg["vocab"], 263 + i, seed=200 + i) for i in range(3)}
    steps = [{"step": 0, "entries": [{"id": rid, "tokens": toks[:3 + i], "want": [2 + i]}
                                     for i, (rid, toks) in enumerate(reqs.items())], "end": []}]
    for t in range(260):
        steps.append({"step": t + 1, "entries": [{"id": rid, "tokens": [toks[3 + i + t]], "want": [0]}
                                                 for i, (rid, toks) in enumerate(reqs.items())],
                      "end": list(reqs) if t == 259 else []})
    eng = engine_for(folders[name], dtype, traces.max_tokens(steps))
    routing = {} if dtype == "bfloat16" else None
    got = traces.replay(eng, steps, routing)
    if routing is None:
        assert eng.runner.graph_replays > 200
        ref = {rid: plain.forward(cfg, w, toks) for rid, toks in reqs.items()}
    else:
        # the rows before the first wanted one were routed too: the trace holds every row of every step
        ref = reference_for(folders[name], reqs, routing, None, dtype)
    err, where = traces.worst_error(got, ref)
    assert err < TOL[dtype], (err, where)


@pytest.mark.parametrize("name", sorted(CASES))
def test_greedy_generation_through_the_scheduler(folders, name):
    """``Engine.generate``: admission, portions under a small token budget, decoding in one batch, sampling
    (greedy) and the release of pages and slots, against the plain model generating token by token."""
    from sharpinference_b200 import Engine, EngineOptions, SamplingParams
    cfg, w = plain.load_folder(folders[name])
    prompts = [traces.random_tokens(cfg["vocab"], n, seed=300 + n) for n in (5, 41, 90, 17, 2)]
    opts = EngineOptions()
    opts.max_cache_tokens, opts.max_batch, opts.max_tokens_per_step = 1024, 3, 48
    eng = Engine(folders[name], dtype="float32", device=DEV, options=opts)
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_new_tokens=12))
    for prompt, out in zip(prompts, outs):
        assert out == plain.generate_greedy(cfg, w, prompt, 12)
    m = eng.metrics()
    assert m["state_slots_free"] == 3 and all(g["held"] == 0 for g in m["cache_groups"].values())


def test_command_line_generates_greedily(folders, capsys):
    """``sharpi-cli`` on a Notedra folder: greedy tokens as JSON, with the per-layer trace switched on."""
    import json

    from sharpinference_b200 import cli
    cfg, w = plain.load_folder(folders["R"])
    prompt = traces.random_tokens(cfg["vocab"], 21, seed=9)
    rc = cli.main(["-m", folders["R"], "--tokens", ",".join(map(str, prompt)), "-n", "6", "--temp", "0", "--dtype", "float32",
                   "--repeat-penalty", "1.0", "--json", "--max-cache-tokens", "256", "--trace-layers"])
    out = capsys.readouterr()
    assert rc == 0
    assert json.loads(out.out.strip().splitlines()[-1])["outputs"][0]["tokens"] == plain.generate_greedy(cfg, w, prompt, 6)
    assert "layer 2" in out.err and "expert" in out.err


def test_parts_are_registered_with_their_constants():
    from sharpinference_b200.parts import part_kinds
    assert "mlstm" in part_kinds("mixer") and "parallel" in part_kinds("block")
    assert {"dense_mlp", "moe_sigmoid_topk"} <= set(part_kinds("feed_forward"))
    assert "reinject_input" in part_kinds("stream")
