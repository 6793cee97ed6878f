"""Zaposun on the GPU: each new kernel against the plain statement of its mechanism, and whole models through the
engine (step function, cache and state manager, scheduler) under every way of cutting the work, in 32-bit and in
bfloat16."""

import pytest
import torch

import plain_zaposun as plain
import traces
from zaposun_models import CASES, write

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

# Relative to the largest |logit| of a request.
TOL = {"float32": 5e-5, "bfloat16": 4e-2}
LENGTHS = {"P": [1, 9, 40, 83, 150, 2], "Q": [150, 5, 67, 200, 31], "R": [3, 70, 12, 45, 100, 64, 65],
           "S": [1, 2, 30, 5], "T": [140, 66, 3, 129], "U": [33, 1, 80], "V": [70, 5, 41, 100]}


def requests_for(name):
    vocab = CASES[name][0]["vocab"]
    return {f"r{i}": traces.random_tokens(vocab, n, seed=37 * i + n) for i, n in enumerate(LENGTHS[name])}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {name: write(name, str(tmp_path_factory.mktemp(f"zaposun_{name}"))) for name in CASES}


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


def run_and_compare(folder, name, dtype, steps, expected, page_size=None, max_batch=4):
    reqs = requests_for(name)
    eng = engine_for(folder, dtype, traces.max_tokens(steps, page_size or 64), max_batch=max_batch, page_size=page_size)
    got = traces.replay(eng, steps)
    eng.runner.flush_status()
    eng.cache.check_invariants()
    assert not eng.cache.requests and all(g.pages.held_count == 0 for g in eng.cache.groups)
    wanted = sum(len(e["want"]) for st in steps for e in st["entries"])
    assert len({rid for rid, _ in got}) == len(reqs) and len(got) == wanted
    err, where = traces.worst_error(got, expected[name])
    assert err < TOL[dtype], f"{name} {dtype}: error {err} at {where}"
    return eng


# ------------------------------------------------------------------------------------------
# kernels alone
# ------------------------------------------------------------------------------------------
def _step_meta(lengths, slots):
    """row_request, row_offsets, state_slots of a step whose requests bring ``lengths`` rows."""
    rr, off = [], [0]
    for b, n in enumerate(lengths):
        rr += [b] * n
        off.append(off[-1] + n)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    return i32(rr), i32(off), i32(slots)


@pytest.mark.parametrize("S,G,H", [(1, 1, 40), (2, 2, 64), (4, 4, 96), (3, 1, 52), (8, 13, 13 * 24)])
def test_stream_update_and_group_norm(S, G, H):
    from sharpinference_b200.kernels import ops
    g = torch.Generator().manual_seed(S * 100 + G)
    T = 9
    x = torch.randn(T, S, H, generator=g, dtype=torch.float64)
    y = torch.randn(T, H, generator=g, dtype=torch.float64)
    mix = torch.eye(S, dtype=torch.float64) + 0.3 * torch.randn(S, S, generator=g, dtype=torch.float64)
    outc, inc = torch.randn(S, generator=g, dtype=torch.float64), torch.randn(S, generator=g, dtype=torch.float64)
    w = 1 + 0.1 * torch.randn(H, generator=g, dtype=torch.float64)
    new = torch.einsum("tsh,sr->trh", x, mix) + outc[None, :, None] * y[:, None, :]
    f = lambda t: t.float().to(DEV).contiguous()
    # with a pending update: the streams are replaced and the weighted sum is normed
    xd = f(x.reshape(T, S * H))
    h = ops.hc_mix_norm(xd, (f(y), f(mix), f(outc)), f(inc), f(w), streams=S, groups=G, eps=1e-5, out_dtype=torch.float32)
    want = plain.group_norm(torch.einsum("tsh,s->th", new, inc), w, G, 1e-5)
    assert torch.allclose(xd.double().cpu().view(T, S, H), new, atol=1e-5)
    assert torch.allclose(h.double().cpu(), want, atol=2e-5)
    # nothing pending, the plain sum, gathered rows: the streams stay as they are
    rows = torch.tensor([7, 0, 3], dtype=torch.int32, device=DEV)
    before = xd.clone()
    h = ops.hc_mix_norm(xd, None, None, f(w), streams=S, groups=G, eps=1e-5, out_dtype=torch.float32, rows=rows)
    assert torch.equal(xd, before)
    assert torch.allclose(h.double().cpu(), plain.group_norm(new.sum(1), w, G, 1e-5)[[7, 0, 3]], atol=2e-5)
    # a pending update with gathered rows is applied for the norm but not stored
    xd2 = f(x.reshape(T, S * H))
    h = ops.hc_mix_norm(xd2, (f(y), f(mix), f(outc)), None, f(w), streams=S, groups=G, eps=1e-5,
                        out_dtype=torch.float32, rows=rows)
    assert torch.equal(xd2, f(x.reshape(T, S * H)))
    assert torch.allclose(h.double().cpu(), plain.group_norm(new.sum(1), w, G, 1e-5)[[7, 0, 3]], atol=2e-5)


def test_token_shift_carries_the_previous_row_across_portions():
    from sharpinference_b200.kernels import ops
    g = torch.Generator().manual_seed(5)
    H, K = 24, 5
    mu = torch.rand(K, H, generator=g, dtype=torch.float64)
    seqs = [torch.randn(n, H, generator=g, dtype=torch.float64) for n in (11, 4, 7)]
    want = [torch.stack([plain.token_shift(s, mu[k]) for k in range(K)]) for s in seqs]
    state = torch.zeros(4, H, device=DEV)
    state[3] = 99.0                                          # a slot that no request of the step holds stays as it is
    slots = [2, 0, 1]
    got = [[] for _ in seqs]
    at = [0, 0, 0]
    for cut in ([3, 4, 1], [1, 0, 2], [5, 0, 4], [2, 0, 0]):          # 0: the request sits the step out
        live = [b for b in range(3) if cut[b]]
        rr, off, sl = _step_meta([cut[b] for b in live], [slots[b] for b in live])
        h = torch.cat([seqs[b][at[b]:at[b] + cut[b]] for b in live]).float().to(DEV)
        out = ops.token_shift(h, mu.float().to(DEV), state, row_request=rr, row_offsets=off, state_slots=sl,
                              out_dtype=torch.float32)
        r = 0
        for b in live:
            got[b].append(out[:, r:r + cut[b]].double().cpu())
            r += cut[b]
            at[b] += cut[b]
    for b in range(3):
        assert torch.allclose(torch.cat(got[b], dim=1), want[b], atol=1e-5)
    assert float(state[3].min()) == 99.0


def test_small_and_large_steps_give_the_same_bits():
    """The stream update with its norm and the token shift have a form for small steps and one for large steps; a
    row's result is the same bits in both."""
    from sharpinference_b200.kernels import ops
    g = torch.Generator().manual_seed(9)
    S, G, H, T = 3, 4, 4 * 300, 700
    x = torch.randn(T, S * H, generator=g).to(DEV)
    y = torch.randn(T, H, generator=g).to(DEV)
    mix, outc, inc = torch.randn(S, S, generator=g).to(DEV), torch.randn(S, generator=g).to(DEV), torch.randn(S, generator=g).to(DEV)
    w = torch.randn(H, generator=g).to(DEV)
    xa, xb = x.clone(), x[:20].clone()
    big = ops.hc_mix_norm(xa, (y, mix, outc), inc, w, streams=S, groups=G, eps=1e-5, out_dtype=torch.float32)
    small = ops.hc_mix_norm(xb, (y[:20].contiguous(), mix, outc), inc, w, streams=S, groups=G, eps=1e-5, out_dtype=torch.float32)
    assert torch.equal(big[:20], small) and torch.equal(xa[:20], xb)
    h = torch.randn(T, H, generator=g).to(DEV)
    mu = torch.rand(2, H, generator=g).to(DEV)
    rr, off, sl = _step_meta([T], [0])
    st_a, st_b = torch.ones(1, H, device=DEV), torch.ones(1, H, device=DEV)
    big = ops.token_shift(h, mu, st_a, row_request=rr, row_offsets=off, state_slots=sl, out_dtype=torch.float32)
    rr, off, sl = _step_meta([20], [0])
    small = ops.token_shift(h[:20].contiguous(), mu, st_b, row_request=rr, row_offsets=off, state_slots=sl, out_dtype=torch.float32)
    assert torch.equal(big[:, :20], small)
    assert torch.equal(st_a[0], h[-1]) and torch.equal(st_b[0], h[19])


def test_pair_embedding_uses_the_previous_token_of_the_request():
    from sharpinference_b200.kernels import ops
    g = torch.Generator().manual_seed(6)
    V, H, buckets, mp, mc, S = 50, 16, 13, 1000003, 7919, 3
    embed = torch.randn(V, H, generator=g).to(torch.bfloat16)
    pairs = torch.randn(buckets + 1, H, generator=g).to(torch.bfloat16)
    seqs = [traces.random_tokens(V, n, seed=n) for n in (9, 5)]
    want = [plain.embedding(s, embed.double(), pairs.double(), buckets, mp, mc) for s in seqs]
    prev = torch.zeros(4, dtype=torch.int32, device=DEV)
    got, at = [[], []], [0, 0]
    for cut in ([4, 1], [1, 3], [4, 1]):
        rr, off, sl = _step_meta(cut, [3, 1])
        ids = torch.tensor(sum((seqs[b][at[b]:at[b] + cut[b]] for b in range(2)), []), dtype=torch.int32, device=DEV)
        x = ops.embed_pair(ids, embed.to(DEV), pairs.to(DEV), row_request=rr, row_offsets=off, state_slots=sl,
                           prev_state=prev, streams=S, buckets=buckets, mul_prev=mp, mul_cur=mc)
        x = x.view(-1, S, H)
        assert torch.equal(x[:, 0], x[:, S - 1])
        r = 0
        for b in range(2):
            got[b].append(x[r:r + cut[b], 0].double().cpu())
            r += cut[b]
            at[b] += cut[b]
    for b in range(2):
        assert torch.allclose(torch.cat(got[b]), want[b], atol=1e-6)


@pytest.mark.parametrize("heads,d", [(2, 24), (1, 2), (3, 64), (1, 128), (2, 48), (1, 160), (1, 17)])
def test_wkv_recurrence_kernel(heads, d):
    """Two requests in portions (the state is carried in its slot) against the plain token-by-token walk."""
    from sharpinference_b200.kernels import ops
    g = torch.Generator().manual_seed(heads * 1000 + d)
    hd = heads * d
    lens = (23, 9)
    mk = lambda n: torch.randn(n, hd, generator=g, dtype=torch.float64)
    data = [{k: mk(n) * (0.5 if k != "wraw" else 0.3) for k in ("r", "k", "v", "wraw", "g")} for n in lens]
    w0 = -3.0 + 2.0 * torch.rand(hd, generator=g, dtype=torch.float64)
    u = torch.randn(hd, generator=g, dtype=torch.float64)
    nw = 1 + 0.1 * torch.randn(hd, generator=g, dtype=torch.float64)
    want = []
    for q in data:
        n = q["r"].shape[0]
        S = torch.zeros(heads, d, d, dtype=torch.float64)
        o = torch.zeros(n, heads, d, dtype=torch.float64)
        w = torch.exp(-torch.exp(q["wraw"] + w0)).view(n, heads, d)
        r, k, v = (q[s].view(n, heads, d) for s in "rkv")
        for t in range(n):
            kv = k[t][:, :, None] * v[t][:, None, :]
            o[t] = torch.einsum("hkv,hk->hv", S + u.view(heads, d)[:, :, None] * kv, r[t])
            S = w[t][:, :, None] * S + kv
        want.append((o.reshape(n, hd), plain.rms(o, 1e-5).reshape(n, hd) * nw * plain.silu(q["g"]), S))
    state = torch.zeros(3, heads * d * d, device=DEV)
    f = lambda t: t.float().to(DEV).contiguous()
    got = [[], []]
    at = [0, 0]
    for cut in ([10, 2], [1, 1], [12, 6]):
        rr, off, sl = _step_meta(cut, [2, 0])
        cat = {k: f(torch.cat([data[b][k][at[b]:at[b] + cut[b]] for b in range(2)])) for k in data[0]}
        o = ops.wkv_recurrence(cat["r"], cat["k"], cat["v"], cat["wraw"], f(w0), f(u), row_offsets=off, state_slots=sl,
                               state=state, heads=heads, d=d)
        out = ops.wkv_out(o, cat["g"], f(nw), 1e-5, heads, d, torch.float32)
        r = 0
        for b in range(2):
            got[b].append((o[r:r + cut[b]].double().cpu(), out[r:r + cut[b]].double().cpu()))
            r += cut[b]
            at[b] += cut[b]
    for b, slot in ((0, 2), (1, 0)):
        o = torch.cat([p[0] for p in got[b]])
        out = torch.cat([p[1] for p in got[b]])
        scale = float(want[b][0].abs().max())
        assert float((o - want[b][0]).abs().max()) < 2e-5 * scale
        assert torch.allclose(out, want[b][1], atol=2e-4)
        assert float((state[slot].double().cpu().view(heads, d, d) - want[b][2]).abs().max()) < 2e-5 * float(want[b][2].abs().max())


@pytest.mark.parametrize("C,N,R,taps", [(40, 5, 3, 3), (8, 200, 2, 4), (33, 16, 4, 1), (2, 1, 1, 2), (70, 64, 5, 5)])
def test_convolution_and_selective_scan_kernels(C, N, R, taps):
    from sharpinference_b200.kernels import ops
    g = torch.Generator().manual_seed(C * 10 + N)
    lens = (19, 6)
    rnd = lambda *s: torch.randn(*s, generator=g, dtype=torch.float64)
    conv_w, conv_b = rnd(C, taps) * 0.5, rnd(C) * 0.2
    dt_b, a_log, dsk = rnd(C) * 0.5, -4.0 + 3.0 * torch.rand(C, N, generator=g, dtype=torch.float64), 1 + 0.1 * rnd(C)
    data = [{"xz": rnd(n, 2 * C), "dbc": rnd(n, R + 2 * N) * 0.5, "dtraw": rnd(n, C)} for n in lens]
    want = []
    for q in data:
        n = q["xz"].shape[0]
        x, z = q["xz"][:, :C], q["xz"][:, C:]
        xp = torch.cat([torch.zeros(taps - 1, C, dtype=torch.float64), x])
        xc = sum(xp[j:j + n] * conv_w[:, j] for j in range(taps))
        xa = plain.silu(xc + conv_b)
        dt = plain.softplus(q["dtraw"] + dt_b)
        B, Cm = q["dbc"][:, R:R + N], q["dbc"][:, R + N:]
        A = -torch.exp(a_log)
        S = torch.zeros(C, N, dtype=torch.float64)
        y = torch.zeros(n, C, dtype=torch.float64)
        for t in range(n):
            S = torch.exp(dt[t][:, None] * A) * S + (dt[t] * xa[t])[:, None] * B[t][None, :]
            y[t] = S @ Cm[t] + dsk * xa[t]
        want.append((xa, y * plain.silu(z), S))
    f = lambda t: t.float().to(DEV).contiguous()
    conv_state = torch.zeros(3, max(taps - 1, 1) * C, device=DEV)
    scan_state = torch.zeros(3, C * N, device=DEV)
    got, at = [[], []], [0, 0]
    for cut in ([1, 2], [1, 1], [2, 0], [15, 3]):                     # portions shorter than the convolution too
        live = [b for b in range(2) if cut[b]]
        rr, off, sl = _step_meta([cut[b] for b in live], [[1, 2][b] for b in live])
        cat = {k: f(torch.cat([data[b][k][at[b]:at[b] + cut[b]] for b in live])) for k in data[0]}
        x32, xact = ops.causal_conv(cat["xz"], C, f(conv_w), f(conv_b), conv_state, row_request=rr, row_offsets=off,
                                    state_slots=sl, act_dtype=torch.float32, gate_col=C)      # the gate's silu in place
        dt = ops.bias_act(cat["dtraw"], f(dt_b), ops.ACT_SOFTPLUS, torch.float32, out=cat["dtraw"])
        y = ops.selective_scan(x32, dt, cat["dbc"], R, R + N, f(a_log), f(dsk), cat["xz"], C,
                               row_offsets=off, state_slots=sl, state=scan_state, out_dtype=torch.float32)
        sliced = ops.slice_cols(cat["dbc"], 0, R, torch.float32)
        assert torch.equal(sliced, cat["dbc"][:, :R].contiguous())
        r = 0
        for b in live:
            got[b].append((x32[r:r + cut[b]].double().cpu(), y[r:r + cut[b]].double().cpu()))
            r += cut[b]
            at[b] += cut[b]
    for b, slot in ((0, 1), (1, 2)):
        assert torch.allclose(torch.cat([p[0] for p in got[b]]), want[b][0], atol=1e-5)
        yw = want[b][1]
        assert float((torch.cat([p[1] for p in got[b]]) - yw).abs().max()) < 3e-5 * max(1.0, float(yw.abs().max()))
        assert float((scan_state[slot].double().cpu().view(C, N) - want[b][2]).abs().max()) < 3e-5 * max(1.0, float(want[b][2].abs().max()))


@pytest.mark.parametrize("layout", ["halves", "interleaved"])
@pytest.mark.parametrize("nq,nkv,dk,dv,rot", [(4, 2, 16, 32, 8), (2, 1, 64, 64, 64), (3, 3, 24, 10, 0), (1, 1, 2, 2, 2)])
def test_rotation_with_norm_first_and_rotated_values(layout, nq, nkv, dk, dv, rot):
    """q and k: weighted RMS norm over the key size, then the rotation of the leading elements; v: rotated over its
    whole size and written to its page; then the inverse rotation of a head's output."""
    from sharpinference_b200.kernels import ops
    from sharpinference_b200.parts.position import leading_rotary_inv_freq
    g = torch.Generator().manual_seed(nq * 100 + dk)
    D = max(dk, dv)
    T, page = 11, 4
    pos = torch.tensor([5, 6, 7, 8, 9, 10, 11, 0, 1, 2, 3])
    req = [0] * 7 + [1] * 4
    table = torch.tensor([[9, 2, 5], [7, 4, -1]], dtype=torch.int32, device=DEV)
    base = 50.0
    wq, wk = (1 + 0.2 * torch.randn(dk, generator=g, dtype=torch.float64) for _ in range(2))
    q, k = torch.randn(T, nq, dk, generator=g, dtype=torch.float64), torch.randn(T, nkv, dk, generator=g, dtype=torch.float64)
    v = torch.randn(T, nkv, dv, generator=g, dtype=torch.float64)
    pad = lambda t: torch.nn.functional.pad(t, (0, D - t.shape[-1]))
    qkv = torch.cat([pad(q).reshape(T, -1), pad(k).reshape(T, -1), pad(v).reshape(T, -1)], dim=1).float().to(DEV)
    want_q = plain.rotate(plain.rms(q, 1e-5) * wq, pos, base, rot, layout)
    want_k = plain.rotate(plain.rms(k, 1e-5) * wk, pos, base, rot, layout)
    want_v = plain.rotate(v, pos, base, dv, layout)
    q_out = torch.zeros(T, nq, D, device=DEV)
    kv = torch.zeros(10, 2, nkv, page, D, device=DEV)
    code = {"halves": ops.ROPE_HALVES, "interleaved": ops.ROPE_INTERLEAVED}[layout]
    f = lambda t: t.float().to(DEV)
    ops.qkv_post_rot(qkv, pos.int().to(DEV), torch.tensor(req, dtype=torch.int32, device=DEV), table, q_out, kv,
                     nq=nq, nkv=nkv, D=D, key_dim=dk, value_dim=dv, page_size=page, pairing=code, q_norm_weight=f(wq),
                     k_norm_weight=f(wk), eps=1e-5, inv_freq=leading_rotary_inv_freq(rot, base).to(DEV) if rot else None,
                     rot_dims=rot, inv_freq_v=leading_rotary_inv_freq(dv, base).to(DEV), v_rot_dims=dv)
    assert torch.allclose(q_out[:, :, :dk].double().cpu(), want_q, atol=2e-5)
    assert float(q_out[:, :, dk:].abs().max()) == 0.0 if D > dk else True
    for t in range(T):
        pg = int(table[req[t], int(pos[t]) // page])
        assert torch.allclose(kv[pg, 0, :, int(pos[t]) % page, :dk].double().cpu(), want_k[t], atol=2e-5)
        assert torch.allclose(kv[pg, 1, :, int(pos[t]) % page, :dv].double().cpu(), want_v[t], atol=2e-5)
    o = torch.randn(T, nq, D, generator=g, dtype=torch.float64)
    back = ops.rotate_heads(o.reshape(T, -1).float().to(DEV), pos.int().to(DEV), leading_rotary_inv_freq(dv, base).to(DEV),
                            heads=nq, D=D, rot_dims=dv, pairing=code, sign=-1.0, out_dtype=torch.float32)
    want = o.clone()
    want[:, :, :dv] = plain.rotate(o[:, :, :dv], pos, base, dv, layout, sign=-1.0)
    assert torch.allclose(back.double().cpu().view(T, nq, D), want, atol=2e-5)


def test_branch_join_gated_activation_and_scale():
    from sharpinference_b200.kernels import ops
    g = torch.Generator().manual_seed(8)
    a, b = torch.randn(6, 52, generator=g, dtype=torch.float64), 3 * torch.randn(6, 52, generator=g, dtype=torch.float64)
    wa, wb = torch.randn(52, generator=g, dtype=torch.float64), torch.randn(52, generator=g, dtype=torch.float64)
    f = lambda t: t.float().to(DEV)
    got = ops.norm_mean2(f(a), f(wa), f(b), f(wb), 1e-4, 0.5)
    assert torch.allclose(got.double().cpu(), 0.5 * (plain.rms(a, 1e-4) * wa + plain.rms(b, 1e-4) * wb), atol=1e-5)
    gu = 2 * torch.randn(5, 2 * 37, generator=g, dtype=torch.float64)
    got = ops.gated_act(f(gu), ops.ACTIVATIONS["gelu_tanh"], torch.float32)
    assert torch.allclose(got.double().cpu(), plain.gelu_tanh(gu[:, :37]) * gu[:, 37:], atol=1e-5)
    assert torch.allclose(ops.tanh(f(gu), torch.float32).double().cpu(), torch.tanh(gu), atol=1e-6)
    y = f(gu)
    assert torch.allclose(ops.scale_(y, 1.75).double().cpu(), gu.float().double() * 1.75, atol=1e-6)


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
    """The last 80 tokens one by one: chunks of 5, 7, 33, 64 and 70 begin and end among decoded tokens, and every
    recurrent state is carried through 80 single-row steps."""
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
    """One state slot for all requests in turn: the previous token, the shifted rows, the convolution's inputs and
    both recurrent states of the request before must be gone."""
    reqs = requests_for(name)
    eng = engine_for(folders[name], "float32", 256, max_batch=1)
    for rid, toks in reqs.items():
        got = traces.replay(eng, traces.whole({rid: toks}))
        err, where = traces.worst_error(got, expected[name])
        assert err < TOL["float32"], (rid, err, where)


@pytest.mark.parametrize("name", ["P", "R", "T"])
def test_a_chunk_one_position_off_would_show(folders, expected, name):
    """The comparison is sharp enough: the plain model with every chunk one position longer or shorter differs from
    the engine by far more than the tolerance once a sequence is longer than the shortest chunk, in prompts and in
    decoded tokens, and not at all before."""
    cfg, w = plain.load_folder(folders[name])
    chunks = [c["mixer"]["left"]["mask"]["size"] for c in cfg["layers"] if c["type"] == "parallel"]
    reqs = {"r": traces.random_tokens(cfg["vocab"], 150, seed=77)}
    eng = engine_for(folders[name], "float32", 256)
    got = traces.replay(eng, traces.tail_decode(reqs, tail=60))
    right = {"r": plain.forward(cfg, w, reqs["r"])}
    assert traces.worst_error(got, right)[0] < TOL["float32"]
    for delta in (-1, 1):
        wrong = plain.forward(cfg, w, reqs["r"], chunk_delta=delta)
        scale = float(right["r"].abs().max())
        early = min(chunks) + min(delta, 0)
        assert float((wrong[:early] - right["r"][:early]).abs().max()) / scale < 1e-9
        late_prompt = float((wrong[early:90] - right["r"][early:90]).abs().max()) / scale
        late_decode = float((wrong[90:] - right["r"][90:]).abs().max()) / scale
        assert late_prompt > 100 * TOL["float32"] and late_decode > 100 * TOL["float32"], (delta, late_prompt, late_decode)


def test_a_lost_state_would_show(folders, expected):
    """A far token matters: the plain model fed a request without its first 30 tokens differs at the request's end,
    200 tokens later, by far more than the tolerance (the recurrent memories reach that far back)."""
    cfg, w = plain.load_folder(folders["Q"])
    toks = requests_for("Q")["r3"]
    full, cut = expected["Q"]["r3"], plain.forward(cfg, w, toks[30:])
    assert float((full[-1] - cut[-1]).abs().max()) / float(full.abs().max()) > 100 * TOL["float32"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_through_graphs(folders, dtype):
    """Three requests decode 260 tokens each side by side, past every chunk edge and over several pages; decode-only
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
    got = traces.replay(eng, steps)
    assert eng.runner.graph_replays > 200
    ref = {rid: plain.forward(cfg, w, toks) for rid, toks in reqs.items()}
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


def test_command_line_and_trace_program(folders, capsys, tmp_path):
    """``sharpi-cli`` generates greedily on a Zaposun folder, and ``bin/trace_run`` as a child process replays a mixed
    schedule from standard input and writes the logits the plain model gives."""
    import json
    import os
    import subprocess
    import sys

    import numpy as np

    from sharpinference_b200 import cli
    cfg, w = plain.load_folder(folders["R"])
    prompt = traces.random_tokens(cfg["vocab"], 21, seed=9)
    rc = cli.main(["-m", folders["R"], "--tokens", ",".join(map(str, prompt)), "-n", "6", "--temp", "0", "--dtype", "float32",
                   "--repeat-penalty", "1.0", "--json", "--max-cache-tokens", "256"])
    out = capsys.readouterr()
    assert rc == 0
    assert json.loads(out.out.strip().splitlines()[-1])["outputs"][0]["tokens"] == plain.generate_greedy(cfg, w, prompt, 6)

    reqs = {f"t{i}": traces.random_tokens(cfg["vocab"], n, seed=50 + i) for i, n in enumerate((40, 3, 77, 18, 66))}
    steps = traces.mixed(reqs, max_live=4)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    res = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folders["R"], "--dtype", "float32",
                          "--out", str(tmp_path), "--max-tokens", str(traces.max_tokens(steps))],
                         input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=900)
    assert res.returncode == 0, res.stderr[-2000:]
    assert [ln for ln in res.stdout.splitlines() if ln.startswith("done ")] == [f"done {s['step']}" for s in steps]
    ref = {rid: plain.forward(cfg, w, toks) for rid, toks in reqs.items()}
    at = {rid: 0 for rid in reqs}
    for st in steps:
        rows = np.fromfile(os.path.join(str(tmp_path), f"{st['step']}.f32"), dtype="<f4").reshape(-1, cfg["vocab"])
        r = 0
        for e in st["entries"]:
            for wpos in e["want"]:
                want = ref[e["id"]][at[e["id"]] + wpos]
                assert float((torch.from_numpy(rows[r]).double() - want).abs().max()) < TOL["float32"] * float(ref[e["id"]].abs().max())
                r += 1
            at[e["id"]] += len(e["tokens"])


def test_parts_are_registered_with_their_constants():
    from sharpinference_b200.parts import part_kinds
    assert {"wkv", "selective_scan", "branch_pair"} <= set(part_kinds("mixer"))
    assert "hyper" in part_kinds("block") and "group_rmsnorm" in part_kinds("norm")
