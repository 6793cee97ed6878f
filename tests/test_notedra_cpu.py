"""Notedra without a GPU: the configuration reader, the tensor declaration, the schedule of a looped model, and
the plain implementation checked against itself (a sequence at once against token by token with carried state;
each mechanism's defining property)."""
import copy
import json
import math

import pytest
import torch

import plain_notedra as plain
from notedra_models import CASE_P, CASE_Q, CASE_R, CASE_S, CASE_T, CASES, write

from sharpinference_b200.config import ConfigError, NotedraConfig
from sharpinference_b200.registry import get_architecture, resolve
from sharpinference_b200.weights.loading import declared_tensors


# -- configuration -------------------------------------------------------------------------
@pytest.mark.parametrize("case", [CASE_P, CASE_Q, CASE_R, CASE_S, CASE_T])
def test_config_round_trip(case):
    arch, cfg = resolve(copy.deepcopy(case), "test")
    assert arch.name == "Notedra" and isinstance(cfg, NotedraConfig)
    assert cfg.to_dict() == case
    assert len(cfg.layers) == len(case["layers"])


def test_architecture_key_forms():
    from sharpinference_b200.config import architecture_name
    assert architecture_name({"architecture": "Notedra"}) == "Notedra"
    assert architecture_name({"architectures": ["X"], "architecture": "Y"}) == "X"
    with pytest.raises(ConfigError):
        architecture_name({"architecture": ""})


def test_layer_runs_and_schedule():
    _, cfg = resolve(copy.deepcopy(CASE_P), "test")
    runs = cfg.layer_runs()
    assert [r[0] for r in runs] == [0, 1, 0, 1, 0, 1, 2, 3]
    assert [r[1] for r in runs] == [0, 0, 1, 1, 2, 2, None, None]
    assert [r[2] for r in runs] == [True, False, True, False, True, False, False, False]
    assert [(layer, t) for layer, t, _ in runs] == plain.layer_runs(CASE_P)
    _, cfg_q = resolve(copy.deepcopy(CASE_Q), "test")
    assert [r[0] for r in cfg_q.layer_runs()] == [0, 1, 2, 3]
    _, cfg_r = resolve(copy.deepcopy(CASE_R), "test")
    assert [(layer, t) for layer, t, _ in cfg_r.layer_runs()] == plain.layer_runs(CASE_R) == [(0, None), (1, 0), (2, 0)]


def test_defaults_of_absent_keys():
    _, cfg = resolve(copy.deepcopy(CASE_Q), "test")
    free = cfg.layers[2]
    assert free.window == 0 and free.rot_dims == 0
    case = copy.deepcopy(CASE_Q)
    del case["layers"][2]["mixer"]["scale"]
    del case["layers"][2]["mixer"]["kv_heads"]
    del case["layers"][2]["mixer"]["vdim"]
    _, cfg = resolve(case, "test")
    assert cfg.layers[2].scale == pytest.approx(32 ** -0.5)
    assert cfg.layers[2].kv_heads == 4 and cfg.layers[2].vdim == 32


def test_config_problems_are_listed_together():
    bad = copy.deepcopy(CASE_P)
    del bad["vocab"]
    bad["layers"][0]["mixer"]["kv_heads"] = 3               # 4 heads are no multiple of 3
    bad["layers"][1]["mlp"]["router"]["top"] = 9            # more than its 4 experts
    bad["layers"][2]["type"] = "conv"
    bad["loop"]["stop"] = 7
    with pytest.raises(ConfigError) as err:
        resolve(bad, "test")
    text = str(err.value)
    for piece in ("vocab", "kv_heads", "top", "conv", "loop"):
        assert piece in text, (piece, text)


def test_declared_tensors_follow_the_configuration():
    arch = get_architecture("Notedra")
    _, cfg = resolve(copy.deepcopy(CASE_P), "test")
    decls = {d.name: d.shape for d in declared_tensors(arch, cfg)}
    assert decls["embed"] == (97, 64) and decls["loop.in"] == (64, 128) and decls["loop.step"] == (3, 64)
    assert decls["l0.mix.q"] == (64, 64) and decls["l0.mix.k"] == (32, 64) and decls["l0.mix.v"] == (32, 64)
    assert decls["l3.mix.v"] == (3 * 48, 64) and decls["l3.mix.o"] == (64, 3 * 48)
    assert decls["l1.mix.i"] == (2, 64) and decls["l1.mix.f.b"] == (2,) and decls["l1.mix.norm"] == (64,)
    assert decls["l1.mlp.e3.up"] == (24, 64) and decls["l1.mlp.correction"] == (4,)
    assert "l2.mlp.up" not in decls and not any(n.startswith("l2.mlp") for n in decls)
    assert decls["l0.mlp.up.b"] == (40,) and decls["l0.mlp.down.b"] == (64,)
    _, cfg_q = resolve(copy.deepcopy(CASE_Q), "test")
    assert not any(n.startswith("loop.") for n in (d.name for d in declared_tensors(arch, cfg_q)))


# -- the plain implementation against itself ---------------------------------------------------
def _rand(*shape, seed=0, scale=1.0):
    return scale * torch.randn(*shape, generator=torch.Generator().manual_seed(seed), dtype=plain.DT)


def test_plain_norms_and_activations():
    x = _rand(5, 12, seed=1, scale=3.0)
    y = plain.unit_rms(x, 0.0)
    assert torch.allclose((y * y).mean(-1), torch.ones(5, dtype=plain.DT))
    assert torch.allclose(plain.offset_norm(x, torch.zeros(12, dtype=plain.DT), 1e-5), plain.unit_rms(x, 1e-5))
    z = torch.tensor([-2.0, 0.0, 0.5, 3.0], dtype=plain.DT)
    assert plain.relu_squared(z).tolist() == [0.0, 0.0, 0.25, 9.0]
    assert plain.gelu_tanh(z)[1] == 0 and plain.gelu_tanh(z)[3] == pytest.approx(2.9964, abs=1e-3)


def test_plain_rotation_is_relative_and_partial():
    q, k = _rand(9, 1, 8, seed=2), _rand(9, 1, 8, seed=3)
    pos = torch.arange(9)
    rq, rk = plain.rotate_pairs(q, pos, 4, 50.0), plain.rotate_pairs(k, pos, 4, 50.0)
    assert torch.equal(rq[..., 4:], q[..., 4:])                      # beyond dims: unchanged
    assert torch.allclose(rq.norm(dim=-1), q.norm(dim=-1))
    same_q, same_k = q[3:4].expand(9, 1, 8), k[5:6].expand(9, 1, 8)   # one vector at every position
    a = plain.rotate_pairs(same_q, pos, 4, 50.0)
    b = plain.rotate_pairs(same_k, pos, 4, 50.0)
    assert (a[6, 0] @ b[4, 0]).item() == pytest.approx((a[3, 0] @ b[1, 0]).item(), abs=1e-12)   # depends on i - j


def test_plain_mlstm_whole_equals_token_by_token():
    m = {"heads": 2, "dim": 6, "vdim": 10, "gate_cap": 7.0}
    W = 14
    w = {"q": _rand(12, W, seed=4), "k": _rand(12, W, seed=5), "v": _rand(20, W, seed=6), "g": _rand(20, W, seed=7),
         "o": _rand(W, 20, seed=8), "norm": _rand(20, seed=9), "i": _rand(2, W, seed=10), "f": _rand(2, W, seed=11),
         "i.b": _rand(2, seed=12), "f.b": _rand(2, seed=13) + 3.0}
    h = _rand(11, W, seed=14)
    whole, _ = plain.mlstm_mixer(h, w, "", m, 1e-5)
    states, rows = None, []
    for cut in ((0, 4), (4, 5), (5, 11)):
        part, states = plain.mlstm_mixer(h[cut[0]:cut[1]], w, "", m, 1e-5, states)
        rows.append(part)
    assert torch.allclose(torch.cat(rows), whole, atol=1e-12)
    # the first token: m_0 = max(f_0, i_0) because the running maximum starts at 0, not at minus infinity
    i0, f0 = plain.mlstm_gates(h[:1], w, "", 7.0)
    (S, n, m0), _ = plain.mlstm_step(None, h[0, :6], h[0, :6], h[0, :10], i0[0, 0], f0[0, 0])
    assert m0 == torch.maximum(f0[0, 0], i0[0, 0])


def test_plain_router_correction_chooses_but_does_not_weigh():
    W, E = 10, 5
    w = {"router": _rand(E, W, seed=20), "correction": torch.tensor([0.0, 0.0, 5.0, 0.0, 0.0], dtype=plain.DT)}
    for e in range(E):
        w[f"e{e}.up"], w[f"e{e}.down"] = _rand(6, W, seed=30 + e), _rand(W, 6, seed=40 + e)
    h = _rand(4, W, seed=21)
    mlp = {"router": {"experts": E, "top": 1, "scale": 2.0}}
    out = plain.mixture_ff(h, w, "", mlp)
    s, _ = plain.router_scores(h, w, "")
    for t in range(4):          # expert 2 always wins the choice, and is weighted by its own score only
        y = plain.relu_squared(h[t] @ w["e2.up"].T) @ w["e2.down"].T
        assert torch.allclose(out[t], 2.0 * s[t, 2] * y)


def test_plain_window_counts_the_query_itself(tmp_path):
    folder = write("P", str(tmp_path))
    cfg, w = plain.load_folder(folder)
    h = _rand(12, cfg["width"], seed=50)
    m = dict(cfg["layers"][0]["mixer"])
    a = plain.window_attention(h, w, "l0.mix.", m, 1e-5)
    m1 = dict(m, mask={"size": 1})
    one = plain.window_attention(h, w, "l0.mix.", m1, 1e-5)
    v = (h @ w["l0.mix.v"].T).view(12, m["kv_heads"], m["vdim"])
    alone = v.repeat_interleave(m["heads"] // m["kv_heads"], dim=1).reshape(12, -1) @ w["l0.mix.o"].T
    assert torch.allclose(one, alone, atol=1e-12)                   # a window of one is the token's own value
    assert not torch.allclose(a[6:], plain.window_attention(h, w, "l0.mix.", m, 1e-5, window_shift=1)[6:], atol=1e-3)
    assert torch.allclose(a[:5], plain.window_attention(h, w, "l0.mix.", m, 1e-5, window_shift=1)[:5], atol=1e-12)


@pytest.mark.parametrize("name", sorted(CASES))
def test_random_folder_loads_and_runs_plain(tmp_path, name):
    folder = write(name, str(tmp_path))
    cfg, w = plain.load_folder(folder)
    assert json.load(open(folder + "/config.json")) == CASES[name][0]
    logits = plain.forward(cfg, w, [1, 2, 3, 4, 5, 6, 7])
    assert logits.shape == (7, cfg["vocab"]) and torch.isfinite(logits).all()
    assert logits.std() > 0.05            # the weights are large enough for the logits to mean something
    again = plain.forward(cfg, w, [1, 2, 3, 4])
    assert torch.allclose(again, logits[:4], atol=1e-10)      # causal
