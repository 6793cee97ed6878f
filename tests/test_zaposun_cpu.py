"""Zaposun without a GPU: the configuration reader, the tensor declaration, the state that the cache manager hands
to blocks, mixers and the model, and the plain implementation checked against each mechanism's defining property."""
import copy
import math

import pytest
import torch

import plain_zaposun as plain
import traces
from zaposun_models import CASE_P, CASE_Q, CASE_R, CASE_S, CASE_T, CASE_U, CASE_V, CASES, write

from sharpinference_b200.config import ConfigError, ZaposunConfig
from sharpinference_b200.registry import get_architecture, resolve
from sharpinference_b200.weights.loading import declared_tensors

F64 = torch.float64


# -- configuration -------------------------------------------------------------------------
@pytest.mark.parametrize("case", [CASE_P, CASE_Q, CASE_R, CASE_S, CASE_T, CASE_U, CASE_V])
def test_config_round_trip(case):
    arch, cfg = resolve(copy.deepcopy(case), "test")
    assert arch.name == "Zaposun" and isinstance(cfg, ZaposunConfig)
    assert ZaposunConfig.from_dict(cfg.to_dict()) == cfg
    assert [layer.type for layer in cfg.layers] == [c["type"] for c in case["layers"]]
    assert cfg.streams == case["streams"] and cfg.groups == case["norm"]["groups"]


def test_defaults_of_absent_keys():
    case = copy.deepcopy(CASE_R)
    left = case["layers"][1]["mixer"]["left"]
    for key in ("scale", "kv_heads", "vdim", "mask"):
        del left[key]
    del case["streams"], case["logit_scale"], case["norm"]["groups"]
    del case["layers"][0]["mixer"]["decay_rank"]
    _, cfg = resolve(case, "test")
    att = cfg.layers[1].left
    assert att.scale == pytest.approx(24 ** -0.5) and att.kv_heads == 2 and att.vdim == 24 and att.chunk == 0
    assert att.rot_dims == 0 and att.rot_layout == "halves"
    assert cfg.streams == 1 and cfg.groups == 1 and cfg.logit_scale == 1.0 and cfg.layers[0].decay_rank == 0
    assert cfg.layers[2].ff == 0 and cfg.layers[1].ff == 18


def test_config_problems_are_listed_together():
    bad = copy.deepcopy(CASE_P)
    del bad["vocab"]
    bad["layers"][0]["mixer"]["left"]["kv_heads"] = 3           # 4 heads are no multiple of 3
    bad["layers"][0]["mixer"]["right"]["state"] = 0
    bad["layers"][1]["type"] = "conv"
    bad["layers"][2]["mixer"]["left"]["rot"]["dims"] = 34       # beyond the head size
    bad["norm"]["groups"] = 5                                   # does not divide the width
    with pytest.raises(ConfigError) as err:
        resolve(bad, "test")
    text = str(err.value)
    for piece in ("vocab", "kv_heads", "state", "conv", "rot.dims"):
        assert piece in text, (piece, text)
    bad = copy.deepcopy(CASE_P)
    bad["norm"]["groups"] = 5
    with pytest.raises(ConfigError, match="groups"):
        resolve(bad, "test")


def test_declared_tensors_follow_the_configuration():
    arch = get_architecture("Zaposun")
    _, cfg = resolve(copy.deepcopy(CASE_P), "test")
    decls = {d.name: d.shape for d in declared_tensors(arch, cfg)}
    assert decls["embed"] == (97, 64) and decls["bigram"] == (54, 64) and decls["head"] == (97, 64)
    assert decls["l0.mix.left.q"] == (64, 64) and decls["l0.mix.left.k"] == (32, 64) and decls["l0.mix.left.v"] == (64, 64)
    assert decls["l0.mix.left.o"] == (64, 4 * 32) and decls["l0.mix.left.q.norm"] == (16,)
    assert decls["l0.mix.right.in"] == (80, 64) and decls["l0.mix.right.x"] == (3 + 10, 40)
    assert decls["l0.mix.right.conv"] == (40, 3) and decls["l0.mix.right.A_log"] == (40, 5)
    assert decls["l0.mix.right.dt"] == (40, 3) and decls["l0.mix.left.out"] == (64,)
    assert decls["l1.mix.w1"] == (6, 64) and decls["l1.mix.w2"] == (48, 6) and decls["l1.mix.u"] == (2, 24)
    assert decls["l1.mix.mu.w"] == (64,) and decls["l1.shift"] == (64,)
    assert decls["l1.hc1.mix"] == (2, 2) and decls["l1.hc2.in"] == (2,)
    assert not any(n.startswith("l1.mlp") for n in decls) and decls["l2.mlp.gate"] == (24, 64)


def test_the_decay_rank_comes_from_the_stored_tensor_when_the_configuration_is_silent():
    arch = get_architecture("Zaposun")
    case = copy.deepcopy(CASE_P)
    del case["layers"][1]["mixer"]["decay_rank"]
    _, cfg = resolve(case, "test")
    with pytest.raises(ValueError, match="decay"):
        declared_tensors(arch, cfg)
    decls = {d.name: d.shape for d in declared_tensors(arch, cfg, stored_names={"l1.mix.w1": (11, 64)})}
    assert decls["l1.mix.w1"] == (11, 64) and decls["l1.mix.w2"] == (48, 11)


def test_state_of_blocks_mixers_and_the_model_in_the_cache_manager():
    """Every layer gets its token-shift row, a wkv layer its previous input and matrix state, a parallel layer the
    scan's state and convolution inputs under the branch's name, the model its previous token; a slot that is
    handed out again is zero."""
    from sharpinference_b200.cache import CacheManager
    from sharpinference_b200.weights.source import DeclaringWeights
    arch = get_architecture("Zaposun")
    _, cfg = resolve(copy.deepcopy(CASE_P), "test")
    model = arch.build(cfg, DeclaringWeights(torch.float32))
    cache = CacheManager(model.schedule, model.blocks, page_size=4, num_pages=8, max_requests=2, dtype=torch.float32,
                         device="cpu", model_state_specs=model.state_specs)
    slots = cache.layer_slots()
    assert set(slots[0].states) == {"shift", "right.S", "right.conv"}
    assert slots[0].states["right.S"].shape == (2, 40 * 5) and slots[0].states["right.conv"].shape == (2, 2 * 40)
    assert set(slots[1].states) == {"shift", "prev", "S"} and slots[1].states["S"].shape == (2, 2 * 24 * 24)
    assert cache.model_states["prev_token"].shape == (2,) and cache.model_states["prev_token"].dtype == torch.int32
    assert len(cache.groups) == 2 and {g.spec.kind for g in cache.groups} == {"chunk"}
    assert sorted(g.spec.span for g in cache.groups) == [7, 70]
    a = cache.add_request("a")
    for t in list(slots[1].states.values()) + [cache.model_states["prev_token"]]:
        t[a.state_slot] = 3
    cache.free_request("a")
    b = cache.add_request("b")
    assert b.state_slot == a.state_slot
    assert all(float(t[b.state_slot].abs().sum()) == 0 for t in slots[1].states.values())
    assert int(cache.model_states["prev_token"][b.state_slot]) == 0


def test_cache_groups_of_models_with_one_kind_of_mixer():
    from sharpinference_b200.cache import CacheManager
    from sharpinference_b200.weights.source import DeclaringWeights
    arch = get_architecture("Zaposun")
    for case, kinds in ((CASE_U, []), (CASE_V, [("chunk", 9, 2), ("full", 0, 1)])):
        _, cfg = resolve(copy.deepcopy(case), "test")
        model = arch.build(cfg, DeclaringWeights(torch.float32))
        cache = CacheManager(model.schedule, model.blocks, page_size=4, num_pages=8, max_requests=2, dtype=torch.float32,
                             device="cpu", model_state_specs=model.state_specs)
        assert [(g.spec.kind, g.spec.span, len(g.entries)) for g in cache.groups] == kinds


# -- the plain implementation against itself ---------------------------------------------------
def _rand(*shape, seed=0, scale=1.0):
    return scale * torch.randn(*shape, generator=torch.Generator().manual_seed(seed), dtype=F64)


def test_plain_group_norm_and_activation():
    x = _rand(5, 12, seed=1, scale=3.0)
    y = plain.group_norm(x, torch.ones(12, dtype=F64), 3, 0.0)
    assert torch.allclose((y * y).view(5, 3, 4).mean(-1), torch.ones(5, 3, dtype=F64))
    assert torch.allclose(plain.group_norm(x, torch.ones(12, dtype=F64), 1, 1e-5), plain.rms(x, 1e-5))
    z = torch.tensor([-3.0, 0.0, 0.5, 4.0], dtype=F64)
    assert torch.allclose(plain.gelu_tanh(z), torch.nn.functional.gelu(z, approximate="tanh"))
    assert float(plain.softplus(torch.tensor(50.0, dtype=F64))) == 50.0


def test_plain_rotation_is_relative_and_leaves_the_tail():
    q, k = _rand(1, 1, 12, seed=2), _rand(1, 1, 12, seed=3)
    for layout in ("halves", "interleaved"):
        dots = []
        for shift in (0, 17):
            qr = plain.rotate(q, torch.tensor([5 + shift]), 100.0, 8, layout)
            kr = plain.rotate(k, torch.tensor([2 + shift]), 100.0, 8, layout)
            assert torch.equal(qr[..., 8:], q[..., 8:])
            dots.append(float((qr * kr).sum()))
        assert dots[0] == pytest.approx(dots[1], abs=1e-12)
        back = plain.rotate(plain.rotate(q, torch.tensor([9]), 100.0, 12, layout), torch.tensor([9]), 100.0, 12, layout, sign=-1.0)
        assert torch.allclose(back, q)
    h = plain.rotate(q, torch.tensor([1]), 100.0, 4, "halves")
    assert float(h[0, 0, 0]) == pytest.approx(float(q[0, 0, 0] * math.cos(1.0) - q[0, 0, 2] * math.sin(1.0)))


def test_plain_pair_embedding_rows():
    embed, pairs = _rand(10, 4, seed=4), _rand(6, 4, seed=5)
    x = plain.embedding([3, 7, 7], embed, pairs, 5, 11, 2)
    assert torch.equal(x[0], embed[3] + pairs[5])
    assert torch.equal(x[1], embed[7] + pairs[(3 * 11 + 7 * 2) % 5]) and torch.equal(x[2], embed[7] + pairs[(7 * 13) % 5])


def test_plain_chunks_count_from_position_zero(tmp_path):
    """Inside a chunk a token's output does not depend on anything before the chunk's first position (attention
    alone; the recurrent branch is what carries the past)."""
    folder = write("P", str(tmp_path))
    cfg, w = plain.load_folder(folder)
    m = cfg["layers"][0]["mixer"]["left"]
    h = _rand(20, cfg["width"], seed=6)
    full = plain.chunk_attention(h, w, "l0.mix.left.", m, 1e-5)
    h2 = h.clone()
    h2[:7] = _rand(7, cfg["width"], seed=7)
    other = plain.chunk_attention(h2, w, "l0.mix.left.", m, 1e-5)
    assert torch.allclose(full[7:], other[7:]) and not torch.allclose(full[:7], other[:7])
    assert not torch.allclose(plain.chunk_attention(h, w, "l0.mix.left.", m, 1e-5, chunk_delta=1)[7:8], full[7:8])


@pytest.mark.parametrize("name", sorted(CASES))
def test_random_folder_loads_and_runs_plain(tmp_path, name):
    folder = write(name, str(tmp_path))
    cfg, w = plain.load_folder(folder)
    arch, typed = resolve(cfg, "test")
    assert {d.name for d in declared_tensors(arch, typed)} == set(w)
    toks = traces.random_tokens(cfg["vocab"], 12, seed=1)
    logits, layers = plain.forward(cfg, w, toks, want_layers=True)
    assert logits.shape == (12, cfg["vocab"]) and len(layers) == len(cfg["layers"]) and bool(torch.isfinite(logits).all())
    # a prefix gives the same logits: everything is causal
    assert torch.allclose(plain.forward(cfg, w, toks[:7]), logits[:7], atol=1e-12)
