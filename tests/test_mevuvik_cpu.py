"""Mevuvik without a GPU: its configuration, its tensor declarations, the plain implementation's
own mechanisms, and the engine's host side (cache manager with two caches for one call, batch
packing, step function) driven through the plain kernel references against the plain
implementation of the whole design."""
import math
import random

import numpy as np
import pytest
import torch

import mevuvik_tiny as mv
import plain_mevuvik as plain
import schedules
from plain_ops import PlainOps
from rvllm_b200.config import config_from_dict
from rvllm_b200.config.registry import architecture
from rvllm_b200.engine import ModelRunner, load_model, make_cache
from rvllm_b200.errors import ConfigError
from rvllm_b200.parts.base import PagedNeed, SeveralNeeds, StateNeed
from rvllm_b200.parts.model import param_decls


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = str(tmp_path_factory.mktemp("mv"))
    return {n: mv.write(root, n) for n in mv.CONFIGS}


def test_config_round_trip_and_errors():
    for name in mv.CONFIGS:
        cfg = config_from_dict(mv.config(name))
        assert config_from_dict(cfg.to_dict()) == cfg
        assert cfg.architecture == "Mevuvik"
    bad = mv.config("A")
    bad["layers"][0]["mixer"]["rot"]["dims"] = 4              # only the whole part turns
    with pytest.raises(ConfigError):
        config_from_dict(bad)
    bad = mv.config("A")
    bad["layers"][1]["mixer"]["left"]["kv_heads"] = 4         # does not divide the heads
    with pytest.raises(ConfigError):
        config_from_dict(bad)
    bad = mv.config("A")
    bad["loop"]["stop"] = 5                                   # beyond the last layer
    with pytest.raises(ConfigError):
        config_from_dict(bad)
    bad = mv.config("B")
    bad["layers"][0]["mlp"]["router"]["top"] = 6              # more than the experts
    with pytest.raises(ConfigError):
        config_from_dict(bad)
    bad = mv.config("B")
    del bad["layers"][1]["mixer"]["q_rank"]
    with pytest.raises(ConfigError):
        config_from_dict(bad)
    bad = mv.config("B")
    bad["layers"][2]["type"] = "sideways"
    with pytest.raises(ConfigError):
        config_from_dict(bad)


def test_declared_tensors_and_run_order():
    cfg = config_from_dict(mv.config("A"))
    spec = architecture("Mevuvik").build_spec(cfg)
    decls = param_decls(spec)
    assert decls["embed"].shape == (300, 96) and decls["embed.norm"].shape == ()
    assert decls["final.norm"].shape == () and decls["l2.norm1"].shape == ()
    assert decls["loop.step"].shape == (3, 96)
    assert decls["l0.mix.dq"].shape == (40, 96) and decls["l0.mix.dq.norm"].shape == (40,)
    assert decls["l0.mix.uq"].shape == (4 * (16 + 8), 40)
    assert decls["l0.mix.dkv"].shape == (32 + 8, 96) and decls["l0.mix.dkv.norm"].shape == (32,)
    assert decls["l0.mix.uk"].shape == (4 * 16, 32) and decls["l0.mix.uv"].shape == (4 * 24, 32)
    assert decls["l0.ls1"].shape == (96,) and decls["l0.ls2"].shape == (96,)
    assert decls["l0.mlp.router"].shape == (6, 96) and decls["l0.mlp.correction"].shape == (6,)
    assert decls["l0.mlp.e5.up"].shape == (48, 96) and "l0.mlp.e0.gate" not in decls
    assert decls["l1.mix.left.q"].shape == (6 * 32, 96) and decls["l1.mix.left.g"].shape == (6, 96)
    assert decls["l1.mix.left.v"].shape == (2 * 16, 96) and decls["l1.mix.left.o"].shape == (96, 6 * 16)
    assert decls["l1.mix.right.q"].shape == (2 * 24, 96) and decls["l1.mix.right.v"].shape == (2 * 16, 96)
    assert decls["l1.mix.right.i"].shape == (2, 96) and decls["l1.mix.right.f.b"].shape == (2,)
    assert decls["l1.mix.right.norm"].shape == (2 * 16,)
    assert decls["l1.mlp.up"].shape == (80, 96) and "l2.norm2" not in decls and "l2.ls2" not in decls
    # layer 0, then layers 1 and 2 three times (each pass adds its row before layer 1), then layer 3
    assert [(c.layer, c.add) for c in spec.order] == [
        (0, None), (1, ("loop.step", 0)), (2, None), (1, ("loop.step", 1)), (2, None),
        (1, ("loop.step", 2)), (2, None), (3, None)]
    spec_b = architecture("Mevuvik").build_spec(config_from_dict(mv.config("B")))
    assert [(c.layer, c.add) for c in spec_b.order] == [(0, None), (1, None), (2, None)]
    assert "loop.step" not in param_decls(spec_b)


def test_every_pass_and_every_branch_has_a_cache_of_its_own(folders):
    model, _ = load_model(folders["A"], "float32", "cpu", PlainOps())
    needs = model.cache_needs()
    assert len(needs) == 8
    assert needs[0] == PagedNeed(1, 32 + 8, values=False)
    par = SeveralNeeds((PagedNeed(2, 32, v_head_dim=16), StateNeed((2 * (16 + 1) * 24 + 2,))))
    assert needs[1] == needs[3] == needs[5] == par
    assert needs[2] == needs[4] == needs[6] == PagedNeed(1, 16 + 16, values=False)
    cache = make_cache(model, 4, 32, 2)
    views = cache.views()
    assert views[1].kind == "several" and [p.kind for p in views[1].parts] == ["paged", "state"]
    # the three passes write different pages and different records
    assert views[1].parts[0].k.data_ptr() != views[3].parts[0].k.data_ptr()
    assert views[1].parts[1].state.data_ptr() != views[5].parts[1].state.data_ptr()
    assert views[2].k.data_ptr() != views[4].k.data_ptr()
    # a slot's records are zero for whoever receives it
    cache.add("a")
    slot = cache.requests["a"].slot
    views[3].parts[1].state[slot].fill_(7.0)
    cache.free("a")
    cache.add("b")
    assert cache.requests["b"].slot == slot and float(views[3].parts[1].state[slot].abs().max()) == 0


# ---- the plain implementation's mechanisms, each against a form written another way -----------

def test_plain_rotation_keeps_lengths_and_relative_angles():
    rng = np.random.default_rng(0)
    a, b = rng.standard_normal(12), rng.standard_normal(12)
    for p, q in ((0, 0), (5, 3), (1000, 990)):
        ra, rb = plain.rotate_half(a, p, 100.0), plain.rotate_half(b, q, 100.0)
        assert abs(np.linalg.norm(ra) - np.linalg.norm(a)) < 1e-12
        # the product depends on the distance only
        assert abs(ra @ rb - plain.rotate_half(a, p - q, 100.0) @ b) < 1e-9
    assert np.allclose(plain.rotate_half(a, 0, 100.0), a)
    # pair (0, 6) turns by p, pair (5, 11) by p * base^(-10/12)
    one = np.zeros(12); one[5] = 1.0
    t = plain.rotate_half(one, 2, 100.0)
    ang = 2 * 100.0 ** (-10 / 12)
    assert abs(t[5] - math.cos(ang)) < 1e-12 and abs(t[11] - math.sin(ang)) < 1e-12


def test_plain_matrix_memory_equals_its_unrolled_sum():
    """With the maxima divided out, C_t = sum_j prod_{l>j} f_l i_j k_j v_j^T: the stabilised
    recurrence equals the direct sum whenever the direct form does not overflow."""
    rng = np.random.default_rng(1)
    W, H, d, dv, T = 12, 2, 3, 4, 9
    m = {"heads": H, "dim": d, "vdim": dv, "gate_cap": 6.0}
    t = {k: rng.standard_normal(s) for k, s in (("q", (H * d, W)), ("k", (H * d, W)),
         ("v", (H * dv, W)), ("g", (H * dv, W)), ("i", (H, W)), ("f", (H, W)), ("i.b", (H,)),
         ("f.b", (H,)), ("norm", (H * dv,)), ("o", (W, H * dv)))}
    h = rng.standard_normal((T, W))
    got, state = plain.matrix_memory(h, m, t, 1e-5)
    li = 6.0 * np.tanh((h @ t["i"].T + t["i.b"]) / 6.0)
    lf = plain.log_sigmoid(6.0 * np.tanh((h @ t["f"].T + t["f.b"]) / 6.0))
    q = (h @ t["q"].T).reshape(T, H, d) / math.sqrt(d)
    k = (h @ t["k"].T).reshape(T, H, d)
    v = (h @ t["v"].T).reshape(T, H, dv)
    out = np.zeros((T, H, dv))
    for hh in range(H):
        for i in range(T):
            w = np.array([math.exp(li[j, hh] + lf[j + 1:i + 1, hh].sum()) for j in range(i + 1)])
            C = sum(w[j] * np.outer(k[j, hh], v[j, hh]) for j in range(i + 1))
            n = sum(w[j] * k[j, hh] for j in range(i + 1))
            # the running maximum starts at 0, so exp(-m) is at most 1 and bounds the divisor
            mx = 0.0
            for j in range(i + 1):
                mx = max(lf[j, hh] + mx, li[j, hh])
            out[i, hh] = C.T @ q[i, hh] / (max(abs(n @ q[i, hh]), 1.0) + 1e-6 * math.exp(mx))
    want = plain.rms(out, 1e-5).reshape(T, H * dv) * t["norm"] * plain.sigmoid(h @ t["g"].T)
    assert np.allclose(got, want @ t["o"].T, atol=1e-9)
    # carried in two portions: the same
    a, st = plain.matrix_memory(h[:4], m, t, 1e-5)
    b, _ = plain.matrix_memory(h[4:], m, t, 1e-5, st)
    assert np.allclose(np.concatenate([a, b]), got, atol=1e-12)


def test_plain_route_compares_with_the_correction_and_weighs_without():
    z = np.array([2.0, 1.0, 0.0, -1.0])
    corr = np.array([-5.0, 0.0, 0.0, 3.0])
    chosen, w = plain.route(z, corr, 2, 2.0)
    s = plain.sigmoid(z)
    assert list(chosen) == [3, 1]                       # 0.27 + 3 and 0.73 + 0
    assert np.allclose(w, s[[3, 1]] / s[[3, 1]].sum() * 2.0) and abs(w.sum() - 2.0) < 1e-12
    chosen, w = plain.route(z, np.zeros(4), 4, 1.0)     # all of them: weights sum to 1
    assert sorted(chosen) == [0, 1, 2, 3] and abs(w.sum() - 1.0) < 1e-12


def test_plain_run_order():
    cfg = {"layers": [0] * 5, "loop": {"start": 1, "stop": 3, "times": 2}}
    assert plain.run_order(cfg) == [(0, None), (1, 0), (2, None), (1, 1), (2, None), (3, None),
                                    (4, None)]
    assert plain.run_order({"layers": [0, 0]}) == [(0, None), (1, None)]


# ---- the engine's host side -----------------------------------------------------------------------

@pytest.mark.parametrize("name", ["A", "B", "C"])
@pytest.mark.parametrize("schedule", ["whole", "tail_decode", "portions", "mixed"])
def test_engine_host_side_under_every_cut(folders, name, schedule):
    model, _ = load_model(folders[name], "float32", "cpu", PlainOps())
    vocab = mv.config(name)["vocab"]
    rng = random.Random(5)
    reqs = {f"q{i}": [rng.randrange(vocab) for _ in range(n)]
            for i, n in enumerate((61, 2, 35, 1, 90, 17))}
    steps = schedules.tail_decode(reqs, 12) if schedule == "tail_decode" else \
        getattr(schedules, schedule)(reqs)
    page = 4
    cache = make_cache(model, page, schedules.tokens_held(steps, 64) // page, 4)
    runner = ModelRunner(model, cache, PlainOps())
    got = schedules.replay(runner, steps)
    tensors = mv.read_tensors(folders[name])
    for rid, ids in reqs.items():
        ref = mv.plain_logits(folders[name], name, ids, tensors=tensors).to(torch.float32)
        scale = float(ref.abs().max())
        for p in range(len(ids)):
            assert float((got[(rid, p)] - ref[p]).abs().max()) < 2e-5 * scale, (rid, p)
    assert not cache.requests and all(g.pool.in_use == 0 for g in cache.groups)
