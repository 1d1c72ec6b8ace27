"""Vifanex without a GPU: its configuration, its tensor declarations, and the engine's host
side (cache manager, batch packing, step function) driven through the plain kernel references
against the plain implementation of the whole design."""
import random

import numpy as np
import pytest
import torch

import plain_vifanex as plain
import schedules
import vifanex_tiny as vf
from plain_ops import PlainOps
from rvllm_b200.config import config_from_dict
from rvllm_b200.config.registry import architecture
from rvllm_b200.engine import ModelRunner, load_model, make_cache
from rvllm_b200.errors import ConfigError
from rvllm_b200.parts.base import PagedNeed, StateNeed
from rvllm_b200.parts.model import param_decls


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = str(tmp_path_factory.mktemp("vf"))
    return {n: vf.write(root, n) for n in vf.CONFIGS}


def test_config_round_trip_and_errors():
    for name in vf.CONFIGS:
        cfg = config_from_dict(vf.config(name))
        assert config_from_dict(cfg.to_dict()) == cfg
        assert cfg.architecture == "Vifanex"
    bad = vf.config("A")
    bad["layers"][1]["mixer"]["kv_heads"] = 4                 # does not divide the heads
    with pytest.raises(ConfigError):
        config_from_dict(bad)
    bad = vf.config("A")
    bad["layers"][2]["mixer"]["vdim"] = 24                    # mixed values of another size
    with pytest.raises(ConfigError):
        config_from_dict(bad)
    bad = vf.config("A")
    bad["layers"][1]["mixer"]["rot"]["dims"] = 15             # pairs need an even count
    with pytest.raises(ConfigError):
        config_from_dict(bad)
    bad = vf.config("A")
    bad["layers"][0]["mlp"]["router"]["groups"]["count"] = 4  # 6 experts in 4 groups
    with pytest.raises(ConfigError):
        config_from_dict(bad)
    bad = vf.config("B")
    bad["layers"][0]["mlp"]["router"]["top"] = 4              # one group of 3 cannot give 4
    with pytest.raises(ConfigError):
        config_from_dict(bad)
    bad = vf.config("B")
    bad["layers"][1]["type"] = "delta"
    with pytest.raises(ConfigError):
        config_from_dict(bad)
    bad = vf.config("B")
    del bad["layers"][1]["mixer"]["conv"]
    with pytest.raises(ConfigError):
        config_from_dict(bad)
    bad = vf.config("C")
    bad["layers"][1]["mlp"]["limit"] = 0.0
    with pytest.raises(ConfigError):
        config_from_dict(bad)


def test_ranks_come_from_the_tensor_file(folders):
    """The ranks of the decay and gate products are in no key of a model folder made
    elsewhere: they are the shapes of two tensors."""
    raw = vf.config("A")
    for layer in raw["layers"]:
        layer["mixer"].pop("decay_rank", None)
        layer["mixer"].pop("gate_rank", None)
    cfg = config_from_dict(raw)
    with pytest.raises(ConfigError):
        architecture("Vifanex").build_spec(cfg)
    from rvllm_b200.weights.loader import tensor_shapes
    full = cfg.with_tensor_shapes(tensor_shapes(folders["A"]))
    assert full == config_from_dict(vf.config("A"))
    wrong = vf.config("A")
    wrong["layers"][0]["mixer"]["decay_rank"] = 9
    with pytest.raises(ConfigError):
        config_from_dict(wrong).with_tensor_shapes(tensor_shapes(folders["A"]))


def test_declared_tensors():
    cfg = config_from_dict(vf.config("A"))
    decls = param_decls(architecture("Vifanex").build_spec(cfg))
    assert decls["embed"].shape == (300, 96) and decls["head"].shape == (300, 96)
    assert decls["l0.mix.q"].shape == (2 * 16, 96) and decls["l0.mix.v"].shape == (4 * 24, 96)
    assert decls["l0.mix.q.conv"].shape == (32, 3) and decls["l0.mix.v.conv"].shape == (96, 3)
    assert decls["l0.mix.b"].shape == (4, 96) and decls["l0.mix.A_log"].shape == (4,)
    assert decls["l0.mix.a1"].shape == (8, 96) and decls["l0.mix.a2"].shape == (4 * 16, 8)
    assert decls["l0.mix.g1"].shape == (12, 96) and decls["l0.mix.g2"].shape == (4 * 24, 12)
    assert decls["l0.mix.dt_bias"].shape == (64,) and decls["l0.mix.norm"].shape == (24,)
    assert decls["l0.mix.o"].shape == (96, 96)
    assert decls["l0.hc1.in"].shape == (3,) and decls["l0.hc2.mix"].shape == (3, 3)
    assert decls["l0.mlp.router"].shape == (6, 96) and decls["l0.mlp.e5.down"].shape == (96, 48)
    assert decls["l0.mlp.shared.gate"].shape == (32, 96) and "l0.mlp.e6.gate" not in decls
    assert "l0.mlp.e0.gate.b" not in decls and "l0.mlp.shared.up.b" not in decls
    assert decls["l1.mix.q"].shape == (6 * 32, 96) and decls["l1.mix.q.norm"].shape == (192,)
    assert decls["l1.mix.k.norm"].shape == (64,) and decls["l1.mix.v.b"].shape == (32,)
    assert decls["l1.mix.vmix"].shape == () and decls["l1.mix.o"].shape == (96, 6 * 16)
    assert decls["l1.mlp.gate.b"].shape == (80,) and decls["l1.mlp.down.b"].shape == (96,)
    assert "l2.norm2" not in decls and "l2.hc2.in" not in decls and "l2.hc1.out" in decls
    assert "l3.mlp.shared.gate" not in decls and decls["final.norm"].shape == (96,)
    plainer = param_decls(architecture("Vifanex").build_spec(config_from_dict(vf.config("B"))))
    assert not any(".hc" in k for k in plainer) and "l0.mix.vmix" not in plainer


def test_cache_needs(folders):
    model, _ = load_model(folders["A"], "float32", "cpu", PlainOps())
    needs = model.cache_needs()
    assert needs[1] == PagedNeed(2, 32, window=20, v_head_dim=16)
    assert needs[2] == PagedNeed(2, 16, window=7)
    # taps - 1 rows of q | k | v inputs, then a [dim, vdim] matrix per head
    assert needs[0] == StateNeed((2 * (2 * 2 * 16 + 4 * 24) + 4 * 16 * 24,))
    assert needs[3] == StateNeed((3 * (2 * 2 * 32 + 2 * 8) + 2 * 32 * 8,))
    model_b, _ = load_model(folders["B"], "float32", "cpu", PlainOps())
    assert model_b.cache_needs()[1] == StateNeed((3 * 8 * 40,))     # one tap: the matrices alone


def test_plain_mechanisms_one_by_one():
    """The plain implementation's own pieces on cases worked by hand."""
    f = plain.rotation_frequencies({"dims": 4, "base": 100.0})
    assert np.allclose(f, [1.0, 0.1])
    # wavelengths 2 pi, 20 pi, 200 pi against an original length of 100: kept (below 100/4),
    # between, divided by the factor (above 100/1)
    f = plain.rotation_frequencies({"dims": 6, "base": 1000.0,
                                    "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 100}})
    s = (100 / (20 * np.pi) - 1.0) / 3.0
    assert np.allclose(f, [1.0, (1 - s) * 0.1 / 8 + s * 0.1, 0.01 / 8])
    x = np.array([1.0, 0.0, 0.0, 2.0, 5.0])
    y = plain.rotate_pairs(x, 3, np.array([np.pi / 6, np.pi / 3]))
    assert np.allclose(y, [0.0, 1.0, 0.0, -2.0, 5.0])
    # groups of neighbours: the best single score decides; ties go to the lower index
    s = np.array([0.05, 0.3, 0.2, 0.21, 0.04, 0.2])
    assert list(plain.route(s, 2, 3, 1)) == [1, 0]
    assert list(plain.route(s, 3, 3, 2)) == [1, 3, 2]
    assert list(plain.route(s, 2, 1, 1)) == [1, 3]
    # one delta step: decay first, then the correction, and the read-out sees the write
    S = np.array([[1.0, 2.0], [0.0, 4.0]])
    S2, o = plain.delta_step(S, np.array([1.0, 1.0]), np.array([1.0, 0.0]), np.array([3.0, 3.0]),
                             0.5, np.array([0.5, 0.25]))
    assert np.allclose(S2, [[1.75, 2.0], [0.0, 1.0]]) and np.allclose(o, [1.75, 3.0])
    t = {"gate": np.array([[2.0], [-1.0]]), "up": np.array([[3.0], [0.25]]), "down": np.eye(2)}
    y = plain.glu_clamp(np.array([1.0]), t, 1.5, False)
    assert np.allclose(y, [1.5 * plain.sigmoid(1.702 * 1.5) * 2.5,
                           -plain.sigmoid(-1.702) * 1.25])
    xs = np.arange(12.0).reshape(2, 2, 3)
    mix = np.array([[1.0, 2.0], [0.0, -1.0]])
    out = plain.streams_write(xs, np.ones((2, 3)), mix, np.array([10.0, 0.0]))
    assert np.allclose(out[0], xs[0] + 10.0) and np.allclose(out[1], 2 * xs[0] - xs[1])


@pytest.mark.parametrize("name", ["A", "B", "C"])
@pytest.mark.parametrize("schedule", ["whole", "tail_decode", "portions", "mixed"])
def test_engine_host_side_under_every_cut(folders, name, schedule):
    model, _ = load_model(folders[name], "float32", "cpu", PlainOps())
    vocab = vf.config(name)["vocab"]
    rng = random.Random(5)
    reqs = {f"q{i}": [rng.randrange(vocab) for _ in range(n)]
            for i, n in enumerate((61, 2, 35, 1, 90, 17))}
    steps = schedules.tail_decode(reqs, 12) if schedule == "tail_decode" else \
        getattr(schedules, schedule)(reqs)
    page = 4
    cache = make_cache(model, page, schedules.tokens_held(steps, 64) // page, 4)
    runner = ModelRunner(model, cache, PlainOps())
    got = schedules.replay(runner, steps)
    tensors = vf.read_tensors(folders[name])
    for rid, ids in reqs.items():
        ref = vf.plain_logits(folders[name], name, ids, tensors=tensors).to(torch.float32)
        for p in range(len(ids)):
            assert torch.allclose(got[(rid, p)], ref[p], atol=3e-5, rtol=0), (rid, p)
    assert not cache.requests and all(g.pool.in_use == 0 for g in cache.groups)
