"""Mevuvik on the GPU against the plain implementation (tests/plain_mevuvik.py): each new
kernel alone at sizes other than any model's, with inputs made so that a fault shows; models of
one mechanism each, with attention made sharp so that one lost key changes the result; then the
engine under every way of cutting requests into steps, in float32 and bfloat16, with and without
replayed launch sequences; then greedy generation through the Python entry point and its
scheduler, and the programs a user starts."""
import copy
import math
import os
import random
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import mevuvik_tiny as mv
import plain_mevuvik as plain
import schedules

pytestmark = pytest.mark.gpu
BOUND = {"float32": 2e-5, "bfloat16": 3e-2}


@pytest.fixture(scope="module")
def ops():
    from rvllm_b200.kernels import cuda_ops
    return cuda_ops()


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = str(tmp_path_factory.mktemp("mv"))
    return {n: mv.write(root, n) for n in mv.CONFIGS}


def dev(t, dtype=None):
    return t.to("cuda", dtype) if dtype is not None else t.to("cuda")


def close(got, want, dtype, scale=None, bound=None):
    want = torch.as_tensor(np.asarray(want), dtype=torch.float64)
    got = got.detach().to("cpu", torch.float64).reshape(want.shape)
    s = float(want.abs().max()) if scale is None else scale
    err = float((got - want).abs().max()) / max(s, 1e-30)
    assert err < max(bound or 0.0, 1e-5 if dtype == torch.float32 else 2e-2), err


def rnd(gen, dtype, *shape, std=1.0):
    """Random values that both sides can hold exactly."""
    return (torch.randn(*shape, generator=gen) * std).to(dtype).double()


# ---- norm with a scaled pending sub-layer and an added vector -------------------------------------

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width", [176, 50, 1024])
def test_norm_adds_scaled_rows_and_a_vector(ops, dtype, width):
    g = torch.Generator().manual_seed(width)
    n = 37
    resid, delta = rnd(g, torch.float32, n, width), rnd(g, dtype, n, width)
    scale, add = rnd(g, torch.float32, width), rnd(g, torch.float32, width)
    weight = torch.full((width,), 1.3, dtype=torch.float64)
    eps = 1e-3
    for use_scale, use_add, use_delta in ((1, 1, 1), (1, 0, 1), (0, 1, 1), (0, 1, 0)):
        x = resid.clone()
        if use_delta:
            x = x + (delta * scale if use_scale else delta)
        if use_add:
            x = x + add
        want = plain.rms(x.numpy(), eps) * 1.3
        r = dev(resid.float())
        out = torch.empty(n, width, device="cuda", dtype=dtype)
        ops.add_rmsnorm(r, dev(delta, dtype) if use_delta else None, dev(weight.float()), eps, out,
                        None, delta_scale=dev(scale.float()) if use_scale and use_delta else None,
                        add=dev(add.float()) if use_add else None)
        close(out, want, dtype)
        close(r, x, torch.float32)                        # the stream has moved on
        rows = torch.tensor([5, 0, 36], dtype=torch.int32)
        r2 = dev(resid.float())
        out2 = torch.empty(3, width, device="cuda", dtype=dtype)
        ops.add_rmsnorm(r2, dev(delta, dtype) if use_delta else None, dev(weight.float()), eps,
                        out2, dev(rows),
                        delta_scale=dev(scale.float()) if use_scale and use_delta else None,
                        add=dev(add.float()) if use_add else None)
        close(out2, want[rows.long().numpy()], dtype)
        close(r2, resid, torch.float32)                   # with a row list the stream stays


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_relu_squared_sum_of_two_and_gate_per_head(ops, dtype):
    g = torch.Generator().manual_seed(1)
    for n, w in ((5, 48), (33, 50), (64, 256)):
        z = rnd(g, dtype, n, w)
        out = torch.empty(n, w, device="cuda", dtype=dtype)
        ops.relu2(dev(z, dtype), out)
        close(out, plain.relu_squared(z.numpy()), dtype)
        a, b = rnd(g, dtype, n, w), rnd(g, dtype, n, w)
        ops.weighted_sum(dev(a, dtype), 1.2, dev(b, dtype), -0.9, out)
        close(out, 1.2 * a - 0.9 * b, dtype)
    for n, H, size, extra in ((7, 3, 10, 5), (40, 8, 48, 16)):
        x = rnd(g, dtype, n, H * size)
        rows = rnd(g, dtype, n, extra + H, std=2.0)
        y = dev(x, dtype)
        ops.head_gate(y, H, size, dev(rows, dtype), extra)
        want = x.reshape(n, H, size) * torch.sigmoid(rows[:, extra:])[:, :, None]
        close(y, want, dtype)


# ---- latent rows: two norms, the turned key part, the cache write; turned query parts -----------------

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("sizes", [(80, 112, 16, 5, 48), (9, 14, 6, 3, 10), (40, 48, 2, 2, 8),
                                   (0, 16, 16, 4, 24)])
def test_latent_rows_and_turned_parts(ops, dtype, sizes):
    q_rank, rank, rot, H, d = sizes
    g = torch.Generator().manual_seed(rank)
    n, eps, base = 21, 1e-4, 777.0
    gate_cols = 5
    rows = rnd(g, dtype, n, q_rank + gate_cols + rank + rot)
    wq, wkv = rnd(g, torch.float32, max(q_rank, 1)), rnd(g, torch.float32, rank)
    positions = torch.tensor([0, 1, 2, 3, 1000, 4095, 17] * 3, dtype=torch.int32)
    slots = torch.tensor(random.Random(3).sample(range(40), n), dtype=torch.int32)
    slots[4] = -1                                            # a filling token writes nothing
    freq = torch.tensor([base ** (-2.0 * i / rot) for i in range(rot // 2)], dtype=torch.float32)
    cache = torch.full((10, 4, 1, rank + rot), 9.0, device="cuda", dtype=dtype)
    cq = torch.empty(n, q_rank, device="cuda", dtype=dtype) if q_rank else None
    kv_off = q_rank + gate_cols
    ops.latent_prepare(dev(rows, dtype), 0, q_rank, dev(wq.float()) if q_rank else None, cq, kv_off,
                       rank, rot, dev(wkv.float()), eps, dev(freq), dev(positions), dev(slots), cache)
    r = rows.numpy()
    if q_rank:
        close(cq, plain.rms(r[:, :q_rank], eps) * wq.numpy(), dtype)
    pages = cache.cpu().double().reshape(40, rank + rot)
    for t in range(n):
        s = int(slots[t])
        if s < 0:
            continue
        want = np.concatenate([plain.rms(r[t, kv_off:kv_off + rank], eps) * wkv.numpy(),
                               plain.rotate_half(r[t, kv_off + rank:], int(positions[t]), base)])
        # angles are float32 products of position and frequency: at position 4095 their
        # rounding is 2^-12 of a turn at most
        close(pages[s], want, dtype, bound=2e-3 if int(positions[t]) > 100 else None)
    untouched = [s for s in range(40) if s not in slots.tolist()]
    assert float((pages[untouched] - 9.0).abs().max()) == 0
    # queries: in every head the last `rot` of d + rot values turn, the rest stay
    q = rnd(g, dtype, n, H * (d + rot) + 3)
    x = dev(q, dtype)
    ops.rope_heads(x, H, d + rot, d, rot, dev(freq), dev(positions))
    want = q.clone().numpy()
    for t in range(n):
        for h in range(H):
            a = h * (d + rot) + d
            want[t, a:a + rot] = plain.rotate_half(q[t, a:a + rot].numpy(), int(positions[t]), base)
    small = [t for t in range(n) if int(positions[t]) <= 100]
    close(x.cpu()[small], want[small], dtype)
    close(x, want, dtype, bound=2e-3 if dtype == torch.float32 else None)


# ---- the router with a correction; experts without a gate ---------------------------------------------

def test_router_compares_with_the_correction_and_weighs_without(ops):
    g = torch.Generator().manual_seed(2)
    for E, top, W, n in ((12, 3, 176, 50), (5, 1, 50, 9), (8, 8, 64, 20), (64, 6, 128, 33)):
        x = rnd(g, torch.bfloat16, n, W)
        router = rnd(g, torch.float32, E, W, std=W ** -0.5)
        corr = rnd(g, torch.float32, E, std=0.5)
        corr[0] = -10.0                                      # never chosen unless all are
        corr[E - 1] = 10.0                                   # always chosen
        for xt in (torch.float32, torch.bfloat16):
            ids = torch.empty(n, top, dtype=torch.int32, device="cuda")
            wts = torch.empty(n, top, dtype=torch.float32, device="cuda")
            ops.moe_route(dev(x, xt), dev(router.float()), 1, 1, 2, 1e-20, ids, wts,
                          route_scale=2.5, choice_bias=dev(corr.float()))
            logits = torch.empty(n, E, dtype=torch.float32, device="cuda")
            logits.copy_(dev((x @ router.T).float()))
            ids2, wts2 = torch.empty_like(ids), torch.empty_like(wts)
            ops.moe_select(logits, 1, 1, 2, 1e-20, ids2, wts2, route_scale=2.5,
                           choice_bias=dev(corr.float()))
            for t in range(n):
                chosen, w = plain.route((router @ x[t]).numpy(), corr.numpy(), top, 2.5)
                for got_i, got_w in ((ids, wts), (ids2, wts2)):
                    assert got_i[t].tolist() == list(chosen), (E, t)
                    assert np.allclose(got_w[t].cpu().numpy(), w, rtol=2e-5, atol=1e-7)
                assert chosen[0] == E - 1 and (top == E or 0 not in chosen)
    # without a correction the kernel is what it was: the largest scores, weights summing to one
    logits = dev(torch.tensor([[0.3, 2.0, -1.0, 2.0, 0.1]]))
    ids = torch.empty(1, 2, dtype=torch.int32, device="cuda")
    wts = torch.empty(1, 2, dtype=torch.float32, device="cuda")
    ops.moe_select(logits, 1, 1, 2, 1e-20, ids, wts)
    assert ids.tolist() == [[1, 3]] and abs(float(wts.sum()) - 1.0) < 1e-6


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("sizes", [(12, 3, 176, 56, 300), (5, 2, 48, 24, 7), (4, 4, 64, 136, 130),
                                   (3, 1, 50, 22, 40)])
def test_experts_without_a_gate(ops, dtype, sizes):
    E, top, W, F, n = sizes
    g = torch.Generator().manual_seed(E + n)
    x = rnd(g, dtype, n, W)
    up, down = rnd(g, dtype, E, F, W, std=W ** -0.5), rnd(g, dtype, E, W, F, std=F ** -0.5)
    rng = random.Random(n)
    ids = torch.tensor([rng.sample(range(E), top) for _ in range(n)], dtype=torch.int32)
    wts = torch.rand(n, top, generator=g).float()
    out = torch.empty(n, W, device="cuda", dtype=dtype)
    modes = ["simple", "grouped"] if dtype == torch.bfloat16 and W % 8 == 0 and F % 8 == 0 else ["simple"]
    for mode in modes:
        keep = ops.moe_mode
        ops.moe_mode = mode
        try:
            ops.moe_experts(dev(x, dtype), dev(ids), dev(wts), dev(up, dtype), dev(down, dtype), out,
                            activation="relu2")
        finally:
            ops.moe_mode = keep
        want = np.zeros((n, W))
        for t in range(n):
            for k in range(top):
                e = int(ids[t, k])
                act = plain.relu_squared(up[e].numpy() @ x[t].numpy())
                if dtype == torch.bfloat16:
                    act = torch.from_numpy(act).to(torch.bfloat16).double().numpy()
                want[t] += float(wts[t, k]) * (down[e].numpy() @ act)
        close(out, want, dtype)
    ops.check_status()


# ---- the matrix memory ----------------------------------------------------------------------------

def _memory_case(H, d, dv, W, seed):
    g = torch.Generator().manual_seed(seed)
    t = {"q": rnd(g, torch.float32, H * d, W, std=W ** -0.5), "k": rnd(g, torch.float32, H * d, W, std=W ** -0.5),
         "v": rnd(g, torch.float32, H * dv, W, std=W ** -0.5), "g": rnd(g, torch.float32, H * dv, W, std=W ** -0.5),
         "i": rnd(g, torch.float32, H, W, std=2 * W ** -0.5), "f": rnd(g, torch.float32, H, W, std=2 * W ** -0.5),
         "i.b": rnd(g, torch.float32, H), "f.b": rnd(g, torch.float32, H) + 2.0,
         "norm": 1.0 + 0.1 * rnd(g, torch.float32, H * dv)}
    t = {k: v.numpy() for k, v in t.items()}
    t["o"] = np.eye(H * dv)                                   # the mixer's inner rows come out
    return t, g


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("sizes", [(3, 48, 72), (2, 6, 5), (1, 64, 64), (3, 24, 40), (2, 130, 33),
                                   (1, 300, 16), (5, 16, 130)])
def test_matrix_memory_kernel(ops, dtype, sizes):
    """Three requests of unequal length in portions of unequal size, one of them token by
    token, in state slots that are not in order; a slot used again starts from zero."""
    H, d, dv = sizes
    W, cap, eps = 32, 5.0, 1e-5
    t, g = _memory_case(H, d, dv, W, d + dv)
    m = {"heads": H, "dim": d, "vdim": dv, "gate_cap": cap}
    w_in = np.concatenate([t[k] for k in ("q", "k", "v", "i", "f", "g")])
    lengths = {"a": 70, "b": 9, "c": 33}
    hs = {r: rnd(g, torch.float32, n, W).numpy() for r, n in lengths.items()}
    want = {r: plain.matrix_memory(h, m, t, eps)[0] for r, h in hs.items()}
    rec = ops.mlstm_record(H, d, dv)
    state = torch.zeros(6, rec, device="cuda")
    state[4].fill_(3.0)                                      # never touched
    slot = {"a": 5, "b": 0, "c": 2}
    cuts = {"a": [40, 2, 1, 27], "b": [1] * 9, "c": [3, 30]}
    done = {r: 0 for r in lengths}
    got = {r: [] for r in lengths}
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device="cuda")
    for step in range(9):
        parts = [(r, cuts[r][step]) for r in ("b", "a", "c") if step < len(cuts[r])]
        parts.sort(key=lambda p: p[1] != 1)                  # single tokens first
        if not parts:
            break
        rows, starts, slots, token_req = [], [0], [], []
        # an empty request in the middle and a filling request at the end, as padded steps have
        layout = parts[:1] + [(None, 0)] + parts[1:] + [(None, 2)]
        for ri, (r, n) in enumerate(layout):
            h = hs[r][done[r]:done[r] + n] if r else np.full((n, W), 1e3)
            rows.append(h @ w_in.T)
            starts.append(starts[-1] + n)
            slots.append(slot[r] if r else -1)
            token_req += [ri] * n
        x = dev(torch.from_numpy(np.concatenate(rows)).float())
        ctx = SimpleNamespace(q_start=i32(starts), state_slot=i32(slots), token_req=i32(token_req),
                              n_reqs=len(layout))
        out = torch.full((x.shape[0], H * dv), float("nan"), device="cuda", dtype=dtype)
        ops.mlstm(x, dev(torch.from_numpy(t["i.b"]).float()), dev(torch.from_numpy(t["f.b"]).float()),
                  dev(torch.from_numpy(t["norm"]).float()), state, ctx, out, H, d, dv, cap, eps)
        for ri, (r, n) in enumerate(layout):
            if r:
                got[r].append(out[starts[ri]:starts[ri + 1]].cpu())
                done[r] += n
            else:
                assert float(out[starts[ri]:starts[ri + 1]].abs().max() if n else 0.0) == 0.0
    for r in lengths:
        close(torch.cat(got[r]), want[r], dtype, bound=3e-5 if dtype == torch.float32 else None)
    assert float((state[4] - 3.0).abs().max()) == 0 and float(state[1].abs().max()) == 0
    # the record after the last token: columns of C with n as the last one, then the maxima
    _, st = plain.matrix_memory(hs["c"], m, t, eps)
    recd = state[2].cpu().double()
    for h in range(H):
        C, n, mx = st[h]
        cols = recd[h * (dv + 1) * d:(h + 1) * (dv + 1) * d].reshape(dv + 1, d)
        close(cols[:dv], C.T, torch.float32, bound=3e-5, scale=max(1.0, float(np.abs(C).max())))
        close(cols[dv], n, torch.float32, bound=3e-5, scale=max(1.0, float(np.abs(n).max())))
        assert abs(float(recd[H * (dv + 1) * d + h]) - mx) < 1e-5 * max(1.0, abs(mx))


def test_matrix_memory_long_and_with_strong_gates(ops):
    """600 tokens with input gates far above and forget gates far below the cap's middle: the
    running maximum keeps every exponential in range, and the first tokens still show."""
    H, d, dv, W, cap, eps = 2, 32, 24, 16, 12.0, 1e-6
    t, g = _memory_case(H, d, dv, W, 77)
    t["i"] *= 8.0
    t["f"] *= 8.0
    m = {"heads": H, "dim": d, "vdim": dv, "gate_cap": cap}
    h = rnd(g, torch.float32, 600, W).numpy()
    want = plain.matrix_memory(h, m, t, eps)[0]
    w_in = np.concatenate([t[k] for k in ("q", "k", "v", "i", "f", "g")])
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device="cuda")
    state = torch.zeros(1, ops.mlstm_record(H, d, dv), device="cuda")
    outs, at = [], 0
    for n in [500] + [1] * 100:
        x = dev(torch.from_numpy(h[at:at + n] @ w_in.T).float())
        ctx = SimpleNamespace(q_start=i32([0, n]), state_slot=i32([0]), token_req=i32([0] * n), n_reqs=1)
        out = torch.empty(n, H * dv, device="cuda")
        ops.mlstm(x, dev(torch.from_numpy(t["i.b"]).float()), dev(torch.from_numpy(t["f.b"]).float()),
                  dev(torch.from_numpy(t["norm"]).float()), state, ctx, out, H, d, dv, cap, eps)
        outs.append(out.cpu())
        at += n
    close(torch.cat(outs), want, torch.float32, bound=1e-4)


# ---- the engine -------------------------------------------------------------------------------------

_models = {}


def engine(folder, dtype):
    from rvllm_b200.engine import load_model
    if (folder, dtype) not in _models:
        _models[(folder, dtype)] = load_model(folder, dtype, "cuda")[0]
    return _models[(folder, dtype)]


def run_schedule(model, steps, page, slots=4, graphs=False):
    from rvllm_b200.engine import ModelRunner, make_cache
    cache = make_cache(model, page, schedules.tokens_held(steps, 64) // page, slots)
    runner = ModelRunner(model, cache, model.ops, use_graphs=graphs)
    got = schedules.replay(runner, steps)
    model.ops.check_status()
    assert not cache.requests and all(g.pool.in_use == 0 for g in cache.groups)
    return got, runner


_plain = {}


def compare(got, folder, cfg, reqs, dtype, share=0.04):
    """float32: every position within the bound.  bfloat16: a router score that is a close call
    may fall the other way after rounding and change a token's experts, which is no fault; so a
    few positions in a hundred may lie outside the bound."""
    over, total = [], 0
    for rid, ids in reqs.items():
        key = (folder, tuple(ids))
        if key not in _plain:
            _plain[key] = mv.plain_logits(folder, None, ids, cfg=cfg)
        ref = _plain[key]
        scale = float(ref.abs().max())
        for p in range(len(ids)):
            err = float((got[(rid, p)].double() - ref[p]).abs().max()) / scale
            total += 1
            if not err < BOUND[dtype]:
                over.append((rid, p, err))
    assert len(over) <= (0 if dtype == "float32" else share * total), (len(over), total, over[:5])


def _requests(vocab, lengths, seed):
    rng = random.Random(seed)
    return {f"q{i}": [rng.randrange(vocab) for _ in range(n)] for i, n in enumerate(lengths)}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_every_cut_equals_plain(folders, name, dtype):
    """Whole prompts; a prompt then its last tokens one by one; portions down to two tokens;
    mixed batches of unequal requests on four slots, with more requests than slots, so that
    pages and slots are used again."""
    model = engine(folders[name], dtype)
    cfg = mv.config(name)
    reqs = _requests(cfg["vocab"], (130, 1, 2, 67, 200, 33, 64, 65), 3)
    f = folders[name]
    compare(run_schedule(model, schedules.whole(reqs), 16)[0], f, cfg, reqs, dtype)
    compare(run_schedule(model, schedules.tail_decode(reqs, 90), 8)[0], f, cfg, reqs, dtype)
    compare(run_schedule(model, schedules.portions(reqs), 16)[0], f, cfg, reqs, dtype)
    compare(run_schedule(model, schedules.portions(reqs, (64, 2, 100, 3)), 4)[0], f, cfg, reqs, dtype)
    for seed in (0, 1):
        compare(run_schedule(model, schedules.mixed(reqs, seed), 16)[0], f, cfg, reqs, dtype)


def _one_mechanism(tmp, which):
    """A model of one layer whose attention is sharp (a large scale, large projections), so that
    a single lost or misplaced key changes the result by much more than the bound."""
    from rvllm_b200.config import config_from_dict
    from rvllm_b200.weights import write_random_model
    from rvllm_b200.weights.safetensors_io import SafetensorsFile, write_streamed
    if which == "latent":
        layer = {"type": "latent_attention", "mlp": None,
                 "mixer": mv._latent(4, 24, 8, 16, 40, 24, 6.0, 50.0)}
    elif which == "left":
        layer = {"type": "parallel", "mlp": None,
                 "mixer": mv._parallel((6, 3, 24, 40, 8.0), (1, 8, 8, 6.0), 1.0, 0.0)}
    else:
        layer = {"type": "parallel", "mlp": None,
                 "mixer": mv._parallel((1, 1, 8, 8, 1.0), (3, 40, 24, 9.0), 0.0, 1.0)}
    cfg = {"architecture": "Mevuvik", "vocab": 150, "width": 72, "norm": {"eps": 1e-5},
           "residual_mult": 1.0, "layers": [layer]}
    folder = write_random_model(os.path.join(tmp, which), config_from_dict(copy.deepcopy(cfg)), 7)
    path = os.path.join(folder, "model.safetensors")
    f = SafetensorsFile(path)
    tensors = {n: f.tensor(n).clone() for n in f.names()}
    del f
    for n, t in tensors.items():                              # projections that give scores of size
        if n.endswith((".dq", ".uq", ".dkv", ".uk", ".q", ".k", ".i", ".f", "embed")):
            tensors[n] = (t.float() * 6.0).to(t.dtype)
    write_streamed(path, [(n, tuple(t.shape), t.dtype) for n, t in tensors.items()],
                   lambda n: tensors[n])
    return folder, cfg


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["latent", "left", "right"])
def test_one_mechanism_alone_with_sharp_scores(tmp_path_factory, which, dtype):
    """Keys far away (hundreds of positions back), at page borders and in the first tokens,
    in prompts, in portions that begin inside a page and in single tokens."""
    folder, cfg = _one_mechanism(str(tmp_path_factory.mktemp("one")), which)
    model = engine(folder, dtype)
    reqs = _requests(cfg["vocab"], (400, 63, 17), 11)
    ref = mv.plain_logits(folder, None, reqs["q0"], cfg=cfg)
    if which != "right":
        # the scores are sharp: most queries put most of their weight on one key
        assert float(ref.abs().max()) > 0.05
    for steps, page in ((schedules.whole(reqs), 16), (schedules.tail_decode(reqs, 40), 8),
                        (schedules.portions(reqs, (15, 2, 17, 130, 3)), 16),
                        (schedules.mixed(reqs, 4), 4)):
        compare(run_schedule(model, steps, page)[0], folder, cfg, reqs, dtype, share=0.05)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "D"])
def test_replayed_steps_equal_plain(folders, name, dtype):
    """The same with captured launch sequences: single-token steps and padded mixtures are
    replayed from graphs; requests come and go, so slots and pages are used again."""
    model = engine(folders[name], dtype)
    cfg = mv.config(name)
    reqs = _requests(cfg["vocab"], (90, 5, 41, 120, 33, 70, 18), 8)
    for steps, page in ((schedules.tail_decode(reqs, 40), 16), (schedules.mixed(reqs, 2), 8),
                        (schedules.mixed(reqs, 3, max_live=3, decode_tail=20), 16)):
        got, runner = run_schedule(model, steps, page, graphs=True)
        compare(got, folders[name], cfg, reqs, dtype)
        assert runner.graph_steps > 0


def test_long_decoding(folders):
    """400 tokens one by one after a short prompt, across many pages and splits."""
    model = engine(folders["B"], "float32")
    cfg = mv.config("B")
    reqs = _requests(cfg["vocab"], (420,), 6)
    got, _ = run_schedule(model, schedules.tail_decode(reqs, 400), 16, graphs=True)
    compare(got, folders["B"], cfg, reqs, "float32")


def test_a_batch_does_not_change_a_request(folders):
    """A request beside others gives what it gives alone, in the same cut."""
    model = engine(folders["A"], "float32")
    reqs = _requests(mv.config("A")["vocab"], (70, 31, 5), 12)
    alone, _ = run_schedule(model, schedules.whole({"q0": reqs["q0"]}), 16)
    steps = [{"step": 0, "entries": [{"id": r, "tokens": ids, "want": list(range(len(ids)))}
                                      for r, ids in reqs.items()], "end": list(reqs)}]
    together, _ = run_schedule(model, steps, 16)
    scale = max(float(alone[("q0", p)].abs().max()) for p in range(70))
    for p in range(70):
        assert float((alone[("q0", p)] - together[("q0", p)]).abs().max()) < 1e-5 * scale


@pytest.mark.parametrize("name", ["A", "C"])
def test_greedy_generation_through_the_entry_point(folders, name):
    """Greedy tokens through `Generator` (scheduler, portions, preemption by a small pool) equal
    the plain implementation's argmax chain."""
    from rvllm_b200 import GenerateOptions, Generator
    rng = random.Random(9)
    cfg = mv.config(name)
    new = 20
    tensors = mv.read_tensors(folders[name])

    def plain_greedy(ids):
        """The argmax chain, or None when two logits on the way are too close to call."""
        ids = list(ids)
        for _ in range(new):
            row = mv.plain_logits(folders[name], name, ids, tensors=tensors)[-1]
            top = torch.topk(row, 2).values
            if float(top[0] - top[1]) < 1e-3 * float(row.abs().max()):
                return None
            ids.append(int(row.argmax()))
        return ids[-new:]

    prompts, want = [], []
    for n in (5, 37, 70):
        for attempt in range(20):
            p = [rng.randrange(cfg["vocab"]) for _ in range(n)]
            w = plain_greedy(p)
            if w is not None:
                prompts.append(p)
                want.append(w)
                break
    assert len(prompts) == 3
    gen = Generator.load(folders[name], dtype="float32")
    for opts in (GenerateOptions(max_tokens=new, block_size=16, stop_tokens=[]),
                 GenerateOptions(max_tokens=new, block_size=8, stop_tokens=[], prefill_chunk=7,
                                 max_batched_tokens=12),
                 GenerateOptions(max_tokens=new, block_size=8, stop_tokens=[], num_blocks=16,
                                 prefill_chunk=20)):
        assert gen.complete_batch(prompts, opts) == want


def test_command_line_and_trace_replay(folders, tmp_path):
    """The design through the programs a user starts: `rvllm random-model` writes a folder from a
    config.json, `rvllm cli` completes prompts of token ids, `bin/trace_run` replays steps from
    standard input and writes logits that equal the plain implementation's."""
    import json
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg_path = tmp_path / "config.json"
    cfg_path.write_text(json.dumps(mv.config("B")))
    folder = str(tmp_path / "model")
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "rvllm"), "random-model",
                        "--config", str(cfg_path), "--seed", "5", "--out", folder],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    tensors = mv.read_tensors(folder)
    prompt = [3, 1, 4, 1, 5, 9, 2, 6]
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "rvllm"), "cli", "--model", folder,
                        "--dtype", "float32", "--token-ids", "--prompt", " ".join(map(str, prompt)),
                        "--max-tokens", "5", "--block-size", "8"],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    got = [int(t) for t in r.stdout.strip().splitlines()[0].split()]
    ids = list(prompt)
    for tok in got:                           # each token is the plain argmax at its place
        row = mv.plain_logits(folder, "B", ids, tensors=tensors)[-1]
        assert float(row.max() - row[tok]) < 1e-3 * float(row.abs().max())
        ids.append(tok)
    assert len(got) == 5
    reqs = _requests(mv.config("B")["vocab"], (70, 33, 90, 41, 12), 4)
    steps = schedules.mixed(reqs, seed=2)
    vocab = mv.config("B")["vocab"]
    for dtype in ("float32", "bfloat16"):
        out = tmp_path / dtype
        cmd = [sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folder,
               "--dtype", dtype, "--out", str(out), "--max-tokens",
               str(schedules.tokens_held(steps, 64))]
        r = subprocess.run(cmd, input="\n".join(json.dumps(s) for s in steps) + "\n",
                           capture_output=True, text=True, timeout=900)
        assert r.returncode == 0, r.stderr[-2000:]
        assert [l for l in r.stdout.split("\n") if l.startswith("done")] == \
            [f"done {s['step']}" for s in steps]
        got, pos = {}, {k: 0 for k in reqs}
        for s in steps:
            arr = np.fromfile(out / f"{s['step']}.f32", dtype="<f4").reshape(-1, vocab)
            k = 0
            for e in s["entries"]:
                for w in e["want"]:
                    got[(e["id"], pos[e["id"]] + w)] = torch.from_numpy(arr[k].copy())
                    k += 1
                pos[e["id"]] += len(e["tokens"])
            assert k == arr.shape[0]
        over, total = 0, 0
        for rid, ids in reqs.items():
            ref = mv.plain_logits(folder, "B", ids, tensors=tensors)
            for p in range(len(ids)):
                err = float((got[(rid, p)].double() - ref[p]).abs().max() / ref.abs().max())
                total += 1
                over += not err < BOUND[dtype]
        assert over <= (0 if dtype == "float32" else 0.04 * total), (dtype, over, total)
