"""Vifanex on the GPU against the plain implementation (tests/plain_vifanex.py): each new
kernel alone at sizes other than any model's, with inputs made so that a lost state, a window
that is one token off or a forgotten stream shows; then the engine under every way of cutting
requests into steps, in float32 and bfloat16, with and without replayed launch sequences; then
greedy generation through the Python entry point and its scheduler, and the programs a user
starts."""
import math
import random
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_vifanex as plain
import schedules
import vifanex_tiny as vf

pytestmark = pytest.mark.gpu
BOUND = {"float32": 2e-5, "bfloat16": 3e-2}


@pytest.fixture(scope="module")
def ops():
    from rvllm_b200.kernels import cuda_ops
    return cuda_ops()


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = str(tmp_path_factory.mktemp("vf"))
    return {n: vf.write(root, n) for n in vf.CONFIGS}


def dev(t, dtype=None):
    return t.to("cuda", dtype) if dtype is not None else t.to("cuda")


def i32(x):
    return torch.tensor(x, dtype=torch.int32, device="cuda")


def close(got, want, dtype, scale=None):
    want = torch.as_tensor(np.asarray(want), dtype=torch.float64)
    got = got.detach().to("cpu", torch.float64).reshape(want.shape)
    s = float(want.abs().max()) if scale is None else scale
    err = float((got - want).abs().max()) / max(s, 1e-30)
    assert err < (1e-5 if dtype == torch.float32 else 2e-2), err


def rounded(g, dtype, *shape, scale=1.0):
    """Random values that `dtype` holds exactly, as float64."""
    return (torch.randn(*shape, generator=g) * scale).to(dtype).double()


# ---- several residual streams -------------------------------------------------------------

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(1, 50), (2, 128), (3, 96), (4, 256), (5, 2050), (16, 33)])
def test_streams_between_sublayers(ops, dtype, shape):
    """Write-back of a pending output, read-in and norm in one kernel: from equal streams
    (the embedding rows), from streams that differ, in place, and for chosen rows only with
    the plain sum (the model's last norm)."""
    S, W = shape
    g = torch.Generator().manual_seed(S * 1000 + W)
    n, eps = 23, 1e-5
    emb = rounded(g, torch.float32, n, W, scale=3.0)
    y = rounded(g, dtype, n, W)
    mix = rounded(g, torch.float32, S, S, scale=0.7)
    a, b, w = (rounded(g, torch.float32, k) for k in (S, S, W))
    # first sub-layer: nothing pending, every stream the embedding row
    streams = torch.full((n, S, W), float("nan"), device="cuda")
    out = torch.empty(n, W, device="cuda", dtype=dtype)
    ops.hyper_norm(dev(emb.float()), streams, None, None, None, dev(a.float()), dev(w.float()), eps,
                   out)
    xs = np.stack([emb.numpy()] * S)
    close(streams.transpose(0, 1), xs, torch.float32)
    close(out, plain.rms_norm(plain.streams_read(xs, a.numpy()), w.numpy(), eps), dtype)
    # a pending output, in place
    ops.hyper_norm(streams, streams, dev(y, dtype), dev(mix.float()), dev(b.float()),
                   dev(a.float()), dev(w.float()), eps, out)
    xs2 = plain.streams_write(xs, y.numpy(), mix.numpy(), b.numpy())
    close(streams.transpose(0, 1), xs2, torch.float32)
    close(out, plain.rms_norm(plain.streams_read(xs2, a.numpy()), w.numpy(), eps), dtype)
    # chosen rows, the plain sum, nothing written back
    before = streams.clone()
    rows = [n - 1, 0, 7]
    out3 = torch.empty(3, W, device="cuda", dtype=dtype)
    ops.hyper_norm(streams, None, dev(y, dtype), dev(mix.float()), dev(b.float()), None,
                   dev(w.float()), eps, out3, i32(rows))
    xs3 = plain.streams_write(xs2, y.numpy(), mix.numpy(), b.numpy())
    close(out3, plain.rms_norm(xs3.sum(axis=0), w.numpy(), eps)[rows], dtype)
    assert torch.equal(before, streams)


def test_streams_mixing_is_from_to(ops):
    """mix[s, t] carries stream s into stream t: a matrix with one entry off the diagonal
    moves the first stream into the second and not the other way."""
    n, W = 4, 40
    x = torch.zeros(n, 2, W)
    x[:, 0] = 1.0
    x[:, 1] = 10.0
    mix = torch.tensor([[1.0, 1.0], [0.0, 1.0]])
    zero = torch.zeros(n, W)
    out = torch.empty(n, W, device="cuda")
    dst = torch.empty(n, 2, W, device="cuda")
    ops.hyper_norm(dev(x), dst, dev(zero), dev(mix), dev(torch.zeros(2)), dev(torch.ones(2)),
                   dev(torch.ones(W)), 0.0, out)
    assert torch.equal(dst[:, 0].cpu(), torch.full((n, W), 1.0))
    assert torch.equal(dst[:, 1].cpu(), torch.full((n, W), 11.0))


# ---- whole-projection norm, rotation of neighbours, value mixing ----------------------------

def plain_qkv(rows, bias, H, G, d, dv, wq, wk, eps, rot, positions, first, lam):
    """rows [N, Q + K + V] float64 -> (q [N, H, d], k [N, G, d], own v, cached v [N, G, dv])."""
    Q, K = H * d, G * d
    x = rows + (bias if bias is not None else 0.0)
    q = plain.rms_norm(x[:, :Q], wq, eps) if wq is not None else x[:, :Q].copy()
    k = plain.rms_norm(x[:, Q:Q + K], wk, eps) if wk is not None else x[:, Q:Q + K].copy()
    q, k = q.reshape(-1, H, d), k.reshape(-1, G, d)
    if rot is not None:
        # the angle is a float32 product of the position and a float32 frequency
        f = plain.rotation_frequencies(rot).astype(np.float32)
        for n, p in enumerate(positions):
            angles = (np.float32(p) * f).astype(np.float64)
            for a in range(H):
                q[n, a] = plain.rotate_pairs(q[n, a], 1.0, angles)
            for a in range(G):
                k[n, a] = plain.rotate_pairs(k[n, a], 1.0, angles)
    own = x[:, Q + K:].reshape(-1, G, dv)
    v = own if first is None else (1.0 - lam) * own + lam * first.reshape(-1, G, dv)
    return q, k, own, v


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("sizes", [(6, 2, 32, 16, 16), (3, 3, 10, 6, 6), (4, 1, 16, 48, 16), (8, 2, 64, 64, 32),
                                   (2, 2, 48, 16, 8), (16, 2, 128, 128, 128), (5, 5, 24, 40, 0)])
def test_projection_norm_rotation_and_value_mixing(ops, dtype, sizes):
    from rvllm_b200.parts.base import position_class
    from rvllm_b200.parts.spec import PositionSpec
    H, G, d, dv, rd = sizes
    g = torch.Generator().manual_seed(H * 100 + d)
    n, eps = 19, 1e-5
    Q, K, V = H * d, G * d, G * dv
    rows = rounded(g, torch.float32, n, Q + K + V, scale=2.0)
    bias, wq, wk = (rounded(g, torch.float32, k) for k in (Q + K + V, Q, K))
    positions = [0, 1, 2, 3, 300, 301, 4095, 77, 78, 5, 100000, 9, 10, 11, 12, 13, 14, 15, 16]
    slots = list(range(40, 40 + n))
    slots[4] = -1                                   # a padding row writes nothing
    scaling = (4.0, 1.0, 3.0, 64)
    rot = None if rd == 0 else {"dims": rd, "base": 500.0,
                                "scaling": dict(zip(("factor", "low", "high", "original"), scaling))}
    freq, rot_dims = None, 0
    if rd:
        pos = position_class("rope_pairs")(PositionSpec("rope_pairs", d, 500.0, 1 << 24, rd, scaling), "cuda")
        freq, rot_dims = pos.frequencies()
        close(freq, plain.rotation_frequencies(rot), torch.float32)
    first = rounded(g, torch.float32, n, V)
    for mode in ("none", "source", "mix"):
        kc = torch.full((64, G, d), float("nan"), device="cuda", dtype=dtype)
        vc = torch.full((64, G, dv), float("nan"), device="cuda", dtype=dtype)
        q_out = torch.empty(n, Q, device="cuda", dtype=dtype)
        own_out = torch.empty(n, V, device="cuda") if mode == "source" else None
        ops.qkv_full_norm_rope_write(
            dev(rows.float()), dev(bias.float()), H, G, d, dv, dev(wq.float()), dev(wk.float()), eps,
            freq, rot_dims, i32(positions), i32(slots), q_out, kc, vc,
            dev(first.float()) if mode == "mix" else None, own_out,
            dev(torch.tensor([0.3])) if mode == "mix" else None)
        q, k, own, v = plain_qkv(rows.numpy(), bias.numpy(), H, G, d, dv, wq.numpy(), wk.numpy(), eps,
                                 rot, positions, first.numpy() if mode == "mix" else None, 0.3)
        close(q_out, q.reshape(n, Q), dtype)
        keep = [i for i in range(n) if slots[i] >= 0]
        close(kc[[slots[i] for i in keep]], k[keep], dtype)
        close(vc[[slots[i] for i in keep]], v[keep], dtype)
        if mode == "source":
            close(own_out, own.reshape(n, V), torch.float32)
        used = torch.zeros(64, dtype=torch.bool)
        used[[slots[i] for i in keep]] = True
        assert bool(torch.isnan(kc.float().cpu()[~used]).all())


def test_rotation_pairs_neighbours_not_halves(ops):
    """A head whose only non-zero entry is dimension 0 turns into dimensions 0 and 1, not
    into 0 and d/2; dimensions from `dims` on do not move."""
    from rvllm_b200.parts.base import position_class
    from rvllm_b200.parts.spec import PositionSpec
    d, rd = 16, 8
    freq, rot_dims = position_class("rope_pairs")(
        PositionSpec("rope_pairs", d, 100.0, 1 << 24, rd, None), "cuda").frequencies()
    rows = torch.zeros(1, 3 * d)
    rows[0, 0] = 1.0          # q: dimension 0
    rows[0, d + 10] = 1.0     # k: dimension 10, beyond the turning ones
    kc = torch.zeros(1, 1, d, device="cuda")
    vc = torch.zeros(1, 1, d, device="cuda")
    q = torch.empty(1, d, device="cuda")
    ops.qkv_full_norm_rope_write(dev(rows), None, 1, 1, d, d, None, None, 0.0, freq, rot_dims,
                                 i32([3]), i32([0]), q, kc, vc)
    want = torch.zeros(d, dtype=torch.float64)
    want[0], want[1] = math.cos(3.0), math.sin(3.0)
    close(q[0], want, torch.float32)
    assert float(kc[0, 0, 10]) == 1.0 and float(kc.abs().sum()) == 1.0


# ---- the gated delta rule -------------------------------------------------------------------

def plain_delta(proj, low, filt, a_log, dt_bias, norm_w, H, G, d, dv, eps):
    """One request's whole sequence in float64.  proj [T, C + H]: q | k | v | beta before the
    convolution; low [T, H d + H dv]: the decays' and the output gates' pre-activations.
    Returns (y [T, H dv], the state after the last token [H, d, dv])."""
    T = proj.shape[0]
    C = 2 * G * d + H * dv
    x = plain.conv_silu(proj[:, :C], filt)
    q = plain.unit(x[:, :G * d].reshape(T, G, d)) * d ** -0.5
    k = plain.unit(x[:, G * d:2 * G * d].reshape(T, G, d))
    v = x[:, 2 * G * d:].reshape(T, H, dv)
    beta = plain.sigmoid(proj[:, C:C + H])
    g = np.exp(-np.exp(a_log)[None, :, None] * plain.softplus(low[:, :H * d] + dt_bias).reshape(T, H, d))
    gate = plain.sigmoid(low[:, H * d:]).reshape(T, H, dv)
    o = np.zeros((T, H, dv))
    S = np.zeros((H, d, dv))
    for a in range(H):
        for i in range(T):
            S[a], o[i, a] = plain.delta_step(S[a], q[i, a // (H // G)], k[i, a // (H // G)], v[i, a],
                                             beta[i, a], g[i, a])
    y = o / np.sqrt((o ** 2).mean(axis=-1, keepdims=True) + eps) * norm_w * gate
    return y.reshape(T, H * dv), S


def run_delta(ops, seqs, cuts, H, G, d, dv, taps, filt, a_log, dt_bias, norm_w, eps, dtype, slots):
    """The kernels on several requests at once, each cut into portions (cycled sizes, a
    request's next portion in every call until it is done), with a request that has no slot
    and no tokens in every batch.  seqs: [(proj, low)] float64.  Returns (y per request, state)."""
    C = 2 * G * d + H * dv
    rec = ops.gated_delta_record(H, G, d, dv, taps)
    state = torch.full((max(slots) + 2, rec), float("nan"), device="cuda")
    for s in slots:
        state[s] = 0.0
    done = [0] * len(seqs)
    ys = [[] for _ in seqs]
    k = 0
    while any(done[i] < seqs[i][0].shape[0] for i in range(len(seqs))):
        batch = []
        for i, (proj, low) in enumerate(seqs):
            left = proj.shape[0] - done[i]
            if left > 0:
                take = min(cuts[k % len(cuts)], left)
                k += 1
                batch.append((i, done[i], take))
        batch.sort(key=lambda e: e[2] != 1)                    # single tokens first
        proj = torch.cat([seqs[i][0][a:a + n] for i, a, n in batch])
        low = torch.cat([seqs[i][1][a:a + n] for i, a, n in batch])
        q_start, token_req = [0], []
        for r, (i, a, n) in enumerate(batch):
            q_start.append(q_start[-1] + n)
            token_req += [r] * n
        q_start.append(q_start[-1])                            # the request without a slot
        ctx = SimpleNamespace(token_req=i32(token_req), q_start=i32(q_start),
                              state_slot=i32([slots[i] for i, _, _ in batch] + [-1]),
                              n_reqs=len(batch) + 1)
        y = torch.full((proj.shape[0], H * dv), float("nan"), device="cuda", dtype=dtype)
        # wider rows than the kernel reads: what follows beta belongs to someone else
        wide = torch.cat([proj, torch.full((proj.shape[0], 3), float("nan"), dtype=proj.dtype)], dim=1)
        ops.gated_delta(dev(wide.float().contiguous()), dev(low.float().contiguous()), dev(filt.float()),
                        dev(a_log.float()), dev(dt_bias.float()), dev(norm_w.float()), state, ctx, y,
                        H, G, d, dv, taps, 1e-6, eps)
        for r, (i, a, n) in enumerate(batch):
            ys[i].append(y[q_start[r]:q_start[r + 1]].cpu())
            done[i] = a + n
    assert bool(torch.isnan(state[max(slots) + 1]).all())
    return [torch.cat(y) for y in ys], state


def delta_case(g, T, H, G, d, dv, taps, memory=False):
    C = 2 * G * d + H * dv
    proj = rounded(g, torch.float32, T, C + H, scale=1.5)
    low = rounded(g, torch.float32, T, H * d + H * dv)
    filt = rounded(g, torch.float32, C, taps, scale=0.6)
    a_log = rounded(g, torch.float32, H, scale=0.5) - (14.0 if memory else 1.0)
    dt_bias = rounded(g, torch.float32, H * d) - 1.0
    norm_w = rounded(g, torch.float32, dv) + 1.0
    return proj, low, filt, a_log, dt_bias, norm_w


# heads, key heads, key size, value size, taps: every way the scan deals a state out to threads
DELTA_SIZES = [(4, 2, 16, 24, 3), (2, 2, 32, 8, 4), (3, 1, 8, 40, 1), (3, 1, 10, 6, 5), (4, 2, 64, 64, 4),
               (2, 1, 128, 128, 4), (3, 3, 64, 96, 3), (2, 1, 160, 48, 2), (1, 1, 260, 20, 2),
               (8, 2, 32, 32, 4), (2, 2, 5, 3, 2), (1, 1, 520, 9, 3)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("sizes", DELTA_SIZES)
def test_gated_delta_against_plain(ops, dtype, sizes):
    """Three requests of unequal length in one batch, cut into portions down to one and two
    tokens, in slots that are not 0, 1, 2; the record (convolution inputs and state) carries
    everything from call to call."""
    H, G, d, dv, taps = sizes
    g = torch.Generator().manual_seed(d * 7 + dv)
    eps = 1e-5
    _, _, filt, a_log, dt_bias, norm_w = delta_case(g, 1, H, G, d, dv, taps)
    seqs = []
    for T in (41, 3, 18):
        proj, low, *_ = delta_case(g, T, H, G, d, dv, taps)
        seqs.append((proj, low))
    want = [plain_delta(p.numpy(), l.numpy(), filt.numpy(), a_log.numpy(), dt_bias.numpy(),
                        norm_w.numpy(), H, G, d, dv, eps) for p, l in seqs]
    C = 2 * G * d + H * dv
    # (2, 1, 1): as many tokens as requests, one request without any, so one has two
    for cuts in ((64,), (1,), (7, 2, 1, 1, 5, 3, 2), (taps, 1, taps + 1), (2, 1, 1)):
        slots = [5, 2, 3]
        got, state = run_delta(ops, seqs, cuts, H, G, d, dv, taps, filt, a_log, dt_bias, norm_w, eps,
                               dtype, slots)
        for i in range(3):
            close(got[i], want[i][0], dtype)
            S = state[slots[i], (taps - 1) * C:].reshape(H, dv, d).transpose(1, 2)   # a column's rows lie together
            close(S, want[i][1], torch.float32, scale=max(1.0, float(np.abs(want[i][1]).max())))
            # the record's first part: the last taps-1 inputs, oldest first, zeros before the start
            T = seqs[i][0].shape[0]
            tail = torch.zeros(taps - 1, C, dtype=torch.float64)
            n = min(T, taps - 1)
            if n:
                tail[taps - 1 - n:] = seqs[i][0][T - n:, :C]
            if taps > 1:
                close(state[slots[i], :(taps - 1) * C], tail, torch.float32, scale=1.0)


@pytest.mark.parametrize("sizes", [(2, 1, 32, 16, 4), (2, 2, 128, 64, 2)])
def test_gated_delta_remembers_far_tokens(ops, sizes):
    """With decays next to 1 the state keeps what the first tokens wrote: 400 tokens later,
    through portions and single tokens, the read-out still equals the plain one, and differs
    from the one of a sequence whose first tokens were others."""
    H, G, d, dv, taps = sizes
    g = torch.Generator().manual_seed(11)
    T, eps = 420, 1e-6
    proj, low, filt, a_log, dt_bias, norm_w = delta_case(g, T, H, G, d, dv, taps, memory=True)
    want, S = plain_delta(proj.numpy(), low.numpy(), filt.numpy(), a_log.numpy(), dt_bias.numpy(),
                          norm_w.numpy(), H, G, d, dv, eps)
    other = proj.clone()
    other[:8] = rounded(g, torch.float32, 8, proj.shape[1], scale=1.5)
    changed, _ = plain_delta(other.numpy(), low.numpy(), filt.numpy(), a_log.numpy(), dt_bias.numpy(),
                             norm_w.numpy(), H, G, d, dv, eps)
    assert np.abs(changed[-1] - want[-1]).max() > 1e-2 * np.abs(want[-1]).max()
    for cuts in ((300, 100, 1), (33, 2, 1, 64)):
        got, state = run_delta(ops, [(proj, low)], cuts, H, G, d, dv, taps, filt, a_log, dt_bias, norm_w,
                               eps, torch.float32, [1])
        assert float((got[0].double() - torch.from_numpy(want)).abs().max()) < 2e-4 * np.abs(want).max()


def test_gated_delta_order_within_a_token(ops):
    """Decay, then the correction with the decayed state, then the read-out of the written
    state: one head, two tokens, numbers worked by the plain step."""
    H = G = 1
    d, dv, taps = 8, 4, 1
    g = torch.Generator().manual_seed(3)
    proj, low, filt, a_log, dt_bias, norm_w = delta_case(g, 2, H, G, d, dv, taps)
    a_log[:] = 0.5                                  # strong decay, so that its place matters
    want, S = plain_delta(proj.numpy(), low.numpy(), filt.numpy(), a_log.numpy(), dt_bias.numpy(),
                          norm_w.numpy(), H, G, d, dv, 1e-5)
    got, state = run_delta(ops, [(proj, low)], (1,), H, G, d, dv, taps, filt, a_log, dt_bias, norm_w, 1e-5,
                           torch.float32, [0])
    close(got[0], want, torch.float32)
    close(state[0].reshape(H, dv, d).transpose(1, 2), S, torch.float32)


# ---- the clamped gated feed-forward and the mixture -------------------------------------------

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_glu_clamp_kernel(ops, dtype):
    g = torch.Generator().manual_seed(2)
    for n, f in ((1, 7), (13, 96), (40, 1000)):
        gate_up = rounded(g, dtype, n, 2 * f, scale=3.0)
        bias = rounded(g, torch.float32, 2 * f)
        gate_up[0, :f] = 50.0                        # far beyond the limit
        gate_up[0, f:] = -50.0
        for limit, b in ((1.0, bias), (2.5, None), (0.25, bias)):
            out = torch.empty(n, f, device="cuda", dtype=dtype)
            ops.glu_clamp(dev(gate_up, dtype), None if b is None else dev(b.float()), out, limit, 1.702)
            x = gate_up.numpy() + (0.0 if b is None else b.numpy())
            gg, uu = np.minimum(x[:, :f], limit), np.clip(x[:, f:], -limit, limit)
            close(out, gg * plain.sigmoid(1.702 * gg) * (uu + 1.0), dtype)


def _ff_part(ops, spec, dtype, seed):
    from rvllm_b200.parts.base import feed_forward_class
    from rvllm_b200.weights.random_init import random_tensor
    cls = feed_forward_class(spec.kind)
    host = {n: random_tensor(n, d, seed, torch.bfloat16) for n, d in cls.params(spec).items()}
    part = cls(spec, {n: t.to("cuda", dtype) for n, t in host.items()}, ops, dtype)
    return part, {n: t.double().numpy() for n, t in host.items()}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(50, 34, 0.5), (96, 80, 1.0), (128, 256, 4.0)])
def test_dense_feed_forward_part(ops, dtype, shape):
    from rvllm_b200.parts.spec import GluClampSpec
    W, F, limit = shape
    part, t = _ff_part(ops, GluClampSpec("glu_clamp", W, ffn_dim=F, limit=limit, alpha=1.702, bias=True),
                       dtype, 4)
    g = torch.Generator().manual_seed(W)
    for n in (1, 9, 70):
        x = rounded(g, dtype, n, W, scale=2.0)
        got = part.forward(dev(x, dtype), None)
        want = np.stack([plain.glu_clamp(r, t, limit, True) for r in x.numpy()])
        close(got, want, dtype)


# width, experts, chosen, (groups, kept), expert width, factor, shared width
MOE_SHAPES = [(50, 6, 2, (3, 2), 34, 2.0, 20), (96, 9, 3, (3, 1), 48, 1.0, None), (64, 5, 2, (5, 3), 32, 1.25, 16),
              (128, 16, 4, (4, 3), 64, 1.5, 128), (72, 3, 3, None, 22, 3.0, 10), (128, 32, 6, (8, 4), 72, 0.5, None)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", MOE_SHAPES)
def test_mixture_part(ops, dtype, shape):
    """Softmax over all experts, groups of neighbours, scores scaled and not renormalised, a
    shared expert: the part against the plain mixture token by token.  Tokens whose choice is a
    close call (two scores nearer than rounding tells apart) are left out."""
    from rvllm_b200.parts.spec import GluClampSpec, MoESpec
    W, E, top, groups, F, factor, shared = shape
    spec = MoESpec("moe", W, ffn_dim=F, experts=E, top=top, groups=groups[0] if groups else 1,
                   keep=groups[1] if groups else 1, group_top=1, score="softmax", renormalize=False,
                   route_scale=factor, activation="glu_clamp", limit=1.5, alpha=1.702,
                   shared=None if shared is None else
                   GluClampSpec("glu_clamp", W, ffn_dim=shared, limit=0.7, alpha=1.702, bias=False))
    part, t = _ff_part(ops, spec, dtype, 6)
    mlp = {"router": {"experts": E, "top": top, "scale": factor}, "expert": {"ff": F, "limit": 1.5}}
    if groups:
        mlp["router"]["groups"] = {"count": groups[0], "keep": groups[1]}
    if shared is not None:
        mlp["shared"] = {"ff": shared, "limit": 0.7}
    g = torch.Generator().manual_seed(E)
    checked = 0
    for n in (1, 5, 64, 150):
        x = rounded(g, dtype, n, W, scale=2.0)
        got = part.forward(dev(x, dtype), None).to("cpu", torch.float64)
        want = plain.moe(x.numpy(), mlp, t)
        z = x.numpy() @ t["router"].T
        for i in range(n):
            s = np.sort(np.exp(z[i] - z[i].max()) / np.exp(z[i] - z[i].max()).sum())
            if np.min(np.diff(s)) < 1e-5 * s[-1]:      # the rows are exact in both types
                continue
            err = np.abs(got[i].numpy() - want[i]).max() / max(np.abs(want).max(), 1e-30)
            assert err < (1e-5 if dtype == torch.float32 else 2e-2), (n, i, err)
            checked += 1
    assert checked > 100


def test_router_weights_are_scores_times_factor(ops):
    """The chosen experts keep their softmax scores (over all experts, not only the chosen),
    times the factor; a group is as good as its best member; ties go to the lower index."""
    logits = torch.tensor([[0.0, 3.0, 2.0, 2.1, -1.0, 2.0],
                           [1.0, 1.0, 1.0, 1.0, 1.0, 1.0],
                           [5.0, 4.9, 0.0, 0.1, 4.0, 3.9]])
    for top, groups, keep in ((2, 3, 1), (3, 3, 2), (2, 1, 1), (4, 6, 4)):
        ids = torch.empty(3, top, dtype=torch.int32, device="cuda")
        wts = torch.empty(3, top, dtype=torch.float32, device="cuda")
        ops.moe_select(dev(logits), groups, keep, 1, 0.0, ids, wts, score="softmax", renormalize=False,
                       route_scale=1.5)
        for i in range(3):
            z = logits[i].double().numpy()
            s = np.exp(z - z.max()) / np.exp(z - z.max()).sum()
            chosen = plain.route(s, top, groups, keep)
            assert ids[i].tolist() == list(chosen), (top, groups, keep, i, ids[i].tolist(), list(chosen))
            assert np.allclose(wts[i].cpu().numpy(), 1.5 * s[chosen], rtol=1e-5)


# ---- a sliding window over keys with a value size of its own ----------------------------------

def plain_window_attend(q, k, v, scale, window, first):
    """q [T, H, d] at positions first.., k [S, G, d], v [S, G, dv] (float64 arrays): position i
    sees j with 0 <= i - j < window."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = np.zeros((T, H, v.shape[2]))
    for i in range(T):
        p = first + i
        lo = 0 if window is None else max(0, p - window + 1)
        for h in range(H):
            g = h // (H // G)
            s = k[lo:p + 1, g] @ q[i, h] * scale
            w = np.exp(s - s.max())
            out[i, h] = (w / w.sum()) @ v[lo:p + 1, g]
    return out


def window_attend(ops, q, k, v, first, page, dtype, scale, window, seed=0):
    """The kernels on queries at positions first.. of one sequence whose keys lie in shuffled
    pages, beside requests without tokens."""
    T, H, d = q.shape
    S, G, dv = v.shape
    n_pages = -(-S // page)
    order = list(range(n_pages + 3))
    random.Random(seed).shuffle(order)
    kc = torch.zeros(n_pages + 3, page, G, d, dtype=dtype)
    vc = torch.zeros(n_pages + 3, page, G, dv, dtype=dtype)
    for j in range(S):
        kc[order[j // page], j % page] = k[j].to(dtype)
        vc[order[j // page], j % page] = v[j].to(dtype)
    rows = q.reshape(T, H * d).to(dtype)
    if T == 1:
        rows = torch.cat([rows, torch.full_like(rows, float("nan"))])
        ctx = SimpleNamespace(q_start=i32([0, 1, 2]), ctx_lens=i32([first + 1, 0]), token_req=i32([0, 1]),
                              n_tokens=2, n_reqs=2, n_decode=2, max_q_len=1, max_ctx_len=first + 1)
        real = 0
    else:
        ctx = SimpleNamespace(q_start=i32([0, 0, T, T]), ctx_lens=i32([0, first + T, 0]),
                              token_req=i32([1] * T), n_tokens=T, n_reqs=3, n_decode=0,
                              max_q_len=T + 5, max_ctx_len=first + T)
        real = 1
    tab = torch.full((ctx.n_reqs, n_pages + 2), -1, dtype=torch.int32)
    tab[real, :n_pages] = torch.tensor(order[:n_pages])
    group = SimpleNamespace(block_table=dev(tab), max_blocks=tab.shape[1], page_size=page, window=window)
    out = torch.full((rows.shape[0], H * dv), float("nan"), device="cuda", dtype=dtype)
    ops.paged_attention(dev(rows), H, G, d, dev(kc), dev(vc), ctx, group, scale, window, out,
                        v_head_dim=dv)
    return out[:T].cpu().reshape(T, H, dv)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("sizes", [(6, 2, 32, 16), (4, 1, 16, 48), (3, 3, 10, 6), (8, 2, 64, 64), (4, 2, 96, 64),
                                   (2, 2, 48, 16), (4, 4, 128, 128)])
@pytest.mark.parametrize("window", [1, 7, 20, 33, 64, 130, None])
def test_window_edges_with_a_standout_key(ops, dtype, sizes, window):
    """One key's score towers over the rest.  Placed on the window's first position it takes
    all the weight; one position earlier it must take none.  In a prompt's portion and for a
    single token, at pages of 4 and 16, far into the sequence."""
    H, G, d, dv = sizes
    S = 300
    g = torch.Generator().manual_seed(H + d + (window or 0))
    q = rounded(g, dtype, S, H, d)
    k = rounded(g, dtype, S, G, d, scale=0.3)
    v = rounded(g, dtype, S, G, dv)
    scale = 0.25
    for first, T, page in ((299, 1, 16), (270, 30, 4), (0, 300, 16), (150, 1, 4), (140, 2, 16)):
        p = first + T - 1                                 # the last query of the portion
        inside = 0 if window is None else max(0, p - window + 1)
        for target in (inside, inside - 1):
            if target < 0:
                continue
            kk = k.clone()
            for a in range(G):                            # this key answers every head of its group
                m = q[p, a * (H // G):(a + 1) * (H // G)].mean(0)
                kk[target, a] = m * (24.0 / (scale * float(m @ m)))     # a score of 24
            kk = kk.to(dtype).double()
            want = plain_window_attend(q[first:first + T].numpy(), kk[:p + 1].numpy(), v[:p + 1].numpy(),
                                       scale, window, first)
            got = window_attend(ops, q[first:first + T], kk[:p + 1], v[:p + 1], first, page, dtype, scale,
                                window)
            close(got, want, dtype)
            if H == G and window not in (None, 1):
                near = np.abs(want[-1] - v[target].numpy()).max() < 0.05
                assert near == (target == inside)


# ---- the engine ---------------------------------------------------------------------------

_models = {}


def engine(folders, name, dtype):
    from rvllm_b200.engine import load_model
    if (name, dtype) not in _models:
        _models[(name, dtype)] = load_model(folders[name], dtype, "cuda")[0]
    return _models[(name, dtype)]


def run_schedule(model, steps, page, slots=4, graphs=False):
    from rvllm_b200.engine import ModelRunner, make_cache
    cache = make_cache(model, page, schedules.tokens_held(steps, 64) // page, slots)
    runner = ModelRunner(model, cache, model.ops, use_graphs=graphs)
    got = schedules.replay(runner, steps)
    model.ops.check_status()
    assert not cache.requests and all(g.pool.in_use == 0 for g in cache.groups)
    return got, runner


_plain = {}


def compare(got, folders, name, reqs, dtype):
    """float32: every position within the bound.  bfloat16: a router score that is a close call
    may fall the other way after rounding and change a token's experts, which is no fault; so a
    few positions in a hundred may lie outside the bound."""
    over, total = [], 0
    for rid, ids in reqs.items():
        key = (name, tuple(ids))
        if key not in _plain:
            _plain[key] = vf.plain_logits(folders[name], name, ids)
        ref = _plain[key]
        scale = float(ref.abs().max())
        for p in range(len(ids)):
            err = float((got[(rid, p)].double() - ref[p]).abs().max()) / scale
            total += 1
            if not err < BOUND[dtype]:
                over.append((rid, p, err))
    assert len(over) <= (0 if dtype == "float32" else 0.04 * total), (len(over), total, over[:5])


def _requests(name, lengths, seed):
    rng = random.Random(seed)
    vocab = vf.config(name)["vocab"]
    return {f"q{i}": [rng.randrange(vocab) for _ in range(n)] for i, n in enumerate(lengths)}


def test_layers_one_by_one(folders):
    """The sum of the residual streams after every layer, float32, against the plain one."""
    from rvllm_b200.engine import ModelRunner, StepEntry, make_cache
    for name in ("A", "C"):
        model = engine(folders, name, "float32")
        ids = _requests(name, (45,), 1)["q0"]
        want = []
        plain.forward(vf.config(name), vf.read_tensors(folders[name]), ids, layers_out=want)
        cache = make_cache(model, 16, 8, 1)
        runner = ModelRunner(model, cache, model.ops, use_graphs=False)
        runner.add_request("a")
        seen = []

        def watched(block):
            inner = block.forward

            def forward(stream, ctx, cache):
                out = inner(stream, ctx, cache)
                # the last sub-layer's output is still pending: x_t = sum_s M[s, t] x_s + b[t] y
                mix, b = out.pending_hyper
                x = torch.einsum("st,nsw->ntw", mix.double(), out.resid.double()) + \
                    b.double()[None, :, None] * out.pending.double()[:, None, :]
                seen.append(x.sum(dim=1)[:len(ids)])
                return out
            return forward
        for b in model.blocks:
            b.forward = watched(b)
        try:
            runner.step([StepEntry("a", ids, ())])
        finally:
            for b in model.blocks:
                del b.forward
        runner.end_request("a")
        assert len(seen) == len(want)
        for i, (x, w) in enumerate(zip(seen, want)):
            close(x, w, torch.float32, scale=float(np.abs(w).max()))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_every_cut_equals_plain(folders, name, dtype):
    """Whole prompts; a prompt then its last tokens one by one (a window passes over decoded
    tokens); portions down to two tokens; mixed batches of unequal requests on four slots,
    with more requests than slots, so that pages and slots are used again."""
    model = engine(folders, name, dtype)
    reqs = _requests(name, (130, 1, 2, 67, 200, 33, 64, 65), 3)
    compare(run_schedule(model, schedules.whole(reqs), 16)[0], folders, name, reqs, dtype)
    compare(run_schedule(model, schedules.tail_decode(reqs, 90), 8)[0], folders, name, reqs, dtype)
    compare(run_schedule(model, schedules.portions(reqs), 16)[0], folders, name, reqs, dtype)
    compare(run_schedule(model, schedules.portions(reqs, (64, 2, 100, 3)), 4)[0], folders, name, reqs, dtype)
    for seed in (0, 1):
        compare(run_schedule(model, schedules.mixed(reqs, seed), 16)[0], folders, name, reqs, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "D"])
def test_replayed_steps_equal_plain(folders, name, dtype):
    """The same with captured launch sequences: single-token steps and padded mixtures are
    replayed from graphs; requests come and go, so slots and pages are used again."""
    model = engine(folders, name, dtype)
    reqs = _requests(name, (90, 5, 41, 120, 33, 70, 18), 8)
    for steps, page in ((schedules.tail_decode(reqs, 40), 16), (schedules.mixed(reqs, 2), 8),
                        (schedules.mixed(reqs, 3, max_live=3, decode_tail=20), 16)):
        got, runner = run_schedule(model, steps, page, graphs=True)
        compare(got, folders, name, reqs, dtype)
        assert runner.graph_steps > 0


def test_long_decoding(folders):
    """400 tokens one by one after a short prompt: across many pages, with every window and
    the recurrent state far past the prompt."""
    model = engine(folders, "B", "float32")
    reqs = _requests("B", (420,), 6)
    got, _ = run_schedule(model, schedules.tail_decode(reqs, 400), 16, graphs=True)
    compare(got, folders, "B", reqs, "float32")


def test_a_batch_does_not_change_a_request(folders):
    """A request beside others gives what it gives alone, in the same cut."""
    model = engine(folders, "A", "float32")
    reqs = _requests("A", (70, 31, 5), 12)
    alone, _ = run_schedule(model, schedules.whole({"q0": reqs["q0"]}), 16)
    steps = [{"step": 0, "entries": [{"id": r, "tokens": ids, "want": list(range(len(ids)))}
                                      for r, ids in reqs.items()], "end": list(reqs)}]
    together, _ = run_schedule(model, steps, 16)
    for p in range(70):
        assert float((alone[("q0", p)] - together[("q0", p)]).abs().max()) < 1e-5


def test_a_used_slot_starts_from_zero(folders):
    """A request that takes the slot and pages of one that ended sees nothing of it: the same
    request run first and run after three others gives the same logits."""
    model = engine(folders, "A", "float32")
    reqs = _requests("A", (50, 60, 70, 40), 13)
    first, _ = run_schedule(model, schedules.whole({"q3": reqs["q3"]}), 16, slots=1)
    later, _ = run_schedule(model, schedules.whole(reqs), 16, slots=1)
    for p in range(40):
        assert float((first[("q3", p)] - later[("q3", p)]).abs().max()) < 1e-5


@pytest.mark.parametrize("name", ["A", "D"])
def test_greedy_generation_through_the_entry_point(folders, name):
    """Greedy tokens through `Generator` (scheduler, portions, preemption by a small pool) equal
    the plain implementation's argmax chain."""
    from rvllm_b200 import GenerateOptions, Generator
    rng = random.Random(9)
    vocab = vf.config(name)["vocab"]
    new = 24
    tensors = vf.read_tensors(folders[name])

    def plain_greedy(ids):
        """The argmax chain, or None when two logits on the way are too close to call."""
        ids = list(ids)
        for _ in range(new):
            row = vf.plain_logits(folders[name], name, ids, tensors=tensors)[-1]
            top = torch.topk(row, 2).values
            if float(top[0] - top[1]) < 1e-3 * float(row.abs().max()):
                return None
            ids.append(int(row.argmax()))
        return ids[-new:]

    prompts, want = [], []
    for n in (5, 37, 70):
        for attempt in range(20):
            p = [rng.randrange(vocab) for _ in range(n)]
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
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg_path = tmp_path / "config.json"
    cfg_path.write_text(json.dumps(vf.config("B")))
    folder = str(tmp_path / "model")
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "rvllm"), "random-model",
                        "--config", str(cfg_path), "--seed", "5", "--out", folder],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    tensors = vf.read_tensors(folder)
    prompt = [3, 1, 4, 1, 5, 9, 2, 6]
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "rvllm"), "cli", "--model", folder,
                        "--dtype", "float32", "--token-ids", "--prompt", " ".join(map(str, prompt)),
                        "--max-tokens", "5", "--block-size", "8"],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    got = [int(t) for t in r.stdout.strip().splitlines()[0].split()]
    ids = list(prompt)
    for tok in got:                           # each token is the plain argmax at its place
        row = vf.plain_logits(folder, "B", ids, tensors=tensors)[-1]
        assert float(row.max() - row[tok]) < 1e-3 * float(row.abs().max())
        ids.append(tok)
    assert len(got) == 5
    reqs = _requests("B", (70, 33, 90, 41, 12), 4)
    steps = schedules.mixed(reqs, seed=2)
    vocab = vf.config("B")["vocab"]
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
            ref = vf.plain_logits(folder, "B", ids, tensors=tensors)
            for p in range(len(ids)):
                err = float((got[(rid, p)].double() - ref[p]).abs().max() / ref.abs().max())
                total += 1
                over += not err < BOUND[dtype]
        assert over <= (0 if dtype == "float32" else 0.04 * total), (dtype, over, total)
