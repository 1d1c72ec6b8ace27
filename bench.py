"""Throughput of the LFM2 engine on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A step is one decode step.  The default run uses the layer sizes of LFM2-1.2B (16
layers: 10 gated short-convolution, 6 attention at [2,5,8,10,12,14]; hidden 2048; 32
query heads, 8 KV heads, head size 64; feed-forward 12288 adjusted to 8192; filter
length 3; vocabulary 65536; tied head) with random bfloat16 weights, a batch of 8 and
a context of 4,096 tokens: every request is prefilled so that after the W warm-up
steps it holds 4096 - K tokens, then K steps are timed with CUDA events and end at
4,096.  The one JSON line printed holds

  value      decoded tokens a second over the K timed steps, tokens fed back on the
             device (no host round trip inside the timed region)
  e2e        the same through the Python entry point (`Engine.step`): every step copies
             its index arrays from pinned host memory and reads the sampled ids back
  prefill    one step over a 2,048-token prompt: tokens a second, and its FLOPs / time /
             the bfloat16 peak
  roofline   the decode step's bytes (every weight once, the live requests' keys and
             values and convolution states) / its time, against the HBM peak
  points     decoded tokens a second at batch 1 and batch 64 (context 2,048 + steps), each
             with its bytes / time as a fraction of the HBM peak (`decode_b1_frac`, ...)
  workloads  two scheduler runs through `Engine.step` with requests that come and go
             (`--workloads none` leaves them out; `--only workload --workload NAME` runs one):
             350m-mixed      LFM2-350M sizes, 32 requests, prompts U[128, 2048], prompt
                             portions of 512 beside the running decodes, 256 new tokens each
             700m-staggered  LFM2-700M sizes, 64 requests arriving four steps apart, prompts
                             U[512, 8192], 512 new tokens each, a page pool of 90 % of the
                             free device memory
             each after one untimed run of the same requests: output and total tokens a
             second, steps, preemptions, the share of steps replayed from a captured graph,
             and per step the host time of `Engine.step` against the device time between
             events recorded around it (`gpu_idle_frac`: the share of the run's wall time in
             which the device waited for the host)

`--only bizenex` (not part of the default run) measures Bizenex (latent and grouped-query
attention with sinks, a mixture of experts) beside an all-attention LFM2 of equal sizes.
`--only vifanex` (not part of the default run) measures Vifanex (gated delta rule and windowed
attention in turn on several residual streams, a softmax-routed mixture with a shared expert)
beside Bizenex at equal sizes.
`--only mevuvik` (not part of the default run) measures Mevuvik (latent attention with a query
latent and a turned shared key part, and a gated grouped-query attention beside a matrix memory
with exponential gates, in turn; relu-squared dense and routed feed-forwards; a stretch of layers
run twice) beside Bizenex with as many layer runs at equal sizes.
`--only retorax` (not part of the default run) measures another design, Retorax, beside LFM2
at equal sizes (width 1024 and 2048, eight layers): a 2,048-token prompt, single tokens at
batch 8 and 64, and the device time of every kernel of a step against its roofline.

RVLLM_BENCH_PAGE sets the tokens per cache page (16; 64 measured the same).

Peaks come from MEASURED_PEAKS.json beside this file when it exists ("of measured"),
else from the fallback figures 6.65 TB/s and 1.59 PFLOP/s ("of fallback").
"""
import argparse
import json
import os
import shutil
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LFM2_1_2B = {
    "architectures": ["Lfm2ForCausalLM"],
    "num_hidden_layers": 16, "full_attn_idxs": [2, 5, 8, 10, 12, 14],
    "hidden_size": 2048, "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 64,
    "block_ff_dim": 12288, "block_auto_adjust_ff_dim": True, "block_multiple_of": 256,
    "conv_L_cache": 3, "conv_bias": False, "vocab_size": 65536, "rope_theta": 1000000.0,
    "max_position_embeddings": 4096, "norm_eps": 1e-5, "tie_embedding": True,
    "torch_dtype": "bfloat16", "bos_token_id": 1, "eos_token_id": 7,
}
# The other published sizes differ in these keys only.
SIZES = {
    "1.2b": {},
    "700m": {"hidden_size": 1536, "num_attention_heads": 24, "block_ff_dim": 10240},
    "350m": {"hidden_size": 1024, "num_attention_heads": 16, "block_ff_dim": 6656},
}
WORKLOADS = {
    "350m-mixed": {"size": "350m", "requests": 32, "prompt": (128, 2048), "new": 256,
                   "chunk": 512, "arrival_gap": 0, "pool": "fit", "positions": 4096},
    "700m-staggered": {"size": "700m", "requests": 64, "prompt": (512, 8192), "new": 512,
                       "chunk": 2048, "arrival_gap": 4, "pool": "90% of free HBM",
                       "positions": 16384},
    # not one of the two that the default run reports: the mixed workload at the headline's sizes
    "1.2b-mixed": {"size": "1.2b", "requests": 32, "prompt": (128, 2048), "new": 256,
                   "chunk": 512, "arrival_gap": 2, "pool": "fit", "positions": 4096},
}
DEFAULT_WORKLOADS = ("350m-mixed", "700m-staggered")
CONTEXT = 4096
PREFILL_TOKENS = 2048
PAGE = int(os.environ.get("RVLLM_BENCH_PAGE", "16"))      # tokens per cache page


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as f:
            m = json.load(f)
        return {"hbm_gbs": float(m["hbm_gbs"]), "bf16_tflops": float(m["bf16_tflops"]),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi samples during the timed region: SM clock and throttle reasons."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc = None
        self.path = None

    @staticmethod
    def _device_id() -> str:
        """What nvidia-smi calls the device CUDA runs on: its UUID when torch can tell it
        (CUDA_VISIBLE_DEVICES may renumber the devices), else index 0."""
        try:
            import torch
            uuid = str(torch.cuda.get_device_properties(torch.cuda.current_device()).uuid)
            return uuid if uuid.startswith("GPU-") else "GPU-" + uuid
        except Exception:
            return "0"

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", self._device_id(), f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        clocks, reasons, mx = [], set(), None
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        with open(self.path) as f:
            for line in f:
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 6:
                    continue
                try:
                    clocks.append(float(parts[0]))
                    mx = float(parts[1])
                except ValueError:
                    continue
                for name, val in zip(names, parts[2:6]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
        os.remove(self.path)
        if clocks:
            clocks.sort()
            out["sm_mhz"] = clocks[len(clocks) // 2]
            out["sm_max_mhz"] = mx
        out["reasons"] = sorted(reasons)
        return out


def model_bytes_and_flops(cfg, spec_decls):
    """Bytes of every weight a step reads once, and matrix FLOPs per token."""
    weight_bytes = 0
    matmul_params = 0
    for name, decl in spec_decls.items():
        n = 1
        for d in decl.shape:
            n *= d
        weight_bytes += n * 2
        if len(decl.shape) == 2 and "embed_tokens" not in name and "conv.conv" not in name:
            matmul_params += n
    return weight_bytes, matmul_params


def run_ours(args):
    import torch

    from rvllm_b200.config import architecture, config_from_dict
    from rvllm_b200.engine import (Engine, ModelRunner, Request, SchedulerConfig, StepEntry,
                                   graphs_default, load_model, make_cache)
    from rvllm_b200.parts.model import param_decls
    from rvllm_b200.sampling import SamplingParams
    from rvllm_b200.weights import write_random_model

    pk = peaks()
    layers_full = LFM2_1_2B["num_hidden_layers"]
    data = dict(LFM2_1_2B)
    data.update(SIZES[args.size])
    cfg = config_from_dict(data)
    K, W, B = args.steps, args.warmup, args.batch
    if K + W > CONTEXT - 64:
        raise SystemExit(f"--steps + --warmup must stay below {CONTEXT - 64}")
    tmp = tempfile.mkdtemp(prefix="rvllm_bench_")
    t0 = time.time()
    try:
        folder = write_random_model(os.path.join(tmp, "lfm2_1_2b"), cfg, seed=0)
        model, cfg = load_model(folder, "bfloat16", "cuda")
    finally:                     # gigabytes of weights: never leave them behind
        shutil.rmtree(tmp, ignore_errors=True)
    setup_s = time.time() - t0
    ops = model.ops
    spec = architecture(cfg.architecture).build_spec(cfg)
    weight_bytes, matmul_params = model_bytes_and_flops(cfg, param_decls(spec))
    n_attn = len(cfg.full_attn_idxs)
    n_conv = cfg.num_hidden_layers - n_attn
    kv_bytes_per_token = n_attn * 2 * cfg.num_key_value_heads * cfg.head_dim * 2
    conv_state_bytes = n_conv * (cfg.conv_L_cache - 1) * cfg.hidden_size * 4 * 2   # read + write
    gen = torch.Generator().manual_seed(0)

    def prompts(n, length):
        return torch.randint(0, cfg.vocab_size, (n, length), generator=gen).tolist()

    def fresh_runner(batch):
        pages = batch * (CONTEXT // PAGE)
        cache = make_cache(model, PAGE, pages, batch)
        return ModelRunner(model, cache, ops, use_graphs=graphs_default())

    def do_prefill(runner, ids_list, chunk=2048):
        for i, ids in enumerate(ids_list):
            runner.add_request(i)
            for a in range(0, len(ids), chunk):
                runner.step([StepEntry(i, ids[a:a + chunk], ())])

    def timed_decode(batch, start_ctx, steps, warmup):
        """Device-timed greedy decode: tokens fed back on the device."""
        runner = fresh_runner(batch)
        do_prefill(runner, prompts(batch, start_ctx - warmup))
        reqs = list(range(batch))
        first = [1] * batch
        out = runner.decode_greedy(reqs, first, warmup)
        first = out[-1].tolist() if warmup else first
        torch.cuda.synchronize()
        launches0 = ops.launches
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        runner.decode_greedy(reqs, first, steps)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        return batch * steps / (ms / 1e3), ms / steps, ops.launches - launches0

    if args.only == "prefill":
        return run_prefill_only(torch, fresh_runner, prompts, StepEntry)

    # ---- the headline: batch B, K steps ending at the full context ------------------
    sampler = ClockSampler()
    sampler.start()
    value, ms_per_step, launches = timed_decode(B, CONTEXT - K, K, W)
    clocks = sampler.stop()
    mean_ctx = CONTEXT - K / 2
    step_bytes = weight_bytes + B * mean_ctx * kv_bytes_per_token + B * conv_state_bytes
    achieved = step_bytes / (ms_per_step / 1e3) / 1e9

    if args.only == "breakdown":
        return run_breakdown(torch, fresh_runner, do_prefill, prompts, B, ops)

    if args.only == "decode":
        print(json.dumps({"only": "decode", "value": round(value, 1),
                          "ms_per_step": round(ms_per_step, 4), "gpu_launches": launches,
                          "roofline_gbs": round(achieved, 1), "clocks": clocks}))
        return 0

    # ---- end to end through Engine.step ------------------------------------------------
    runner = fresh_runner(B)
    sched = SchedulerConfig(block_size=PAGE, num_blocks=B * (CONTEXT // PAGE),
                            max_num_batched_tokens=8192, prefill_chunk=2048)
    engine = Engine(runner, sched, CONTEXT, lookahead=True)
    e2e_steps = min(K, 512)
    budget = e2e_steps + W + 16          # requests start decoding a few steps apart
    for i, ids in enumerate(prompts(B, CONTEXT - budget)):
        engine.add_request(Request(i, ids, budget, (), SamplingParams()))
    seqs = list(engine.scheduler.seqs.values())
    while min(len(s.generated) for s in seqs) < W:
        engine.step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    done = 0
    for _ in range(e2e_steps):
        done += len(engine.step())
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    e2e = {"value": round(done / e2e_s, 1), "unit": "tokens/s",
           "h2d_bytes_per_step": runner.builder.last_h2d_bytes, "d2h_bytes_per_step": 4 * B}
    del engine, runner

    # ---- prefill of 2,048 tokens -----------------------------------------------------
    runner = fresh_runner(1)
    ids = prompts(1, PREFILL_TOKENS)[0]
    times = []
    for it in range(5):
        runner.add_request("p")
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        runner.step([StepEntry("p", ids, (PREFILL_TOKENS - 1,))])
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
        runner.end_request("p")
    pre_ms = sorted(times[2:])[len(times[2:]) // 2]
    T = PREFILL_TOKENS
    flops = 2.0 * T * matmul_params + 2.0 * cfg.vocab_size * cfg.hidden_size \
        + n_attn * 4.0 * cfg.num_attention_heads * cfg.head_dim * T * (T + 1) / 2
    prefill = {"value": round(T / (pre_ms / 1e3), 1), "tokens": T, "ms": round(pre_ms, 3),
               "frac": round(flops / (pre_ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4)}
    del runner

    # ---- other batch sizes -------------------------------------------------------------
    points = {}
    for b in (1, 64):
        # 2,048 prompt tokens, then 8 untimed steps: the padded block-table width grows at
        # 2,049 tokens, and the graph of the new width is captured there, outside the timing
        v, ms, _ = timed_decode(b, 2048 + 8, 256, 8)
        points[f"decode_b{b}"] = round(v, 1)
        nbytes = weight_bytes + b * (2048 + 8 + 128) * kv_bytes_per_token + b * conv_state_bytes
        points[f"decode_b{b}_frac"] = round(nbytes / (ms / 1e3) / 1e9 / pk["hbm_gbs"], 4)

    del model
    workloads = {}
    if args.workloads != "none":
        import gc
        gc.collect()
        torch.cuda.empty_cache()
        for name in (DEFAULT_WORKLOADS if args.workloads == "both" else [args.workloads]):
            workloads[name] = run_workload(name)

    line = {
        "metric": f"decode tok/s at batch {B} (LFM2-{args.size.upper()} sizes, context to 4,096)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic: random weights (seed 0), "
        "uniform random token ids", "impl": "ours",
        "config": {"model": f"LFM2-{args.size.upper()} sizes", "layers": cfg.num_hidden_layers,
                   "layers_full": layers_full, "hidden": cfg.hidden_size,
                   "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "ffn": cfg.ffn_dim, "vocab": cfg.vocab_size,
                   "conv_taps": cfg.conv_L_cache, "attn_layers": n_attn,
                   "global_batch": B, "seq_len": CONTEXT, "page": PAGE,
                   "parallelism": "single GPU", "l2": "inputs larger than L2 (2.3 GB weights)",
                   "peaks": pk["source"]},
        "e2e": e2e, "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"],
                     "unit": "GB/s", "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points, "workloads": workloads, "gpu_launches": launches, "clocks": clocks,
        "setup_s": round(setup_s, 1),
    }
    print(json.dumps(line))
    return 0


def run_prefill_only(torch, fresh_runner, prompts, StepEntry):
    runner = fresh_runner(1)
    ids = prompts(1, PREFILL_TOKENS)[0]
    times = []
    for it in range(3):
        runner.add_request("p")
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        runner.step([StepEntry("p", ids, (PREFILL_TOKENS - 1,))])
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
        runner.end_request("p")
    print(json.dumps({"only": "prefill", "ms": [round(t, 3) for t in times]}))
    return 0


def run_breakdown(torch, fresh_runner, do_prefill, prompts, B, ops, ctx=3000, steps=20):
    """Per-kernel device time inside replayed decode steps (torch.profiler over `steps`
    steps at context `ctx`), the wall time of a step, and the host time of an engine step.
    With programmatic dependent launch a kernel's time includes its wait for the previous
    kernel, so the kernel times can add up to more than the wall time."""
    import collections
    import re

    from torch.profiler import ProfilerActivity, profile
    runner = fresh_runner(B)
    do_prefill(runner, prompts(B, ctx))
    reqs = list(range(B))
    runner.decode_greedy(reqs, [1] * B, 8)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    runner.decode_greedy(reqs, [1] * B, 50)
    e1.record()
    torch.cuda.synchronize()
    wall_us = e0.elapsed_time(e1) / 50 * 1e3
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        runner.decode_greedy(reqs, [1] * B, steps)
        torch.cuda.synchronize()
    agg = collections.defaultdict(lambda: [0, 0.0])
    for ev in prof.events():
        if ev.device_type == torch.autograd.DeviceType.CUDA:
            name = re.sub(r"<.*", "", ev.name).replace("void ", "")[:48]
            agg[name][0] += 1
            agg[name][1] += ev.device_time
    ops.check_status()
    kernels = {k: {"per_step": round(n / steps, 1), "us_each": round(t / n, 2),
                   "us_per_step": round(t / steps, 1)}
               for k, (n, t) in sorted(agg.items(), key=lambda x: -x[1][1])[:16]}
    print(json.dumps({"only": "breakdown", "batch": B, "context": ctx,
                      "wall_us_per_step": round(wall_us, 1), "kernels": kernels}))
    return 0


def run_kernels(args):
    """Single kernels at LFM2-1.2B sizes, timed as launches captured in one CUDA graph (no
    host gaps), over operands larger than L2.  One JSON line."""
    import math
    from types import SimpleNamespace

    import torch

    from rvllm_b200.kernels import cuda_ops
    ops = cuda_ops()
    pk = peaks()
    nh, nkv, hd, ps = args.kernel_heads, 8, 64, args.kernel_page
    out = {"only": "kernels", "peaks": pk["source"]}

    def graph_time(fns, reps=5):
        for f in fns[:2]:
            f()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for f in fns:
                f()
        g.replay()
        torch.cuda.synchronize()
        ts = []
        for _ in range(reps):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            g.replay()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) * 1e3 / len(fns))
        return sorted(ts)[len(ts) // 2]

    if args.kernel == "copy_rate":
        # the copy probe (csrc/copy_probe.cu): what one SM, a quarter of the SMs and all of
        # them can copy into shared memory, as tensor-map boxes and as contiguous bulk copies
        import ctypes
        K, iters = 2048, 512
        sms = torch.cuda.get_device_properties(0).multi_processor_count
        rows = sms * iters * 16384 // (K * 2) + 128
        w = torch.randn(rows, K, device="cuda", dtype=torch.bfloat16)      # 1.2 GB: larger than L2
        status = ops.status_word("cuda")
        for mode, name, chunk in ((0, "box", 16384), (1, "bulk", 16384), (1, "bulk32k", 32768),
                                  (1, "bulk64k", 65536)):
            for grid in (sms, sms // 4, 1):
                for stages in (3, 4, 10):
                    if stages * chunk > 200 * 1024:
                        continue

                    def call():
                        ops._check(ops.lib.rv_copy_probe(
                            ctypes.c_void_p(w.data_ptr()), ctypes.c_longlong(rows), ctypes.c_int(K),
                            ctypes.c_int(mode), ctypes.c_int(grid), ctypes.c_int(iters * 16384 // chunk),
                            ctypes.c_int(stages), ctypes.c_int(chunk), ctypes.c_void_p(status.data_ptr()),
                            ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)), "copy_probe")
                    call()
                    torch.cuda.synchronize()
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    call()
                    e1.record()
                    torch.cuda.synchronize()
                    gbs = grid * (iters * 16384 // chunk) * chunk / (e0.elapsed_time(e1) * 1e-3) / 1e9
                    out[f"copy_{name}_sms{grid}_stages{stages}"] = {
                        "GB/s": round(gbs, 1), "GB/s_per_sm": round(gbs / grid, 1)}
        ops.check_status()
        print(json.dumps(out))
        return 0
    if args.kernel in ("all", "attn_decode"):
        B, ctx = args.kernel_batch, args.kernel_ctx
        blocks = -(-ctx // ps)
        layers = max(2, min(6, (400 << 20) // (B * ctx * nkv * hd * 4)))   # distinct caches > L2
        caches = [(torch.randn(B * blocks, ps, nkv, hd, device="cuda", dtype=torch.bfloat16),
                   torch.randn(B * blocks, ps, nkv, hd, device="cuda", dtype=torch.bfloat16))
                  for _ in range(layers)]
        table = torch.randperm(B * blocks, device="cuda").to(torch.int32).view(B, blocks)
        q = torch.randn(B, (nh + 2 * nkv) * hd, device="cuda", dtype=torch.bfloat16)
        o = torch.empty(B, nh * hd, device="cuda", dtype=torch.bfloat16)
        cl = torch.full((B,), ctx, dtype=torch.int32, device="cuda")
        qs = torch.arange(B + 1, dtype=torch.int32, device="cuda")
        scale = 1 / math.sqrt(hd)
        nbytes = B * ctx * nkv * hd * 2 * 2
        for name, fn in (("mma", lambda k, v: ops.paged_attention_decode_mma(
                q, nh, nkv, hd, k, v, table, qs, cl, B, ctx, ps, scale, None, o)),
                         ("simt", lambda k, v: ops.paged_attention_decode(
                q, nh, nkv, hd, k, v, table, cl, B, ctx, ps, scale, None, o))):
            us = graph_time([(lambda k=k, v=v: fn(k, v)) for k, v in caches])
            out[f"attn_decode_{name}_b{B}_ctx{ctx}"] = {
                "us": round(us, 1), "GB/s": round(nbytes / us / 1e3, 1),
                "frac_hbm": round(nbytes / us / 1e3 / pk["hbm_gbs"], 3)}
    if args.kernel in ("all", "attn_prefill"):
        # the whole prompt in one portion, and (--kernel-ctx above the portion) its last portion:
        # the same number of query tokens at the end of a longer context
        T = args.kernel_tokens
        for C in sorted({T, max(T, args.kernel_ctx if args.kernel == "attn_prefill" else T)}):
            blocks = -(-C // ps)
            kc = torch.randn(blocks, ps, nkv, hd, device="cuda", dtype=torch.bfloat16)
            vc = torch.randn_like(kc)
            table = torch.randperm(blocks, device="cuda").to(torch.int32).view(1, blocks)
            q = torch.randn(T, (nh + 2 * nkv) * hd, device="cuda", dtype=torch.bfloat16)
            o = torch.empty(T, nh * hd, device="cuda", dtype=torch.bfloat16)
            ctx = SimpleNamespace(n_tokens=T, n_reqs=1, n_decode=0, max_ctx_len=C, max_q_len=T,
                                  q_start=torch.tensor([0, T], dtype=torch.int32, device="cuda"),
                                  ctx_lens=torch.tensor([C], dtype=torch.int32, device="cuda"),
                                  token_req=torch.zeros(T, dtype=torch.int32, device="cuda"))
            group = SimpleNamespace(block_table=table, max_blocks=blocks, page_size=ps, window=None)
            us = graph_time([lambda: ops.paged_attention(q, nh, nkv, hd, kc, vc, ctx, group,
                                                         1 / math.sqrt(hd), None, o)] * 4)
            flops = 4 * nh * hd * (T * (C - T) + T * (T + 1) / 2)
            name = f"attn_prefill_t{T}" + (f"_ctx{C}" if C != T else "")
            out[name] = {"us": round(us, 1), "TFLOP/s": round(flops / us / 1e6, 1),
                         "frac_bf16": round(flops / us / 1e6 / pk["bf16_tflops"], 3)}
    if args.kernel == "elementwise":
        # the memory-bound kernels between the products of a 2,048-token prompt portion, each on
        # buffers in rotation that together exceed the L2 (bytes = what the kernel has to move)
        T = PREFILL_TOKENS
        cfgd = dict(LFM2_1_2B)
        cfgd.update(SIZES[args.size])
        from rvllm_b200.config import config_from_dict
        mc = config_from_dict(cfgd)
        H, F, taps = mc.hidden_size, mc.ffn_dim, mc.conv_L_cache
        bf = torch.bfloat16
        n = 6
        res = {}

        def timed(name, fns, nbytes):
            us = graph_time(fns)
            res[name] = {"us": round(us, 1), "GB/s": round(nbytes / us / 1e3, 1),
                         "frac_hbm": round(nbytes / us / 1e3 / pk["hbm_gbs"], 3)}

        gu = [torch.randn(T, 2 * F, device="cuda", dtype=bf) for _ in range(n)]
        act = [torch.empty(T, F, device="cuda", dtype=bf) for _ in range(n)]
        timed("swiglu", [(lambda a=a, b=b: ops.swiglu(a, b)) for a, b in zip(gu, act)], T * F * 6)
        del gu, act
        resid = [torch.randn(T, H, device="cuda", dtype=torch.float32) for _ in range(n * 2)]
        delta = [torch.randn(T, H, device="cuda", dtype=bf) for _ in range(n * 2)]
        outs = [torch.empty(T, H, device="cuda", dtype=bf) for _ in range(n * 2)]
        wn = torch.ones(H, device="cuda", dtype=torch.float32)
        timed("add_rmsnorm", [(lambda r=r, d=d, o=o: ops.add_rmsnorm(r, d, wn, 1e-5, o))
                              for r, d, o in zip(resid, delta, outs)], T * H * 12)
        del resid, delta
        proj = [torch.randn(T, 3 * H, device="cuda", dtype=bf) for _ in range(n * 2)]
        filt = torch.randn(H, taps, device="cuda", dtype=torch.float32)
        state = torch.zeros(2, taps - 1, H, device="cuda", dtype=torch.float32)
        cctx = SimpleNamespace(n_reqs=1, max_q_len=T,
                               q_start=torch.tensor([0, T], dtype=torch.int32, device="cuda"),
                               state_slot=torch.tensor([1], dtype=torch.int32, device="cuda"),
                               start_pos=torch.tensor([0], dtype=torch.int32, device="cuda"))
        timed("short_conv", [(lambda a=a, o=o: ops.short_conv(a, filt, None, None, state, cctx, o))
                             for a, o in zip(proj, outs)], T * H * 8)
        del proj
        qkv = [torch.randn(T, (nh + 2 * nkv) * hd, device="cuda", dtype=bf) for _ in range(n * 3)]
        blocks = -(-T // ps)
        kcs = [torch.empty(blocks, ps, nkv, hd, device="cuda", dtype=bf) for _ in range(n * 3)]
        vcs = [torch.empty_like(k) for k in kcs]
        pos = torch.arange(T, dtype=torch.int32, device="cuda")
        slots = torch.randperm(blocks * ps, device="cuda").to(torch.int32)[:T].contiguous()
        qw = torch.ones(hd, device="cuda", dtype=torch.float32)
        inv = 1.0 / (1e6 ** (torch.arange(0, hd, 2, device="cuda", dtype=torch.float32) / hd))
        ang = pos.float()[:, None] * inv[None, :]
        table = (ang.cos().contiguous(), ang.sin().contiguous())
        timed("qk_norm_rope_write",
              [(lambda a=a, k=k, v=v: ops.qk_norm_rope_write(a, nh, nkv, hd, qw, qw, 1e-5, table, pos,
                                                            slots, k, v))
               for a, k, v in zip(qkv, kcs, vcs)],
              T * hd * 2 * ((nh + nkv) * 2 + nkv + 2 * nkv))
        print(json.dumps({"only": "kernels", "peaks": pk["source"], "tokens": T, **res}))
        return 0
    if args.kernel == "all" or args.kernel.startswith("gemm"):
        M = args.kernel_m
        x = torch.randn(M, 8192, device="cuda", dtype=torch.bfloat16)
        shapes = ((6144, 2048), (2048, 2048), (3072, 2048), (16384, 2048), (2048, 8192),
                  (65536, 2048))
        if ":" in args.kernel:                       # gemm:NxK, one shape (for profiling)
            shapes = (tuple(int(v) for v in args.kernel.split(":")[1].split("x")),)
        for N, K in shapes:
            copies = max(4, min(48, (300 << 20) // (N * K * 2)))
            ws = [torch.randn(N, K, device="cuda", dtype=torch.bfloat16) for _ in range(copies)]
            xs = x[:, :K].contiguous()
            t_lib = graph_time([(lambda w=w: torch.mm(xs, w.t())) for w in ws])
            t_own = graph_time([(lambda w=w: ops.linear_tcgen05(xs, w, torch.bfloat16)) for w in ws])
            out[f"gemm_m{M}_n{N}_k{K}"] = {
                "cublas_us": round(t_lib, 1), "tcgen05_us": round(t_own, 1),
                "tcgen05_GB/s": round(N * K * 2 / t_own / 1e3, 1),
                "frac_hbm": round(N * K * 2 / t_own / 1e3 / pk["hbm_gbs"], 3)}
            del ws
        ops.check_status()
    print(json.dumps(out))
    return 0


def run_workload(name, verbose=False):
    """One scheduler workload through `Engine.step`, after two untimed runs of the same
    requests (the reference's bench discards a warm-up run too, src/bin/bench.rs:215-232;
    prompts are seeded uniform random ids like its own, src/bin/bench.rs:93-109; random
    weights never produce a meaningful stop token, so none is set and every request
    generates its full length)."""
    import random

    import torch

    from rvllm_b200.config import config_from_dict
    import gc

    from rvllm_b200.engine import (Engine, ModelRunner, Request, SchedulerConfig, graphs_default,
                                   load_model, make_cache, settled_heap)
    from rvllm_b200.sampling import SamplingParams
    from rvllm_b200.weights import write_random_model

    w = WORKLOADS[name]
    data = dict(LFM2_1_2B)
    data.update(SIZES[w["size"]])
    data["max_position_embeddings"] = w["positions"]
    cfg = config_from_dict(data)
    tmp = tempfile.mkdtemp(prefix="rvllm_bench_")
    try:
        folder = write_random_model(os.path.join(tmp, "model"), cfg, seed=0)
        model, cfg = load_model(folder, "bfloat16", "cuda")
    finally:
        shutil.rmtree(tmp, ignore_errors=True)
    rng = random.Random(17)
    lengths = [rng.randint(*w["prompt"]) for _ in range(w["requests"])]
    prompts = [[rng.randrange(cfg.vocab_size) for _ in range(n)] for n in lengths]
    per_token = 2 * len(cfg.full_attn_idxs) * cfg.num_key_value_heads * cfg.head_dim * 2
    if w["pool"] == "fit":
        pages = sum(-(-(n + w["new"]) // PAGE) for n in lengths)
    else:
        torch.cuda.synchronize()
        free, _ = torch.cuda.mem_get_info()
        pages = int(0.9 * free) // (per_token * PAGE)
    cache = make_cache(model, PAGE, pages, w["requests"])
    runner = ModelRunner(model, cache, model.ops, use_graphs=graphs_default())
    sched = SchedulerConfig(block_size=PAGE, num_blocks=pages,
                            max_num_batched_tokens=w["chunk"] + w["requests"],
                            prefill_chunk=w["chunk"])

    def one_run(timed):
        engine = Engine(runner, sched, cfg.max_position_embeddings, lookahead=True)
        for i, ids in enumerate(prompts):
            engine.add_request(Request(i, ids, w["new"], (), SamplingParams(),
                                       arrival_step=i * w["arrival_gap"]))
        steps0, graph0 = runner.steps, runner.graph_steps
        captures0 = runner.captures
        marks, host = [], []
        out_tokens = 0
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        while engine.has_work():
            a = torch.cuda.Event(enable_timing=True)
            b = torch.cuda.Event(enable_timing=True)
            a.record()
            h0 = time.perf_counter()
            out_tokens += len(engine.step())
            host.append(time.perf_counter() - h0)
            b.record()
            marks.append((a, b))
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        model.ops.check_status()
        if not timed:
            return None
        device = [a.elapsed_time(b) for a, b in marks]
        if os.environ.get("RVLLM_BENCH_STEPS"):              # the slowest steps, for a look
            worst = sorted(range(len(device)), key=lambda i: -host[i])[:12]
            print("slowest steps (index, host ms, device ms):",
                  [(i, round(1e3 * host[i], 2), round(device[i], 2)) for i in sorted(worst)],
                  file=sys.stderr)
        st = engine.scheduler.stats
        n_steps = runner.steps - steps0
        busy = sum(device) / 1e3
        return {
            "model": f"LFM2-{w['size'].upper()} sizes", "requests": w["requests"],
            "prompt_tokens": sum(lengths), "new_tokens": out_tokens,
            "pool_pages": pages, "pool": w["pool"],
            "wall_s": round(wall, 3),
            "output_tok_s": round(out_tokens / wall, 1),
            "total_tok_s": round((sum(lengths) + out_tokens) / wall, 1),
            "steps": n_steps, "preemptions": st.preemptions,
            "graph_step_share": round((runner.graph_steps - graph0) / max(1, n_steps), 3),
            "host_ms_per_step": round(1e3 * sum(host) / len(host), 3),
            "device_ms_per_step": round(sum(device) / len(device), 3),
            "gpu_idle_frac": round(max(0.0, 1.0 - busy / wall), 3),
            "graphs_captured_meanwhile": runner.captures - captures0,
        }

    # two untimed runs: sizes that come once per run are met in the first and captured in the
    # second, so that the timed run, like steady traffic, replays (a capture costs 4 - 5 ms and
    # now and then 30 - 130 ms on this shared machine)
    one_run(False)
    one_run(False)
    # what earlier parts of the benchmark left on the Python heap is not walked again by the
    # garbage collector during the timed run, as in `rvllm_b200.engine.run`
    with settled_heap():
        result = one_run(True)
    del runner, cache, model
    gc.collect()
    torch.cuda.empty_cache()
    return result


def run_further(args):
    """Speed at further sizes, one JSON line: decode at batch 8 with 16,384 and 32,768 tokens of
    context, a prompt of 8,192 tokens taken in portions of 2,048 (convolution state and attention
    across portion boundaries at the real widths), and the samplers over 65,536 logits."""
    import torch

    from rvllm_b200.config import architecture, config_from_dict
    from rvllm_b200.engine import ModelRunner, StepEntry, graphs_default, load_model, make_cache
    from rvllm_b200.parts.model import param_decls
    from rvllm_b200.weights import write_random_model

    pk = peaks()
    data = dict(LFM2_1_2B)
    data["max_position_embeddings"] = 32768
    cfg = config_from_dict(data)
    tmp = tempfile.mkdtemp(prefix="rvllm_bench_")
    try:
        folder = write_random_model(os.path.join(tmp, "model"), cfg, seed=0)
        model, cfg = load_model(folder, "bfloat16", "cuda")
    finally:
        shutil.rmtree(tmp, ignore_errors=True)
    ops = model.ops
    spec = architecture(cfg.architecture).build_spec(cfg)
    weight_bytes, matmul_params = model_bytes_and_flops(cfg, param_decls(spec))
    n_attn = len(cfg.full_attn_idxs)
    kv_per_token = n_attn * 2 * cfg.num_key_value_heads * cfg.head_dim * 2
    gen = torch.Generator().manual_seed(0)
    out = {"only": "further", "peaks": pk["source"]}

    def ids(n):
        return torch.randint(0, cfg.vocab_size, (n,), generator=gen).tolist()

    B, steps = 8, 128
    for ctx in (16384, 32768):
        cache = make_cache(model, PAGE, B * (ctx // PAGE), B)
        runner = ModelRunner(model, cache, ops, use_graphs=graphs_default())
        for i in range(B):
            runner.add_request(i)
            toks = ids(ctx - steps - 8)
            for a in range(0, len(toks), 2048):
                runner.step([StepEntry(i, toks[a:a + 2048], ())])
        first = runner.decode_greedy(list(range(B)), [1] * B, 8)[-1].tolist()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        runner.decode_greedy(list(range(B)), first, steps)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        nbytes = weight_bytes + B * (ctx - steps / 2) * kv_per_token
        out[f"decode_b{B}_ctx{ctx}"] = {"tok_s": round(B / (ms / 1e3), 1), "ms_per_step": round(ms, 4),
                                         "frac_hbm": round(nbytes / (ms / 1e3) / 1e9 / pk["hbm_gbs"], 4)}
        del runner, cache

    # a prompt of 8,192 tokens in portions of 2,048
    T, portion = 8192, 2048
    cache = make_cache(model, PAGE, T // PAGE, 1)
    runner = ModelRunner(model, cache, ops, use_graphs=False)
    toks = ids(T)
    times = []
    for it in range(4):
        runner.add_request("p")
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for a in range(0, T, portion):
            runner.step([StepEntry("p", toks[a:a + portion], (portion - 1,) if a + portion == T else ())])
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
        runner.end_request("p")
    ms = sorted(times[1:])[1]
    flops = 2.0 * T * matmul_params + 2.0 * cfg.vocab_size * cfg.hidden_size \
        + n_attn * 4.0 * cfg.num_attention_heads * cfg.head_dim * T * (T + 1) / 2
    out["prefill_8192_in_portions_of_2048"] = {
        "tok_s": round(T / (ms / 1e3), 1), "ms": round(ms, 3),
        "frac_bf16": round(flops / (ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4)}
    del runner, cache

    # the samplers over [rows, 65,536] float32 logits
    for rows in (8, 64):
        logits = torch.randn(rows, cfg.vocab_size, device="cuda", generator=None) * 3
        temp = torch.full((rows,), 0.8, device="cuda")
        seed = torch.arange(rows, dtype=torch.int64, device="cuda")
        counter = torch.zeros(rows, dtype=torch.int64, device="cuda")

        def timed(fn, reps=20):
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(reps):
                fn()
            e1.record()
            torch.cuda.synchronize()
            return round(e0.elapsed_time(e1) * 1e3 / reps, 1)
        entry = {"argmax_us": timed(lambda: ops.argmax(logits))}
        for top_p in (1.0, 0.9):
            tp = torch.full((rows,), top_p, device="cuda")
            entry[f"sample_top_p_{top_p}_us"] = timed(lambda: ops.sample(logits, temp, tp, seed, counter))
        entry["logits_MB"] = round(rows * cfg.vocab_size * 4 / 1e6, 1)
        out[f"sampling_rows{rows}"] = entry
    ops.check_status()
    print(json.dumps(out))
    return 0


# ---- another design beside LFM2 ---------------------------------------------------------------

RETORAX_SIZES = {
    # width, layers (recurrence and attention in turn; every second attention reads the keys
    # and values of the one before it), heads / kv heads, key = value size, chunk, ff, vocab
    "w1024": {"width": 1024, "layers": 8, "heads": 16, "kv": 4, "dim": 64, "chunk": 1024,
              "ff": 4096, "vocab": 32768},
    "w2048": {"width": 2048, "layers": 8, "heads": 32, "kv": 8, "dim": 64, "chunk": 2048,
              "ff": 8192, "vocab": 32768},
}
FP32_TFLOPS_NOMINAL = 148 * 128 * 2 * 1.965e9 / 1e12      # CUDA-core FMA rate at the top clock


def retorax_config(sz):
    layers, last_kv = [], None
    for i in range(sz["layers"]):
        mlp = {"kind": "dense", "ff": sz["ff"]}
        if i % 2 == 0:
            layers.append({"type": "mingru", "mixer": {"width": sz["width"]}, "mlp": mlp})
            continue
        mixer = {"heads": sz["heads"], "kv_heads": sz["kv"], "dim": sz["dim"], "vdim": sz["dim"],
                 "scale": sz["dim"] ** -0.5, "rot": {"dims": sz["dim"] // 2, "base": 10000.0},
                 "mask": {"size": sz["chunk"]}}
        if last_kv is not None and (i // 2) % 2 == 1:
            mixer["kv_from"] = last_kv
        else:
            last_kv = i
        layers.append({"type": "attention", "mixer": mixer, "mlp": mlp})
    return {"architecture": "Retorax", "vocab": sz["vocab"], "width": sz["width"],
            "norm": {"eps": 1e-5}, "layers": layers}


BIZENEX_SIZES = {
    # latent and grouped-query attention in turn, every second latent layer reading the one
    # before; `ff` is an expert's inner width, a token uses `top` of `experts`
    "w1024": {"width": 1024, "layers": 8, "heads": 16, "kv": 4, "dim": 64, "rank": 128,
              "experts": 16, "top": 4, "groups": (4, 2), "ff": 1024, "vocab": 32768},
    "w2048": {"width": 2048, "layers": 8, "heads": 32, "kv": 8, "dim": 64, "rank": 128,
              "experts": 16, "top": 4, "groups": (4, 2), "ff": 2048, "vocab": 32768},
}


def bizenex_config(sz):
    layers, last = [], None
    mlp = {"kind": "moe", "expert": {"ff": sz["ff"]},
           "router": {"experts": sz["experts"], "top": sz["top"],
                      "groups": {"count": sz["groups"][0], "keep": sz["groups"][1]}}}
    for i in range(sz["layers"]):
        if i % 2 == 0:
            mixer = {"heads": sz["heads"], "dim": sz["dim"], "vdim": sz["dim"],
                     "kv_rank": sz["rank"], "scale": sz["dim"] ** -0.5}
            if last is not None and (i // 2) % 2 == 1:
                mixer["kv_from"] = last
            else:
                last = i
            layers.append({"type": "latent_attention", "mixer": mixer, "mlp": mlp})
        else:
            mixer = {"heads": sz["heads"], "kv_heads": sz["kv"], "dim": sz["dim"], "vdim": sz["dim"],
                     "scale": 12.0 / sz["dim"] ** 0.5, "q_temp": {"coef": 0.4, "every": 256}}
            layers.append({"type": "attention", "mixer": mixer, "mlp": mlp})
    return {"architecture": "Bizenex", "vocab": sz["vocab"], "width": sz["width"],
            "norm": {"eps": 1e-5}, "logit_softcap": 30.0, "layers": layers}


VIFANEX_SIZES = {
    # gated delta rule and windowed grouped-query attention in turn on `streams` residual
    # streams; the first layer's feed-forward is dense (as wide as the experts a token uses),
    # the others are mixtures with a shared expert.  The fields Bizenex reads are here too, so
    # that it runs beside at equal sizes.
    "w1024": {"width": 1024, "layers": 8, "heads": 16, "kv": 4, "dim": 64, "rank": 128, "window": 1024,
              "delta_heads": 8, "delta_kv": 4, "delta_dim": 128, "low_rank": 64, "taps": 4, "streams": 4,
              "experts": 16, "top": 4, "groups": (4, 2), "ff": 1024, "vocab": 32768},
    "w2048": {"width": 2048, "layers": 8, "heads": 32, "kv": 8, "dim": 64, "rank": 128, "window": 1024,
              "delta_heads": 16, "delta_kv": 8, "delta_dim": 128, "low_rank": 64, "taps": 4, "streams": 4,
              "experts": 16, "top": 4, "groups": (4, 2), "ff": 2048, "vocab": 32768},
}


def vifanex_config(sz):
    layers = []
    moe = {"kind": "moe", "expert": {"ff": sz["ff"], "limit": 7.0},
           "router": {"experts": sz["experts"], "top": sz["top"], "scale": 1.5,
                      "groups": {"count": sz["groups"][0], "keep": sz["groups"][1]}},
           "shared": {"ff": sz["ff"], "limit": 7.0}}
    for i in range(sz["layers"]):
        mlp = {"kind": "dense", "ff": sz["top"] * sz["ff"], "limit": 7.0} if i == 0 else moe
        if i % 2 == 0:
            mixer = {"heads": sz["delta_heads"], "kv_heads": sz["delta_kv"], "dim": sz["delta_dim"],
                     "vdim": sz["delta_dim"], "conv": sz["taps"], "decay_rank": sz["low_rank"],
                     "gate_rank": sz["low_rank"]}
            layers.append({"type": "channel_delta", "mixer": mixer, "mlp": mlp})
        else:
            mixer = {"heads": sz["heads"], "kv_heads": sz["kv"], "dim": sz["dim"], "vdim": sz["dim"],
                     "scale": sz["dim"] ** -0.5, "mask": {"size": sz["window"]}, "v_mix": True,
                     "rot": {"dims": sz["dim"], "base": 10000.0,
                             "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}}
            layers.append({"type": "attention", "mixer": mixer, "mlp": mlp})
    return {"architecture": "Vifanex", "vocab": sz["vocab"], "width": sz["width"], "streams": sz["streams"],
            "norm": {"eps": 1e-6}, "embedding": {"scale": sz["width"] ** 0.5}, "logit_softcap": 30.0,
            "layers": layers}


MEVUVIK_SIZES = {
    # latent attention and (gated grouped-query attention beside a matrix memory) in turn; six
    # layers of which the middle two run twice: eight layer runs, as many as Bizenex has layers.
    # A latent row and its turned part fill a head of `rank` values, as Bizenex's latent rows do.
    # The fields Bizenex reads are here too, so that it runs beside at equal sizes.
    "w1024": {"width": 1024, "layers": 8, "heads": 16, "kv": 4, "dim": 64, "rank": 128, "rot": 16,
              "q_rank": 256, "mem_heads": 8, "mem_dim": 64, "mem_vdim": 128,
              "experts": 16, "top": 4, "groups": (4, 2), "ff": 1024, "vocab": 32768},
    "w2048": {"width": 2048, "layers": 8, "heads": 32, "kv": 8, "dim": 64, "rank": 128, "rot": 16,
              "q_rank": 512, "mem_heads": 16, "mem_dim": 64, "mem_vdim": 128,
              "experts": 16, "top": 4, "groups": (4, 2), "ff": 2048, "vocab": 32768},
}


def mevuvik_config(sz):
    moe = {"kind": "moe", "expert": {"ff": sz["ff"]},
           "router": {"experts": sz["experts"], "top": sz["top"], "scale": 2.5}}
    latent = {"heads": sz["heads"], "dim": sz["dim"], "rot_dim": sz["rot"], "vdim": sz["dim"],
              "kv_rank": sz["rank"] - sz["rot"], "q_rank": sz["q_rank"],
              "scale": (sz["dim"] + sz["rot"]) ** -0.5, "rot": {"base": 10000.0, "dims": sz["rot"]}}
    par = {"left": {"heads": sz["heads"], "kv_heads": sz["kv"], "dim": sz["dim"], "vdim": sz["dim"],
                    "scale": sz["dim"] ** -0.5},
           "right": {"heads": sz["mem_heads"], "dim": sz["mem_dim"], "vdim": sz["mem_vdim"],
                     "gate_cap": 15.0},
           "left_scale": 1.0, "right_scale": 1.0}
    layers = []
    for i in range(sz["layers"] - 2):
        mlp = {"kind": "dense", "ff": sz["top"] * sz["ff"]} if i == 0 else moe
        layers.append({"type": "latent_attention", "mixer": latent, "mlp": mlp} if i % 2 == 0 else
                      {"type": "parallel", "mixer": par, "mlp": mlp})
    return {"architecture": "Mevuvik", "vocab": sz["vocab"], "width": sz["width"],
            "norm": {"eps": 1e-5}, "residual_mult": 0.7, "logit_softcap": 25.0,
            "loop": {"start": 2, "stop": 4, "times": 2}, "layers": layers}


def lfm2_all_attention(sz):
    """LFM2 with the same width and layer count, attention in every layer with the same head
    counts and sizes, and a SwiGLU as wide as the experts a token uses together."""
    d = dict(LFM2_1_2B)
    d.update(num_hidden_layers=sz["layers"], full_attn_idxs=list(range(sz["layers"])),
             hidden_size=sz["width"], num_attention_heads=sz["heads"],
             num_key_value_heads=sz["kv"], head_dim=sz["dim"], block_ff_dim=sz["top"] * sz["ff"],
             block_auto_adjust_ff_dim=False, vocab_size=sz["vocab"], max_position_embeddings=8192)
    return d


def lfm2_like(sz):
    """LFM2 with the same width, layer count, attention places and head sizes, and a SwiGLU of
    as many parameters as the dense feed-forward (three matrices of 2/3 the inner width)."""
    d = dict(LFM2_1_2B)
    d.update(num_hidden_layers=sz["layers"], full_attn_idxs=list(range(1, sz["layers"], 2)),
             hidden_size=sz["width"], num_attention_heads=sz["heads"],
             num_key_value_heads=sz["kv"], head_dim=sz["dim"], block_ff_dim=sz["ff"],
             block_auto_adjust_ff_dim=True, block_multiple_of=256, vocab_size=sz["vocab"],
             max_position_embeddings=8192)
    return d


class OpTimer:
    """Device time of each call of the kernel set's methods, by CUDA events around the call."""
    NAMES = ("embed", "add_rmsnorm", "add_layernorm", "linear", "linear_qk_norm_rope_write",
             "qk_norm_rope_write", "rope_partial_write", "paged_attention", "paged_attention_mixed",
             "short_conv", "mingru_scan", "swiglu", "xielu", "qk_unit_write", "latent_norm_write",
             "heads_product", "sigmoid_gate", "moe_select", "moe_route", "moe_experts", "softcap",
             "hyper_norm", "qkv_full_norm_rope_write", "gated_delta", "glu_clamp", "relu2",
             "weighted_sum", "latent_prepare", "rope_heads", "head_gate", "mlstm")

    def __init__(self, torch, ops):
        self.torch, self.ops, self.events, self.saved = torch, ops, [], {}

    def __enter__(self):
        for name in self.NAMES:
            fn = getattr(self.ops, name)
            self.saved[name] = fn

            def wrapped(*a, _fn=fn, _name=name, **kw):
                e0 = self.torch.cuda.Event(enable_timing=True)
                e1 = self.torch.cuda.Event(enable_timing=True)
                e0.record()
                out = _fn(*a, **kw)
                e1.record()
                self.events.append((_name, e0, e1))
                return out
            setattr(self.ops, name, wrapped)
        return self

    def __exit__(self, *exc):
        for name in self.saved:
            delattr(self.ops, name)           # the class's method shows again
        return False

    def totals(self):
        self.torch.cuda.synchronize()
        out = {}
        for name, e0, e1 in self.events:
            t = out.setdefault(name, [0, 0.0])
            t[0] += 1
            t[1] += e0.elapsed_time(e1) * 1e3
        return {k: {"calls": v[0], "us": round(v[1], 1)} for k, v in out.items()}


def run_designs(args, which="retorax"):
    """Retorax (`--only retorax`) or Bizenex (`--only bizenex`) beside LFM2, Mevuvik (`--only mevuvik`) beside Bizenex, or Vifanex
    (`--only vifanex`) beside Bizenex, at equal sizes:
    prompt and single-token throughput, and the device time of every kernel of one prompt step
    and one single-token step with its share of the roofline.  One JSON line."""
    import torch

    from rvllm_b200.config import config_from_dict
    from rvllm_b200.engine import ModelRunner, StepEntry, graphs_default, load_model, make_cache
    from rvllm_b200.weights import write_random_model

    pk = peaks()
    out = {"only": which, "peaks": pk["source"], "fp32_tflops_nominal": round(FP32_TFLOPS_NOMINAL, 1)}
    gen = torch.Generator().manual_seed(0)
    T, CTX = 2048, 1024
    sampler = ClockSampler()
    sampler.start()
    sizes = {"retorax": RETORAX_SIZES, "bizenex": BIZENEX_SIZES, "vifanex": VIFANEX_SIZES,
             "mevuvik": MEVUVIK_SIZES}[which]
    for size_name, sz in sizes.items():
        if args.design_size not in ("all", size_name):
            continue
        entry = {}
        if which == "retorax":
            pair = (("retorax", retorax_config(sz)), ("lfm2", lfm2_like(sz)))
        elif which == "bizenex":
            pair = (("bizenex", bizenex_config(sz)), ("lfm2", lfm2_all_attention(sz)))
        elif which == "mevuvik":
            pair = (("mevuvik", mevuvik_config(sz)), ("bizenex", bizenex_config(sz)))
        else:
            pair = (("vifanex", vifanex_config(sz)), ("bizenex", bizenex_config(sz)))
        for design, data in pair:
            cfg = config_from_dict(data)
            tmp = tempfile.mkdtemp(prefix="rvllm_bench_")
            try:
                folder = write_random_model(os.path.join(tmp, "m"), cfg, seed=0)
                model, cfg = load_model(folder, "bfloat16", "cuda")
            finally:
                shutil.rmtree(tmp, ignore_errors=True)
            ops = model.ops
            vocab = model.spec.vocab_size
            res = {"weights_MB": round(sum(t.numel() * t.element_size() for t in
                                           [model.embedding] + [w for b in model.blocks for w in _block_tensors(b)]) / 1e6, 1)}

            def ids(n):
                return torch.randint(0, vocab, (n,), generator=gen).tolist()

            # a prompt of T tokens in one step
            cache = make_cache(model, PAGE, T // PAGE + 1, 1)
            runner = ModelRunner(model, cache, ops, use_graphs=False)
            toks = ids(T)
            times = []
            for it in range(5):
                runner.add_request("p")
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                runner.step([StepEntry("p", toks, (T - 1,))])
                e1.record()
                torch.cuda.synchronize()
                times.append(e0.elapsed_time(e1))
                runner.end_request("p")
            ms = sorted(times[2:])[1]
            res["prefill_2048"] = {"tok_s": round(T / (ms / 1e3), 1), "ms": round(ms, 3)}
            runner.add_request("p")
            with OpTimer(torch, ops) as timer:
                runner.step([StepEntry("p", toks, (T - 1,))])
            res["prefill_2048_kernels_us"] = timer.totals()
            runner.end_request("p")
            del runner, cache
            # single tokens at batch 8 and 64, contexts around CTX
            for b in (8, 64):
                steps, warm = 128, 8
                cache = make_cache(model, PAGE, b * ((CTX + steps + warm) // PAGE + 2), b)
                runner = ModelRunner(model, cache, ops, use_graphs=graphs_default())
                for i in range(b):
                    runner.add_request(i)
                    runner.step([StepEntry(i, ids(CTX - steps // 2), ())])
                reqs = list(range(b))
                first = runner.decode_greedy(reqs, [1] * b, warm)[-1].tolist()
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                runner.decode_greedy(reqs, first, steps)
                e1.record()
                torch.cuda.synchronize()
                ms = e0.elapsed_time(e1) / steps
                res[f"decode_b{b}"] = {"tok_s": round(b / (ms / 1e3), 1), "ms_per_step": round(ms, 4)}
                if b == 64:
                    plain = ModelRunner(model, cache, ops, use_graphs=False)
                    plain.step([StepEntry(i, (1,), ()) for i in reqs])          # shapes met once
                    with OpTimer(torch, ops) as timer:
                        plain.step([StepEntry(i, (1,), ()) for i in reqs])
                    res["decode_b64_kernels_us"] = timer.totals()
                    del plain
                del runner, cache
            ops.check_status()
            entry[design] = res
            del model
            torch.cuda.empty_cache()
        entry["rooflines"] = {"retorax": design_rooflines, "bizenex": bizenex_rooflines,
                              "vifanex": vifanex_rooflines,
                              "mevuvik": mevuvik_rooflines}[which](sz, entry, pk, T, CTX)
        out[size_name] = entry
    out["clocks"] = sampler.stop()
    print(json.dumps(out))
    return 0


def _block_tensors(block):
    for part in (block.mixer, block.feed_forward):
        for v in vars(part).values() if part is not None else ():
            if hasattr(v, "element_size") and v.dim() >= 2:
                yield v


def design_rooflines(sz, entry, pk, T, CTX):
    """Per kernel pair (the new design's kernel, LFM2's like kernel): device time of all calls in
    the prompt step, and the time the roofline allows (bytes / measured copy rate; for attention
    tensor FLOPs / measured GEMM rate, plus, for the mixed heads, 2 H^2 float32 FLOPs a score on
    the CUDA cores at their nominal rate)."""
    W, F, H, G, D = sz["width"], sz["ff"], sz["heads"], sz["kv"], sz["dim"]
    L = sz["layers"]
    hbm = pk["hbm_gbs"] * 1e3                       # bytes per microsecond
    tens = pk["bf16_tflops"] * 1e6                  # FLOPs per microsecond
    fp32 = FP32_TFLOPS_NOMINAL * 1e6
    n_attn = L // 2
    f_lfm = -(-int(2 * F / 3) // 256) * 256
    chunk = sz["chunk"]
    pairs = sum(min(p % chunk, p) + 1 for p in range(T))          # (query, key) pairs of a prompt
    pairs_full = T * (T + 1) // 2
    ideal = {
        # per call: stream read and written, the added rows read, the normalised rows written
        "add_layernorm": (2 * L + 1) * T * W * (4 + 4 + 2 + 2) / hbm,
        "add_rmsnorm": (2 * L + 1) * T * W * (4 + 4 + 2 + 2) / hbm,
        "xielu": L * T * F * 4 / hbm,
        "swiglu": L * T * f_lfm * 6 / hbm,
        "mingru_scan": (L // 2) * T * W * (12 + 2) / hbm,
        "short_conv": (L // 2) * T * W * (6 + 2) / hbm,
        "paged_attention_mixed": n_attn * (pairs * 4.0 * H * D / tens + pairs * 2.0 * H * H / fp32),
        "paged_attention": n_attn * pairs_full * 4.0 * H * D / tens,
    }
    rows = {}
    like = (("add_layernorm", "add_rmsnorm"), ("xielu", "swiglu"), ("mingru_scan", "short_conv"),
            ("paged_attention_mixed", "paged_attention"))
    for ours, theirs in like:
        a = entry["retorax"]["prefill_2048_kernels_us"].get(ours)
        b = entry["lfm2"]["prefill_2048_kernels_us"].get(theirs)
        if a and b:
            rows[ours] = {"us": a["us"], "roofline_us": round(ideal[ours], 1),
                          "times_roofline": round(a["us"] / ideal[ours], 2),
                          "like": theirs, "like_us": b["us"], "like_roofline_us": round(ideal[theirs], 1),
                          "like_times_roofline": round(b["us"] / ideal[theirs], 2)}
    return rows



def bizenex_rooflines(sz, entry, pk, T, CTX):
    """Per kernel pair (Bizenex's kernel, LFM2's like kernel): device time of all calls in the
    prompt step, and the time the roofline allows: bytes / measured copy rate for the elementwise
    kernels, tensor FLOPs / measured GEMM rate for attention and for the matrix products."""
    W, F, H, G, D, R = sz["width"], sz["ff"], sz["heads"], sz["kv"], sz["dim"], sz["rank"]
    L, E, top, V = sz["layers"], sz["experts"], sz["top"], sz["vocab"]
    hbm = pk["hbm_gbs"] * 1e3                       # bytes per microsecond
    tens = pk["bf16_tflops"] * 1e6                  # FLOPs per microsecond
    n_lat, n_att = (L + 1) // 2, L // 2
    pairs = T * (T + 1) // 2                        # (query, key) pairs of a prompt
    qkv_cols = (H + 2 * G) * D
    ideal = {
        "add_layernorm": (2 * L + 1) * T * W * (4 + 4 + 2 + 2) / hbm,
        "add_rmsnorm": (2 * L + 1) * T * W * (4 + 4 + 2 + 2) / hbm,
        # scores and values of every pair: latent heads of size R, grouped heads of size D
        "paged_attention": (n_lat * pairs * 4.0 * H * R + n_att * pairs * 4.0 * H * D) / tens,
        "paged_attention_lfm2": L * pairs * 4.0 * H * D / tens,
        # q and k read and written, k and v written to the pages
        "qk_unit_write": n_att * T * ((H + G) * D * 4 + 2 * G * D * 2) / hbm,
        "qk_norm_rope_write": L * T * ((H + G) * D * 4 + 2 * G * D * 2) / hbm,
        "latent_norm_write": (n_lat + 1) // 2 * T * R * 4 / hbm,
        "sigmoid_gate": n_lat * T * H * D * 6 / hbm,
        # the rows read, ids and weights written
        "moe_route": L * T * (W * 2 + top * 8) / hbm,
        # the experts' three matrices for `top` experts a token, against the library's products
        "moe_experts": L * T * top * 6.0 * F * W / tens,
        "linear_lfm2": (L * T * 2.0 * W * (qkv_cols + H * D + 3 * top * F) + 2.0 * W * V) / tens,
        "swiglu": L * T * top * F * 6 / hbm,
        "heads_product": n_lat * T * 2.0 * H * (D * R + R * D) / tens,
    }
    ours, theirs = entry["bizenex"]["prefill_2048_kernels_us"], entry["lfm2"]["prefill_2048_kernels_us"]
    like = (("add_layernorm", "add_rmsnorm", "add_rmsnorm"),
            ("paged_attention", "paged_attention", "paged_attention_lfm2"),
            ("qk_unit_write", "qk_norm_rope_write", "qk_norm_rope_write"),
            ("latent_norm_write", "qk_norm_rope_write", "qk_norm_rope_write"),
            ("sigmoid_gate", "swiglu", "swiglu"), ("moe_route", "swiglu", "swiglu"),
            ("moe_experts", "linear", "linear_lfm2"), ("heads_product", "linear", "linear_lfm2"))
    rows = {}
    for mine, other, other_ideal in like:
        a, b = ours.get(mine), theirs.get(other)
        if a and b:
            rows[mine] = {"us": a["us"], "roofline_us": round(ideal[mine], 1),
                          "times_roofline": round(a["us"] / ideal[mine], 2),
                          "like": other, "like_us": b["us"],
                          "like_roofline_us": round(ideal[other_ideal], 1),
                          "like_times_roofline": round(b["us"] / ideal[other_ideal], 2)}
    return rows


def vifanex_rooflines(sz, entry, pk, T, CTX):
    """Per kernel pair (Vifanex's kernel, Bizenex's like kernel): device time of all calls in the
    prompt step, and the time the roofline allows: bytes / measured copy rate for the elementwise
    kernels, tensor FLOPs / measured GEMM rate for attention and the experts' products, and for
    the delta rule's recurrence its float32 FLOPs (7 a state element a token) on the CUDA cores at
    their nominal rate.  The recurrence has no like kernel in Bizenex; it stands alone."""
    W, F, H, G, D, R = sz["width"], sz["ff"], sz["heads"], sz["kv"], sz["dim"], sz["rank"]
    L, E, top, S = sz["layers"], sz["experts"], sz["top"], sz["streams"]
    Hd, Gd, Dd, ranks, taps = sz["delta_heads"], sz["delta_kv"], sz["delta_dim"], sz["low_rank"], sz["taps"]
    hbm = pk["hbm_gbs"] * 1e3                       # bytes per microsecond
    tens = pk["bf16_tflops"] * 1e6                  # FLOPs per microsecond
    fp32 = FP32_TFLOPS_NOMINAL * 1e6
    n_delta, n_att = (L + 1) // 2, L // 2
    n_lat = (L + 1) // 2                            # Bizenex: latent layers, grouped ones n_att
    window = sz["window"]
    pairs_w = sum(min(p + 1, window) for p in range(T))
    pairs = T * (T + 1) // 2
    C = 2 * Gd * Dd + Hd * Dd
    ideal = {
        # per call: S streams read and written, the pending rows read, the normalised rows written
        "hyper_norm": 2 * L * T * W * (8 * S + 2 + 2) / hbm,
        "add_layernorm": (2 * L + 1) * T * W * (4 + 4 + 2 + 2) / hbm,
        # the float32 q|k|v rows read, q written, k and v written to the pages, the first values
        "qkv_full_norm_rope_write": n_att * T * ((H + 2 * G) * D * 4 + (H + 2 * G) * D * 2 + G * D * 4) / hbm,
        "qk_unit_write": n_att * T * ((H + G) * D * 4 + 2 * G * D * 2) / hbm,
        "paged_attention": n_att * pairs_w * 4.0 * H * D / tens,
        "paged_attention_bizenex": (n_lat * pairs * 4.0 * H * R + n_att * pairs * 4.0 * H * D) / tens,
        # gate|up rows read, the activation written: the dense layer and the shared experts
        "glu_clamp": (T * top * F * 6 + (L - 1) * T * F * 6) / hbm,
        "sigmoid_gate": n_lat * T * H * D * 6 / hbm,
        "moe_route": (L - 1) * T * (W * 2 + top * 8) / hbm,
        "moe_route_bizenex": L * T * (W * 2 + top * 8) / hbm,
        "moe_experts": (L - 1) * T * top * 6.0 * F * W / tens,
        "moe_experts_bizenex": L * T * top * 6.0 * F * W / tens,
        # the recurrence: decay, correction and read-out touch every state element of every token
        "gated_delta": n_delta * max(T * Hd * 7.0 * Dd * Dd / fp32,
                                     T * ((C + Hd) * 4 + 2 * Hd * Dd * 4 + Hd * Dd * 2) / hbm),
    }
    ours, theirs = entry["vifanex"]["prefill_2048_kernels_us"], entry["bizenex"]["prefill_2048_kernels_us"]
    like = (("hyper_norm", "add_layernorm", "add_layernorm"),
            ("qkv_full_norm_rope_write", "qk_unit_write", "qk_unit_write"),
            ("paged_attention", "paged_attention", "paged_attention_bizenex"),
            ("glu_clamp", "sigmoid_gate", "sigmoid_gate"),
            ("moe_route", "moe_route", "moe_route_bizenex"),
            ("moe_experts", "moe_experts", "moe_experts_bizenex"),
            ("gated_delta", None, None))
    rows = {}
    for mine, other, other_ideal in like:
        a, b = ours.get(mine), theirs.get(other) if other else None
        if not a:
            continue
        rows[mine] = {"us": a["us"], "roofline_us": round(ideal[mine], 1),
                      "times_roofline": round(a["us"] / ideal[mine], 2)}
        if b:
            rows[mine].update({"like": other, "like_us": b["us"],
                               "like_roofline_us": round(ideal[other_ideal], 1),
                               "like_times_roofline": round(b["us"] / ideal[other_ideal], 2)})
    # single tokens at batch 64: the state of every request is read and written once a layer
    dec = entry["vifanex"].get("decode_b64_kernels_us", {}).get("gated_delta")
    if dec:
        state_bytes = n_delta * 64 * 2.0 * Hd * Dd * Dd * 4
        rows["gated_delta_decode_b64"] = {"us": dec["us"], "roofline_us": round(state_bytes / hbm, 1),
                                          "times_roofline": round(dec["us"] / (state_bytes / hbm), 2)}
    return rows


def mevuvik_rooflines(sz, entry, pk, T, CTX):
    """Per kernel pair (Mevuvik's kernel, Bizenex's like kernel): device time of all calls in the
    prompt step, and the time the roofline allows: bytes / measured copy rate for the elementwise
    kernels, tensor FLOPs / measured GEMM rate for attention and the experts' products, and for
    the matrix memory its float32 FLOPs (5 a state element a token: the decay, the write, the
    read-out) on the CUDA cores at their nominal rate.  The memory has no like kernel in Bizenex."""
    W, F, H, G, D, R = sz["width"], sz["ff"], sz["heads"], sz["kv"], sz["dim"], sz["rank"]
    E, top, rot, Rq = sz["experts"], sz["top"], sz["rot"], sz["q_rank"]
    Hm, Dm, Vm = sz["mem_heads"], sz["mem_dim"], sz["mem_vdim"]
    runs = sz["layers"]                              # layer runs of both designs
    n_lat = n_par = runs // 2                        # Mevuvik: latent runs and parallel runs
    n_moe = runs - 1                                 # its first feed-forward is dense
    hbm = pk["hbm_gbs"] * 1e3                        # bytes per microsecond
    tens = pk["bf16_tflops"] * 1e6                   # FLOPs per microsecond
    fp32 = FP32_TFLOPS_NOMINAL * 1e6
    pairs = T * (T + 1) // 2
    mem_cols = 2 * Hm * Dm + 2 * Hm * Vm + 2 * Hm    # q, k, v, two gates, the output gate
    ideal = {
        # the stream read and written, the pending rows and the scale read, the normed rows written
        "add_rmsnorm": (2 * runs + 2) * T * W * (4 + 4 + 2 + 2) / hbm,
        "add_layernorm": (2 * runs + 1) * T * W * (4 + 4 + 2 + 2) / hbm,
        # both latents read, the query latent and the page slot written
        "latent_prepare": n_lat * T * (Rq + R) * 4 / hbm,
        "latent_norm_write": ((runs + 1) // 2 + 1) // 2 * T * R * 4 / hbm,
        "rope_heads": n_lat * T * H * rot * 4 / hbm,
        "paged_attention": (n_lat * pairs * 4.0 * H * R + n_par * pairs * 4.0 * H * D) / tens,
        "paged_attention_bizenex": ((runs + 1) // 2 * pairs * 4.0 * H * R + runs // 2 * pairs * 4.0 * H * D) / tens,
        "qk_unit_write": n_par * T * ((H + 2 * G) * D * 2 + 2 * G * D * 2) / hbm,
        "qk_unit_write_bizenex": runs // 2 * T * ((H + G) * D * 4 + 2 * G * D * 2) / hbm,
        "head_gate": n_par * T * H * D * 4 / hbm,
        "weighted_sum": n_par * T * W * 6 / hbm,
        "sigmoid_gate": (runs + 1) // 2 * T * H * D * 6 / hbm,
        "relu2": T * top * F * 4 / hbm,
        "moe_route": n_moe * T * (W * 2 + top * 8) / hbm,
        "moe_route_bizenex": runs * T * (W * 2 + top * 8) / hbm,
        "moe_experts": n_moe * T * top * 4.0 * F * W / tens,
        "moe_experts_bizenex": runs * T * top * 6.0 * F * W / tens,
        "mlstm": n_par * max(T * Hm * 5.0 * Dm * (Vm + 1) / fp32,
                             T * (mem_cols * 4 + Hm * Vm * 2) / hbm),
    }
    ours, theirs = entry["mevuvik"]["prefill_2048_kernels_us"], entry["bizenex"]["prefill_2048_kernels_us"]
    like = (("add_rmsnorm", "add_layernorm", "add_layernorm"),
            ("latent_prepare", "latent_norm_write", "latent_norm_write"),
            ("rope_heads", "latent_norm_write", "latent_norm_write"),
            ("paged_attention", "paged_attention", "paged_attention_bizenex"),
            ("qk_unit_write", "qk_unit_write", "qk_unit_write_bizenex"),
            ("head_gate", "sigmoid_gate", "sigmoid_gate"),
            ("weighted_sum", "sigmoid_gate", "sigmoid_gate"),
            ("relu2", "sigmoid_gate", "sigmoid_gate"),
            ("moe_route", "moe_route", "moe_route_bizenex"),
            ("moe_experts", "moe_experts", "moe_experts_bizenex"),
            ("mlstm", None, None))
    rows = {}
    for mine, other, other_ideal in like:
        a, b = ours.get(mine), theirs.get(other) if other else None
        if not a:
            continue
        rows[mine] = {"us": a["us"], "calls": a["calls"], "roofline_us": round(ideal[mine], 1),
                      "times_roofline": round(a["us"] / ideal[mine], 2)}
        if b:
            rows[mine].update({"like": other, "like_us": b["us"],
                               "like_roofline_us": round(ideal[other_ideal], 1),
                               "like_times_roofline": round(b["us"] / ideal[other_ideal], 2)})
    # single tokens at batch 64: the state of every request is read and written once a layer run
    dec = entry["mevuvik"].get("decode_b64_kernels_us", {}).get("mlstm")
    if dec:
        state_bytes = n_par * 64 * 2.0 * Hm * Dm * (Vm + 1) * 4
        rows["mlstm_decode_b64"] = {"us": dec["us"], "roofline_us": round(state_bytes / hbm, 1),
                                    "times_roofline": round(dec["us"] / (state_bytes / hbm), 2)}
    return rows


def run_reference(args):
    print(json.dumps({
        "impl": "reference",
        "unavailable": "ermolushka/rvllm is a Rust crate (no setup.py/pyproject.toml: pip says "
                       "'not installable'); no cargo/rustc and no vendored crates offline"}))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1024)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--size", default="1.2b", choices=sorted(SIZES),
                    help="layer sizes: LFM2-1.2B (the default and the headline), 700M or 350M")
    ap.add_argument("--only", default="all", choices=["all", "decode", "prefill", "kernels", "breakdown", "workload", "further", "retorax", "bizenex", "vifanex", "mevuvik"],
                    help="run one part only (for profiling); the JSON line then lacks the rest")
    ap.add_argument("--workloads", default="both", choices=["both", "none"] + sorted(WORKLOADS),
                    help="scheduler workloads to add to the line (default: both)")
    ap.add_argument("--workload", default="350m-mixed", choices=sorted(WORKLOADS),
                    help="with --only workload: which one")
    ap.add_argument("--design-size", default="all", choices=["all"] + sorted(set(RETORAX_SIZES) | set(VIFANEX_SIZES)),
                    help="with --only retorax, bizenex, vifanex or mevuvik: which of the sizes")
    ap.add_argument("--kernel", default="all",
                    help="with --only kernels: attn_decode, attn_prefill, gemm, gemm:NxK, elementwise, copy_rate or all")
    ap.add_argument("--kernel-batch", type=int, default=64)
    ap.add_argument("--kernel-m", type=int, default=8, help="tokens of the gemm micro-benchmark")
    ap.add_argument("--kernel-ctx", type=int, default=4096)
    ap.add_argument("--kernel-tokens", type=int, default=PREFILL_TOKENS,
                    help="query tokens of the prefill attention micro-benchmark")
    ap.add_argument("--kernel-heads", type=int, default=32,
                    help="query heads of the attention micro-benchmarks (8 key/value heads)")
    ap.add_argument("--kernel-page", type=int, default=PAGE, help="page size of the attention micro-benchmarks")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    if args.only == "kernels":
        return run_kernels(args)
    if args.only == "further":
        return run_further(args)
    if args.only == "retorax":
        return run_designs(args)
    if args.only == "bizenex":
        return run_designs(args, "bizenex")
    if args.only == "vifanex":
        return run_designs(args, "vifanex")
    if args.only == "mevuvik":
        return run_designs(args, "mevuvik")
    if args.only == "workload":
        print(json.dumps({"only": "workload", args.workload: run_workload(args.workload)}))
        return 0
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
