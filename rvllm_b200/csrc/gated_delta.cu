// The gated delta rule with one decay per key channel, over any mixture of prompt portions and
// single tokens.  Per request a float32 record holds the last taps-1 inputs of the short
// convolutions, [taps-1, C] oldest first with C = 2 G d + H dv channels (q | k | v), and then
// the state S [H, d, dv].  G key heads of size d, H value heads of size dv; value head h reads
// key head h / (H / G).
//
//   gdr_prepare  (one block per token)
//     proj [N, P] float32: q | k | v | beta (H) | anything else; the first C columns pass a
//     causal convolution over time per channel (filter [C, taps], last column the current
//     token's; the inputs before a request's first token of the step come from its record)
//     and then silu; q and k become unit vectors per head, x / sqrt(sum x^2 + unit_eps), q also
//     times d^(-1/2); beta = sigmoid(proj beta); decay g = exp(-exp(A_log[h]) * softplus(a +
//     dt_bias)) with a = lowrank[n, h d + i].  Output prep [N, PW] float32, every part a
//     multiple of four floats so that it can be copied 16 bytes at a time:
//     q [G, dp] | k [G, dp] | g [H, dp] | v [H dv] | beta [H] | q.k [G], where dp >= d is the
//     number of state rows the scan's threads hold together; rows d .. dp-1 carry q = k = 0,
//     g = 1.
//   gdr_scan  (one block of 64 threads per (value head, group of value channels, request))
//     S <- g * S (rows);  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q.  With S' = g * S
//     the read-out is o = S'^T q + (q.k) u, so one pass over the rows gives both sums, and the
//     write k u^T is folded into the next token's pass: a token costs one walk over the state,
//     not two.  Column j of S never meets another column, so the columns of a head are spread over blocks; P threads
//     share a column and each keeps R of its rows in registers for the whole portion (P
//     neighbouring lanes, rows dealt out four at a time, sums by shuffles).  q, k and g of the
//     coming tokens (with the block's values and beta) arrive in a ring of shared-memory
//     slots by asynchronous copies, three tokens ahead, one barrier a token.  The record's
//     state is read before the first token and written after the last; o goes out as float32
//     [N, H dv].
//   gdr_finish  (one block per token, and one per request)
//     y = o / sqrt(mean_j o^2 + eps) * norm[j] * sigmoid(gate[n, h dv + j]), gate being the
//     columns lowrank[n, H d + ...]; and the request's convolution inputs move on (the last
//     taps-1 of old record | this step's rows).
// All arithmetic is float32; y is the compute type.  Plain reference: tests/plain_ops.py
// gated_delta.
#include "common.cuh"

__device__ __forceinline__ float gd_sigmoid(float x) { return 1.f / (1.f + expf(-x)); }
__device__ __forceinline__ float gd_softplus(float a) { return a > 20.f ? a : log1pf(expf(a)); }
static inline int gd_pad4(int n) { return (n + 3) & ~3; }

__global__ void gdr_prepare_kernel(const float* __restrict__ proj, int P,
                                   const float* __restrict__ lowrank, int LW,
                                   const float* __restrict__ filt, const float* __restrict__ a_log,
                                   const float* __restrict__ dt_bias,
                                   const float* __restrict__ state, long long rec,
                                   const int* __restrict__ token_req,
                                   const int* __restrict__ q_start,
                                   const int* __restrict__ state_slot, float* __restrict__ prep,
                                   int PW, int H, int G, int d, int dp, int dv, int taps,
                                   float unit_eps) {
    rv_pdl_launch_dependents();
    extern __shared__ float act[];                 // [C]
    const int n = blockIdx.x;
    const int r = token_req[n];
    const int slot = state_slot[r];
    if (slot < 0) return;
    const int t0 = q_start[r];
    const int C = 2 * G * d + H * dv;
    rv_pdl_wait();
    const float* conv_state = state + (size_t)slot * rec;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        float acc = 0.f;
        for (int j = 0; j < taps; ++j) {
            const int m = n - (taps - 1 - j);              // the token this tap reads
            const float x = m >= t0 ? proj[(size_t)m * P + c]
                                    : conv_state[(size_t)(taps - 1 + (m - t0)) * C + c];
            acc += filt[(size_t)c * taps + j] * x;
        }
        act[c] = acc * gd_sigmoid(acc);
    }
    __syncthreads();
    float* out = prep + (size_t)n * PW;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    float* kq_out = out + (2 * G + H) * dp + ((H * dv + 3) & ~3) + ((H + 3) & ~3);
    for (int head = warp; head < G; head += nwarps) {      // a query head and its key head
        const float* xq = act + head * d;
        const float* xk = act + (G + head) * d;
        float sq = 0.f, sk = 0.f;
        for (int i = lane; i < d; i += 32) {
            sq += xq[i] * xq[i];
            sk += xk[i] * xk[i];
        }
        sq = rv_warp_sum(sq);
        sk = rv_warp_sum(sk);
        const float iq = 1.f / sqrtf((float)d) / sqrtf(sq + unit_eps), ik = 1.f / sqrtf(sk + unit_eps);
        float dot = 0.f;
        for (int i = lane; i < dp; i += 32) {
            const float qv = i < d ? xq[i] * iq : 0.f, kv = i < d ? xk[i] * ik : 0.f;
            out[head * dp + i] = qv;
            out[(G + head) * dp + i] = kv;
            dot += qv * kv;
        }
        dot = rv_warp_sum(dot);
        if (lane == 0) kq_out[head] = dot;
    }
    float* gout = out + 2 * G * dp;
    for (int e = threadIdx.x; e < H * dp; e += blockDim.x) {
        const int h = e / dp, i = e - h * dp;
        float g = 1.f;
        if (i < d) {
            const float a = lowrank[(size_t)n * LW + h * d + i] + dt_bias[h * d + i];
            g = expf(-expf(a_log[h]) * gd_softplus(a));
        }
        gout[e] = g;
    }
    float* vout = gout + H * dp;
    for (int c = threadIdx.x; c < H * dv; c += blockDim.x) vout[c] = act[2 * G * d + c];
    float* bout = vout + ((H * dv + 3) & ~3);
    for (int h = threadIdx.x; h < H; h += blockDim.x)
        bout[h] = gd_sigmoid(proj[(size_t)n * P + C + h]);
}

__device__ __forceinline__ void gd_copy16(float* dst, const float* src) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(s), "l"(src) : "memory");
}
__device__ __forceinline__ void gd_copy4(float* dst, const float* src) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(s), "l"(src) : "memory");
}
__device__ __forceinline__ void gd_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void gd_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

#define GD_THREADS 64
#define GD_STAGES 4

// Row of the state that register r of the thread with number `part` among the P of a column
// holds: rows are dealt out four at a time, so that the P threads read neighbouring float4s.
template <int P>
__device__ __forceinline__ int gd_row(int r, int part) {
    return (r >> 2) * (4 * P) + part * 4 + (r & 3);
}

template <int R, int P>
__global__ void __launch_bounds__(GD_THREADS)
gdr_scan_kernel(const float* __restrict__ prep, int PW, float* __restrict__ state, long long rec,
                const int* __restrict__ q_start, const int* __restrict__ state_slot,
                float* __restrict__ o_out, int H, int G, int d, int dv, int taps, int col_blocks) {
    constexpr int COLS = GD_THREADS / P;
    constexpr int DP = R * P;
    rv_pdl_launch_dependents();
    constexpr int SLOT = 3 * DP + ((COLS + 2 + 3) & ~3);   // q | k | g [DP each] | v [COLS] | beta | q.k
    extern __shared__ __align__(16) float ring[];          // [GD_STAGES][SLOT]
    const int h = blockIdx.x / col_blocks, cb = blockIdx.x - h * col_blocks;
    const int r = blockIdx.y;
    const int slot = state_slot[r];
    const int t0 = q_start[r], qlen = q_start[r + 1] - t0;
    if (slot < 0 || qlen <= 0) return;
    const int tid = threadIdx.x;
    const int part = tid % P, col = cb * COLS + tid / P;
    const bool live = col < dv;
    const int kvh = h / (H / G);
    const int C = 2 * G * d + H * dv;
    const int v_off = (2 * G + H) * DP + h * dv + cb * COLS;
    const int b_off = (2 * G + H) * DP + ((H * dv + 3) & ~3) + h;
    const int kq_off = (2 * G + H) * DP + ((H * dv + 3) & ~3) + ((H + 3) & ~3) + kvh;
    rv_pdl_wait();

    auto fetch = [&](int t) {
        const float* row = prep + (size_t)(t0 + t) * PW;
        float* dst = ring + (size_t)(t % GD_STAGES) * SLOT;
        if (tid < COLS && cb * COLS + tid < dv) gd_copy4(dst + 3 * DP + tid, row + v_off + tid);
        if (tid == GD_THREADS - 1) gd_copy4(dst + 3 * DP + COLS, row + b_off);
        if (tid == GD_THREADS - 2) gd_copy4(dst + 3 * DP + COLS + 1, row + kq_off);
        for (int e = tid; e < 3 * DP / 4; e += GD_THREADS) {
            const int seg = e / (DP / 4), off = e - seg * (DP / 4);
            const int from = (seg == 0 ? kvh : seg == 1 ? G + kvh : 2 * G + h) * DP;
            gd_copy16(dst + seg * DP + off * 4, row + from + off * 4);
        }
    };
    for (int s = 0; s < GD_STAGES - 1; ++s) {
        if (s < qlen) fetch(s);
        gd_commit();
    }
    float* Sg = state + (size_t)slot * rec + (size_t)(taps - 1) * C + (size_t)h * d * dv;
    float S[R], kp[R];                             // state rows; the last token's key, not yet written
#pragma unroll
    for (int i = 0; i < R; ++i) {
        const int row = gd_row<P>(i, part);
        S[i] = (live && row < d) ? Sg[(size_t)row * dv + col] : 0.f;
        kp[i] = 0.f;
    }
    float up = 0.f;                                // the last token's correction
    for (int t = 0; t < qlen; ++t) {
        gd_wait<GD_STAGES - 2>();
        __syncthreads();                           // token t has arrived; slot of t-1 is free
        if (t + GD_STAGES - 1 < qlen) fetch(t + GD_STAGES - 1);
        gd_commit();
        const float* slot_t = ring + (size_t)(t % GD_STAGES) * SLOT;
        const float v = live ? slot_t[3 * DP + tid / P] : 0.f;
        const float beta = slot_t[3 * DP + COLS], kq = slot_t[3 * DP + COLS + 1];
        const float4* q4 = reinterpret_cast<const float4*>(slot_t);
        const float4* k4 = q4 + DP / 4;
        const float4* g4 = k4 + DP / 4;
        float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f, o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
        for (int i = 0; i < R / 4; ++i) {
            const float4 kk = k4[i * P + part], gg = g4[i * P + part], qq = q4[i * P + part];
            float s0 = fmaf(kp[4 * i + 0], up, S[4 * i + 0]) * gg.x;
            float s1 = fmaf(kp[4 * i + 1], up, S[4 * i + 1]) * gg.y;
            float s2 = fmaf(kp[4 * i + 2], up, S[4 * i + 2]) * gg.z;
            float s3 = fmaf(kp[4 * i + 3], up, S[4 * i + 3]) * gg.w;
            S[4 * i + 0] = s0; a0 = fmaf(s0, kk.x, a0); o0 = fmaf(s0, qq.x, o0); kp[4 * i + 0] = kk.x;
            S[4 * i + 1] = s1; a1 = fmaf(s1, kk.y, a1); o1 = fmaf(s1, qq.y, o1); kp[4 * i + 1] = kk.y;
            S[4 * i + 2] = s2; a2 = fmaf(s2, kk.z, a2); o2 = fmaf(s2, qq.z, o2); kp[4 * i + 2] = kk.z;
            S[4 * i + 3] = s3; a3 = fmaf(s3, kk.w, a3); o3 = fmaf(s3, qq.w, o3); kp[4 * i + 3] = kk.w;
        }
        float acc = (a0 + a1) + (a2 + a3), o = (o0 + o1) + (o2 + o3);
#pragma unroll
        for (int s = P / 2; s > 0; s >>= 1) {
            acc += __shfl_xor_sync(0xffffffffu, acc, s);
            o += __shfl_xor_sync(0xffffffffu, o, s);
        }
        up = beta * (v - acc);
        if (live && part == 0) o_out[(size_t)(t0 + t) * H * dv + h * dv + col] = fmaf(kq, up, o);
    }
#pragma unroll
    for (int i = 0; i < R; ++i) S[i] = fmaf(kp[i], up, S[i]);
#pragma unroll
    for (int i = 0; i < R; ++i) {
        const int row = gd_row<P>(i, part);
        if (live && row < d) Sg[(size_t)row * dv + col] = S[i];
    }
}

template <typename TO>
__global__ void gdr_finish_kernel(const float* __restrict__ o_in, const float* __restrict__ proj,
                                  int P, const float* __restrict__ lowrank, int LW,
                                  const float* __restrict__ norm_w, float* __restrict__ state,
                                  long long rec, const int* __restrict__ token_req,
                                  const int* __restrict__ q_start,
                                  const int* __restrict__ state_slot, TO* __restrict__ y,
                                  int n_tokens, int H, int G, int d, int dv, int taps, float eps) {
    rv_pdl_launch_dependents();
    const int C = 2 * G * d + H * dv;
    if ((int)blockIdx.x >= n_tokens) {
        // the convolutions' inputs move on: channel by channel, oldest first, so that what a
        // place receives is read from a later place before that one is overwritten
        const int r = blockIdx.x - n_tokens;
        const int slot = state_slot[r];
        const int t0 = q_start[r], qlen = q_start[r + 1] - t0;
        if (slot < 0 || qlen <= 0) return;
        rv_pdl_wait();
        float* record = state + (size_t)slot * rec;
        for (int c = threadIdx.x; c < C; c += blockDim.x)
            for (int i = 0; i < taps - 1; ++i) {
                const int idx = qlen - (taps - 1) + i;     // among this step's rows; negative: older
                record[(size_t)i * C + c] = idx >= 0 ? proj[(size_t)(t0 + idx) * P + c]
                                                     : record[(size_t)(taps - 1 + idx) * C + c];
            }
        return;
    }
    const int n = blockIdx.x;
    if (state_slot[token_req[n]] < 0) return;
    rv_pdl_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    for (int h = warp; h < H; h += nwarps) {
        const float* o = o_in + (size_t)n * H * dv + (size_t)h * dv;
        float ss = 0.f;
        for (int j = lane; j < dv; j += 32) ss += o[j] * o[j];
        ss = rv_warp_sum(ss);
        const float inv = 1.f / sqrtf(ss / (float)dv + eps);
        for (int j = lane; j < dv; j += 32) {
            const float gate = gd_sigmoid(lowrank[(size_t)n * LW + H * d + h * dv + j]);
            rv_store(y + (size_t)n * H * dv + h * dv + j, o[j] * inv * norm_w[j] * gate);
        }
    }
}

// Floats of one request's record.
extern "C" long long rv_gated_delta_record(int H, int G, int d, int dv, int taps) {
    return (long long)(taps - 1) * (2 * G * d + H * dv) + (long long)H * d * dv;
}

// State rows a thread keeps (R) and threads that share a column (P) for key heads of size d.
static bool gd_shape(int d, int* R, int* P) {
    static const int table[][3] = {{8, 8, 1},    {16, 8, 2},   {32, 8, 4},    {64, 16, 4},
                                   {128, 32, 4}, {256, 32, 8}, {512, 32, 16}, {1024, 32, 32}};
    for (const auto& row : table)
        if (d <= row[0]) {
            *R = row[1];
            *P = row[2];
            return true;
        }
    return false;
}

// Floats of a row of the scratch `prep`, and of the whole scratch for n tokens (prep, then
// the raw read-outs [n, H dv]).
extern "C" long long rv_gated_delta_scratch(int n_tokens, int H, int G, int d, int dv) {
    int R = 0, P = 0;
    if (!gd_shape(d, &R, &P)) return -1;
    const long long pw = (long long)(2 * G + H) * R * P + gd_pad4(H * dv) + gd_pad4(H) + gd_pad4(G);
    return (long long)n_tokens * (pw + (long long)H * dv);
}

template <int R, int P>
static void gd_launch_scan(const float* prep, int PW, float* state, long long rec, const int* q_start,
                           const int* state_slot, float* o, int n_reqs, int H, int G, int d, int dv,
                           int taps, cudaStream_t s) {
    const int cols = GD_THREADS / P;
    const int col_blocks = (dv + cols - 1) / cols;
    const size_t smem = (size_t)GD_STAGES * (3 * R * P + ((cols + 2 + 3) & ~3)) * sizeof(float);
    if (smem > 48 * 1024)
        cudaFuncSetAttribute(gdr_scan_kernel<R, P>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    rv_launch(gdr_scan_kernel<R, P>, dim3(H * col_blocks, n_reqs), dim3(GD_THREADS), smem, s, prep, PW,
              state, rec, q_start, state_slot, o, H, G, d, dv, taps, col_blocks);
}

// proj [N, P] float32 (P >= C + H); lowrank [N, LW] float32 (LW >= H d + H dv: the decays'
// pre-activations, then the output gates'); filt [C, taps]; a_log [H]; dt_bias [H d]; norm_w
// [dv]; state [slots, record]; scratch: rv_gated_delta_scratch floats; y [N, H dv].
extern "C" int rv_gated_delta(const float* proj, int P, const float* lowrank, int LW,
                              const float* filt, const float* a_log, const float* dt_bias,
                              const float* norm_w, float* state, const int* token_req,
                              const int* q_start, const int* state_slot, float* scratch, void* y,
                              int out_dtype, int n_tokens, int n_reqs, int H, int G, int d, int dv,
                              int taps, float unit_eps, float eps, void* stream) {
    if (n_tokens == 0 || n_reqs == 0) return 0;
    if (n_tokens < 0 || n_reqs < 0 || H < 1 || G < 1 || H % G || d < 1 || dv < 1 || taps < 1)
        RV_FAIL("gated_delta: bad sizes");
    const int C = 2 * G * d + H * dv;
    if (P < C + H || LW < H * d + H * dv) RV_FAIL("gated_delta: rows are too narrow");
    int R = 0, TP = 0;
    if (!gd_shape(d, &R, &TP))
        RV_FAIL("gated_delta: key heads of %d are not supported (at most 1024)", d);
    if (n_reqs > 65535) RV_FAIL("gated_delta: batch too large");
    const int dp = R * TP;
    const int PW = (2 * G + H) * dp + gd_pad4(H * dv) + gd_pad4(H) + gd_pad4(G);
    const long long rec = rv_gated_delta_record(H, G, d, dv, taps);
    const size_t smem1 = (size_t)C * sizeof(float);
    if (smem1 > 200 * 1024) RV_FAIL("gated_delta: %d channels do not fit shared memory", C);
    float* prep = scratch;
    float* o = scratch + (size_t)n_tokens * PW;
    cudaStream_t s = (cudaStream_t)stream;
    if (smem1 > 48 * 1024)
        cudaFuncSetAttribute(gdr_prepare_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem1);
    rv_launch(gdr_prepare_kernel, dim3(n_tokens), dim3(256), smem1, s, proj, P, lowrank, LW, filt, a_log,
              dt_bias, (const float*)state, rec, token_req, q_start, state_slot, prep, PW, H, G, d, dp, dv,
              taps, unit_eps);
    RV_CHECK_LAUNCH("gated_delta prepare");
#define GD_CASE(r_, p_)                                                                                \
    if (R == r_ && TP == p_)                                                                           \
        gd_launch_scan<r_, p_>(prep, PW, state, rec, q_start, state_slot, o, n_reqs, H, G, d, dv, taps, s);
    GD_CASE(8, 1) GD_CASE(8, 2) GD_CASE(8, 4) GD_CASE(16, 4) GD_CASE(32, 4) GD_CASE(32, 8) GD_CASE(32, 16)
    GD_CASE(32, 32)
#undef GD_CASE
    RV_CHECK_LAUNCH("gated_delta scan");
    RV_DISPATCH_DTYPE(out_dtype, "gated_delta", {
        rv_launch(gdr_finish_kernel<T>, dim3(n_tokens + n_reqs), dim3(128), 0, s, (const float*)o, proj, P,
                  lowrank, LW, norm_w, state, rec, token_req, q_start, state_slot, (T*)y, n_tokens, H, G, d,
                  dv, taps, eps);
    });
    RV_CHECK_LAUNCH("gated_delta finish");
    return 0;
}
