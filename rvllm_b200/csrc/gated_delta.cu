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
//     dt_bias)) with a = lowrank[n, h d + i].  Output prep [N, 2 G d + H dv + H + H d] float32:
//     q | k | v | beta | g.
//   gdr_scan  (one block per (value head, request), one thread per value channel j)
//     S <- g * S (rows);  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q;  then
//     y = o / sqrt(mean_j o^2 + eps) * norm[j] * sigmoid(gate[n, h dv + j]), gate being the
//     columns lowrank[n, H d + ...].  Column j of S never meets another column, so a thread
//     keeps its column (in shared memory, [d][dv]) for the whole portion; the record is read
//     before the first token and written after the last.  The blocks of a request also move
//     its convolution inputs on (the last taps-1 of old record | this step's rows).
// All arithmetic is float32; y is the compute type.  Plain reference: tests/plain_ops.py
// gated_delta.
#include "common.cuh"

__device__ __forceinline__ float gd_sigmoid(float x) { return 1.f / (1.f + expf(-x)); }
__device__ __forceinline__ float gd_softplus(float a) { return a > 20.f ? a : log1pf(expf(a)); }

__global__ void gdr_prepare_kernel(const float* __restrict__ proj, int P,
                                   const float* __restrict__ lowrank, int LW,
                                   const float* __restrict__ filt, const float* __restrict__ a_log,
                                   const float* __restrict__ dt_bias,
                                   const float* __restrict__ state, long long rec,
                                   const int* __restrict__ token_req,
                                   const int* __restrict__ q_start,
                                   const int* __restrict__ state_slot, float* __restrict__ prep,
                                   int H, int G, int d, int dv, int taps, float unit_eps) {
    rv_pdl_launch_dependents();
    extern __shared__ float act[];                 // [C]
    const int n = blockIdx.x;
    const int r = token_req[n];
    const int slot = state_slot[r];
    if (slot < 0) return;
    const int t0 = q_start[r];
    const int C = 2 * G * d + H * dv;
    const int PW = C + H + H * d;
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
    for (int head = warp; head < 2 * G; head += nwarps) {  // q heads, then k heads
        const float* x = act + head * d;
        float ss = 0.f;
        for (int i = lane; i < d; i += 32) ss += x[i] * x[i];
        ss = rv_warp_sum(ss);
        const float inv = (head < G ? 1.f / sqrtf((float)d) : 1.f) / sqrtf(ss + unit_eps);
        for (int i = lane; i < d; i += 32) out[head * d + i] = x[i] * inv;
    }
    for (int c = 2 * G * d + threadIdx.x; c < C; c += blockDim.x) out[c] = act[c];
    for (int h = threadIdx.x; h < H; h += blockDim.x)
        out[C + h] = gd_sigmoid(proj[(size_t)n * P + C + h]);
    for (int e = threadIdx.x; e < H * d; e += blockDim.x) {
        const float a = lowrank[(size_t)n * LW + e] + dt_bias[e];
        out[C + H + e] = expf(-expf(a_log[e / d]) * gd_softplus(a));
    }
}

template <typename TO>
__global__ void gdr_scan_kernel(const float* __restrict__ prep, const float* __restrict__ proj,
                                int P, const float* __restrict__ lowrank, int LW,
                                const float* __restrict__ norm_w, float* __restrict__ state,
                                long long rec, const int* __restrict__ q_start,
                                const int* __restrict__ state_slot, TO* __restrict__ y, int H, int G,
                                int d, int dv, int taps, float eps) {
    rv_pdl_launch_dependents();
    extern __shared__ float smem[];
    float* S = smem;                               // [d][dv]
    float* qs = S + (size_t)d * dv;                // [d]
    float* ks = qs + d;
    float* gs = ks + d;
    float* red = gs + d;                           // [33]
    const int h = blockIdx.x, r = blockIdx.y;
    const int slot = state_slot[r];
    const int t0 = q_start[r], t1 = q_start[r + 1];
    if (slot < 0 || t1 <= t0) return;
    const int j = threadIdx.x;
    const bool live = j < dv;
    const int kvh = h / (H / G);
    const int C = 2 * G * d + H * dv;
    const int PW = C + H + H * d;
    const float nw = live ? norm_w[j] : 0.f;
    rv_pdl_wait();
    float* record = state + (size_t)slot * rec;
    // the convolutions' inputs move on: channel by channel, oldest first, so that what a place
    // receives is read from a later place before that one is overwritten
    const int qlen = t1 - t0;
    for (int c = h * blockDim.x + threadIdx.x; c < C; c += H * blockDim.x)
        for (int i = 0; i < taps - 1; ++i) {
            const int idx = qlen - (taps - 1) + i;         // among this step's rows; negative: older
            record[(size_t)i * C + c] = idx >= 0 ? proj[(size_t)(t0 + idx) * P + c]
                                                 : record[(size_t)(taps - 1 + idx) * C + c];
        }
    float* Sg = record + (size_t)(taps - 1) * C + (size_t)h * d * dv;
    if (live)
        for (int i = 0; i < d; ++i) S[i * dv + j] = Sg[(size_t)i * dv + j];
    for (int t = t0; t < t1; ++t) {
        const float* row = prep + (size_t)t * PW;
        __syncthreads();
        for (int i = threadIdx.x; i < d; i += blockDim.x) {
            qs[i] = row[kvh * d + i];
            ks[i] = row[G * d + kvh * d + i];
            gs[i] = row[C + H + h * d + i];
        }
        __syncthreads();
        float o = 0.f;
        if (live) {
            const float v = row[2 * G * d + h * dv + j], beta = row[C + h];
            float acc = 0.f;
            for (int i = 0; i < d; ++i) {
                const float s = gs[i] * S[i * dv + j];
                S[i * dv + j] = s;
                acc += s * ks[i];
            }
            const float u = beta * (v - acc);
            for (int i = 0; i < d; ++i) {
                const float s = S[i * dv + j] + ks[i] * u;
                S[i * dv + j] = s;
                o += s * qs[i];
            }
        }
        const float ss = rv_block_sum(o * o, red);
        if (live) {
            const float gate = gd_sigmoid(lowrank[(size_t)t * LW + H * d + h * dv + j]);
            rv_store(y + (size_t)t * H * dv + h * dv + j, o / sqrtf(ss / (float)dv + eps) * nw * gate);
        }
    }
    if (live)
        for (int i = 0; i < d; ++i) Sg[(size_t)i * dv + j] = S[i * dv + j];
}

// Floats of one request's record.
extern "C" long long rv_gated_delta_record(int H, int G, int d, int dv, int taps) {
    return (long long)(taps - 1) * (2 * G * d + H * dv) + (long long)H * d * dv;
}

// proj [N, P] float32 (P >= C + H); lowrank [N, LW] float32 (LW >= H d + H dv: the decays'
// pre-activations, then the output gates'); filt [C, taps]; a_log [H]; dt_bias [H d]; norm_w
// [dv]; state [slots, record]; prep: scratch [N, C + H + H d] float32; y [N, H dv].
extern "C" int rv_gated_delta(const float* proj, int P, const float* lowrank, int LW,
                              const float* filt, const float* a_log, const float* dt_bias,
                              const float* norm_w, float* state, const int* token_req,
                              const int* q_start, const int* state_slot, float* prep, void* y,
                              int out_dtype, int n_tokens, int n_reqs, int H, int G, int d, int dv,
                              int taps, float unit_eps, float eps, void* stream) {
    if (n_tokens == 0 || n_reqs == 0) return 0;
    if (n_tokens < 0 || n_reqs < 0 || H < 1 || G < 1 || H % G || d < 1 || dv < 1 || taps < 1)
        RV_FAIL("gated_delta: bad sizes");
    const int C = 2 * G * d + H * dv;
    if (P < C + H || LW < H * d + H * dv) RV_FAIL("gated_delta: rows are too narrow");
    if (dv > 1024) RV_FAIL("gated_delta: value heads of %d are not supported (at most 1024)", dv);
    if (n_reqs > 65535) RV_FAIL("gated_delta: batch too large");
    const long long rec = rv_gated_delta_record(H, G, d, dv, taps);
    const size_t smem1 = (size_t)C * sizeof(float);
    const size_t smem2 = ((size_t)d * dv + 3 * d + 33) * sizeof(float);
    if (smem1 > 200 * 1024 || smem2 > 200 * 1024)
        RV_FAIL("gated_delta: a state of %d x %d does not fit shared memory", d, dv);
    cudaStream_t s = (cudaStream_t)stream;
    if (smem1 > 48 * 1024)
        cudaFuncSetAttribute(gdr_prepare_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem1);
    rv_launch(gdr_prepare_kernel, dim3(n_tokens), dim3(256), smem1, s, proj, P, lowrank, LW, filt, a_log,
              dt_bias, (const float*)state, rec, token_req, q_start, state_slot, prep, H, G, d, dv, taps,
              unit_eps);
    RV_CHECK_LAUNCH("gated_delta prepare");
    const int threads = ((dv + 31) / 32) * 32;
    RV_DISPATCH_DTYPE(out_dtype, "gated_delta", {
        if (smem2 > 48 * 1024)
            cudaFuncSetAttribute(gdr_scan_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem2);
        rv_launch(gdr_scan_kernel<T>, dim3(H, n_reqs), dim3(threads), smem2, s, (const float*)prep, proj, P,
                  lowrank, LW, norm_w, state, rec, q_start, state_slot, (T*)y, H, G, d, dv, taps, eps);
    });
    RV_CHECK_LAUNCH("gated_delta scan");
    return 0;
}
