// The matrix memory with exponential gates (mLSTM): per head a float32 matrix C [d, dv], a
// vector n [d] and a running maximum m (0 at the start) that keeps the exponentials in range.
// For a token with log input gate li and log forget gate lf:
//
//     m'  = max(lf + m, li);   a = exp(lf + m - m');   b = exp(li - m')
//     C  <- a C + b k v^T;     n <- a n + b k;          m <- m'
//     o   = C^T q / (max(|n . q|, exp(-m)) + 1e-6)
//     y   = o / sqrt(mean(o^2) + eps) * w * sigmoid(g)                      per head
//
// with li = cap tanh((i + bi) / cap), lf = logsigmoid(cap tanh((f + bf) / cap)) and q scaled
// by d^(-1/2).  Everything here is float32.  n is kept as one more column of C whose value is
// always 1, so that n . q comes out of the same pass as C^T q.
//
// rows [N, stride] float32: q [H d] | k [H d] | v [H dv] | i [H] | f [H] | g [H dv].
// A request's record [H (dv + 1) d + H]: per head the dv + 1 columns, a column's d rows side by
// side; then the H maxima.  Three launches for any mixture of portions and single tokens:
//
//   gates   block per (request, head): li and lf of all the request's tokens in parallel, the
//           maxima one after another by one thread (an add and a max a token), then a, b and
//           exp(-m) of all tokens in parallel -> gate [N, H, 4]; the record's maximum moves on.
//   scan    block per (tile of columns, head, request): P neighbouring lanes share a column and
//           each holds R of its rows in registers for the whole portion; q, k, v and the gates
//           of sixteen tokens at a time arrive in a ring of shared-memory buffers by cp.async
//           while the sixteen before them are worked on; per token every lane does R
//           multiply-adds into its rows and R into its part of the column's sum; the sums of
//           sixteen tokens are added over the P lanes together -> num [N, H, dv + 1].  A
//           column never meets another, so the columns of a head are spread over blocks, and a
//           row's sums are formed token after token in the same order however a prompt was cut.
//   finish  warp per (token, head): the division, the head's norm, weight and gate.
// Plain reference: tests/plain_ops.py mlstm.
#include "common.cuh"

#define ML_TC 16            // tokens staged at a time
#define ML_THREADS 128

__device__ __forceinline__ float ml_logsigmoid(float z) {
    return fminf(z, 0.f) - log1pf(expf(-fabsf(z)));
}

__global__ void __launch_bounds__(512) mlstm_gates_kernel(
    const float* __restrict__ rows, int stride, int i_off, int f_off, const float* __restrict__ bi,
    const float* __restrict__ bf, float cap, const int* __restrict__ q_start,
    const int* __restrict__ state_slot, float* __restrict__ state, long long rec, int m_off,
    float* __restrict__ gate, int H) {
    rv_pdl_launch_dependents();
    const int r = blockIdx.x, h = blockIdx.y;
    const int slot = state_slot[r];
    const int a0 = q_start[r], a1 = q_start[r + 1];
    const float b_i = bi[h], b_f = bf[h];
    rv_pdl_wait();
    if (slot < 0 || a1 <= a0) return;
    constexpr int CH = 1024;
    __shared__ float li[CH], lf[CH], ms[CH + 1];
    float* m_rec = state + (size_t)slot * rec + m_off + h;
    if (threadIdx.x == 0) ms[0] = *m_rec;
    for (int c0 = a0; c0 < a1; c0 += CH) {
        const int n = min(CH, a1 - c0);
        for (int t = threadIdx.x; t < n; t += blockDim.x) {
            const float* row = rows + (size_t)(c0 + t) * stride;
            li[t] = cap * tanhf((row[i_off + h] + b_i) / cap);
            lf[t] = ml_logsigmoid(cap * tanhf((row[f_off + h] + b_f) / cap));
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            // the one chain of the layer: an add and a max a token, eight tokens' gates fetched
            // before the eight links that use them
            float m = ms[0];
            int t = 0;
            for (; t + 8 <= n; t += 8) {
                float gi[8], gf[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    gi[u] = li[t + u];
                    gf[u] = lf[t + u];
                }
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    m = fmaxf(gf[u] + m, gi[u]);
                    ms[t + u + 1] = m;
                }
            }
            for (; t < n; ++t) {
                m = fmaxf(lf[t] + m, li[t]);
                ms[t + 1] = m;
            }
        }
        __syncthreads();
        for (int t = threadIdx.x; t < n; t += blockDim.x) {
            const float m_old = ms[t], m_new = ms[t + 1];
            *(float4*)(gate + ((size_t)(c0 + t) * H + h) * 4) =
                make_float4(expf(lf[t] + m_old - m_new), expf(li[t] - m_new), expf(-m_new), 0.f);
        }
        __syncthreads();
        if (threadIdx.x == 0) ms[0] = ms[n];
        __syncthreads();
    }
    if (threadIdx.x == 0) *m_rec = ms[0];
}

__device__ __forceinline__ void ml_cp4(float* smem, const float* gmem) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(
                     (unsigned)__cvta_generic_to_shared(smem)), "l"(gmem));
}
__device__ __forceinline__ void ml_cp8(float* smem, const float* gmem) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;\n" ::"r"(
                     (unsigned)__cvta_generic_to_shared(smem)), "l"(gmem));
}
__device__ __forceinline__ void ml_cp16(float* smem, const float* gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(
                     (unsigned)__cvta_generic_to_shared(smem)), "l"(gmem));
}

// P lanes a column, R rows a lane: P * R >= d.  Rows beyond d are zeros and stay zeros.
// Sixteen tokens at a time lie in one of `nb` shared-memory buffers; the chunks after them are
// requested (cp.async, 16 bytes a piece where `vec` says the rows allow it) before these are
// worked on.  Only a row's own multiply-add links one token to the next: the column sums of
// sixteen tokens are kept in registers and added over the P lanes afterwards, sixteen
// independent shuffles a round, and the query's factor d^(-1/2) multiplies the finished sum.
template <int R>
__global__ void __launch_bounds__(ML_THREADS) mlstm_scan_kernel(
    const float* __restrict__ rows, int stride, int H, int d, int dv, int P,
    const int* __restrict__ q_start, const int* __restrict__ state_slot, float* __restrict__ state,
    long long rec, const float* __restrict__ gate, float* __restrict__ num, float q_scale, int vec,
    int nb) {
    rv_pdl_launch_dependents();
    const int h = blockIdx.y, r = blockIdx.z;
    const int slot = state_slot[r];
    const int a0 = q_start[r], a1 = q_start[r + 1];
    extern __shared__ __align__(16) float sm[];
    const int DP = P * R;                        // padded rows
    const int CPB = ML_THREADS / P;              // columns a block
    const int stage = 2 * ML_TC * DP + ML_TC * CPB + 2 * ML_TC;      // a multiple of 4 floats
    const int tid = threadIdx.x;
    const int part = tid % P, cl = tid / P;
    const int col = blockIdx.x * CPB + cl;       // dv: the column of n
    const bool live = col <= dv;
    const int r0 = part * R;
    if (slot < 0 || a1 <= a0) {
        rv_pdl_wait();
        return;
    }
    if (a1 - a0 == 1) {
        // a single token: nothing is staged; every lane reads its rows of the column, its
        // stretch of k and q, and forms the same sums in the same order as below
        rv_pdl_wait();
        const float* row = rows + (size_t)a0 * stride;
        const float* gt = gate + ((size_t)a0 * H + h) * 4;
        const float a = gt[0];
        const float bv = gt[1] * ((live && col < dv) ? row[2 * H * d + h * dv + col] : 1.f);
        float* cr = state + (size_t)slot * rec + ((size_t)h * (dv + 1) + col) * d;
        const float* kr = row + H * d + h * d;
        const float* qr = row + h * d;
        float sum = 0.f;
        if (R >= 4 && (vec & 2)) {
#pragma unroll
            for (int j = 0; j + 3 < R; j += 4) {
                if (live && r0 + j < d) {
                    float4 s4 = *(const float4*)(cr + r0 + j);
                    const float4 k4 = *(const float4*)(kr + r0 + j), q4 = *(const float4*)(qr + r0 + j);
                    s4.x = fmaf(a, s4.x, bv * k4.x);
                    s4.y = fmaf(a, s4.y, bv * k4.y);
                    s4.z = fmaf(a, s4.z, bv * k4.z);
                    s4.w = fmaf(a, s4.w, bv * k4.w);
                    sum = fmaf(s4.x, q4.x, sum);
                    sum = fmaf(s4.y, q4.y, sum);
                    sum = fmaf(s4.z, q4.z, sum);
                    sum = fmaf(s4.w, q4.w, sum);
                    *(float4*)(cr + r0 + j) = s4;
                }
            }
        } else {
#pragma unroll
            for (int j = 0; j < R; ++j) {
                if (live && r0 + j < d) {
                    const float sj = fmaf(a, cr[r0 + j], bv * kr[r0 + j]);
                    sum = fmaf(sj, qr[r0 + j], sum);
                    cr[r0 + j] = sj;
                }
            }
        }
        for (int o = P >> 1; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        if (part == 0 && live) num[((size_t)a0 * H + h) * (dv + 1) + col] = sum * q_scale;
        return;
    }
    // A buffer: q [16][DP], k [16][DP], v [CPB][16], a [16], b [16].  Zeros where no copy ever
    // writes (rows beyond d, columns beyond dv); ones as the values of the column of n.
    const int sh_cpb = __ffs(CPB) - 1;           // CPB = 128 / P is a power of two
    for (int i = tid; i < nb * stage; i += ML_THREADS) {
        const int x = i % stage - 2 * ML_TC * DP;
        const bool n_col = x >= 0 && x < ML_TC * CPB && blockIdx.x * CPB + (x >> 4) == dv;
        sm[i] = n_col ? 1.f : 0.f;
    }
    // every lane's part of a column's sum: [16][CPB][P + 1].  A column's P parts lie side by
    // side; the one float between columns keeps the lanes that write and the threads that add
    // them on different banks.
    float* psum = sm + nb * stage;
    const int pitch = ML_THREADS + CPB;
    rv_pdl_wait();
    float S[R];
    float* col_rec = state + (size_t)slot * rec + ((size_t)h * (dv + 1) + col) * d;
#pragma unroll
    for (int j = 0; j < R; ++j) S[j] = (live && r0 + j < d) ? col_rec[r0 + j] : 0.f;
    const int q_off = h * d, k_off = H * d + h * d, v_off = 2 * H * d + h * dv;
    const int W = dv + 1;
    // this thread's first copy of q and k in a chunk (the same in every chunk): token and place
    const int per_row = (vec & 1) ? (d >> 2) : d;
    const int t_first = tid / per_row, x_first = tid - t_first * per_row;
    const int t_step = ML_THREADS / per_row, x_step = ML_THREADS - t_step * per_row;
    const int v_c = tid & (CPB - 1), v_t = tid >> sh_cpb;
    const bool v_real = blockIdx.x * CPB + v_c < dv;
    __syncthreads();                             // the buffers are set before any copy lands
    auto request = [&](int c0, float* buf) {
        const int n = min(ML_TC, a1 - c0);
        float* qs = buf;
        float* ks = buf + ML_TC * DP;
        float* vs = ks + ML_TC * DP;
        float* gab = vs + ML_TC * CPB;
        int t = t_first, x = x_first;
        while (t < n) {
            const float* row = rows + (size_t)(c0 + t) * stride;
            if (vec & 1) {
                ml_cp16(qs + t * DP + 4 * x, row + q_off + 4 * x);
                ml_cp16(ks + t * DP + 4 * x, row + k_off + 4 * x);
            } else {
                ml_cp4(qs + t * DP + x, row + q_off + x);
                ml_cp4(ks + t * DP + x, row + k_off + x);
            }
            x += x_step;
            t += t_step;
            if (x >= per_row) {
                x -= per_row;
                ++t;
            }
        }
        if (v_real)
            for (int tv = v_t; tv < n; tv += P)
                ml_cp4(vs + v_c * ML_TC + tv,
                       rows + (size_t)(c0 + tv) * stride + v_off + blockIdx.x * CPB + v_c);
        if (tid < 2 * n)
            ml_cp4(gab + (tid & 1) * ML_TC + (tid >> 1),
                   gate + ((size_t)(c0 + (tid >> 1)) * H + h) * 4 + (tid & 1));
        asm volatile("cp.async.commit_group;\n" ::);
    };
    // a ring of nb buffers: nb - 1 chunks are on their way while one is worked on (a chunk's
    // arithmetic is shorter than a trip to memory); a group is committed for every chunk, also an
    // empty one past the end, so that "all but the newest nb - 1" always names this chunk
    for (int i = 0; i < nb - 1; ++i) {
        if (a0 + i * ML_TC < a1) request(a0 + i * ML_TC, sm + i * stage);
        else asm volatile("cp.async.commit_group;\n" ::);
    }
    int which = 0;
    for (int c0 = a0; c0 < a1; c0 += ML_TC, which = which + 1 == nb ? 0 : which + 1) {
        const int n = min(ML_TC, a1 - c0);
        const int ahead = c0 + (nb - 1) * ML_TC;
        if (ahead < a1) request(ahead, sm + (which == 0 ? nb - 1 : which - 1) * stage);
        else asm volatile("cp.async.commit_group;\n" ::);
        if (nb == 4) asm volatile("cp.async.wait_group 3;\n" ::);
        else if (nb == 3) asm volatile("cp.async.wait_group 2;\n" ::);
        else asm volatile("cp.async.wait_group 1;\n" ::);
        __syncthreads();                         // this chunk has landed for every thread
        const float* qs = sm + which * stage;
        const float* ks = qs + ML_TC * DP;
        const float* vs = ks + ML_TC * DP + cl * ML_TC;       // this lane's column
        const float* ga = ks + ML_TC * DP + ML_TC * CPB;
        const float* gb = ga + ML_TC;
        if (n == ML_TC) {
            float a_[ML_TC], bv_[ML_TC];
#pragma unroll
            for (int g = 0; g < ML_TC / 4; ++g) {
                const float4 A = ((const float4*)ga)[g], B = ((const float4*)gb)[g],
                             V = ((const float4*)vs)[g];
                a_[4 * g] = A.x; a_[4 * g + 1] = A.y; a_[4 * g + 2] = A.z; a_[4 * g + 3] = A.w;
                bv_[4 * g] = B.x * V.x; bv_[4 * g + 1] = B.y * V.y;
                bv_[4 * g + 2] = B.z * V.z; bv_[4 * g + 3] = B.w * V.w;
            }
#pragma unroll
            for (int t = 0; t < ML_TC; ++t) {
                const float a = a_[t], bv = bv_[t];
                const float4* kq = (const float4*)(ks + t * DP + r0);
                const float4* qq = (const float4*)(qs + t * DP + r0);
                float sum = 0.f;
#pragma unroll
                for (int j = 0; j < R / 4; ++j) {
                    const float4 k4 = kq[j], q4 = qq[j];
                    S[4 * j] = fmaf(a, S[4 * j], bv * k4.x);
                    S[4 * j + 1] = fmaf(a, S[4 * j + 1], bv * k4.y);
                    S[4 * j + 2] = fmaf(a, S[4 * j + 2], bv * k4.z);
                    S[4 * j + 3] = fmaf(a, S[4 * j + 3], bv * k4.w);
                    sum = fmaf(S[4 * j], q4.x, sum);
                    sum = fmaf(S[4 * j + 1], q4.y, sum);
                    sum = fmaf(S[4 * j + 2], q4.z, sum);
                    sum = fmaf(S[4 * j + 3], q4.w, sum);
                }
                psum[t * pitch + cl * (P + 1) + part] = sum;
            }
            __syncthreads();
            // a thread adds the P parts of one (token, column) in the lanes' order and writes it
            for (int o = tid; o < ML_TC * CPB; o += ML_THREADS) {
                const int t = o >> sh_cpb, c = o & (CPB - 1);
                const int colg = blockIdx.x * CPB + c;
                if (colg <= dv) {
                    const float* pp = psum + t * pitch + c * (P + 1);
                    float sum = 0.f;
                    for (int i = 0; i < P; ++i) sum += pp[i];
                    num[((size_t)(c0 + t) * H + h) * W + colg] = sum * q_scale;
                }
            }
        } else {
            for (int t = 0; t < n; ++t) {
                const float a = ga[t], bv = gb[t] * vs[t];
                const float* kq = ks + t * DP + r0;
                const float* qq = qs + t * DP + r0;
                float sum = 0.f;
#pragma unroll
                for (int j = 0; j < R; ++j) {
                    S[j] = fmaf(a, S[j], bv * kq[j]);
                    sum = fmaf(S[j], qq[j], sum);
                }
                for (int o = P >> 1; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
                if (part == 0 && live) num[((size_t)(c0 + t) * H + h) * W + col] = sum * q_scale;
            }
        }
        __syncthreads();                         // done with this buffer before it is asked for again
    }
    if (live) {
#pragma unroll
        for (int j = 0; j < R; ++j)
            if (r0 + j < d) col_rec[r0 + j] = S[j];
    }
}

template <typename T>
__global__ void mlstm_finish_kernel(const float* __restrict__ num, const float* __restrict__ gate,
                                    const float* __restrict__ rows, int stride, int g_off,
                                    const float* __restrict__ norm_w, float eps,
                                    const int* __restrict__ token_req,
                                    const int* __restrict__ state_slot, T* __restrict__ out,
                                    int n_tokens, int H, int dv) {
    rv_pdl_launch_dependents();
    const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (warp >= (long long)n_tokens * H) return;
    const int t = (int)(warp / H), h = (int)(warp - (long long)t * H);
    const bool pad = state_slot[token_req[t]] < 0;
    rv_pdl_wait();
    T* o = out + (size_t)t * H * dv + (size_t)h * dv;
    if (pad) {
        for (int c = lane; c < dv; c += 32) rv_store(o + c, 0.f);
        return;
    }
    const float* nm = num + ((size_t)t * H + h) * (dv + 1);
    const float den = fmaxf(fabsf(nm[dv]), gate[((size_t)t * H + h) * 4 + 2]) + 1e-6f;
    float ss = 0.f;
    for (int c = lane; c < dv; c += 32) {
        const float x = nm[c] / den;
        ss += x * x;
    }
    ss = rv_warp_sum(ss);
    const float rms = sqrtf(ss / (float)dv + eps);
    const float* g = rows + (size_t)t * stride + g_off + h * dv;
    const float* w = norm_w + h * dv;
    for (int c = lane; c < dv; c += 32)
        rv_store(o + c, nm[c] / den / rms * w[c] / (1.f + expf(-g[c])));
}

// Floats of one request's record.
extern "C" long long rv_mlstm_record(int H, int d, int dv) {
    return (long long)H * (dv + 1) * d + H;
}

// Floats of scratch for n tokens: gate [n, H, 4], then num [n, H, dv + 1].
extern "C" long long rv_mlstm_scratch(int n_tokens, int H, int dv) {
    return (long long)n_tokens * H * (4 + dv + 1);
}

// Rows of a column a lane holds.  (Two rows a lane, which doubles the warps of a single prompt,
// measured slower at key size 64: 437 against 274 us for 2,048 tokens of 8 heads; what a block
// does per chunk besides its multiply-adds is what costs.)
static int ml_rows_per_lane(int d) { return d <= 64 ? 4 : d <= 256 ? 8 : 16; }

extern "C" int rv_mlstm(const float* rows, int stride, const float* bi, const float* bf,
                        const float* norm_w, float* state, const int* token_req, const int* q_start,
                        const int* state_slot, float* scratch, void* out, int out_dtype,
                        int n_tokens, int n_reqs, int H, int d, int dv, float cap, float eps,
                        void* stream) {
    if (n_tokens == 0 || n_reqs == 0) return 0;
    if (n_tokens < 0 || n_reqs < 0 || H < 1 || d < 1 || dv < 1) RV_FAIL("mlstm: bad sizes");
    if (d > 512) RV_FAIL("mlstm: key heads of %d exceed 512", d);
    if (stride < 2 * H * d + 2 * H * dv + 2 * H) RV_FAIL("mlstm: rows are too short");
    if (!(cap > 0.f)) RV_FAIL("mlstm: the gate cap must be positive");
    if (n_reqs > 65535 || H > 65535) RV_FAIL("mlstm: too many requests or heads");
    if ((uintptr_t)scratch & 15) RV_FAIL("mlstm: the scratch must be 16-byte aligned");
    cudaStream_t s = (cudaStream_t)stream;
    const long long rec = rv_mlstm_record(H, d, dv);
    const int i_off = 2 * H * d + H * dv, f_off = i_off + H, g_off = f_off + H;
    float* gate = scratch;
    float* num = scratch + (size_t)n_tokens * H * 4;
    // the gates of a long portion are formed by many threads; the chain between them is one thread's
    const int gate_threads = n_tokens / n_reqs >= 256 ? 512 : ML_THREADS;
    rv_launch(mlstm_gates_kernel, dim3(n_reqs, H), dim3(gate_threads), 0, s, rows, stride, i_off, f_off,
              bi, bf, cap, q_start, state_slot, state, rec, H * (dv + 1) * d, gate, H);
    RV_CHECK_LAUNCH("mlstm_gates");
    const int R = ml_rows_per_lane(d);
    int P = 1;
    while (P * R < d) P <<= 1;
    const int CPB = ML_THREADS / P;
    const dim3 grid((dv + 1 + CPB - 1) / CPB, H, n_reqs);
    const size_t stage_bytes = (size_t)(2 * ML_TC * P * R + ML_TC * CPB + 2 * ML_TC) * sizeof(float);
    const int nb = stage_bytes * 4 <= 64 * 1024 ? 4 : stage_bytes * 3 <= 128 * 1024 ? 3 : 2;   // ring
    const size_t smem = nb * stage_bytes + (size_t)ML_TC * (ML_THREADS + CPB) * sizeof(float);
    // 16-byte copies of q and k: every row and every head's stretch begins on a 16-byte boundary
    // (bit 0); and of a single token's rows of the state as well (bit 1)
    int vec = d % 4 == 0 && stride % 4 == 0 && ((uintptr_t)rows & 15) == 0;
    if (vec && rec % 4 == 0 && ((uintptr_t)state & 15) == 0) vec |= 2;
    const float q_scale = 1.f / sqrtf((float)d);
#define ML_SCAN(RR)                                                                               \
    {                                                                                             \
        if (smem > 48 * 1024 &&                                                                   \
            cudaFuncSetAttribute(mlstm_scan_kernel<RR>,                                           \
                                 cudaFuncAttributeMaxDynamicSharedMemorySize,                     \
                                 (int)smem) != cudaSuccess)                                       \
            RV_FAIL("mlstm: %zu bytes of shared memory are not to be had", smem);                 \
        rv_launch(mlstm_scan_kernel<RR>, grid, dim3(ML_THREADS), smem, s, rows, stride, H, d, dv, \
                  P, q_start, state_slot, state, rec, (const float*)gate, num, q_scale, vec, nb); \
    }
    if (R == 4) ML_SCAN(4)
    else if (R == 8) ML_SCAN(8)
    else ML_SCAN(16)
#undef ML_SCAN
    RV_CHECK_LAUNCH("mlstm_scan");
    const long long warps = (long long)n_tokens * H;
    const long long blocks = (warps + 3) / 4;
    if (blocks > 0x7fffffffLL) RV_FAIL("mlstm: too many tokens");
    RV_DISPATCH_DTYPE(out_dtype, "mlstm",
                      (rv_launch(mlstm_finish_kernel<T>, dim3((int)blocks), dim3(128), 0, s,
                                 (const float*)num, (const float*)gate, rows, stride, g_off, norm_w,
                                 eps, token_req, state_slot, (T*)out, n_tokens, H, dv)));
    RV_CHECK_LAUNCH("mlstm_finish");
    return 0;
}
