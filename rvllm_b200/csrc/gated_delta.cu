// The gated delta rule with one decay per key channel, over any mixture of prompt portions and
// single tokens.  Per request a float32 record holds the last taps-1 inputs of the short
// convolutions, [taps-1, C] oldest first with C = 2 G d + H dv channels (q | k | v), and then
// the state S, stored [H, dv, d]: the d rows of a column lie side by side, because a thread owns
// rows of one column.  G key heads of size d, H value heads of size dv; value head h reads key
// head h / (H / G).
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
//   gdr_scan  (one block per (value head, group of value channels, request): up to 128 working
//   threads and a warp that brings the inputs)
//     S <- g * S (rows);  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q.  Column j of S
//     never meets another column, so the columns of a head are spread over blocks; P threads
//     share a column and each keeps R of its rows in registers for the whole portion (P
//     neighbouring lanes, rows dealt out four at a time, sums by shuffles).  A token is one step
//     of a dependent chain, so R is small (8 up to key size 256): a warp issues few
//     instructions per token and a head's work is spread over many warps.
//     The rows lag two writes behind: after token t the state is Z + a u' + k_t u, with u' and u
//     the corrections of tokens t-1 and t and a = k_{t-1} * g_t.  Then Z_t = (Z + a u'') * g_t
//     needs only the correction before last, and u' enters the token's sums through
//     kk = sum_i k_{t-1}[i] g_t[i] k_t[i] and kq = sum_i k_{t-1}[i] g_t[i] q_t[i]:
//     S_t^T k_t = Z_t^T k_t + u' kk,  o = Z_t^T q_t + u' kq + u (q_t . k_t).  One pass over the
//     rows gives both sums of a token, and two tokens' passes and shuffles are independent, so
//     tokens are worked in pairs.  At a portion's end the two writes are added and the record
//     holds the state itself.
//     q, k and g of the tokens (with the block's values, beta and q.k) arrive sixteen tokens
//     at a time in one of three shared-memory buffers by asynchronous copies of the bringing
//     warp, two chunks ahead; that warp also forms kk and kq of the chunk that has arrived.
//     One barrier per sixteen tokens, none between tokens.  The record's state is read before
//     the first token and written after the last; o goes out as float32 [N, H dv].
//   gdr_single  (a step in which every request brings one token; same grid, no bringing warp)
//     the same update without the lag: every thread copies its share of the token, reads its
//     rows meanwhile, and writes them back with the write added.  Small blocks, so that many
//     fit a multiprocessor: the step is bound by reading and writing every state once.
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
    // the scan is let in only now: let in at the start, its few long-lived blocks would settle
    // several to a multiprocessor on whichever had room beside this kernel's blocks
    rv_pdl_launch_dependents();
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

#define GD_MAX_THREADS 128      // working threads of a scan block
#define GD_SINGLE_THREADS 128   // threads of a single-token block
#define GD_CHUNK 16             // tokens that arrive together
#define GD_BUFFER_FLOATS 8192   // one of the three buffers holds at most this much

// Row of the state that register r of the thread with number `part` among the P of a column
// holds: rows are dealt out four at a time, so that the P threads read neighbouring float4s.
template <int P>
__device__ __forceinline__ int gd_row(int r, int part) {
    return (r >> 2) * (4 * P) + part * 4 + (r & 3);
}

template <int R, int P>
__global__ void __launch_bounds__(GD_MAX_THREADS + 32, R <= 8 ? 4 : 1)
gdr_scan_kernel(const float* __restrict__ prep, int PW, float* __restrict__ state, long long rec,
                const int* __restrict__ q_start, const int* __restrict__ state_slot,
                float* __restrict__ o_out, int H, int G, int d, int dv, int taps, int col_blocks, int chunk) {
    constexpr int DP = R * P;
    const int workers = blockDim.x - 32, COLS = workers / P;   // the last warp only brings the inputs
    rv_pdl_launch_dependents();
    const int SLOT = 3 * DP + ((COLS + 4 + 3) & ~3);       // q | k | g [DP each] | beta | q.k | kk | kq | v [COLS]
    extern __shared__ __align__(16) float ring[];          // [3][chunk][SLOT]
    const int h = blockIdx.x / col_blocks, cb = blockIdx.x - h * col_blocks;
    const int r = blockIdx.y;
    const int slot = state_slot[r];
    const int t0 = q_start[r], qlen = q_start[r + 1] - t0;
    if (slot < 0 || qlen <= 0) return;
    const int tid = threadIdx.x;
    const bool brings = tid >= workers;
    const int part = tid % P, col = cb * COLS + tid / P;
    const bool live = !brings && col < dv;
    const int kvh = h / (H / G);
    const int C = 2 * G * d + H * dv;
    rv_pdl_wait();

    // tokens arrive a chunk at a time, in one of three buffers [chunk][SLOT]: while the others
    // work on chunk c, the bringing warp starts the copies of chunk c+2, waits for those of
    // chunk c+1 and adds that chunk's sums, all before the barrier that ends chunk c
    const int n_chunks = (qlen + chunk - 1) / chunk;
    auto start = [&](int c) {
        if (c >= n_chunks) return;
        const int lane = tid - workers;
        const int first = c * chunk, n = min(chunk, qlen - first);
        const float* rows = prep + (size_t)(t0 + first) * PW;
        float* buf = ring + (size_t)(c % 3) * chunk * SLOT;
        // q, k and g of a token: DP floats each, 16 bytes a lane, pointers that walk the tokens
#pragma unroll
        for (int seg = 0; seg < 3; ++seg) {
            const float* src = rows + (seg == 0 ? kvh : seg == 1 ? G + kvh : 2 * G + h) * DP + lane * 4;
            unsigned dst = (unsigned)__cvta_generic_to_shared(buf + seg * DP + lane * 4);
            for (int j = 0; j < n; ++j, src += PW, dst += SLOT * 4) {
#pragma unroll
                for (int off = 0; off < DP / 4; off += 32)
                    if (DP / 4 - off >= 32 || lane < DP / 4 - off)
                        asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(dst + off * 16),
                                     "l"(src + off * 4) : "memory");
            }
        }
        // beta and q.k, then the block's values: 4 bytes a lane
        const int tail = (2 * G + H) * DP;
        const int b_off = tail + ((H * dv + 3) & ~3) + h;
        const int kq_off = b_off - h + ((H + 3) & ~3) + kvh;
        for (int w = lane; w < COLS + 2; w += 32) {
            const bool value = w < COLS;
            if (value && cb * COLS + w >= dv) continue;
            const float* src = rows + (value ? tail + h * dv + cb * COLS + w : w == COLS ? b_off : kq_off);
            unsigned dst = (unsigned)__cvta_generic_to_shared(buf + 3 * DP + (value ? 4 + w : w - COLS));
            for (int j = 0; j < n; ++j, src += PW, dst += SLOT * 4)
                asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
        }
    };
    // what the last token's key, still to be written, adds to a token's two sums:
    // kk = sum_i k'[i] g[i] k[i] and kq = sum_i k'[i] g[i] q[i], k' the key before; nothing is
    // pending before a portion's first token.  Two lanes a token.
    auto sums = [&](int c) {
        if (c >= n_chunks) return;
        const int lane = tid - workers, sub = lane & 1;
        const int n = min(chunk, qlen - c * chunk);
        float* buf = ring + (size_t)(c % 3) * chunk * SLOT;
        for (int j0 = 0; j0 < n; j0 += 16) {
            const int j = j0 + (lane >> 1);
            float* cur = buf + (size_t)j * SLOT;
            float kk = 0.f, kq = 0.f;
            if (j < n && (j > 0 || c > 0)) {
                const float* before = j > 0 ? cur - SLOT
                                            : ring + ((size_t)((c - 1) % 3) * chunk + (chunk - 1)) * SLOT;
                const float4* bk = reinterpret_cast<const float4*>(before + DP);
                const float4* cq = reinterpret_cast<const float4*>(cur);
                const float4* ck = cq + DP / 4;
                const float4* cg = ck + DP / 4;
                for (int i = sub; i < DP / 4; i += 2) {
                    const float4 b = bk[i], g = cg[i], k = ck[i], q = cq[i];
                    const float w0 = b.x * g.x, w1 = b.y * g.y, w2 = b.z * g.z, w3 = b.w * g.w;
                    kk = fmaf(w0, k.x, kk); kk = fmaf(w1, k.y, kk); kk = fmaf(w2, k.z, kk); kk = fmaf(w3, k.w, kk);
                    kq = fmaf(w0, q.x, kq); kq = fmaf(w1, q.y, kq); kq = fmaf(w2, q.z, kq); kq = fmaf(w3, q.w, kq);
                }
            }
            kk += __shfl_xor_sync(0xffffffffu, kk, 1);
            kq += __shfl_xor_sync(0xffffffffu, kq, 1);
            if (j < n && sub == 0) {
                cur[3 * DP + 2] = kk;
                cur[3 * DP + 3] = kq;
            }
        }
    };
    // this column of the head's state: its d rows lie side by side in the record
    float* Sg = state + (size_t)slot * rec + (size_t)(taps - 1) * C + ((size_t)h * dv + (live ? col : 0)) * d;
    const bool wide = (d & 3) == 0 && (reinterpret_cast<size_t>(Sg) & 15) == 0;
    // The thread's rows Z of the state lack the last two tokens' writes: the state after token
    // t is Z + a u' + kp u with u', u the corrections of tokens t-1 and t, kp = k_t and
    // a = k_{t-1} * g_t.  Token t+1 needs u' for its rows but u only for one product with a sum
    // the bringing warp has made, so the long way from a correction through the rows and the
    // shuffles to a correction spans two tokens, and two tokens' sums are in flight together.
    float S[R], kp[R], ka[R];
    if (brings) {
        start(0);
        gd_commit();
        start(1);
        gd_commit();
        gd_wait<1>();
        __syncwarp();
        sums(0);
    } else {
#pragma unroll
        for (int i = 0; i < R; i += 4) {
            const int row = gd_row<P>(i, part);
            if (wide && live && row < d) {
                const float4 x = *reinterpret_cast<const float4*>(Sg + row);
                S[i] = x.x; S[i + 1] = x.y; S[i + 2] = x.z; S[i + 3] = x.w;
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j) S[i + j] = (live && row + j < d) ? Sg[row + j] : 0.f;
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) kp[i + j] = ka[i + j] = 0.f;
        }
    }
    __syncthreads();                               // chunk 0 has arrived
    float up = 0.f, up2 = 0.f;                     // the corrections of the last token and the one before
    float* o_ptr = o_out + (size_t)t0 * H * dv + h * dv + (live ? col : 0);
    const size_t o_step = (size_t)H * dv;
    const bool writes = live && part == 0;
    for (int c = 0; c < n_chunks; ++c) {
        if (brings) {
            start(c + 2);                          // into the buffer that chunk c-1 was read from
            gd_commit();
            gd_wait<1>();                          // chunk c+1 is here
            __syncwarp();
            sums(c + 1);
        } else {
            const int n = min(chunk, qlen - c * chunk);
            const float* slot_t = ring + (size_t)(c % 3) * chunk * SLOT;
            const int v_at = 3 * DP + 4 + tid / P;
            // one token's pass over the thread's rows: they receive the write before last
            // (correction `lag`) and the decay, and give this thread's share of Z^T k and Z^T q
            auto rows = [&](const float* at, float lag, float& acc, float& o) {
                const float4* q4 = reinterpret_cast<const float4*>(at) + part;
                const float4* k4 = q4 + DP / 4;
                const float4* g4 = k4 + DP / 4;
                float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f, o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
                for (int i = 0; i < R / 4; ++i) {
                    const float4 kk = k4[i * P], gg = g4[i * P], qq = q4[i * P];
                    const float s0 = fmaf(ka[4 * i + 0], lag, S[4 * i + 0]) * gg.x;
                    const float s1 = fmaf(ka[4 * i + 1], lag, S[4 * i + 1]) * gg.y;
                    const float s2 = fmaf(ka[4 * i + 2], lag, S[4 * i + 2]) * gg.z;
                    const float s3 = fmaf(ka[4 * i + 3], lag, S[4 * i + 3]) * gg.w;
                    S[4 * i + 0] = s0; a0 = fmaf(s0, kk.x, a0); o0 = fmaf(s0, qq.x, o0);
                    S[4 * i + 1] = s1; a1 = fmaf(s1, kk.y, a1); o1 = fmaf(s1, qq.y, o1);
                    S[4 * i + 2] = s2; a2 = fmaf(s2, kk.z, a2); o2 = fmaf(s2, qq.z, o2);
                    S[4 * i + 3] = s3; a3 = fmaf(s3, kk.w, a3); o3 = fmaf(s3, qq.w, o3);
                    ka[4 * i + 0] = kp[4 * i + 0] * gg.x; kp[4 * i + 0] = kk.x;
                    ka[4 * i + 1] = kp[4 * i + 1] * gg.y; kp[4 * i + 1] = kk.y;
                    ka[4 * i + 2] = kp[4 * i + 2] * gg.z; kp[4 * i + 2] = kk.z;
                    ka[4 * i + 3] = kp[4 * i + 3] * gg.w; kp[4 * i + 3] = kk.w;
                }
                acc = (a0 + a1) + (a2 + a3);
                o = (o0 + o1) + (o2 + o3);
            };
            int j = 0;
            // two tokens at a time: the second token's rows need only the first's lagging
            // correction, which is known, so both passes and all four sums run together
            for (; j + 1 < n; j += 2, slot_t += 2 * SLOT, o_ptr += 2 * o_step) {
                const float* next = slot_t + SLOT;
                const float v0 = slot_t[v_at], v1 = next[v_at];
                const float4 e0 = *reinterpret_cast<const float4*>(slot_t + 3 * DP);   // beta, q.k, kk, kq
                const float4 e1 = *reinterpret_cast<const float4*>(next + 3 * DP);
                float acc0, o0, acc1, o1;
                rows(slot_t, up2, acc0, o0);
                rows(next, up, acc1, o1);
#pragma unroll
                for (int s = P / 2; s > 0; s >>= 1) {
                    acc0 += __shfl_xor_sync(0xffffffffu, acc0, s);
                    acc1 += __shfl_xor_sync(0xffffffffu, acc1, s);
                    o0 += __shfl_xor_sync(0xffffffffu, o0, s);
                    o1 += __shfl_xor_sync(0xffffffffu, o1, s);
                }
                const float u0 = e0.x * (v0 - fmaf(up, e0.z, acc0));
                const float u1 = e1.x * (v1 - fmaf(u0, e1.z, acc1));
                if (writes) {
                    o_ptr[0] = fmaf(e0.y, u0, fmaf(up, e0.w, o0));
                    o_ptr[o_step] = fmaf(e1.y, u1, fmaf(u0, e1.w, o1));
                }
                up2 = u0;
                up = u1;
            }
            if (j < n) {
                const float v = slot_t[v_at];
                const float4 e = *reinterpret_cast<const float4*>(slot_t + 3 * DP);
                float acc, o;
                rows(slot_t, up2, acc, o);
#pragma unroll
                for (int s = P / 2; s > 0; s >>= 1) {
                    acc += __shfl_xor_sync(0xffffffffu, acc, s);
                    o += __shfl_xor_sync(0xffffffffu, o, s);
                }
                const float u = e.x * (v - fmaf(up, e.z, acc));
                if (writes) *o_ptr = fmaf(e.y, u, fmaf(up, e.w, o));
                up2 = up;
                up = u;
                o_ptr += o_step;
            }
        }
        __syncthreads();                           // chunk c is read, chunk c+1 has arrived
    }
    if (brings) return;
#pragma unroll
    for (int i = 0; i < R; ++i) S[i] = fmaf(kp[i], up, fmaf(ka[i], up2, S[i]));
#pragma unroll
    for (int i = 0; i < R; i += 4) {
        const int row = gd_row<P>(i, part);
        if (wide && live && row < d) {
            *reinterpret_cast<float4*>(Sg + row) = make_float4(S[i], S[i + 1], S[i + 2], S[i + 3]);
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (live && row + j < d) Sg[row + j] = S[i + j];
        }
    }
}

// The scan for steps in which every request brings one token (and, slowly but rightly, for
// any other step): no bringing warp and no buffers in turn, so that a block is small and many
// fit a multiprocessor.  Every thread copies its share of the token's q, k and g, reads its
// rows of the state meanwhile, and writes them back with the token's write added.
template <int R, int P>
__global__ void __launch_bounds__(GD_SINGLE_THREADS)
gdr_single_kernel(const float* __restrict__ prep, int PW, float* __restrict__ state, long long rec,
                  const int* __restrict__ q_start, const int* __restrict__ state_slot,
                  float* __restrict__ o_out, int H, int G, int d, int dv, int taps, int col_blocks) {
    constexpr int DP = R * P;
    const int threads = blockDim.x, COLS = threads / P;
    rv_pdl_launch_dependents();
    extern __shared__ __align__(16) float ring[];          // q | k | g [DP each] | beta | q.k | v [COLS]
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
    const int tail = (2 * G + H) * DP;
    const int b_off = tail + ((H * dv + 3) & ~3) + h;
    const int kq_off = b_off - h + ((H + 3) & ~3) + kvh;
    rv_pdl_wait();
    float* Sg = state + (size_t)slot * rec + (size_t)(taps - 1) * C + ((size_t)h * dv + (live ? col : 0)) * d;
    const bool wide = (d & 3) == 0 && (reinterpret_cast<size_t>(Sg) & 15) == 0;
    float S[R];
    for (int t = 0; t < qlen; ++t) {
        if (t) __syncthreads();                    // the token before is read
        const float* row = prep + (size_t)(t0 + t) * PW;
        for (int e = tid; e < 3 * DP / 4; e += threads) {
            const int seg = e / (DP / 4), off = e - seg * (DP / 4);
            const int from = (seg == 0 ? kvh : seg == 1 ? G + kvh : 2 * G + h) * DP;
            gd_copy16(ring + seg * DP + off * 4, row + from + off * 4);
        }
        if (tid < COLS && cb * COLS + tid < dv) gd_copy4(ring + 3 * DP + 2 + tid, row + tail + h * dv + cb * COLS + tid);
        if (tid == threads - 1) gd_copy4(ring + 3 * DP, row + b_off);
        if (tid == threads - 2) gd_copy4(ring + 3 * DP + 1, row + kq_off);
        gd_commit();
        if (t == 0) {
#pragma unroll
            for (int i = 0; i < R; i += 4) {
                const int at = gd_row<P>(i, part);
                if (wide && live && at < d) {
                    const float4 x = *reinterpret_cast<const float4*>(Sg + at);
                    S[i] = x.x; S[i + 1] = x.y; S[i + 2] = x.z; S[i + 3] = x.w;
                } else {
#pragma unroll
                    for (int j = 0; j < 4; ++j) S[i + j] = (live && at + j < d) ? Sg[at + j] : 0.f;
                }
            }
        }
        gd_wait<0>();
        __syncthreads();
        const float v = ring[3 * DP + 2 + tid / P], beta = ring[3 * DP], qk = ring[3 * DP + 1];
        const float4* q4 = reinterpret_cast<const float4*>(ring) + part;
        const float4* k4 = q4 + DP / 4;
        const float4* g4 = k4 + DP / 4;
        float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f, o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
        float4 kk[R / 4];
#pragma unroll
        for (int i = 0; i < R / 4; ++i) {
            const float4 gg = g4[i * P], qq = q4[i * P];
            kk[i] = k4[i * P];
            S[4 * i + 0] *= gg.x; a0 = fmaf(S[4 * i + 0], kk[i].x, a0); o0 = fmaf(S[4 * i + 0], qq.x, o0);
            S[4 * i + 1] *= gg.y; a1 = fmaf(S[4 * i + 1], kk[i].y, a1); o1 = fmaf(S[4 * i + 1], qq.y, o1);
            S[4 * i + 2] *= gg.z; a2 = fmaf(S[4 * i + 2], kk[i].z, a2); o2 = fmaf(S[4 * i + 2], qq.z, o2);
            S[4 * i + 3] *= gg.w; a3 = fmaf(S[4 * i + 3], kk[i].w, a3); o3 = fmaf(S[4 * i + 3], qq.w, o3);
        }
        float acc = (a0 + a1) + (a2 + a3), o = (o0 + o1) + (o2 + o3);
#pragma unroll
        for (int s = P / 2; s > 0; s >>= 1) {
            acc += __shfl_xor_sync(0xffffffffu, acc, s);
            o += __shfl_xor_sync(0xffffffffu, o, s);
        }
        const float u = beta * (v - acc);
        if (live && part == 0) o_out[(size_t)(t0 + t) * H * dv + h * dv + col] = fmaf(qk, u, o);
#pragma unroll
        for (int i = 0; i < R / 4; ++i) {
            S[4 * i + 0] = fmaf(kk[i].x, u, S[4 * i + 0]);
            S[4 * i + 1] = fmaf(kk[i].y, u, S[4 * i + 1]);
            S[4 * i + 2] = fmaf(kk[i].z, u, S[4 * i + 2]);
            S[4 * i + 3] = fmaf(kk[i].w, u, S[4 * i + 3]);
        }
    }
#pragma unroll
    for (int i = 0; i < R; i += 4) {
        const int at = gd_row<P>(i, part);
        if (wide && live && at < d) {
            *reinterpret_cast<float4*>(Sg + at) = make_float4(S[i], S[i + 1], S[i + 2], S[i + 3]);
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (live && at + j < d) Sg[at + j] = S[i + j];
        }
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
    static const int table[][3] = {{8, 8, 1},    {16, 8, 2},   {32, 8, 4},    {64, 8, 8},
                                   {128, 8, 16}, {256, 8, 32}, {512, 16, 32}, {1024, 32, 32}};
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
static void gd_launch_single(const float* prep, int PW, float* state, long long rec, const int* q_start,
                             const int* state_slot, float* o, int n_reqs, int H, int G, int d, int dv,
                             int taps, cudaStream_t s) {
    int threads = ((dv * P + 31) / 32) * 32;
    if (threads > GD_SINGLE_THREADS) threads = GD_SINGLE_THREADS;
    const int cols = threads / P;
    const int col_blocks = (dv + cols - 1) / cols;
    const size_t smem = (size_t)(3 * R * P + ((cols + 2 + 3) & ~3)) * sizeof(float);
    if (smem > 48 * 1024)
        cudaFuncSetAttribute(gdr_single_kernel<R, P>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    rv_launch(gdr_single_kernel<R, P>, dim3(H * col_blocks, n_reqs), dim3(threads), smem, s, prep, PW, state,
              rec, q_start, state_slot, o, H, G, d, dv, taps, col_blocks);
}

template <int R, int P>
static void gd_launch_scan(const float* prep, int PW, float* state, long long rec, const int* q_start,
                           const int* state_slot, float* o, int n_reqs, int longest, int H, int G, int d,
                           int dv, int taps, cudaStream_t s) {
    // as many working threads as the head's columns need, in whole warps, at most
    // GD_MAX_THREADS, and one more warp that brings the inputs
    int threads = ((dv * P + 31) / 32) * 32;
    if (threads > GD_MAX_THREADS) threads = GD_MAX_THREADS;
    const int cols = threads / P;
    const int col_blocks = (dv + cols - 1) / cols;
    // tokens per buffer: 16, fewer where three buffers of them would pass 96 KB, and no more
    // than the longest portion can have
    const int slot = 3 * R * P + ((cols + 4 + 3) & ~3);
    int chunk = GD_BUFFER_FLOATS / slot;
    chunk = chunk < 1 ? 1 : chunk > GD_CHUNK ? GD_CHUNK : chunk;
    if (H * col_blocks * n_reqs > rv_sm_count() && chunk > GD_CHUNK / 2) chunk = GD_CHUNK / 2;
    if (chunk > longest) chunk = longest;
    const size_t smem = (size_t)3 * chunk * slot * sizeof(float);
    if (smem > 48 * 1024)
        cudaFuncSetAttribute(gdr_scan_kernel<R, P>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    rv_launch(gdr_scan_kernel<R, P>, dim3(H * col_blocks, n_reqs), dim3(threads + 32), smem, s, prep, PW,
              state, rec, q_start, state_slot, o, H, G, d, dv, taps, col_blocks, chunk);
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
    // the staging buffers are sized for the longest portion the step can have if every request
    // brings a token; the size changes only how often the scan's blocks meet, not what they compute
    const int longest = n_tokens - n_reqs + 1 > 1 ? n_tokens - n_reqs + 1 : 1;
    if (longest == 1) {
#define GD_CASE(r_, p_)                                                                                \
    if (R == r_ && TP == p_)                                                                           \
        gd_launch_single<r_, p_>(prep, PW, state, rec, q_start, state_slot, o, n_reqs, H, G, d, dv, taps, s);
        GD_CASE(8, 1) GD_CASE(8, 2) GD_CASE(8, 4) GD_CASE(8, 8) GD_CASE(8, 16) GD_CASE(8, 32) GD_CASE(16, 32)
        GD_CASE(32, 32)
#undef GD_CASE
    } else {
#define GD_CASE(r_, p_)                                                                                \
    if (R == r_ && TP == p_)                                                                           \
        gd_launch_scan<r_, p_>(prep, PW, state, rec, q_start, state_slot, o, n_reqs, longest, H, G, d, dv, taps, s);
        GD_CASE(8, 1) GD_CASE(8, 2) GD_CASE(8, 4) GD_CASE(8, 8) GD_CASE(8, 16) GD_CASE(8, 32) GD_CASE(16, 32)
        GD_CASE(32, 32)
#undef GD_CASE
    }
    RV_CHECK_LAUNCH("gated_delta scan");
    RV_DISPATCH_DTYPE(out_dtype, "gated_delta", {
        rv_launch(gdr_finish_kernel<T>, dim3(n_tokens + n_reqs), dim3(128), 0, s, (const float*)o, proj, P,
                  lowrank, LW, norm_w, state, rec, token_req, q_start, state_slot, (T*)y, n_tokens, H, G, d,
                  dv, taps, eps);
    });
    RV_CHECK_LAUNCH("gated_delta finish");
    return 0;
}
