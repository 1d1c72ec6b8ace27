// Mixture of experts: the choice of a token's experts, and the experts' SwiGLU feed-forwards
// walked token by token (the form for few tokens and for float32; moe_grouped.cu has the
// grouped matrix products for many bfloat16 tokens).
//
//   moe_select     logits float32 [N, E] -> ids int32 [N, top], weights float32 [N, top].
//                  s = sigmoid(logits); with `groups` > 1 the experts form that many equal
//                  groups of neighbours, a group's score is the sum of its `group_top` largest
//                  s, and only experts of the `keep` best groups can be chosen; the `top`
//                  largest allowed s are chosen (ties: the lower index first, for groups too);
//                  weights = chosen s / (their sum + weight_eps).  One warp per token.
//                  Options: score_mode 1 makes s the softmax of the logits over all experts
//                  instead of their sigmoids; renorm 0 leaves the chosen s undivided; every
//                  weight is multiplied by route_scale.  `choice_bias` float32 [E], if given,
//                  is added to s wherever experts (and groups) are compared; the weights are
//                  made from s without it.
//   moe_route      the router's product (x [N, W] of any type, router float32 [E, W]) and the same
//                  choice in one kernel.
//   moe_gate_up    act[pair, f] = silu(<gate_e[f], x_t>) * <up_e[f], x_t> for pair = t * top + k,
//                  e = ids[t, k]; gate_up is [E, 2F, W] with gate and up rows alternating
//                  (row 2f: gate f, row 2f + 1: up f).  act_mode 1: with g = min(gate, limit) and
//                  u = clamp(up, -limit, limit) the value is g * sigmoid(alpha g) * (u + 1).
//                  act_mode 2: experts without a gate; the matrix is [E, F, W] and the value is
//                  max(<up_e[f], x_t>, 0)^2.
//   moe_down       out[t, w] = sum_k weights[t, k] * <down_e(k)[w], act[t * top + k]>, the sum in
//                  the order of k; down is [E, W, F].  `addend` [N, W], if given, is where each sum
//                  starts (the output of an expert that every token uses).
// Dot products and the activation are float32; act is rounded to the storage type.
// Plain references: tests/plain_ops.py moe_select, moe_experts.
#include "common.cuh"

#define MOE_MAX_GROUP_TOP 8

// (value, index) of the largest sc[e] over e in [lo, hi), ties to the lower index; whole warp.
__device__ __forceinline__ void moe_warp_argmax(const float* sc, int lo, int hi, int lane,
                                                float& best, int& idx) {
    best = -INFINITY;
    idx = 0x7fffffff;
    for (int e = lo + lane; e < hi; e += 32) {
        const float v = sc[e];
        if (v > best) {
            best = v;
            idx = e;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ov > best || (ov == best && oi < idx)) {
            best = ov;
            idx = oi;
        }
    }
    if (idx == 0x7fffffff) idx = lo;             // nothing compared greater (NaN scores)
}

// One token's choice, by one warp.  sc [E]: router logits on entry (scores afterwards);
// gs [groups]: scratch.  Writes ids[top] and weights[top].
__device__ __forceinline__ void moe_select_warp(float* sc, float* gs, int E, int top, int groups,
                                                int keep, int group_top, float weight_eps,
                                                int* __restrict__ ids, float* __restrict__ weights,
                                                int lane, int score_mode = 0, int renorm = 1,
                                                float route_scale = 1.f,
                                                const float* __restrict__ choice_bias = nullptr,
                                                float* orig = nullptr) {
    if (score_mode == 1) {                           // softmax over all experts
        float m = -INFINITY;
        for (int e = lane; e < E; e += 32) m = fmaxf(m, sc[e]);
        m = rv_warp_max(m);
        float tot = 0.f;
        for (int e = lane; e < E; e += 32) {
            const float v = expf(sc[e] - m);
            sc[e] = v;
            tot += v;
        }
        tot = rv_warp_sum(tot);
        for (int e = lane; e < E; e += 32) sc[e] = sc[e] / tot;
    } else {
        for (int e = lane; e < E; e += 32) sc[e] = 1.f / (1.f + expf(-sc[e]));
    }
    if (choice_bias) {                               // compare s + bias, weigh with s
        for (int e = lane; e < E; e += 32) {
            orig[e] = sc[e];
            sc[e] += choice_bias[e];
        }
    }
    __syncwarp();
    if (groups > 1) {
        const int size = E / groups;
        for (int g = 0; g < groups; ++g) {
            // the sum of the group's largest scores: take them out one by one, then put them back
            float sum = 0.f, taken_v[MOE_MAX_GROUP_TOP];
            int taken_i[MOE_MAX_GROUP_TOP];
            const int n_take = min(group_top, size);
            for (int k = 0; k < n_take; ++k) {
                float v;
                int i;
                moe_warp_argmax(sc, g * size, (g + 1) * size, lane, v, i);
                sum += v;
                taken_v[k] = v;
                taken_i[k] = i;
                __syncwarp();
                if (lane == 0) sc[i] = -INFINITY;
                __syncwarp();
            }
            if (lane == 0) {
                for (int k = 0; k < n_take; ++k) sc[taken_i[k]] = taken_v[k];
                gs[g] = sum;
            }
            __syncwarp();
        }
        // the `keep` best groups stay: their score becomes +inf, then the others' experts go
        for (int k = 0; k < keep; ++k) {
            float best = -INFINITY;
            int idx = 0x7fffffff;
            for (int g = lane; g < groups; g += 32) {
                const float v = gs[g];
                if (v != INFINITY && v > best) {
                    best = v;
                    idx = g;
                }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, best, o);
                const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
                if (ov > best || (ov == best && oi < idx)) {
                    best = ov;
                    idx = oi;
                }
            }
            __syncwarp();
            if (lane == 0 && idx < groups) gs[idx] = INFINITY;
            __syncwarp();
        }
        for (int e = lane; e < E; e += 32)
            if (gs[e / size] != INFINITY) sc[e] = -3.0e38f;      // below every score
        __syncwarp();
    }
    float sum = 0.f, mine = 0.f;
    int mine_id = 0;
    for (int k = 0; k < top; ++k) {
        float v;
        int i;
        moe_warp_argmax(sc, 0, E, lane, v, i);
        if (choice_bias) v = orig[i];
        sum += v;
        if (lane == (k & 31) && k < 32) {
            mine = v;
            mine_id = i;
        }
        if (k >= 32 && lane == 0) {                  // more than 32 experts a token: written at once
            ids[k] = i;
            weights[k] = v;                          // divided below
        }
        __syncwarp();
        if (lane == 0) sc[i] = -INFINITY;            // taken: below the experts left out
        __syncwarp();
    }
    const float inv = (renorm ? 1.f / (sum + weight_eps) : 1.f) * route_scale;
    if (lane < top) {
        ids[lane] = mine_id;
        weights[lane] = mine * inv;
    }
    if (lane == 0)
        for (int k = 32; k < top; ++k) weights[k] *= inv;
}

__global__ void moe_select_kernel(const float* __restrict__ logits, int n_tokens, int E, int top,
                                  int groups, int keep, int group_top, float weight_eps,
                                  int* __restrict__ ids, float* __restrict__ weights, int score_mode,
                                  int renorm, float route_scale,
                                  const float* __restrict__ choice_bias) {
    rv_pdl_prologue();
    extern __shared__ float smem[];
    const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
    const int t = blockIdx.x * (blockDim.x >> 5) + wib;
    if (t >= n_tokens) return;
    float* sc = smem + (size_t)wib * (2 * E + groups);   // [E] scores, [groups], [E] unbiased scores
    for (int e = lane; e < E; e += 32) sc[e] = logits[(size_t)t * E + e];
    __syncwarp();
    moe_select_warp(sc, sc + E, E, top, groups, keep, group_top, weight_eps,
                    ids + (size_t)t * top, weights + (size_t)t * top, lane, score_mode, renorm,
                    route_scale, choice_bias, sc + E + groups);
}

// The router's product and the choice in one kernel: a block takes MOE_ROUTE_TOK tokens; each
// warp walks the router's rows (float32) e = warp, warp + 8, ... and forms the logit of every
// token of the block (so a row is read once per block, the tokens' rows come from L1), then
// warp t makes token t's choice.  Products and sums are float32 whatever the rows' type.
#define MOE_ROUTE_TOK 8
__device__ __forceinline__ void moe_load8(const float* p, float (&v)[8]) {
    const float4 a = *(const float4*)p, b = *(const float4*)(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void moe_load8(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 raw = *(const uint4*)p;
    const __nv_bfloat162* h = (const __nv_bfloat162*)&raw;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(h[j]);
        v[2 * j] = f.x;
        v[2 * j + 1] = f.y;
    }
}
template <typename T>
__global__ void __launch_bounds__(MOE_ROUTE_TOK * 32) moe_route_kernel(
    const T* __restrict__ x, const float* __restrict__ router, int n_tokens, int W, int E, int top,
    int groups, int keep, int group_top, float weight_eps, int* __restrict__ ids,
    float* __restrict__ weights, int stage_rows, int score_mode, int renorm, float route_scale,
    const float* __restrict__ choice_bias) {
    rv_pdl_prologue();
    extern __shared__ __align__(16) float smem[];        // [MOE_ROUTE_TOK][2 E + groups], then the rows
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int t0 = blockIdx.x * MOE_ROUTE_TOK;
    const int nt = min(MOE_ROUTE_TOK, n_tokens - t0);
    const int stride = 2 * E + groups;
    // eight values a lane and step (16-byte loads) when the width allows
    const bool vec = W % 8 == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)router & 15) == 0;
    // The block's rows go to shared memory first (one round trip for all of them), so that the
    // loop over a router row waits only for that row, whose loads the compiler can then issue
    // several steps ahead.  Rows beyond the last token are zeros.
    T* xs = (T*)(smem + ((MOE_ROUTE_TOK * stride + 3) & ~3));
    const T* rows = x + (size_t)t0 * W;
    if (stage_rows) {
        if (vec) {
            const int ppr = W * (int)sizeof(T) / 16;          // 16-byte pieces per row
            const uint4* src = (const uint4*)rows;
            for (int i = threadIdx.x; i < MOE_ROUTE_TOK * ppr; i += blockDim.x)
                ((uint4*)xs)[i] = i / ppr < nt ? src[i] : make_uint4(0, 0, 0, 0);
        } else {
            for (int i = threadIdx.x; i < MOE_ROUTE_TOK * W; i += blockDim.x)
                xs[i] = i / W < nt ? rows[i] : T(0.f);
        }
        __syncthreads();
        rows = xs;
    }
    const int last = stage_rows ? MOE_ROUTE_TOK - 1 : nt - 1;   // staged rows are all there
    for (int e = warp; e < E; e += MOE_ROUTE_TOK) {
        const float* w_row = router + (size_t)e * W;
        float acc[MOE_ROUTE_TOK];
#pragma unroll
        for (int t = 0; t < MOE_ROUTE_TOK; ++t) acc[t] = 0.f;
        if (vec) {
#pragma unroll 4
            for (int i = lane * 8; i < W; i += 256) {
                const float4 w0 = *(const float4*)(w_row + i), w1 = *(const float4*)(w_row + i + 4);
#pragma unroll
                for (int t = 0; t < MOE_ROUTE_TOK; ++t) {
                    float xv[8];
                    moe_load8(rows + (size_t)min(t, last) * W + i, xv);
                    acc[t] += w0.x * xv[0] + w0.y * xv[1] + w0.z * xv[2] + w0.w * xv[3] +
                              w1.x * xv[4] + w1.y * xv[5] + w1.z * xv[6] + w1.w * xv[7];
                }
            }
        } else {
            for (int i = lane; i < W; i += 32) {
                const float w = w_row[i];
#pragma unroll
                for (int t = 0; t < MOE_ROUTE_TOK; ++t)
                    if (t <= last) acc[t] += w * rv_load(rows + (size_t)t * W + i);
            }
        }
#pragma unroll
        for (int t = 0; t < MOE_ROUTE_TOK; ++t) {
            const float v = rv_warp_sum(acc[t]);
            if (lane == 0) smem[t * stride + e] = v;
        }
    }
    __syncthreads();
    if (warp < nt) {
        float* sc = smem + warp * stride;
        int* my_ids = ids + (size_t)(t0 + warp) * top;
        float* my_weights = weights + (size_t)(t0 + warp) * top;
        moe_select_warp(sc, sc + E, E, top, groups, keep, group_top, weight_eps, my_ids, my_weights,
                        lane, score_mode, renorm, route_scale, choice_bias, sc + E + groups);
    }
}

// ---------------------------------------------------------------------------------
#define MOE_ROWS 32        // output rows per block of the two simple kernels

template <typename T>
__global__ void moe_gate_up_kernel(const T* __restrict__ x, const int* __restrict__ ids,
                                   const T* __restrict__ gate_up, T* __restrict__ act, int top,
                                   int E, int W, int F, int act_mode, float limit, float alpha) {
    rv_pdl_prologue();
    extern __shared__ float xs[];                      // [W]
    const int pair = blockIdx.x;
    const int t = pair / top;
    const int e = ids[pair];
    for (int i = threadIdx.x; i < W; i += blockDim.x) xs[i] = rv_load(x + (size_t)t * W + i);
    __syncthreads();
    if (e < 0 || e >= E) return;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int f_end = min(F, (int)(blockIdx.y + 1) * MOE_ROWS);
    if (act_mode == 2) {                               // no gate: [E, F, W], relu squared
        const T* wu = gate_up + (size_t)e * F * W;
        for (int f = blockIdx.y * MOE_ROWS + warp; f < f_end; f += nwarps) {
            const T* u_row = wu + (size_t)f * W;
            float u = 0.f;
            for (int i = lane; i < W; i += 32) u += xs[i] * rv_load(u_row + i);
            u = fmaxf(rv_warp_sum(u), 0.f);
            if (lane == 0) rv_store(act + (size_t)pair * F + f, u * u);
        }
        return;
    }
    const T* wg = gate_up + (size_t)e * 2 * F * W;
    for (int f = blockIdx.y * MOE_ROWS + warp; f < f_end; f += nwarps) {
        const T* g_row = wg + (size_t)(2 * f) * W;
        const T* u_row = g_row + W;
        float g = 0.f, u = 0.f;
        for (int i = lane; i < W; i += 32) {
            const float xv = xs[i];
            g += xv * rv_load(g_row + i);
            u += xv * rv_load(u_row + i);
        }
        g = rv_warp_sum(g);
        u = rv_warp_sum(u);
        if (lane == 0) {
            float v;
            if (act_mode == 1) {
                g = fminf(g, limit);
                u = fminf(fmaxf(u, -limit), limit);
                v = g / (1.f + expf(-alpha * g)) * (u + 1.f);
            } else {
                v = g / (1.f + expf(-g)) * u;
            }
            rv_store(act + (size_t)pair * F + f, v);
        }
    }
}

template <typename T>
__global__ void moe_down_kernel(const T* __restrict__ act, const int* __restrict__ ids,
                                const float* __restrict__ weights, const T* __restrict__ down,
                                const T* __restrict__ addend, T* __restrict__ out, int top, int E,
                                int W, int F) {
    rv_pdl_prologue();
    extern __shared__ float as[];                      // [top * F]
    const int t = blockIdx.x;
    for (int i = threadIdx.x; i < top * F; i += blockDim.x)
        as[i] = rv_load(act + (size_t)t * top * F + i);
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int w_end = min(W, (int)(blockIdx.y + 1) * MOE_ROWS);
    for (int w = blockIdx.y * MOE_ROWS + warp; w < w_end; w += nwarps) {
        float y = addend ? rv_load(addend + (size_t)t * W + w) : 0.f;
        for (int k = 0; k < top; ++k) {
            const int e = ids[(size_t)t * top + k];
            if (e < 0 || e >= E) continue;
            const T* row = down + ((size_t)e * W + w) * F;
            float s = 0.f;
            for (int i = lane; i < F; i += 32) s += as[k * F + i] * rv_load(row + i);
            s = rv_warp_sum(s);
            y += weights[(size_t)t * top + k] * s;
        }
        if (lane == 0) rv_store(out + (size_t)t * W + w, y);
    }
}

extern "C" int rv_moe_select(const float* logits, int n_tokens, int E, int top, int groups,
                             int keep, int group_top, float weight_eps, int* ids, float* weights,
                             int score_mode, int renorm, float route_scale, const float* choice_bias,
                             void* stream) {
    if (n_tokens == 0) return 0;
    if (n_tokens < 0 || E < 1 || top < 1 || top > E) RV_FAIL("moe_select: bad sizes");
    if (groups < 1 || E % groups || keep < 1 || keep > groups || keep * (E / groups) < top)
        RV_FAIL("moe_select: %d experts in %d groups of which %d are kept cannot give %d", E,
                groups, keep, top);
    if (group_top < 1 || group_top > MOE_MAX_GROUP_TOP)
        RV_FAIL("moe_select: a group's score sums 1 to %d scores", MOE_MAX_GROUP_TOP);
    const int wpb = 4;
    const size_t smem = (size_t)wpb * (2 * E + groups) * sizeof(float);
    if (smem > 48 * 1024) RV_FAIL("moe_select: too many experts");
    rv_launch(moe_select_kernel, dim3((n_tokens + wpb - 1) / wpb), dim3(wpb * 32), smem,
              (cudaStream_t)stream, logits, n_tokens, E, top, groups, keep, group_top, weight_eps,
              ids, weights, score_mode, renorm, route_scale, choice_bias);
    RV_CHECK_LAUNCH("moe_select");
    return 0;
}

extern "C" int rv_moe_route(const void* x, int dtype, const float* router, int n_tokens, int W,
                            int E, int top, int groups, int keep, int group_top, float weight_eps,
                            int* ids, float* weights, int score_mode, int renorm, float route_scale,
                            const float* choice_bias, void* stream) {
    if (n_tokens == 0) return 0;
    if (n_tokens < 0 || W < 1 || E < 1 || top < 1 || top > E) RV_FAIL("moe_route: bad sizes");
    if (groups < 1 || E % groups || keep < 1 || keep > groups || keep * (E / groups) < top)
        RV_FAIL("moe_route: %d experts in %d groups of which %d are kept cannot give %d", E, groups,
                keep, top);
    if (group_top < 1 || group_top > MOE_MAX_GROUP_TOP)
        RV_FAIL("moe_route: a group's score sums 1 to %d scores", MOE_MAX_GROUP_TOP);
    size_t smem = (size_t)((MOE_ROUTE_TOK * (2 * E + groups) + 3) & ~3) * sizeof(float);
    if (smem > 40 * 1024) RV_FAIL("moe_route: too many experts");
    // the block's rows in shared memory when they fit beside the logits in 48 KB
    const size_t row_bytes = (size_t)MOE_ROUTE_TOK * W * (dtype == RV_DTYPE_BF16 ? 2 : 4);
    const int stage_rows = smem + row_bytes <= 48 * 1024;
    if (stage_rows) smem += row_bytes;
    const int blocks = (n_tokens + MOE_ROUTE_TOK - 1) / MOE_ROUTE_TOK;
    RV_DISPATCH_DTYPE(dtype, "moe_route",
                      (rv_launch(moe_route_kernel<T>, dim3(blocks), dim3(MOE_ROUTE_TOK * 32), smem,
                                 (cudaStream_t)stream, (const T*)x, router, n_tokens, W, E, top,
                                 groups, keep, group_top, weight_eps, ids, weights, stage_rows,
                                 score_mode, renorm, route_scale, choice_bias)));
    RV_CHECK_LAUNCH("moe_route");
    return 0;
}

// act: scratch [n_tokens * top, F] of the storage type.
extern "C" int rv_moe_experts_simple(const void* x, int dtype, const int* ids, const float* weights,
                                     const void* gate_up, const void* down, void* act, void* out,
                                     int n_tokens, int top, int E, int W, int F, int act_mode,
                                     float limit, float alpha, const void* addend, void* stream) {
    if (n_tokens == 0) return 0;
    if (n_tokens < 0 || top < 1 || E < 1 || W < 1 || F < 1) RV_FAIL("moe_experts: bad sizes");
    if ((size_t)W * 4 > 200 * 1024 || (size_t)top * F * 4 > 200 * 1024)
        RV_FAIL("moe_experts: rows of %d or %d x %d values do not fit shared memory", W, top, F);
    if ((long long)n_tokens * top > 0x7fffffffLL) RV_FAIL("moe_experts: too many rows");
    cudaStream_t s = (cudaStream_t)stream;
    const size_t smem1 = (size_t)W * 4, smem2 = (size_t)top * F * 4;
    RV_DISPATCH_DTYPE(dtype, "moe_experts", {
        if (smem1 > 48 * 1024)
            cudaFuncSetAttribute(moe_gate_up_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)smem1);
        if (smem2 > 48 * 1024)
            cudaFuncSetAttribute(moe_down_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)smem2);
        rv_launch(moe_gate_up_kernel<T>, dim3(n_tokens * top, (F + MOE_ROWS - 1) / MOE_ROWS),
                  dim3(128), smem1, s, (const T*)x, ids, (const T*)gate_up, (T*)act, top, E, W, F,
                  act_mode, limit, alpha);
        rv_launch(moe_down_kernel<T>, dim3(n_tokens, (W + MOE_ROWS - 1) / MOE_ROWS), dim3(128),
                  smem2, s, (const T*)act, ids, weights, (const T*)down, (const T*)addend, (T*)out, top,
                  E, W, F);
    });
    RV_CHECK_LAUNCH("moe_experts");
    return 0;
}
