// Mixture of experts for many bfloat16 tokens: the tokens' (token, expert) pairs are sorted by
// expert, and each expert's rows pass its two matrices as tiles of one grouped matrix product
// on the 5th-generation tensor cores.
//
//   moe_sort      ids [N, top] -> a layout of rows in which expert e owns a stretch that
//                 begins at a multiple of TN rows: sorted_token[row] = the pair's token (-1: a
//                 filling row), pair_pos[pair] = its row, and the list of token tiles
//                 (tile_expert, tile_row0, n_tiles).  Counts stay on the device, so a captured
//                 launch sequence serves any routing.
//   moe_gather    xs[row] = x[sorted_token[row]] (zeros for filling rows).
//   moe_grouped   out[row0 + t, n] = <xs[row0 + t], W[e][n]> for the rows of one token tile and
//                 128 rows of W[e] per block: 128 rows of W are the M side of a tcgen05.mma
//                 (cta_group::1, kind::f16, M = 128), the TN tokens its N side, the accumulator
//                 [128 lanes x TN columns] lives in TMEM; operands come by TMA
//                 (cp.async.bulk.tensor.2d, 128-byte swizzle, K tiles of 64) through a ring of
//                 stages guarded by mbarriers; one elected thread issues the copies, one the
//                 MMAs; four warps read the accumulator with tcgen05.ld.  W is the stack
//                 [E * n_out, K], so expert e's tile is a row offset.  With SWIGLU the rows of W
//                 alternate gate and up (row 2f: gate f, row 2f + 1: up f), neighbouring lanes
//                 hold a pair, and the epilogue writes silu(gate) * up [rows, n_out / 2].
//   moe_combine   out[t] = sum_k weights[t, k] * ys[pair_pos[t * top + k]], in the order of k.
//
// A row's sums depend on its own expert and values only, never on which other rows share its
// tile, so a token's result does not depend on the batch.  Every wait on an mbarrier is
// bounded (RV_WAIT_CYCLES); a wait that runs out records code 31-34 in `status`, every role
// leaves its loop, copies in flight are waited for (bounded), TMEM is freed, the block returns.
// No TMA multicast.  Plain reference: tests/plain_ops.py moe_experts.
#include "tcgen05_common.cuh"

#define MG_BM 128
#define MG_BK 64
#define MG_MAX_STAGES 8
#define MG_SMEM_LIMIT (110 * 1024)     // two blocks an SM: one's epilogue beside the other's products
#define MG_SMEM_MAX (200 * 1024)

__global__ void moe_sort_kernel(const int* __restrict__ ids, int P, int E, int top, int TN,
                                int rows_pad, int max_tiles, int* __restrict__ sorted_token,
                                int* __restrict__ pair_pos, int* __restrict__ tile_expert,
                                int* __restrict__ tile_row0, int* __restrict__ n_tiles) {
    rv_pdl_prologue();
    extern __shared__ int sm[];
    int* cnt = sm;             // [E]
    int* off = cnt + E;        // [E]
    int* cur = off + E;        // [E]
    for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = cur[e] = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < P; p += blockDim.x) {
        const int e = ids[p];
        if (e >= 0 && e < E) atomicAdd(&cnt[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int row = 0, tiles = 0;
        for (int e = 0; e < E; ++e) {
            off[e] = row;
            const int nt = (cnt[e] + TN - 1) / TN;
            for (int i = 0; i < nt && tiles < max_tiles; ++i) {
                tile_expert[tiles] = e;
                tile_row0[tiles] = row + i * TN;
                ++tiles;
            }
            row += nt * TN;
        }
        n_tiles[0] = tiles;
    }
    for (int r = threadIdx.x; r < rows_pad; r += blockDim.x) sorted_token[r] = -1;
    __syncthreads();
    for (int p = threadIdx.x; p < P; p += blockDim.x) {
        const int e = ids[p];
        int pos = 0;
        if (e >= 0 && e < E) {
            pos = off[e] + atomicAdd(&cur[e], 1);
            if (pos < rows_pad) sorted_token[pos] = p / top;
        }
        pair_pos[p] = pos;
    }
}

// one warp per row; width a multiple of 8
__global__ void moe_gather_kernel(const bf16* __restrict__ x, const int* __restrict__ sorted_token,
                                  bf16* __restrict__ xs, int rows, int W) {
    rv_pdl_prologue();
    const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (warp >= rows) return;
    const int t = sorted_token[warp];
    uint4* dst = (uint4*)(xs + (size_t)warp * W);
    if (t < 0) {
        for (int i = lane; i < W / 8; i += 32) dst[i] = make_uint4(0, 0, 0, 0);
        return;
    }
    const uint4* src = (const uint4*)(x + (size_t)t * W);
    for (int i = lane; i < W / 8; i += 32) dst[i] = src[i];
}

// one block per token; width a multiple of 8
__global__ void moe_combine_kernel(const bf16* __restrict__ ys, const int* __restrict__ pair_pos,
                                   const float* __restrict__ weights, const bf16* __restrict__ addend,
                                   bf16* __restrict__ out, int top, int W) {
    rv_pdl_prologue();
    const int t = blockIdx.x;
    for (int i = threadIdx.x; i < W / 8; i += blockDim.x) {
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.f;
        if (addend) {                                  // rows that every token gets (a shared expert)
            const uint4 raw = *((const uint4*)(addend + (size_t)t * W) + i);
            const __nv_bfloat162* h = (const __nv_bfloat162*)&raw;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 f = __bfloat1622float2(h[j]);
                acc[2 * j] = f.x;
                acc[2 * j + 1] = f.y;
            }
        }
        for (int k = 0; k < top; ++k) {
            const float wgt = weights[(size_t)t * top + k];
            const uint4 raw = *((const uint4*)(ys + (size_t)pair_pos[(size_t)t * top + k] * W) + i);
            const __nv_bfloat162* h = (const __nv_bfloat162*)&raw;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 f = __bfloat1622float2(h[j]);
                acc[2 * j] += wgt * f.x;
                acc[2 * j + 1] += wgt * f.y;
            }
        }
        uint4 res;
        __nv_bfloat162* o = (__nv_bfloat162*)&res;
#pragma unroll
        for (int j = 0; j < 4; ++j) o[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
        *((uint4*)(out + (size_t)t * W) + i) = res;
    }
}

// grid (ceil(n_out / (128 MT)), max_tiles); block 128 threads.  MT (1 or 2): how many tiles of
// 128 rows of W a block multiplies with its token tile; with two, the tokens' tile is copied
// once for twice the products (the kernel is bound by what an SM copies from L2: 32 KB per 64
// of K with one tile, 48 KB for two), each with an accumulator of its own in TMEM.
// ACT: 0 = the sums as they are; 1 = silu(gate) * up; 2 = the clamped form
//   g = min(gate, limit), u = clamp(up, -limit, limit), g * sigmoid(alpha g) * (u + 1)
// of pairs of neighbouring rows of W; 3 = max(sum, 0)^2 of every row (experts without a gate).
template <int ACT>
__global__ void __launch_bounds__(128, 2) moe_grouped_kernel(
    const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
    bf16* __restrict__ out, int* __restrict__ status, const int* __restrict__ tile_expert,
    const int* __restrict__ tile_row0, const int* __restrict__ n_tiles, int n_out, int kblocks,
    int TN, int stages, int MT, float limit, float alpha) {
    constexpr bool SWIGLU = ACT == 1 || ACT == 2;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* base = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const int w_half = MG_BM * MG_BK * 2;                     // one tile of 128 rows of W
    const int w_tile = MT * w_half, x_tile = TN * MG_BK * 2;
    unsigned char* w_tiles = base;
    unsigned char* x_tiles = base + stages * w_tile;
    __shared__ __align__(8) unsigned long long full_bar[MG_MAX_STAGES];
    __shared__ __align__(8) unsigned long long empty_bar[MG_MAX_STAGES];
    __shared__ __align__(8) unsigned long long accum_bar;
    __shared__ unsigned tmem_base_smem;
    __shared__ volatile int failed;

    rv_pdl_launch_dependents();
    rv_pdl_wait();                       // the list of tiles is written by an earlier kernel
    if ((int)blockIdx.y >= n_tiles[0]) return;
    const int expert = tile_expert[blockIdx.y], row0 = tile_row0[blockIdx.y];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int tile = blockIdx.x;
    const int w_row = expert * n_out + tile * MT * MG_BM;
    unsigned tmem_cols = 32;
    while ((int)tmem_cols < MT * TN) tmem_cols <<= 1;

    if (tid == 0) {
        failed = 0;
        for (int s = 0; s < stages; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        mbar_init(&accum_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&tmem_base_smem)), "r"(tmem_cols));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned tmem_base = tmem_base_smem;

    if (warp == 0 && lane == 0) {
        // ---- producer ------------------------------------------------------------------------
        auto load = [&](int s, int kb) {
            mbar_expect_tx(&full_bar[s], (unsigned)(w_tile + x_tile));
            for (int m = 0; m < MT; ++m)
                tma_load_2d(w_tiles + s * w_tile + m * w_half, &map_w, &full_bar[s], kb * MG_BK,
                            w_row + m * MG_BM);
            tma_load_2d(x_tiles + s * x_tile, &map_x, &full_bar[s], kb * MG_BK, row0);
        };
        const int pre = min(kblocks, stages);
        for (int i = 0; i < pre; ++i) load(i, i);
        int issued = pre;
        for (int i = pre; i < kblocks; ++i) {
            const int s = i % stages;
            if (!mbar_wait(&empty_bar[s], ((i / stages) - 1) & 1, &failed)) {
                if (!failed) { failed = 1; atomicCAS(status, 0, 31); }
                break;
            }
            load(s, i);
            issued = i + 1;
        }
        // no copy of this block may still be in flight when it returns
        for (int i = max(0, issued - stages); i < issued; ++i) {
            const int s = i % stages;
            bool ok = false;
            const long long start = clock64();
            while (!ok && clock64() - start < RV_WAIT_CYCLES)
                ok = mbar_try_wait(&full_bar[s], (i / stages) & 1);
            if (!ok && !failed) { failed = 1; atomicCAS(status, 0, 32); }
        }
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer: D float32, A and B bfloat16, both K-major, N = TN, M = 128 --------------
        const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(TN >> 3) << 17) |
                               ((unsigned)(MG_BM >> 4) << 24);
        for (int i = 0; i < kblocks; ++i) {
            const int s = i % stages;
            if (!mbar_wait(&full_bar[s], (i / stages) & 1, &failed)) {
                if (!failed) { failed = 1; atomicCAS(status, 0, 33); }
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const unsigned long long b0 = smem_desc_sw128(x_tiles + s * x_tile);
            for (int m = 0; m < MT; ++m) {
                const unsigned long long a0 = smem_desc_sw128(w_tiles + s * w_tile + m * w_half);
#pragma unroll
                for (int k = 0; k < MG_BK / 16; ++k)
                    tcgen05_mma_f16(tmem_base + (unsigned)(m * TN), a0 + 2 * k, b0 + 2 * k, idesc,
                                    (i | k) != 0);
            }
            tcgen05_commit(&empty_bar[s]);
        }
        tcgen05_commit(&accum_bar);
        if (!failed && !mbar_wait(&accum_bar, 0, &failed) && !failed) {
            failed = 1;
            atomicCAS(status, 0, 34);
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }
    __syncwarp();
    __syncthreads();          // the accumulator is complete, `failed` is final, copies are drained
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const bool good = !failed;
    // The accumulator [128 rows of W x TN tokens] leaves through shared memory (the ring is free:
    // every MMA that read it is done), turned to [token][column], so that the rows of the output
    // are written in 16-byte pieces.  With SWIGLU a lane and its neighbour hold gate and up of
    // one column, and half as many columns leave.
    constexpr int CW = SWIGLU ? MG_BM / 2 : MG_BM;            // columns of the output per tile of W
    constexpr int SW = CW + 8;                                // a staged row: padded against bank conflicts
    bf16* stage_out = (bf16*)base;                            // [TN][SW]
    const int n_local = warp * 32 + lane;
    const int out_cols = SWIGLU ? (n_out >> 1) : n_out;       // a multiple of 8
    constexpr int CPR = CW / 8;                               // 16-byte pieces per row
    for (int m = 0; m < MT; ++m) {
        if (m > 0) __syncthreads();                           // the staged tile has left
        for (int c = 0; c < TN; c += 16) {
            unsigned r[16];
            tmem_load_16(tmem_base + ((unsigned)(warp * 32) << 16) + (unsigned)(m * TN + c), r);
            if (SWIGLU) {
                // An even lane holds the gate sums of its column, its neighbour the up sums.  For
                // a pair of tokens the two lanes swap one value each way, so that the even lane
                // has token j's pair and the odd lane token j + 1's: half the arithmetic a lane.
                // The quotient is rounded to bfloat16, so the fast exponential and division do.
                const bool odd = lane & 1;
#pragma unroll
                for (int j = 0; j < 16; j += 2) {
                    const float mine0 = good ? __uint_as_float(r[j]) : 0.f;
                    const float mine1 = good ? __uint_as_float(r[j + 1]) : 0.f;
                    const float got = __shfl_xor_sync(0xffffffffu, odd ? mine0 : mine1, 1);
                    const float g = odd ? got : mine0;         // odd: the gate of token j + 1
                    const float u = odd ? mine1 : got;         // even: the up value of token j
                    float res;
                    if (ACT == 2) {
                        const float gc = fminf(g, limit), uc = fminf(fmaxf(u, -limit), limit);
                        res = __fdividef(gc, 1.f + __expf(-alpha * gc)) * (uc + 1.f);
                    } else {
                        res = __fdividef(g, 1.f + __expf(-g)) * u;
                    }
                    stage_out[(c + j + (odd ? 1 : 0)) * SW + (n_local >> 1)] =
                        __float2bfloat16_rn(res);
                }
            } else {
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    float v = good ? __uint_as_float(r[j]) : 0.f;
                    if (ACT == 3) {
                        v = fmaxf(v, 0.f);
                        v *= v;
                    }
                    stage_out[(c + j) * SW + n_local] = __float2bfloat16_rn(v);
                }
            }
        }
        __syncthreads();
        for (int idx = tid; idx < TN * CPR; idx += 128) {
            const int t = idx / CPR, ch = idx - t * CPR;
            const int col = (tile * MT + m) * CW + ch * 8;
            if (col < out_cols)
                *(uint4*)(out + (size_t)(row0 + t) * out_cols + col) =
                    *(const uint4*)(stage_out + t * SW + ch * 8);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                     "r"(tmem_cols));
    }
}

// Rows of the sorted layout for `pairs` (token, expert) pairs over E experts in tiles of TN.
extern "C" long long rv_moe_grouped_rows(int pairs, int E, int TN) {
    return ((long long)(pairs + TN - 1) / TN + E) * TN;
}

extern "C" int rv_moe_grouped_init() {
    cudaError_t e = cudaFuncSetAttribute(moe_grouped_kernel<0>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, MG_SMEM_MAX);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(moe_grouped_kernel<1>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, MG_SMEM_MAX);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(moe_grouped_kernel<2>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, MG_SMEM_MAX);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(moe_grouped_kernel<3>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, MG_SMEM_MAX);
    if (e != cudaSuccess) RV_FAIL("moe_grouped: %s", cudaGetErrorString(e));
    if (!encode_fn()) RV_FAIL("moe_grouped: cuTensorMapEncodeTiled is not available in this driver");
    return 0;
}

static int grouped_product(const void* xs, const void* w, void* out, int* status, const int* tile_expert,
                           const int* tile_row0, const int* n_tiles, long long rows, int E, int n_out,
                           int K, int TN, int max_tiles, int act, float limit, float alpha,
                           cudaStream_t stream) {
    CUtensorMap map_w, map_x;
    if (make_map(&map_w, w, (long long)E * n_out, K, MG_BM)) return 1;
    if (make_map(&map_x, xs, rows, K, TN)) return 1;
    const int kblocks = (K + MG_BK - 1) / MG_BK;
    // two tiles of W a block where there are many tokens an expert and rows of W enough
    // (RVLLM_MOE_MT=1 or 2 forces it)
    static int forced_mt = getenv("RVLLM_MOE_MT") ? atoi(getenv("RVLLM_MOE_MT")) : 0;
    int MT = (TN >= 128 && n_out >= 4 * MG_BM) ? 2 : 1;
    if (forced_mt == 1 || forced_mt == 2) MT = forced_mt;
    static int smem_limit = getenv("RVLLM_MOE_SMEM_KB") ? atoi(getenv("RVLLM_MOE_SMEM_KB")) * 1024 : MG_SMEM_LIMIT;
    const int per_stage = MT * MG_BM * MG_BK * 2 + TN * MG_BK * 2;
    int stages = (smem_limit - 1024) / per_stage;
    if (stages > 6) stages = 6;
    if (stages < 2) stages = 2;
    const size_t smem = (size_t)stages * per_stage + 1024;
    dim3 grid((n_out + MT * MG_BM - 1) / (MT * MG_BM), max_tiles);
    if (act == 3)
        rv_launch(moe_grouped_kernel<3>, grid, dim3(128), smem, stream, map_w, map_x, (bf16*)out,
                  status, tile_expert, tile_row0, n_tiles, n_out, kblocks, TN, stages, MT, limit, alpha);
    else if (act == 2)
        rv_launch(moe_grouped_kernel<2>, grid, dim3(128), smem, stream, map_w, map_x, (bf16*)out,
                  status, tile_expert, tile_row0, n_tiles, n_out, kblocks, TN, stages, MT, limit, alpha);
    else if (act == 1)
        rv_launch(moe_grouped_kernel<1>, grid, dim3(128), smem, stream, map_w, map_x, (bf16*)out,
                  status, tile_expert, tile_row0, n_tiles, n_out, kblocks, TN, stages, MT, limit, alpha);
    else
        rv_launch(moe_grouped_kernel<0>, grid, dim3(128), smem, stream, map_w, map_x, (bf16*)out,
                  status, tile_expert, tile_row0, n_tiles, n_out, kblocks, TN, stages, MT, limit, alpha);
    RV_CHECK_LAUNCH("moe_grouped");
    return 0;
}

// Bytes of scratch rv_moe_experts_grouped needs for n_tokens tokens.
extern "C" long long rv_moe_grouped_scratch_bytes(int n_tokens, int top, int E, int W, int F, int TN) {
    const long long pairs = (long long)n_tokens * top;
    const long long rows = rv_moe_grouped_rows((int)pairs, E, TN);
    const long long ints = rows + pairs + 2 * (rows / TN) + 4;
    return ((ints * 4 + 255) & ~255ll) + rows * ((long long)W * 2 + (long long)F * 2 + (long long)W * 2) + 256;
}

// x [n_tokens, W] bf16; gate_up [E, 2F, W] with gate and up rows alternating; down [E, W, F].
// act_mode 2: experts without a gate, `gate_up` is the up matrices [E, F, W] and the activation
// the square of relu.
extern "C" int rv_moe_experts_grouped(const void* x, const int* ids, const float* weights,
                                      const void* gate_up, const void* down, void* out,
                                      void* scratch, long long scratch_bytes, int* status,
                                      int n_tokens, int top, int E, int W, int F, int TN,
                                      int act_mode, float limit, float alpha, const void* addend,
                                      void* stream) {
    if (n_tokens == 0) return 0;
    if (n_tokens < 0 || top < 1 || E < 1 || W < 8 || F < 8 || W % 8 || F % 8)
        RV_FAIL("moe_experts_grouped: widths must be multiples of 8");
    if (TN != 16 && TN != 32 && TN != 64 && TN != 128) RV_FAIL("moe_experts_grouped: bad token tile");
    if (act_mode < 0 || act_mode > 2) RV_FAIL("moe_experts_grouped: unknown activation %d", act_mode);
    if ((uintptr_t)addend & 15) RV_FAIL("moe_experts_grouped: the added rows must be 16-byte aligned");
    if ((size_t)3 * E * sizeof(int) > 48 * 1024) RV_FAIL("moe_experts_grouped: too many experts");
    const long long pairs = (long long)n_tokens * top;
    if (pairs > 0x3fffffffLL) RV_FAIL("moe_experts_grouped: too many rows");
    if (rv_moe_grouped_scratch_bytes(n_tokens, top, E, W, F, TN) > scratch_bytes)
        RV_FAIL("moe_experts_grouped: scratch of %lld bytes is too small", scratch_bytes);
    if (((uintptr_t)scratch & 255) || ((uintptr_t)x & 15) || ((uintptr_t)out & 15))
        RV_FAIL("moe_experts_grouped: buffers must be 16-byte aligned (scratch 256)");
    const long long rows = rv_moe_grouped_rows((int)pairs, E, TN);
    const int max_tiles = (int)(rows / TN);
    if (max_tiles > 65535) RV_FAIL("moe_experts_grouped: too many token tiles");
    int* sorted_token = (int*)scratch;
    int* pair_pos = sorted_token + rows;
    int* tile_expert = pair_pos + pairs;
    int* tile_row0 = tile_expert + max_tiles;
    int* n_tiles = tile_row0 + max_tiles;
    const long long ints = rows + pairs + 2 * (long long)max_tiles + 4;
    bf16* xs = (bf16*)((char*)scratch + ((ints * 4 + 255) & ~255ll));
    bf16* act = xs + rows * W;
    bf16* ys = act + rows * F;
    cudaStream_t s = (cudaStream_t)stream;
    rv_launch(moe_sort_kernel, dim3(1), dim3(1024), (size_t)3 * E * sizeof(int), s, ids, (int)pairs, E,
              top, TN, (int)rows, max_tiles, sorted_token, pair_pos, tile_expert, tile_row0, n_tiles);
    RV_CHECK_LAUNCH("moe_sort");
    rv_launch(moe_gather_kernel, dim3((unsigned)((rows + 7) / 8)), dim3(256), 0, s, (const bf16*)x,
              (const int*)sorted_token, xs, (int)rows, W);
    RV_CHECK_LAUNCH("moe_gather");
    if (grouped_product(xs, gate_up, act, status, tile_expert, tile_row0, n_tiles, rows, E,
                        act_mode == 2 ? F : 2 * F, W, TN, max_tiles,
                        act_mode == 2 ? 3 : act_mode == 1 ? 2 : 1, limit, alpha, s))
        return 1;
    if (grouped_product(act, down, ys, status, tile_expert, tile_row0, n_tiles, rows, E, W, F, TN,
                        max_tiles, 0, 0.f, 0.f, s))
        return 1;
    rv_launch(moe_combine_kernel, dim3(n_tokens), dim3(W / 8 < 256 ? ((W / 8 + 31) / 32) * 32 : 256), 0,
              s, (const bf16*)ys, (const int*)pair_pos, weights, (const bf16*)addend, (bf16*)out, top,
              W);
    RV_CHECK_LAUNCH("moe_combine");
    return 0;
}
