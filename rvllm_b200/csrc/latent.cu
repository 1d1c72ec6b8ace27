// Small kernels around an attention over latent rows.
//
//   latent_norm_write   rows [N, row_stride] carry a latent row of `rank` values at column
//                       `offset`; it is RMS-normed (x / sqrt(mean(x^2) + eps) * weight, float32)
//                       and written to the page slot of its token, which is all that the cache
//                       keeps of the token.  One warp per token.
//   sigmoid_gate        x[n, i] <- x[n, i] * sigmoid(rows[n, gate_off + i]): the gate on the
//                       concatenated heads before the output product.  Sigmoid and product are
//                       float32, rounded once.
//   latent_prepare      the same for a layer whose queries pass a latent of their own and whose
//                       tokens leave a turned key part beside the latent row: columns
//                       [q_off, q_off + q_rank) are RMS-normed with their weight into `cq`
//                       [N, q_rank]; columns [kv_off, kv_off + rank) are RMS-normed into the first
//                       `rank` values of the token's page slot; the `rot` columns after them are
//                       turned by the token's position (dimension i with i + rot/2, angle
//                       position * freq[i], float32) into the slot's last `rot` values.
//   rope_heads          x [N, heads * size] in place: in every head the `rot` values from `off` on
//                       are turned the same way.
//   head_gate           x[n, h * size + c] <- x[n, h * size + c] * sigmoid(rows[n, gate_off + h]):
//                       one gate per head.
// Plain references: tests/plain_ops.py latent_norm_write, sigmoid_gate, latent_prepare, rope_heads,
// head_gate.
#include "common.cuh"

template <typename T>
__global__ void latent_norm_write_kernel(const T* __restrict__ rows, int row_stride, int n_tokens,
                                         int offset, int rank, const float* __restrict__ weight,
                                         float eps, const int* __restrict__ slot_mapping,
                                         T* __restrict__ cache) {
    rv_pdl_launch_dependents();
    const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (warp >= n_tokens) return;
    const int t = (int)warp;
    const int slot = slot_mapping[t];
    rv_pdl_wait();
    if (slot < 0) return;
    const T* src = rows + (size_t)t * row_stride + offset;
    float ss = 0.f;
    for (int i = lane; i < rank; i += 32) {
        const float x = rv_load(src + i);
        ss += x * x;
    }
    ss = rv_warp_sum(ss);
    const float rms = sqrtf(ss / (float)rank + eps);
    T* dst = cache + (size_t)slot * rank;
    for (int i = lane; i < rank; i += 32) rv_store(dst + i, rv_load(src + i) / rms * weight[i]);
}

template <typename T>
__global__ void sigmoid_gate_kernel(T* __restrict__ x, int width, const T* __restrict__ rows,
                                    int row_stride, int gate_off, long long total) {
    rv_pdl_prologue();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const long long n = i / width;
    const int c = (int)(i - n * width);
    const float g = rv_load(rows + n * row_stride + gate_off + c);
    rv_store(x + i, rv_load(x + i) / (1.f + expf(-g)));
}

// eight bfloat16 values a thread, 16-byte accesses
__global__ void sigmoid_gate_bf16x8_kernel(__nv_bfloat16* __restrict__ x, int width8,
                                           const __nv_bfloat16* __restrict__ rows, int row_stride,
                                           int gate_off, long long total8) {
    rv_pdl_prologue();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total8) return;
    const long long n = i / width8;
    const int c = (int)(i - n * width8) * 8;
    uint4 xv = *(const uint4*)(x + i * 8);
    const uint4 gv = *(const uint4*)(rows + n * row_stride + gate_off + c);
    __nv_bfloat162* xp = (__nv_bfloat162*)&xv;
    const __nv_bfloat162* gp = (const __nv_bfloat162*)&gv;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float2 a = __bfloat1622float2(xp[j]), g = __bfloat1622float2(gp[j]);
        xp[j] = __floats2bfloat162_rn(a.x / (1.f + expf(-g.x)), a.y / (1.f + expf(-g.y)));
    }
    *(uint4*)(x + i * 8) = xv;
}

extern "C" int rv_latent_norm_write(const void* rows, int dtype, int row_stride, int n_tokens,
                                    int offset, int rank, const float* weight, float eps,
                                    const int* slot_mapping, void* cache, void* stream) {
    if (n_tokens == 0) return 0;
    if (n_tokens < 0 || rank <= 0 || offset < 0 || row_stride < offset + rank)
        RV_FAIL("latent_norm_write: bad sizes");
    if (!weight || !slot_mapping || !cache) RV_FAIL("latent_norm_write: a pointer is missing");
    const long long blocks = ((long long)n_tokens + 3) / 4;
    RV_DISPATCH_DTYPE(dtype, "latent_norm_write",
                      (rv_launch(latent_norm_write_kernel<T>, dim3((int)blocks), dim3(128), 0,
                                 (cudaStream_t)stream, (const T*)rows, row_stride, n_tokens, offset,
                                 rank, weight, eps, slot_mapping, (T*)cache)));
    RV_CHECK_LAUNCH("latent_norm_write");
    return 0;
}

extern "C" int rv_sigmoid_gate(void* x, int dtype, int n, int width, const void* rows,
                               int row_stride, int gate_off, void* stream) {
    if (n == 0) return 0;
    if (n < 0 || width <= 0 || gate_off < 0 || row_stride < gate_off + width)
        RV_FAIL("sigmoid_gate: bad sizes");
    const long long total = (long long)n * width;
    if (dtype == RV_DTYPE_BF16 && width % 8 == 0 && row_stride % 8 == 0 && gate_off % 8 == 0 &&
        ((uintptr_t)x & 15) == 0 && ((uintptr_t)rows & 15) == 0) {
        const long long total8 = total / 8;
        rv_launch(sigmoid_gate_bf16x8_kernel, dim3((unsigned)((total8 + 255) / 256)), dim3(256), 0,
                  (cudaStream_t)stream, (__nv_bfloat16*)x, width / 8, (const __nv_bfloat16*)rows,
                  row_stride, gate_off, total8);
        RV_CHECK_LAUNCH("sigmoid_gate");
        return 0;
    }
    const long long blocks = (total + 255) / 256;
    if (blocks > 0x7fffffffLL) RV_FAIL("sigmoid_gate: too many values");
    RV_DISPATCH_DTYPE(dtype, "sigmoid_gate",
                      (rv_launch(sigmoid_gate_kernel<T>, dim3((int)blocks), dim3(256), 0,
                                 (cudaStream_t)stream, (T*)x, width, (const T*)rows, row_stride,
                                 gate_off, total)));
    RV_CHECK_LAUNCH("sigmoid_gate");
    return 0;
}



// ---------------------------------------------------------------------------------
template <typename T>
__global__ void latent_prepare_kernel(const T* __restrict__ rows, int row_stride, int n_tokens,
                                      int q_off, int q_rank, const float* __restrict__ q_weight,
                                      T* __restrict__ cq, int kv_off, int rank, int rot,
                                      const float* __restrict__ kv_weight, float eps,
                                      const float* __restrict__ freq,
                                      const int* __restrict__ positions,
                                      const int* __restrict__ slot_mapping, T* __restrict__ cache) {
    rv_pdl_launch_dependents();
    const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (warp >= n_tokens) return;
    const int t = (int)warp;
    const int slot = slot_mapping[t];
    const float pos = (float)positions[t];
    rv_pdl_wait();
    const T* row = rows + (size_t)t * row_stride;
    if (q_rank > 0) {
        const T* src = row + q_off;
        float ss = 0.f;
        for (int i = lane; i < q_rank; i += 32) {
            const float x = rv_load(src + i);
            ss += x * x;
        }
        ss = rv_warp_sum(ss);
        const float rms = sqrtf(ss / (float)q_rank + eps);
        T* dst = cq + (size_t)t * q_rank;
        for (int i = lane; i < q_rank; i += 32)
            rv_store(dst + i, rv_load(src + i) / rms * q_weight[i]);
    }
    if (slot < 0) return;
    const T* src = row + kv_off;
    float ss = 0.f;
    for (int i = lane; i < rank; i += 32) {
        const float x = rv_load(src + i);
        ss += x * x;
    }
    ss = rv_warp_sum(ss);
    const float rms = sqrtf(ss / (float)rank + eps);
    T* dst = cache + (size_t)slot * (rank + rot);
    for (int i = lane; i < rank; i += 32) rv_store(dst + i, rv_load(src + i) / rms * kv_weight[i]);
    const int half = rot >> 1;
    for (int i = lane; i < half; i += 32) {
        float sn, cs;
        sincosf(pos * freq[i], &sn, &cs);
        const float u = rv_load(src + rank + i), v = rv_load(src + rank + half + i);
        rv_store(dst + rank + i, u * cs - v * sn);
        rv_store(dst + rank + half + i, v * cs + u * sn);
    }
}

template <typename T>
__global__ void rope_heads_kernel(T* __restrict__ x, int row_stride, int heads, int size, int off,
                                  int half, const float* __restrict__ freq,
                                  const int* __restrict__ positions, long long total) {
    rv_pdl_launch_dependents();
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int i = (int)(idx % half);
    const long long th = idx / half;
    const int h = (int)(th % heads);
    const long long t = th / heads;
    const float ang = (float)positions[t] * freq[i];
    rv_pdl_wait();
    float sn, cs;
    sincosf(ang, &sn, &cs);
    T* p = x + t * row_stride + (size_t)h * size + off;
    const float u = rv_load(p + i), v = rv_load(p + half + i);
    rv_store(p + i, u * cs - v * sn);
    rv_store(p + half + i, v * cs + u * sn);
}

template <typename T>
__global__ void head_gate_kernel(T* __restrict__ x, int width, int size, const T* __restrict__ rows,
                                 int row_stride, int gate_off, long long total) {
    rv_pdl_prologue();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const long long n = i / width;
    const int h = (int)(i - n * width) / size;
    const float g = rv_load(rows + n * row_stride + gate_off + h);
    rv_store(x + i, rv_load(x + i) / (1.f + expf(-g)));
}

extern "C" int rv_latent_prepare(const void* rows, int dtype, int row_stride, int n_tokens, int q_off,
                                 int q_rank, const float* q_weight, void* cq, int kv_off, int rank,
                                 int rot, const float* kv_weight, float eps, const float* freq,
                                 const int* positions, const int* slot_mapping, void* cache,
                                 void* stream) {
    if (n_tokens == 0) return 0;
    if (n_tokens < 0 || rank <= 0 || rot < 0 || rot % 2 || q_rank < 0 || q_off < 0 || kv_off < 0 ||
        row_stride < kv_off + rank + rot || row_stride < q_off + q_rank)
        RV_FAIL("latent_prepare: bad sizes");
    if (!kv_weight || !slot_mapping || !cache || !positions || (rot && !freq) ||
        (q_rank && (!q_weight || !cq)))
        RV_FAIL("latent_prepare: a pointer is missing");
    const long long blocks = ((long long)n_tokens + 3) / 4;
    RV_DISPATCH_DTYPE(dtype, "latent_prepare",
                      (rv_launch(latent_prepare_kernel<T>, dim3((int)blocks), dim3(128), 0,
                                 (cudaStream_t)stream, (const T*)rows, row_stride, n_tokens, q_off,
                                 q_rank, q_weight, (T*)cq, kv_off, rank, rot, kv_weight, eps, freq,
                                 positions, slot_mapping, (T*)cache)));
    RV_CHECK_LAUNCH("latent_prepare");
    return 0;
}

extern "C" int rv_rope_heads(void* x, int dtype, int row_stride, int n_tokens, int heads, int size,
                             int off, int rot, const float* freq, const int* positions,
                             void* stream) {
    if (n_tokens == 0 || rot == 0) return 0;
    if (n_tokens < 0 || heads <= 0 || size <= 0 || off < 0 || rot < 0 || rot % 2 || off + rot > size ||
        row_stride < heads * size)
        RV_FAIL("rope_heads: bad sizes");
    if (!freq || !positions) RV_FAIL("rope_heads: a pointer is missing");
    const long long total = (long long)n_tokens * heads * (rot / 2);
    const long long blocks = (total + 255) / 256;
    if (blocks > 0x7fffffffLL) RV_FAIL("rope_heads: too many values");
    RV_DISPATCH_DTYPE(dtype, "rope_heads",
                      (rv_launch(rope_heads_kernel<T>, dim3((int)blocks), dim3(256), 0,
                                 (cudaStream_t)stream, (T*)x, row_stride, heads, size, off, rot / 2,
                                 freq, positions, total)));
    RV_CHECK_LAUNCH("rope_heads");
    return 0;
}

// eight bfloat16 values a thread (all of one head), 16-byte accesses
__global__ void head_gate_bf16x8_kernel(__nv_bfloat16* __restrict__ x, int width8, int size8,
                                        const __nv_bfloat16* __restrict__ rows, int row_stride,
                                        int gate_off, long long total8) {
    rv_pdl_prologue();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total8) return;
    const long long n = i / width8;
    const int h = (int)(i - n * width8) / size8;
    const float den = 1.f + expf(-__bfloat162float(rows[n * row_stride + gate_off + h]));
    uint4 xv = *(const uint4*)(x + i * 8);
    __nv_bfloat162* xp = (__nv_bfloat162*)&xv;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float2 a = __bfloat1622float2(xp[j]);
        xp[j] = __floats2bfloat162_rn(a.x / den, a.y / den);
    }
    *(uint4*)(x + i * 8) = xv;
}

extern "C" int rv_head_gate(void* x, int dtype, int n, int heads, int size, const void* rows,
                            int row_stride, int gate_off, void* stream) {
    if (n == 0) return 0;
    if (n < 0 || heads <= 0 || size <= 0 || gate_off < 0 || row_stride < gate_off + heads)
        RV_FAIL("head_gate: bad sizes");
    const long long total = (long long)n * heads * size;
    if (dtype == RV_DTYPE_BF16 && size % 8 == 0 && ((uintptr_t)x & 15) == 0) {
        const long long total8 = total / 8;
        rv_launch(head_gate_bf16x8_kernel, dim3((unsigned)((total8 + 255) / 256)), dim3(256), 0,
                  (cudaStream_t)stream, (__nv_bfloat16*)x, heads * size / 8, size / 8,
                  (const __nv_bfloat16*)rows, row_stride, gate_off, total8);
        RV_CHECK_LAUNCH("head_gate");
        return 0;
    }
    const long long blocks = (total + 255) / 256;
    if (blocks > 0x7fffffffLL) RV_FAIL("head_gate: too many values");
    RV_DISPATCH_DTYPE(dtype, "head_gate",
                      (rv_launch(head_gate_kernel<T>, dim3((int)blocks), dim3(256), 0,
                                 (cudaStream_t)stream, (T*)x, heads * size, size, (const T*)rows,
                                 row_stride, gate_off, total)));
    RV_CHECK_LAUNCH("head_gate");
    return 0;
}
