// Hyper-connections: the residual is S parallel streams x_1 .. x_S per token, [N, S, W] float32.
// One kernel does what lies between two sub-layers:
//
//   1. the write-back of the sub-layer output y that is still pending, with that sub-layer's
//      mixing matrix M [S, S] (indexed [from, to]) and output weights b [S]:
//          x'_t = sum_s M[s, t] x_s + b[t] y          (all streams at once, from the old ones)
//   2. the read-in of the next sub-layer with its weights a [S]:  u = sum_t a[t] x'_t
//   3. RMSNorm of u:  out = u / sqrt(mean(u^2) + eps) * w
//
// Without a pending output step 1 is the identity.  `src` may be the embedding rows [N, W]
// read with a stream stride of 0 (every stream starts as the embedding output); `dst`, if
// given, receives x' as [N, S, W] (it may be `src`).  With a row list only those rows are read
// and nothing is written back (the model's last norm, where `a` absent means all ones: the sum
// of the streams).  One block per row; everything is float32, `out` the compute type.
// Plain reference: tests/plain_ops.py hyper_norm.
#include "common.cuh"

#define RV_HC_MAX_STREAMS 16

template <typename TD, typename TO>
__global__ void hyper_norm_kernel(const float* __restrict__ src, long long src_row_stride,
                                  int src_stream_stride, float* __restrict__ dst,
                                  const TD* __restrict__ delta, const float* __restrict__ mix,
                                  const float* __restrict__ out_w, const float* __restrict__ in_w,
                                  const float* __restrict__ weight, TO* __restrict__ out,
                                  const int* __restrict__ rows, int S, int W, float eps) {
    rv_pdl_launch_dependents();
    extern __shared__ float smem[];
    float* u_row = smem;                       // [W]
    float* red = smem + W;                     // [33]
    float* m_s = red + 33;                     // [S * S]
    float* b_s = m_s + S * S;                  // [S]
    float* a_s = b_s + S;                      // [S]
    for (int i = threadIdx.x; i < S * S; i += blockDim.x) m_s[i] = mix ? mix[i] : (i / S == i % S ? 1.f : 0.f);
    for (int i = threadIdx.x; i < S; i += blockDim.x) {
        b_s[i] = out_w ? out_w[i] : 0.f;
        a_s[i] = in_w ? in_w[i] : 1.f;
    }
    const int row = rows ? rows[blockIdx.x] : blockIdx.x;
    rv_pdl_wait();
    __syncthreads();
    const float* x_row = src + (size_t)row * src_row_stride;
    float ss = 0.f;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        float x[RV_HC_MAX_STREAMS];
#pragma unroll
        for (int s = 0; s < RV_HC_MAX_STREAMS; ++s)
            if (s < S) x[s] = x_row[(size_t)s * src_stream_stride + c];
        float u = 0.f;
        if (delta) {
            const float y = rv_load(delta + (size_t)row * W + c);
            for (int t = 0; t < S; ++t) {
                float v = 0.f;
#pragma unroll
                for (int s = 0; s < RV_HC_MAX_STREAMS; ++s)
                    if (s < S) v += m_s[s * S + t] * x[s];
                v += b_s[t] * y;
                if (dst) dst[((size_t)row * S + t) * W + c] = v;
                u += a_s[t] * v;
            }
        } else {
#pragma unroll
            for (int s = 0; s < RV_HC_MAX_STREAMS; ++s)
                if (s < S) {
                    if (dst && dst + ((size_t)row * S + s) * W + c != x_row + (size_t)s * src_stream_stride + c)
                        dst[((size_t)row * S + s) * W + c] = x[s];
                    u += a_s[s] * x[s];
                }
        }
        u_row[c] = u;
        ss += u * u;
    }
    ss = rv_block_sum(ss, red);
    const float denom = sqrtf(ss / (float)W + eps);
    for (int c = threadIdx.x; c < W; c += blockDim.x)
        rv_store(out + (size_t)blockIdx.x * W + c, u_row[c] / denom * weight[c]);
}

// The same for widths that four divides and up to eight streams, the number of streams known at
// compile time: a thread takes four neighbouring columns (16-byte accesses), the weights sit in
// registers, and nothing is predicated.
__device__ __forceinline__ float4 hc_load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 hc_load4(const __nv_bfloat16* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
    const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    return make_float4(__low2float(lo), __high2float(lo), __low2float(hi), __high2float(hi));
}
__device__ __forceinline__ void hc_store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void hc_store4(__nv_bfloat16* p, float4 v) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 raw;
    raw.x = *reinterpret_cast<const unsigned*>(&lo);
    raw.y = *reinterpret_cast<const unsigned*>(&hi);
    *reinterpret_cast<uint2*>(p) = raw;
}

template <int S, typename TD, typename TO>
__global__ void hyper_norm_vec_kernel(const float* __restrict__ src, long long src_row_stride,
                                      int src_stream_stride, float* __restrict__ dst,
                                      const TD* __restrict__ delta, const float* __restrict__ mix,
                                      const float* __restrict__ out_w, const float* __restrict__ in_w,
                                      const float* __restrict__ weight, TO* __restrict__ out,
                                      const int* __restrict__ rows, int W, float eps) {
    rv_pdl_launch_dependents();
    extern __shared__ __align__(16) float smem[];
    float* u_row = smem;                       // [W]
    float* red = smem + W;                     // [33]
    float m[S][S], b[S], a[S];
#pragma unroll
    for (int i = 0; i < S; ++i) {
#pragma unroll
        for (int j = 0; j < S; ++j) m[i][j] = mix ? mix[i * S + j] : (i == j ? 1.f : 0.f);
        b[i] = out_w ? out_w[i] : 0.f;
        a[i] = in_w ? in_w[i] : 1.f;
    }
    const int row = rows ? rows[blockIdx.x] : blockIdx.x;
    rv_pdl_wait();
    const float* x_row = src + (size_t)row * src_row_stride;
    const bool in_place = dst && dst + (size_t)row * S * W == x_row && src_stream_stride == W;
    float ss = 0.f;
    for (int c = 4 * threadIdx.x; c < W; c += 4 * blockDim.x) {
        float4 x[S];
#pragma unroll
        for (int s = 0; s < S; ++s) x[s] = hc_load4(x_row + (size_t)s * src_stream_stride + c);
        float4 u = make_float4(0.f, 0.f, 0.f, 0.f);
        if (delta) {
            const float4 y = hc_load4(delta + (size_t)row * W + c);
#pragma unroll
            for (int t = 0; t < S; ++t) {
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int s = 0; s < S; ++s) {
                    v.x += m[s][t] * x[s].x; v.y += m[s][t] * x[s].y;
                    v.z += m[s][t] * x[s].z; v.w += m[s][t] * x[s].w;
                }
                v.x += b[t] * y.x; v.y += b[t] * y.y; v.z += b[t] * y.z; v.w += b[t] * y.w;
                if (dst) hc_store4(dst + ((size_t)row * S + t) * W + c, v);
                u.x += a[t] * v.x; u.y += a[t] * v.y; u.z += a[t] * v.z; u.w += a[t] * v.w;
            }
        } else {
#pragma unroll
            for (int s = 0; s < S; ++s) {
                if (dst && !in_place) hc_store4(dst + ((size_t)row * S + s) * W + c, x[s]);
                u.x += a[s] * x[s].x; u.y += a[s] * x[s].y; u.z += a[s] * x[s].z; u.w += a[s] * x[s].w;
            }
        }
        hc_store4(u_row + c, u);
        ss += u.x * u.x + u.y * u.y + u.z * u.z + u.w * u.w;
    }
    ss = rv_block_sum(ss, red);
    const float denom = sqrtf(ss / (float)W + eps);
    for (int c = 4 * threadIdx.x; c < W; c += 4 * blockDim.x) {
        const float4 u = hc_load4(u_row + c), w = hc_load4(weight + c);
        hc_store4(out + (size_t)blockIdx.x * W + c,
                  make_float4(u.x / denom * w.x, u.y / denom * w.y, u.z / denom * w.z, u.w / denom * w.w));
    }
}

template <typename TD, typename TO>
static bool hc_launch_vec(int S, dim3 grid, dim3 block, size_t smem, cudaStream_t s, const float* src,
                          long long row_stride, int stream_stride, float* dst, const void* delta,
                          const float* mix, const float* out_w, const float* in_w, const float* weight,
                          void* out, const int* rows, int W, float eps) {
#define RV_HC_CASE(n)                                                                                  \
    case n:                                                                                            \
        if (smem > 48 * 1024)                                                                          \
            cudaFuncSetAttribute(hyper_norm_vec_kernel<n, TD, TO>,                                     \
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);              \
        rv_launch(hyper_norm_vec_kernel<n, TD, TO>, grid, block, smem, s, src, row_stride, stream_stride, \
                  dst, (const TD*)delta, mix, out_w, in_w, weight, (TO*)out, rows, W, eps);            \
        return true;
    switch (S) {
        RV_HC_CASE(1) RV_HC_CASE(2) RV_HC_CASE(3) RV_HC_CASE(4) RV_HC_CASE(5) RV_HC_CASE(6) RV_HC_CASE(7)
        RV_HC_CASE(8)
    }
#undef RV_HC_CASE
    return false;
}

// src [N, W] (src_streams == 1: every stream reads the same row) or [N, S, W]; dst [N, S, W] or
// null; delta [N, W] of type delta_dtype or null (then mix and out_w are not read); rows: int32
// [n_out] or null (then n_out rows 0 .. n_out-1).
extern "C" int rv_hyper_norm(const float* src, int src_streams, float* dst, const void* delta,
                             int delta_dtype, const float* mix, const float* out_w,
                             const float* in_w, const float* weight, void* out, int out_dtype,
                             const int* rows, int n_out, int S, int W, float eps, void* stream) {
    if (n_out == 0) return 0;
    if (n_out < 0 || W <= 0 || S < 1 || S > RV_HC_MAX_STREAMS)
        RV_FAIL("hyper_norm: bad sizes (1 to %d streams)", RV_HC_MAX_STREAMS);
    if (src_streams != 1 && src_streams != S) RV_FAIL("hyper_norm: the source has 1 or S streams");
    if (rows && dst) RV_FAIL("hyper_norm: with a row list nothing is written back");
    if (delta && (!mix || !out_w)) RV_FAIL("hyper_norm: a pending output needs its mixing weights");
    const size_t smem = ((size_t)W + 33 + (size_t)S * S + 2 * S) * sizeof(float);
    if (smem > 200 * 1024) RV_FAIL("hyper_norm: a row of %d values does not fit shared memory", W);
    const int threads = W >= 2048 ? 512 : (W >= 256 ? 256 : 128);
    const long long row_stride = src_streams == 1 ? W : (long long)S * W;
    const int stream_stride = src_streams == 1 ? 0 : W;
    cudaStream_t s = (cudaStream_t)stream;
#define RV_HC_LAUNCH(TD, TO)                                                                     \
    do {                                                                                         \
        if (smem > 48 * 1024)                                                                    \
            cudaFuncSetAttribute(hyper_norm_kernel<TD, TO>,                                      \
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);        \
        rv_launch(hyper_norm_kernel<TD, TO>, dim3(n_out), dim3(threads), smem, s, src, row_stride, \
                  stream_stride, dst, (const TD*)delta, mix, out_w, in_w, weight, (TO*)out, rows, \
                  S, W, eps);                                                                    \
    } while (0)
    const int dd = delta ? delta_dtype : RV_DTYPE_F32;
    if (W % 4 == 0 && S <= 8) {
        const int vthreads = W >= 2048 ? 256 : 128;
        const size_t vsmem = ((size_t)W + 33) * sizeof(float);
        bool done = false;
        if (dd == RV_DTYPE_F32 && out_dtype == RV_DTYPE_F32)
            done = hc_launch_vec<float, float>(S, dim3(n_out), dim3(vthreads), vsmem, s, src, row_stride,
                                               stream_stride, dst, delta, mix, out_w, in_w, weight, out, rows, W, eps);
        else if (dd == RV_DTYPE_F32 && out_dtype == RV_DTYPE_BF16)
            done = hc_launch_vec<float, __nv_bfloat16>(S, dim3(n_out), dim3(vthreads), vsmem, s, src, row_stride,
                                                       stream_stride, dst, delta, mix, out_w, in_w, weight, out, rows, W, eps);
        else if (dd == RV_DTYPE_BF16 && out_dtype == RV_DTYPE_BF16)
            done = hc_launch_vec<__nv_bfloat16, __nv_bfloat16>(S, dim3(n_out), dim3(vthreads), vsmem, s, src, row_stride,
                                                               stream_stride, dst, delta, mix, out_w, in_w, weight, out, rows, W, eps);
        else if (dd == RV_DTYPE_BF16 && out_dtype == RV_DTYPE_F32)
            done = hc_launch_vec<__nv_bfloat16, float>(S, dim3(n_out), dim3(vthreads), vsmem, s, src, row_stride,
                                                       stream_stride, dst, delta, mix, out_w, in_w, weight, out, rows, W, eps);
        if (done) {
            RV_CHECK_LAUNCH("hyper_norm");
            return 0;
        }
    }
    if (dd == RV_DTYPE_F32 && out_dtype == RV_DTYPE_F32) RV_HC_LAUNCH(float, float);
    else if (dd == RV_DTYPE_F32 && out_dtype == RV_DTYPE_BF16) RV_HC_LAUNCH(float, __nv_bfloat16);
    else if (dd == RV_DTYPE_BF16 && out_dtype == RV_DTYPE_BF16) RV_HC_LAUNCH(__nv_bfloat16, __nv_bfloat16);
    else if (dd == RV_DTYPE_BF16 && out_dtype == RV_DTYPE_F32) RV_HC_LAUNCH(__nv_bfloat16, float);
    else RV_FAIL("hyper_norm: unknown dtype codes %d, %d", delta_dtype, out_dtype);
#undef RV_HC_LAUNCH
    RV_CHECK_LAUNCH("hyper_norm");
    return 0;
}
