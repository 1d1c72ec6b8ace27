// Activations of the dense feed-forward, element by element.
//   xIELU with two learned numbers p, q:
//     z > 0 :  softplus(p) z^2 + z/2
//     z <= 0:  (1/2 + softplus(q)) (e^z - 1 - z) + z/2
//   relu squared: max(z, 0)^2 (at the end of the file).
// Arithmetic in float32 whatever the storage type.  Plain reference: tests/plain_ops.py xielu.
#include "common.cuh"

__device__ __forceinline__ float rv_softplus(float a) { return a > 20.f ? a : log1pf(expf(a)); }

__device__ __forceinline__ float rv_xielu(float z, float ap, float an) {
    return z > 0.f ? ap * z * z + 0.5f * z : an * (expm1f(z) - z) + 0.5f * z;
}

template <typename T>
__global__ void xielu_kernel(const T* __restrict__ in, const float* __restrict__ act,
                             T* __restrict__ out, size_t total) {
    rv_pdl_launch_dependents();
    const float ap = rv_softplus(act[0]), an = 0.5f + rv_softplus(act[1]);
    rv_pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (size_t)gridDim.x * blockDim.x)
        rv_store(out + i, rv_xielu(rv_load(in + i), ap, an));
}

// For results that are rounded to bfloat16: e^z - 1 - z without the library's expm1f.  Below
// -1/2 the difference e^z - 1 loses nothing; above, the series z^2/2 + ... + z^8/8! (its first
// missing term is below 2^-27 there).  Both sides are evaluated, so a warp does not diverge.
__device__ __forceinline__ float rv_xielu_bf16(float z, float ap, float an) {
    const float zn = fminf(z, 0.f);
    float ser = 1.f / 40320.f;
    ser = fmaf(ser, zn, 1.f / 5040.f);
    ser = fmaf(ser, zn, 1.f / 720.f);
    ser = fmaf(ser, zn, 1.f / 120.f);
    ser = fmaf(ser, zn, 1.f / 24.f);
    ser = fmaf(ser, zn, 1.f / 6.f);
    ser = fmaf(ser, zn, 0.5f);
    ser *= zn * zn;
    const float far = __expf(zn) - 1.f - zn;
    const float neg = an * (zn < -0.5f ? far : ser);
    return fmaf(0.5f, z, z > 0.f ? ap * z * z : neg);
}

// bfloat16, eight values per 16-byte access
__global__ void xielu_bf16x8_kernel(const uint4* __restrict__ in, const float* __restrict__ act,
                                    uint4* __restrict__ out, size_t total8) {
    rv_pdl_launch_dependents();
    const float ap = rv_softplus(act[0]), an = 0.5f + rv_softplus(act[1]);
    rv_pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total8;
         i += (size_t)gridDim.x * blockDim.x) {
        const uint4 raw = in[i];
        uint4 o4;
        const __nv_bfloat162* x2 = (const __nv_bfloat162*)&raw;
        __nv_bfloat162* o2 = (__nv_bfloat162*)&o4;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 z = __bfloat1622float2(x2[k]);
            o2[k] = __floats2bfloat162_rn(rv_xielu_bf16(z.x, ap, an), rv_xielu_bf16(z.y, ap, an));
        }
        out[i] = o4;
    }
}

extern "C" int rv_xielu_act(const void* in, const float* act, void* out, int dtype, int n_rows,
                            int width, void* stream) {
    if (n_rows == 0) return 0;
    if (n_rows < 0 || width <= 0) RV_FAIL("xielu: bad sizes");
    const size_t total = (size_t)n_rows * width;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == RV_DTYPE_BF16 && total % 8 == 0 && (uintptr_t)in % 16 == 0 && (uintptr_t)out % 16 == 0) {
        const size_t total8 = total / 8;
        const int blocks = (int)((total8 + 255) / 256 < 148 * 16 ? (total8 + 255) / 256 : 148 * 16);
        rv_launch(xielu_bf16x8_kernel, dim3(blocks), dim3(256), 0, s, (const uint4*)in, act,
                  (uint4*)out, total8);
    } else {
        const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
        RV_DISPATCH_DTYPE(dtype, "xielu",
                          (rv_launch(xielu_kernel<T>, dim3(blocks), dim3(256), 0, s, (const T*)in, act,
                                     (T*)out, total)));
    }
    RV_CHECK_LAUNCH("xielu");
    return 0;
}

// ---------------------------------------------------------------------------------
// The clamped gated activation of a feed-forward whose gate and up rows come out of one product
// as [N, 2F] (gate values, then up values), with an optional bias [2F] added first:
//   g = min(gate, limit);  u = clamp(up, -limit, limit);  out = g * sigmoid(alpha g) * (u + 1)
// Arithmetic in float32.  Plain reference: tests/plain_ops.py glu_clamp.
template <typename T>
__global__ void glu_clamp_kernel(const T* __restrict__ in, const float* __restrict__ bias,
                                 T* __restrict__ out, size_t total, int F, float limit,
                                 float alpha) {
    rv_pdl_prologue();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (size_t)gridDim.x * blockDim.x) {
        const size_t row = i / F;
        const int f = (int)(i - row * F);
        float g = rv_load(in + row * 2 * F + f), u = rv_load(in + row * 2 * F + F + f);
        if (bias) {
            g += bias[f];
            u += bias[F + f];
        }
        g = fminf(g, limit);
        u = fminf(fmaxf(u, -limit), limit);
        rv_store(out + i, g / (1.f + expf(-alpha * g)) * (u + 1.f));
    }
}

extern "C" int rv_glu_clamp(const void* in, const float* bias, void* out, int dtype, int n_rows,
                            int F, float limit, float alpha, void* stream) {
    if (n_rows == 0) return 0;
    if (n_rows < 0 || F <= 0) RV_FAIL("glu_clamp: bad sizes");
    const size_t total = (size_t)n_rows * F;
    const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    RV_DISPATCH_DTYPE(dtype, "glu_clamp",
                      (rv_launch(glu_clamp_kernel<T>, dim3(blocks), dim3(256), 0, (cudaStream_t)stream,
                                 (const T*)in, bias, (T*)out, total, F, limit, alpha)));
    RV_CHECK_LAUNCH("glu_clamp");
    return 0;
}

// ---------------------------------------------------------------------------------
// The square of relu: out = max(z, 0)^2.  Arithmetic in float32.  Plain reference:
// tests/plain_ops.py relu2.
template <typename T>
__global__ void relu2_kernel(const T* __restrict__ in, T* __restrict__ out, size_t total) {
    rv_pdl_prologue();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (size_t)gridDim.x * blockDim.x) {
        const float z = fmaxf(rv_load(in + i), 0.f);
        rv_store(out + i, z * z);
    }
}

// bfloat16, eight values per 16-byte access
__global__ void relu2_bf16x8_kernel(const uint4* __restrict__ in, uint4* __restrict__ out,
                                    size_t total8) {
    rv_pdl_prologue();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total8;
         i += (size_t)gridDim.x * blockDim.x) {
        const uint4 raw = in[i];
        uint4 o4;
        const __nv_bfloat162* x2 = (const __nv_bfloat162*)&raw;
        __nv_bfloat162* o2 = (__nv_bfloat162*)&o4;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            float2 z = __bfloat1622float2(x2[k]);
            z.x = fmaxf(z.x, 0.f);
            z.y = fmaxf(z.y, 0.f);
            o2[k] = __floats2bfloat162_rn(z.x * z.x, z.y * z.y);
        }
        out[i] = o4;
    }
}

extern "C" int rv_relu2(const void* in, void* out, int dtype, int n_rows, int width, void* stream) {
    if (n_rows == 0) return 0;
    if (n_rows < 0 || width <= 0) RV_FAIL("relu2: bad sizes");
    const size_t total = (size_t)n_rows * width;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == RV_DTYPE_BF16 && total % 8 == 0 && (uintptr_t)in % 16 == 0 && (uintptr_t)out % 16 == 0) {
        const size_t total8 = total / 8;
        const int blocks = (int)((total8 + 255) / 256 < 148 * 16 ? (total8 + 255) / 256 : 148 * 16);
        rv_launch(relu2_bf16x8_kernel, dim3(blocks), dim3(256), 0, s, (const uint4*)in, (uint4*)out,
                  total8);
    } else {
        const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
        RV_DISPATCH_DTYPE(dtype, "relu2",
                          (rv_launch(relu2_kernel<T>, dim3(blocks), dim3(256), 0, s, (const T*)in,
                                     (T*)out, total)));
    }
    RV_CHECK_LAUNCH("relu2");
    return 0;
}
