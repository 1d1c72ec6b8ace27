// What lies between the q|k|v product and attention for a layer whose query and key norms span
// the whole projection, in one kernel, one block per token:
//
//   rows [N, Q + K + V] float32, the product of each token (Q = heads * d, K = kv_heads * d,
//   V = kv_heads * dv), to which `bias` [Q + K + V] is added when given;
//   q <- q / sqrt(mean_{all Q}(q^2) + eps) * wq,  k likewise over all K values with wk
//   (one statistic for the whole projection, before it is split into heads; without wq and
//   wk this step is left out);
//   rotation of q and k: in every head the pair (2i, 2i + 1), i < rot_dims / 2, at position p
//   turns by the angle p * freq[i] (float32): (u, v) -> (u cos - v sin, v cos + u sin); the
//   dimensions from rot_dims on pass;
//   value mixing: v <- (1 - lambda) v + lambda v_first, where v_first [N, V] float32 holds the
//   values an earlier layer made for the same tokens (`v_first_in`, with `lambda` a scalar on
//   the device); a layer that is the source writes its own values to `v_first_out` instead;
//   q goes to q_out [N, Q], k and the mixed v to the cache rows at slot_mapping[n] (none when
//   it is negative), all in the cache's storage type.
// Sums, norms, angles and the mix are float32.  Plain reference: tests/plain_ops.py
// qkv_full_norm_rope_write.
#include "common.cuh"

template <typename T>
__global__ void qkv_full_kernel(const float* __restrict__ rows, const float* __restrict__ bias,
                                const float* __restrict__ wq, const float* __restrict__ wk,
                                float eps, const float* __restrict__ freq, int rot_dims,
                                const int* __restrict__ positions,
                                const int* __restrict__ slot_mapping, T* __restrict__ q_out,
                                T* __restrict__ k_cache, T* __restrict__ v_cache,
                                const float* __restrict__ v_first_in,
                                float* __restrict__ v_first_out, const float* __restrict__ lambda,
                                int Q, int K, int V, int d) {
    rv_pdl_launch_dependents();
    extern __shared__ float smem[];
    float* qk = smem;                         // [Q + K]
    float* red = smem + Q + K;                // [33]
    const int n = blockIdx.x;
    const int pos = positions[n];
    const int slot = slot_mapping[n];
    const float lam = v_first_in ? lambda[0] : 0.f;
    rv_pdl_wait();
    const float* row = rows + (size_t)n * (Q + K + V);
    float sq = 0.f, sk = 0.f;
    for (int e = threadIdx.x; e < Q + K; e += blockDim.x) {
        const float x = row[e] + (bias ? bias[e] : 0.f);
        qk[e] = x;
        if (e < Q) sq += x * x;
        else sk += x * x;
    }
    sq = rv_block_sum(sq, red);
    sk = rv_block_sum(sk, red);
    // without norm weights the projections stay as they are
    const float dq = wq ? sqrtf(sq / (float)Q + eps) : 1.f, dk = wk ? sqrtf(sk / (float)K + eps) : 1.f;
    if ((d & 1) == 0) {
        // heads of even size: a thread takes a pair (2i, 2i + 1), so one division by the head
        // size, one sine and one cosine serve two values
        for (int p = threadIdx.x; p < (Q + K) / 2; p += blockDim.x) {
            const int e = 2 * p;
            const bool is_q = e < Q;
            const int j = (is_q ? e : e - Q) % d;             // place in its head, even
            const float den = is_q ? dq : dk;
            const float* w = is_q ? wq : (wk ? wk - Q : nullptr);
            float a = qk[e], b = qk[e + 1];
            if (w) {
                a = a / den * w[e];
                b = b / den * w[e + 1];
            }
            if (j < rot_dims) {
                const float ang = (float)pos * freq[j >> 1];
                const float c = cosf(ang), sn = sinf(ang);
                const float ra = a * c - b * sn, rb = b * c + a * sn;
                a = ra;
                b = rb;
            }
            if (is_q) {
                rv_store(q_out + (size_t)n * Q + e, a);
                rv_store(q_out + (size_t)n * Q + e + 1, b);
            } else if (slot >= 0) {
                rv_store(k_cache + (size_t)slot * K + (e - Q), a);
                rv_store(k_cache + (size_t)slot * K + (e - Q) + 1, b);
            }
        }
    } else {
        for (int e = threadIdx.x; e < Q + K; e += blockDim.x) {
            const bool is_q = e < Q;
            const int j = (is_q ? e : e - Q) % d;             // place in its head
            const float den = is_q ? dq : dk;
            const float* w = is_q ? wq : (wk ? wk - Q : nullptr);
            float val = w ? qk[e] / den * w[e] : qk[e];
            if (j < rot_dims) {
                const float other = w ? qk[e ^ 1] / den * w[e ^ 1] : qk[e ^ 1];   // heads start at even places
                const float ang = (float)pos * freq[j >> 1];
                const float c = cosf(ang), s = sinf(ang);
                val = (j & 1) ? val * c + other * s : val * c - other * s;
            }
            if (is_q) rv_store(q_out + (size_t)n * Q + e, val);
            else if (slot >= 0) rv_store(k_cache + (size_t)slot * K + (e - Q), val);
        }
    }
    for (int e = threadIdx.x; e < V; e += blockDim.x) {
        float val = row[Q + K + e] + (bias ? bias[Q + K + e] : 0.f);
        if (v_first_out) v_first_out[(size_t)n * V + e] = val;
        if (v_first_in) val = (1.f - lam) * val + lam * v_first_in[(size_t)n * V + e];
        if (slot >= 0) rv_store(v_cache + (size_t)slot * V + e, val);
    }
}

extern "C" int rv_qkv_full_norm_rope_write(const float* rows, const float* bias, const float* wq,
                                           const float* wk, float eps, const float* freq,
                                           int rot_dims, const int* positions,
                                           const int* slot_mapping, void* q_out, void* k_cache,
                                           void* v_cache, int dtype, const float* v_first_in,
                                           float* v_first_out, const float* lambda, int n_tokens,
                                           int num_heads, int num_kv_heads, int head_dim,
                                           int v_head_dim, void* stream) {
    if (n_tokens == 0) return 0;
    if (n_tokens < 0 || num_heads < 1 || num_kv_heads < 1 || head_dim < 1 || v_head_dim < 1)
        RV_FAIL("qkv_full_norm_rope_write: bad sizes");
    if (rot_dims < 0 || rot_dims > head_dim || rot_dims % 2 || (rot_dims > 0 && head_dim % 2))
        RV_FAIL("qkv_full_norm_rope_write: %d turning dimensions do not fit pairs of a head of %d",
                rot_dims, head_dim);
    if (rot_dims > 0 && !freq) RV_FAIL("qkv_full_norm_rope_write: a rotation needs its frequencies");
    if (v_first_in && !lambda) RV_FAIL("qkv_full_norm_rope_write: mixing needs its weight");
    const int Q = num_heads * head_dim, K = num_kv_heads * head_dim, V = num_kv_heads * v_head_dim;
    const size_t smem = ((size_t)Q + K + 33) * sizeof(float);
    if (smem > 200 * 1024) RV_FAIL("qkv_full_norm_rope_write: the projection does not fit shared memory");
    const int threads = Q + K >= 2048 ? 512 : 256;
    RV_DISPATCH_DTYPE(dtype, "qkv_full_norm_rope_write", {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(qkv_full_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)smem);
        rv_launch(qkv_full_kernel<T>, dim3(n_tokens), dim3(threads), smem, (cudaStream_t)stream, rows,
                  bias, wq, wk, eps, freq, rot_dims, positions, slot_mapping, (T*)q_out, (T*)k_cache,
                  (T*)v_cache, v_first_in, v_first_out, lambda, Q, K, V, head_dim);
    });
    RV_CHECK_LAUNCH("qkv_full_norm_rope_write");
    return 0;
}
