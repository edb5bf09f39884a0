// Attention over a cached latent: the two kernels around the paged attention kernels.
//
// A latent-attention mixer keeps ONE row c_t of `rank` values per position (c_t = rmsnorm(Wd h_t) * gain) and makes every
// head's keys and values from it: k = Wuk c, v = Wuv c. With q' = Wuk_h^T q_h the score q_h . k_j equals q' . c_j, and
// sum_j p_j v_j = Wuv_h (sum_j p_j c_j): attention with one key/value head of width `rank` whose keys and values are the
// same cached rows, between two small products per head. The attention itself is the engine's paged attention
// (kv_heads = 1, head_dim = rank). Here:
//
//   latent_norm_store   RMSNorm of the down-projected rows (float32 arithmetic) and their write into the paged cache
//   gemm_heads          out[r, h, :] = f(r, h) * W[h] a[r, h, :] for every head h at once (W [heads, N, K]), on the CUDA
//                       cores with one float32 accumulator per element in ascending k, so that a row's result does not
//                       depend on the batch; f = alpha, or alpha * sigmoid(gate[r, h]) (the mixer's output gate)
#include "common.cuh"

namespace {

template <typename T>
__global__ void __launch_bounds__(128)
latent_norm_store_kernel(const T* __restrict__ src, int ld, VecRef gain, const int* __restrict__ slots, T* __restrict__ cache,
                         int rank, float eps, long long cache_rows) {
    __shared__ float scratch[33];
    pdl_wait();
    pdl_trigger();
    const int r = blockIdx.x;
    const T* row = src + (size_t)r * ld;
    float ss = 0.f;
    for (int i = threadIdx.x; i < rank; i += blockDim.x) {
        const float v = to_float(row[i]);
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.f / sqrtf(ss / (float)rank + eps);
    const int slot = slots[r];
    if (!jllm_in_bounds(slot, cache_rows, BOUNDS_SLOT)) return;
    T* dst = cache + (size_t)slot * rank;
    for (int i = threadIdx.x; i < rank; i += blockDim.x)
        dst[i] = from_float<T>(__fmul_rn(__fmul_rn(to_float(row[i]), inv), gain[i]));
}

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

template <typename T>
__global__ void __launch_bounds__(256)
gemm_heads_kernel(const T* __restrict__ a, int lda, const T* __restrict__ w, T* __restrict__ out, int ldo,
                  const T* __restrict__ gate, int ld_gate, float alpha, int M, int N, int K) {
    __shared__ float as[BK][BM + 4];
    __shared__ float ws[BK][BN + 4];
    pdl_wait();
    pdl_trigger();
    const int tid = threadIdx.x, h = blockIdx.z;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int tx = tid % 16, ty = tid / 16;
    const T* ah = a + (size_t)h * K;
    const T* wh = w + (size_t)h * N * K;
    float acc[TM][TN] = {};
    const int lr = tid / 4, lk = (tid % 4) * 4;
    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int k = k0 + lk + j;
            const int m = m0 + lr, n = n0 + lr;
            as[lk + j][lr] = (m < M && k < K) ? to_float(ah[(size_t)m * lda + k]) : 0.f;
            ws[lk + j][lr] = (n < N && k < K) ? to_float(wh[(size_t)n * K + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float av[TM], wv[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) av[i] = as[k][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) wv[j] = ws[k][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int m = m0 + ty * TM + i;
        if (m >= M) continue;
        float f = alpha;
        if (gate != nullptr) {
            const float gv = to_float(gate[(size_t)m * ld_gate + h]);
            f = __fmul_rn(alpha, 1.f / (1.f + expf(-gv)));
        }
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int n = n0 + tx * TN + j;
            if (n < N) out[(size_t)m * ldo + (size_t)h * N + n] = from_float<T>(__fmul_rn(acc[i][j], f));
        }
    }
}

}  // namespace

JLLM_BOUNDS_READER(latent_attention)

// src [rows, ld] (the down-projected rows), cache [cache_rows, rank] (a page pool seen as rows: slot = page * page_size
// + offset), both of type `dtype`.
JLLM_EXPORT int jllm_latent_norm_store(const void* src, int dtype, int ld, const void* gain, int gain_dtype,
                                       const int* slots, void* cache, long long cache_rows, int rows, int rank, float eps,
                                       cudaStream_t stream) {
    JLLM_REQUIRE(rows >= 0 && rank > 0 && ld >= rank, "latent_norm_store: rows=%d rank=%d ld=%d", rows, rank, ld);
    if (rows == 0) return JLLM_OK;
    const VecRef g{gain, gain_dtype};
    if (dtype == JLLM_F32)
        jllm_launch(latent_norm_store_kernel<float>, dim3(rows), dim3(128), 0, stream, LAUNCH_DEPENDENT, (const float*)src,
                    ld, g, slots, (float*)cache, rank, eps, cache_rows);
    else
        jllm_launch(latent_norm_store_kernel<__nv_bfloat16>, dim3(rows), dim3(128), 0, stream, LAUNCH_DEPENDENT,
                    (const __nv_bfloat16*)src, ld, g, slots, (__nv_bfloat16*)cache, rank, eps, cache_rows);
    return jllm_check_launch("latent_norm_store");
}

// a [M, lda] with head h's K values at column h * K; w [heads, N, K]; out [M, ldo] with head h's N values at h * N;
// gate (or null) [M, ld_gate] with head h's gate at column h.
JLLM_EXPORT int jllm_gemm_heads(const void* a, int dtype, int lda, const void* w, void* out, int ldo, const void* gate,
                                int ld_gate, float alpha, int M, int heads, int N, int K, cudaStream_t stream) {
    JLLM_REQUIRE(M >= 0 && heads > 0 && N > 0 && K > 0, "gemm_heads: M=%d heads=%d N=%d K=%d", M, heads, N, K);
    JLLM_REQUIRE(lda >= heads * K && ldo >= heads * N && heads <= 65535 && (M + BM - 1) / BM <= 65535,
                 "gemm_heads: lda=%d ldo=%d for %d heads of K=%d, N=%d", lda, ldo, heads, K, N);
    if (M == 0) return JLLM_OK;
    const dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM, heads);
    if (dtype == JLLM_F32)
        jllm_launch(gemm_heads_kernel<float>, grid, dim3(256), 0, stream, LAUNCH_DEPENDENT, (const float*)a, lda,
                    (const float*)w, (float*)out, ldo, (const float*)gate, ld_gate, alpha, M, N, K);
    else
        jllm_launch(gemm_heads_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, LAUNCH_DEPENDENT,
                    (const __nv_bfloat16*)a, lda, (const __nv_bfloat16*)w, (__nv_bfloat16*)out, ldo,
                    (const __nv_bfloat16*)gate, ld_gate, alpha, M, N, K);
    return jllm_check_launch("gemm_heads");
}
