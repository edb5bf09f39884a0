// Attention over a cached latent: the two kernels around the paged attention kernels.
//
// A latent-attention mixer keeps ONE row c_t of `rank` values per position (c_t = rmsnorm(Wd h_t) * gain) and makes every
// head's keys and values from it: k = Wuk c, v = Wuv c. With q' = Wuk_h^T q_h the score q_h . k_j equals q' . c_j, and
// sum_j p_j v_j = Wuv_h (sum_j p_j c_j): attention with one key/value head of width `rank` whose keys and values are the
// same cached rows, between two small products per head. The attention itself is the engine's paged attention
// (kv_heads = 1, head_dim = rank). Here:
//
//   latent_norm_store   RMSNorm of the down-projected rows (float32 arithmetic) and their write into the paged cache
//   gemm_heads          out[r, h, :] = f(r, h) * W[h] a[r, h, :] for every head h at once (W [heads, N, K]); f = alpha, or
//                       alpha * sigmoid(gate[r, h]) (the mixer's output gate). float32: on the CUDA cores with one
//                       accumulator per element in ascending k. bfloat16: 64 x 64 tiles per (head, block) on the tensor
//                       cores (mma.sync m16n8k16, float32 accumulation), operands staged in shared memory 32 k at a
//                       time. Either way a row's result depends on that row alone, not on the batch.
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

// The bfloat16 product on the tensor cores. Four warps; warp w holds rows [16 w, 16 w + 16) of the block's 64 x 64 tile
// as eight m16n8 accumulators. Shared rows are padded to 40 values, so that the eight rows a fragment load touches fall
// into different banks. VEC: K, the row strides and the base addresses allow 16-byte loads.
constexpr int HK = 32, HPAD = 40;

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                               uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <bool VEC>
__global__ void __launch_bounds__(128)
gemm_heads_mma_kernel(const __nv_bfloat16* __restrict__ a, int lda, const __nv_bfloat16* __restrict__ w,
                      __nv_bfloat16* __restrict__ out, int ldo, const __nv_bfloat16* __restrict__ gate, int ld_gate,
                      float alpha, int M, int N, int K) {
    __shared__ __align__(16) __nv_bfloat16 as[64][HPAD];
    __shared__ __align__(16) __nv_bfloat16 ws[64][HPAD];
    pdl_wait();
    pdl_trigger();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3, h = blockIdx.z;
    const int m0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
    const __nv_bfloat16* ah = a + (size_t)h * K;
    const __nv_bfloat16* wh = w + (size_t)h * N * K;
    float acc[8][4] = {};
    const __nv_bfloat16 zero = __float2bfloat16_rn(0.f);
    for (int k0 = 0; k0 < K; k0 += HK) {
        if (VEC) {
            // 64 rows x 4 chunks of 8 values per tile: two chunks a thread and tile
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int c = tid + 128 * j, row = c >> 2, kc = (c & 3) * 8, k = k0 + kc;
                uint4 va = make_uint4(0, 0, 0, 0), vw = va;
                if (k < K) {        // (K is a multiple of 8 here: a chunk is inside or outside as a whole)
                    if (m0 + row < M) va = *reinterpret_cast<const uint4*>(ah + (size_t)(m0 + row) * lda + k);
                    if (n0 + row < N) vw = *reinterpret_cast<const uint4*>(wh + (size_t)(n0 + row) * K + k);
                }
                *reinterpret_cast<uint4*>(&as[row][kc]) = va;
                *reinterpret_cast<uint4*>(&ws[row][kc]) = vw;
            }
        } else {
            for (int e = tid; e < 64 * HK; e += 128) {
                const int row = e / HK, kc = e - row * HK, k = k0 + kc;
                as[row][kc] = (m0 + row < M && k < K) ? ah[(size_t)(m0 + row) * lda + k] : zero;
                ws[row][kc] = (n0 + row < N && k < K) ? wh[(size_t)(n0 + row) * K + k] : zero;
            }
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < HK; kk += 16) {
            const int r = warp * 16 + g;
            const uint32_t a0 = *reinterpret_cast<const uint32_t*>(&as[r][kk + 2 * t]);
            const uint32_t a1 = *reinterpret_cast<const uint32_t*>(&as[r + 8][kk + 2 * t]);
            const uint32_t a2 = *reinterpret_cast<const uint32_t*>(&as[r][kk + 2 * t + 8]);
            const uint32_t a3 = *reinterpret_cast<const uint32_t*>(&as[r + 8][kk + 2 * t + 8]);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const uint32_t b0 = *reinterpret_cast<const uint32_t*>(&ws[8 * j + g][kk + 2 * t]);
                const uint32_t b1 = *reinterpret_cast<const uint32_t*>(&ws[8 * j + g][kk + 2 * t + 8]);
                mma_bf16_16816(acc[j], a0, a1, a2, a3, b0, b1);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int m = m0 + warp * 16 + g + 8 * half;
        if (m >= M) continue;
        float f = alpha;
        if (gate != nullptr) {
            const float gv = to_float(gate[(size_t)m * ld_gate + h]);
            f = __fmul_rn(alpha, 1.f / (1.f + expf(-gv)));
        }
        __nv_bfloat16* dst = out + (size_t)m * ldo + (size_t)h * N;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int n = n0 + 8 * j + 2 * t;
            if (n < N) dst[n] = __float2bfloat16_rn(__fmul_rn(acc[j][2 * half], f));
            if (n + 1 < N) dst[n + 1] = __float2bfloat16_rn(__fmul_rn(acc[j][2 * half + 1], f));
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
    static_assert(BM == 64 && BN == 64, "both kernels take 64 x 64 tiles");
    if (dtype == JLLM_F32) {
        jllm_launch(gemm_heads_kernel<float>, grid, dim3(256), 0, stream, LAUNCH_DEPENDENT, (const float*)a, lda,
                    (const float*)w, (float*)out, ldo, (const float*)gate, ld_gate, alpha, M, N, K);
        return jllm_check_launch("gemm_heads");
    }
    const bool vec = K % 8 == 0 && lda % 8 == 0 && ((uintptr_t)a % 16) == 0 && ((uintptr_t)w % 16) == 0;
    if (vec)
        jllm_launch(gemm_heads_mma_kernel<true>, grid, dim3(128), 0, stream, LAUNCH_DEPENDENT, (const __nv_bfloat16*)a, lda,
                    (const __nv_bfloat16*)w, (__nv_bfloat16*)out, ldo, (const __nv_bfloat16*)gate, ld_gate, alpha, M, N, K);
    else
        jllm_launch(gemm_heads_mma_kernel<false>, grid, dim3(128), 0, stream, LAUNCH_DEPENDENT, (const __nv_bfloat16*)a, lda,
                    (const __nv_bfloat16*)w, (__nv_bfloat16*)out, ldo, (const __nv_bfloat16*)gate, ld_gate, alpha, M, N, K);
    return jllm_check_launch("gemm_heads");
}
