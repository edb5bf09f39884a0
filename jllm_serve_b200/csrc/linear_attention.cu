// Gated linear attention: the recurrence over a request's tokens, and the per-head norm and gate of its output.
//
// Per head, with dk key channels and dv value channels, a request carries a state S [dk, dv] in 32-bit floats:
//     S_t = diag(d_t) S_(t-1) + k_t v_t^T,    o_t = S_t^T (scale * q_t),    d_t = sigmoid(z_t)^(1 / tau)
// d_t is formed as exp(log_sigmoid(z_t) / tau) in float32. The columns of S do not depend on one another, so a block
// owns 32 columns of one (segment, head): warp g of the block holds rows [g * R, (g + 1) * R) of those columns in
// registers (lane = column), every token's k, d, q and v are staged through shared memory eight tokens at a time, and
// the G partial sums of o_t are added in the order of g. A token's arithmetic is the same sequence of operations
// wherever its portion begins and whatever else the batch holds, so the result has the same bits for every cut.
//
// A segment is a run of consecutive rows of one request (a prompt portion, or one decoded token); its state lies in
// `state[slot]` ([slots, heads, dk, dv]), is read at the segment's first token and written back after its last. The
// same kernel serves a prompt and a decode step; the float32 and the bfloat16 path differ in the type of q, k, v only.
#include "common.cuh"

namespace {

constexpr int TOKENS = 8;       // tokens staged at a time
constexpr int COLS = 32;        // state columns per block: one per lane

template <typename T, int R>
__global__ void __launch_bounds__(1024)
gla_recurrent_kernel(const T* __restrict__ proj, int ld, int q_off, int k_off, int v_off, const float* __restrict__ z,
                     float* __restrict__ state, const int* __restrict__ seg_start, const int* __restrict__ seg_len,
                     const int* __restrict__ state_slots, float* __restrict__ o, int heads, int dk, int dv, float q_scale,
                     float inv_tau, int num_slots) {
    extern __shared__ float smem[];
    const int G = blockDim.x / COLS;
    float* ks = smem;                       // [TOKENS][dk]
    float* ds = ks + TOKENS * dk;           // [TOKENS][dk]
    float* qs = ds + TOKENS * dk;           // [TOKENS][dk]
    float* vs = qs + TOKENS * dk;           // [TOKENS][COLS]
    float* part = vs + TOKENS * COLS;       // [TOKENS][G][COLS]
    pdl_wait();
    pdl_trigger();
    const int seg = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * COLS;
    const int lane = threadIdx.x & 31, g = threadIdx.x >> 5, j = c0 + lane;
    const int first = seg_start[seg], n = seg_len[seg], slot = state_slots[seg];
    if (!jllm_in_bounds(slot, num_slots, BOUNDS_SLOT)) return;
    float* S = state + (((size_t)slot * heads + h) * dk) * dv;
    float s[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int i = g * R + r;
        s[r] = (i < dk && j < dv) ? S[(size_t)i * dv + j] : 0.f;
    }
    for (int t0 = 0; t0 < n; t0 += TOKENS) {
        const int nt = min(TOKENS, n - t0);
        __syncthreads();            // the staging of the last round has been read
        for (int e = threadIdx.x; e < nt * dk; e += blockDim.x) {
            const int t = e / dk, i = e - t * dk;
            const size_t row = (size_t)(first + t0 + t);
            const T* p = proj + row * ld + (size_t)h * dk + i;
            ks[t * dk + i] = to_float(p[k_off]);
            qs[t * dk + i] = __fmul_rn(to_float(p[q_off]), q_scale);
            const float zz = z[row * ((size_t)heads * dk) + (size_t)h * dk + i];
            // log(sigmoid(z)) = min(z, 0) - log1p(exp(-|z|)), then the 1 / tau-th power
            ds[t * dk + i] = expf(__fmul_rn(fminf(zz, 0.f) - log1pf(expf(-fabsf(zz))), inv_tau));
        }
        for (int e = threadIdx.x; e < nt * COLS; e += blockDim.x) {
            const int t = e / COLS, c = e - t * COLS;
            vs[e] = c0 + c < dv ? to_float(proj[(size_t)(first + t0 + t) * ld + v_off + (size_t)h * dv + c0 + c]) : 0.f;
        }
        __syncthreads();
        for (int t = 0; t < nt; ++t) {
            const float v = vs[t * COLS + lane];
            const float* kt = ks + t * dk + g * R;
            const float* dt = ds + t * dk + g * R;
            const float* qt = qs + t * dk + g * R;
            float acc = 0.f;
#pragma unroll
            for (int r = 0; r < R; ++r) {
                if (g * R + r < dk) {
                    s[r] = fmaf(dt[r], s[r], __fmul_rn(kt[r], v));
                    acc = fmaf(s[r], qt[r], acc);
                }
            }
            part[(t * G + g) * COLS + lane] = acc;
        }
        __syncthreads();
        for (int e = threadIdx.x; e < nt * COLS; e += blockDim.x) {
            const int t = e / COLS, c = e - t * COLS;
            if (c0 + c >= dv) continue;
            float acc = 0.f;
            for (int gg = 0; gg < G; ++gg) acc += part[(t * G + gg) * COLS + c];
            o[(size_t)(first + t0 + t) * ((size_t)heads * dv) + (size_t)h * dv + c0 + c] = acc;
        }
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int i = g * R + r;
        if (i < dk && j < dv) S[(size_t)i * dv + j] = s[r];
    }
}

template <typename T, int R>
int launch_recurrent(const void* proj, int ld, int q_off, int k_off, int v_off, const float* z, float* state,
                     const int* seg_start, const int* seg_len, const int* state_slots, float* o, int segments, int heads,
                     int dk, int dv, float q_scale, float inv_tau, int num_slots, cudaStream_t stream) {
    const int G = (dk + R - 1) / R;
    const size_t smem = (size_t)(TOKENS * (3 * dk + COLS) + TOKENS * G * COLS) * sizeof(float);
    auto kernel = gla_recurrent_kernel<T, R>;
    if (smem > 48 * 1024 &&
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return jllm_fail(JLLM_CUDA_ERROR, "gla_recurrent: %zu bytes of shared memory refused", smem);
    jllm_launch(kernel, dim3(segments, heads, (dv + COLS - 1) / COLS), dim3(G * COLS), smem, stream, LAUNCH_DEPENDENT,
                (const T*)proj, ld, q_off, k_off, v_off, z, state, seg_start, seg_len, state_slots, o, heads, dk, dv,
                q_scale, inv_tau, num_slots);
    return jllm_check_launch("gla_recurrent");
}

// y[r, h, :] = o[r, h, :] / sqrt(mean(o[r, h, :]^2) + eps) * gain * silu(gate[r, h, :]) * scale; one warp per (row, head)
template <typename T>
__global__ void __launch_bounds__(256)
gated_head_norm_kernel(const float* __restrict__ o, const T* __restrict__ gate, int ld_gate, VecRef gain, T* __restrict__ y,
                       int rows, int heads, int dv, float eps, float scale) {
    pdl_wait();
    pdl_trigger();
    const int w = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (w >= rows * heads) return;
    const int r = w / heads, h = w - r * heads;
    const float* src = o + ((size_t)r * heads + h) * dv;
    float ss = 0.f;
    for (int i = lane; i < dv; i += 32) ss = fmaf(src[i], src[i], ss);
    ss = warp_sum(ss);
    const float inv = 1.f / sqrtf(ss / (float)dv + eps);
    const T* gp = gate + (size_t)r * ld_gate + (size_t)h * dv;
    T* dst = y + ((size_t)r * heads + h) * dv;
    for (int i = lane; i < dv; i += 32) {
        const float gv = to_float(gp[i]);
        const float silu = gv / (1.f + expf(-gv));
        dst[i] = from_float<T>(__fmul_rn(__fmul_rn(__fmul_rn(__fmul_rn(src[i], inv), gain[i]), silu), scale));
    }
}

}  // namespace

JLLM_BOUNDS_READER(linear_attention)

// proj [rows, ld]: q at column q_off (heads x dk), k at k_off, v at v_off (heads x dv); z [rows, heads x dk] float32;
// state [num_slots, heads, dk, dv] float32; o [rows, heads x dv] float32.
JLLM_EXPORT int jllm_gla_recurrent(const void* proj, int dtype, int ld, int q_off, int k_off, int v_off, const float* z,
                                   float* state, int num_slots, const int* seg_start, const int* seg_len,
                                   const int* state_slots, float* o, int segments, int heads, int dk, int dv, float q_scale,
                                   float tau, cudaStream_t stream) {
    JLLM_REQUIRE(segments >= 0 && heads > 0 && dk > 0 && dv > 0 && tau > 0.f, "gla_recurrent: segments=%d heads=%d dk=%d dv=%d",
                 segments, heads, dk, dv);
    JLLM_REQUIRE(dk <= 512 && heads <= 65535 && (dv + COLS - 1) / COLS <= 65535, "gla_recurrent: dk=%d is above 512", dk);
    if (segments == 0) return JLLM_OK;
    const float inv_tau = 1.f / tau;
#define JLLM_GLA(T, R)                                                                                                  \
    return launch_recurrent<T, R>(proj, ld, q_off, k_off, v_off, z, state, seg_start, seg_len, state_slots, o, segments, \
                                  heads, dk, dv, q_scale, inv_tau, num_slots, stream)
    if (dtype == JLLM_F32) {
        if (dk <= 64) JLLM_GLA(float, 4);
        if (dk <= 256) JLLM_GLA(float, 8);
        JLLM_GLA(float, 16);
    }
    if (dk <= 64) JLLM_GLA(__nv_bfloat16, 4);
    if (dk <= 256) JLLM_GLA(__nv_bfloat16, 8);
    JLLM_GLA(__nv_bfloat16, 16);
#undef JLLM_GLA
}

JLLM_EXPORT int jllm_gated_head_norm(const float* o, const void* gate, int dtype, int ld_gate, const void* gain,
                                     int gain_dtype, void* y, int rows, int heads, int dv, float eps, float scale,
                                     cudaStream_t stream) {
    JLLM_REQUIRE(rows >= 0 && heads > 0 && dv > 0, "gated_head_norm: rows=%d heads=%d dv=%d", rows, heads, dv);
    if (rows == 0) return JLLM_OK;
    const VecRef g{gain, gain_dtype};
    const long long warps = (long long)rows * heads;
    const dim3 grid((unsigned)((warps + 7) / 8));
    if (dtype == JLLM_F32)
        jllm_launch(gated_head_norm_kernel<float>, grid, dim3(256), 0, stream, LAUNCH_DEPENDENT, o, (const float*)gate,
                    ld_gate, g, (float*)y, rows, heads, dv, eps, scale);
    else
        jllm_launch(gated_head_norm_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, LAUNCH_DEPENDENT, o,
                    (const __nv_bfloat16*)gate, ld_gate, g, (__nv_bfloat16*)y, rows, heads, dv, eps, scale);
    return jllm_check_launch("gated_head_norm");
}
