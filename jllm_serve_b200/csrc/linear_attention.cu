// Gated linear attention: the recurrence over a request's tokens, and the per-head norm and gate of its output.
//
// Per head, with dk key channels and dv value channels, a request carries a state S [dk, dv] in 32-bit floats:
//     S_t = diag(d_t) S_(t-1) + k_t v_t^T,    o_t = S_t^T (scale * q_t),    d_t = sigmoid(z_t)^(1 / tau)
// d_t is formed as exp(log_sigmoid(z_t) / tau) in float32 by a kernel in front. The columns of S do not depend on one
// another, so a block owns CB columns (32, or 16 where that gives more SMs a block) of one (segment, head). A thread holds R
// rows of one column in registers (row group g, column c); every token's k, d, q and v are staged through shared
// memory eight tokens at a time, the next eight being fetched into registers while these are worked on, and the G
// partial sums of o_t are added in the order of g. A token's arithmetic is the same sequence of operations wherever its
// portion begins, whatever else the batch holds and however the columns are dealt out, so the result has the same
// bits for every cut.
//
// A segment is a run of consecutive rows of one request (a prompt portion, or one decoded token); its state lies in
// `state[slot]` ([slots, heads, dk, dv]), is read at the segment's first token and written back after its last. The
// same kernel serves a prompt and a decode step; the float32 and the bfloat16 path differ in the type of q, k, v only.
#include "common.cuh"

namespace {

constexpr int TOKENS = 8;       // tokens staged at a time

// d = sigmoid(z)^(1 / tau), in place over [rows, heads x dk] float32: log(sigmoid(z)) = min(z, 0) - log1p(exp(-|z|)),
// times 1 / tau, exponentiated. Done once per step and element, in front of the recurrence (whose blocks would
// otherwise each redo it for the columns they own).
__global__ void gla_decay_kernel(float* __restrict__ z, float inv_tau, size_t total) {
    pdl_wait();
    pdl_trigger();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const float v = z[i];
        z[i] = expf(__fmul_rn(fminf(v, 0.f) - log1pf(expf(-fabsf(v))), inv_tau));
    }
}

template <typename T, int R, int CB, bool V4>
__global__ void __launch_bounds__(1024)
gla_recurrent_kernel(const T* __restrict__ proj, int ld, int q_off, int k_off, int v_off, const float* __restrict__ decay,
                     float* __restrict__ state, const int* __restrict__ seg_start, const int* __restrict__ seg_len,
                     const int* __restrict__ state_slots, float* __restrict__ o, int heads, int dk, int dv, float q_scale,
                     int num_slots) {
    constexpr int EPT = TOKENS * R / CB;            // staged values of k (and of q, of d) a thread fetches per round
    extern __shared__ __align__(16) float smem[];
    const int threads = blockDim.x, G = threads / CB;
    const int stage = TOKENS * (3 * dk + CB);       // floats of one staging buffer: k, d, q [TOKENS][dk], v [TOKENS][CB]
    float* part = smem + 2 * stage;                 // [TOKENS][G][CB]
    pdl_wait();
    pdl_trigger();
    const int seg = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * CB;
    const int tid = threadIdx.x, c = tid % CB, g = tid / CB, j = c0 + c;
    const int first = seg_start[seg], n = seg_len[seg], slot = state_slots[seg];
    if (!jllm_in_bounds(slot, num_slots, BOUNDS_SLOT)) return;
    float* S = state + (((size_t)slot * heads + h) * dk) * dv;
    float s[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int i = g * R + r;
        s[r] = (i < dk && j < dv) ? S[(size_t)i * dv + j] : 0.f;
    }
    // which staged values this thread fetches: the same places of every round, worked out once
    int st[EPT], sp[EPT], sd[EPT];                  // token within the round (TOKENS: none), offsets into proj and decay
#pragma unroll
    for (int u = 0; u < EPT; ++u) {
        const int e = tid + u * threads;
        st[u] = e < TOKENS * dk ? e / dk : TOKENS;
        const int i = e - st[u] * dk;
        sp[u] = st[u] * ld + h * dk + i;
        sd[u] = st[u] * heads * dk + h * dk + i;
    }
    const int vt = tid / CB, vc = tid - vt * CB;    // the one value of v this thread fetches (threads >= TOKENS x CB / 1)
    const int vpt = (TOKENS * CB + threads - 1) / threads;
    float fk[EPT], fq[EPT], fd[EPT], fv[TOKENS];

    auto fetch = [&](int t0) {      // the round that starts at token t0: from global memory into registers
        const int nt = min(TOKENS, n - t0);
        const size_t base = (size_t)(first + t0);
#pragma unroll
        for (int u = 0; u < EPT; ++u) {
            fk[u] = fq[u] = 0.f;
            fd[u] = 1.f;
            if (st[u] < nt) {
                const T* p = proj + base * ld + sp[u];
                fk[u] = to_float(p[k_off]);
                fq[u] = to_float(p[q_off]);
                fd[u] = decay[base * ((size_t)heads * dk) + sd[u]];
            }
        }
#pragma unroll
        for (int u = 0; u < TOKENS; ++u) {
            fv[u] = 0.f;
            if (u < vpt) {
                const int t = vt + u * (threads / CB);
                if (t < nt && c0 + vc < dv) fv[u] = to_float(proj[(base + t) * ld + v_off + (size_t)h * dv + c0 + vc]);
            }
        }
    };
    auto park = [&](int b) {        // ... and from the registers into staging buffer b
        float* ks = smem + b * stage;
        float* ds = ks + TOKENS * dk;
        float* qs = ds + TOKENS * dk;
        float* vs = qs + TOKENS * dk;
#pragma unroll
        for (int u = 0; u < EPT; ++u) {
            const int e = tid + u * threads;
            if (e < TOKENS * dk) {
                ks[e] = fk[u];
                ds[e] = fd[u];
                qs[e] = __fmul_rn(fq[u], q_scale);
            }
        }
#pragma unroll
        for (int u = 0; u < TOKENS; ++u) {
            const int t = vt + u * (threads / CB);
            if (u < vpt && t < TOKENS) vs[t * CB + vc] = fv[u];
        }
    };

    if (n > 0) {
        fetch(0);
        park(0);
    }
    __syncthreads();
    const bool rows_in = g * R < dk;
    for (int t0 = 0, b = 0; t0 < n; t0 += TOKENS, b ^= 1) {
        const int nt = min(TOKENS, n - t0);
        const bool more = t0 + TOKENS < n;
        if (more) fetch(t0 + TOKENS);               // on their way while this round's tokens are worked on
        const float* ks = smem + b * stage + g * R;
        const float* ds = ks + TOKENS * dk;
        const float* qs = ds + TOKENS * dk;
        const float* vs = smem + b * stage + 3 * TOKENS * dk;
        for (int t = 0; t < nt; ++t) {
            const float v = vs[t * CB + c];
            float acc0 = 0.f, acc1 = 0.f;
            if constexpr (V4) {     // dk a multiple of 4: four rows' k, d and q in one load each
                if (rows_in) {
#pragma unroll
                    for (int r = 0; r < R; r += 4) {
                        if (g * R + r < dk) {
                            const float4 kk = *reinterpret_cast<const float4*>(ks + t * dk + r);
                            const float4 dd = *reinterpret_cast<const float4*>(ds + t * dk + r);
                            const float4 qq = *reinterpret_cast<const float4*>(qs + t * dk + r);
                            s[r] = fmaf(dd.x, s[r], __fmul_rn(kk.x, v));
                            s[r + 1] = fmaf(dd.y, s[r + 1], __fmul_rn(kk.y, v));
                            s[r + 2] = fmaf(dd.z, s[r + 2], __fmul_rn(kk.z, v));
                            s[r + 3] = fmaf(dd.w, s[r + 3], __fmul_rn(kk.w, v));
                            acc0 = fmaf(s[r], qq.x, acc0);
                            acc1 = fmaf(s[r + 1], qq.y, acc1);
                            acc0 = fmaf(s[r + 2], qq.z, acc0);
                            acc1 = fmaf(s[r + 3], qq.w, acc1);
                        }
                    }
                }
            } else {
#pragma unroll
                for (int r = 0; r < R; r += 2) {
                    if (g * R + r < dk) {
                        s[r] = fmaf(ds[t * dk + r], s[r], __fmul_rn(ks[t * dk + r], v));
                        acc0 = fmaf(s[r], qs[t * dk + r], acc0);
                    }
                    if (g * R + r + 1 < dk) {
                        s[r + 1] = fmaf(ds[t * dk + r + 1], s[r + 1], __fmul_rn(ks[t * dk + r + 1], v));
                        acc1 = fmaf(s[r + 1], qs[t * dk + r + 1], acc1);
                    }
                }
            }
            part[(t * G + g) * CB + c] = acc0 + acc1;
        }
        if (more) park(b ^ 1);                      // (the other buffer: its last readers passed the barrier below)
        __syncthreads();
        for (int e = tid; e < nt * CB; e += threads) {
            const int t = e / CB, cc = e - t * CB;
            if (c0 + cc >= dv) continue;
            float acc = 0.f;
            for (int gg = 0; gg < G; ++gg) acc += part[(t * G + gg) * CB + cc];
            o[(size_t)(first + t0 + t) * ((size_t)heads * dv) + (size_t)h * dv + c0 + cc] = acc;
        }
        __syncthreads();                            // `part` and buffer b may be written again
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int i = g * R + r;
        if (i < dk && j < dv) S[(size_t)i * dv + j] = s[r];
    }
}

template <typename T, int R, int CB, bool V4>
int launch_recurrent(const void* proj, int ld, int q_off, int k_off, int v_off, const float* decay, float* state,
                     const int* seg_start, const int* seg_len, const int* state_slots, float* o, int segments, int heads,
                     int dk, int dv, float q_scale, int num_slots, cudaStream_t stream) {
    const int per_warp = 32 / CB;
    const int G = ((dk + R - 1) / R + per_warp - 1) / per_warp * per_warp;       // row groups: whole warps
    const size_t smem = (size_t)(2 * TOKENS * (3 * dk + CB) + TOKENS * G * CB) * sizeof(float);
    auto kernel = gla_recurrent_kernel<T, R, CB, V4>;
    if (smem > 48 * 1024 &&
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return jllm_fail(JLLM_CUDA_ERROR, "gla_recurrent: %zu bytes of shared memory refused", smem);
    jllm_launch(kernel, dim3(segments, heads, (dv + CB - 1) / CB), dim3(G * CB), smem, stream, LAUNCH_DEPENDENT,
                (const T*)proj, ld, q_off, k_off, v_off, decay, state, seg_start, seg_len, state_slots, o, heads, dk, dv,
                q_scale, num_slots);
    return jllm_check_launch("gla_recurrent");
}

// Columns per block: 32 (a warp is one row group), or 16 where 32 columns per block leave SMs without one. The choice
// changes which thread holds which value, not what is computed.
template <typename T, int R>
int launch_recurrent_cols(const void* proj, int ld, int q_off, int k_off, int v_off, const float* decay, float* state,
                          const int* seg_start, const int* seg_len, const int* state_slots, float* o, int segments,
                          int heads, int dk, int dv, float q_scale, int num_slots, cudaStream_t stream) {
    const long long sms = max(1, jllm_device_sm_count());
    const long long units = (long long)segments * heads;
    const bool wide = units * ((dv + 31) / 32) >= sms || dv <= 16;
#define JLLM_GLA_COLS(CB, V4)                                                                                                  \
    return launch_recurrent<T, R, CB, V4>(proj, ld, q_off, k_off, v_off, decay, state, seg_start, seg_len, state_slots, o, \
                                          segments, heads, dk, dv, q_scale, num_slots, stream)
    if (dk % 4 == 0) {
        if (wide) JLLM_GLA_COLS(32, true);
        JLLM_GLA_COLS(16, true);
    }
    if (wide) JLLM_GLA_COLS(32, false);
    JLLM_GLA_COLS(16, false);
#undef JLLM_GLA_COLS
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

// proj [rows, ld]: q at column q_off (heads x dk), k at k_off, v at v_off (heads x dv); z [rows, heads x dk] float32:
// the decay logits, which this call turns into the decays in place; state [num_slots, heads, dk, dv] float32; o [rows,
// heads x dv] float32. Two launches.
JLLM_EXPORT int jllm_gla_recurrent(const void* proj, int dtype, int ld, int q_off, int k_off, int v_off, float* z, int rows,
                                   float* state, int num_slots, const int* seg_start, const int* seg_len,
                                   const int* state_slots, float* o, int segments, int heads, int dk, int dv, float q_scale,
                                   float tau, cudaStream_t stream) {
    JLLM_REQUIRE(segments >= 0 && rows >= 0 && heads > 0 && dk > 0 && dv > 0 && tau > 0.f,
                 "gla_recurrent: segments=%d heads=%d dk=%d dv=%d", segments, heads, dk, dv);
    JLLM_REQUIRE(dk <= 512 && heads <= 65535 && (dv + 7) / 8 <= 65535, "gla_recurrent: dk=%d is above 512", dk);
    if (segments == 0 || rows == 0) return JLLM_OK;
    const float inv_tau = 1.f / tau;
    {       // the decay logits become decays, in place
        const size_t total = (size_t)rows * heads * dk;
        const int blocks = (int)min((size_t)65535, (total + 255) / 256);
        jllm_launch(gla_decay_kernel, dim3(blocks), dim3(256), 0, stream, LAUNCH_DEPENDENT, z, inv_tau, total);
        const int code = jllm_check_launch("gla_decay");
        if (code) return code;
    }
#define JLLM_GLA(T, R)                                                                                                       \
    return launch_recurrent_cols<T, R>(proj, ld, q_off, k_off, v_off, z, state, seg_start, seg_len, state_slots, o, segments, \
                                       heads, dk, dv, q_scale, num_slots, stream)
    if (dtype == JLLM_F32) {
        if (dk <= 128) JLLM_GLA(float, 4);
        if (dk <= 256) JLLM_GLA(float, 8);
        JLLM_GLA(float, 16);
    }
    // few rows a thread: the kernel waits more than it computes, and more threads hide more of the waiting (at most
    // 32 row groups of 32 columns: 1,024 threads)
    if (dk <= 128) JLLM_GLA(__nv_bfloat16, 4);
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
