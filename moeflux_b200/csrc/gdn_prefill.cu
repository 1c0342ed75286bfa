// Chunked GatedDeltaNet prefill (chunk of 64 tokens) for sm_100a.
//
// The reference prefills by running its five-kernel decode step once per token
// (crates/moeflux/src/riir/mod.rs:1206-1212 driving linear_attn_forward.rs:
// 607-664).  Here T tokens of one (layer, sequence) are processed by three
// launches that together compute exactly that sequence of steps:
//
//   1. gdn_prefill_conv_kernel   causal 4-tap depthwise conv + SiLU over the T
//      tokens (history from the conv ring), q/k normalisation, decay g and beta
//      per token (shaders.metal conv1d_step :1213, rms_norm_qk :1254,
//      compute_decay_beta :1312) -> q^,k^ (bf16), v (fp32), log g, beta scratch.
//   2. the delta rule in chunked form.  For a chunk of C = 64 tokens with cumulative
//      decay gamma_t = prod_{i<=t} g_i (kept as base-2 logs; only ratios
//      gamma_t/gamma_i with i <= t are ever formed):
//        A_ti = beta_t (gamma_t/gamma_i) (k_t.k_i), i < t        (strictly lower)
//        (I + A) U = diag(beta) (V - diag(gamma) K S0^T)
//        O = diag(gamma) Q S0^T + (M o Q K^T) U,  M_ti = gamma_t/gamma_i, i <= t
//        S_C = gamma_C S0 + U^T diag(gamma_C/gamma_i) K
//      which is the recurrence of gated_delta_net_step (shaders.metal:1154-1194)
//      unrolled over the chunk.  The solve is linear in its right-hand side, so
//      U = Ut - Wt S0^T with (I + A) Ut = diag(beta) V and (I + A) Wt = diag(beta gamma) K,
//      neither of which needs the state:
//      2a. gdn_prefill_intra_kernel  all chunks in parallel: A, the two forward
//          substitutions (fp32) and the masked Q K^T;
//      2b. gdn_prefill_state_kernel  serial over chunks: one CTA owns 64 of the 128
//          value rows of one v-head (state rows are independent), keeps that
//          half-state in registers in fp32 and runs the four remaining contractions
//          per chunk on the tensor cores (mma.sync m16n8k16, bf16 operands, fp32
//          accumulate).
//   3. gdn_prefill_out_kernel    read-out epilogue: gated RMSNorm with z
//      (shaders.metal:1337-1370) or a plain copy, to bf16.
#include <math.h>

#include "common.cuh"
#include "kernels.h"

namespace mfc {

namespace {

constexpr int CH = 64;          // tokens per chunk
constexpr int DVC = 64;         // value rows per CTA
constexpr int LDK = GDN_DIM + 8;  // padded leading dim (bf16) of [.][128] operand tiles
constexpr int LDT = CH + 8;       // padded leading dim (bf16) of [.][64] operand tiles

// ------------------------------------------------------------------ 1. conv / norm / gates
// grid (T, conv_dim / 2048), 256 threads: a thread owns 8 consecutive channels of one
// token (16-byte loads of the four input rows and of the weights).  A q or k head is
// 128 channels = 16 neighbouring lanes, reduced by shuffles.  Block y == 0 also
// computes the per-head gates of the token.
__global__ void __launch_bounds__(256)
gdn_prefill_conv_kernel(const __nv_bfloat16 *x, const __nv_bfloat16 *alpha, const __nv_bfloat16 *beta,
                        float *ring, int slot0, const uint16_t *conv_w, const float *a_log,
                        const uint16_t *dt_bias, __nv_bfloat16 *q_hat, __nv_bfloat16 *k_hat, float *v_out,
                        float *lg_out, float *beta_out, int T, int Hk, int Hv, int conv_dim) {
    const int t = blockIdx.x, tid = threadIdx.x;
    const int c0 = (blockIdx.y * 256 + tid) * 8;
    const int total_key = Hk * GDN_DIM;
    if (c0 < conv_dim) {
        float xr[4][8];  // rows t-3 .. t
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const int tt = t - 3 + k;
            if (tt >= 0) {
                const uint4 raw = *reinterpret_cast<const uint4 *>(x + (size_t)tt * conv_dim + c0);
                const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    xr[k][2 * e] = bf16_bits_to_f32((uint16_t)(w[e] & 0xffffu));
                    xr[k][2 * e + 1] = bf16_bits_to_f32((uint16_t)(w[e] >> 16));
                }
            } else {  // history row from the ring: token -1 sits in slot0-1, etc.
                const float *hr = ring + (size_t)((slot0 + tt) & 3) * conv_dim + c0;
#pragma unroll
                for (int e = 0; e < 8; e++) xr[k][e] = hr[e];
            }
        }
        float y[8];
#pragma unroll
        for (int e2 = 0; e2 < 4; e2++) {  // weights of two channels per 16-byte load
            const uint4 wr = *reinterpret_cast<const uint4 *>(conv_w + (size_t)(c0 + 2 * e2) * 4);
            const uint32_t w[4] = {wr.x, wr.y, wr.z, wr.w};
#pragma unroll
            for (int u = 0; u < 2; u++) {
                const int e = 2 * e2 + u;
                float acc = fmaf(xr[0][e], bf16_bits_to_f32((uint16_t)(w[2 * u] & 0xffffu)), 0.0f);
                acc = fmaf(xr[1][e], bf16_bits_to_f32((uint16_t)(w[2 * u] >> 16)), acc);
                acc = fmaf(xr[2][e], bf16_bits_to_f32((uint16_t)(w[2 * u + 1] & 0xffffu)), acc);
                acc = fmaf(xr[3][e], bf16_bits_to_f32((uint16_t)(w[2 * u + 1] >> 16)), acc);
                y[e] = acc / (1.0f + expf(-acc));
            }
        }
        if (c0 < 2 * total_key) {  // q or k: normalise over the head (16 lanes x 8 channels)
            float ss = 0.0f;
#pragma unroll
            for (int e = 0; e < 8; e++) ss += y[e] * y[e];
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            const float inv_scale = 1.0f / sqrtf((float)GDN_DIM);
            const float inv = 1.0f / sqrtf(ss / (float)GDN_DIM + 1e-6f);
            const bool is_q = c0 < total_key;
            const int cc = is_q ? c0 : c0 - total_key;
            uint32_t pk[4];
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const float a0 = is_q ? y[2 * e] * inv * inv_scale * inv_scale : y[2 * e] * inv * inv_scale;
                const float a1 = is_q ? y[2 * e + 1] * inv * inv_scale * inv_scale : y[2 * e + 1] * inv * inv_scale;
                pk[e] = pack_bf16x2(a0, a1);
            }
            __nv_bfloat16 *dst = (is_q ? q_hat : k_hat) + (size_t)t * total_key + cc;
            *reinterpret_cast<uint4 *>(dst) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
        } else {
            float *dst = v_out + (size_t)t * Hv * GDN_DIM + (c0 - 2 * total_key);
            *reinterpret_cast<float4 *>(dst) = make_float4(y[0], y[1], y[2], y[3]);
            *reinterpret_cast<float4 *>(dst + 4) = make_float4(y[4], y[5], y[6], y[7]);
        }
    }
    if (blockIdx.y == 0 && tid < Hv) {
        const float a_val = __bfloat162float(alpha[(size_t)t * Hv + tid]);
        const float dt_b = bf16_bits_to_f32(dt_bias[tid]);
        const float softplus = logf(1.0f + expf(a_val + dt_b));
        lg_out[(size_t)t * Hv + tid] = -expf(a_log[tid]) * softplus * 1.4426950408889634f;  // log2 of the decay g
        beta_out[(size_t)t * Hv + tid] = 1.0f / (1.0f + expf(-__bfloat162float(beta[(size_t)t * Hv + tid])));
    }
}

// The last three inputs become the conv history (token t goes to slot (slot0 + t) & 3).
__global__ void gdn_prefill_ring_kernel(const __nv_bfloat16 *x, float *ring, int slot0, int T, int conv_dim) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= conv_dim) return;
    for (int t = max(0, T - 3); t < T; t++) ring[(size_t)((slot0 + t) & 3) * conv_dim + c] = __bfloat162float(x[(size_t)t * conv_dim + c]);
}

// ------------------------------------------------------------------ warp-level GEMM pieces
// acc[NT][4] (16 rows x NT*8 cols, fp32) += A(16 x K) * B, A row-major bf16 (lda), K = KS*16.
// B given "n-major": element (n, k) at B[n*ldb + k].
template <int NT, int KS>
__device__ __forceinline__ void warp_gemm_nmajor(float (&acc)[NT][4], const __nv_bfloat16 *A, int lda,
                                                 const __nv_bfloat16 *B, int ldb, int lane) {
#pragma unroll
    for (int ks = 0; ks < KS; ks++) {
        uint32_t a[4];
        ldmatrix_x4(a[0], a[1], a[2], a[3], smem_u32(A + (lane & 15) * lda + ks * 16 + (lane >> 4) * 8));
#pragma unroll
        for (int nt = 0; nt < NT; nt += 2) {
            uint32_t b0, b1, b2, b3;
            ldmatrix_x4(b0, b1, b2, b3,
                        smem_u32(B + (nt * 8 + (lane & 7) + ((lane >> 4) << 3)) * ldb + ks * 16 + ((lane >> 3) & 1) * 8));
            mma_bf16_16816(acc[nt], a, b0, b1);
            mma_bf16_16816(acc[nt + 1], a, b2, b3);
        }
    }
}
// Same with B given "k-major": element (k, n) at B[k*ldb + n].
template <int NT, int KS>
__device__ __forceinline__ void warp_gemm_kmajor(float (&acc)[NT][4], const __nv_bfloat16 *A, int lda,
                                                 const __nv_bfloat16 *B, int ldb, int lane) {
#pragma unroll
    for (int ks = 0; ks < KS; ks++) {
        uint32_t a[4];
        ldmatrix_x4(a[0], a[1], a[2], a[3], smem_u32(A + (lane & 15) * lda + ks * 16 + (lane >> 4) * 8));
#pragma unroll
        for (int nt = 0; nt < NT; nt += 2) {
            uint32_t b0, b1, b2, b3;
            ldmatrix_x4_trans(b0, b1, b2, b3,
                              smem_u32(B + (ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * ldb + nt * 8 + (lane >> 4) * 8));
            mma_bf16_16816(acc[nt], a, b0, b1);
            mma_bf16_16816(acc[nt + 1], a, b2, b3);
        }
    }
}

// Same as warp_gemm_kmajor with A given transposed: element (m, k) at At[k*lda + m].
template <int NT, int KS>
__device__ __forceinline__ void warp_gemm_at_kmajor(float (&acc)[NT][4], const __nv_bfloat16 *At, int lda,
                                                    const __nv_bfloat16 *B, int ldb, int lane) {
#pragma unroll
    for (int ks = 0; ks < KS; ks++) {
        uint32_t a[4];
        ldmatrix_x4_trans(a[0], a[1], a[2], a[3],
                          smem_u32(At + (ks * 16 + (lane & 7) + ((lane >> 4) & 1) * 8) * lda + ((lane >> 3) & 1) * 8));
#pragma unroll
        for (int nt = 0; nt < NT; nt += 2) {
            uint32_t b0, b1, b2, b3;
            ldmatrix_x4_trans(b0, b1, b2, b3,
                              smem_u32(B + (ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * ldb + nt * 8 + (lane >> 4) * 8));
            mma_bf16_16816(acc[nt], a, b0, b1);
            mma_bf16_16816(acc[nt + 1], a, b2, b3);
        }
    }
}
// Two products that share the n-major B operand: acc1 += A1 B, acc2 += A2 B.
template <int NT, int KS>
__device__ __forceinline__ void warp_gemm2_nmajor(float (&acc1)[NT][4], float (&acc2)[NT][4], const __nv_bfloat16 *A1,
                                                  const __nv_bfloat16 *A2, int lda, const __nv_bfloat16 *B, int ldb,
                                                  int lane) {
#pragma unroll
    for (int ks = 0; ks < KS; ks++) {
        uint32_t a1[4], a2[4];
        ldmatrix_x4(a1[0], a1[1], a1[2], a1[3], smem_u32(A1 + (lane & 15) * lda + ks * 16 + (lane >> 4) * 8));
        ldmatrix_x4(a2[0], a2[1], a2[2], a2[3], smem_u32(A2 + (lane & 15) * lda + ks * 16 + (lane >> 4) * 8));
#pragma unroll
        for (int nt = 0; nt < NT; nt += 2) {
            uint32_t b0, b1, b2, b3;
            ldmatrix_x4(b0, b1, b2, b3,
                        smem_u32(B + (nt * 8 + (lane & 7) + ((lane >> 4) << 3)) * ldb + ks * 16 + ((lane >> 3) & 1) * 8));
            mma_bf16_16816(acc1[nt], a1, b0, b1);
            mma_bf16_16816(acc1[nt + 1], a1, b2, b3);
            mma_bf16_16816(acc2[nt], a2, b0, b1);
            mma_bf16_16816(acc2[nt + 1], a2, b2, b3);
        }
    }
}

// ------------------------------------------------------------------ 2a. per-chunk work that does not need the state
// grid (chunks, Hv), 256 threads.  Everything of a chunk that is independent of the
// running state is done here, for all chunks in parallel:
//   lg      <- inclusive prefix sum of log2 g inside the chunk (in place)
//   A_ti    = beta_t (gamma_t/gamma_i) (k_t.k_i), i < t                     shared memory, fp32
//   Wm_ti   = (gamma_t/gamma_i) (q_t.k_i), i <= t                           -> w_mask (bf16)
//   (I + A) Wt = diag(beta gamma) K      forward substitution, fp32         -> w_tilde (bf16)
//   (I + A) Ut = diag(beta) V            forward substitution, fp32         -> v_io in place (fp32)
// so that the serial kernel is left with U = Ut - Wt S0^T.  A thread owns one of the
// 128 + 128 right-hand-side columns and keeps its 64 unknowns in registers.
constexpr int LDA4 = CH + 4;  // fp32 [64][64] tile, rows 16-byte aligned
struct IntraSmem {
    __nv_bfloat16 K[CH][LDK];
    __nv_bfloat16 Q[CH][LDK];
    float A[CH][LDA4];
    float V[CH][GDN_DIM];
    float lg[CH];
    float bt[CH];
};

__global__ void __launch_bounds__(256, 2)
gdn_prefill_intra_kernel(const __nv_bfloat16 *q_hat, const __nv_bfloat16 *k_hat, float *v_io, float *lg_io,
                         const float *beta_in, __nv_bfloat16 *w_tilde, __nv_bfloat16 *w_mask, int T, int Hk, int Hv) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    IntraSmem &sm = *reinterpret_cast<IntraSmem *>(smem_raw);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t4 = lane & 3;
    const int tok0 = blockIdx.x * CH, h = blockIdx.y;
    const int j = h / (Hv / Hk);
    const size_t vrow = (size_t)Hv * GDN_DIM;

    // ---- operands: k^, q^ (bf16) and v (fp32) of the chunk; rows past T are zero ----
    for (int i = tid; i < CH * (GDN_DIM / 8); i += 256) {
        const int r = i >> 4, col = (i & 15) * 8;
        const bool in = tok0 + r < T;
        const size_t goff = ((size_t)(in ? tok0 + r : 0) * Hk + j) * GDN_DIM + col;
        const unsigned nbytes = in ? 16u : 0u;
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(&sm.K[r][col])), "l"(k_hat + goff),
                     "r"(nbytes)
                     : "memory");
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(&sm.Q[r][col])), "l"(q_hat + goff),
                     "r"(nbytes)
                     : "memory");
    }
    for (int i = tid; i < CH * (GDN_DIM / 4); i += 256) {
        const int r = i >> 5, col = (i & 31) * 4;
        const bool in = tok0 + r < T;
        const size_t goff = (size_t)(in ? tok0 + r : 0) * vrow + (size_t)h * GDN_DIM + col;
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(&sm.V[r][col])), "l"(v_io + goff),
                     "r"(in ? 16u : 0u)
                     : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    if (warp == 0) {  // inclusive prefix sum of log2 g over the 64 tokens; tokens past T leave gamma unchanged
        const bool ina = tok0 + lane < T, inb = tok0 + 32 + lane < T;
        float a = ina ? lg_io[(size_t)(tok0 + lane) * Hv + h] : 0.0f;
        float b = inb ? lg_io[(size_t)(tok0 + 32 + lane) * Hv + h] : 0.0f;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float ua = __shfl_up_sync(0xffffffffu, a, o), ub = __shfl_up_sync(0xffffffffu, b, o);
            if (lane >= o) {
                a += ua;
                b += ub;
            }
        }
        b += __shfl_sync(0xffffffffu, a, 31);
        sm.lg[lane] = a;
        sm.lg[32 + lane] = b;
        if (ina) lg_io[(size_t)(tok0 + lane) * Hv + h] = a;
        if (inb) lg_io[(size_t)(tok0 + 32 + lane) * Hv + h] = b;
        sm.bt[lane] = ina ? beta_in[(size_t)(tok0 + lane) * Hv + h] : 0.0f;
        sm.bt[32 + lane] = inb ? beta_in[(size_t)(tok0 + 32 + lane) * Hv + h] : 0.0f;
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();

    // ---- A and Wm: warp = (16-token row tile, 32-column half) ----
    {
        const int mt = warp & 3, nh = warp >> 2;
        const int r0 = 16 * mt + g, r1 = r0 + 8;
        const float lg0 = sm.lg[r0], lg1 = sm.lg[r1], b0 = sm.bt[r0], b1 = sm.bt[r1];
        float acc[4][4], acq[4][4];
#pragma unroll
        for (int n = 0; n < 4; n++)
#pragma unroll
            for (int e = 0; e < 4; e++) acc[n][e] = acq[n][e] = 0.0f;
        warp_gemm2_nmajor<4, 8>(acc, acq, &sm.K[16 * mt][0], &sm.Q[16 * mt][0], LDK, &sm.K[32 * nh][0], LDK, lane);
        const bool in0 = tok0 + r0 < T, in1 = tok0 + r1 < T;
#pragma unroll
        for (int n = 0; n < 4; n++) {
            const int col = 32 * nh + 8 * n + 2 * t4;
            const float d00 = ex2_approx(lg0 - sm.lg[col]), d01 = ex2_approx(lg0 - sm.lg[col + 1]);
            const float d10 = ex2_approx(lg1 - sm.lg[col]), d11 = ex2_approx(lg1 - sm.lg[col + 1]);
            sm.A[r0][col] = (col < r0) ? b0 * d00 * acc[n][0] : 0.0f;
            sm.A[r0][col + 1] = (col + 1 < r0) ? b0 * d01 * acc[n][1] : 0.0f;
            sm.A[r1][col] = (col < r1) ? b1 * d10 * acc[n][2] : 0.0f;
            sm.A[r1][col + 1] = (col + 1 < r1) ? b1 * d11 * acc[n][3] : 0.0f;
            if (in0)
                *reinterpret_cast<uint32_t *>(&w_mask[((size_t)(tok0 + r0) * Hv + h) * CH + col]) =
                    pack_bf16x2((col <= r0) ? d00 * acq[n][0] : 0.0f, (col + 1 <= r0) ? d01 * acq[n][1] : 0.0f);
            if (in1)
                *reinterpret_cast<uint32_t *>(&w_mask[((size_t)(tok0 + r1) * Hv + h) * CH + col]) =
                    pack_bf16x2((col <= r1) ? d10 * acq[n][2] : 0.0f, (col + 1 <= r1) ? d11 * acq[n][3] : 0.0f);
        }
    }
    __syncthreads();

    // ---- forward substitution, one right-hand-side column per thread ----
    {
        const int col = tid & 127;
        const bool is_v = tid >= 128;  // warp-uniform
        float u[CH];
        if (is_v) {
#pragma unroll
            for (int t = 0; t < CH; t++) u[t] = sm.bt[t] * sm.V[t][col];
        } else {
#pragma unroll
            for (int t = 0; t < CH; t++) u[t] = sm.bt[t] * ex2_approx(sm.lg[t]) * __bfloat162float(sm.K[t][col]);
        }
#pragma unroll
        for (int t = 1; t < CH; t++) {
            // A[t][i] is zero for i >= t, so whole groups of four can be taken; four partial sums keep the chain short
            float s0 = u[t], s1 = 0.0f, s2 = 0.0f, s3 = 0.0f;
#pragma unroll
            for (int i = 0; i < t; i += 4) {
                const float4 a = *reinterpret_cast<const float4 *>(&sm.A[t][i]);
                s0 = fmaf(-a.x, u[i], s0);
                s1 = fmaf(-a.y, u[i + 1], s1);
                s2 = fmaf(-a.z, u[i + 2], s2);
                s3 = fmaf(-a.w, u[i + 3], s3);
            }
            u[t] = (s0 + s1) + (s2 + s3);
        }
        const int n_in = min(CH, T - tok0);
        if (is_v) {
            float *dst = v_io + (size_t)tok0 * vrow + (size_t)h * GDN_DIM + col;
#pragma unroll
            for (int t = 0; t < CH; t++)
                if (t < n_in) dst[(size_t)t * vrow] = u[t];
        } else {
            __nv_bfloat16 *dst = w_tilde + ((size_t)tok0 * Hv + h) * GDN_DIM + col;
#pragma unroll
            for (int t = 0; t < CH; t++)
                if (t < n_in) dst[(size_t)t * vrow] = __float2bfloat16_rn(u[t]);
        }
    }
}

// ------------------------------------------------------------------ 2b. the serial part: state across chunks
// grid 2*Hv, 256 threads.  One CTA owns 64 of the 128 value rows of one v-head, keeps
// that half-state in registers in fp32 across all chunks (a bf16 operand copy in shared
// memory) and per chunk runs
//   U = Ut - Wt S0^T;   O = diag(gamma) Q S0^T + Wm U;   S = gamma_C S0 + (diag(gamma_C/gamma) U)^T K
// on the tensor cores (mma.sync m16n8k16, bf16 operands, fp32 accumulate).  Operands of
// chunk c+1 are requested while chunk c is worked on.
struct StateSmem {
    __nv_bfloat16 K[2][CH][LDK];
    __nv_bfloat16 Q[2][CH][LDK];
    __nv_bfloat16 Wt[2][CH][LDK];
    __nv_bfloat16 Wm[2][CH][LDT];
    __nv_bfloat16 Sb[DVC][LDK];   // bf16 operand copy of the state rows
    __nv_bfloat16 U[CH][LDT];     // [token][value row]
    __nv_bfloat16 Us[CH][LDT];    // rows scaled by gamma_C/gamma_t
};

__global__ void __launch_bounds__(256, 1)
gdn_prefill_state_kernel(float *ssm, const __nv_bfloat16 *q_hat, const __nv_bfloat16 *k_hat, float *v_io,
                         const float *lgc, const __nv_bfloat16 *w_tilde, const __nv_bfloat16 *w_mask, int T, int Hk,
                         int Hv) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    StateSmem &sm = *reinterpret_cast<StateSmem *>(smem_raw);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t4 = lane & 3;
    const int h = blockIdx.x >> 1, half = blockIdx.x & 1;
    const int j = h / (Hv / Hk);
    const size_t vrow = (size_t)Hv * GDN_DIM;
    float *Sg = ssm + ((size_t)h * GDN_DIM + half * DVC) * GDN_DIM;
    const int vcol0 = h * GDN_DIM + half * DVC;  // first value channel of this CTA in [T][Hv*128] arrays
    const int n_chunks = (T + CH - 1) / CH;

    // roles: products over tokens: (16-token tile mt, 32-value-row half nh); state update: (16 value rows sm_, 64 key columns sn)
    const int mt = warp & 3, nh = warp >> 2;
    const int r0 = 16 * mt + g, r1 = r0 + 8;
    const int srow0 = 16 * (warp & 3) + g, scol0 = 64 * (warp >> 2);

    auto prefetch = [&](int cc_) {
        const int base = cc_ * CH, buf = cc_ & 1;
        for (int i = tid; i < CH * (GDN_DIM / 8); i += 256) {
            const int r = i >> 4, col = (i & 15) * 8;
            const bool in = base + r < T;
            const unsigned nbytes = in ? 16u : 0u;
            const size_t tk = (size_t)(in ? base + r : 0);
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(&sm.K[buf][r][col])),
                         "l"(k_hat + (tk * Hk + j) * GDN_DIM + col), "r"(nbytes)
                         : "memory");
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(&sm.Q[buf][r][col])),
                         "l"(q_hat + (tk * Hk + j) * GDN_DIM + col), "r"(nbytes)
                         : "memory");
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(&sm.Wt[buf][r][col])),
                         "l"(w_tilde + (tk * Hv + h) * GDN_DIM + col), "r"(nbytes)
                         : "memory");
        }
        for (int i = tid; i < CH * (CH / 8); i += 256) {
            const int r = i >> 3, col = (i & 7) * 8;
            const bool in = base + r < T;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(&sm.Wm[buf][r][col])),
                         "l"(w_mask + ((size_t)(in ? base + r : 0) * Hv + h) * CH + col), "r"(in ? 16u : 0u)
                         : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    // per-thread values of a chunk that come straight from global memory: its Ut elements and decay logs
    struct ChunkRegs {
        float2 ut[4][2];
        float lg0, lg1, lgC;
    };
    auto fetch_regs = [&](int cc_, ChunkRegs &cr) {
        const int base = cc_ * CH;
        const bool in0 = base + r0 < T, in1 = base + r1 < T;
#pragma unroll
        for (int n = 0; n < 4; n++) {
            const int col = vcol0 + 32 * nh + 8 * n + 2 * t4;
            cr.ut[n][0] = in0 ? *reinterpret_cast<const float2 *>(&v_io[(size_t)(base + r0) * vrow + col]) : make_float2(0.0f, 0.0f);
            cr.ut[n][1] = in1 ? *reinterpret_cast<const float2 *>(&v_io[(size_t)(base + r1) * vrow + col]) : make_float2(0.0f, 0.0f);
        }
        cr.lg0 = lgc[(size_t)min(base + r0, T - 1) * Hv + h];
        cr.lg1 = lgc[(size_t)min(base + r1, T - 1) * Hv + h];
        cr.lgC = lgc[(size_t)min(base + CH - 1, T - 1) * Hv + h];
    };

    prefetch(0);
    ChunkRegs nxt;
    fetch_regs(0, nxt);
    float S[8][4];  // state rows srow0, srow0+8; columns scol0 + 8n + 2*t4 + {0,1}
#pragma unroll
    for (int n = 0; n < 8; n++) {
        const int col = scol0 + 8 * n + 2 * t4;
        const float2 a = *reinterpret_cast<const float2 *>(&Sg[(size_t)srow0 * GDN_DIM + col]);
        const float2 b = *reinterpret_cast<const float2 *>(&Sg[(size_t)(srow0 + 8) * GDN_DIM + col]);
        S[n][0] = a.x;
        S[n][1] = a.y;
        S[n][2] = b.x;
        S[n][3] = b.y;
        *reinterpret_cast<uint32_t *>(&sm.Sb[srow0][col]) = pack_bf16x2(a.x, a.y);
        *reinterpret_cast<uint32_t *>(&sm.Sb[srow0 + 8][col]) = pack_bf16x2(b.x, b.y);
    }

    for (int c = 0; c < n_chunks; c++) {
        const int buf = c & 1, tok0 = c * CH;
        asm volatile("cp.async.wait_group 0;" ::: "memory");  // this thread's copies of chunk c have landed
        __syncthreads();  // everyone's have; Sb holds the current state; the other buffers are free
        const ChunkRegs cur = nxt;
        if (c + 1 < n_chunks) {
            prefetch(c + 1);
            fetch_regs(c + 1, nxt);
        }
        // ---- U = Ut - Wt S0^T and Q S0^T (same B operand) ----
        float aw[4][4], o[4][4];
#pragma unroll
        for (int n = 0; n < 4; n++)
#pragma unroll
            for (int e = 0; e < 4; e++) aw[n][e] = o[n][e] = 0.0f;
        warp_gemm2_nmajor<4, 8>(aw, o, &sm.Wt[buf][16 * mt][0], &sm.Q[buf][16 * mt][0], LDK, &sm.Sb[32 * nh][0], LDK, lane);
        {
            const float f0 = ex2_approx(cur.lgC - cur.lg0), f1 = ex2_approx(cur.lgC - cur.lg1);
            const float e0 = ex2_approx(cur.lg0), e1 = ex2_approx(cur.lg1);
#pragma unroll
            for (int n = 0; n < 4; n++) {
                const int col = 32 * nh + 8 * n + 2 * t4;
                const float u00 = cur.ut[n][0].x - aw[n][0], u01 = cur.ut[n][0].y - aw[n][1];
                const float u10 = cur.ut[n][1].x - aw[n][2], u11 = cur.ut[n][1].y - aw[n][3];
                *reinterpret_cast<uint32_t *>(&sm.U[r0][col]) = pack_bf16x2(u00, u01);
                *reinterpret_cast<uint32_t *>(&sm.U[r1][col]) = pack_bf16x2(u10, u11);
                *reinterpret_cast<uint32_t *>(&sm.Us[r0][col]) = pack_bf16x2(u00 * f0, u01 * f0);
                *reinterpret_cast<uint32_t *>(&sm.Us[r1][col]) = pack_bf16x2(u10 * f1, u11 * f1);
                o[n][0] *= e0;
                o[n][1] *= e0;
                o[n][2] *= e1;
                o[n][3] *= e1;
            }
        }
        __syncthreads();  // U and Us are complete; nobody reads Sb any more
        // ---- O += Wm U -> written over v_io (fp32) ----
        warp_gemm_kmajor<4, 4>(o, &sm.Wm[buf][16 * mt][0], LDT, &sm.U[0][32 * nh], LDT, lane);
        {
            const bool in0 = tok0 + r0 < T, in1 = tok0 + r1 < T;
#pragma unroll
            for (int n = 0; n < 4; n++) {
                const int col = vcol0 + 32 * nh + 8 * n + 2 * t4;
                if (in0) *reinterpret_cast<float2 *>(&v_io[(size_t)(tok0 + r0) * vrow + col]) = make_float2(o[n][0], o[n][1]);
                if (in1) *reinterpret_cast<float2 *>(&v_io[(size_t)(tok0 + r1) * vrow + col]) = make_float2(o[n][2], o[n][3]);
            }
        }
        // ---- S = gamma_C S + Us^T K ----
        {
            const float gC = ex2_approx(cur.lgC);
#pragma unroll
            for (int n = 0; n < 8; n++)
#pragma unroll
                for (int e = 0; e < 4; e++) S[n][e] *= gC;
            warp_gemm_at_kmajor<8, 4>(S, &sm.Us[0][16 * (warp & 3)], LDT, &sm.K[buf][0][scol0], LDK, lane);
#pragma unroll
            for (int n = 0; n < 8; n++) {
                const int col = scol0 + 8 * n + 2 * t4;
                *reinterpret_cast<uint32_t *>(&sm.Sb[srow0][col]) = pack_bf16x2(S[n][0], S[n][1]);
                *reinterpret_cast<uint32_t *>(&sm.Sb[srow0 + 8][col]) = pack_bf16x2(S[n][2], S[n][3]);
            }
        }
    }
#pragma unroll
    for (int n = 0; n < 8; n++) {
        const int col = scol0 + 8 * n + 2 * t4;
        *reinterpret_cast<float2 *>(&Sg[(size_t)srow0 * GDN_DIM + col]) = make_float2(S[n][0], S[n][1]);
        *reinterpret_cast<float2 *>(&Sg[(size_t)(srow0 + 8) * GDN_DIM + col]) = make_float2(S[n][2], S[n][3]);
    }
}

// ------------------------------------------------------------------ 3. read-out epilogue
// grid (T), 256 threads: a warp takes one head at a time (4 values per lane):
// out = o * rsqrt(mean o^2 + eps) * w * silu(z), or out = o.
__global__ void __launch_bounds__(256)
gdn_prefill_out_kernel(const float *o_raw, const __nv_bfloat16 *z, const uint16_t *norm_w, __nv_bfloat16 *out,
                       int Hv, float eps) {
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int h = warp; h < Hv; h += 8) {
        const size_t idx = ((size_t)t * Hv + h) * GDN_DIM + lane * 4;
        const float4 o = *reinterpret_cast<const float4 *>(o_raw + idx);
        float r[4] = {o.x, o.y, o.z, o.w};
        if (z != nullptr) {
            const float tot = warp_sum(o.x * o.x + o.y * o.y + o.z * o.z + o.w * o.w);
            const float inv_rms = 1.0f / sqrtf(tot / (float)GDN_DIM + eps);
            const uint2 zz = *reinterpret_cast<const uint2 *>(z + idx);
            const uint2 ww = *reinterpret_cast<const uint2 *>(norm_w + lane * 4);
            const float zf[4] = {bf16_bits_to_f32((uint16_t)(zz.x & 0xffffu)), bf16_bits_to_f32((uint16_t)(zz.x >> 16)),
                                 bf16_bits_to_f32((uint16_t)(zz.y & 0xffffu)), bf16_bits_to_f32((uint16_t)(zz.y >> 16))};
            const float wf[4] = {bf16_bits_to_f32((uint16_t)(ww.x & 0xffffu)), bf16_bits_to_f32((uint16_t)(ww.x >> 16)),
                                 bf16_bits_to_f32((uint16_t)(ww.y & 0xffffu)), bf16_bits_to_f32((uint16_t)(ww.y >> 16))};
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const float silu_z = zf[e] / (1.0f + expf(-zf[e]));
                r[e] = r[e] * inv_rms * wf[e] * silu_z;
            }
        }
        *reinterpret_cast<uint2 *>(out + idx) = make_uint2(pack_bf16x2(r[0], r[1]), pack_bf16x2(r[2], r[3]));
    }
}

}  // namespace

cudaError_t gdn_prefill_configure() {
    cudaError_t e = cudaFuncSetAttribute(gdn_prefill_intra_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)sizeof(IntraSmem));
    if (e != cudaSuccess) return e;
    return cudaFuncSetAttribute(gdn_prefill_state_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                (int)sizeof(StateSmem));
}

cudaError_t launch_gdn_prefill(const GdnPrefillParams &p, cudaStream_t stream) {
    if (p.T <= 0) return cudaSuccess;
    const __nv_bfloat16 *x = reinterpret_cast<const __nv_bfloat16 *>(p.qkv);
    dim3 g1((unsigned)p.T, (unsigned)((p.conv_dim + 2047) / 2048), 1);
    gdn_prefill_conv_kernel<<<g1, 256, 0, stream>>>(
        x, reinterpret_cast<const __nv_bfloat16 *>(p.alpha), reinterpret_cast<const __nv_bfloat16 *>(p.beta), p.ring,
        p.slot0, p.conv_w, p.a_log, p.dt_bias, reinterpret_cast<__nv_bfloat16 *>(p.q_hat),
        reinterpret_cast<__nv_bfloat16 *>(p.k_hat), p.v_io, p.lg, p.beta_gate, p.T, p.Hk, p.Hv, p.conv_dim);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    gdn_prefill_ring_kernel<<<(p.conv_dim + 255) / 256, 256, 0, stream>>>(x, p.ring, p.slot0, p.T, p.conv_dim);
    if ((e = cudaGetLastError()) != cudaSuccess) return e;
    const int n_chunks = (p.T + CH - 1) / CH;
    gdn_prefill_intra_kernel<<<dim3((unsigned)n_chunks, (unsigned)p.Hv, 1), 256, sizeof(IntraSmem), stream>>>(
        reinterpret_cast<const __nv_bfloat16 *>(p.q_hat), reinterpret_cast<const __nv_bfloat16 *>(p.k_hat), p.v_io, p.lg,
        p.beta_gate, reinterpret_cast<__nv_bfloat16 *>(p.w_tilde), reinterpret_cast<__nv_bfloat16 *>(p.w_mask), p.T, p.Hk,
        p.Hv);
    if ((e = cudaGetLastError()) != cudaSuccess) return e;
    gdn_prefill_state_kernel<<<2 * p.Hv, 256, sizeof(StateSmem), stream>>>(
        p.ssm, reinterpret_cast<const __nv_bfloat16 *>(p.q_hat), reinterpret_cast<const __nv_bfloat16 *>(p.k_hat), p.v_io,
        p.lg, reinterpret_cast<const __nv_bfloat16 *>(p.w_tilde), reinterpret_cast<const __nv_bfloat16 *>(p.w_mask), p.T,
        p.Hk, p.Hv);
    if ((e = cudaGetLastError()) != cudaSuccess) return e;
    gdn_prefill_out_kernel<<<(unsigned)p.T, 256, 0, stream>>>(p.v_io, reinterpret_cast<const __nv_bfloat16 *>(p.z), p.norm_w,
                                                   reinterpret_cast<__nv_bfloat16 *>(p.out), p.Hv, p.eps);
    return cudaGetLastError();
}

}  // namespace mfc
