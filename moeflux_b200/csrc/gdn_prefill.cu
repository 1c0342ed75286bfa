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
//   2. gdn_prefill_chunk_kernel  the delta rule in chunked form.  For a chunk of
//      C = 64 tokens with cumulative decay gamma_t = prod_{i<=t} g_i (kept as
//      base-2 logs; only ratios gamma_t/gamma_i with i <= t are ever formed):
//        A_ti = beta_t (gamma_t/gamma_i) (k_t.k_i), i < t        (strictly lower)
//        (I + A) U = diag(beta) (V - diag(gamma) K S0^T)          forward substitution, fp32
//        O = diag(gamma) Q S0^T + (M o Q K^T) U,  M_ti = gamma_t/gamma_i, i <= t
//        S_C = gamma_C S0 + U^T diag(gamma_C/gamma_i) K
//      which is the recurrence of gated_delta_net_step (shaders.metal:1154-1194)
//      unrolled over the chunk.  One CTA owns 64 of the 128 value rows of one
//      v-head (state rows are independent), keeps that half-state in shared
//      memory in fp32 across all chunks, and runs the six dense contractions on
//      the tensor cores (mma.sync m16n8k16, bf16 operands, fp32 accumulate).
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
constexpr int LDA = CH + 1;       // fp32 [64][64] tiles

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

// ------------------------------------------------------------------ 2. chunked delta rule
struct ChunkSmem {
    float S[DVC][GDN_DIM];            // fp32 master copy of this CTA's state rows   32 KiB
    __nv_bfloat16 Sb[DVC][LDK];       // bf16 operand copy                           17 KiB
    __nv_bfloat16 K[2][CH][LDK];      // k^ of the chunk (later scaled in place), double buffered  34 KiB
    __nv_bfloat16 Q[2][CH][LDK];      //                                                           34 KiB
    float A[CH][LDA];                 // strictly lower triangular system            16.25 KiB
    float Bm[CH][DVC + 1];            // right-hand side                             16.25 KiB
    __nv_bfloat16 W[CH][LDT];         // decay-masked Q K^T                           9 KiB
    __nv_bfloat16 Ut[DVC][LDT];       // U transposed: [value row][token]             9 KiB
    float lg[CH];                     // cumulative log2 decay, inclusive
    float bt[CH];                     // beta
};

__global__ void __launch_bounds__(128, 1)
gdn_prefill_chunk_kernel(float *ssm, const __nv_bfloat16 *q_hat, const __nv_bfloat16 *k_hat, float *v_io,
                         const float *lg_in, const float *beta_in, int T, int Hk, int Hv) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    ChunkSmem &sm = *reinterpret_cast<ChunkSmem *>(smem_raw);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t4 = lane & 3;
    const int h = blockIdx.x >> 1, half = blockIdx.x & 1;
    const int j = h / (Hv / Hk);
    float *Sg = ssm + ((size_t)h * GDN_DIM + half * DVC) * GDN_DIM;
    const int vcol0 = h * GDN_DIM + half * DVC;  // first value channel of this CTA in [T][Hv*128] arrays

    for (int i = tid; i < DVC * GDN_DIM / 4; i += 128)
        reinterpret_cast<float4 *>(&sm.S[0][0])[i] = reinterpret_cast<const float4 *>(Sg)[i];

    const int n_chunks = (T + CH - 1) / CH;
    // k^ and q^ rows of chunk cc -> buffer cc & 1 (16-byte cp.async, rows past T zero-filled)
    auto prefetch_kq = [&](int cc_) {
        const int base = cc_ * CH, buf = cc_ & 1;
        for (int i = tid; i < CH * (GDN_DIM / 8); i += 128) {
            const int r = i >> 4, col = (i & 15) * 8;
            const bool in = base + r < T;
            const size_t goff = ((size_t)(in ? base + r : 0) * Hk + j) * GDN_DIM + col;
            const unsigned nbytes = in ? 16u : 0u;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(&sm.K[buf][r][col])),
                         "l"(k_hat + goff), "r"(nbytes)
                         : "memory");
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(&sm.Q[buf][r][col])),
                         "l"(q_hat + goff), "r"(nbytes)
                         : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    prefetch_kq(0);
    for (int c = 0; c < n_chunks; c++) {
        __nv_bfloat16(*Kc)[LDK] = sm.K[c & 1];
        __nv_bfloat16(*Qc)[LDK] = sm.Q[c & 1];
        const int tok0 = c * CH;
        __syncthreads();  // previous chunk is done with every buffer
        // ---- stage 0: operands of the chunk; tokens past T act as "no token" ----
        // operands of chunk c were requested one chunk ago; request those of chunk c+1 now
        if (c + 1 < n_chunks) {
            prefetch_kq(c + 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");  // everything but the newest group has landed
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        for (int i = tid; i < DVC * GDN_DIM / 2; i += 128) {
            const int r = i >> 6, cc = (i & 63) * 2;
            *reinterpret_cast<uint32_t *>(&sm.Sb[r][cc]) = pack_bf16x2(sm.S[r][cc], sm.S[r][cc + 1]);
        }
        if (warp == 0) {  // inclusive prefix sum of log g over the 64 tokens
            float a = (tok0 + lane < T) ? lg_in[(size_t)(tok0 + lane) * Hv + h] : 0.0f;
            float b = (tok0 + 32 + lane < T) ? lg_in[(size_t)(tok0 + 32 + lane) * Hv + h] : 0.0f;
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
            sm.bt[lane] = (tok0 + lane < T) ? beta_in[(size_t)(tok0 + lane) * Hv + h] : 0.0f;
            sm.bt[32 + lane] = (tok0 + 32 + lane < T) ? beta_in[(size_t)(tok0 + 32 + lane) * Hv + h] : 0.0f;
        }
        __syncthreads();

        const int r0 = 16 * warp + g, r1 = r0 + 8;  // this thread's two token rows in 64-row results
        const float lg0 = sm.lg[r0], lg1 = sm.lg[r1];
        // this thread's v values of the chunk, requested now, used in stage 2
        float2 vpre[8][2];
        {
            const bool in0 = tok0 + r0 < T, in1 = tok0 + r1 < T;
#pragma unroll
            for (int n = 0; n < 8; n++) {
                const int col = 8 * n + 2 * t4;
                vpre[n][0] = in0 ? *reinterpret_cast<const float2 *>(&v_io[(size_t)(tok0 + r0) * Hv * GDN_DIM + vcol0 + col])
                                 : make_float2(0.0f, 0.0f);
                vpre[n][1] = in1 ? *reinterpret_cast<const float2 *>(&v_io[(size_t)(tok0 + r1) * Hv * GDN_DIM + vcol0 + col])
                                 : make_float2(0.0f, 0.0f);
            }
        }
        // ---- stage 1: A = beta (gamma_t/gamma_i) K K^T (i < t);  W = (gamma_t/gamma_i) Q K^T (i <= t) ----
        {
            float acc[8][4];
#pragma unroll
            for (int n = 0; n < 8; n++) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.0f;
            warp_gemm_nmajor<8, 8>(acc, &Kc[16 * warp][0], LDK, &Kc[0][0], LDK, lane);
            const float b0 = sm.bt[r0], b1 = sm.bt[r1];
#pragma unroll
            for (int n = 0; n < 8; n++)
#pragma unroll
                for (int e = 0; e < 2; e++) {
                    const int col = 8 * n + 2 * t4 + e;
                    sm.A[r0][col] = (col < r0) ? b0 * ex2_approx(lg0 - sm.lg[col]) * acc[n][e] : 0.0f;
                    sm.A[r1][col] = (col < r1) ? b1 * ex2_approx(lg1 - sm.lg[col]) * acc[n][2 + e] : 0.0f;
                }
#pragma unroll
            for (int n = 0; n < 8; n++) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.0f;
            warp_gemm_nmajor<8, 8>(acc, &Qc[16 * warp][0], LDK, &Kc[0][0], LDK, lane);
#pragma unroll
            for (int n = 0; n < 8; n++) {
                const int col = 8 * n + 2 * t4;
                const float w00 = (col <= r0) ? ex2_approx(lg0 - sm.lg[col]) * acc[n][0] : 0.0f;
                const float w01 = (col + 1 <= r0) ? ex2_approx(lg0 - sm.lg[col + 1]) * acc[n][1] : 0.0f;
                const float w10 = (col <= r1) ? ex2_approx(lg1 - sm.lg[col]) * acc[n][2] : 0.0f;
                const float w11 = (col + 1 <= r1) ? ex2_approx(lg1 - sm.lg[col + 1]) * acc[n][3] : 0.0f;
                *reinterpret_cast<uint32_t *>(&sm.W[r0][col]) = pack_bf16x2(w00, w01);
                *reinterpret_cast<uint32_t *>(&sm.W[r1][col]) = pack_bf16x2(w10, w11);
            }
        }
        // ---- stage 2: Bm = beta (V - gamma K S0^T) ----
        {
            float acc[8][4];
#pragma unroll
            for (int n = 0; n < 8; n++) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.0f;
            warp_gemm_nmajor<8, 8>(acc, &Kc[16 * warp][0], LDK, &sm.Sb[0][0], LDK, lane);
            const float b0 = sm.bt[r0], b1 = sm.bt[r1], e0 = ex2_approx(lg0), e1 = ex2_approx(lg1);
#pragma unroll
            for (int n = 0; n < 8; n++) {
                const int col = 8 * n + 2 * t4;
                sm.Bm[r0][col] = b0 * (vpre[n][0].x - e0 * acc[n][0]);
                sm.Bm[r0][col + 1] = b0 * (vpre[n][0].y - e0 * acc[n][1]);
                sm.Bm[r1][col] = b1 * (vpre[n][1].x - e1 * acc[n][2]);
                sm.Bm[r1][col + 1] = b1 * (vpre[n][1].y - e1 * acc[n][3]);
            }
        }
        __syncthreads();
        // ---- stage 3: forward substitution (I + A) U = Bm, one thread per value column ----
        if (tid < DVC) {
            float u[CH];
#pragma unroll
            for (int t = 0; t < CH; t++) {
                // four independent partial sums keep the dependent FMA chain of a row short
                float s0 = sm.Bm[t][tid], s1 = 0.0f, s2 = 0.0f, s3 = 0.0f;
#pragma unroll
                for (int i = 0; i + 3 < t; i += 4) {
                    s0 = fmaf(-sm.A[t][i], u[i], s0);
                    s1 = fmaf(-sm.A[t][i + 1], u[i + 1], s1);
                    s2 = fmaf(-sm.A[t][i + 2], u[i + 2], s2);
                    s3 = fmaf(-sm.A[t][i + 3], u[i + 3], s3);
                }
#pragma unroll
                for (int i = t & ~3; i < t; i++) s0 = fmaf(-sm.A[t][i], u[i], s0);
                u[t] = (s0 + s1) + (s2 + s3);
            }
#pragma unroll
            for (int t = 0; t < CH; t += 2) *reinterpret_cast<uint32_t *>(&sm.Ut[tid][t]) = pack_bf16x2(u[t], u[t + 1]);
        }
        __syncthreads();
        // ---- stage 4: O = gamma Q S0^T + W U  -> written over v_io (fp32) ----
        {
            float acc[8][4];
#pragma unroll
            for (int n = 0; n < 8; n++) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.0f;
            warp_gemm_nmajor<8, 8>(acc, &Qc[16 * warp][0], LDK, &sm.Sb[0][0], LDK, lane);
            const float e0 = ex2_approx(lg0), e1 = ex2_approx(lg1);
#pragma unroll
            for (int n = 0; n < 8; n++) {
                acc[n][0] *= e0;
                acc[n][1] *= e0;
                acc[n][2] *= e1;
                acc[n][3] *= e1;
            }
            warp_gemm_nmajor<8, 4>(acc, &sm.W[16 * warp][0], LDT, &sm.Ut[0][0], LDT, lane);
            const bool in0 = tok0 + r0 < T, in1 = tok0 + r1 < T;
#pragma unroll
            for (int n = 0; n < 8; n++) {
                const int col = 8 * n + 2 * t4;
                if (in0)
                    *reinterpret_cast<float2 *>(&v_io[(size_t)(tok0 + r0) * Hv * GDN_DIM + vcol0 + col]) =
                        make_float2(acc[n][0], acc[n][1]);
                if (in1)
                    *reinterpret_cast<float2 *>(&v_io[(size_t)(tok0 + r1) * Hv * GDN_DIM + vcol0 + col]) =
                        make_float2(acc[n][2], acc[n][3]);
            }
        }
        __syncthreads();  // every warp is done reading K and Q of this chunk
        // ---- stage 5: K <- (gamma_C/gamma_i) K;  S = gamma_C S + U^T K ----
        const float lgC = sm.lg[CH - 1];
        for (int i = tid; i < CH * (GDN_DIM / 2); i += 128) {
            const int r = i >> 6, cc = (i & 63) * 2;
            const float f = ex2_approx(lgC - sm.lg[r]);
            __nv_bfloat162 kv = *reinterpret_cast<__nv_bfloat162 *>(&Kc[r][cc]);
            *reinterpret_cast<uint32_t *>(&Kc[r][cc]) = pack_bf16x2(__low2float(kv) * f, __high2float(kv) * f);
        }
        __syncthreads();
        {
            float acc[16][4];
#pragma unroll
            for (int n = 0; n < 16; n++) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.0f;
            warp_gemm_kmajor<16, 4>(acc, &sm.Ut[16 * warp][0], LDT, &Kc[0][0], LDK, lane);
            const float gC = ex2_approx(lgC);
#pragma unroll
            for (int n = 0; n < 16; n++) {
                const int col = 8 * n + 2 * t4;
                float2 *p0 = reinterpret_cast<float2 *>(&sm.S[r0][col]);
                float2 *p1 = reinterpret_cast<float2 *>(&sm.S[r1][col]);
                const float2 s0 = *p0, s1 = *p1;
                *p0 = make_float2(fmaf(gC, s0.x, acc[n][0]), fmaf(gC, s0.y, acc[n][1]));
                *p1 = make_float2(fmaf(gC, s1.x, acc[n][2]), fmaf(gC, s1.y, acc[n][3]));
            }
        }
    }
    __syncthreads();
    for (int i = tid; i < DVC * GDN_DIM / 4; i += 128)
        reinterpret_cast<float4 *>(Sg)[i] = reinterpret_cast<const float4 *>(&sm.S[0][0])[i];
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
    return cudaFuncSetAttribute(gdn_prefill_chunk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                (int)sizeof(ChunkSmem));
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
    gdn_prefill_chunk_kernel<<<2 * p.Hv, 128, sizeof(ChunkSmem), stream>>>(
        p.ssm, reinterpret_cast<const __nv_bfloat16 *>(p.q_hat), reinterpret_cast<const __nv_bfloat16 *>(p.k_hat),
        p.v_io, p.lg, p.beta_gate, p.T, p.Hk, p.Hv);
    if ((e = cudaGetLastError()) != cudaSuccess) return e;
    gdn_prefill_out_kernel<<<(unsigned)p.T, 256, 0, stream>>>(p.v_io, reinterpret_cast<const __nv_bfloat16 *>(p.z), p.norm_w,
                                                   reinterpret_cast<__nv_bfloat16 *>(p.out), p.Hv, p.eps);
    return cudaGetLastError();
}

}  // namespace mfc
