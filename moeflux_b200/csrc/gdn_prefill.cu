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
#include "tcgen05.cuh"

namespace mfc {

namespace {

constexpr int CH = 64;          // tokens per chunk
constexpr int DVC = 64;         // value rows per CTA
constexpr int LDK = GDN_DIM + 8;  // padded leading dim (bf16) of [.][128] operand tiles

// ------------------------------------------------------------------ 1. conv / norm / gates
// grid (ceil(T / CONV_TT), conv_dim / 2048), 256 threads: a thread owns 8 consecutive channels and walks CONV_TT
// consecutive tokens with the three previous input rows in registers, so every input row is loaded once (one
// 16-byte load per token and thread, eight of them in flight) and the taps once per CONV_TT tokens.  (The first
// version gave every thread one token: four row loads and a re-read of the taps per token, 225 us for 8192 tokens.)
// A q or k head is 128 channels = 16 neighbouring lanes, reduced by shuffles.  Block y == 0 also computes the
// per-head gates.  SiLU uses ex2.approx and an approximate division (the results feed bf16 operands).
constexpr int CONV_TT = 32;
constexpr int CONV_UNROLL = 8;
__global__ void __launch_bounds__(256, 2)
gdn_prefill_conv_kernel(const __nv_bfloat16 *x, const __nv_bfloat16 *alpha, const __nv_bfloat16 *beta,
                        float *ring, int slot0, const uint16_t *conv_w, const float *a_log,
                        const uint16_t *dt_bias, __nv_bfloat16 *q_hat, __nv_bfloat16 *k_hat, float *v_out,
                        float *lg_out, float *beta_out, int T, int Hk, int Hv, int conv_dim) {
    const int t0 = blockIdx.x * CONV_TT, tid = threadIdx.x;
    const int c0 = (blockIdx.y * 256 + tid) * 8;
    const int total_key = Hk * GDN_DIM;
    const bool in_c = c0 < conv_dim;
    const int t_end = min(t0 + CONV_TT, T);
    float win[3][8];  // the rows before the current token: win[0] is the oldest
    float wf[8][4];   // taps of the 8 channels
    auto unpack = [](const uint4 &raw, float (&dst)[8]) {
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int e = 0; e < 4; e++) {
            dst[2 * e] = bf16_bits_to_f32((uint16_t)(w[e] & 0xffffu));
            dst[2 * e + 1] = bf16_bits_to_f32((uint16_t)(w[e] >> 16));
        }
    };
#pragma unroll
    for (int k = 0; k < 3; k++) {
        const int tt = t0 - 3 + k;
#pragma unroll
        for (int e = 0; e < 8; e++) win[k][e] = 0.0f;
        if (in_c) {
            if (tt >= 0) {
                unpack(*reinterpret_cast<const uint4 *>(x + (size_t)tt * conv_dim + c0), win[k]);
            } else {  // history row from the ring: token -1 sits in slot0-1, etc.
                const float *hr = ring + (size_t)((slot0 + tt) & 3) * conv_dim + c0;
#pragma unroll
                for (int e = 0; e < 8; e++) win[k][e] = hr[e];
            }
        }
    }
#pragma unroll
    for (int e2 = 0; e2 < 4; e2++) {  // weights of two channels per 16-byte load
        uint4 wr = make_uint4(0, 0, 0, 0);
        if (in_c) wr = *reinterpret_cast<const uint4 *>(conv_w + (size_t)(c0 + 2 * e2) * 4);
        const uint32_t w[4] = {wr.x, wr.y, wr.z, wr.w};
#pragma unroll
        for (int u = 0; u < 2; u++) {
            wf[2 * e2 + u][0] = bf16_bits_to_f32((uint16_t)(w[2 * u] & 0xffffu));
            wf[2 * e2 + u][1] = bf16_bits_to_f32((uint16_t)(w[2 * u] >> 16));
            wf[2 * e2 + u][2] = bf16_bits_to_f32((uint16_t)(w[2 * u + 1] & 0xffffu));
            wf[2 * e2 + u][3] = bf16_bits_to_f32((uint16_t)(w[2 * u + 1] >> 16));
        }
    }
    const bool is_qk = c0 < 2 * total_key, is_q = c0 < total_key;
    const float inv_scale = 1.0f / sqrtf((float)GDN_DIM);
    for (int tb = t0; tb < t_end; tb += CONV_UNROLL) {  // uniform over the block
        uint4 raw[CONV_UNROLL];
#pragma unroll
        for (int u = 0; u < CONV_UNROLL; u++) {
            raw[u] = make_uint4(0, 0, 0, 0);
            if (in_c && tb + u < t_end) raw[u] = *reinterpret_cast<const uint4 *>(x + (size_t)(tb + u) * conv_dim + c0);
        }
#pragma unroll
        for (int u = 0; u < CONV_UNROLL; u++) {
            const int t = tb + u;
            if (t >= t_end) break;
            float cur[8], y[8];
            unpack(raw[u], cur);
            float ss = 0.0f;
#pragma unroll
            for (int e = 0; e < 8; e++) {
                float acc = fmaf(win[0][e], wf[e][0], 0.0f);
                acc = fmaf(win[1][e], wf[e][1], acc);
                acc = fmaf(win[2][e], wf[e][2], acc);
                acc = fmaf(cur[e], wf[e][3], acc);
                y[e] = __fdividef(acc, 1.0f + __expf(-acc));
                ss += y[e] * y[e];
                win[0][e] = win[1][e];
                win[1][e] = win[2][e];
                win[2][e] = cur[e];
            }
            // q or k: normalise over the head (16 lanes x 8 channels); every lane takes part in the shuffles
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            if (!in_c) continue;
            if (is_qk) {
                const float inv = 1.0f / sqrtf(ss / (float)GDN_DIM + 1e-6f);
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
    }
    if (blockIdx.y == 0 && tid < Hv) {
        const float dt_b = bf16_bits_to_f32(dt_bias[tid]);
        const float neg_a = -expf(a_log[tid]);
        for (int t = t0; t < t_end; t++) {
            const float a_val = __bfloat162float(alpha[(size_t)t * Hv + tid]);
            const float softplus = logf(1.0f + expf(a_val + dt_b));
            lg_out[(size_t)t * Hv + tid] = neg_a * softplus * 1.4426950408889634f;  // log2 of the decay g
            beta_out[(size_t)t * Hv + tid] = 1.0f / (1.0f + expf(-__bfloat162float(beta[(size_t)t * Hv + tid])));
        }
    }
}

// The last three inputs become the conv history (token t goes to slot (slot0 + t) & 3).
__global__ void gdn_prefill_ring_kernel(const __nv_bfloat16 *x, float *ring, int slot0, int T, int conv_dim) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= conv_dim) return;
    for (int t = max(0, T - 3); t < T; t++) ring[(size_t)((slot0 + t) & 3) * conv_dim + c] = __bfloat162float(x[(size_t)t * conv_dim + c]);
}

// ------------------------------------------------------------------ warp-level MMA pieces
// (x0, x1) -> bf16x2 registers hi and mid with x = hi + mid + O(2^-18 |x|); x0 in the low half.
__device__ __forceinline__ void split_bf16x2(float x0, float x1, uint32_t &hi, uint32_t &mid) {
    hi = pack_bf16x2(x0, x1);
    mid = pack_bf16x2(x0 - __uint_as_float(hi << 16), x1 - __uint_as_float(hi & 0xffff0000u));
}
// Two products that share the n-major B operand (element (n, k) at B[n*ldb + k]): acc1 += A1 B, acc2 += A2 B,
// A row-major bf16 (lda), K = KS*16.
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
// acc (16 x 16, two n-tiles) += X (16 x 16, A fragments in hi/mid form) * B^T, where the 16 x 16 block B is
// given in hi/mid form, row-major with leading dimension ldb (element (n, k) at B[n*ldb + k]); the three
// cross products hi*hi, mid*hi, hi*mid are kept.
__device__ __forceinline__ void mma_block_split(float (&acc)[2][4], const uint32_t (&xh)[4], const uint32_t (&xm)[4],
                                                const __nv_bfloat16 *Bh, const __nv_bfloat16 *Bm, int ldb, int lane) {
    const int off = ((lane & 7) + ((lane >> 4) << 3)) * ldb + ((lane >> 3) & 1) * 8;
    uint32_t h0, h1, h2, h3, m0, m1, m2, m3;
    ldmatrix_x4(h0, h1, h2, h3, smem_u32(Bh + off));
    ldmatrix_x4(m0, m1, m2, m3, smem_u32(Bm + off));
    mma_bf16_16816(acc[0], xh, h0, h1);
    mma_bf16_16816(acc[0], xm, h0, h1);
    mma_bf16_16816(acc[0], xh, m0, m1);
    mma_bf16_16816(acc[1], xh, h2, h3);
    mma_bf16_16816(acc[1], xm, h2, h3);
    mma_bf16_16816(acc[1], xh, m2, m3);
}

// ------------------------------------------------------------------ 2a. per-chunk work that does not need the state
// grid (chunks, Hv), 256 threads.  Everything of a chunk that is independent of the
// running state is done here, for all chunks in parallel:
//   lg      <- inclusive prefix sum of log2 g inside the chunk (in place)
//   A_ti    = beta_t (gamma_t/gamma_i) (k_t.k_i), i < t;  L = I + A
//   Wm_ti   = (gamma_t/gamma_i) (q_t.k_i), i <= t                           -> w_mask (bf16)
//   L Wt = diag(beta gamma) K                                               -> w_tilde (bf16)
//   L Ut = diag(beta) V                                                     -> v_io in place (fp32)
// so that the serial kernel is left with U = Ut - Wt S0^T.  The two triangular solves are
// one blocked forward substitution over 16-row blocks with 256 right-hand-side columns:
//   X_k = D_k (B_k - sum_{m<k} A_km X_m),   D_k = L_kk^-1 (16 x 16, by scalar substitution in fp32),
// run transposed (rows = right-hand-side columns) so that the accumulator fragments of X_m^T
// are directly the A operand of the next product; a warp owns 32 of the columns and never
// synchronises with the others inside the solve.  fp32 operands enter mma.sync m16n8k16 as
// two-piece bf16 expansions (hi + mid, three products each), which keeps ~2^-17 relative.
constexpr int LDM = CH + 8;        // bf16 [64][64] tiles
constexpr int LDV = GDN_DIM + 4;   // fp32 [64][128] tile: rows 16-byte aligned, conflict-free column walks
struct IntraSmem {
    __nv_bfloat16 K[CH][LDK];      // k^ of the chunk; overwritten in place by Wt
    union {
        __nv_bfloat16 Q[CH][LDK];  // q^ of the chunk, dead once the products with k^ are in registers
        struct {
            __nv_bfloat16 Mh[CH][LDM];  // hi parts: block (k, m < k) = -A_km, block (k, k) = D_k
            __nv_bfloat16 Mm[CH][LDM];  // mid parts of the same
        };
    };
    float V[CH][LDV];              // v of this head; overwritten in place by Ut
    float Ad[4][16][17];           // diagonal 16 x 16 blocks of A, fp32
    float lg[CH];
    float bt[CH];
};

__global__ void __launch_bounds__(256, 3)
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

    // ---- A and Wm: warp = (16-token row tile mt, 32-column half nh); blocks above the diagonal are skipped ----
    {
        const int mt = warp & 3, nh = warp >> 2;
        const int r0 = 16 * mt + g, r1 = r0 + 8;
        const bool in0 = tok0 + r0 < T, in1 = tok0 + r1 < T;
        const bool active = 32 * nh <= 16 * mt + 15;
        float acc[4][4], acq[4][4];
#pragma unroll
        for (int n = 0; n < 4; n++)
#pragma unroll
            for (int e = 0; e < 4; e++) acc[n][e] = acq[n][e] = 0.0f;
        if (active)
            warp_gemm2_nmajor<4, 8>(acc, acq, &sm.K[16 * mt][0], &sm.Q[16 * mt][0], LDK, &sm.K[32 * nh][0], LDK, lane);
        __syncthreads();  // q^ has been consumed: its memory now takes the M tiles
        if (active) {
            const float lg0 = sm.lg[r0], lg1 = sm.lg[r1], b0 = sm.bt[r0], b1 = sm.bt[r1];
#pragma unroll
            for (int n = 0; n < 4; n++) {
                const int col = 32 * nh + 8 * n + 2 * t4;  // even: col and col+1 lie in the same 16-block
                const float d00 = ex2_approx(lg0 - sm.lg[col]), d01 = ex2_approx(lg0 - sm.lg[col + 1]);
                const float d10 = ex2_approx(lg1 - sm.lg[col]), d11 = ex2_approx(lg1 - sm.lg[col + 1]);
                const float a00 = (col < r0) ? b0 * d00 * acc[n][0] : 0.0f, a01 = (col + 1 < r0) ? b0 * d01 * acc[n][1] : 0.0f;
                const float a10 = (col < r1) ? b1 * d10 * acc[n][2] : 0.0f, a11 = (col + 1 < r1) ? b1 * d11 * acc[n][3] : 0.0f;
                if ((col >> 4) == mt) {  // diagonal block (r0 and r1 are in block mt): kept in fp32
                    sm.Ad[mt][r0 & 15][col & 15] = a00;
                    sm.Ad[mt][r0 & 15][(col & 15) + 1] = a01;
                    sm.Ad[mt][r1 & 15][col & 15] = a10;
                    sm.Ad[mt][r1 & 15][(col & 15) + 1] = a11;
                } else if ((col >> 4) < mt) {
                    uint32_t hi, mid;
                    split_bf16x2(-a00, -a01, hi, mid);
                    *reinterpret_cast<uint32_t *>(&sm.Mh[r0][col]) = hi;
                    *reinterpret_cast<uint32_t *>(&sm.Mm[r0][col]) = mid;
                    split_bf16x2(-a10, -a11, hi, mid);
                    *reinterpret_cast<uint32_t *>(&sm.Mh[r1][col]) = hi;
                    *reinterpret_cast<uint32_t *>(&sm.Mm[r1][col]) = mid;
                }
                if (in0)
                    *reinterpret_cast<uint32_t *>(&w_mask[((size_t)(tok0 + r0) * Hv + h) * CH + col]) =
                        pack_bf16x2((col <= r0) ? d00 * acq[n][0] : 0.0f, (col + 1 <= r0) ? d01 * acq[n][1] : 0.0f);
                if (in1)
                    *reinterpret_cast<uint32_t *>(&w_mask[((size_t)(tok0 + r1) * Hv + h) * CH + col]) =
                        pack_bf16x2((col <= r1) ? d10 * acq[n][2] : 0.0f, (col + 1 <= r1) ? d11 * acq[n][3] : 0.0f);
            }
        } else {  // nothing to the right of the diagonal: Wm is zero there
#pragma unroll
            for (int n = 0; n < 4; n++) {
                const int col = 32 * nh + 8 * n + 2 * t4;
                if (in0) *reinterpret_cast<uint32_t *>(&w_mask[((size_t)(tok0 + r0) * Hv + h) * CH + col]) = 0u;
                if (in1) *reinterpret_cast<uint32_t *>(&w_mask[((size_t)(tok0 + r1) * Hv + h) * CH + col]) = 0u;
            }
        }
    }
    __syncthreads();

    // ---- D_k = (I + A_kk)^-1: thread = (block k, column c), 16-step substitution in fp32 ----
    if (tid < 64) {
        const int k = tid >> 4, c = tid & 15;
        float x[16];
#pragma unroll
        for (int i = 0; i < 16; i++) {
            float s = (i == c) ? 1.0f : 0.0f;
#pragma unroll
            for (int jj = 0; jj < i; jj++) s = fmaf(-sm.Ad[k][i][jj], x[jj], s);
            x[i] = s;
        }
#pragma unroll
        for (int i = 0; i < 16; i++) {
            const __nv_bfloat16 hi = __float2bfloat16_rn(x[i]);
            sm.Mh[16 * k + i][16 * k + c] = hi;
            sm.Mm[16 * k + i][16 * k + c] = __float2bfloat16_rn(x[i] - __bfloat162float(hi));
        }
    }
    __syncthreads();

    // ---- blocked forward substitution, transposed: a warp owns right-hand-side columns
    //      [16 warp, 16 warp + 16) of diag(beta gamma) K and the same columns of diag(beta) V ----
#pragma unroll 1
    for (int which = 0; which < 2; which++) {
        const int n0 = 16 * warp;  // this warp's 16 columns; fragment rows g and g+8 are columns n0+g, n0+g+8
        uint32_t xh[3][4], xm[3][4];
#pragma unroll
        for (int k = 0; k < 4; k++) {
            float acc[2][4];
#pragma unroll
            for (int jn = 0; jn < 2; jn++) {
                const int t = 16 * k + 8 * jn + 2 * t4;
                if (which == 0) {
                    const float f0 = sm.bt[t] * ex2_approx(sm.lg[t]), f1 = sm.bt[t + 1] * ex2_approx(sm.lg[t + 1]);
                    acc[jn][0] = f0 * __bfloat162float(sm.K[t][n0 + g]);
                    acc[jn][1] = f1 * __bfloat162float(sm.K[t + 1][n0 + g]);
                    acc[jn][2] = f0 * __bfloat162float(sm.K[t][n0 + g + 8]);
                    acc[jn][3] = f1 * __bfloat162float(sm.K[t + 1][n0 + g + 8]);
                } else {
                    const float f0 = sm.bt[t], f1 = sm.bt[t + 1];
                    acc[jn][0] = f0 * sm.V[t][n0 + g];
                    acc[jn][1] = f1 * sm.V[t + 1][n0 + g];
                    acc[jn][2] = f0 * sm.V[t][n0 + g + 8];
                    acc[jn][3] = f1 * sm.V[t + 1][n0 + g + 8];
                }
            }
#pragma unroll
            for (int m = 0; m < k; m++)
                mma_block_split(acc, xh[m], xm[m], &sm.Mh[16 * k][16 * m], &sm.Mm[16 * k][16 * m], LDM, lane);
            // Y^T (accumulator fragments) -> A fragments, then X_k^T = Y^T D_k^T
            uint32_t yh[4], ym[4];
            split_bf16x2(acc[0][0], acc[0][1], yh[0], ym[0]);
            split_bf16x2(acc[0][2], acc[0][3], yh[1], ym[1]);
            split_bf16x2(acc[1][0], acc[1][1], yh[2], ym[2]);
            split_bf16x2(acc[1][2], acc[1][3], yh[3], ym[3]);
            float out[2][4];
#pragma unroll
            for (int jn = 0; jn < 2; jn++) out[jn][0] = out[jn][1] = out[jn][2] = out[jn][3] = 0.0f;
            mma_block_split(out, yh, ym, &sm.Mh[16 * k][16 * k], &sm.Mm[16 * k][16 * k], LDM, lane);
            if (k < 3) {
                split_bf16x2(out[0][0], out[0][1], xh[k][0], xm[k][0]);
                split_bf16x2(out[0][2], out[0][3], xh[k][1], xm[k][1]);
                split_bf16x2(out[1][0], out[1][1], xh[k][2], xm[k][2]);
                split_bf16x2(out[1][2], out[1][3], xh[k][3], xm[k][3]);
            }
            // in place: element (t, column) is read and written by this thread only
#pragma unroll
            for (int jn = 0; jn < 2; jn++) {
                const int t = 16 * k + 8 * jn + 2 * t4;
                if (which == 0) {
                    sm.K[t][n0 + g] = __float2bfloat16_rn(out[jn][0]);
                    sm.K[t + 1][n0 + g] = __float2bfloat16_rn(out[jn][1]);
                    sm.K[t][n0 + g + 8] = __float2bfloat16_rn(out[jn][2]);
                    sm.K[t + 1][n0 + g + 8] = __float2bfloat16_rn(out[jn][3]);
                } else {
                    sm.V[t][n0 + g] = out[jn][0];
                    sm.V[t + 1][n0 + g] = out[jn][1];
                    sm.V[t][n0 + g + 8] = out[jn][2];
                    sm.V[t + 1][n0 + g + 8] = out[jn][3];
                }
            }
        }
    }
    __syncthreads();

    // ---- copy out: Wt (bf16) and Ut (fp32), 16-byte stores, valid rows only ----
    const int n_in = min(CH, T - tok0);
    for (int i = tid; i < CH * (GDN_DIM / 8); i += 256) {
        const int r = i >> 4, col = (i & 15) * 8;
        if (r < n_in)
            *reinterpret_cast<uint4 *>(w_tilde + ((size_t)(tok0 + r) * Hv + h) * GDN_DIM + col) =
                *reinterpret_cast<const uint4 *>(&sm.K[r][col]);
    }
    for (int i = tid; i < CH * (GDN_DIM / 4); i += 256) {
        const int r = i >> 5, col = (i & 31) * 4;
        if (r < n_in)
            *reinterpret_cast<float4 *>(v_io + (size_t)(tok0 + r) * vrow + (size_t)h * GDN_DIM + col) =
                *reinterpret_cast<const float4 *>(&sm.V[r][col]);
    }
}

// ------------------------------------------------------------------ 2b. the serial part: state across chunks
// grid 2*Hv, 320 threads.  One CTA owns 64 of the 128 value rows of one v-head and keeps
// that half-state, transposed (key index = TMEM lane, value row = column), in tensor
// memory in fp32 across all chunks.  Per chunk, three groups of tcgen05.mma (M = 128,
// N = 64, bf16 operands, fp32 accumulate):
//   D1 = [Wt ; Q] S0^T          rows 0-63: Wt S0^T, rows 64-127: Q S0^T        (K = 128 key dims)
//   ST = gamma_C ST + K^T Us    Us = diag(gamma_C/gamma_t) U                   (K = 64 tokens)
//   D2 = [ . ; Wm] U            rows 64-127: Wm U                              (K = 64 tokens)
// with U = Ut - D1[0:64] and O = diag(gamma) D1[64:128] + D2[64:128] computed by eight
// epilogue warps (thread = TMEM lane x half of the 64 columns).  Operands arrive by TMA
// (128-byte swizzle) into a ring (two stages for what a chunk needs first, three for the rest); S0 (bf16), U and Us are written to shared
// memory by the epilogue warps as MN-major operands.  Warp 8 issues every MMA, warp 9
// every TMA load.  The recurrence S0 -> D1 -> U -> ST -> S0 is the critical path; the read-out
// (D2, O) of chunk c is finished under the first product of chunk c+1.  Every mbarrier
// wait is bounded; a wait that expires sets a status bit and the CTA frees its TMEM and
// leaves.
// operand ring: two A stages (Wt, q^, Ut: needed first in a chunk) and three B stages (k^, Wm: needed last)
constexpr uint32_t SA_A1 = 0;                    // [2 boxes][128 rows][128 B]: rows 0-63 Wt, rows 64-127 q^
constexpr uint32_t SA_UT = SA_A1 + 32768;        // [2 boxes][64 rows][128 B] fp32
constexpr uint32_t STAGE_A_BYTES = SA_UT + 16384;  // 48 KiB
constexpr uint32_t SB_K = 0;                     // [2 boxes][64 rows][128 B]
constexpr uint32_t SB_WM = SB_K + 16384;         // [64 rows][128 B]
constexpr uint32_t STAGE_B_BYTES = SB_WM + 8192;   // 24 KiB
constexpr uint32_t TC_OFF_B = 2 * STAGE_A_BYTES;
constexpr uint32_t TC_OFF_SB = TC_OFF_B + 3 * STAGE_B_BYTES;  // [128 key rows][128 B]
constexpr uint32_t TC_OFF_U = TC_OFF_SB + 16384;  // [64 token rows][128 B]
constexpr uint32_t TC_OFF_US = TC_OFF_U + 8192;
constexpr uint32_t TC_OFF_BAR = TC_OFF_US + 8192;
constexpr uint32_t TC_SMEM = TC_OFF_BAR + 128 + 1024;
constexpr uint32_t TC_TMEM_COLS = 256;
constexpr uint32_t TM_ST = 0, TM_D1 = 64, TM_D2 = 128;
constexpr int TC_THREADS = 320;

// one arrival for the whole warp, after every lane's earlier writes and fences
__device__ __forceinline__ void warp_arrive(uint64_t *bar) {
    __syncwarp();
    if ((threadIdx.x & 31) == 0) mbar_arrive(bar);
}
// address of 16-byte chunk c of row r in a [rows][128 B] region laid out with the 128-byte swizzle
__device__ __forceinline__ uint8_t *sw128_chunk(uint8_t *base, int r, int c) { return base + r * 128 + ((c ^ (r & 7)) << 4); }

__global__ void __launch_bounds__(TC_THREADS, 1)
gdn_prefill_state_kernel(const __grid_constant__ CUtensorMap wt_map, const __grid_constant__ CUtensorMap q_map,
                         const __grid_constant__ CUtensorMap k_map, const __grid_constant__ CUtensorMap wm_map,
                         const __grid_constant__ CUtensorMap ut_map, float *ssm, float *v_io, const float *lgc, int T,
                         int Hk, int Hv, unsigned *status) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + TC_OFF_BAR);
    uint64_t *full_a = bars + 0;    // [2] TMA: an A stage has landed
    uint64_t *full_b = bars + 2;    // [3] TMA: a B stage has landed
    uint64_t *d1_ready = bars + 5;  // tcgen05.commit
    uint64_t *d2_ready = bars + 6;  // tcgen05.commit
    uint64_t *g3_done = bars + 7;   // tcgen05.commit: the state update of a chunk has been accumulated
    // the next four are arrived on once per warp (lane 0, after __syncwarp): hundreds of per-thread arrivals on
    // one barrier serialise in the shared-memory unit and were the larger part of a chunk's latency
    uint64_t *u_ready = bars + 8;   // 4 warps: U and Us are in shared memory, D1[0:64] and Ut have been read
    uint64_t *s_ready = bars + 9;   // 8 warps: S0 (bf16) is in shared memory, D1 has been read
    uint64_t *st_ready = bars + 10; // 8 warps: ST has been scaled by the decay of the coming chunk
    uint64_t *o_done = bars + 11;   // 4 warps: D2 of the previous chunk has been read
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 12);
    volatile int *s_fail = reinterpret_cast<volatile int *>(bars + 13);

    const int tid = threadIdx.x, warp = tid >> 5, lane_id = tid & 31;
    const int h = blockIdx.x >> 1, half = blockIdx.x & 1;
    const int j = h / (Hv / Hk);
    const size_t vrow = (size_t)Hv * GDN_DIM;
    const int vcol0 = h * GDN_DIM + half * DVC;  // first value channel of this CTA in [T][Hv*128] arrays
    float *Sg = ssm + ((size_t)h * GDN_DIM + half * DVC) * GDN_DIM;
    const int n_chunks = (T + CH - 1) / CH;

    if (tid == 0) {
        prefetch_tmap(&wt_map);
        prefetch_tmap(&q_map);
        prefetch_tmap(&k_map);
        prefetch_tmap(&wm_map);
        prefetch_tmap(&ut_map);
        for (int i = 0; i < 5; i++) mbar_init(&bars[i], 1);
        mbar_init(d1_ready, 1);
        mbar_init(d2_ready, 1);
        mbar_init(g3_done, 1);
        mbar_init(u_ready, 4);
        mbar_init(s_ready, 8);
        mbar_init(st_ready, 8);
        mbar_init(o_done, 4);
        *s_fail = 0;
        mbar_fence_init();
    }
    if (warp == 0) {
        tmem_alloc(tmem_slot, TC_TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    bool ok = true;
    auto lg_at = [&](int tok) { return lgc[(size_t)min(tok, T - 1) * Hv + h]; };

    if (warp == 9) {
        // ================= producer: one lane issues every TMA load =================
        if (lane_id == 0) {
            auto load_a = [&](int cc) {  // Wt, q^ and Ut of chunk cc
                uint8_t *st = smem + (cc & 1) * STAGE_A_BYTES;
                uint64_t *bar = &full_a[cc & 1];
                mbar_expect_tx(bar, STAGE_A_BYTES);
#pragma unroll
                for (int b = 0; b < 2; b++) {
                    tma_load_2d(st + SA_A1 + b * 16384, &wt_map, h * GDN_DIM + b * 64, cc * CH, bar);
                    tma_load_2d(st + SA_A1 + b * 16384 + 8192, &q_map, j * GDN_DIM + b * 64, cc * CH, bar);
                    tma_load_2d(st + SA_UT + b * 8192, &ut_map, vcol0 + b * 32, cc * CH, bar);
                }
            };
            auto load_b = [&](int cc) {  // k^ and Wm of chunk cc
                uint8_t *st = smem + TC_OFF_B + (cc % 3) * STAGE_B_BYTES;
                uint64_t *bar = &full_b[cc % 3];
                mbar_expect_tx(bar, STAGE_B_BYTES);
#pragma unroll
                for (int b = 0; b < 2; b++) tma_load_2d(st + SB_K + b * 8192, &k_map, j * GDN_DIM + b * 64, cc * CH, bar);
                tma_load_2d(st + SB_WM, &wm_map, h * CH, cc * CH, bar);
            };
            load_a(0);
            load_b(0);
            if (n_chunks > 1) {
                load_a(1);
                load_b(1);
            }
            if (n_chunks > 2) load_b(2);
            for (int c = 0; c + 2 < n_chunks && ok; c++) {
                if (c >= 1) {
                    // the B stage of chunk c-1 is free once its read-out product (issued after its state update) has completed
                    ok = mbar_wait_bounded(d2_ready, (unsigned)(c - 1) & 1u);
                    if (!ok) break;
                    load_b(c + 2);
                }
                // Wt, q^ (read by the first product, complete once D1 was read) and Ut of chunk c's A stage are free at u_ready
                ok = mbar_wait_bounded(u_ready, (unsigned)c & 1u);
                if (!ok) break;
                load_a(c + 2);
            }
            if (!ok) *s_fail = 1;
        }
    } else if (warp == 8) {
        // ================= issuer: one lane drives the tensor core =================
        if (lane_id == 0) {
            constexpr uint32_t IDESC_KN = idesc_bf16(DVC, 1, 0);  // A K-major, B MN-major
            constexpr uint32_t IDESC_MN = idesc_bf16(DVC, 1, 1);  // A and B MN-major
            const uint32_t sbase = smem_u32(smem);
            const uint64_t sb_desc = smem_desc_sw128(sbase + TC_OFF_SB, 16384, 1024);
            const uint64_t u_desc = smem_desc_sw128(sbase + TC_OFF_U, 8192, 1024);
            const uint64_t us_desc = smem_desc_sw128(sbase + TC_OFF_US, 8192, 1024);
            for (int c = 0; c < n_chunks && ok; c++) {
                const uint32_t sta = sbase + (c & 1) * STAGE_A_BYTES;
                const uint32_t stb = sbase + TC_OFF_B + (c % 3) * STAGE_B_BYTES;
                const unsigned par = (unsigned)c & 1u;
                ok = mbar_wait_bounded(&full_a[c & 1], (unsigned)(c >> 1) & 1u) && mbar_wait_bounded(s_ready, par);
                if (!ok) break;
                tc_fence_after();
                {
                    const uint64_t a1 = smem_desc_sw128(sta + SA_A1, 16, 1024);
#pragma unroll
                    for (int ks = 0; ks < 8; ks++)
                        tc_mma_bf16(tmem + TM_D1, a1 + (uint64_t)(((ks >> 2) * 16384 + (ks & 3) * 32) >> 4),
                                    sb_desc + (uint64_t)((ks * 2048) >> 4), IDESC_KN, ks > 0);
                    tc_commit(d1_ready);
                }
                ok = mbar_wait_bounded(u_ready, par) && mbar_wait_bounded(st_ready, par) &&
                     mbar_wait_bounded(&full_b[c % 3], (unsigned)(c / 3) & 1u);
                if (!ok) break;
                tc_fence_after();
                {
                    const uint64_t kd = smem_desc_sw128(stb + SB_K, 8192, 1024);  // m = key dim: two 64-wide atoms 8 KiB apart
#pragma unroll
                    for (int ks = 0; ks < 4; ks++)
                        tc_mma_bf16(tmem + TM_ST, kd + (uint64_t)((ks * 2048) >> 4), us_desc + (uint64_t)((ks * 2048) >> 4),
                                    IDESC_MN, 1);
                    tc_commit(g3_done);
                }
                ok = mbar_wait_bounded(o_done, par);  // D2 of chunk c-1 has been read
                if (!ok) break;
                tc_fence_after();
                {
                    // rows 0-63 of this A operand are the 8 KiB in front of Wm (finite k^ data); only rows 64-127 of D2 are used
                    const uint64_t wm = smem_desc_sw128(stb + SB_WM - 8192, 16, 1024);
#pragma unroll
                    for (int ks = 0; ks < 4; ks++)
                        tc_mma_bf16(tmem + TM_D2, wm + (uint64_t)((ks * 32) >> 4), u_desc + (uint64_t)((ks * 2048) >> 4),
                                    IDESC_KN, ks > 0);
                    tc_commit(d2_ready);
                }
            }
            if (!ok) *s_fail = 1;
        }
    } else {
        // ================= epilogue warps: thread = (TMEM lane, half of the 64 columns) =================
        const int quad = warp & 3, ch = warp >> 2;       // lane quadrant, column half
        const int lane = 32 * quad + lane_id;            // TMEM lane = key dim of ST / row of D1, D2
        const int r = lane & 63;                         // token row in D1 / D2 (quadrants 0-1: U rows, 2-3: O rows)
        const uint32_t lane_base = tmem + ((uint32_t)(32 * quad) << 16) + 32 * ch;
        const bool u_role = quad < 2;
        // ---- initial state: element (key dim = lane) of value rows 32 ch .. 32 ch + 31 ----
        {
            float sv[32];
#pragma unroll
            for (int d = 0; d < 32; d++) sv[d] = Sg[(size_t)(32 * ch + d) * GDN_DIM + lane];
#pragma unroll
            for (int cc = 0; cc < 4; cc++) {
                uint32_t w[4];
#pragma unroll
                for (int e = 0; e < 4; e++) w[e] = pack_bf16x2(sv[8 * cc + 2 * e], sv[8 * cc + 2 * e + 1]);
                *reinterpret_cast<uint4 *>(sw128_chunk(smem + TC_OFF_SB, lane, 4 * ch + cc)) = make_uint4(w[0], w[1], w[2], w[3]);
            }
            fence_proxy_async_smem();
            warp_arrive(s_ready);
            const float g0 = ex2_approx(lg_at(CH - 1));
#pragma unroll
            for (int d = 0; d < 32; d++) sv[d] *= g0;
            tmem_st32(lane_base + TM_ST, *reinterpret_cast<float(*)[32]>(&sv[0]));
            tc_wait_st();
            tc_fence_before();
            warp_arrive(st_ready);
        }
        float lg_r = lg_at(r), lg_c = lg_at(CH - 1);
        float o1[32];  // O rows: gamma_t (Q S0^T) of the chunk whose read-out is still open
        // finishes the read-out of chunk cc: O = o1 + D2 -> written over v_io (fp32)
        auto finish_o = [&](int cc) -> bool {
            if (!__all_sync(0xffffffffu, mbar_wait_bounded(d2_ready, (unsigned)cc & 1u))) return false;
            tc_fence_after();
            float d2[32];
            tmem_ld32(lane_base + TM_D2, d2);
            tc_wait_ld();
            const int tok = cc * CH + r;
            if (tok < T) {
                float *dst = v_io + (size_t)tok * vrow + vcol0 + 32 * ch;
#pragma unroll
                for (int q4 = 0; q4 < 8; q4++)
                    *reinterpret_cast<float4 *>(dst + 4 * q4) =
                        make_float4(o1[4 * q4] + d2[4 * q4], o1[4 * q4 + 1] + d2[4 * q4 + 1], o1[4 * q4 + 2] + d2[4 * q4 + 2],
                                    o1[4 * q4 + 3] + d2[4 * q4 + 3]);
            }
            return true;
        };
        for (int c = 0; c < n_chunks && ok; c++) {
            uint8_t *st = smem + (c & 1) * STAGE_A_BYTES;
            const unsigned par = (unsigned)c & 1u;
            // decay logs of the next chunk, requested now
            const float lg_r_next = lg_at((c + 1) * CH + r), lg_c_next = lg_at((c + 1) * CH + CH - 1);
            if (!u_role) {
                if (c > 0) {
                    ok = finish_o(c - 1);
                    if (!ok) break;
                }
                tc_fence_before();
                warp_arrive(o_done);
            } else if (c > 0) {
                // U of chunk c-1 is still the operand of its read-out product until that has completed
                ok = __all_sync(0xffffffffu, mbar_wait_bounded(d2_ready, (unsigned)(c - 1) & 1u));
                if (!ok) break;
            }
            ok = __all_sync(0xffffffffu, mbar_wait_bounded(d1_ready, par) && *s_fail == 0);
            if (!ok) break;
            tc_fence_after();
            float d1[32];
            tmem_ld32(lane_base + TM_D1, d1);
            tc_wait_ld();
            if (u_role) {
                // ---- U = Ut - Wt S0^T ; Us = (gamma_C/gamma_t) U : value rows 32 ch .. 32 ch + 31 of token r ----
                const float f = ex2_approx(lg_c - lg_r);
#pragma unroll
                for (int cc = 0; cc < 4; cc++) {
                    uint32_t wu[4], ws[4];
#pragma unroll
                    for (int e2 = 0; e2 < 2; e2++) {
                        const int d0 = 8 * cc + 4 * e2;
                        const float4 ut = *reinterpret_cast<const float4 *>(sw128_chunk(st + SA_UT + ch * 8192, r, d0 >> 2));
                        const float u0 = ut.x - d1[d0], u1 = ut.y - d1[d0 + 1], u2 = ut.z - d1[d0 + 2], u3 = ut.w - d1[d0 + 3];
                        wu[2 * e2] = pack_bf16x2(u0, u1);
                        wu[2 * e2 + 1] = pack_bf16x2(u2, u3);
                        ws[2 * e2] = pack_bf16x2(u0 * f, u1 * f);
                        ws[2 * e2 + 1] = pack_bf16x2(u2 * f, u3 * f);
                    }
                    *reinterpret_cast<uint4 *>(sw128_chunk(smem + TC_OFF_U, r, 4 * ch + cc)) = make_uint4(wu[0], wu[1], wu[2], wu[3]);
                    *reinterpret_cast<uint4 *>(sw128_chunk(smem + TC_OFF_US, r, 4 * ch + cc)) = make_uint4(ws[0], ws[1], ws[2], ws[3]);
                }
                fence_proxy_async_smem();
                tc_fence_before();
                warp_arrive(u_ready);
            } else {
                const float e = ex2_approx(lg_r);
#pragma unroll
                for (int d = 0; d < 32; d++) o1[d] = d1[d] * e;
            }
            // ---- state pass: S of this chunk -> bf16 operand copy; then the decay of the next chunk ----
            ok = __all_sync(0xffffffffu, mbar_wait_bounded(g3_done, par));
            if (!ok) break;
            tc_fence_after();
            float sv[32];
            tmem_ld32(lane_base + TM_ST, sv);
            tc_wait_ld();
            if (c + 1 < n_chunks) {
#pragma unroll
                for (int cc = 0; cc < 4; cc++) {
                    uint32_t w[4];
#pragma unroll
                    for (int e = 0; e < 4; e++) w[e] = pack_bf16x2(sv[8 * cc + 2 * e], sv[8 * cc + 2 * e + 1]);
                    *reinterpret_cast<uint4 *>(sw128_chunk(smem + TC_OFF_SB, lane, 4 * ch + cc)) = make_uint4(w[0], w[1], w[2], w[3]);
                }
                fence_proxy_async_smem();
                tc_fence_before();
                warp_arrive(s_ready);
                const float gn = ex2_approx(lg_c_next);
#pragma unroll
                for (int d = 0; d < 32; d++) sv[d] *= gn;
                tmem_st32(lane_base + TM_ST, *reinterpret_cast<float(*)[32]>(&sv[0]));
                tc_wait_st();
                tc_fence_before();
                warp_arrive(st_ready);
            } else {
#pragma unroll
                for (int d = 0; d < 32; d++) Sg[(size_t)(32 * ch + d) * GDN_DIM + lane] = sv[d];
            }
            lg_r = lg_r_next;
            lg_c = lg_c_next;
        }
        if (ok && !u_role && n_chunks > 0) ok = finish_o(n_chunks - 1);
        if (!ok && lane_id == 0) *s_fail = 1;
    }
    tc_fence_before();
    __syncthreads();
    if (tid == 0 && *s_fail) atomicOr(status, STATUS_TMA_TIMEOUT);
    if (warp == 0) tmem_dealloc(tmem, TC_TMEM_COLS);
}

// ------------------------------------------------------------------ 3. read-out epilogue
// grid (T), 256 threads: a warp takes heads warp, warp+8, ... (4 values per lane), four heads
// in flight at a time: out = o * rsqrt(mean o^2 + eps) * w * silu(z), or out = o.
__global__ void __launch_bounds__(256)
gdn_prefill_out_kernel(const float *o_raw, const __nv_bfloat16 *z, const uint16_t *norm_w, __nv_bfloat16 *out,
                       int Hv, float eps) {
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float wf[4] = {1.0f, 1.0f, 1.0f, 1.0f};
    if (z != nullptr) {
        const uint2 ww = *reinterpret_cast<const uint2 *>(norm_w + lane * 4);
        wf[0] = bf16_bits_to_f32((uint16_t)(ww.x & 0xffffu));
        wf[1] = bf16_bits_to_f32((uint16_t)(ww.x >> 16));
        wf[2] = bf16_bits_to_f32((uint16_t)(ww.y & 0xffffu));
        wf[3] = bf16_bits_to_f32((uint16_t)(ww.y >> 16));
    }
    for (int hb = warp; hb < Hv; hb += 32) {
        float4 o[4];
        uint2 zz[4];
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const int h = hb + 8 * u;
            if (h < Hv) {
                const size_t idx = ((size_t)t * Hv + h) * GDN_DIM + lane * 4;
                o[u] = *reinterpret_cast<const float4 *>(o_raw + idx);
                if (z != nullptr) zz[u] = *reinterpret_cast<const uint2 *>(z + idx);
            }
        }
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const int h = hb + 8 * u;
            if (h >= Hv) break;  // uniform over the warp
            const size_t idx = ((size_t)t * Hv + h) * GDN_DIM + lane * 4;
            float r[4] = {o[u].x, o[u].y, o[u].z, o[u].w};
            if (z != nullptr) {
                const float tot = warp_sum(o[u].x * o[u].x + o[u].y * o[u].y + o[u].z * o[u].z + o[u].w * o[u].w);
                const float inv_rms = 1.0f / sqrtf(tot / (float)GDN_DIM + eps);
                const float zf[4] = {bf16_bits_to_f32((uint16_t)(zz[u].x & 0xffffu)), bf16_bits_to_f32((uint16_t)(zz[u].x >> 16)),
                                     bf16_bits_to_f32((uint16_t)(zz[u].y & 0xffffu)), bf16_bits_to_f32((uint16_t)(zz[u].y >> 16))};
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const float silu_z = zf[e] / (1.0f + expf(-zf[e]));
                    r[e] = r[e] * inv_rms * wf[e] * silu_z;
                }
            }
            *reinterpret_cast<uint2 *>(out + idx) = make_uint2(pack_bf16x2(r[0], r[1]), pack_bf16x2(r[2], r[3]));
        }
    }
}

}  // namespace

cudaError_t gdn_prefill_configure() {
    cudaError_t e = cudaFuncSetAttribute(gdn_prefill_intra_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)sizeof(IntraSmem));
    if (e != cudaSuccess) return e;
    return cudaFuncSetAttribute(gdn_prefill_state_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TC_SMEM);
}

cudaError_t launch_gdn_prefill(const GdnPrefillParams &p, const GdnPrefillMaps &m, cudaStream_t stream) {
    if (p.T <= 0) return cudaSuccess;
    const __nv_bfloat16 *x = reinterpret_cast<const __nv_bfloat16 *>(p.qkv);
    dim3 g1((unsigned)((p.T + CONV_TT - 1) / CONV_TT), (unsigned)((p.conv_dim + 2047) / 2048), 1);
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
    gdn_prefill_state_kernel<<<2 * p.Hv, TC_THREADS, TC_SMEM, stream>>>(m.wt, m.q, m.k, m.wm, m.ut, p.ssm, p.v_io, p.lg, p.T, p.Hk,
                                                               p.Hv, p.status);
    if ((e = cudaGetLastError()) != cudaSuccess) return e;
    gdn_prefill_out_kernel<<<(unsigned)p.T, 256, 0, stream>>>(p.v_io, reinterpret_cast<const __nv_bfloat16 *>(p.z), p.norm_w,
                                                   reinterpret_cast<__nv_bfloat16 *>(p.out), p.Hv, p.eps);
    return cudaGetLastError();
}

}  // namespace mfc
