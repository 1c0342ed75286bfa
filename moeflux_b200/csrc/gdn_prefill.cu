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
//      logs; only ratios gamma_t/gamma_i with i <= t are ever formed):
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
// grid (T, 2*Hk): block (t, b): b < Hk -> q and k channels of k-head b (+ norms);
// b >= Hk -> a 512-channel slice of v, and block b == Hk also the per-head gates.
__global__ void __launch_bounds__(128)
gdn_prefill_conv_kernel(const __nv_bfloat16 *x, const __nv_bfloat16 *alpha, const __nv_bfloat16 *beta,
                        float *ring, int slot0, const uint16_t *conv_w, const float *a_log,
                        const uint16_t *dt_bias, __nv_bfloat16 *q_hat, __nv_bfloat16 *k_hat, float *v_out,
                        float *lg_out, float *beta_out, int T, int Hk, int Hv, int conv_dim) {
    __shared__ float s_red[8];
    const int t = blockIdx.x, b = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int total_key = Hk * GDN_DIM;
    // input of token tt (< 0: history row from the ring), channel c
    auto xin = [&](int tt, int c) -> float {
        if (tt >= 0) return __bfloat162float(x[(size_t)tt * conv_dim + c]);
        return ring[(size_t)((slot0 + tt) & 3) * conv_dim + c];  // token -1 sits in slot0-1, etc.
    };
    auto conv = [&](int c) -> float {
        const uint2 wb = *reinterpret_cast<const uint2 *>(conv_w + (size_t)c * 4);
        float acc = fmaf(xin(t - 3, c), bf16_bits_to_f32((uint16_t)(wb.x & 0xffffu)), 0.0f);
        acc = fmaf(xin(t - 2, c), bf16_bits_to_f32((uint16_t)(wb.x >> 16)), acc);
        acc = fmaf(xin(t - 1, c), bf16_bits_to_f32((uint16_t)(wb.y & 0xffffu)), acc);
        acc = fmaf(xin(t, c), bf16_bits_to_f32((uint16_t)(wb.y >> 16)), acc);
        return acc / (1.0f + expf(-acc));
    };
    if (b < Hk) {
        const float yq = conv(b * GDN_DIM + tid);
        const float yk = conv(total_key + b * GDN_DIM + tid);
        const float sq = warp_sum(yq * yq), sk = warp_sum(yk * yk);
        if (lane == 0) {
            s_red[warp] = sq;
            s_red[4 + warp] = sk;
        }
        __syncthreads();
        const float tq = (s_red[0] + s_red[1]) + (s_red[2] + s_red[3]);
        const float tk = (s_red[4] + s_red[5]) + (s_red[6] + s_red[7]);
        const float inv_scale = 1.0f / sqrtf((float)GDN_DIM);
        const float iq = 1.0f / sqrtf(tq / (float)GDN_DIM + 1e-6f), ik = 1.0f / sqrtf(tk / (float)GDN_DIM + 1e-6f);
        q_hat[((size_t)t * Hk + b) * GDN_DIM + tid] = __float2bfloat16_rn(yq * iq * inv_scale * inv_scale);
        k_hat[((size_t)t * Hk + b) * GDN_DIM + tid] = __float2bfloat16_rn(yk * ik * inv_scale);
    } else {
        const int v_per_block = (Hv * GDN_DIM) / Hk;  // channels of v handled by one block
        const int c0 = (b - Hk) * v_per_block;
        for (int i = tid; i < v_per_block; i += blockDim.x) v_out[(size_t)t * Hv * GDN_DIM + c0 + i] = conv(2 * total_key + c0 + i);
        if (b == Hk && tid < Hv) {
            const float a_val = __bfloat162float(alpha[(size_t)t * Hv + tid]);
            const float dt_b = bf16_bits_to_f32(dt_bias[tid]);
            const float softplus = logf(1.0f + expf(a_val + dt_b));
            lg_out[(size_t)t * Hv + tid] = -expf(a_log[tid]) * softplus;  // log of the decay g
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
    __nv_bfloat16 K[CH][LDK];         // k^ of the chunk (later scaled in place)     17 KiB
    __nv_bfloat16 Q[CH][LDK];         //                                             17 KiB
    float A[CH][LDA];                 // strictly lower triangular system            16.25 KiB
    float Bm[CH][DVC + 1];            // right-hand side                             16.25 KiB
    __nv_bfloat16 W[CH][LDT];         // decay-masked Q K^T                           9 KiB
    __nv_bfloat16 Ut[DVC][LDT];       // U transposed: [value row][token]             9 KiB
    float lg[CH];                     // cumulative log decay, inclusive
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
    for (int c = 0; c < n_chunks; c++) {
        const int tok0 = c * CH;
        __syncthreads();  // previous chunk is done with every buffer
        // ---- stage 0: operands of the chunk; tokens past T act as "no token" ----
        for (int i = tid; i < CH * (GDN_DIM / 8); i += 128) {
            const int r = i >> 4, cc = (i & 15) * 8;
            uint4 kq = make_uint4(0, 0, 0, 0), qq = make_uint4(0, 0, 0, 0);
            if (tok0 + r < T) {
                kq = *reinterpret_cast<const uint4 *>(k_hat + ((size_t)(tok0 + r) * Hk + j) * GDN_DIM + cc);
                qq = *reinterpret_cast<const uint4 *>(q_hat + ((size_t)(tok0 + r) * Hk + j) * GDN_DIM + cc);
            }
            *reinterpret_cast<uint4 *>(&sm.K[r][cc]) = kq;
            *reinterpret_cast<uint4 *>(&sm.Q[r][cc]) = qq;
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
        // ---- stage 1: A = beta (gamma_t/gamma_i) K K^T (i < t);  W = (gamma_t/gamma_i) Q K^T (i <= t) ----
        {
            float acc[8][4];
#pragma unroll
            for (int n = 0; n < 8; n++) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.0f;
            warp_gemm_nmajor<8, 8>(acc, &sm.K[16 * warp][0], LDK, &sm.K[0][0], LDK, lane);
            const float b0 = sm.bt[r0], b1 = sm.bt[r1];
#pragma unroll
            for (int n = 0; n < 8; n++)
#pragma unroll
                for (int e = 0; e < 2; e++) {
                    const int col = 8 * n + 2 * t4 + e;
                    sm.A[r0][col] = (col < r0) ? b0 * expf(lg0 - sm.lg[col]) * acc[n][e] : 0.0f;
                    sm.A[r1][col] = (col < r1) ? b1 * expf(lg1 - sm.lg[col]) * acc[n][2 + e] : 0.0f;
                }
#pragma unroll
            for (int n = 0; n < 8; n++) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.0f;
            warp_gemm_nmajor<8, 8>(acc, &sm.Q[16 * warp][0], LDK, &sm.K[0][0], LDK, lane);
#pragma unroll
            for (int n = 0; n < 8; n++) {
                const int col = 8 * n + 2 * t4;
                const float w00 = (col <= r0) ? expf(lg0 - sm.lg[col]) * acc[n][0] : 0.0f;
                const float w01 = (col + 1 <= r0) ? expf(lg0 - sm.lg[col + 1]) * acc[n][1] : 0.0f;
                const float w10 = (col <= r1) ? expf(lg1 - sm.lg[col]) * acc[n][2] : 0.0f;
                const float w11 = (col + 1 <= r1) ? expf(lg1 - sm.lg[col + 1]) * acc[n][3] : 0.0f;
                *reinterpret_cast<uint32_t *>(&sm.W[r0][col]) = pack_bf16x2(w00, w01);
                *reinterpret_cast<uint32_t *>(&sm.W[r1][col]) = pack_bf16x2(w10, w11);
            }
        }
        // ---- stage 2: Bm = beta (V - gamma K S0^T) ----
        {
            float acc[8][4];
#pragma unroll
            for (int n = 0; n < 8; n++) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.0f;
            warp_gemm_nmajor<8, 8>(acc, &sm.K[16 * warp][0], LDK, &sm.Sb[0][0], LDK, lane);
            const float b0 = sm.bt[r0], b1 = sm.bt[r1], e0 = expf(lg0), e1 = expf(lg1);
            const bool in0 = tok0 + r0 < T, in1 = tok0 + r1 < T;
#pragma unroll
            for (int n = 0; n < 8; n++)
#pragma unroll
                for (int e = 0; e < 2; e++) {
                    const int col = 8 * n + 2 * t4 + e;
                    const float v0 = in0 ? v_io[(size_t)(tok0 + r0) * Hv * GDN_DIM + vcol0 + col] : 0.0f;
                    const float v1 = in1 ? v_io[(size_t)(tok0 + r1) * Hv * GDN_DIM + vcol0 + col] : 0.0f;
                    sm.Bm[r0][col] = b0 * (v0 - e0 * acc[n][e]);
                    sm.Bm[r1][col] = b1 * (v1 - e1 * acc[n][2 + e]);
                }
        }
        __syncthreads();
        // ---- stage 3: forward substitution (I + A) U = Bm, one thread per value column ----
        if (tid < DVC) {
            float u[CH];
#pragma unroll
            for (int t = 0; t < CH; t++) {
                float s = sm.Bm[t][tid];
#pragma unroll
                for (int i = 0; i < t; i++) s = fmaf(-sm.A[t][i], u[i], s);
                u[t] = s;
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
            warp_gemm_nmajor<8, 8>(acc, &sm.Q[16 * warp][0], LDK, &sm.Sb[0][0], LDK, lane);
            const float e0 = expf(lg0), e1 = expf(lg1);
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
            const float f = expf(lgC - sm.lg[r]);
            __nv_bfloat162 kv = *reinterpret_cast<__nv_bfloat162 *>(&sm.K[r][cc]);
            *reinterpret_cast<uint32_t *>(&sm.K[r][cc]) = pack_bf16x2(__low2float(kv) * f, __high2float(kv) * f);
        }
        __syncthreads();
        {
            float acc[16][4];
#pragma unroll
            for (int n = 0; n < 16; n++) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.0f;
            warp_gemm_kmajor<16, 4>(acc, &sm.Ut[16 * warp][0], LDT, &sm.K[0][0], LDK, lane);
            const float gC = expf(lgC);
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
// grid (T, Hv), 128 threads: out = o * rsqrt(mean o^2 + eps) * w * silu(z), or out = o.
__global__ void __launch_bounds__(128)
gdn_prefill_out_kernel(const float *o_raw, const __nv_bfloat16 *z, const uint16_t *norm_w, __nv_bfloat16 *out,
                       int Hv, float eps) {
    __shared__ float s_red[4];
    const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    const size_t idx = ((size_t)t * Hv + h) * GDN_DIM + tid;
    const float o = o_raw[idx];
    if (z == nullptr) {
        out[idx] = __float2bfloat16_rn(o);
        return;
    }
    const float ss = warp_sum(o * o);
    if ((tid & 31) == 0) s_red[tid >> 5] = ss;
    __syncthreads();
    const float tot = (s_red[0] + s_red[1]) + (s_red[2] + s_red[3]);
    const float inv_rms = 1.0f / sqrtf(tot / (float)GDN_DIM + eps);
    const float zv = __bfloat162float(z[idx]);
    const float silu_z = zv / (1.0f + expf(-zv));
    out[idx] = __float2bfloat16_rn(o * inv_rms * bf16_bits_to_f32(norm_w[tid]) * silu_z);
}

}  // namespace

cudaError_t gdn_prefill_configure() {
    return cudaFuncSetAttribute(gdn_prefill_chunk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                (int)sizeof(ChunkSmem));
}

cudaError_t launch_gdn_prefill(const GdnPrefillParams &p, cudaStream_t stream) {
    if (p.T <= 0) return cudaSuccess;
    const __nv_bfloat16 *x = reinterpret_cast<const __nv_bfloat16 *>(p.qkv);
    dim3 g1((unsigned)p.T, (unsigned)(2 * p.Hk), 1);
    gdn_prefill_conv_kernel<<<g1, 128, 0, stream>>>(
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
    dim3 g3((unsigned)p.T, (unsigned)p.Hv, 1);
    gdn_prefill_out_kernel<<<g3, 128, 0, stream>>>(p.v_io, reinterpret_cast<const __nv_bfloat16 *>(p.z), p.norm_w,
                                                   reinterpret_cast<__nv_bfloat16 *>(p.out), p.Hv, p.eps);
    return cudaGetLastError();
}

}  // namespace mfc
