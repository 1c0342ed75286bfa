// Fused GatedDeltaNet decode step for sm_100a.
//
// One launch performs, for every (layer, sequence) item in the list, what the
// reference does with five kernels (crates/moeflux/shaders/shaders.metal:
// conv1d_step :1213-1244, rms_norm_qk :1254-1303, compute_decay_beta :1312-1327,
// gated_delta_net_step :1154-1194, gated_rms_norm :1337-1370):
//
//   y      = silu(conv4(history, x))               per channel, history advanced
//   q̂, k̂  = q * rsqrt(mean q² + 1e-6) / 128,  k * rsqrt(mean k² + 1e-6) / sqrt(128)
//   g, β   = exp(-exp(A_log) * softplus(α + dt_bias)),  sigmoid(b)
//   per state row vi:  S = g S;  kv = S·k̂;  δ = (v[vi] - kv) β;  S += k̂ δ;  o[vi] = S·q̂
//   out    = o * rsqrt(mean o² + eps) * w * silu(z)          (only when z is given)
//
// Work split.  The 128x128 fp32 state of one (item, v-head) is cut into blocks
// of ROWS value rows; one CTA owns one block and the 128/ROWS CTAs of a head
// form a thread-block cluster (the gated norm needs the head-wide mean of o²,
// exchanged through distributed shared memory).  A warp owns ROWS/8 rows; a
// lane holds four consecutive key elements of a row, so one row is one 512-byte
// coalesced access per warp, read once and written once.  All state loads of
// the first four rows of each warp are issued before the conv/norm prologue so
// that HBM latency overlaps it.
//
// Conv history.  The reference shifts a [3][conv_dim] history in place, which
// would race here (the CTAs of four v-heads read the same q/k channels).  The
// history is a 4-slot ring instead: step t reads slots t+1, t+2, t+3 (mod 4)
// and writes x into slot t (mod 4), which nobody reads during that step.
#include <cooperative_groups.h>

#include "common.cuh"
#include "kernels.h"

namespace cg = cooperative_groups;

namespace mfc {

namespace {

__device__ __forceinline__ float conv_channel(const float *ring, const float *x,
                                              const uint16_t *w, int conv_dim, int slot, int c,
                                              bool write_ring, float *ring_w) {
    const uint2 wb = *reinterpret_cast<const uint2 *>(w + (size_t)c * 4);
    const float w0 = bf16_bits_to_f32((uint16_t)(wb.x & 0xffffu));
    const float w1 = bf16_bits_to_f32((uint16_t)(wb.x >> 16));
    const float w2 = bf16_bits_to_f32((uint16_t)(wb.y & 0xffffu));
    const float w3 = bf16_bits_to_f32((uint16_t)(wb.y >> 16));
    const float h0 = ring[(size_t)((slot + 1) & 3) * conv_dim + c];
    const float h1 = ring[(size_t)((slot + 2) & 3) * conv_dim + c];
    const float h2 = ring[(size_t)((slot + 3) & 3) * conv_dim + c];
    const float xi = x[c];
    float acc = fmaf(h0, w0, 0.0f);
    acc = fmaf(h1, w1, acc);
    acc = fmaf(h2, w2, acc);
    acc = fmaf(xi, w3, acc);
    if (write_ring) ring_w[(size_t)slot * conv_dim + c] = xi;
    return acc / (1.0f + expf(-acc));
}

template <int ROWS>
__global__ void __launch_bounds__(256) gdn_decode_kernel(const __grid_constant__ GdnParams p) {
    constexpr int CS = GDN_DIM / ROWS;  // CTAs per head (cluster size)
    constexpr int RPW = ROWS / 8;       // rows per warp
    constexpr int NB = RPW / 4;         // batches of four rows per warp
    static_assert(RPW % 4 == 0 && NB >= 1, "ROWS must be a multiple of 32");

    __shared__ __align__(16) float s_q[GDN_DIM];
    __shared__ __align__(16) float s_k[GDN_DIM];
    __shared__ float s_v[ROWS];
    __shared__ float s_o[ROWS];
    __shared__ float s_red[8];
    __shared__ float s_gb[2];
    __shared__ float s_ss;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int bid = blockIdx.x;
    const int rb = bid % CS;
    const int h = (bid / CS) % p.Hv;
    const int item = bid / (CS * p.Hv);
    const GdnItem it = p.items ? p.items[item] : p.inline_items[item];
    const int vpk = p.Hv / p.Hk;
    const int j = h / vpk;
    const int total_key = p.Hk * GDN_DIM;

    float *S = p.ssm_base + ((size_t)it.state_idx * p.Hv + h) * (GDN_DIM * GDN_DIM) +
               (size_t)(rb * ROWS + warp * RPW) * GDN_DIM + lane * 4;

    // ---- state loads of the first batch go out before anything else ----
    float4 cur[4];
#pragma unroll
    for (int i = 0; i < 4; i++) cur[i] = *reinterpret_cast<const float4 *>(S + (size_t)i * GDN_DIM);

    // ---- prologue: conv + SiLU for q_j, k_j and this block's v rows ----
    const float *x = p.qkv + (size_t)item * p.conv_dim;
    float *ring = p.conv_base + (size_t)it.state_idx * CONV_TAPS * p.conv_dim;
    const uint16_t *cw = p.conv_w + (size_t)it.w_layer * p.conv_dim * 4;
    const bool qk_writer = (h % vpk == 0) && (rb == 0);
    {
        const int c = (tid < GDN_DIM) ? (j * GDN_DIM + tid) : (total_key + j * GDN_DIM + tid - GDN_DIM);
        const float y = conv_channel(ring, x, cw, p.conv_dim, it.slot, c, qk_writer, ring);
        const float ss = warp_sum(y * y);
        if (lane == 0) s_red[warp] = ss;
        if (tid < ROWS) {
            const int cv = 2 * total_key + h * GDN_DIM + rb * ROWS + tid;
            s_v[tid] = conv_channel(ring, x, cw, p.conv_dim, it.slot, cv, true, ring);
        }
        if (tid == 0) {
            const float a_val = p.alpha[(size_t)item * p.Hv + h];
            const float dt_b = bf16_bits_to_f32(p.dt_bias[(size_t)it.w_layer * p.Hv + h]);
            const float a_cap = expf(p.a_log[(size_t)it.w_layer * p.Hv + h]);
            const float softplus = logf(1.0f + expf(a_val + dt_b));
            s_gb[0] = expf(-a_cap * softplus);
            s_gb[1] = 1.0f / (1.0f + expf(-p.beta[(size_t)item * p.Hv + h]));
        }
        __syncthreads();
        const float inv_scale = 1.0f / sqrtf((float)GDN_DIM);
        if (tid < GDN_DIM) {
            const float tot = (s_red[0] + s_red[1]) + (s_red[2] + s_red[3]);
            const float inv = 1.0f / sqrtf(tot / (float)GDN_DIM + 1e-6f);
            s_q[tid] = y * inv * inv_scale * inv_scale;
        } else {
            const float tot = (s_red[4] + s_red[5]) + (s_red[6] + s_red[7]);
            const float inv = 1.0f / sqrtf(tot / (float)GDN_DIM + 1e-6f);
            s_k[tid - GDN_DIM] = y * inv * inv_scale;
        }
        __syncthreads();
    }
    const float4 kk = *reinterpret_cast<const float4 *>(s_k + lane * 4);
    const float4 qq = *reinterpret_cast<const float4 *>(s_q + lane * 4);
    const float g = s_gb[0], bgate = s_gb[1];

    // ---- delta rule over this warp's rows, four rows per batch ----
#pragma unroll
    for (int b = 0; b < NB; b++) {
        float4 nxt[4];
        if (b + 1 < NB) {
#pragma unroll
            for (int i = 0; i < 4; i++)
                nxt[i] = *reinterpret_cast<const float4 *>(S + (size_t)((b + 1) * 4 + i) * GDN_DIM);
        }
        float kv[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            cur[i].x *= g;
            cur[i].y *= g;
            cur[i].z *= g;
            cur[i].w *= g;
            float a = cur[i].x * kk.x;
            a = fmaf(cur[i].y, kk.y, a);
            a = fmaf(cur[i].z, kk.z, a);
            a = fmaf(cur[i].w, kk.w, a);
            kv[i] = a;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
            for (int i = 0; i < 4; i++) kv[i] += __shfl_xor_sync(0xffffffffu, kv[i], o);
        }
        float ov[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int lr = warp * RPW + b * 4 + i;
            const float delta = (s_v[lr] - kv[i]) * bgate;
            cur[i].x = fmaf(kk.x, delta, cur[i].x);
            cur[i].y = fmaf(kk.y, delta, cur[i].y);
            cur[i].z = fmaf(kk.z, delta, cur[i].z);
            cur[i].w = fmaf(kk.w, delta, cur[i].w);
            *reinterpret_cast<float4 *>(S + (size_t)(b * 4 + i) * GDN_DIM) = cur[i];
            float a = cur[i].x * qq.x;
            a = fmaf(cur[i].y, qq.y, a);
            a = fmaf(cur[i].z, qq.z, a);
            a = fmaf(cur[i].w, qq.w, a);
            ov[i] = a;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
            for (int i = 0; i < 4; i++) ov[i] += __shfl_xor_sync(0xffffffffu, ov[i], o);
        }
        if (lane == 0) {
#pragma unroll
            for (int i = 0; i < 4; i++) s_o[warp * RPW + b * 4 + i] = ov[i];
        }
        if (b + 1 < NB) {
#pragma unroll
            for (int i = 0; i < 4; i++) cur[i] = nxt[i];
        }
    }
    __syncthreads();

    // ---- epilogue: plain read-out, or gated RMSNorm over the whole head ----
    float *out = p.out + (size_t)item * p.Hv * GDN_DIM + h * GDN_DIM + rb * ROWS;
    if (p.z == nullptr) {
        if (tid < ROWS) out[tid] = s_o[tid];
        return;
    }
    if (warp == 0) {
        float v = 0.0f;
        for (int i = lane; i < ROWS; i += 32) v += s_o[i] * s_o[i];
        v = warp_sum(v);
        if (lane == 0) s_ss = v;
    }
    float total;
    if constexpr (CS > 1) {
        cg::cluster_group cluster = cg::this_cluster();
        cluster.sync();
        total = 0.0f;
#pragma unroll
        for (int r = 0; r < CS; r++) total += *cluster.map_shared_rank(&s_ss, r);
        cluster.sync();  // peers may still be reading s_ss of this CTA
    } else {
        __syncthreads();
        total = s_ss;
    }
    if (tid < ROWS) {
        const float inv_rms = 1.0f / sqrtf(total / (float)GDN_DIM + p.eps);
        const int row = rb * ROWS + tid;
        const float zv = p.z[(size_t)item * p.Hv * GDN_DIM + h * GDN_DIM + row];
        const float w = bf16_bits_to_f32(p.norm_w[(size_t)it.w_layer * GDN_DIM + row]);
        const float silu_z = zv / (1.0f + expf(-zv));
        out[tid] = s_o[tid] * inv_rms * w * silu_z;
    }
}

template <int ROWS>
cudaError_t launch_rows(const GdnParams &p, cudaStream_t stream) {
    constexpr int CS = GDN_DIM / ROWS;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(p.n_items * p.Hv * CS), 1, 1);
    cfg.blockDim = dim3(256, 1, 1);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = CS;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, gdn_decode_kernel<ROWS>, p);
}

}  // namespace

cudaError_t launch_gdn_decode(const GdnParams &p, int rows_per_cta, cudaStream_t stream) {
    if (p.n_items <= 0) return cudaSuccess;
    switch (rows_per_cta) {
        case 32: return launch_rows<32>(p, stream);
        case 64: return launch_rows<64>(p, stream);
        case 128: return launch_rows<128>(p, stream);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace mfc
