// Folded MLA attention for decode (the third attention flavour of the reference), for sm_100a.
//
// What it computes (crates/moeflux/shaders/shaders.metal: mla_sdpa_folded :1717-1822, the tiled form
// mla_sdpa_tile_accumulate :1845-1966 and mla_sdpa_tile_finalize :1971-1987; dispatch
// crates/moeflux/src/riir/gpu_mla.rs:146-274), for every head h:
//     s[t]         = (q'[h] . latent[t] + q_pe[h] . rope_k[t]) * softmax_scale
//     p            = softmax(s)
//     v_combine[h] = sum_t p[t] * latent[t]
// with q' [H][512] (the query folded through kv_b_proj), q_pe [H][64], and the compressed cache latent [len][512],
// rope_k [len][64], fp32 as the reference stores them.  The cached row doubles as key (all 576 numbers) and value
// (the first 512): it is read from HBM once and serves both contractions out of shared memory.
//
// The reference runs one threadgroup per head with the scores of up to 4096 positions in threadgroup memory and,
// beyond that, one dispatch per 4096-position tile merged by an online softmax in device memory.  Here a CTA owns
// 16 heads (the M rows of mma.sync m16n8k16) and a chunk of positions; tiles of 16 positions arrive by TMA
// (cp.async.bulk.tensor, 128-byte swizzle) into a two-stage ring with bounded mbarrier waits; fp32
// operands enter the tensor cores as two-piece bf16 expansions (hi + mid, three products, fp32 accumulate: about
// 2^-16 relative, inside the reference's 1e-3 bound).  Each warp owns a quarter of the 576 key dims for the scores
// (partial score blocks are summed through shared memory) and a quarter of the 512 value dims for the output.  The
// chunks of a head block write un-normalised (o, m, l) partials that a second kernel merges by log-sum-exp -- the
// algebra of the reference's tile merge (:1933-1968).  CTAs of the same chunk are neighbours in the grid, so the
// eight head blocks of a 128-head model find the chunk's rows in L2 after the first of them has read them.
#include <math.h>

#include "common.cuh"
#include "kernels.h"

namespace mfc {

namespace {

constexpr int MLA_TILE = 16;                                   // positions per pipeline stage
constexpr int MLA_STAGES = 2;
constexpr int MLA_BOX_BYTES = MLA_TILE * 128;                  // one [16 rows x 32 floats] box
constexpr int MLA_LAT_BOXES = MLA_RANK / 32;                   // 16
constexpr int MLA_ROPE_BOXES = MLA_ROPE / 32;                  // 2
constexpr int MLA_KD = MLA_RANK + MLA_ROPE;                    // 576 key dims
constexpr int MLA_TILE_BYTES = MLA_TILE * MLA_KD * 4;          // 36,864
constexpr int MLA_KSTEPS = MLA_KD / 16;                        // 36 k-steps of 16 dims
constexpr int MLA_KSTEPS_PER_WARP = MLA_KSTEPS / 4;            // 9
constexpr int MLA_SP_STRIDE = 24;                              // padded row stride of a partial score block
constexpr int MLA_Q_STRIDE = MLA_KD + 4;                       // floats: staged q rows, spread over the banks
constexpr float MLA_LOG2E = 1.4426950408889634f;

__device__ __forceinline__ void split2(float x0, float x1, uint32_t &hi, uint32_t &mid) {
    hi = pack_bf16x2(x0, x1);
    mid = pack_bf16x2(x0 - __uint_as_float(hi << 16), x1 - __uint_as_float(hi & 0xffff0000u));
}

__global__ void __launch_bounds__(128, 2)
mla_decode_kernel(const __grid_constant__ CUtensorMap lat_map, const __grid_constant__ CUtensorMap rope_map,
                  const MlaParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *stages = smem;  // [STAGES][16 latent boxes | 2 rope boxes]
    float *s_sp = reinterpret_cast<float *>(smem + MLA_STAGES * MLA_TILE_BYTES);  // [2][4][16][24]
    uint64_t *full = reinterpret_cast<uint64_t *>(s_sp + 2 * 4 * 16 * MLA_SP_STRIDE);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    if (tid == 0) {
        prefetch_tmap(&lat_map);
        prefetch_tmap(&rope_map);
#pragma unroll
        for (int s = 0; s < MLA_STAGES; s++) mbar_init(&full[s], 1);
        mbar_fence_init();
    }
    __syncthreads();

    const int chunk = (int)blockIdx.x / p.n_head_blocks, hb = (int)blockIdx.x % p.n_head_blocks;
    const int c0 = chunk * p.rows_per_chunk;
    const int c1 = min(c0 + p.rows_per_chunk, p.cache_len);
    const int ntiles = (c1 - c0 + MLA_TILE - 1) / MLA_TILE;
    const int heads = min(16, p.H - 16 * hb);
    const unsigned spins = p.wait_spins ? p.wait_spins : (1u << 22);

    auto issue_tile = [&](int tile) {
        const int st = tile % MLA_STAGES;
        uint8_t *dst = stages + (size_t)st * MLA_TILE_BYTES;
        mbar_expect_tx(&full[st], MLA_TILE_BYTES);
        const int y = c0 + tile * MLA_TILE;  // rows past cache_len are outside the maps: the copy fills zeros
#pragma unroll
        for (int b = 0; b < MLA_LAT_BOXES; b++) tma_load_2d(dst + b * MLA_BOX_BYTES, &lat_map, b * 32, y, &full[st]);
#pragma unroll
        for (int b = 0; b < MLA_ROPE_BOXES; b++)
            tma_load_2d(dst + (MLA_LAT_BOXES + b) * MLA_BOX_BYTES, &rope_map, b * 32, y, &full[st]);
    };
    if (tid == 0 && ntiles > 0) issue_tile(0);

    // ---- the 16 query rows [q' (512) | q_pe (64)] through the stage that is still free, then as fragments ----
    // (16 rows of 580 floats: the last stage of the ring plus the first 256 bytes of the score exchange behind it,
    // which is idle until the first tile)
    float *s_q = reinterpret_cast<float *>(stages + (size_t)(MLA_STAGES - 1) * MLA_TILE_BYTES);
    for (int i = tid; i < 16 * (MLA_KD / 4); i += 128) {
        const int r = i / (MLA_KD / 4), c = (i % (MLA_KD / 4)) * 4;
        float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (r < heads) {
            const int h = 16 * hb + r;
            v = c < MLA_RANK ? *reinterpret_cast<const float4 *>(p.q_prime + (size_t)h * MLA_RANK + c)
                             : *reinterpret_cast<const float4 *>(p.q_pe + (size_t)h * MLA_ROPE + (c - MLA_RANK));
        }
        *reinterpret_cast<float4 *>(s_q + r * MLA_Q_STRIDE + c) = v;
    }
    __syncthreads();
    // A (16x16, bf16): a0 (g, k=2t,2t+1)  a1 (g+8, same k)  a2 (g, k=2t+8,2t+9)  a3 (g+8, same k); the k index of a
    // 16-dim step is permuted, k = 2t -> dim t, 2t+1 -> t+4, 2t+8 -> t+8, 2t+9 -> t+12, so that the two floats one
    // ldmatrix row delivers to a lane form one bf16x2 register of the B operand.
    uint32_t qh[MLA_KSTEPS_PER_WARP][4], qm[MLA_KSTEPS_PER_WARP][4];
#pragma unroll
    for (int j = 0; j < MLA_KSTEPS_PER_WARP; j++) {
        const int ks = MLA_KSTEPS_PER_WARP * warp + j;
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const int row = g + ((e & 1) ? 8 : 0);
            const int d = 16 * ks + t + ((e & 2) ? 8 : 0);
            split2(s_q[row * MLA_Q_STRIDE + d], s_q[row * MLA_Q_STRIDE + d + 4], qh[j][e], qm[j][e]);
        }
    }
    fence_proxy_async();  // the staging area goes back to the ring
    __syncthreads();
    if (tid == 0 && ntiles > 1) issue_tile(1);

    float o[16][4];  // this warp's 128 value dims: n-tile nt covers dims 128 w + 8 nt .. + 7
#pragma unroll
    for (int i = 0; i < 16; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
    float m_r[2] = {-INFINITY, -INFINITY};
    float l_r[2] = {0.0f, 0.0f};
    const float sl2 = p.scale * MLA_LOG2E;
    int failed_at = -1;

    for (int i = 0; i < ntiles; i++) {
        const int st = i % MLA_STAGES;
        const unsigned par = (unsigned)(i / MLA_STAGES) & 1u;
        const bool ok = mbar_wait_bounded(&full[st], par, spins);
        const uint8_t *gen = stages + (size_t)st * MLA_TILE_BYTES;
        const uint32_t kst = smem_u32(gen);

        // partial scores of the 16 positions over this warp's 144 key dims
        // (the three products of the expansion accumulate separately: six independent chains of MMAs per warp
        // instead of two)
        float sp[2][4], sp_mid[2][4], sp_kmid[2][4];
#pragma unroll
        for (int nt = 0; nt < 2; nt++)
#pragma unroll
            for (int e = 0; e < 4; e++) sp[nt][e] = sp_mid[nt][e] = sp_kmid[nt][e] = 0.0f;
        if (ok) {
            const int r = lane & 7, mi = lane >> 3;
#pragma unroll
            for (int j = 0; j < MLA_KSTEPS_PER_WARP; j++) {
                const int ks = MLA_KSTEPS_PER_WARP * warp + j;
                const int box = ks >> 1, chunk16 = ((ks & 1) << 2) + mi;
#pragma unroll
                for (int nt = 0; nt < 2; nt++) {
                    const int row = 8 * nt + r;
                    const uint32_t addr = kst + box * MLA_BOX_BYTES + row * 128 + ((chunk16 ^ (row & 7)) << 4);
                    uint32_t r0, r1, r2, r3;  // K[row][16 ks + t, + 4, + 8, + 12]
                    ldmatrix_x4(r0, r1, r2, r3, addr);
                    uint32_t h0, m0, h1, m1;
                    split2(__uint_as_float(r0), __uint_as_float(r1), h0, m0);
                    split2(__uint_as_float(r2), __uint_as_float(r3), h1, m1);
                    mma_bf16_16816(sp[nt], qh[j], h0, h1);
                    mma_bf16_16816(sp_mid[nt], qm[j], h0, h1);
                    mma_bf16_16816(sp_kmid[nt], qh[j], m0, m1);
                }
            }
#pragma unroll
            for (int nt = 0; nt < 2; nt++)
#pragma unroll
                for (int e = 0; e < 4; e++) sp[nt][e] += sp_mid[nt][e] + sp_kmid[nt][e];
        }
        float *spw = s_sp + ((i & 1) * 4 + warp) * 16 * MLA_SP_STRIDE;
#pragma unroll
        for (int nt = 0; nt < 2; nt++) {
            *reinterpret_cast<float2 *>(spw + g * MLA_SP_STRIDE + 8 * nt + 2 * t) = make_float2(sp[nt][0], sp[nt][1]);
            *reinterpret_cast<float2 *>(spw + (g + 8) * MLA_SP_STRIDE + 8 * nt + 2 * t) = make_float2(sp[nt][2], sp[nt][3]);
        }
        if (!__syncthreads_and(ok ? 1 : 0)) {
            failed_at = i;
            break;
        }
        // every warp is past its reads of tile i-1: refill that stage
        if (tid == 0 && i >= 1 && (i - 1 + MLA_STAGES) < ntiles) issue_tile(i - 1 + MLA_STAGES);

        float sv[2][4];
#pragma unroll
        for (int nt = 0; nt < 2; nt++) sv[nt][0] = sv[nt][1] = sv[nt][2] = sv[nt][3] = 0.0f;
#pragma unroll
        for (int w = 0; w < 4; w++) {
            const float *src = s_sp + ((i & 1) * 4 + w) * 16 * MLA_SP_STRIDE;
#pragma unroll
            for (int nt = 0; nt < 2; nt++) {
                const float2 a = *reinterpret_cast<const float2 *>(src + g * MLA_SP_STRIDE + 8 * nt + 2 * t);
                const float2 b = *reinterpret_cast<const float2 *>(src + (g + 8) * MLA_SP_STRIDE + 8 * nt + 2 * t);
                sv[nt][0] += a.x;
                sv[nt][1] += a.y;
                sv[nt][2] += b.x;
                sv[nt][3] += b.y;
            }
        }
        const int tile_row0 = c0 + i * MLA_TILE;
        if (tile_row0 + MLA_TILE > c1) {
#pragma unroll
            for (int nt = 0; nt < 2; nt++) {
                const int col = tile_row0 + 8 * nt + 2 * t;
                if (col >= c1) sv[nt][0] = sv[nt][2] = -INFINITY;
                if (col + 1 >= c1) sv[nt][1] = sv[nt][3] = -INFINITY;
            }
        }
        float corr[2];
#pragma unroll
        for (int x = 0; x < 2; x++) {
            float mx = fmaxf(fmaxf(sv[0][2 * x], sv[0][2 * x + 1]), fmaxf(sv[1][2 * x], sv[1][2 * x + 1]));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            const float m_new = fmaxf(m_r[x], mx);
            corr[x] = ex2_approx((m_r[x] - m_new) * sl2);
            m_r[x] = m_new;
            const float mb = m_new * sl2;
            float rs = 0.0f;
#pragma unroll
            for (int nt = 0; nt < 2; nt++) {
                sv[nt][2 * x] = ex2_approx(fmaf(sv[nt][2 * x], sl2, -mb));
                sv[nt][2 * x + 1] = ex2_approx(fmaf(sv[nt][2 * x + 1], sl2, -mb));
                rs += sv[nt][2 * x] + sv[nt][2 * x + 1];
            }
            l_r[x] = l_r[x] * corr[x] + rs;
        }
        // O[:, 128w .. 128w+127] = corr * O + P (16 x 16) * latent (16 x 128): the same tile, as the value operand.
        // Rows past the end of the cache were filled with zeros by the copy and carry weight zero.  The tile's
        // products are summed by the tensor core from zero and joined to the running output by a fused multiply-add
        // that rounds to nearest: an accumulator kept in the tensor core is truncated after every instruction and
        // drifts towards zero over thousands of tiles.
        {
            uint32_t ph[4], pm[4];
            split2(sv[0][0], sv[0][1], ph[0], pm[0]);  // (g,   rows 2t, 2t+1)
            split2(sv[0][2], sv[0][3], ph[1], pm[1]);  // (g+8, rows 2t, 2t+1)
            split2(sv[1][0], sv[1][1], ph[2], pm[2]);  // (g,   rows 2t+8, 2t+9)
            split2(sv[1][2], sv[1][3], ph[3], pm[3]);  // (g+8, rows 2t+8, 2t+9)
            auto v_at = [&](const uint8_t *bx, int r, int col) {
                return *reinterpret_cast<const float *>(bx + r * 128 + ((((col >> 2) ^ (r & 7))) << 4) + (col & 3) * 4);
            };
#pragma unroll
            for (int nt = 0; nt < 16; nt++) {
                const uint8_t *bx = gen + (4 * warp + (nt >> 2)) * MLA_BOX_BYTES;
                const int col = 8 * (nt & 3) + g;
                uint32_t h0, m0, h1, m1;
                split2(v_at(bx, 2 * t, col), v_at(bx, 2 * t + 1, col), h0, m0);
                split2(v_at(bx, 2 * t + 8, col), v_at(bx, 2 * t + 9, col), h1, m1);
                float d[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                mma_bf16_16816(d, pm, h0, h1);
                mma_bf16_16816(d, ph, m0, m1);
                mma_bf16_16816(d, ph, h0, h1);
                o[nt][0] = fmaf(o[nt][0], corr[0], d[0]);
                o[nt][1] = fmaf(o[nt][1], corr[0], d[1]);
                o[nt][2] = fmaf(o[nt][2], corr[1], d[2]);
                o[nt][3] = fmaf(o[nt][3], corr[1], d[3]);
            }
        }
    }
    if (failed_at >= 0) {
        // a load did not arrive within the limit: wait (bounded again) for the one other load that may be in flight
        // into this CTA's shared memory, report, and leave without writing results
        if (tid == 0) atomicOr(p.status, STATUS_TMA_TIMEOUT);
        const int last_issued = min(ntiles - 1, max(MLA_STAGES - 1, failed_at + 1));
        for (int j = failed_at + 1; j <= last_issued; j++)
            mbar_wait_bounded(&full[j % MLA_STAGES], (unsigned)(j / MLA_STAGES) & 1u, spins);
        return;
    }

    // ---- epilogue: the final rows when the head block has one chunk, else the un-normalised partial ----
#pragma unroll
    for (int x = 0; x < 2; x++) {
        l_r[x] += __shfl_xor_sync(0xffffffffu, l_r[x], 1);
        l_r[x] += __shfl_xor_sync(0xffffffffu, l_r[x], 2);
    }
    const bool single = p.n_chunks == 1;
#pragma unroll
    for (int x = 0; x < 2; x++) {
        const int row = g + 8 * x;
        if (row >= heads) continue;
        const int h = 16 * hb + row;
        float *dst;
        float inv = 1.0f;
        if (single) {
            dst = p.out + (size_t)h * MLA_RANK;
            inv = 1.0f / l_r[x];
        } else {
            dst = p.part_o + ((size_t)chunk * p.H + h) * MLA_RANK;
            if (warp == 0 && t == 0) {
                p.part_m[(size_t)chunk * p.H + h] = m_r[x] * p.scale;
                p.part_l[(size_t)chunk * p.H + h] = l_r[x];
            }
        }
#pragma unroll
        for (int nt = 0; nt < 16; nt++)
            *reinterpret_cast<float2 *>(dst + 128 * warp + 8 * nt + 2 * t) =
                make_float2(o[nt][2 * x] * inv, o[nt][2 * x + 1] * inv);
    }
}

// ---- bf16 latent cache -----------------------------------------------------------------------------------------
// The same work split for a cache stored as bf16 (latent [len][512], rope_k [len][64]; not a reference format: the
// reference stores fp32).  Half the HBM bytes per position, tiles of 32 positions, and one product per contraction
// instead of three: q and P are rounded to bf16 for the MMAs as in the bf16 GQA kernel (tolerance 2e-2 against the
// oracle on the rounded cache).  K fragments come from ldmatrix, V fragments from ldmatrix.trans on the same tile.
constexpr int MLB_TILE = 32;
constexpr int MLB_BOX_BYTES = MLB_TILE * 128;                  // one [32 rows x 64 bf16] box
constexpr int MLB_LAT_BOXES = MLA_RANK / 64;                   // 8
constexpr int MLB_ROPE_BOXES = MLA_ROPE / 64;                  // 1
constexpr int MLB_TILE_BYTES = MLB_TILE * MLA_KD * 2;          // 36,864
constexpr int MLB_SP_STRIDE = 40;

__global__ void __launch_bounds__(128, 2)
mla_decode_bf16_kernel(const __grid_constant__ CUtensorMap lat_map, const __grid_constant__ CUtensorMap rope_map,
                       const MlaParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *stages = smem;  // [STAGES][8 latent boxes | 1 rope box]
    float *s_sp = reinterpret_cast<float *>(smem + MLA_STAGES * MLB_TILE_BYTES);  // [2][4][16][40]
    uint64_t *full = reinterpret_cast<uint64_t *>(s_sp + 2 * 4 * 16 * MLB_SP_STRIDE);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    if (tid == 0) {
        prefetch_tmap(&lat_map);
        prefetch_tmap(&rope_map);
#pragma unroll
        for (int s = 0; s < MLA_STAGES; s++) mbar_init(&full[s], 1);
        mbar_fence_init();
    }
    __syncthreads();

    const int chunk = (int)blockIdx.x / p.n_head_blocks, hb = (int)blockIdx.x % p.n_head_blocks;
    const int c0 = chunk * p.rows_per_chunk;
    const int c1 = min(c0 + p.rows_per_chunk, p.cache_len);
    const int ntiles = (c1 - c0 + MLB_TILE - 1) / MLB_TILE;
    const int heads = min(16, p.H - 16 * hb);
    const unsigned spins = p.wait_spins ? p.wait_spins : (1u << 22);

    auto issue_tile = [&](int tile) {
        const int st = tile % MLA_STAGES;
        uint8_t *dst = stages + (size_t)st * MLB_TILE_BYTES;
        mbar_expect_tx(&full[st], MLB_TILE_BYTES);
        const int y = c0 + tile * MLB_TILE;  // rows past cache_len are outside the maps: the copy fills zeros
#pragma unroll
        for (int b = 0; b < MLB_LAT_BOXES; b++) tma_load_2d(dst + b * MLB_BOX_BYTES, &lat_map, b * 64, y, &full[st]);
        tma_load_2d(dst + MLB_LAT_BOXES * MLB_BOX_BYTES, &rope_map, 0, y, &full[st]);
    };
    if (tid == 0 && ntiles > 0) issue_tile(0);

    // the 16 query rows through the last ring stage (and the head of the score exchange behind it), as bf16 fragments
    float *s_q = reinterpret_cast<float *>(stages + (size_t)(MLA_STAGES - 1) * MLB_TILE_BYTES);
    for (int i = tid; i < 16 * (MLA_KD / 4); i += 128) {
        const int r = i / (MLA_KD / 4), c = (i % (MLA_KD / 4)) * 4;
        float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (r < heads) {
            const int h = 16 * hb + r;
            v = c < MLA_RANK ? *reinterpret_cast<const float4 *>(p.q_prime + (size_t)h * MLA_RANK + c)
                             : *reinterpret_cast<const float4 *>(p.q_pe + (size_t)h * MLA_ROPE + (c - MLA_RANK));
        }
        *reinterpret_cast<float4 *>(s_q + r * MLA_Q_STRIDE + c) = v;
    }
    __syncthreads();
    uint32_t qa[MLA_KSTEPS_PER_WARP][4];  // A (16x16): a0 (g, 2t..)  a1 (g+8, 2t..)  a2 (g, 2t+8..)  a3 (g+8, 2t+8..)
#pragma unroll
    for (int j = 0; j < MLA_KSTEPS_PER_WARP; j++) {
        const int d = 16 * (MLA_KSTEPS_PER_WARP * warp + j) + 2 * t;
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const float *src = s_q + (g + ((e & 1) ? 8 : 0)) * MLA_Q_STRIDE + d + ((e & 2) ? 8 : 0);
            qa[j][e] = pack_bf16x2(src[0], src[1]);
        }
    }
    fence_proxy_async();
    __syncthreads();
    if (tid == 0 && ntiles > 1) issue_tile(1);

    float o[16][4];
#pragma unroll
    for (int i = 0; i < 16; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
    float m_r[2] = {-INFINITY, -INFINITY};
    float l_r[2] = {0.0f, 0.0f};
    const float sl2 = p.scale * MLA_LOG2E;
    int failed_at = -1;

    for (int i = 0; i < ntiles; i++) {
        const int st = i % MLA_STAGES;
        const unsigned par = (unsigned)(i / MLA_STAGES) & 1u;
        const bool ok = mbar_wait_bounded(&full[st], par, spins);
        const uint32_t kst = smem_u32(stages + (size_t)st * MLB_TILE_BYTES);

        // partial scores of the 32 positions over this warp's 144 key dims: one ldmatrix.x4 = one k-step of two
        // 8-row groups (matrices: rows A dims 0-7, rows A dims 8-15, rows B dims 0-7, rows B dims 8-15)
        float sp[4][4];
#pragma unroll
        for (int nt = 0; nt < 4; nt++) sp[nt][0] = sp[nt][1] = sp[nt][2] = sp[nt][3] = 0.0f;
        if (ok) {
            const int r = lane & 7, mi = lane >> 3;
#pragma unroll
            for (int j = 0; j < MLA_KSTEPS_PER_WARP; j++) {
                const int ks = MLA_KSTEPS_PER_WARP * warp + j;
                const int box = ks >> 2, c16 = ((ks & 3) << 1) + (mi & 1);
#pragma unroll
                for (int np = 0; np < 2; np++) {
                    const int row = 16 * np + 8 * (mi >> 1) + r;
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4(b0, b1, b2, b3, kst + box * MLB_BOX_BYTES + row * 128 + ((c16 ^ (row & 7)) << 4));
                    mma_bf16_16816(sp[2 * np], qa[j], b0, b1);
                    mma_bf16_16816(sp[2 * np + 1], qa[j], b2, b3);
                }
            }
        }
        float *spw = s_sp + ((i & 1) * 4 + warp) * 16 * MLB_SP_STRIDE;
#pragma unroll
        for (int nt = 0; nt < 4; nt++) {
            *reinterpret_cast<float2 *>(spw + g * MLB_SP_STRIDE + 8 * nt + 2 * t) = make_float2(sp[nt][0], sp[nt][1]);
            *reinterpret_cast<float2 *>(spw + (g + 8) * MLB_SP_STRIDE + 8 * nt + 2 * t) = make_float2(sp[nt][2], sp[nt][3]);
        }
        if (!__syncthreads_and(ok ? 1 : 0)) {
            failed_at = i;
            break;
        }
        if (tid == 0 && i >= 1 && (i - 1 + MLA_STAGES) < ntiles) issue_tile(i - 1 + MLA_STAGES);

        float sv[4][4];
#pragma unroll
        for (int nt = 0; nt < 4; nt++) sv[nt][0] = sv[nt][1] = sv[nt][2] = sv[nt][3] = 0.0f;
#pragma unroll
        for (int w = 0; w < 4; w++) {
            const float *src = s_sp + ((i & 1) * 4 + w) * 16 * MLB_SP_STRIDE;
#pragma unroll
            for (int nt = 0; nt < 4; nt++) {
                const float2 a = *reinterpret_cast<const float2 *>(src + g * MLB_SP_STRIDE + 8 * nt + 2 * t);
                const float2 b = *reinterpret_cast<const float2 *>(src + (g + 8) * MLB_SP_STRIDE + 8 * nt + 2 * t);
                sv[nt][0] += a.x;
                sv[nt][1] += a.y;
                sv[nt][2] += b.x;
                sv[nt][3] += b.y;
            }
        }
        const int tile_row0 = c0 + i * MLB_TILE;
        if (tile_row0 + MLB_TILE > c1) {
#pragma unroll
            for (int nt = 0; nt < 4; nt++) {
                const int col = tile_row0 + 8 * nt + 2 * t;
                if (col >= c1) sv[nt][0] = sv[nt][2] = -INFINITY;
                if (col + 1 >= c1) sv[nt][1] = sv[nt][3] = -INFINITY;
            }
        }
        float corr[2];
#pragma unroll
        for (int x = 0; x < 2; x++) {
            float mx = fmaxf(fmaxf(sv[0][2 * x], sv[0][2 * x + 1]), fmaxf(sv[1][2 * x], sv[1][2 * x + 1]));
            mx = fmaxf(mx, fmaxf(fmaxf(sv[2][2 * x], sv[2][2 * x + 1]), fmaxf(sv[3][2 * x], sv[3][2 * x + 1])));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            const float m_new = fmaxf(m_r[x], mx);
            corr[x] = ex2_approx((m_r[x] - m_new) * sl2);
            m_r[x] = m_new;
            const float mb = m_new * sl2;
            float rs = 0.0f;
#pragma unroll
            for (int nt = 0; nt < 4; nt++) {
                sv[nt][2 * x] = ex2_approx(fmaf(sv[nt][2 * x], sl2, -mb));
                sv[nt][2 * x + 1] = ex2_approx(fmaf(sv[nt][2 * x + 1], sl2, -mb));
                rs += sv[nt][2 * x] + sv[nt][2 * x + 1];
            }
            l_r[x] = l_r[x] * corr[x] + rs;
        }
#pragma unroll
        for (int nt = 0; nt < 16; nt++) {
            o[nt][0] *= corr[0];
            o[nt][1] *= corr[0];
            o[nt][2] *= corr[1];
            o[nt][3] *= corr[1];
        }
        // O[:, 128w .. 128w+127] += P (16 x 32) * latent (32 x 128): the tile again, transposed by ldmatrix
#pragma unroll
        for (int kk = 0; kk < 2; kk++) {
            uint32_t pa[4];
            pa[0] = pack_bf16x2(sv[2 * kk][0], sv[2 * kk][1]);
            pa[1] = pack_bf16x2(sv[2 * kk][2], sv[2 * kk][3]);
            pa[2] = pack_bf16x2(sv[2 * kk + 1][0], sv[2 * kk + 1][1]);
            pa[3] = pack_bf16x2(sv[2 * kk + 1][2], sv[2 * kk + 1][3]);
            const int r = lane & 7, mi = lane >> 3;
            const int prow = 16 * kk + 8 * (mi & 1) + r;
#pragma unroll
            for (int bx = 0; bx < 2; bx++) {
#pragma unroll
                for (int cp = 0; cp < 4; cp++) {
                    const int c16 = 2 * cp + (mi >> 1);
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4_trans(b0, b1, b2, b3,
                                      kst + (2 * warp + bx) * MLB_BOX_BYTES + prow * 128 + ((c16 ^ (prow & 7)) << 4));
                    mma_bf16_16816(o[8 * bx + 2 * cp], pa, b0, b1);
                    mma_bf16_16816(o[8 * bx + 2 * cp + 1], pa, b2, b3);
                }
            }
        }
    }
    if (failed_at >= 0) {
        if (tid == 0) atomicOr(p.status, STATUS_TMA_TIMEOUT);
        const int last_issued = min(ntiles - 1, max(MLA_STAGES - 1, failed_at + 1));
        for (int j = failed_at + 1; j <= last_issued; j++)
            mbar_wait_bounded(&full[j % MLA_STAGES], (unsigned)(j / MLA_STAGES) & 1u, spins);
        return;
    }
#pragma unroll
    for (int x = 0; x < 2; x++) {
        l_r[x] += __shfl_xor_sync(0xffffffffu, l_r[x], 1);
        l_r[x] += __shfl_xor_sync(0xffffffffu, l_r[x], 2);
    }
    const bool single = p.n_chunks == 1;
#pragma unroll
    for (int x = 0; x < 2; x++) {
        const int row = g + 8 * x;
        if (row >= heads) continue;
        const int h = 16 * hb + row;
        float *dst;
        float inv = 1.0f;
        if (single) {
            dst = p.out + (size_t)h * MLA_RANK;
            inv = 1.0f / l_r[x];
        } else {
            dst = p.part_o + ((size_t)chunk * p.H + h) * MLA_RANK;
            if (warp == 0 && t == 0) {
                p.part_m[(size_t)chunk * p.H + h] = m_r[x] * p.scale;
                p.part_l[(size_t)chunk * p.H + h] = l_r[x];
            }
        }
#pragma unroll
        for (int nt = 0; nt < 16; nt++)
            *reinterpret_cast<float2 *>(dst + 128 * warp + 8 * nt + 2 * t) =
                make_float2(o[nt][2 * x] * inv, o[nt][2 * x + 1] * inv);
    }
}

// v_combine[h] = sum_c e^{m_c - M} o_c / sum_c e^{m_c - M} l_c over the chunks of head h: one CTA per head, 128 threads
// x 4 dims.  The reference's tile merge (shaders.metal:1933-1968) walks the tiles in order and rescales a running
// accumulator; taking the maximum first gives the same sums with one rounding per term.
__global__ void __launch_bounds__(128) mla_merge_kernel(const MlaParams p) {
    const int h = blockIdx.x, tid = threadIdx.x;
    float M = -INFINITY;
    for (int c = 0; c < p.n_chunks; c++) M = fmaxf(M, p.part_m[(size_t)c * p.H + h]);
    float L = 0.0f;
    float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    for (int c = 0; c < p.n_chunks; c++) {
        const float m = p.part_m[(size_t)c * p.H + h];
        const float w = (m == -INFINITY) ? 0.0f : expf(m - M);
        L += w * p.part_l[(size_t)c * p.H + h];
        const float4 o = *reinterpret_cast<const float4 *>(p.part_o + ((size_t)c * p.H + h) * MLA_RANK + 4 * tid);
        acc.x = fmaf(w, o.x, acc.x);
        acc.y = fmaf(w, o.y, acc.y);
        acc.z = fmaf(w, o.z, acc.z);
        acc.w = fmaf(w, o.w, acc.w);
    }
    const float inv = L > 0.0f ? 1.0f / L : 0.0f;
    *reinterpret_cast<float4 *>(p.out + (size_t)h * MLA_RANK + 4 * tid) =
        make_float4(acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv);
}

constexpr size_t MLA_SMEM = 1024 + (size_t)MLA_STAGES * MLA_TILE_BYTES + sizeof(float) * 2 * 4 * 16 * MLA_SP_STRIDE +
                            sizeof(uint64_t) * MLA_STAGES;
static_assert(16 * MLA_Q_STRIDE * 4 <= MLA_TILE_BYTES + (int)sizeof(float) * 2 * 4 * 16 * MLA_SP_STRIDE,
              "the staged query rows must fit the last ring stage and the score exchange behind it");

}  // namespace

constexpr size_t MLB_SMEM = 1024 + (size_t)MLA_STAGES * MLB_TILE_BYTES + sizeof(float) * 2 * 4 * 16 * MLB_SP_STRIDE +
                            sizeof(uint64_t) * MLA_STAGES;

cudaError_t mla_decode_configure() {
    cudaError_t e = cudaFuncSetAttribute(mla_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)MLA_SMEM);
    if (e != cudaSuccess) return e;
    return cudaFuncSetAttribute(mla_decode_bf16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)MLB_SMEM);
}

cudaError_t launch_mla_decode(const CUtensorMap &lat_map, const CUtensorMap &rope_map, const MlaParams &p,
                              cudaStream_t stream) {
    if (p.n_chunks <= 0 || p.n_head_blocks <= 0) return cudaSuccess;
    if (p.cache_bf16) mla_decode_bf16_kernel<<<p.n_chunks * p.n_head_blocks, 128, MLB_SMEM, stream>>>(lat_map, rope_map, p);
    else mla_decode_kernel<<<p.n_chunks * p.n_head_blocks, 128, MLA_SMEM, stream>>>(lat_map, rope_map, p);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess || p.n_chunks == 1) return e;
    mla_merge_kernel<<<p.H, 128, 0, stream>>>(p);
    return cudaGetLastError();
}

}  // namespace mfc
