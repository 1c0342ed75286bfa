// Split-K flash-decoding for GQA full attention, fp32 KV cache (the reference's
// storage type), for sm_100a.  Same work split, TMA pipeline, RoPE/append fusion
// and epilogue as the bf16 kernel (gqa_decode.cu); the tile maths differs.
//
// fp32 operands run on the tensor cores as a two-piece bf16 expansion: every
// operand x is split into hi = bf16(x) and mid = bf16(x - hi) (16 mantissa bits,
// fp32's exponent range), and a product a*b is accumulated in fp32 as
// a_hi*b_hi + a_mid*b_hi + a_hi*b_mid.  What is dropped (a_mid*b_mid and the two
// remainders) is below 2^-16 of |a||b| per term, which leaves the attention output
// within about 1e-5 relative of the fp32 reference (crates/moeflux/src/riir/sdpa.rs:
// 114-169) at half the tensor-pipe instructions of a 3xTF32 scheme: mma.sync
// m16n8k16 covers 16 k per instruction where the tf32 shape covers 8, and this
// kernel is bound by that pipe, not by memory.  Each warp owns 64 of the 256 dims
// for BOTH contractions: it computes a partial score block over its dims, the four
// partial blocks are summed through shared memory, and P V is accumulated for
// the same 64 dims.  Tiles are 16 rows; K fragments come from ldmatrix (an 8x8
// b16 matrix is an 8x4 fp32 block) with the k index of the MMA permuted so that the
// two floats a lane receives form one bf16x2 operand register; V fragments come
// from conflict-free scalar loads.
#include <math.h>

#include "gqa_common.cuh"

namespace mfc {

namespace {

#ifndef F32_SCORE_CHAINS
#define F32_SCORE_CHAINS 3  // 3: one accumulator per product of the two-piece expansion; 1: a single chain
#endif
constexpr int F32_TILE = KV_TILE_F32;
constexpr int F32_STAGES = 3;
constexpr int TILE_BYTES_F32 = F32_TILE * HEAD_DIM * 4;  // 16 KiB per tensor per stage
constexpr int BOX_BYTES = F32_TILE * 128;                // one [16 rows x 32 floats] box
constexpr int SP_STRIDE = 24;                            // padded row stride of a partial score block

// (x0, x1) -> bf16x2 registers hi and mid with x = hi + mid + O(2^-18 |x|); x0 in the low half.
__device__ __forceinline__ void split_bf16x2(float x0, float x1, uint32_t &hi, uint32_t &mid) {
    hi = pack_bf16x2(x0, x1);
    mid = pack_bf16x2(x0 - __uint_as_float(hi << 16), x1 - __uint_as_float(hi & 0xffff0000u));
}

__global__ void __launch_bounds__(128, 2)
gqa_decode_f32_kernel(const __grid_constant__ CUtensorMap kmap,
                      const __grid_constant__ CUtensorMap vmap, const __grid_constant__ GqaParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *stages = smem;  // [STAGES][K tile | V tile]
    float *s_sp = reinterpret_cast<float *>(smem + F32_STAGES * 2 * TILE_BYTES_F32);  // [2][4][16][24]
    float *s_cos = s_sp + 2 * 4 * 16 * SP_STRIDE;  // [128]
    float *s_sin = s_cos + 128;                    // [128]
    uint64_t *full = reinterpret_cast<uint64_t *>(s_sin + 128);
    // merge scratch aliases the stage ring: it is touched only after the last tile
    float *s_w = reinterpret_cast<float *>(stages);  // [MAX_SPLITS*16]
    float *s_M = s_w + MAX_SPLITS * 16;              // [16]
    float *s_L = s_M + 16;                           // [16]
    __shared__ int s_flag;
    __shared__ int s_begin[LOCATE_SMEM_ITEMS];
    __shared__ float s_inv[16];
    __shared__ float s_kred[4];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    if (tid == 0) {
        prefetch_tmap(&kmap);
        prefetch_tmap(&vmap);
#pragma unroll
        for (int s = 0; s < F32_STAGES; s++) mbar_init(&full[s], 1);
        mbar_fence_init();
    }
    stage_tile_begins(p, s_begin);  // also publishes the barrier initialisation

    // This CTA's share of the launch-wide tile sequence, one unit segment at a time.
    int gt = (int)blockIdx.x * p.tiles_per_cta;
    const int gt_end = min(gt + p.tiles_per_cta, p.total_tiles);
    unsigned pc = 0;  // tiles pushed through the stage ring so far: stage and phase follow from it
    const unsigned spins = p.wait_spins ? p.wait_spins : (1u << 22);
    bool abandoned = false;  // a bounded wait ran out, or an item failed its checks: no further loads, tickets only
    int seg_no = 0;
    trace_phase(p, 0);
    while (gt < gt_end) {
    const Located L = locate_tile<F32_TILE>(p, gt, gt_end, s_begin);
    const GqaItem &it = L.it;
    const int group = p.group;
    if (L.bad && !abandoned) {
        if (tid == 0) atomicOr(p.status, STATUS_BAD_ITEM);
        abandoned = true;
    }
    if (abandoned) {  // take the unit's tickets so that the counters return to zero, touch nothing else
        float o0[8][4] = {};
        float m0[2] = {-INFINITY, -INFINITY}, l0[2] = {0.0f, 0.0f};
        finish_unit(p, L, o0, m0, l0, s_w, s_M, s_L, &s_flag, s_L + 16, true);
        gt += L.seg;
        __syncthreads();
        continue;
    }

    const int c0 = L.t0 * F32_TILE;
    const int c1 = min(c0 + L.seg * F32_TILE, it.local_len);
    const int ntiles = (c1 > c0) ? (c1 - c0 + F32_TILE - 1) / F32_TILE : 0;
    const int row_base = (it.kv_slot * p.Hkv + L.kvh) * p.cap_rows;
    const bool appender = it.append_row >= c0 && it.append_row < c0 + L.seg * F32_TILE;

    const bool lose_load = p.inject_lost_load && blockIdx.x == 0 && seg_no == 0;
    auto issue_tile = [&](int tile) {
        const int st = (int)((pc + (unsigned)tile) % F32_STAGES);
        uint8_t *kdst = stages + (size_t)st * 2 * TILE_BYTES_F32;
        uint8_t *vdst = kdst + TILE_BYTES_F32;
        mbar_expect_tx(&full[st], 2 * TILE_BYTES_F32);
        if (lose_load && tile == 0) return;  // diagnostic: the barrier is armed and nothing will ever arrive
        const int y = row_base + c0 + tile * F32_TILE;
#pragma unroll
        for (int b = 0; b < 8; b++) {
            tma_load_2d(kdst + b * BOX_BYTES, &kmap, b * 32, y, &full[st]);
            tma_load_2d(vdst + b * BOX_BYTES, &vmap, b * 32, y, &full[st]);
        }
    };

    // (the last stage of the ring first carries the Q rows)
    float *s_q = reinterpret_cast<float *>(stages + (size_t)((pc + F32_STAGES - 1) % F32_STAGES) * 2 * TILE_BYTES_F32);
    stage_q_rows(p.q + ((size_t)it.in_idx * p.H + (size_t)L.kvh * group) * (size_t)p.q_row_stride, group, p.q_row_stride, s_q);
    const int half = p.rotary_dim >> 1;
    if (tid < half) {
        float sn, cs;
        sincosf((float)it.pos * p.inv_freq[tid], &sn, &cs);
        s_cos[tid] = cs;
        s_sin[tid] = sn;
    }
    __syncthreads();
    // the first tiles of the segment are requested only now, with the query rows already in shared memory (rows asked
    // for behind the first tiles of every CTA of the launch came back after microseconds, with the ring full and idle)
    if (tid == 0 && !appender) {
        const int n0 = min(ntiles, F32_STAGES - 1);
        for (int i = 0; i < n0; i++) issue_tile(i);
    }

    if (appender) {
        const float *ksrc = p.k + ((size_t)it.in_idx * p.Hkv + L.kvh) * HEAD_DIM;
        const float *vsrc = p.v + ((size_t)it.in_idx * p.Hkv + L.kvh) * HEAD_DIM;
        const int d = 2 * tid;
        float k_inv = 1.0f;
        const uint16_t *knw = p.knorm_w ? p.knorm_w + (size_t)(it.kv_slot / p.n_seqs) * HEAD_DIM : nullptr;
        if (knw) {  // per-head RMSNorm of k before the rotation
            const float2 kr = *reinterpret_cast<const float2 *>(ksrc + d);
            const float ss = warp_sum(kr.x * kr.x + kr.y * kr.y);
            if (lane == 0) s_kred[warp] = ss;
            __syncthreads();
            k_inv = 1.0f / sqrtf(((s_kred[0] + s_kred[1]) + (s_kred[2] + s_kred[3])) / (float)HEAD_DIM + p.norm_eps);
        }
        const float2 kx = load_rot2(ksrc, d, p.rotary_dim, half, s_cos, s_sin, k_inv, knw);
        const float2 vx = *reinterpret_cast<const float2 *>(vsrc + d);
        const size_t roff = ((size_t)row_base + it.append_row) * HEAD_DIM + d;
        *reinterpret_cast<float2 *>(reinterpret_cast<float *>(p.k_base) + roff) = kx;
        *reinterpret_cast<float2 *>(reinterpret_cast<float *>(p.v_base) + roff) = vx;
        __threadfence();
        fence_proxy_async();
        __syncthreads();
        if (tid == 0) {
            const int n0 = min(ntiles, F32_STAGES - 1);
            for (int i = 0; i < n0; i++) issue_tile(i);
        }
    }

    // ---- Q fragments for this warp's 64 dims: 4 k-steps of 16, hi and mid ----
    // A (16x16, bf16): a0 (g, k=2t,2t+1)  a1 (g+8, same k)  a2 (g, k=2t+8,2t+9)  a3 (g+8, same k).
    // k -> dim map inside a 16-dim step: 2t -> t, 2t+1 -> t+4, 2t+8 -> t+8, 2t+9 -> t+12 (see the K fragments).
    // The rows are first normalised / rotated in shared memory by compact loops (an unrolled build straight from
    // the inputs runs once per segment from a cold instruction cache); the fragments are then plain loads.
    uint32_t qh[4][4], qm[4][4];
    {
        const uint16_t *qnw = p.qnorm_w ? p.qnorm_w + (size_t)(it.kv_slot / p.n_seqs) * HEAD_DIM : nullptr;
        if (qnw) head_inv_rms(s_q, group, Q_STAGE_STRIDE, p.norm_eps, s_inv);
        // in place: the thread that owns dims (d, d+1) below `half` also owns their partners (d + half, d + half + 1)
#pragma unroll 1
        for (int idx = tid; idx < 16 * (HEAD_DIM / 2); idx += 128) {
            const int row = idx >> 7, d = (idx & 127) * 2;
            if (row >= group) continue;  // rows past the group were staged as zeros
            float *qr = s_q + row * Q_STAGE_STRIDE;
            const float qinv = qnw ? s_inv[row] : 1.0f;
            if (d < half) {
                const float2 lo = load_norm2(qr, d, qinv, qnw), hi = load_norm2(qr, d + half, qinv, qnw);
                *reinterpret_cast<float2 *>(qr + d) =
                    make_float2(lo.x * s_cos[d] - hi.x * s_sin[d], lo.y * s_cos[d + 1] - hi.y * s_sin[d + 1]);
                *reinterpret_cast<float2 *>(qr + d + half) =
                    make_float2(lo.x * s_sin[d] + hi.x * s_cos[d], lo.y * s_sin[d + 1] + hi.y * s_cos[d + 1]);
            } else if (d >= p.rotary_dim && qnw) {
                *reinterpret_cast<float2 *>(qr + d) = load_norm2(qr, d, qinv, qnw);
            }
        }
        __syncthreads();
#pragma unroll
        for (int ks = 0; ks < 4; ks++) {
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int row = g + ((e & 1) ? 8 : 0);
                const int d = 64 * warp + 16 * ks + t + ((e & 2) ? 8 : 0);
                split_bf16x2(s_q[row * Q_STAGE_STRIDE + d], s_q[row * Q_STAGE_STRIDE + d + 4], qh[ks][e], qm[ks][e]);
            }
        }
    }

    fence_proxy_async();  // the Q staging area goes back to the ring
    __syncthreads();
    if (tid == 0 && ntiles >= F32_STAGES) issue_tile(F32_STAGES - 1);
    if (seg_no == 0) trace_phase(p, 1);

    float o[8][4];
#pragma unroll
    for (int i = 0; i < 8; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
    float m_r[2] = {-INFINITY, -INFINITY};
    float l_r[2] = {0.0f, 0.0f};
    const float sl2 = p.scale * LOG2E;
    int failed_at = -1;

    for (int i = 0; i < ntiles; i++) {
        const int st = (int)((pc + (unsigned)i) % F32_STAGES);
        const unsigned par = ((pc + (unsigned)i) / F32_STAGES) & 1u;
        const bool ok = mbar_wait_bounded(&full[st], par, spins);
        const uint8_t *kgen = stages + (size_t)st * 2 * TILE_BYTES_F32;
        const uint32_t kst = smem_u32(kgen);
        const uint8_t *vgen = kgen + TILE_BYTES_F32;

        // partial scores over dims 64w..64w+63 for the 16 rows of the tile
        // (the three products of the expansion accumulate separately: six independent chains of MMAs per warp
        // instead of two chains of twelve dependent ones)
        float sp[2][4], sp_mid[2][4], sp_kmid[2][4];
#pragma unroll
        for (int nt = 0; nt < 2; nt++)
#pragma unroll
            for (int e = 0; e < 4; e++) sp[nt][e] = sp_mid[nt][e] = sp_kmid[nt][e] = 0.0f;
        if (ok) {
            const int r = lane & 7, mi = lane >> 3;
#pragma unroll
            for (int jx = 0; jx < 4; jx++) {  // one 16-dim k-step per ldmatrix.x4
                const int box = 2 * warp + (jx >> 1);
                const int chunk = ((jx & 1) << 2) + mi;
#pragma unroll
                for (int nt = 0; nt < 2; nt++) {
                    const int row = 8 * nt + r;
                    const uint32_t addr = kst + box * BOX_BYTES + row * 128 + ((chunk ^ (row & 7)) << 4);
                    uint32_t r0, r1, r2, r3;  // K[row g][16 jx + t, + 4, + 8, + 12] of this warp's dims
                    ldmatrix_x4(r0, r1, r2, r3, addr);
                    uint32_t h0, m0, h1, m1;
                    split_bf16x2(__uint_as_float(r0), __uint_as_float(r1), h0, m0);
                    split_bf16x2(__uint_as_float(r2), __uint_as_float(r3), h1, m1);
#if F32_SCORE_CHAINS == 3
                    mma_bf16_16816(sp[nt], qh[jx], h0, h1);
                    mma_bf16_16816(sp_mid[nt], qm[jx], h0, h1);
                    mma_bf16_16816(sp_kmid[nt], qh[jx], m0, m1);
#else
                    mma_bf16_16816(sp[nt], qh[jx], h0, h1);
                    mma_bf16_16816(sp[nt], qm[jx], h0, h1);
                    mma_bf16_16816(sp[nt], qh[jx], m0, m1);
#endif
                }
            }
#if F32_SCORE_CHAINS == 3
#pragma unroll
            for (int nt = 0; nt < 2; nt++)
#pragma unroll
                for (int e = 0; e < 4; e++) sp[nt][e] += sp_mid[nt][e] + sp_kmid[nt][e];
#endif
        }
        float *spw = s_sp + ((i & 1) * 4 + warp) * 16 * SP_STRIDE;
#pragma unroll
        for (int nt = 0; nt < 2; nt++) {
            *reinterpret_cast<float2 *>(spw + g * SP_STRIDE + 8 * nt + 2 * t) = make_float2(sp[nt][0], sp[nt][1]);
            *reinterpret_cast<float2 *>(spw + (g + 8) * SP_STRIDE + 8 * nt + 2 * t) =
                make_float2(sp[nt][2], sp[nt][3]);
        }
        if (!__syncthreads_and(ok ? 1 : 0)) {
            failed_at = i;
            break;
        }
        if (tid == 0 && i >= 1 && (i - 1 + F32_STAGES) < ntiles) issue_tile(i - 1 + F32_STAGES);

        // full scores = sum of the four partial blocks
        float sv[2][4];
#pragma unroll
        for (int nt = 0; nt < 2; nt++) sv[nt][0] = sv[nt][1] = sv[nt][2] = sv[nt][3] = 0.0f;
#pragma unroll
        for (int w = 0; w < 4; w++) {
            const float *src = s_sp + ((i & 1) * 4 + w) * 16 * SP_STRIDE;
#pragma unroll
            for (int nt = 0; nt < 2; nt++) {
                const float2 a = *reinterpret_cast<const float2 *>(src + g * SP_STRIDE + 8 * nt + 2 * t);
                const float2 b = *reinterpret_cast<const float2 *>(src + (g + 8) * SP_STRIDE + 8 * nt + 2 * t);
                sv[nt][0] += a.x;
                sv[nt][1] += a.y;
                sv[nt][2] += b.x;
                sv[nt][3] += b.y;
            }
        }
        const int tile_row0 = c0 + i * F32_TILE;
        if (tile_row0 + F32_TILE > c1) {
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
        if (tile_row0 + F32_TILE > c1) {
            // Rows of the tile past the end of the sequence carry weight zero, but 0 * NaN is NaN: whatever the
            // cache holds there (a caller's uninitialised memory) must not reach the product.  Each warp clears
            // those rows of the two 32-column boxes it reads.
            const int first_bad = c1 - tile_row0;
            uint8_t *vbox = stages + (size_t)st * 2 * TILE_BYTES_F32 + TILE_BYTES_F32 + 2 * warp * BOX_BYTES;
            for (int b = 0; b < 2; b++)
                for (int idx = first_bad * 8 + lane; idx < F32_TILE * 8; idx += 32)
                    *reinterpret_cast<uint4 *>(vbox + b * BOX_BYTES + idx * 16) = make_uint4(0u, 0u, 0u, 0u);
            __syncwarp();
        }
        // O[:, 64w..64w+63] = corr * O + P (16x16) * V (16 x 64): one k-step of 16 tile rows; the score
        // fragment (columns 2t, 2t+1 of each 8-column block) is already in A-operand order.
        // The tile's three products are summed by the tensor core starting from zero (smallest terms first) and
        // joined to the running output by one fused multiply-add per element.  The tensor core truncates its
        // accumulator after every instruction; run through thousands of tiles, an accumulator kept there shrinks
        // by half a unit in the last place each time (1e-4 of its size after 13000 rows), which the fp32 contract
        // has no room for.  Here the long sum rounds to nearest, once per tile.
        {
            uint32_t ph[4], pm[4];
            split_bf16x2(sv[0][0], sv[0][1], ph[0], pm[0]);  // (g,   rows 2t, 2t+1)
            split_bf16x2(sv[0][2], sv[0][3], ph[1], pm[1]);  // (g+8, rows 2t, 2t+1)
            split_bf16x2(sv[1][0], sv[1][1], ph[2], pm[2]);  // (g,   rows 2t+8, 2t+9)
            split_bf16x2(sv[1][2], sv[1][3], ph[3], pm[3]);  // (g+8, rows 2t+8, 2t+9)
            auto v_at = [&](const uint8_t *bx, int r, int col) {
                return *reinterpret_cast<const float *>(bx + r * 128 + ((((col >> 2) ^ (r & 7))) << 4) + (col & 3) * 4);
            };
#pragma unroll
            for (int nt = 0; nt < 8; nt++) {
                const uint8_t *bx = vgen + (2 * warp + (nt >> 2)) * BOX_BYTES;
                const int col = 8 * (nt & 3) + g;
                uint32_t h0, m0, h1, m1;
                split_bf16x2(v_at(bx, 2 * t, col), v_at(bx, 2 * t + 1, col), h0, m0);
                split_bf16x2(v_at(bx, 2 * t + 8, col), v_at(bx, 2 * t + 9, col), h1, m1);
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
        // A load did not arrive within the limit.  The loads that are still in flight write into this CTA's shared
        // memory: wait for them (bounded again) before anything else, then stop streaming for good.
        if (tid == 0) atomicOr(p.status, STATUS_TMA_TIMEOUT);
        const int last_issued = min(ntiles - 1, max(F32_STAGES - 1, failed_at + 1));
        for (int j = failed_at + 1; j <= last_issued; j++)
            mbar_wait_bounded(&full[(pc + (unsigned)j) % F32_STAGES], ((pc + (unsigned)j) / F32_STAGES) & 1u, spins);
        abandoned = true;
        __syncthreads();
    }
    if (seg_no == 0) trace_phase(p, 2);
    finish_unit(p, L, o, m_r, l_r, s_w, s_M, s_L, &s_flag, s_L + 16, abandoned);  // the stage ring is idle here: scratch for the merge
    if (seg_no == 0) trace_phase(p, 3);
    pc += (unsigned)ntiles;
    gt += L.seg;
    seg_no++;
    fence_proxy_async();  // the next segment's TMA loads overwrite memory this segment touched
    __syncthreads();  // shared scratch (RoPE table, score exchange, merge weights) is reused by the next segment
    }
    trace_phase(p, 4);
    publish_exchange_flags(p, &s_flag);
}

constexpr size_t F32_SMEM = 1024 + (size_t)F32_STAGES * 2 * TILE_BYTES_F32 +
                            sizeof(float) * (2 * 4 * 16 * SP_STRIDE + 256) +
                            sizeof(uint64_t) * F32_STAGES;

}  // namespace

cudaError_t gqa_decode_f32_configure() {
    return cudaFuncSetAttribute(gqa_decode_f32_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                (int)F32_SMEM);
}

cudaError_t launch_gqa_decode_f32(const CUtensorMap &kmap, const CUtensorMap &vmap,
                                  const GqaParams &p, cudaStream_t stream) {
    if (p.total_ctas <= 0) return cudaSuccess;
    if (p.coop_merge) {
        // every CTA resident at once: CTAs that share a unit may wait for one another (merge_unit_slices)
        void *args[] = {const_cast<CUtensorMap *>(&kmap), const_cast<CUtensorMap *>(&vmap), const_cast<GqaParams *>(&p)};
        return cudaLaunchCooperativeKernel(reinterpret_cast<void *>(gqa_decode_f32_kernel), dim3(p.total_ctas), dim3(128), args, F32_SMEM, stream);
    }
    gqa_decode_f32_kernel<<<p.total_ctas, 128, F32_SMEM, stream>>>(kmap, vmap, p);
    return cudaGetLastError();
}

int gqa_decode_f32_coop_capacity() {
    int dev = 0, sms = 0, per_sm = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, gqa_decode_f32_kernel, 128, F32_SMEM) != cudaSuccess)
        return 0;
    int coop = 0;
    cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev);
    return coop ? sms * per_sm : 0;
}

}  // namespace mfc
