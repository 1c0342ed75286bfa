// Causal GQA prefill (flash-attention forward) on the 5th-generation tensor
// cores: tcgen05.mma with operands staged in shared memory by TMA and the
// accumulators in tensor memory (TMEM).
//
// The reference has no batched prefill: eval_prompt runs the decode step once
// per token (crates/moeflux/src/riir/mod.rs:1206-1212).  This kernel computes
// the same result for T tokens at once: for token t (absolute position
// start_pos + t) the full-attention step of crates/moeflux/src/riir/
// full_attn_forward.rs:278-389 -- RoPE(q, k), append, softmax(q K^T / 16) V over
// rows [0, start_pos + t], sigmoid gate -- with bf16 activations.
//
// Two launches:
//   1. prefill_kv_append_kernel: per token, the RoPE table entry (accurate
//      sincosf of pos * inv_freq, shared by all heads), rotated K and V rows
//      stored into the cache.
//   2. gqa_prefill_kernel: CTA = 128 query tokens of one query head (M = 128);
//      eight softmax warps (thread = query row x half of the columns), one warp
//      that issues every tcgen05.mma and one that issues every TMA load.
//      Per 64-row KV tile: S = Q K^T (16 tcgen05.mma of K=16, N=64, fp32 in
//      TMEM), softmax with one thread per query row (tcgen05.ld, no shuffles),
//      P written to shared memory as bf16, O += P V (4 tcgen05.mma, N=256,
//      V as an MN-major operand straight from the cache layout).  S is double
//      buffered in TMEM so Q K^T of tile j+1 runs under the softmax of tile j;
//      O is rescaled in TMEM only when a row maximum grows by more than 2^8
//      (stale-max trick), which is rare after the first tiles.
// Every mbarrier wait is bounded; a wait that expires sets a status bit, the CTA
// frees its TMEM and leaves.
#include <math.h>

#include "common.cuh"
#include "kernels.h"
#include "tcgen05.cuh"

namespace mfc {

namespace {

constexpr int PF_M = 128;        // query rows per CTA
constexpr int PF_N = 64;         // KV rows per tile
constexpr int PF_STAGES = 2;
constexpr float LOG2E_PF = 1.4426950408889634f;

constexpr uint32_t Q_BYTES = PF_M * HEAD_DIM * 2;      // 64 KiB: 4 boxes of [128 x 64]
constexpr uint32_t Q_BOX = PF_M * 128;                 // 16 KiB
constexpr uint32_t KV_TILE_BYTES = PF_N * HEAD_DIM * 2;  // 32 KiB: 4 boxes of [64 x 64]
constexpr uint32_t KV_BOX = PF_N * 128;                // 8 KiB
constexpr uint32_t P_BYTES = PF_M * PF_N * 2;          // 16 KiB
constexpr uint32_t OFF_Q = 0;
constexpr uint32_t OFF_K = OFF_Q + Q_BYTES;
constexpr uint32_t OFF_V = OFF_K + PF_STAGES * KV_TILE_BYTES;
constexpr uint32_t OFF_P = OFF_V + PF_STAGES * KV_TILE_BYTES;
constexpr uint32_t OFF_BAR = OFF_P + 2 * P_BYTES;
constexpr uint32_t OFF_XM = OFF_BAR + 256;               // row-maximum exchange, bf16 [2 tiles][2 halves][128 rows]
constexpr uint32_t PF_SMEM = OFF_XM + 1024 + 1024;      // + alignment slack
constexpr int PF_THREADS = 320;

constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t TM_S = 0;      // two S buffers of 64 columns
constexpr uint32_t TM_O = 128;    // O accumulator, 256 columns

// 320 threads: warps 0-7 own the 128 query rows, two warps (column halves) per TMEM lane
// quadrant (softmax, rescale, epilogue); warp 8 issues every tcgen05.mma and warp 9 every
// TMA load.  The MMA issue of a tile blocks its
// thread for about as long as the tensor core needs (~1350 cycles), so neither the
// softmax nor the issue of the loads (~550 cycles a tile) may share that thread.
__global__ void __launch_bounds__(PF_THREADS, 1)
gqa_prefill_kernel(const __grid_constant__ CUtensorMap qmap, const __grid_constant__ CUtensorMap kmap,
                   const __grid_constant__ CUtensorMap vmap, const PrefillAttnParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + OFF_BAR);
    uint64_t *full_q = bars + 0;    // TMA: Q tile landed
    uint64_t *full_k = bars + 1;    // [2] TMA: K stage landed
    uint64_t *full_v = bars + 3;    // [2] TMA: V stage landed
    uint64_t *s_ready = bars + 5;   // [2] tcgen05.commit: scores of a tile are in TMEM
    uint64_t *pv_done = bars + 7;   // [2] tcgen05.commit: P V of a tile has been accumulated
    uint64_t *p_ready = bars + 9;   // [2] 8 warps: P of a tile is in shared memory, S has been read
    uint64_t *q_ready = bars + 11;  // 8 warps: Q has been rotated in shared memory
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 12);
    volatile int *s_fail = reinterpret_cast<volatile int *>(bars + 13);
    uint64_t *x_ready = bars + 14;  // [4] 2 warps: both column halves of a lane quadrant have published their row maxima

    const int tid = threadIdx.x, warp = tid >> 5;
    const int n_qt = (p.T + PF_M - 1) / PF_M;
    const int qt = n_qt - 1 - (int)blockIdx.x;  // longest tiles first
    const int h = blockIdx.y;
    const int kvh = h / p.group;
    const int t0 = qt * PF_M;
    const int kv_need = p.start_pos + min(p.T, t0 + PF_M);  // rows this tile may attend to
    const int ntiles = (kv_need + PF_N - 1) / PF_N;
    const int kv_row0 = (p.kv_slot * p.Hkv + kvh) * p.cap_rows;

    if (tid == 0) {
        prefetch_tmap(&qmap);
        prefetch_tmap(&kmap);
        prefetch_tmap(&vmap);
        for (int i = 0; i < 9; i++) mbar_init(&bars[i], 1);
        mbar_init(&p_ready[0], 8);  // one arrival per softmax warp
        mbar_init(&p_ready[1], 8);
        mbar_init(q_ready, 8);
        for (int i = 0; i < 4; i++) mbar_init(&x_ready[i], 2);
        *s_fail = 0;
        mbar_fence_init();
    }
    if (warp == 0) {
        tmem_alloc(tmem_slot, TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    bool ok = true;

    if (warp == 9) {
        // ================= producer warp: one lane issues every TMA load =================
        if ((tid & 31) == 0) {
            auto load_k = [&](int tile) {
                const int st = tile & 1;
                mbar_expect_tx(&full_k[st], KV_TILE_BYTES);
#pragma unroll
                for (int b = 0; b < 4; b++)
                    tma_load_2d(smem + OFF_K + st * KV_TILE_BYTES + b * KV_BOX, &kmap, b * 64, kv_row0 + tile * PF_N,
                                &full_k[st]);
            };
            auto load_v = [&](int tile) {
                const int st = tile & 1;
                mbar_expect_tx(&full_v[st], KV_TILE_BYTES);
#pragma unroll
                for (int b = 0; b < 4; b++)
                    tma_load_2d(smem + OFF_V + st * KV_TILE_BYTES + b * KV_BOX, &vmap, b * 64, kv_row0 + tile * PF_N,
                                &full_v[st]);
            };
            mbar_expect_tx(full_q, Q_BYTES);
#pragma unroll
            for (int b = 0; b < 4; b++) tma_load_3d(smem + OFF_Q + b * Q_BOX, &qmap, b * 64, h, t0, full_q);
            load_k(0);
            load_v(0);
            if (ntiles > 1) {
                load_k(1);
                load_v(1);
            }
            for (int j = 0; j + 2 < ntiles && ok; j++) {
                const int b = j & 1;
                const unsigned par = (unsigned)(j >> 1) & 1u;
                // the K stage of tile j is free once Q K^T of tile j has completed, its V stage once P V of tile j has
                ok = mbar_wait_bounded(&s_ready[b], par);
                if (!ok) break;
                load_k(j + 2);
                ok = mbar_wait_bounded(&pv_done[b], par);
                if (!ok) break;
                load_v(j + 2);
            }
            if (!ok) *s_fail = 1;
        }
    } else if (warp == 8) {
        // ================= issuer warp: one lane drives the tensor core =================
        if ((tid & 31) == 0) {
            constexpr uint32_t IDESC_QK = idesc_bf16(PF_N, 0);
            constexpr uint32_t IDESC_PV = idesc_bf16(HEAD_DIM, 1);
            // descriptors differ only in their start-address field: build the bases once
            const uint64_t q_desc = smem_desc_sw128(smem_u32(smem + OFF_Q), 16, 1024);
            const uint64_t k_desc0 = smem_desc_sw128(smem_u32(smem + OFF_K), 16, 1024);
            const uint64_t p_desc0 = smem_desc_sw128(smem_u32(smem + OFF_P), 16, 1024);
            // V: MN-major; 64-dim atoms KV_BOX apart (LBO), 8-row groups 1024 B apart (SBO)
            const uint64_t v_desc0 = smem_desc_sw128(smem_u32(smem + OFF_V), KV_BOX, 1024);
            auto issue_qk = [&](int tile) {  // S[tile&1] = Q K^T
                const uint64_t kd = k_desc0 + (uint64_t)(((tile & 1) * KV_TILE_BYTES) >> 4);
#pragma unroll
                for (int ks = 0; ks < 16; ks++)
                    tc_mma_bf16(tmem + TM_S + (tile & 1) * PF_N, q_desc + (uint64_t)(((ks >> 2) * Q_BOX + (ks & 3) * 32) >> 4),
                                kd + (uint64_t)(((ks >> 2) * KV_BOX + (ks & 3) * 32) >> 4), IDESC_QK, ks > 0);
                tc_commit(&s_ready[tile & 1]);
            };
            auto issue_pv = [&](int tile) {  // O += P V
                const uint64_t pd = p_desc0 + (uint64_t)(((tile & 1) * P_BYTES) >> 4);
                const uint64_t vd = v_desc0 + (uint64_t)(((tile & 1) * KV_TILE_BYTES) >> 4);
#pragma unroll
                for (int ks = 0; ks < PF_N / 16; ks++)
                    tc_mma_bf16(tmem + TM_O, pd + (uint64_t)((ks * 32) >> 4), vd + (uint64_t)((ks * 2048) >> 4), IDESC_PV,
                                (tile > 0) || (ks > 0));
                tc_commit(&pv_done[tile & 1]);
            };
            ok = mbar_wait_bounded(q_ready, 0) && mbar_wait_bounded(&full_k[0], 0);
            if (ok) {
                tc_fence_after();
                issue_qk(0);
            }
            for (int j = 0; j < ntiles && ok; j++) {
                const int b = j & 1;
                const unsigned par = (unsigned)(j >> 1) & 1u;
                if (j + 1 < ntiles) {
                    // S[(j+1)&1] was read by the softmax of tile j-1, which this thread saw finish (p_ready) last turn
                    ok = mbar_wait_bounded(&full_k[(j + 1) & 1], (unsigned)((j + 1) >> 1) & 1u);
                    if (!ok) break;
                    tc_fence_after();
                    issue_qk(j + 1);
                }
                // P of tile j is in shared memory, V of tile j has landed
                ok = mbar_wait_bounded(&p_ready[b], par) && mbar_wait_bounded(&full_v[b], par);
                if (!ok) break;
                tc_fence_after();
                issue_pv(j);
            }
            if (!ok) *s_fail = 1;
        }
    } else {
        // ================= softmax warps: thread = (query row, half of the columns) =================
        // warps w and w+4 share TMEM lane quadrant w: warp w takes columns 0-31 of a 64-column score tile (and
        // dims 0-127 of O), warp w+4 the rest; the two exchange their row maxima through shared memory.
        const int quad = warp & 3, hf = warp >> 2;
        const int row = 32 * quad + (tid & 31);  // query row of the tile = TMEM lane
        const int row_tok = t0 + row;            // this thread's query token
        const int qpos = p.start_pos + row_tok;  // its absolute position
        const uint32_t lane_base = tmem + ((uint32_t)(32 * quad) << 16);
        __nv_bfloat16 *xm = reinterpret_cast<__nv_bfloat16 *>(smem + OFF_XM);
        auto warp_arrive = [&](uint64_t *bar) {
            __syncwarp();
            if ((tid & 31) == 0) mbar_arrive(bar);
        };
        // exchange point of the two warps of a quadrant (bounded, like every other wait here)
        unsigned x_phase = 0;
        auto pair_sync = [&]() -> bool {
            warp_arrive(&x_ready[quad]);
            const bool done = __all_sync(0xffffffffu, mbar_wait_bounded(&x_ready[quad], x_phase & 1u));
            x_phase++;
            return done;
        };

        // ---- RoPE on this thread's share of its Q row, in shared memory (dims 0..63 live in box 0) ----
        ok = __all_sync(0xffffffffu, mbar_wait_bounded(full_q, 0));
        if (ok && p.rotary_dim > 0 && row_tok < p.T) {
            const int half = p.rotary_dim >> 1;  // <= 32 here (rotary_dim <= 64)
            uint8_t *rowp = smem + OFF_Q + row * 128;
            const float2 *cs = reinterpret_cast<const float2 *>(p.cos_sin) + (size_t)row_tok * 32;
            for (int i0 = 8 * hf; i0 < half; i0 += 16) {
                const int c_lo = i0 >> 3, c_hi = (i0 + half) >> 3;
                uint4 *plo = reinterpret_cast<uint4 *>(rowp + ((c_lo ^ (row & 7)) << 4));
                uint4 *phi = reinterpret_cast<uint4 *>(rowp + ((c_hi ^ (row & 7)) << 4));
                uint4 lo = *plo, hi = *phi;
                __nv_bfloat16 *a = reinterpret_cast<__nv_bfloat16 *>(&lo);
                __nv_bfloat16 *b = reinterpret_cast<__nv_bfloat16 *>(&hi);
#pragma unroll
                for (int e = 0; e < 8; e++) {
                    const float2 c = cs[i0 + e];  // (cos, sin)
                    const float x0 = __bfloat162float(a[e]), x1 = __bfloat162float(b[e]);
                    a[e] = __float2bfloat16_rn(x0 * c.x - x1 * c.y);
                    b[e] = __float2bfloat16_rn(x0 * c.y + x1 * c.x);
                }
                *plo = lo;
                *phi = hi;
            }
        }
        fence_proxy_async_smem();
        warp_arrive(q_ready);

        float m_run = -INFINITY, l_run = 0.0f;  // l_run: this thread's 32 columns of every tile only
        const float sl2 = p.scale * LOG2E_PF;
        for (int j = 0; j < ntiles && ok; j++) {
            const int b = j & 1;
            const unsigned par = (unsigned)(j >> 1) & 1u;
            ok = __all_sync(0xffffffffu, mbar_wait_bounded(&s_ready[b], par) && *s_fail == 0);
            if (!ok) break;
            tc_fence_after();
            float s[32];
            tmem_ld32(lane_base + TM_S + b * PF_N + 32 * hf, s);
            tc_wait_ld();
            const int kv0 = j * PF_N + 32 * hf;
            if (j * PF_N + PF_N - 1 > p.start_pos + t0) {  // tile touches the diagonal
#pragma unroll
                for (int c = 0; c < 32; c++)
                    if (kv0 + c > qpos) s[c] = -INFINITY;
            }
            float mx = s[0];
#pragma unroll
            for (int c = 1; c < 32; c++) mx = fmaxf(mx, s[c]);
            // The two halves of a row must agree on the maximum they use: both round their own up to bf16 (the
            // running maximum only has to bound the scores from above, roughly) and take the larger.
            __nv_bfloat16 mx_b = __float2bfloat16_ru(mx);
            xm[(b * 2 + hf) * PF_M + row] = mx_b;
            ok = pair_sync();
            if (!ok) break;
            const float m_tile = fmaxf(__bfloat162float(mx_b), __bfloat162float(xm[(b * 2 + (hf ^ 1)) * PF_M + row]));
            const float m_new = fmaxf(m_run, m_tile);
            // rescale O only when some row of the quadrant moved its maximum by more than 2^8
            const bool need = (m_new - m_run) * sl2 > 8.0f;  // also true on the first tile (m_run = -inf)
            const bool warp_rescale = __any_sync(0xffffffffu, need);
            float corr = 1.0f;
            if (warp_rescale) {
                corr = ex2_approx((m_run - m_new) * sl2);
                m_run = m_new;
            }
            const float mb = m_run * sl2;
            float rs = 0.0f;
            uint32_t pk[16];
#pragma unroll
            for (int c = 0; c < 32; c += 2) {
                const float p0 = ex2_approx(fmaf(s[c], sl2, -mb));
                const float p1 = ex2_approx(fmaf(s[c + 1], sl2, -mb));
                rs += p0 + p1;
                pk[c >> 1] = pack_bf16x2(p0, p1);
            }
            l_run = l_run * corr + rs;

            // P buffer b last fed P V of tile j-2, which the commit behind s_ready[b] already covers.
            // O may be touched only once P V of tile j-1 has completed.
            if (warp_rescale && j > 0) {
                ok = __all_sync(0xffffffffu, mbar_wait_bounded(&pv_done[(j - 1) & 1], (unsigned)((j - 1) >> 1) & 1u));
                if (!ok) break;
                tc_fence_after();
#pragma unroll 1
                for (int c0 = 128 * hf; c0 < 128 * hf + 128; c0 += 32) {
                    float o[32];
                    tmem_ld32(lane_base + TM_O + c0, o);
                    tc_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; i++) o[i] *= corr;
                    tmem_st32(lane_base + TM_O + c0, *reinterpret_cast<float(*)[32]>(&o[0]));
                }
                tc_wait_st();
            }
            {
                uint8_t *prow = smem + OFF_P + b * P_BYTES + row * 128;
#pragma unroll
                for (int c = 0; c < 4; c++)
                    *reinterpret_cast<uint4 *>(prow + (((4 * hf + c) ^ (row & 7)) << 4)) =
                        make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
            }
            fence_proxy_async_smem();
            tc_fence_before();
            warp_arrive(&p_ready[b]);
        }
        if (ok && ntiles > 0) {
            ok = __all_sync(0xffffffffu,
                            mbar_wait_bounded(&pv_done[(ntiles - 1) & 1], (unsigned)((ntiles - 1) >> 1) & 1u));
            tc_fence_after();
        }
        // row sum = the two halves' partial sums (both carry the same running maximum); every MMA has completed,
        // so the P buffers are free to carry the exchange
        float *xl = reinterpret_cast<float *>(smem + OFF_P);
        if (ok) {
            xl[hf * PF_M + row] = l_run;
            ok = pair_sync();
            l_run += xl[(hf ^ 1) * PF_M + row];
        }
        if (ok) {
            // every lane takes part in the warp-wide TMEM loads; only the global accesses are predicated
            const bool valid = row_tok < p.T;
            const float inv = 1.0f / l_run;
            const size_t off = ((size_t)(valid ? row_tok : 0) * p.H + h) * HEAD_DIM;
#pragma unroll 1
            for (int c0 = 128 * hf; c0 < 128 * hf + 128; c0 += 32) {
                float o[32];
                tmem_ld32(lane_base + TM_O + c0, o);
                tc_wait_ld();
                if (valid) {
#pragma unroll
                    for (int v8 = 0; v8 < 4; v8++) {
                        uint4 g4 = make_uint4(0, 0, 0, 0);
                        if (p.gate) g4 = *reinterpret_cast<const uint4 *>(p.gate + off + c0 + v8 * 8);
                        const __nv_bfloat16 *gb = reinterpret_cast<const __nv_bfloat16 *>(&g4);
                        uint32_t w[4];
#pragma unroll
                        for (int e = 0; e < 4; e++) {
                            float x0 = o[v8 * 8 + 2 * e] * inv, x1 = o[v8 * 8 + 2 * e + 1] * inv;
                            if (p.gate) {
                                x0 *= 1.0f / (1.0f + expf(-__bfloat162float(gb[2 * e])));
                                x1 *= 1.0f / (1.0f + expf(-__bfloat162float(gb[2 * e + 1])));
                            }
                            w[e] = pack_bf16x2(x0, x1);
                        }
                        *reinterpret_cast<uint4 *>(p.out + off + c0 + v8 * 8) = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                }
            }
        } else if ((tid & 31) == 0) {
            *s_fail = 1;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (tid == 0 && *s_fail) atomicOr(p.status, STATUS_TMA_TIMEOUT);
    if (warp == 0) tmem_dealloc(tmem, TMEM_COLS);
}

// ---- RoPE table + KV append for T tokens ------------------------------------------
template <typename CacheT>
__global__ void __launch_bounds__(128)
prefill_kv_append_kernel(const __nv_bfloat16 *k, const __nv_bfloat16 *v, CacheT *k_cache, CacheT *v_cache,
                         float *cos_sin, const float *inv_freq, int T, int Hkv, int rotary_dim, int start_pos,
                         size_t slot_row0, int cap_rows, int rank, int world, int block) {
    __shared__ float s_cos[128], s_sin[128];
    const int t = blockIdx.x;
    const int pos = start_pos + t;
    const int half = rotary_dim >> 1;
    if (threadIdx.x < half) {
        float sn, cs;
        sincosf((float)pos * inv_freq[threadIdx.x], &sn, &cs);
        s_cos[threadIdx.x] = cs;
        s_sin[threadIdx.x] = sn;
        if (threadIdx.x < 32) reinterpret_cast<float2 *>(cos_sin)[(size_t)t * 32 + threadIdx.x] = make_float2(cs, sn);
    }
    __syncthreads();
    int row = pos;
    if (world > 1) {
        const int blk = pos / block;
        if (blk % world != rank) return;  // another context stores this position
        row = (blk / world) * block + pos % block;
    }
    for (int idx = threadIdx.x; idx < Hkv * HEAD_DIM; idx += blockDim.x) {
        const int hh = idx / HEAD_DIM, d = idx % HEAD_DIM;
        const __nv_bfloat16 *kr = k + ((size_t)t * Hkv + hh) * HEAD_DIM;
        float x = __bfloat162float(kr[d]);
        if (d < rotary_dim) {
            if (d < half) x = x * s_cos[d] - __bfloat162float(kr[d + half]) * s_sin[d];
            else x = __bfloat162float(kr[d - half]) * s_sin[d - half] + x * s_cos[d - half];
        }
        const size_t o = (slot_row0 + (size_t)hh * cap_rows + row) * HEAD_DIM + d;
        k_cache[o] = (CacheT)x;
        v_cache[o] = (CacheT)__bfloat162float(v[((size_t)t * Hkv + hh) * HEAD_DIM + d]);
    }
}

}  // namespace

cudaError_t gqa_prefill_configure() {
    return cudaFuncSetAttribute(gqa_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PF_SMEM);
}

cudaError_t launch_prefill_kv_append(const void *k_bf16, const void *v_bf16, void *k_cache, void *v_cache,
                                     int kv_bf16, float *cos_sin, const float *inv_freq, int T, int Hkv,
                                     int rotary_dim, int start_pos, size_t slot_row0, int cap_rows, int rank,
                                     int world, int block, cudaStream_t stream) {
    if (T <= 0) return cudaSuccess;
    const __nv_bfloat16 *k = reinterpret_cast<const __nv_bfloat16 *>(k_bf16);
    const __nv_bfloat16 *v = reinterpret_cast<const __nv_bfloat16 *>(v_bf16);
    if (kv_bf16)
        prefill_kv_append_kernel<__nv_bfloat16><<<T, 128, 0, stream>>>(
            k, v, reinterpret_cast<__nv_bfloat16 *>(k_cache), reinterpret_cast<__nv_bfloat16 *>(v_cache), cos_sin,
            inv_freq, T, Hkv, rotary_dim, start_pos, slot_row0, cap_rows, rank, world, block);
    else
        prefill_kv_append_kernel<float><<<T, 128, 0, stream>>>(k, v, reinterpret_cast<float *>(k_cache),
                                                               reinterpret_cast<float *>(v_cache), cos_sin, inv_freq,
                                                               T, Hkv, rotary_dim, start_pos, slot_row0, cap_rows,
                                                               rank, world, block);
    return cudaGetLastError();
}

cudaError_t launch_gqa_prefill(const CUtensorMap &qmap, const CUtensorMap &kmap, const CUtensorMap &vmap,
                               const PrefillAttnParams &p, cudaStream_t stream) {
    if (p.T <= 0) return cudaSuccess;
    dim3 grid((unsigned)((p.T + PF_M - 1) / PF_M), (unsigned)p.H, 1);
    gqa_prefill_kernel<<<grid, PF_THREADS, PF_SMEM, stream>>>(qmap, kmap, vmap, p);
    return cudaGetLastError();
}

}  // namespace mfc
