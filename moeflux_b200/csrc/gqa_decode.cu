// Split-K flash-decoding for GQA full attention with the sigmoid output gate,
// bf16 KV cache, for sm_100a.
//
// One launch performs, for every (layer, sequence) item, what the reference
// does with RoPE + KV append on the host and four GPU kernels
// (crates/moeflux/src/riir/rope.rs:65-131, full_attn_forward.rs:281-323,
// crates/moeflux/shaders/shaders.metal: attn_scores_batched :976-1019,
// attn_softmax_batched :1026-1084, attn_values_batched :1095-1117,
// sigmoid_gate :1125-1134), or with sdpa_cpu (sdpa.rs:63-172) outside
// 32 <= kv_len < 8192.
//
// Work split ("stream-K" over KV tiles).  The 32-row tiles of all (item, kv head)
// units of a launch form one sequence, cut into equal runs, one CTA (4 warps) per
// run, across unit boundaries; a CTA walks its run one unit segment at a time.
// The up-to-16 query heads that share the kv head are the M=16 rows of mma.sync
// m16n8k16, so a cached row is read from HBM once for all of them.  K/V tiles
// arrive by TMA (cp.async.bulk.tensor, 128-byte swizzle, four 64-column boxes
// per tensor) into a multi-stage shared-memory ring guarded by mbarriers with
// bounded waits.  Per tile: warp w computes the scores of rows 8w..8w+7 over
// all 256 dims (Q fragments live in registers), the four 16x8 score blocks are
// exchanged through shared memory, every warp runs the same online softmax
// (warp-shuffle row max) and then accumulates P·V for its own 64 output dims.
// A unit that lies inside one run is finished in place; a unit cut by run
// boundaries is merged from the un-normalised (o, m, l) partials of the CTAs
// that share it by the last of them to finish (atomic tickets, no spinning, two
// levels when more than eight CTAs share it), which applies the sigmoid gate
// and writes the output.  With partial_mode the merged un-normalised partial is
// written instead, for the cross-GPU KV split -- to local memory, or straight
// into the receive buffer of the GPU that finishes the item (peer stores).
//
// RoPE and the append are fused: every CTA rotates q while building its
// fragments; the CTA whose chunk holds the new row rotates k, stores k and v
// into the cache, fences, and only then starts its TMA loads.
#include <math.h>

#include "gqa_common.cuh"

namespace mfc {

namespace {

constexpr int BF16_STAGES = 3;
constexpr int TILE_BYTES_BF16 = KV_TILE * HEAD_DIM * 2;  // 16 KiB per tensor per stage
constexpr int SX_STRIDE = 40;                            // padded row stride of the score exchange

__global__ void __launch_bounds__(128, 2)
gqa_decode_bf16_kernel(const __grid_constant__ CUtensorMap kmap,
                       const __grid_constant__ CUtensorMap vmap, const __grid_constant__ GqaParams p) {
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment for the 128-byte swizzle atoms
    uint8_t *smem = reinterpret_cast<uint8_t *>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *stages = smem;  // [STAGES][K tile | V tile]
    float *s_sx = reinterpret_cast<float *>(smem + BF16_STAGES * 2 * TILE_BYTES_BF16);  // [2][16][40]
    float *s_cos = s_sx + 2 * 16 * SX_STRIDE;  // [128]
    float *s_sin = s_cos + 128;                // [128]
    float *s_w = s_sin + 128;                  // [MAX_SPLITS*16]
    float *s_M = s_w + MAX_SPLITS * 16;        // [16]
    float *s_L = s_M + 16;                     // [16]
    uint64_t *full = reinterpret_cast<uint64_t *>(s_L + 16);  // [STAGES]
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
        for (int s = 0; s < BF16_STAGES; s++) mbar_init(&full[s], 1);
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
    const Located L = locate_tile<KV_TILE>(p, gt, gt_end, s_begin);
    const GqaItem &it = L.it;
    const int group = p.group;
    if (L.bad && !abandoned) {
        if (tid == 0) atomicOr(p.status, STATUS_BAD_ITEM);
        abandoned = true;
    }
    if (abandoned) {  // take the unit's tickets so that the counters return to zero, touch nothing else
        float o0[8][4] = {};
        float m0[2] = {-INFINITY, -INFINITY}, l0[2] = {0.0f, 0.0f};
        finish_unit(p, L, o0, m0, l0, s_w, s_M, s_L, &s_flag, reinterpret_cast<float *>(stages), true);
        gt += L.seg;
        __syncthreads();
        continue;
    }

    const int c0 = L.t0 * KV_TILE;
    const int c1 = min(c0 + L.seg * KV_TILE, it.local_len);
    const int ntiles = (c1 > c0) ? (c1 - c0 + KV_TILE - 1) / KV_TILE : 0;
    const int row_base = (it.kv_slot * p.Hkv + L.kvh) * p.cap_rows;
    const bool appender = it.append_row >= c0 && it.append_row < c0 + L.seg * KV_TILE;

    const bool lose_load = p.inject_lost_load && blockIdx.x == 0 && seg_no == 0;
    auto issue_tile = [&](int tile) {
        const int st = (int)((pc + (unsigned)tile) % BF16_STAGES);
        uint8_t *kdst = stages + (size_t)st * 2 * TILE_BYTES_BF16;
        uint8_t *vdst = kdst + TILE_BYTES_BF16;
        mbar_expect_tx(&full[st], 2 * TILE_BYTES_BF16);
        if (lose_load && tile == 0) return;  // diagnostic: the barrier is armed and nothing will ever arrive
        const int y = row_base + c0 + tile * KV_TILE;
#pragma unroll
        for (int b = 0; b < 4; b++) {
            tma_load_2d(kdst + b * 4096, &kmap, b * 64, y, &full[st]);
            tma_load_2d(vdst + b * 4096, &vmap, b * 64, y, &full[st]);
        }
    };

    // (the last stage of the ring first carries the Q rows)
    float *s_q = reinterpret_cast<float *>(stages + (size_t)((pc + BF16_STAGES - 1) % BF16_STAGES) * 2 * TILE_BYTES_BF16);
    stage_q_rows(p.q + ((size_t)it.in_idx * p.H + (size_t)L.kvh * group) * (size_t)p.q_row_stride, group, p.q_row_stride, s_q);
    // RoPE table for this token
    const int half = p.rotary_dim >> 1;
    if (tid < half) {
        float sn, cs;
        sincosf((float)it.pos * p.inv_freq[tid], &sn, &cs);
        s_cos[tid] = cs;
        s_sin[tid] = sn;
    }
    __syncthreads();
    // The first tiles of the segment are requested only now, with the query rows already in shared memory: every CTA
    // of a launch starts at the same time, and query rows asked for behind 57 MB of first tiles came back after 8 us
    // while the ring sat full and idle.  (The rows themselves take a microsecond; nothing can be computed before.)
    if (tid == 0 && !appender) {
        const int n0 = min(ntiles, BF16_STAGES - 1);
        for (int i = 0; i < n0; i++) issue_tile(i);
    }
    if (seg_no == 0) trace_phase(p, 5);  // query rows and the RoPE table are in shared memory

    if (appender) {
        // rotate k, store the new K and V rows (bf16), then let thread 0 start the loads
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
        *reinterpret_cast<uint32_t *>(reinterpret_cast<__nv_bfloat16 *>(p.k_base) + roff) =
            pack_bf16x2(kx.x, kx.y);
        *reinterpret_cast<uint32_t *>(reinterpret_cast<__nv_bfloat16 *>(p.v_base) + roff) =
            pack_bf16x2(vx.x, vx.y);
        __threadfence();
        fence_proxy_async();
        __syncthreads();
        if (tid == 0) {
            const int n0 = min(ntiles, BF16_STAGES - 1);
            for (int i = 0; i < n0; i++) issue_tile(i);
        }
    }

    // ---- Q fragments (A operand, 16 heads x 256 dims, bf16), RoPE applied ----
    // Two compact steps (a long unrolled build runs once per segment from a cold instruction cache and cost
    // ~12 us): normalise / rotate into a bf16 tile beside the staged rows, then one ldmatrix per k-step.
    uint32_t qa[16][4];
    {
        constexpr int QB_STRIDE = HEAD_DIM + 8;  // bf16: rows 16-byte aligned, conflict-free for ldmatrix
        __nv_bfloat16 *s_qb = reinterpret_cast<__nv_bfloat16 *>(s_q + 16 * Q_STAGE_STRIDE);
        const uint16_t *qnw = p.qnorm_w ? p.qnorm_w + (size_t)(it.kv_slot / p.n_seqs) * HEAD_DIM : nullptr;
        if (qnw) head_inv_rms(s_q, group, Q_STAGE_STRIDE, p.norm_eps, s_inv);
#pragma unroll 1
        for (int idx = tid; idx < 16 * (HEAD_DIM / 2); idx += 128) {
            const int row = idx >> 7, d = (idx & 127) * 2;
            float2 x = make_float2(0.0f, 0.0f);
            if (row < group)
                x = load_rot2(s_q + row * Q_STAGE_STRIDE, d, p.rotary_dim, half, s_cos, s_sin, qnw ? s_inv[row] : 1.0f, qnw);
            *reinterpret_cast<uint32_t *>(s_qb + row * QB_STRIDE + d) = pack_bf16x2(x.x, x.y);
        }
        __syncthreads();
        if (seg_no == 0) trace_phase(p, 6);  // appended (if this CTA appends), normalised and rotated
#pragma unroll
        for (int ks = 0; ks < 16; ks++)
            ldmatrix_x4(qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3],
                        smem_u32(s_qb + (lane & 15) * QB_STRIDE + 16 * ks + (lane >> 4) * 8));
    }
    fence_proxy_async();  // the Q staging area goes back to the ring
    __syncthreads();
    if (tid == 0 && ntiles >= BF16_STAGES) issue_tile(BF16_STAGES - 1);
    if (seg_no == 0) trace_phase(p, 1);

    float o[8][4];
#pragma unroll
    for (int i = 0; i < 8; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
    float m_r[2] = {-INFINITY, -INFINITY};
    float l_r[2] = {0.0f, 0.0f};
    const float sl2 = p.scale * LOG2E;
    int failed_at = -1;

    for (int i = 0; i < ntiles; i++) {
        const int st = (int)((pc + (unsigned)i) % BF16_STAGES);
        const unsigned par = ((pc + (unsigned)i) / BF16_STAGES) & 1u;
        const bool ok = mbar_wait_bounded(&full[st], par, spins);
        const uint32_t kst = smem_u32(stages + (size_t)st * 2 * TILE_BYTES_BF16);
        const uint32_t vst = kst + TILE_BYTES_BF16;

        // scores of rows 8w..8w+7 against all 16 heads
        float sacc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        if (ok) {
            const int r = lane & 7, mi = lane >> 3;
            const int row = 8 * warp + r;
#pragma unroll
            for (int jx = 0; jx < 8; jx++) {
                const int box = jx >> 1, chunk = ((jx & 1) << 2) + mi;
                const uint32_t addr = kst + box * 4096 + row * 128 + ((chunk ^ (row & 7)) << 4);
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4(b0, b1, b2, b3, addr);
                mma_bf16_16816(sacc, qa[2 * jx], b0, b1);
                mma_bf16_16816(sacc, qa[2 * jx + 1], b2, b3);
            }
        }
        float *sx = s_sx + (i & 1) * 16 * SX_STRIDE;
        *reinterpret_cast<float2 *>(sx + g * SX_STRIDE + 8 * warp + 2 * t) =
            make_float2(sacc[0], sacc[1]);
        *reinterpret_cast<float2 *>(sx + (g + 8) * SX_STRIDE + 8 * warp + 2 * t) =
            make_float2(sacc[2], sacc[3]);
        if (!__syncthreads_and(ok ? 1 : 0)) {
            failed_at = i;
            break;
        }
        // every warp is past its reads of tile i-1: refill that stage
        if (tid == 0 && i >= 1 && (i - 1 + BF16_STAGES) < ntiles) issue_tile(i - 1 + BF16_STAGES);

        float sv[4][4];
#pragma unroll
        for (int nt = 0; nt < 4; nt++) {
            const float2 a = *reinterpret_cast<const float2 *>(sx + g * SX_STRIDE + 8 * nt + 2 * t);
            const float2 b =
                *reinterpret_cast<const float2 *>(sx + (g + 8) * SX_STRIDE + 8 * nt + 2 * t);
            sv[nt][0] = a.x;
            sv[nt][1] = a.y;
            sv[nt][2] = b.x;
            sv[nt][3] = b.y;
        }
        const int tile_row0 = c0 + i * KV_TILE;
        if (tile_row0 + KV_TILE > c1) {
#pragma unroll
            for (int nt = 0; nt < 4; nt++) {
                const int col = tile_row0 + 8 * nt + 2 * t;
                if (col >= c1) sv[nt][0] = sv[nt][2] = -INFINITY;
                if (col + 1 >= c1) sv[nt][1] = sv[nt][3] = -INFINITY;
            }
        }
        // online softmax, rows g (x=0) and g+8 (x=1)
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
        for (int nt = 0; nt < 8; nt++) {
            o[nt][0] *= corr[0];
            o[nt][1] *= corr[0];
            o[nt][2] *= corr[1];
            o[nt][3] *= corr[1];
        }
        if (tile_row0 + KV_TILE > c1) {
            // Rows of the tile past the end of the sequence carry weight zero, but 0 * NaN is NaN: whatever the
            // cache holds there (a caller's uninitialised memory) must not reach the product.  Each warp clears
            // those rows of the 64-column box it reads.
            const int first_bad = c1 - tile_row0;
            uint8_t *vbox = stages + (size_t)st * 2 * TILE_BYTES_BF16 + TILE_BYTES_BF16 + warp * 4096;
            for (int idx = first_bad * 8 + lane; idx < KV_TILE * 8; idx += 32)
                *reinterpret_cast<uint4 *>(vbox + idx * 16) = make_uint4(0u, 0u, 0u, 0u);
            __syncwarp();
        }
        // O[:, 64w..64w+63] += P (16x32) * V (32 x 64)
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
            for (int cp = 0; cp < 4; cp++) {
                const int chunk = 2 * cp + (mi >> 1);
                const uint32_t addr = vst + warp * 4096 + prow * 128 + ((chunk ^ (prow & 7)) << 4);
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4_trans(b0, b1, b2, b3, addr);
                mma_bf16_16816(o[2 * cp], pa, b0, b1);
                mma_bf16_16816(o[2 * cp + 1], pa, b2, b3);
            }
        }
    }
    if (failed_at >= 0) {
        // A load did not arrive within the limit.  The loads that are still in flight write into this CTA's shared
        // memory: wait for them (bounded again) before anything else, then stop streaming for good.
        if (tid == 0) atomicOr(p.status, STATUS_TMA_TIMEOUT);
        const int last_issued = min(ntiles - 1, max(BF16_STAGES - 1, failed_at + 1));
        for (int j = failed_at + 1; j <= last_issued; j++)
            mbar_wait_bounded(&full[(pc + (unsigned)j) % BF16_STAGES], ((pc + (unsigned)j) / BF16_STAGES) & 1u, spins);
        abandoned = true;
        __syncthreads();
    }
    if (seg_no == 0) trace_phase(p, 2);

    finish_unit(p, L, o, m_r, l_r, s_w, s_M, s_L, &s_flag, reinterpret_cast<float *>(stages), abandoned);  // the stage ring is idle here: scratch for the merge
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

constexpr size_t BF16_SMEM = 1024 + (size_t)BF16_STAGES * 2 * TILE_BYTES_BF16 +
                             sizeof(float) * (2 * 16 * SX_STRIDE + 256 + MAX_SPLITS * 16 + 32) +
                             sizeof(uint64_t) * BF16_STAGES;

// ---- stand-alone merge of gathered partials (cross-GPU KV split) ----------
__global__ void __launch_bounds__(128)
lse_merge_gate_kernel(int n_parts, int n, int H, const float *o_parts, const float *m_parts,
                      const float *l_parts, size_t stride_o, size_t stride_ml, size_t item_o, size_t item_ml,
                      const float *gate, float *out, const unsigned *flags, unsigned flag_value, unsigned spins,
                      unsigned *status) {
    // one CTA per (item, head); 128 threads x 2 dims.  Part r, item i, head h:
    // o at o_parts + r*stride_o + i*item_o + h*256, m/l at + r*stride_ml + i*item_ml + h.
    const int item = blockIdx.x / H, head = blockIdx.x % H;
    const int tid = threadIdx.x;
    if (flags) {
        // Fused exchange: part r was stored into this buffer by rank r's decode kernel over NVLink; rank r publishes
        // flags[r] = flag_value (a step number that only grows) once all its stores are visible.  The wait is
        // bounded: when it runs out the CTA reports through the status word and leaves.
        __shared__ int s_ok;
        if (tid == 0) s_ok = 1;
        __syncthreads();
        if (tid < n_parts) {
            bool seen = false;
            for (unsigned i = 0; i < spins && !seen; i++) {
                unsigned v;
                asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flags + tid) : "memory");
                seen = (int)(v - flag_value) >= 0;
                if (!seen) __nanosleep(1000);  // about a microsecond per poll: the limit is a time, give or take
            }
            if (!seen) s_ok = 0;
        }
        __syncthreads();
        if (!s_ok) {
            if (tid == 0) atomicOr(status, STATUS_PEER_TIMEOUT);
            return;
        }
    }
    const size_t oo = (size_t)item * item_o + (size_t)head * HEAD_DIM, mo = (size_t)item * item_ml + head;
    float M = -INFINITY;
    for (int r = 0; r < n_parts; r++) M = fmaxf(M, m_parts[r * stride_ml + mo]);
    float Ls = 0.0f;
    float2 acc = make_float2(0.0f, 0.0f);
    for (int r = 0; r < n_parts; r++) {
        const float m = m_parts[r * stride_ml + mo];
        const float w = (m == -INFINITY) ? 0.0f : expf(m - M);
        Ls += w * l_parts[r * stride_ml + mo];
        const float2 o = *reinterpret_cast<const float2 *>(o_parts + r * stride_o + oo + 2 * tid);
        acc.x = fmaf(w, o.x, acc.x);
        acc.y = fmaf(w, o.y, acc.y);
    }
    const float inv = 1.0f / Ls;
    float2 rv = make_float2(acc.x * inv, acc.y * inv);
    const size_t off = (size_t)blockIdx.x * HEAD_DIM + 2 * tid;
    if (gate) {
        const float2 gt = *reinterpret_cast<const float2 *>(gate + off);
        rv.x *= 1.0f / (1.0f + expf(-gt.x));
        rv.y *= 1.0f / (1.0f + expf(-gt.y));
    }
    *reinterpret_cast<float2 *>(out + off) = rv;
}

// ---- RoPE hook ------------------------------------------------------------------
__global__ void rope_kernel(float *q, float *k, int H, int Hkv, int rotary_dim, int pos,
                            const float *inv_freq) {
    const int half = rotary_dim >> 1;
    const int total = (H + Hkv) * half;
    for (int idx = blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += gridDim.x * blockDim.x) {
        const int hh = idx / half, i = idx % half;
        float *x = (hh < H) ? q + (size_t)hh * HEAD_DIM : k + (size_t)(hh - H) * HEAD_DIM;
        float sn, cs;
        sincosf((float)pos * inv_freq[i], &sn, &cs);
        const float x0 = x[i], x1 = x[i + half];
        x[i] = x0 * cs - x1 * sn;
        x[i + half] = x0 * sn + x1 * cs;
    }
}

// ---- cache <-> wire layout ----------------------------------------------------
// wire rows: [row][Hkv][256] fp32; cache: [Hkv][cap_rows][256] of the storage type
__global__ void kv_pack_kernel(const float *src, void *dst, int n_rows, int Hkv, int cap_rows,
                               int kv_bf16, int pos0, int rank, int world, int block) {
    // wire row i holds whole-sequence position pos0 + i; a context of a KV split
    // keeps only the positions of its own blocks
    const size_t total = (size_t)n_rows * Hkv * HEAD_DIM;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        const int d = (int)(idx % HEAD_DIM);
        const int hh = (int)((idx / HEAD_DIM) % Hkv);
        const int pos = pos0 + (int)(idx / ((size_t)HEAD_DIM * Hkv));
        int row = pos;
        if (world > 1) {
            const int blk = pos / block;
            if (blk % world != rank) continue;
            row = (blk / world) * block + pos % block;
        }
        const size_t o = ((size_t)hh * cap_rows + row) * HEAD_DIM + d;
        if (kv_bf16) reinterpret_cast<__nv_bfloat16 *>(dst)[o] = __float2bfloat16_rn(src[idx]);
        else reinterpret_cast<float *>(dst)[o] = src[idx];
    }
}
__global__ void kv_unpack_kernel(const void *src, float *dst, int n_rows, int Hkv, int cap_rows,
                                 int kv_bf16) {
    const size_t total = (size_t)n_rows * Hkv * HEAD_DIM;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        const int d = (int)(idx % HEAD_DIM);
        const int hh = (int)((idx / HEAD_DIM) % Hkv);
        const size_t row = idx / ((size_t)HEAD_DIM * Hkv);
        const size_t o = ((size_t)hh * cap_rows + row) * HEAD_DIM + d;
        dst[idx] = kv_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(src)[o])
                           : reinterpret_cast<const float *>(src)[o];
    }
}

}  // namespace

cudaError_t gqa_decode_configure() {
    return cudaFuncSetAttribute(gqa_decode_bf16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                (int)BF16_SMEM);
}

cudaError_t launch_gqa_decode_bf16(const CUtensorMap &kmap, const CUtensorMap &vmap,
                                   const GqaParams &p, cudaStream_t stream) {
    if (p.total_ctas <= 0) return cudaSuccess;
    if (p.coop_merge) {
        // every CTA resident at once: CTAs that share a unit may wait for one another (merge_unit_slices)
        void *args[] = {const_cast<CUtensorMap *>(&kmap), const_cast<CUtensorMap *>(&vmap), const_cast<GqaParams *>(&p)};
        return cudaLaunchCooperativeKernel(reinterpret_cast<void *>(gqa_decode_bf16_kernel), dim3(p.total_ctas), dim3(128), args, BF16_SMEM, stream);
    }
    gqa_decode_bf16_kernel<<<p.total_ctas, 128, BF16_SMEM, stream>>>(kmap, vmap, p);
    return cudaGetLastError();
}

int gqa_decode_bf16_coop_capacity() {
    int dev = 0, sms = 0, per_sm = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, gqa_decode_bf16_kernel, 128, BF16_SMEM) != cudaSuccess)
        return 0;
    int coop = 0;
    cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev);
    return coop ? sms * per_sm : 0;
}

cudaError_t launch_lse_merge_gate(int n_parts, int n, int H, const float *o_parts,
                                  const float *m_parts, const float *l_parts, size_t part_stride,
                                  const float *gate, float *out, cudaStream_t stream, size_t o_item_stride,
                                  size_t ml_item_stride, const unsigned *flags, unsigned flag_value, unsigned spins,
                                  unsigned *status) {
    if (n <= 0) return cudaSuccess;
    if (flags && n_parts > 128) return cudaErrorInvalidValue;
    const size_t io = o_item_stride ? o_item_stride : (size_t)H * HEAD_DIM;
    const size_t iml = ml_item_stride ? ml_item_stride : (size_t)H;
    const size_t so = part_stride ? part_stride : (size_t)n * io;
    const size_t sml = part_stride ? part_stride : (size_t)n * iml;
    lse_merge_gate_kernel<<<n * H, 128, 0, stream>>>(n_parts, n, H, o_parts, m_parts, l_parts, so, sml, io, iml, gate,
                                                     out, flags, flag_value, spins ? spins : (1u << 21), status);
    return cudaGetLastError();
}

// ---- gather of the step's query rows over the links (cross-GPU KV split) ----------
// Every rank holds, in its own copy of the step's row table, the rows of the items it finishes (they came from its
// host).  The kernel stores them into the same slot of every peer's table with plain peer stores, then the CTA that
// finishes last publishes flags[my_rank] = flag_value on every peer and waits, bounded, until every peer's flag has
// reached flag_value in this rank's own array: when the kernel ends, the whole table is in this GPU's memory and the
// decode kernel queued behind it reads it like any other device buffer.  The waits are on other GPUs' kernels only.
static __global__ void __launch_bounds__(256)
q_rows_gather_kernel(float *const *peer_rows, unsigned *const *peer_flags, const unsigned *my_flags,
                     unsigned *done_counter, size_t own_floats, int my_rank, int world, unsigned flag_value,
                     unsigned spins, unsigned *status) {
    const int tid = threadIdx.x;
    const size_t n4 = own_floats / 4;
    const float4 *src = reinterpret_cast<const float4 *>(peer_rows[my_rank] + (size_t)my_rank * own_floats);
    for (size_t i = (size_t)blockIdx.x * blockDim.x + tid; i < n4; i += (size_t)gridDim.x * blockDim.x) {
        const float4 v = src[i];
        for (int d = 1; d < world; d++) {
            const int r = (my_rank + d) % world;  // every rank starts at another peer
            reinterpret_cast<float4 *>(peer_rows[r] + (size_t)my_rank * own_floats)[i] = v;
        }
    }
    __threadfence_system();
    __syncthreads();
    __shared__ int s_last;
    if (tid == 0) {
        const unsigned prev = atomicAdd(done_counter, 1u);
        s_last = (prev == gridDim.x - 1);
        if (s_last) *done_counter = 0u;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence_system();
    if (tid < world && tid != my_rank) {
        unsigned *dst = peer_flags[tid] + my_rank;
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(dst), "r"(flag_value) : "memory");
        bool seen = false;
        for (unsigned i = 0; i < spins && !seen; i++) {
            unsigned v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(my_flags + tid) : "memory");
            seen = (int)(v - flag_value) >= 0;
            if (!seen) __nanosleep(500);
        }
        if (!seen) atomicOr(status, STATUS_PEER_TIMEOUT);
    }
}

cudaError_t launch_q_rows_gather(float *const *peer_rows, unsigned *const *peer_flags, const unsigned *my_flags,
                                 unsigned *done_counter, size_t own_floats, int my_rank, int world,
                                 unsigned flag_value, unsigned spins, unsigned *status, cudaStream_t stream) {
    if (world < 2 || world > 128 || own_floats == 0 || own_floats % 4) return cudaErrorInvalidValue;
    const size_t n4 = own_floats / 4;
    int grid = (int)((n4 + 511) / 512);  // two 16-byte chunks per thread and peer
    if (grid > 64) grid = 64;
    q_rows_gather_kernel<<<grid, 256, 0, stream>>>(peer_rows, peer_flags, my_flags, done_counter, own_floats, my_rank,
                                                   world, flag_value, spins ? spins : (1u << 22), status);
    return cudaGetLastError();
}

// out *= sigmoid(gate), four floats per thread: the gate applied after the fact with the fused epilogue's arithmetic
static __global__ void sigmoid_gate_kernel(float *out, const float *gate, size_t n4) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n4) return;
    float4 o = reinterpret_cast<float4 *>(out)[i];
    const float4 g = reinterpret_cast<const float4 *>(gate)[i];
    o.x *= 1.0f / (1.0f + expf(-g.x));
    o.y *= 1.0f / (1.0f + expf(-g.y));
    o.z *= 1.0f / (1.0f + expf(-g.z));
    o.w *= 1.0f / (1.0f + expf(-g.w));
    reinterpret_cast<float4 *>(out)[i] = o;
}

cudaError_t launch_sigmoid_gate(float *out, const float *gate, size_t n, cudaStream_t stream) {
    const size_t n4 = n / 4;
    if (n4 == 0) return cudaSuccess;
    sigmoid_gate_kernel<<<(unsigned)((n4 + 255) / 256), 256, 0, stream>>>(out, gate, n4);
    return cudaGetLastError();
}

cudaError_t launch_rope(float *q, float *k, int H, int Hkv, int rotary_dim, int pos,
                        const float *inv_freq, cudaStream_t stream) {
    const int total = (H + Hkv) * (rotary_dim / 2);
    if (total <= 0) return cudaSuccess;
    rope_kernel<<<(total + 127) / 128, 128, 0, stream>>>(q, k, H, Hkv, rotary_dim, pos, inv_freq);
    return cudaGetLastError();
}

cudaError_t launch_kv_pack(const float *src_rows, void *dst_cache, int n_rows, int Hkv,
                           int cap_rows, int kv_bf16, int pos0, int rank, int world, int block,
                           cudaStream_t stream) {
    if (n_rows <= 0) return cudaSuccess;
    const size_t total = (size_t)n_rows * Hkv * HEAD_DIM;
    const int blocks = (int)((total + 255) / 256 > 4096 ? 4096 : (total + 255) / 256);
    kv_pack_kernel<<<blocks, 256, 0, stream>>>(src_rows, dst_cache, n_rows, Hkv, cap_rows, kv_bf16, pos0, rank,
                                               world, block);
    return cudaGetLastError();
}
cudaError_t launch_kv_unpack(const void *src_cache, float *dst_rows, int n_rows, int Hkv,
                             int cap_rows, int kv_bf16, cudaStream_t stream) {
    if (n_rows <= 0) return cudaSuccess;
    const size_t total = (size_t)n_rows * Hkv * HEAD_DIM;
    const int blocks = (int)((total + 255) / 256 > 4096 ? 4096 : (total + 255) / 256);
    kv_unpack_kernel<<<blocks, 256, 0, stream>>>(src_cache, dst_rows, n_rows, Hkv, cap_rows, kv_bf16);
    return cudaGetLastError();
}

}  // namespace mfc
