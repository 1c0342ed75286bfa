// Pieces shared by the bf16 and fp32 split-K decode kernels: CTA -> work unit
// lookup, RoPE of one float2, and the epilogue (finish in place, or park the
// partial and let the last CTA of the unit merge by log-sum-exp and gate).
#pragma once
#include <math.h>

#include "common.cuh"
#include "kernels.h"

namespace mfc {

constexpr float LOG2E = 1.4426950408889634f;

// x[d], x[d+1] of one head row after the optional per-head RMSNorm (x * inv_rms *
// w[d], crates/moeflux/src/riir/rms_norm.rs:140-152) and partial RoPE (MLX
// half-split pairing, crates/moeflux/src/riir/rope.rs:93-128); d even, tables
// indexed by pair index.  nw == nullptr: no norm.
__device__ __forceinline__ float2 load_norm2(const float *row, int d, float inv_rms, const uint16_t *nw) {
    float2 x = *reinterpret_cast<const float2 *>(row + d);
    if (nw) {
        const uint32_t wb = *reinterpret_cast<const uint32_t *>(nw + d);
        x.x = x.x * inv_rms * bf16_bits_to_f32((uint16_t)(wb & 0xffffu));
        x.y = x.y * inv_rms * bf16_bits_to_f32((uint16_t)(wb >> 16));
    }
    return x;
}
__device__ __forceinline__ float2 load_rot2(const float *row, int d, int rotary_dim, int half,
                                            const float *s_cos, const float *s_sin, float inv_rms = 1.0f,
                                            const uint16_t *nw = nullptr) {
    float2 x = load_norm2(row, d, inv_rms, nw);
    if (d < rotary_dim) {
        if (d < half) {
            const float2 pr = load_norm2(row, d + half, inv_rms, nw);
            x = make_float2(x.x * s_cos[d] - pr.x * s_sin[d], x.y * s_cos[d + 1] - pr.y * s_sin[d + 1]);
        } else {
            const int i = d - half;
            const float2 pr = load_norm2(row, i, inv_rms, nw);
            x = make_float2(pr.x * s_sin[i] + x.x * s_cos[i], pr.y * s_sin[i + 1] + x.y * s_cos[i + 1]);
        }
    }
    return x;
}

// Copies the query head rows of a unit (q_row_stride floats apart in device memory) into shared memory with
// 16-byte loads that are all in flight together; the fragment builders then read shared memory.  (Building the
// fragments straight from device memory serialised ~64 dependent-latency loads per thread: 30 us per segment.)
constexpr int Q_STAGE_STRIDE = HEAD_DIM + 4;  // floats: rows stay 16-byte aligned and spread over the banks
__device__ __forceinline__ void stage_q_rows(const float *qbase, int rows, int q_row_stride, float *s_q) {
#pragma unroll
    for (int k = 0; k < 16 * (HEAD_DIM / 4) / 128; k++) {
        const int i = k * 128 + (int)threadIdx.x;
        const int r = i >> 6, c = (i & 63) * 4;
        float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (r < rows) v = *reinterpret_cast<const float4 *>(qbase + (size_t)r * q_row_stride + c);
        *reinterpret_cast<float4 *>(s_q + r * Q_STAGE_STRIDE + c) = v;
    }
}

// 1/rms of the 16 (or fewer) query head rows of a unit, by 4 warps: s_inv[row].
// qbase points at row 0; rows are q_row_stride floats apart.  Contains a __syncthreads.
__device__ __forceinline__ void head_inv_rms(const float *qbase, int rows, int row_stride, float eps, float *s_inv) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int r = warp; r < 16; r += 4) {
        float ss = 0.0f;
        if (r < rows) {
            const float4 a = *reinterpret_cast<const float4 *>(qbase + (size_t)r * row_stride + lane * 8);
            const float4 b = *reinterpret_cast<const float4 *>(qbase + (size_t)r * row_stride + lane * 8 + 4);
            ss = a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w + b.x * b.x + b.y * b.y + b.z * b.z + b.w * b.w;
        }
        ss = warp_sum(ss);
        if (lane == 0) s_inv[r] = 1.0f / sqrtf(ss / (float)HEAD_DIM + eps);
    }
    __syncthreads();
}

// A segment of work: the part of one (item, kv head) unit that falls into this
// CTA's range of the launch-wide tile sequence.
struct Located {
    GqaItem it;
    int item_idx;
    int kvh;
    int t0;        // first tile of the segment, within the unit
    int seg;       // tiles in the segment
    int n_parts;   // CTAs that share the unit (1: this CTA finishes it alone)
    int part_idx;  // this CTA's rank among them
    int slot0;     // scratch slot of the unit's first partial
    bool bad;      // the item failed its range checks: the unit is skipped (its tickets are still taken)
    bool last_goes_on;  // the unit's last sharer continues with another unit after it (it takes no part in a
                        //   cooperative merge: it must not wait in the middle of its run)
};

constexpr int LOCATE_SMEM_ITEMS = 512;
// Stages the items' first-tile indices in shared memory (one round of global
// loads instead of a dependent chain per lookup).  Contains a __syncthreads.
__device__ __forceinline__ const GqaItem *item_list(const GqaParams &p) { return p.items ? p.items : p.inline_items; }
__device__ __forceinline__ void stage_tile_begins(const GqaParams &p, int *s_begin) {
    const GqaItem *items = item_list(p);
    if (p.n_items <= LOCATE_SMEM_ITEMS)
        for (int i = threadIdx.x; i < p.n_items; i += blockDim.x) s_begin[i] = items[i].tile_begin;
    __syncthreads();
}
// Segment that starts at tile `gt` of the launch-wide sequence and ends at the
// unit's end or at `gt_end`, whichever comes first.
template <int TILE_ROWS>
__device__ __forceinline__ Located locate_tile(const GqaParams &p, int gt, int gt_end, const int *s_begin) {
    int lo = 0, hi = p.n_items - 1;
    const bool in_smem = p.n_items <= LOCATE_SMEM_ITEMS;
    const GqaItem *items = item_list(p);
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        const int tb = in_smem ? s_begin[mid] : items[mid].tile_begin;
        if (tb <= gt) lo = mid;
        else hi = mid - 1;
    }
    Located L;
    L.it = items[lo];
    L.item_idx = lo;
    // tiles a kv head of the item takes in the launch-wide sequence: its own, or (pad0 > 0: a plan that keeps units
    // and CTA runs aligned) that number rounded up to whole runs; the tiles past the item's rows are empty
    const int nt = L.it.pad0 > 0 ? L.it.pad0 : (L.it.local_len > 0 ? (L.it.local_len + TILE_ROWS - 1) / TILE_ROWS : 1);
    const int local = gt - L.it.tile_begin;
    L.kvh = local / nt;
    L.t0 = local - L.kvh * nt;
    L.seg = min(nt - L.t0, gt_end - gt);
    const int tb_u = L.it.tile_begin + L.kvh * nt;
    const int first_cta = tb_u / p.tiles_per_cta, last_cta = (tb_u + nt - 1) / p.tiles_per_cta;
    L.n_parts = last_cta - first_cta + 1;
    L.part_idx = (int)blockIdx.x - first_cta;
    L.last_goes_on = tb_u + nt < min((last_cta + 1) * p.tiles_per_cta, p.total_tiles);
    // (unit index + CTA index) grows strictly along the tile sequence: a unique slot per pair
    L.slot0 = lo * p.Hkv + L.kvh + first_cta;
    // what the kernel indexes memory with must lie inside the caches and the input arrays
    L.bad = L.it.kv_slot < 0 || L.it.kv_slot >= p.n_kv_slots || L.it.local_len < 0 || L.it.local_len > p.cap_rows ||
            L.it.append_row >= L.it.local_len || L.it.in_idx < 0 || L.it.in_idx >= p.n_items ||
            L.n_parts > MAX_UNIT_PARTS;
    return L;
}

// Optional per-CTA phase trace (thread 0 only): word w of this CTA's record.
__device__ __forceinline__ void trace_phase(const GqaParams &p, int w) {
    if (p.phase_trace && threadIdx.x == 0 && w < PHASE_TRACE_WORDS)
        p.phase_trace[(size_t)blockIdx.x * PHASE_TRACE_WORDS + w] = global_timer_ns();
}

// Where a merged un-normalised partial of an item goes in partial mode: the caller's buffers, or (fused exchange of
// the KV-sequence split) the receive buffer of the rank that finishes the item, through its peer-mapped pointer.
struct PartialDst {
    float *o, *m, *l;  // o: [H][256], m / l: [H]
};
__device__ __forceinline__ PartialDst partial_dst(const GqaParams &p, int in_idx) {
    PartialDst d;
    if (p.peer_recv) {
        const int dest = in_idx / p.items_per_dest, j = in_idx - dest * p.items_per_dest;
        float *blk = p.peer_recv[dest] + ((size_t)p.my_rank * p.items_per_dest + j) * p.po_item_stride;
        d.o = blk;
        d.m = blk + (size_t)p.H * HEAD_DIM;
        d.l = d.m + p.H;
    } else {
        d.o = p.po + (size_t)in_idx * p.po_item_stride;
        d.m = p.pm + (size_t)in_idx * p.pml_item_stride;
        d.l = p.pl + (size_t)in_idx * p.pml_item_stride;
    }
    return d;
}

// Merge of n_src partials of one (item, kv head) unit by log-sum-exp; partial c sits in scratch slot
// src_slot0 + c * slot_stride.  to_slot >= 0: first level of a two-level merge, the un-normalised result (o, M, L)
// goes to that scratch slot (it may be one of the sources: every thread reads its elements of all sources before it
// writes them).  to_slot < 0: the unit is finished here, as the gated output or, in partial mode, as the
// un-normalised partial of the item.  Executed by 128 threads; s_w: n_src * 16 floats, s_tmp: n_src * 16 floats.
__device__ __forceinline__ void merge_unit(const GqaParams &p, const Located &L, size_t src_slot0, int slot_stride,
                                           int n_src, long long to_slot, float *s_w, float *s_M, float *s_L,
                                           float *s_tmp) {
    const int tid = threadIdx.x;
    const int group = p.group;
    // m and l of every partial come in with all loads in flight; the reductions then run out of shared memory
    for (int idx = tid; idx < n_src * 16; idx += 128) {
        const size_t so = (src_slot0 + (size_t)(idx >> 4) * slot_stride) * 16 + (idx & 15);
        s_w[idx] = p.sc_m[so];
        s_tmp[idx] = p.sc_l[so];
    }
    __syncthreads();
    if (tid < 16) {
        float M = -INFINITY;
        for (int c = 0; c < n_src; c++) M = fmaxf(M, s_w[c * 16 + tid]);
        s_M[tid] = M;
    }
    __syncthreads();
    for (int idx = tid; idx < n_src * 16; idx += 128) {
        const float m = s_w[idx];
        s_w[idx] = (m == -INFINITY) ? 0.0f : expf(m - s_M[idx & 15]);
    }
    __syncthreads();
    if (tid < 16) {
        float Ls = 0.0f;
        for (int c = 0; c < n_src; c++) Ls += s_w[c * 16 + tid] * s_tmp[c * 16 + tid];
        s_L[tid] = Ls;
    }
    __syncthreads();
    const size_t head0 = (size_t)L.it.in_idx * p.H + (size_t)L.kvh * group;
    const bool final_out = to_slot < 0 && !p.partial_mode;
    PartialDst pd;
    if (to_slot < 0 && p.partial_mode) pd = partial_dst(p, L.it.in_idx);
    // Four heads x eight partials per round, every load of a round in flight together: the merging CTA is the last of
    // its group to finish, often at the very end of the launch, so this latency is on the launch's critical path.
    for (int hr0 = 0; hr0 < group; hr0 += 4) {
        float2 acc[4], gt[4];
#pragma unroll
        for (int u = 0; u < 4; u++) {
            acc[u] = make_float2(0.0f, 0.0f);
            gt[u] = make_float2(0.0f, 0.0f);
            if (final_out && p.gate && hr0 + u < group)
                gt[u] = *reinterpret_cast<const float2 *>(p.gate + (head0 + hr0 + u) * (size_t)p.gate_row_stride + 2 * tid);
        }
        for (int c0 = 0; c0 < n_src; c0 += MERGE_GROUP) {
            float2 o[MERGE_GROUP][4];
#pragma unroll
            for (int k = 0; k < MERGE_GROUP; k++)
#pragma unroll
                for (int u = 0; u < 4; u++)
                    o[k][u] = (c0 + k < n_src && hr0 + u < group)
                                  ? *reinterpret_cast<const float2 *>(
                                        p.sc_o + ((src_slot0 + (size_t)(c0 + k) * slot_stride) * 16 + hr0 + u) * HEAD_DIM + 2 * tid)
                                  : make_float2(0.0f, 0.0f);
#pragma unroll
            for (int k = 0; k < MERGE_GROUP; k++) {  // partials are added in index order
                if (c0 + k >= n_src) break;
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    const float w = s_w[(c0 + k) * 16 + ((hr0 + u) & 15)];
                    acc[u].x = fmaf(w, o[k][u].x, acc[u].x);
                    acc[u].y = fmaf(w, o[k][u].y, acc[u].y);
                }
            }
        }
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const int hr = hr0 + u;
            if (hr >= group) break;
            if (to_slot >= 0) {
                *reinterpret_cast<float2 *>(p.sc_o + ((size_t)to_slot * 16 + hr) * HEAD_DIM + 2 * tid) = acc[u];
            } else if (p.partial_mode) {
                const int hl = L.kvh * group + hr;  // head within the item
                *reinterpret_cast<float2 *>(pd.o + (size_t)hl * HEAD_DIM + 2 * tid) = acc[u];
                if (tid == 0) {
                    pd.m[hl] = s_M[hr];
                    pd.l[hl] = s_L[hr];
                }
            } else {
                const size_t off = (head0 + hr) * HEAD_DIM + 2 * tid;
                const float inv = 1.0f / s_L[hr];
                float2 r = make_float2(acc[u].x * inv, acc[u].y * inv);
                if (p.gate) {
                    r.x *= 1.0f / (1.0f + expf(-gt[u].x));
                    r.y *= 1.0f / (1.0f + expf(-gt[u].y));
                }
                *reinterpret_cast<float2 *>(p.out + off) = r;
            }
        }
    }
    if (to_slot >= 0 && tid < 16) {  // every thread is past its reads of the sources' m and l (staged above)
        p.sc_m[(size_t)to_slot * 16 + tid] = s_M[tid];
        p.sc_l[(size_t)to_slot * 16 + tid] = s_L[tid];
    }
}

// Cooperative merge of a unit shared by many CTAs (a lone long sequence: up to MAX_UNIT_PARTS partials per unit).
// Launched cooperatively, so every CTA of the grid is resident and a CTA may wait for the others.  Each sharer
// parks its partial and takes the unit's ticket; the sharers whose segment ends their run (all but a last sharer
// that goes on to another unit) wait until all tickets are taken and then each merges a slice of the output: slice
// unit = (head, 64 output dims), dealt round-robin over the merging CTAs.  Per slice unit the 128 threads are 8 rows
// of partials x 16 lanes of four dims; the loads of all partials of the slice are in flight together with the loads
// of their (m, l), so the whole merge is one round trip to L2 instead of one per group of partials.
//   s_w: 2 * MAX_UNIT_PARTS floats (m, then l), s_tmp: 8 * 64 floats.
static_assert(MAX_SPLITS * 16 >= 2 * MAX_UNIT_PARTS, "the merge weight area of the kernels must hold m and l of every partial");
__device__ __forceinline__ void merge_unit_slices(const GqaParams &p, const Located &L, size_t slot0, int n_parts,
                                                  int n_mergers, int my_idx, float *s_w, float *s_tmp) {
    const int tid = threadIdx.x, lane = tid & 31;
    const int l16 = tid & 15, prow = tid >> 4;
    const int group = p.group;
    const size_t head0 = (size_t)L.it.in_idx * p.H + (size_t)L.kvh * group;
    float *s_m = s_w, *s_l = s_w + MAX_UNIT_PARTS;
    PartialDst pd;
    if (p.partial_mode) pd = partial_dst(p, L.it.in_idx);
    constexpr int ROWS_PER_THREAD = 20;  // partial rows a thread holds per batch (8 rows of threads: 160 partials, so
                                         // that one wave of CTAs over two units is a single batch)
    for (int su = my_idx; su < group * 4; su += n_mergers) {
        const int hr = su >> 2, j = su & 3;
        float4 o4[ROWS_PER_THREAD];
#pragma unroll
        for (int i = 0; i < ROWS_PER_THREAD; i++) {
            const int c = prow + 8 * i;
            o4[i] = c < n_parts ? *reinterpret_cast<const float4 *>(p.sc_o + ((slot0 + c) * 16 + hr) * HEAD_DIM + 64 * j + 4 * l16)
                                : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        }
        for (int c = tid; c < n_parts; c += 128) {
            s_m[c] = p.sc_m[(slot0 + c) * 16 + hr];
            s_l[c] = p.sc_l[(slot0 + c) * 16 + hr];
        }
        float2 gt2 = make_float2(0.0f, 0.0f);  // gate logits of the dims this thread finishes (threads 0..31: 2 each)
        if (!p.partial_mode && p.gate && tid < 32)
            gt2 = *reinterpret_cast<const float2 *>(p.gate + (head0 + hr) * (size_t)p.gate_row_stride + 64 * j + 2 * tid);
        __syncthreads();
        // every warp forms M and L for the head (the same values in all four)
        float M = -INFINITY;
        for (int c = lane; c < n_parts; c += 32) M = fmaxf(M, s_m[c]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
        float Ls = 0.0f;
        for (int c = lane; c < n_parts; c += 32) Ls += (s_m[c] == -INFINITY ? 0.0f : expf(s_m[c] - M)) * s_l[c];
        Ls = warp_sum(Ls);
        float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        for (int b0 = 0; b0 < n_parts; b0 += 8 * ROWS_PER_THREAD) {
            if (b0 > 0) {  // further batches of 128 partials (units shared by more than 128 CTAs)
#pragma unroll
                for (int i = 0; i < ROWS_PER_THREAD; i++) {
                    const int c = b0 + prow + 8 * i;
                    o4[i] = c < n_parts ? *reinterpret_cast<const float4 *>(p.sc_o + ((slot0 + c) * 16 + hr) * HEAD_DIM + 64 * j + 4 * l16)
                                        : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                }
            }
#pragma unroll
            for (int i = 0; i < ROWS_PER_THREAD; i++) {
                const int c = b0 + prow + 8 * i;
                if (c >= n_parts) break;
                const float w = s_m[c] == -INFINITY ? 0.0f : expf(s_m[c] - M);
                acc.x = fmaf(w, o4[i].x, acc.x);
                acc.y = fmaf(w, o4[i].y, acc.y);
                acc.z = fmaf(w, o4[i].z, acc.z);
                acc.w = fmaf(w, o4[i].w, acc.w);
            }
        }
        *reinterpret_cast<float4 *>(s_tmp + prow * 64 + 4 * l16) = acc;
        __syncthreads();
        if (tid < 32) {  // two dims per thread: sum over the 8 rows of threads, in row order
            float2 r = make_float2(0.0f, 0.0f);
#pragma unroll
            for (int k = 0; k < 8; k++) {
                const float2 v = *reinterpret_cast<const float2 *>(s_tmp + k * 64 + 2 * tid);
                r.x += v.x;
                r.y += v.y;
            }
            if (p.partial_mode) {
                const int hl = L.kvh * group + hr;
                *reinterpret_cast<float2 *>(pd.o + (size_t)hl * HEAD_DIM + 64 * j + 2 * tid) = r;
                if (tid == 0 && j == 0) {
                    pd.m[hl] = M;
                    pd.l[hl] = Ls;
                }
            } else {
                const float inv = 1.0f / Ls;
                r.x *= inv;
                r.y *= inv;
                if (p.gate) {
                    r.x *= 1.0f / (1.0f + expf(-gt2.x));
                    r.y *= 1.0f / (1.0f + expf(-gt2.y));
                }
                *reinterpret_cast<float2 *>(p.out + (head0 + hr) * HEAD_DIM + 64 * j + 2 * tid) = r;
            }
        }
        __syncthreads();  // s_m / s_l / s_tmp are reused by the next slice unit
    }
}

// Epilogue shared by both kernels.  The warp layout of the accumulators is:
// o[nt][2x + e] = row (g + 8x), dim 64*warp + 8*nt + 2t + e;  m_r / l_r per row
// (l_r still split over the four lanes of a row).
__device__ __forceinline__ void finish_unit(const GqaParams &p, const Located &L, float (&o)[8][4],
                                            float (&m_r)[2], float (&l_r)[2], float *s_w,
                                            float *s_M, float *s_L, int *s_flag_p, float *s_tmp, bool abandoned) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const GqaItem &it = L.it;
    const int group = p.group;
#pragma unroll
    for (int x = 0; x < 2; x++) {
        l_r[x] += __shfl_xor_sync(0xffffffffu, l_r[x], 1);
        l_r[x] += __shfl_xor_sync(0xffffffffu, l_r[x], 2);
    }

    const size_t head0 = (size_t)it.in_idx * p.H + (size_t)L.kvh * group;
    if (L.n_parts == 1) {
        if (abandoned) return;
        // the unit was not split: finish in place
        PartialDst pd;
        if (p.partial_mode) pd = partial_dst(p, it.in_idx);
#pragma unroll
        for (int x = 0; x < 2; x++) {
            const int row = g + 8 * x;
            if (row >= group) continue;
            const float m_nat = m_r[x] * p.scale;
            if (p.partial_mode) {
                if (warp == 0 && t == 0) {
                    pd.m[L.kvh * group + row] = m_nat;
                    pd.l[L.kvh * group + row] = l_r[x];
                }
            }
            const float inv = p.partial_mode ? 1.0f : 1.0f / l_r[x];
#pragma unroll
            for (int nt = 0; nt < 8; nt++) {
                const size_t off = (head0 + row) * HEAD_DIM + 64 * warp + 8 * nt + 2 * t;
                float2 rv = make_float2(o[nt][2 * x] * inv, o[nt][2 * x + 1] * inv);
                if (p.partial_mode) {
                    *reinterpret_cast<float2 *>(pd.o + (size_t)(L.kvh * group + row) * HEAD_DIM + 64 * warp + 8 * nt + 2 * t) = rv;
                } else {
                    if (p.gate) {
                        const float2 gt = *reinterpret_cast<const float2 *>(
                            p.gate + (head0 + row) * (size_t)p.gate_row_stride + 64 * warp + 8 * nt + 2 * t);
                        rv.x *= 1.0f / (1.0f + expf(-gt.x));
                        rv.y *= 1.0f / (1.0f + expf(-gt.y));
                    }
                    *reinterpret_cast<float2 *>(p.out + off) = rv;
                }
            }
        }
        return;
    }

    // The unit is shared: park the partial; the last CTA to arrive merges.  Up to MERGE_GROUP partials are merged in
    // one level.  Beyond that, in a cooperative launch, the sharers merge together (merge_unit_slices); in an
    // ordinary launch the partials form groups of MERGE_GROUP consecutive ones: the last arriver of a group
    // merges it into the group's first slot (many groups merge side by side on different SMs), then arrives at the
    // unit's ticket, and the last group to arrive merges the group results.  In an ordinary launch nothing ever
    // spins: a CTA that is not last simply leaves.  A CTA that gave up on its loads still takes its tickets, so that the counters return to
    // zero for the next launch; what it would have merged is not merged (the status word says so to the host).
    const size_t slot0 = (size_t)L.slot0;  // first slot of the unit
    const size_t slot = slot0 + L.part_idx;
    if (!abandoned) {
#pragma unroll
        for (int x = 0; x < 2; x++) {
            const int row = g + 8 * x;
            if (warp == 0 && t == 0) {
                p.sc_m[slot * 16 + row] = m_r[x] * p.scale;
                p.sc_l[slot * 16 + row] = l_r[x];
            }
#pragma unroll
            for (int nt = 0; nt < 8; nt++) {
                *reinterpret_cast<float2 *>(p.sc_o + (slot * 16 + row) * HEAD_DIM + 64 * warp + 8 * nt + 2 * t) =
                    make_float2(o[nt][2 * x], o[nt][2 * x + 1]);
            }
        }
    }
    unsigned *unit_ticket = p.tickets + (size_t)L.item_idx * p.Hkv + L.kvh;
    if (p.coop_merge && L.n_parts > MERGE_GROUP) {
        // cooperative launch: the sharers that are at the end of their run merge the unit together (see above)
        __threadfence();
        __syncthreads();
        if (tid == 0) atomicAdd(unit_ticket, 1u);
        const bool merger = !(L.last_goes_on && L.part_idx == L.n_parts - 1);
        if (!merger) return;
        const int n_mergers = L.n_parts - (L.last_goes_on ? 1 : 0);
        if (tid == 0) {
            bool seen = false;
            const unsigned limit = p.wait_spins ? p.wait_spins : (1u << 22);
            for (unsigned i = 0; i < limit && !seen; i++) {
                unsigned v;
                asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(unit_ticket) : "memory");
                seen = v >= (unsigned)L.n_parts;
                if (!seen) __nanosleep(200);
            }
            *s_flag_p = seen;
            if (!seen) atomicOr(p.status, STATUS_MERGE_TIMEOUT);
        }
        __syncthreads();
        if (!*s_flag_p) return;  // the host clears the counters when it reads the status
        __threadfence();
        if (!abandoned) merge_unit_slices(p, L, slot0, L.n_parts, n_mergers, L.part_idx, s_w, s_tmp);
        __syncthreads();
        if (tid == 0) {  // the last merger to finish puts both counters back to zero for the next launch
            unsigned *done = p.group_tickets + slot0;
            const unsigned prev = atomicAdd(done, 1u);
            if (prev == (unsigned)(n_mergers - 1)) {
                *done = 0u;
                *unit_ticket = 0u;
            }
        }
        return;
    }
    const bool two_level = L.n_parts > MERGE_GROUP;
    const int gi = L.part_idx / MERGE_GROUP;
    const int n_groups = (L.n_parts + MERGE_GROUP - 1) / MERGE_GROUP;
    __threadfence();
    __syncthreads();
    if (two_level) {
        const int gsize = min(MERGE_GROUP, L.n_parts - gi * MERGE_GROUP);
        const size_t gslot = slot0 + (size_t)gi * MERGE_GROUP;
        if (tid == 0) {
            unsigned *tk = p.group_tickets + gslot;
            const unsigned prev = atomicAdd(tk, 1u);
            *s_flag_p = (prev == (unsigned)(gsize - 1));
            if (*s_flag_p) *tk = 0u;  // ready for the next launch
        }
        __syncthreads();
        if (!*s_flag_p) return;
        __threadfence();
        if (!abandoned) merge_unit(p, L, gslot, 1, gsize, (long long)gslot, s_w, s_M, s_L, s_tmp);
        __threadfence();
        __syncthreads();
    }
    if (tid == 0) {
        const unsigned prev = atomicAdd(unit_ticket, 1u);
        *s_flag_p = (prev == (unsigned)((two_level ? n_groups : L.n_parts) - 1));
        if (*s_flag_p) *unit_ticket = 0u;  // ready for the next launch
    }
    __syncthreads();
    if (!*s_flag_p || abandoned) return;
    __threadfence();
    if (two_level) merge_unit(p, L, slot0, MERGE_GROUP, n_groups, -1, s_w, s_M, s_L, s_tmp);
    else merge_unit(p, L, slot0, 1, L.n_parts, -1, s_w, s_M, s_L, s_tmp);
}

// End of a CTA's work in a launch with the fused exchange: once every CTA has made its stores to the peers'
// receive buffers visible system-wide, the last one publishes this rank's flag in every peer's flag array.
__device__ __forceinline__ void publish_exchange_flags(const GqaParams &p, int *s_flag_p) {
    if (!p.peer_flags) return;
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned prev = atomicAdd(p.done_counter, 1u);
        *s_flag_p = (prev == gridDim.x - 1);
        if (*s_flag_p) *p.done_counter = 0u;
    }
    __syncthreads();
    if (!*s_flag_p) return;
    __threadfence_system();
    if ((int)threadIdx.x < p.world) {
        unsigned *dst = p.peer_flags[threadIdx.x] + p.my_rank;
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(dst), "r"(p.flag_value) : "memory");
    }
}

}  // namespace mfc
