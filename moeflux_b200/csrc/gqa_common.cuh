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
};

constexpr int LOCATE_SMEM_ITEMS = 512;
// Stages the items' first-tile indices in shared memory (one round of global
// loads instead of a dependent chain per lookup).  Contains a __syncthreads.
__device__ __forceinline__ void stage_tile_begins(const GqaParams &p, int *s_begin) {
    if (p.n_items <= LOCATE_SMEM_ITEMS)
        for (int i = threadIdx.x; i < p.n_items; i += blockDim.x) s_begin[i] = p.items[i].tile_begin;
    __syncthreads();
}
// Segment that starts at tile `gt` of the launch-wide sequence and ends at the
// unit's end or at `gt_end`, whichever comes first.
template <int TILE_ROWS>
__device__ __forceinline__ Located locate_tile(const GqaParams &p, int gt, int gt_end, const int *s_begin) {
    int lo = 0, hi = p.n_items - 1;
    const bool in_smem = p.n_items <= LOCATE_SMEM_ITEMS;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        const int tb = in_smem ? s_begin[mid] : p.items[mid].tile_begin;
        if (tb <= gt) lo = mid;
        else hi = mid - 1;
    }
    Located L;
    L.it = p.items[lo];
    L.item_idx = lo;
    const int nt = L.it.local_len > 0 ? (L.it.local_len + TILE_ROWS - 1) / TILE_ROWS : 1;
    const int local = gt - L.it.tile_begin;
    L.kvh = local / nt;
    L.t0 = local - L.kvh * nt;
    L.seg = min(nt - L.t0, gt_end - gt);
    const int tb_u = L.it.tile_begin + L.kvh * nt;
    const int first_cta = tb_u / p.tiles_per_cta, last_cta = (tb_u + nt - 1) / p.tiles_per_cta;
    L.n_parts = last_cta - first_cta + 1;
    L.part_idx = (int)blockIdx.x - first_cta;
    // (unit index + CTA index) grows strictly along the tile sequence: a unique slot per pair
    L.slot0 = lo * p.Hkv + L.kvh + first_cta;
    return L;
}

// out = merge of n_src partials (slot stride given) for one (item, kv head):
// final gated output or merged partial.  Executed by 128 threads.
__device__ __forceinline__ void merge_unit(const GqaParams &p, const Located &L, const float *src_o,
                           const float *src_m, const float *src_l, int n_src, float *s_w,
                           float *s_M, float *s_L, float *s_tmp) {
    const int tid = threadIdx.x;
    const int group = p.group;
    // m and l of every partial come in with all loads in flight (s_tmp: n_src * 16 floats of scratch); the
    // reductions then run out of shared memory in the order they always had
    for (int idx = tid; idx < n_src * 16; idx += 128) {
        s_w[idx] = src_m[idx];
        s_tmp[idx] = src_l[idx];
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
    // Four heads x four partials per round, every load of a round in flight together: the merging CTA is the last of
    // its unit to finish, usually at the very end of the launch, so this latency is on the launch's critical path
    // (and with one long sequence per launch a unit has up to MAX_SPLITS partials).
    for (int hr0 = 0; hr0 < group; hr0 += 4) {
        float2 acc[4], gt[4];
#pragma unroll
        for (int u = 0; u < 4; u++) {
            acc[u] = make_float2(0.0f, 0.0f);
            gt[u] = make_float2(0.0f, 0.0f);
            if (!p.partial_mode && p.gate && hr0 + u < group)
                gt[u] = *reinterpret_cast<const float2 *>(p.gate + (head0 + hr0 + u) * (size_t)p.gate_row_stride + 2 * tid);
        }
        for (int c0 = 0; c0 < n_src; c0 += 4) {
            float2 o[4][4];
#pragma unroll
            for (int k = 0; k < 4; k++)
#pragma unroll
                for (int u = 0; u < 4; u++)
                    o[k][u] = (c0 + k < n_src && hr0 + u < group)
                                  ? *reinterpret_cast<const float2 *>(src_o + ((size_t)(c0 + k) * 16 + hr0 + u) * HEAD_DIM + 2 * tid)
                                  : make_float2(0.0f, 0.0f);
#pragma unroll
            for (int k = 0; k < 4; k++) {  // partials are added in index order, as before
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
            const size_t off = (head0 + hr) * HEAD_DIM + 2 * tid;
            if (p.partial_mode) {
                const int hl = L.kvh * group + hr;  // head within the item
                *reinterpret_cast<float2 *>(p.po + (size_t)L.it.in_idx * p.po_item_stride + (size_t)hl * HEAD_DIM + 2 * tid) = acc[u];
                if (tid == 0) {
                    p.pm[(size_t)L.it.in_idx * p.pml_item_stride + hl] = s_M[hr];
                    p.pl[(size_t)L.it.in_idx * p.pml_item_stride + hl] = s_L[hr];
                }
            } else {
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
}

// Epilogue shared by both kernels.  The warp layout of the accumulators is:
// o[nt][2x + e] = row (g + 8x), dim 64*warp + 8*nt + 2t + e;  m_r / l_r per row
// (l_r still split over the four lanes of a row).
__device__ __forceinline__ void finish_unit(const GqaParams &p, const Located &L, float (&o)[8][4],
                                            float (&m_r)[2], float (&l_r)[2], float *s_w,
                                            float *s_M, float *s_L, int *s_flag_p, float *s_tmp) {
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
        // the unit was not split: finish in place
#pragma unroll
        for (int x = 0; x < 2; x++) {
            const int row = g + 8 * x;
            if (row >= group) continue;
            const float m_nat = m_r[x] * p.scale;
            if (p.partial_mode) {
                if (warp == 0 && t == 0) {
                    p.pm[(size_t)it.in_idx * p.pml_item_stride + L.kvh * group + row] = m_nat;
                    p.pl[(size_t)it.in_idx * p.pml_item_stride + L.kvh * group + row] = l_r[x];
                }
            }
            const float inv = p.partial_mode ? 1.0f : 1.0f / l_r[x];
#pragma unroll
            for (int nt = 0; nt < 8; nt++) {
                const size_t off = (head0 + row) * HEAD_DIM + 64 * warp + 8 * nt + 2 * t;
                float2 rv = make_float2(o[nt][2 * x] * inv, o[nt][2 * x + 1] * inv);
                if (p.partial_mode) {
                    *reinterpret_cast<float2 *>(p.po + (size_t)it.in_idx * p.po_item_stride +
                                                (size_t)(L.kvh * group + row) * HEAD_DIM + 64 * warp + 8 * nt + 2 * t) = rv;
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

    // the unit is shared: park the partial, the last CTA of the unit to finish merges
    const size_t slot0 = (size_t)L.slot0;  // first slot of the unit
    const size_t slot = slot0 + L.part_idx;
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
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        unsigned *tk = p.tickets + (size_t)L.item_idx * p.Hkv + L.kvh;
        const unsigned prev = atomicAdd(tk, 1u);
        *s_flag_p = (prev == (unsigned)(L.n_parts - 1));
        if (*s_flag_p) *tk = 0u;  // ready for the next launch
    }
    __syncthreads();
    if (!*s_flag_p) return;
    __threadfence();
    merge_unit(p, L, p.sc_o + slot0 * 16 * HEAD_DIM, p.sc_m + slot0 * 16, p.sc_l + slot0 * 16,
               L.n_parts, s_w, s_M, s_L, s_tmp);
}

}  // namespace mfc
