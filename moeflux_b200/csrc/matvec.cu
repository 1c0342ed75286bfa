// 4-bit group-64 affine-quantised matrix-vector product for sm_100a: the projections on
// either side of the attention path (q/k/v/o_proj, in_proj_qkv/z/a/b, out_proj).
//
// Format and maths follow the reference (crates/moeflux/src/riir/cpu_matvec.rs:83-171,
// shaders/shaders.metal:251-340, dispatch gpu_matvec.rs:84-129):
//   W_packed [out_dim][in_dim/8] u32, eight nibbles per word, least significant first =
//   consecutive input features; scales, biases bf16 [out_dim][in_dim/64];
//   out[r] = sum_c (nibble(r,c) * scale[r][c/64] + bias[r][c/64]) * x[c].
//
// The product is bound by the weight bytes (0.5 B per multiply-add), so the kernel is built
// around 16-byte weight loads and few instructions per nibble:
//   * one launch takes up to eight matrices that share x (q/k/v_proj; in_proj_qkv/z/a/b): a launch costs
//     ~10 us of fixed latency, several times what streaming a 20 MB matrix does;
//   * x (all n_vec vectors) and the sums of x over each 32-feature half group are staged in
//     shared memory once per CTA;
//   * a lane owns 16-byte chunks (32 nibbles, half a group) lane, lane+32, ... of FOUR rows
//     at a time, so a chunk of x read from shared memory serves four rows;
//   * a nibble n becomes the float 1 + n/128 by byte surgery (three ALU operations per word of eight nibbles,
//     then one PRMT per nibble), so per nibble there is about one ALU operation and one FMA;
//     with D = sum (1 + n/128) x and X = sum x over the chunk,
//     sum (n s + b) x = 128 s (D - X) + b X   (D - X cancels ~5 bits of the 24).
#include <stdint.h>

#include "common.cuh"
#include "kernels.h"

namespace mfc {

namespace {

constexpr int MV_ROWS = 4;      // rows a lane works on at a time
constexpr int MV_WARPS = 8;     // warps per CTA
constexpr int MV_THREADS = MV_WARPS * 32;

// The eight nibbles of a packed word as the floats 1 + n/128: with the nibble in the low half of byte 2 and the
// constant 0x80 in its high half, the bit pattern is 0x3F80'0000 | n << 16.  Two masks put 0x80 | n into every byte
// (three ALU operations per word), then one PRMT per nibble assembles the float: byte 3 = 0x3F, byte 2 = 0x80 | n.
__device__ __forceinline__ void nib_floats(uint32_t w, float (&f)[8]) {
    const uint32_t lo = (w & 0x0f0f0f0fu) | 0x80808080u;         // nibbles 0, 2, 4, 6
    const uint32_t hi = ((w >> 4) & 0x0f0f0f0fu) | 0x80808080u;  // nibbles 1, 3, 5, 7
    constexpr uint32_t K = 0x0000003fu;                          // byte 4 of the PRMT pair = 0x3F, bytes 5-7 = 0
    f[0] = __uint_as_float(__byte_perm(lo, K, 0x4055));
    f[1] = __uint_as_float(__byte_perm(hi, K, 0x4055));
    f[2] = __uint_as_float(__byte_perm(lo, K, 0x4155));
    f[3] = __uint_as_float(__byte_perm(hi, K, 0x4155));
    f[4] = __uint_as_float(__byte_perm(lo, K, 0x4255));
    f[5] = __uint_as_float(__byte_perm(hi, K, 0x4255));
    f[6] = __uint_as_float(__byte_perm(lo, K, 0x4355));
    f[7] = __uint_as_float(__byte_perm(hi, K, 0x4355));
}

template <int NV> struct MvDepth { static constexpr int value = NV <= 2 ? 2 : 1; };  // 16-byte chunks per row a lane has in flight

template <int NV>
__global__ void __launch_bounds__(MV_THREADS, NV <= 2 ? 2 : 1)
dequant_matvec_4bit_kernel(const __grid_constant__ MatvecBatch mb, const float *__restrict__ x, int in_dim) {
    extern __shared__ __align__(16) float smem_f[];
    // [NV][in_dim / 32][36]: a chunk of 32 features padded to 36 floats, so that lanes reading consecutive chunks
    // (128 bytes apart unpadded: one bank) spread over the banks
    float *xs = smem_f;
    const int in_dim_p = (in_dim >> 5) * 36;
    float *xh = smem_f + NV * in_dim_p;    // [NV][in_dim / 32]: sums of x over half groups
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n_chunks = in_dim >> 5;      // 16-byte chunks per row
    const int n_groups = in_dim >> 6;
    const int row_stride_w = in_dim >> 3;  // words per row

    constexpr int MV_DEPTH = MvDepth<NV>::value;
    struct Chunk {
        uint4 w[MV_ROWS];
        uint16_t sc[MV_ROWS], bi[MV_ROWS];
    };
    // row group rg (MV_ROWS rows of one matrix) -> matrix and first row; a group never straddles two matrices
    auto locate = [&](int rg, int &m, int &row0) {
        m = 0;
#pragma unroll
        for (int k = 1; k < MATVEC_MAX_MATS; k++)
            if (k < mb.n_mat && rg >= mb.group_begin[k]) m = k;
        row0 = (rg - mb.group_begin[m]) * MV_ROWS;
    };
    auto load_chunk = [&](int m, int row0, int c, Chunk &ch) {
        const uint32_t *W = mb.w[m];
        const uint16_t *scales = mb.scales[m], *biases = mb.biases[m];
        const int out_dim = mb.out_dim[m];
#pragma unroll
        for (int r = 0; r < MV_ROWS; r++) {
            const int row = min(row0 + r, out_dim - 1);  // rows past the end repeat the last one; not stored
            ch.w[r] = __ldg(reinterpret_cast<const uint4 *>(W + (size_t)row * row_stride_w + 4 * c));
            ch.sc[r] = __ldg(scales + (size_t)row * n_groups + (c >> 1));
            ch.bi[r] = __ldg(biases + (size_t)row * n_groups + (c >> 1));
        }
    };
    // the first weights are requested before x is staged, so that their latency runs under the staging
    const int rg_first = blockIdx.x * MV_WARPS + warp;
    Chunk first;
    if (rg_first < mb.total_groups && lane < n_chunks) {
        int m, row0;
        locate(rg_first, m, row0);
        load_chunk(m, row0, lane, first);
    }

    // x and, from the same registers, the sums over 32-feature half groups (8 consecutive threads hold one)
    const int n_f4 = NV * (in_dim >> 2);
    for (int i0 = 0; i0 < n_f4; i0 += 4 * MV_THREADS) {  // four loads in flight per thread
        float4 v[4];
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const int i = i0 + u * MV_THREADS + tid;
            v[u] = i < n_f4 ? __ldg(reinterpret_cast<const float4 *>(x) + i) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        }
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const int i = i0 + u * MV_THREADS + tid;
            if (i < n_f4) {
                const int vec = i / (in_dim >> 2), f = (i - vec * (in_dim >> 2)) * 4;  // feature index of the first float
                *reinterpret_cast<float4 *>(xs + (size_t)vec * in_dim_p + (f >> 5) * 36 + (f & 31)) = v[u];
            }
            float sm = (v[u].x + v[u].y) + (v[u].z + v[u].w);
            sm += __shfl_xor_sync(0xffffffffu, sm, 1);
            sm += __shfl_xor_sync(0xffffffffu, sm, 2);
            sm += __shfl_xor_sync(0xffffffffu, sm, 4);
            if ((tid & 7) == 0 && i < n_f4) xh[i >> 3] = sm;
        }
    }
    __syncthreads();

    // D = sum over the chunk of (1 + n/128) x, for MV_ROWS rows and NV vectors
    auto chunk_dot = [&](const Chunk &ch, int c, float (&acc)[MV_ROWS][NV]) {
        float d[MV_ROWS][NV];
#pragma unroll
        for (int r = 0; r < MV_ROWS; r++)
#pragma unroll
            for (int v = 0; v < NV; v++) d[r][v] = 0.0f;
#pragma unroll
        for (int q = 0; q < 4; q++) {  // one packed word = 8 features at a time
            float xv[NV][8];
#pragma unroll
            for (int v = 0; v < NV; v++) {
                const float4 a = *reinterpret_cast<const float4 *>(xs + (size_t)v * in_dim_p + 36 * c + 8 * q);
                const float4 b = *reinterpret_cast<const float4 *>(xs + (size_t)v * in_dim_p + 36 * c + 8 * q + 4);
                xv[v][0] = a.x; xv[v][1] = a.y; xv[v][2] = a.z; xv[v][3] = a.w;
                xv[v][4] = b.x; xv[v][5] = b.y; xv[v][6] = b.z; xv[v][7] = b.w;
            }
#pragma unroll
            for (int r = 0; r < MV_ROWS; r++) {
                const uint32_t word = q == 0 ? ch.w[r].x : q == 1 ? ch.w[r].y : q == 2 ? ch.w[r].z : ch.w[r].w;
                float f[8];
                nib_floats(word, f);
#pragma unroll
                for (int v = 0; v < NV; v++)
#pragma unroll
                    for (int j = 0; j < 8; j++) d[r][v] = fmaf(f[j], xv[v][j], d[r][v]);
            }
        }
#pragma unroll
        for (int v = 0; v < NV; v++) {
            const float xsum = xh[v * n_chunks + c];
#pragma unroll
            for (int r = 0; r < MV_ROWS; r++)
                acc[r][v] += fmaf(128.0f * bf16_bits_to_f32(ch.sc[r]), d[r][v] - xsum, bf16_bits_to_f32(ch.bi[r]) * xsum);
        }
    };

    for (int rg = rg_first; rg < mb.total_groups; rg += gridDim.x * MV_WARPS) {
        int m, row0;
        locate(rg, m, row0);
        float acc[MV_ROWS][NV];
#pragma unroll
        for (int r = 0; r < MV_ROWS; r++)
#pragma unroll
            for (int v = 0; v < NV; v++) acc[r][v] = 0.0f;
        // MV_DEPTH chunks per row in flight: the loads of a round are all issued before the first is used
        for (int c0 = lane; c0 < n_chunks; c0 += 32 * MV_DEPTH) {
            Chunk ch[MV_DEPTH];
#pragma unroll
            for (int k = 0; k < MV_DEPTH; k++) {
                const int c = c0 + 32 * k;
                if (c >= n_chunks) break;
                if (k == 0 && c0 == lane && rg == rg_first) ch[0] = first;
                else load_chunk(m, row0, c, ch[k]);
            }
#pragma unroll
            for (int k = 0; k < MV_DEPTH; k++) {
                const int c = c0 + 32 * k;
                if (c < n_chunks) chunk_dot(ch[k], c, acc);
            }
        }
#pragma unroll
        for (int r = 0; r < MV_ROWS; r++)
#pragma unroll
            for (int v = 0; v < NV; v++) {
                const float s = warp_sum(acc[r][v]);
                if (lane == 0 && row0 + r < mb.out_dim[m]) mb.out[m][(size_t)v * mb.out_dim[m] + row0 + r] = s;
            }
    }
}

// ------------------------------------------------------------------ several vectors: tensor cores
// With n_vec >= 2 the CUDA-core kernel above spends one FMA per nibble and vector and is bound by instruction
// issue, so batching vectors buys nothing.  Here the vectors are the N = 8 columns of mma.sync m16n8k16 (unused
// columns are zero), 16 rows of W are the M rows and 16 nibbles the K step:
//   * a nibble n enters as the bf16 16 + n = 0x4180 | n << 3, which is exact: one shift and one LOP3 give the
//     bf16x2 {16 + n_j, 16 + n_(j+4)} of a word (a larger offset, e.g. 128 + n, would cost accuracy below);
//   * x enters as a two-piece bf16 expansion (hi + mid, two MMAs per step), staged once per CTA in shared
//     memory in fragment order; the K index of the MMA is permuted to fit the nibble pairs above;
//   * per group of 64 features the 16 x 8 accumulator D = sum (16 + n) x is folded into the result as
//     s (D - 16 X) + b X with X = sum x over the group (cancels under 2 bits);
//   * a lane reads 8 bytes per row and group (a quad reads one 32-byte sector), eight groups in flight.
// The MMA sums over K, so every lane ends with finished outputs: rows g, g+8 x vectors 2t, 2t+1.
constexpr int MM_WARPS = 8;
constexpr int MM_THREADS = MM_WARPS * 32;
constexpr int MM_DEPTH = 8;  // groups of 64 features a lane has in flight

__device__ __forceinline__ void split_bf16x2_mv(float x0, float x1, uint32_t &hi, uint32_t &mid) {
    hi = pack_bf16x2(x0, x1);
    mid = pack_bf16x2(x0 - __uint_as_float(hi << 16), x1 - __uint_as_float(hi & 0xffff0000u));
}

// ks = 1, 2, 4 or 8 warps share a tile of 16 rows, each taking a contiguous range of groups (so that short
// launches still fill every warp slot of the GPU); their partial results are added in a fixed order.
template <int NV>
__global__ void __launch_bounds__(MM_THREADS, NV <= 3 ? 2 : 1)
dequant_matvec_4bit_mma_kernel(const __grid_constant__ MatvecBatch mb, const float *__restrict__ x, int in_dim, int ks) {
    extern __shared__ __align__(16) uint8_t smem_b[];
    // B fragments: [group][step 0/1][hi | mid][g < NV][t] x 16 bytes {m1b0, m1b1, m2b0, m2b1}: the lanes of a
    // quarter warp read consecutive 16-byte words
    uint4 *xb = reinterpret_cast<uint4 *>(smem_b);
    const int n_groups = in_dim >> 6;
    float *xg = reinterpret_cast<float *>(smem_b + (size_t)n_groups * 8 * NV * 32);  // [NV][n_groups] group sums
    float4 *red = reinterpret_cast<float4 *>(xg + NV * n_groups);                     // [MM_WARPS][32] partial results
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int row_stride_w = in_dim >> 3;

    // ---- stage x: entry e = (group, step, t) of vector v covers x[v][64 group + 16 t + 8 step + 0..7] ----
    const int n_entries = n_groups * 8;
    for (int i0 = 0; i0 < NV * n_entries; i0 += 2 * MM_THREADS) {
        float4 a[2], b[2];
        int vv[2], ee[2];
        bool in[2];
#pragma unroll
        for (int u = 0; u < 2; u++) {  // two entries (four 16-byte loads) in flight per thread
            const int i = i0 + u * MM_THREADS + tid;
            in[u] = i < NV * n_entries;
            vv[u] = in[u] ? i / n_entries : 0;
            ee[u] = in[u] ? i - vv[u] * n_entries : 0;
            const int gi = ee[u] >> 3, st = (ee[u] >> 2) & 1, tt = ee[u] & 3;
            const float4 *src = reinterpret_cast<const float4 *>(x + (size_t)vv[u] * in_dim + 64 * gi + 16 * tt + 8 * st);
            a[u] = in[u] ? __ldg(src) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            b[u] = in[u] ? __ldg(src + 1) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        }
#pragma unroll
        for (int u = 0; u < 2; u++) {
            if (in[u]) {
                uint32_t h[4], m[4];
                split_bf16x2_mv(a[u].x, b[u].x, h[0], m[0]);  // MMA 1, b0: k slots (2t, 2t+1)   <- features 0, 4
                split_bf16x2_mv(a[u].y, b[u].y, h[1], m[1]);  // MMA 1, b1: k slots (2t+8, 2t+9) <- features 1, 5
                split_bf16x2_mv(a[u].z, b[u].z, h[2], m[2]);  // MMA 2, b0                        <- features 2, 6
                split_bf16x2_mv(a[u].w, b[u].w, h[3], m[3]);  // MMA 2, b1                        <- features 3, 7
                const int gs = ee[u] >> 2, tt = ee[u] & 3;  // (group, step), t
                xb[((size_t)(gs * 2 + 0) * NV + vv[u]) * 4 + tt] = make_uint4(h[0], h[1], h[2], h[3]);
                xb[((size_t)(gs * 2 + 1) * NV + vv[u]) * 4 + tt] = make_uint4(m[0], m[1], m[2], m[3]);
            }
            // the eight entries of a group sit in eight consecutive threads
            float sm = ((a[u].x + a[u].y) + (a[u].z + a[u].w)) + ((b[u].x + b[u].y) + (b[u].z + b[u].w));
            sm += __shfl_xor_sync(0xffffffffu, sm, 1);
            sm += __shfl_xor_sync(0xffffffffu, sm, 2);
            sm += __shfl_xor_sync(0xffffffffu, sm, 4);
            if ((tid & 7) == 0 && in[u]) xg[vv[u] * n_groups + (ee[u] >> 3)] = sm;
        }
    }
    __syncthreads();

    const int tiles_total = mb.total_groups;  // here: tiles of 16 rows (see the launcher)
    const int tiles_per_cta = MM_WARPS / ks;
    const int tile_in_cta = warp / ks, split = warp - tile_in_cta * ks;
    const int gps = (n_groups + ks - 1) / ks;
    const int g_begin = split * gps, g_end = min(g_begin + gps, n_groups);
    for (int tile0 = blockIdx.x * tiles_per_cta; tile0 < tiles_total; tile0 += gridDim.x * tiles_per_cta) {
        const int tile = tile0 + tile_in_cta;
        const bool active = tile < tiles_total;
        // tile -> matrix (tiles never straddle two matrices: the launcher counts them per matrix)
        int m = 0;
#pragma unroll
        for (int k = 1; k < MATVEC_MAX_MATS; k++)
            if (k < mb.n_mat && tile >= mb.group_begin[k]) m = k;
        const int row0 = active ? (tile - mb.group_begin[m]) * 16 : 0;
        const int out_dim = mb.out_dim[m];
        float tot[4] = {0.0f, 0.0f, 0.0f, 0.0f};  // (row g, vec 2t), (row g, vec 2t+1), (row g+8, ...), (row g+8, ...)
        if (active) {
            const int r_lo = min(row0 + g, out_dim - 1), r_hi = min(row0 + g + 8, out_dim - 1);  // clamped, not stored
            const uint2 *w_lo = reinterpret_cast<const uint2 *>(mb.w[m] + (size_t)r_lo * row_stride_w) + t;
            const uint2 *w_hi = reinterpret_cast<const uint2 *>(mb.w[m] + (size_t)r_hi * row_stride_w) + t;
            const uint16_t *s_lo = mb.scales[m] + (size_t)r_lo * n_groups, *s_hi = mb.scales[m] + (size_t)r_hi * n_groups;
            const uint16_t *b_lo = mb.biases[m] + (size_t)r_lo * n_groups, *b_hi = mb.biases[m] + (size_t)r_hi * n_groups;
            for (int g0 = g_begin; g0 < g_end; g0 += MM_DEPTH) {
                uint2 wl[MM_DEPTH], wh[MM_DEPTH];
                uint16_t sl[MM_DEPTH], sh[MM_DEPTH], bl[MM_DEPTH], bh[MM_DEPTH];
#pragma unroll
                for (int k = 0; k < MM_DEPTH; k++) {
                    const int gi = min(g0 + k, g_end - 1);
                    wl[k] = __ldg(w_lo + 4 * gi);  // 8 words per row and group; this lane takes words 2t, 2t+1
                    wh[k] = __ldg(w_hi + 4 * gi);
                    sl[k] = __ldg(s_lo + gi);
                    sh[k] = __ldg(s_hi + gi);
                    bl[k] = __ldg(b_lo + gi);
                    bh[k] = __ldg(b_hi + gi);
                }
#pragma unroll
                for (int k = 0; k < MM_DEPTH; k++) {
                    const int gi = g0 + k;
                    if (gi >= g_end) break;
                    float d[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                    for (int st = 0; st < 2; st++) {
                        const uint32_t a_lo = st == 0 ? wl[k].x : wl[k].y, a_hi = st == 0 ? wh[k].x : wh[k].y;
                        uint4 bh4 = make_uint4(0, 0, 0, 0), bm4 = make_uint4(0, 0, 0, 0);
                        if (g < NV) {
                            const int gs = gi * 2 + st;
                            bh4 = xb[((size_t)(gs * 2 + 0) * NV + g) * 4 + t];
                            bm4 = xb[((size_t)(gs * 2 + 1) * NV + g) * 4 + t];
                        }
                        // bf16 16 + n = 0x4180 | n << 3 (exact): nibble pairs (j, j + 4) of a word in one register
                        constexpr uint32_t MASK = 0x00780078u, BASE = 0x41804180u;
                        uint32_t a1[4] = {((a_lo << 3) & MASK) | BASE, ((a_hi << 3) & MASK) | BASE,
                                          ((a_lo >> 1) & MASK) | BASE, ((a_hi >> 1) & MASK) | BASE};
                        uint32_t a2[4] = {((a_lo >> 5) & MASK) | BASE, ((a_hi >> 5) & MASK) | BASE,
                                          ((a_lo >> 9) & MASK) | BASE, ((a_hi >> 9) & MASK) | BASE};
                        mma_bf16_16816(d, a1, bh4.x, bh4.y);
                        mma_bf16_16816(d, a1, bm4.x, bm4.y);
                        mma_bf16_16816(d, a2, bh4.z, bh4.w);
                        mma_bf16_16816(d, a2, bm4.z, bm4.w);
                    }
                    const float x0 = (2 * t < NV) ? xg[(2 * t) * n_groups + gi] : 0.0f;
                    const float x1 = (2 * t + 1 < NV) ? xg[(2 * t + 1) * n_groups + gi] : 0.0f;
                    const float s0 = bf16_bits_to_f32(sl[k]), s1 = bf16_bits_to_f32(sh[k]);
                    const float c0 = bf16_bits_to_f32(bl[k]), c1 = bf16_bits_to_f32(bh[k]);
                    tot[0] += fmaf(s0, fmaf(-16.0f, x0, d[0]), c0 * x0);
                    tot[1] += fmaf(s0, fmaf(-16.0f, x1, d[1]), c0 * x1);
                    tot[2] += fmaf(s1, fmaf(-16.0f, x0, d[2]), c1 * x0);
                    tot[3] += fmaf(s1, fmaf(-16.0f, x1, d[3]), c1 * x1);
                }
            }
        }
        if (ks > 1) {  // uniform over the CTA
            red[warp * 32 + lane] = make_float4(tot[0], tot[1], tot[2], tot[3]);
            __syncthreads();
            if (split == 0)
                for (int k = 1; k < ks; k++) {
                    const float4 p = red[(warp + k) * 32 + lane];
                    tot[0] += p.x;
                    tot[1] += p.y;
                    tot[2] += p.z;
                    tot[3] += p.w;
                }
            __syncthreads();
        }
        if (active && split == 0) {
            float *o = mb.out[m];
            if (row0 + g < out_dim) {
                if (2 * t < NV) o[(size_t)(2 * t) * out_dim + row0 + g] = tot[0];
                if (2 * t + 1 < NV) o[(size_t)(2 * t + 1) * out_dim + row0 + g] = tot[1];
            }
            if (row0 + g + 8 < out_dim) {
                if (2 * t < NV) o[(size_t)(2 * t) * out_dim + row0 + g + 8] = tot[2];
                if (2 * t + 1 < NV) o[(size_t)(2 * t + 1) * out_dim + row0 + g + 8] = tot[3];
            }
        }
    }
}

size_t mma_smem(int in_dim, int nv) {
    return (size_t)(in_dim >> 6) * 8 * nv * 32 + sizeof(float) * (size_t)nv * (in_dim >> 6) + sizeof(float4) * MM_WARPS * 32;
}

template <int NV>
cudaError_t launch_mma(MatvecBatch mb, const float *x, int in_dim, int n_sms, cudaStream_t stream) {
    const size_t smem = mma_smem(in_dim, NV);
    static thread_local bool configured[64] = {false};  // per device: the opt-in is a host call of several microseconds
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(dequant_matvec_4bit_mma_kernel<NV>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)(227 * 1024));
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    int tiles = 0;  // here group_begin counts tiles of 16 rows per matrix
    for (int m = 0; m < mb.n_mat; m++) {
        mb.group_begin[m] = tiles;
        tiles += (mb.out_dim[m] + 15) / 16;
    }
    mb.total_groups = tiles;
    // warps per tile: enough to give every warp slot of the GPU work, while a warp keeps at least 8 groups
    const int ctas_per_sm = (NV <= 3 && smem <= 100 * 1024) ? 2 : 1;
    const int slots = n_sms * ctas_per_sm * MM_WARPS;
    int ks = 1;
    while (ks < MM_WARPS && tiles * ks < slots && (in_dim >> 6) / (2 * ks) >= 8) ks *= 2;
    const int tiles_per_cta = MM_WARPS / ks;
    int grid = (tiles + tiles_per_cta - 1) / tiles_per_cta;
    if (grid > n_sms * ctas_per_sm) grid = n_sms * ctas_per_sm;
    dequant_matvec_4bit_mma_kernel<NV><<<grid, MM_THREADS, smem, stream>>>(mb, x, in_dim, ks);
    return cudaGetLastError();
}

template <int NV>
cudaError_t launch_nv(const MatvecBatch &mb, const float *x, int in_dim, int n_sms, cudaStream_t stream) {
    const size_t smem = sizeof(float) * (size_t)NV * ((in_dim >> 5) * 36 + in_dim / 32);
    // the shared-memory opt-in and the occupancy query are host calls of several microseconds: once per size
    static thread_local size_t cfg_smem[16] = {0};
    static thread_local int cfg_dev[16], cfg_per_sm[16];
    int dev = 0;
    cudaGetDevice(&dev);
    int slot = -1;
    for (int i = 0; i < 16; i++)
        if (cfg_smem[i] == smem && cfg_dev[i] == dev) slot = i;
    if (slot < 0) {
        cudaError_t e = cudaFuncSetAttribute(dequant_matvec_4bit_kernel<NV>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)(227 * 1024));
        if (e != cudaSuccess) return e;
        int per_sm = 1;
        e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, dequant_matvec_4bit_kernel<NV>, MV_THREADS, smem);
        if (e != cudaSuccess) return e;
        static thread_local int next = 0;
        slot = next;
        next = (next + 1) & 15;
        cfg_smem[slot] = smem;
        cfg_dev[slot] = dev;
        cfg_per_sm[slot] = per_sm < 1 ? 1 : per_sm;
    }
    int grid = (mb.total_groups + MV_WARPS - 1) / MV_WARPS;
    if (grid > n_sms * cfg_per_sm[slot]) grid = n_sms * cfg_per_sm[slot];  // CTAs stride over the rows: x is staged once per CTA
    dequant_matvec_4bit_kernel<NV><<<grid, MV_THREADS, smem, stream>>>(mb, x, in_dim);
    return cudaGetLastError();
}

}  // namespace

size_t dequant_matvec_4bit_smem(int in_dim, int n_vec) {
    if (n_vec == 1) return sizeof(float) * (size_t)((in_dim >> 5) * 36 + in_dim / 32);
    return mma_smem(in_dim, n_vec);
}

cudaError_t launch_dequant_matvec_4bit(MatvecBatch mb, const float *x, int in_dim, int n_vec, int n_sms,
                                       cudaStream_t stream) {
    if (mb.n_mat < 1 || mb.n_mat > MATVEC_MAX_MATS) return cudaErrorInvalidValue;
    int g = 0;
    for (int m = 0; m < mb.n_mat; m++) {
        mb.group_begin[m] = g;
        g += (mb.out_dim[m] + MV_ROWS - 1) / MV_ROWS;
    }
    mb.total_groups = g;
    switch (n_vec) {
        case 1: return launch_nv<1>(mb, x, in_dim, n_sms, stream);
        case 2: return launch_mma<2>(mb, x, in_dim, n_sms, stream);
        case 3: return launch_mma<3>(mb, x, in_dim, n_sms, stream);
        case 4: return launch_mma<4>(mb, x, in_dim, n_sms, stream);
        case 5: return launch_mma<5>(mb, x, in_dim, n_sms, stream);
        case 6: return launch_mma<6>(mb, x, in_dim, n_sms, stream);
        case 7: return launch_mma<7>(mb, x, in_dim, n_sms, stream);
        case 8: return launch_mma<8>(mb, x, in_dim, n_sms, stream);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace mfc
