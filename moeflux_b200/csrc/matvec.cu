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
    float *xs = smem_f;                    // [NV][in_dim]
    float *xh = smem_f + NV * in_dim;      // [NV][in_dim / 32]: sums of x over half groups
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
            if (i < n_f4) reinterpret_cast<float4 *>(xs)[i] = v[u];
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
                const float4 a = *reinterpret_cast<const float4 *>(xs + (size_t)v * in_dim + 32 * c + 8 * q);
                const float4 b = *reinterpret_cast<const float4 *>(xs + (size_t)v * in_dim + 32 * c + 8 * q + 4);
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

template <int NV>
cudaError_t launch_nv(const MatvecBatch &mb, const float *x, int in_dim, int n_sms, cudaStream_t stream) {
    const size_t smem = sizeof(float) * (size_t)NV * (in_dim + in_dim / 32);
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

size_t dequant_matvec_4bit_smem(int in_dim, int n_vec) { return sizeof(float) * (size_t)n_vec * (in_dim + in_dim / 32); }

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
        case 2: return launch_nv<2>(mb, x, in_dim, n_sms, stream);
        case 3: return launch_nv<3>(mb, x, in_dim, n_sms, stream);
        case 4: return launch_nv<4>(mb, x, in_dim, n_sms, stream);
        case 5: return launch_nv<5>(mb, x, in_dim, n_sms, stream);
        case 6: return launch_nv<6>(mb, x, in_dim, n_sms, stream);
        case 7: return launch_nv<7>(mb, x, in_dim, n_sms, stream);
        case 8: return launch_nv<8>(mb, x, in_dim, n_sms, stream);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace mfc
