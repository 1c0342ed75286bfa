// 4-bit group-64 affine-quantised matrix-vector product for sm_100a: the projections on
// either side of the attention path (q/k/v/o_proj, in_proj_qkv/z/a/b, out_proj).
//
// Format and maths follow the reference (crates/moeflux/src/riir/cpu_matvec.rs:83-171,
// shaders/shaders.metal:251-340, dispatch gpu_matvec.rs:84-129):
//   W_packed [out_dim][in_dim/8] u32, eight nibbles per word, least significant first =
//   consecutive input features; scales, biases bf16 [out_dim][in_dim/64];
//   out[r] = sum_c (nibble(r,c) * scale[r][c/64] + bias[r][c/64]) * x[c].
//
// The product is bound by the weight bytes (0.5 B per multiply-add).  One launch takes up to eight matrices that
// share x (q/k/v_proj; in_proj_qkv/z/a/b): a launch has microseconds of fixed latency, as much as streaming a
// 20 MB matrix takes.  One kernel, instantiated for one to eight vectors.
#include <stdint.h>
#include <string.h>

#include "common.cuh"
#include "kernels.h"

namespace mfc {

namespace {

// ------------------------------------------------------------------ streamed tiles, integer tensor cores
// The product with one vector is the decode step's projection and is bound by the weight bytes, so the kernel is
// organised around keeping HBM busy and spending next to nothing per nibble (what changes with two to eight vectors
// is said where the consumer's two forms are):
//   * persistent CTAs take tiles of 16 rows from a counter in device memory (tiles of a launch cost the same, and the
//     two CTAs of an SM share the queue, so the SMs finish together);
//   * a producer warp streams each tile in stages of 16 rows x 1 KiB (32 groups) into a ring of 3-8 stages
//     (64-128 KiB in flight per SM): eight TMA boxes of 16 rows x 128 bytes with the 128-byte swizzle, completion on
//     mbarriers (a row-by-row cp.async.bulk of the same bytes ran at a third of the rate); it starts before x is staged;
//   * the nibbles go to the tensor core as they are: w & 0x0f0f0f0f and w & 0xf0f0f0f0 (16 n; the features they
//     multiply enter divided by 16) are the u8 A operands of mma.sync m16n8k32: two ALU operations per word of eight
//     nibbles, no offset to cancel afterwards;
//   * x enters as integers: per group of 64 features, q = rint(x / sx) with sx the power of two that puts the
//     group's largest |x| below 2^30, written in four balanced base-256 digits (s8: the bytes of q + 0x808080 with
//     the top bit of the three low bytes flipped).  The four digits of a group are four of the eight B columns, so
//     two groups share one accumulator and every lane of a quad ends up owning one (group, digit pair):
//     sum n x = sx * (D0 + 256 D1 + 256^2 D2 + 256^3 D3) is exact integer arithmetic, and the only roundings are
//     those of x to 31 bits (27 for the features that enter divided by 16) relative to its group's largest element,
//     of the integers to fp32, and of the fp32 sums
//     over groups (the reference's CPU product rounds every multiply-add);
//   * scales and biases of a stage (16 rows x 64 bytes each) are two more boxes of the same stage when their rows
//     are 16-byte aligned (in_dim a multiple of 512), otherwise the consumers read them from global memory;
//   * the launch is a programmatic dependent launch: its CTAs may start while the kernel before it in the stream is
//     still draining, and the producer warps request tensor maps and weights at once (the first box of a cold launch
//     takes 2-3 us to arrive); only the consumers wait for the earlier kernel, before they read x or write results;
//   * the eight consumer warps split the groups of a stage; their partial sums for a tile meet in shared memory, four
//     tiles behind one rendezvous, and are added in a fixed order (results do not depend on timing).
// A NaN or infinity in x makes every output NaN, as it does in the reference's product.
// Consumer warps (a producer warp comes on top): eight, one per box of a stage, for one or two vectors; sixteen, two
// per box (one pair of groups each), from three vectors on, where the work per stage grows with the vectors and one
// CTA per SM is all that fits: twice the warps hide the latencies that eight cannot.
__host__ __device__ constexpr int sv_warps(int n_vec) { return n_vec >= 3 ? 16 : 8; }
constexpr int SV_ROWS = 16;                        // rows per tile: M of the MMA
constexpr int SV_CHUNK_GROUPS = 32;                // groups of 64 features per stage
constexpr int SV_ROW_BYTES = SV_CHUNK_GROUPS * 32; // 1 KiB of a row per stage
constexpr int SV_BOX_BYTES = SV_ROWS * 128;        // one TMA box: 16 rows x 128 bytes (4 groups), 128-byte swizzle
constexpr int SV_BOXES = SV_ROW_BYTES / 128;       // 8 boxes per stage: box w holds the groups consumer warp w takes
constexpr int SV_W_BYTES = SV_BOXES * SV_BOX_BYTES;  // weights of a stage: 16 KiB
constexpr int SV_SB_ROW = SV_CHUNK_GROUPS * 2;     // scales (or biases) of a row in a stage: 64 bytes
constexpr int SV_SB_BOX = SV_ROWS * SV_SB_ROW;     // one TMA box of scales (or of biases): 16 rows x 32 groups, 1 KiB
constexpr int SV_STAGE_BYTES = SV_W_BYTES + 2 * SV_SB_BOX;  // 18 KiB: a multiple of the swizzle atom
static_assert(SV_STAGE_BYTES % 1024 == 0, "stages keep the 1 KiB alignment of the swizzled boxes");
constexpr int SV_MAX_STAGES = 8;
constexpr int SV_BATCH = 4;                        // tiles combined behind one rendezvous (at most)
// ... two with sixteen consumer warps, whose table of partial sums is twice as wide
__host__ __device__ constexpr int sv_batch(int n_vec) { return n_vec >= 3 ? 2 : SV_BATCH; }
constexpr int SV_OFF_HDR = 256;                    // after the mbarriers
constexpr int SV_OFF_SLOT = SV_OFF_HDR + SV_MAX_STAGES * 16;
constexpr int SV_OFF_RED = SV_OFF_SLOT + 2 * SV_BATCH * 8 + 64;  // (64 spare bytes)
static_assert(SV_OFF_RED % 16 == 0, "alignment of the shared-memory regions");
// after the partial sums [2][tiles of a batch][consumer warps][n_vec][SV_ROWS]: per vector and group {sx, sx * 256^2, sum of x, -},
// then per vector and group the 256 bytes of digits in B-fragment order
__host__ __device__ constexpr size_t sv_off_xw(int n_vec) {
    return (size_t)SV_OFF_RED + 2 * sv_batch(n_vec) * sv_warps(n_vec) * SV_ROWS * 4 * (size_t)n_vec;
}
__host__ __device__ inline size_t sv_fixed_bytes(int in_dim, int n_vec) {
    const size_t n_groups = (size_t)(in_dim >> 6);
    return (sv_off_xw(n_vec) + (size_t)n_vec * (n_groups * 16 + n_groups * 256) + 1023) & ~(size_t)1023;
}

__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// D(16x8,s32) += A(16x32,u8,row) * B(32x8,s8,col)
__device__ __forceinline__ void mma_u8s8_16832(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
    asm volatile(  // volatile: the instruction needs the whole warp, so it must stay where it is written
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 "
        "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// One poll of an mbarrier phase that lets the hardware park the thread for up to `ns` nanoseconds (it resumes when the
// phase completes): a waiting warp then spends no issue slots, which the warps that have data need.
__device__ __forceinline__ bool mbar_try_wait_parked(uint64_t *bar, unsigned parity, unsigned ns) {
    unsigned ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(ns)
        : "memory");
    return ok != 0;
}
// Bounded wait (each poll parks for up to a microsecond) that also gives up when another warp of the CTA has.
__device__ __forceinline__ bool sv_wait(uint64_t *bar, unsigned parity, unsigned spins, volatile int *abort_flag) {
    for (unsigned i = 0; i < spins; i++) {
        if (mbar_try_wait_parked(bar, parity, 1000u)) return true;
        if ((i & 15u) == 15u && *abort_flag) return false;
    }
    return false;
}

// Optional per-CTA phase stamps (nanoseconds): 0 entry, 1 barriers set up, 2 x staged (this thread), 3 x staged (all),
// 4 first stage arrived, 5 last stage consumed, 6 results stored; 7 (producer) first ring of stages issued.
__device__ __forceinline__ void sv_trace(const MatvecBatch &mb, int w) {
    if (mb.trace) mb.trace[(size_t)blockIdx.x * PHASE_TRACE_WORDS + w] = global_timer_ns();
}

template <int NV>
__global__ void __launch_bounds__((sv_warps(NV) + 1) * 32, NV <= 2 ? 2 : 1)
dequant_matvec_4bit_stream_kernel(const __grid_constant__ MatvecMaps maps, const __grid_constant__ MatvecBatch mb,
                                  const float *__restrict__ x, int in_dim, int n_stages) {
    extern __shared__ __align__(16) uint8_t sv_smem_raw[];
    uint8_t *sv_smem = sv_smem_raw + ((1024u - (smem_u32(sv_smem_raw) & 1023u)) & 1023u);  // swizzled boxes: 1 KiB alignment
    uint64_t *full = reinterpret_cast<uint64_t *>(sv_smem);         // [SV_MAX_STAGES]
    uint64_t *empty = full + SV_MAX_STAGES;                         // [SV_MAX_STAGES]
    uint64_t *red_bar = empty + SV_MAX_STAGES;                      // rendezvous of the consumer warps
    volatile int *abort_flag = reinterpret_cast<volatile int *>(red_bar + 1);
    int4 *hdr = reinterpret_cast<int4 *>(sv_smem + SV_OFF_HDR);     // per stage: {tile, matrix, first row, chunk}
    int2 *slot_info = reinterpret_cast<int2 *>(sv_smem + SV_OFF_SLOT);  // [2][SV_BATCH]: {matrix, first row}
    constexpr int CW = sv_warps(NV);  // consumer warps
    constexpr int BATCH = sv_batch(NV);
    float *red = reinterpret_cast<float *>(sv_smem + SV_OFF_RED);   // [2][BATCH][CW][NV][SV_ROWS]
    float4 *xw = reinterpret_cast<float4 *>(sv_smem + sv_off_xw(NV));  // [NV][group]: {sx, sx * 256^2, sum of x, -}
    const int n_groups = in_dim >> 6;
    uint8_t *xb = reinterpret_cast<uint8_t *>(xw + (size_t)NV * n_groups);  // [NV][group][digit][word] x {b0, b1}
    uint8_t *stages = sv_smem + sv_fixed_bytes(in_dim, NV);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int row_bytes = in_dim >> 1;
    const int n_chunks = (n_groups + SV_CHUNK_GROUPS - 1) / SV_CHUNK_GROUPS;
    const unsigned spins = mb.spins ? mb.spins : (1u << 21);  // polls of up to a microsecond each

    if (tid == 0) sv_trace(mb, 0);
    if (tid == 0) {
        for (int s = 0; s < n_stages; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], CW);
        }
        mbar_init(red_bar, CW);
        *abort_flag = 0;
        mbar_fence_init();
    }
    __syncthreads();
    if (tid == 0) sv_trace(mb, 1);

    if (warp == CW) {
        // ---------------- producer: tiles from the launch-wide counter, stages into the ring
        if (lane < mb.n_mat) {
            prefetch_tmap(&maps.w[lane]);
            if (mb.sb_bulk) {
                prefetch_tmap(&maps.sc[lane]);
                prefetch_tmap(&maps.bi[lane]);
            }
        }
        unsigned it = 0;  // stages issued
        int st = 0;       // it modulo the ring, and the parity of the ring's previous turn
        unsigned prev_phase = 1;
        bool ok = true;
        int tile = blockIdx.x;  // the first tile is fixed; the rest come from the counter, asked for one tile ahead
        int tile_next = 0;      // (the answer of an atomic takes a microsecond: as long as streaming a tile)
        if (lane == 0) tile_next = (int)(gridDim.x + atomicAdd(mb.sched, 1u));
        while (ok && tile < mb.total_groups) {
            int m = 0;
#pragma unroll
            for (int k = 1; k < MATVEC_MAX_MATS; k++)
                if (k < mb.n_mat && tile >= mb.group_begin[k]) m = k;
            const int row0 = (tile - mb.group_begin[m]) * SV_ROWS;
            for (int chunk = 0; chunk < n_chunks; chunk++) {
                if (it >= (unsigned)n_stages) ok = sv_wait(&empty[st], prev_phase, spins, abort_flag);
                if (!ok) break;
                const int bytes = min(SV_ROW_BYTES, row_bytes - chunk * SV_ROW_BYTES);  // of a row in this stage
                const int n_boxes = (bytes + 127) >> 7;
                if (lane == 0) {
                    hdr[st] = make_int4(tile, m, row0, chunk);
                    mbar_expect_tx(&full[st], (unsigned)(n_boxes * SV_BOX_BYTES + (mb.sb_bulk ? 2 * SV_SB_BOX : 0)));
                }
                __syncwarp();
                uint8_t *dst = stages + (size_t)st * SV_STAGE_BYTES;
                // box b: bytes [128 b, 128 b + 128) of the stage's 1 KiB of rows row0 .. row0 + 15 (rows and bytes
                // past the matrix arrive as zeros); then the rows' scales and biases of the stage's 32 groups
                // (test hook: the first CTA arms its first stage and requests nothing, so that the consumers' bounded
                // wait runs out with nothing in flight)
                if (mb.inject_lost_load && blockIdx.x == 0 && it == 0) {
                } else if (lane < n_boxes)
                    tma_load_2d(dst + lane * SV_BOX_BYTES, &maps.w[m], chunk * SV_ROW_BYTES + lane * 128, row0, &full[st]);
                else if (mb.sb_bulk && lane == 8)
                    tma_load_2d(dst + SV_W_BYTES, &maps.sc[m], chunk * SV_CHUNK_GROUPS, row0, &full[st]);
                else if (mb.sb_bulk && lane == 9)
                    tma_load_2d(dst + SV_W_BYTES + SV_SB_BOX, &maps.bi[m], chunk * SV_CHUNK_GROUPS, row0, &full[st]);
                it++;
                if (++st == n_stages) {
                    st = 0;
                    prev_phase ^= 1u;
                }
            }
            if (!ok) break;
            tile = __shfl_sync(0xffffffffu, tile_next, 0);
            if (lane == 0 && tile < mb.total_groups) tile_next = (int)(gridDim.x + atomicAdd(mb.sched, 1u));
        }
        if (ok) {  // the stage after the last one carries "no more work"
            if (it >= (unsigned)n_stages) ok = sv_wait(&empty[st], prev_phase, spins, abort_flag);
            if (ok && lane == 0) {
                hdr[st] = make_int4(-1, 0, 0, 0);
                mbar_arrive(&full[st]);
            }
        }
        if (!ok) {
            // gave up (or a consumer did): no further copies are issued; the copies still in flight write into this
            // CTA's shared memory, so they are waited for (bounded again) before the warp leaves
            if (lane == 0) {
                *abort_flag = 1;
                atomicOr(mb.status, STATUS_TMA_TIMEOUT);
            }
            const unsigned first = it > (unsigned)n_stages ? it - (unsigned)n_stages : 0u;
            for (unsigned k = first; k < it; k++)
                mbar_wait_bounded(&full[k % (unsigned)n_stages], (k / (unsigned)n_stages) & 1u, spins);
        }
        // the last CTA to finish puts the counters back for the next launch
        if (lane == 0) {
            __threadfence();
            if (atomicAdd(mb.sched + 1, 1u) == gridDim.x - 1) {
                mb.sched[0] = 0u;
                mb.sched[1] = 0u;
                __threadfence();
            }
        }
        return;
    }

    // ---------------- consumers: x as integer digits in B-fragment order, then the stream of stages
    // x is an earlier kernel's result: wait for the kernels before this one to finish and their writes to be visible.
    // Only then may the kernel after this one start (it uses the tile counters this kernel's predecessor used).
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    {
        // the NV vectors are contiguous in x, in xw and in xb: staged as one vector of NV * in_dim features
        const float *xv_src = x;
        float4 *xw_v = xw;
        uint8_t *xb_v = xb;
        const int n_words = NV * (in_dim >> 3);  // a thread handles the 8 features of one packed word; 8 threads hold a group
        constexpr int XU = 4;             // words per thread whose loads are in flight together
        for (int wq0 = 0; wq0 < n_words; wq0 += CW * 32 * XU) {
            float4 va[XU], vb[XU];
#pragma unroll
            for (int u = 0; u < XU; u++) {
                const int wq = wq0 + u * CW * 32 + tid;
                const bool in = wq < n_words;
                va[u] = in ? __ldg(reinterpret_cast<const float4 *>(xv_src) + 2 * wq) : make_float4(0.f, 0.f, 0.f, 0.f);
                vb[u] = in ? __ldg(reinterpret_cast<const float4 *>(xv_src) + 2 * wq + 1) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int u = 0; u < XU; u++) {
                const int wq = wq0 + u * CW * 32 + tid;
                if (wq0 + u * CW * 32 >= n_words) break;  // uniform over the CTA
                const bool in = wq < n_words;
                const float v[8] = {va[u].x, va[u].y, va[u].z, va[u].w, vb[u].x, vb[u].y, vb[u].z, vb[u].w};
                float sm = ((v[0] + v[1]) + (v[2] + v[3])) + ((v[4] + v[5]) + (v[6] + v[7]));
                uint32_t ebits = 0;  // largest exponent field of the group: the scale, and NaN / infinity (255)
#pragma unroll
                for (int j = 0; j < 8; j++) ebits = max(ebits, (__float_as_uint(v[j]) >> 23) & 0xffu);
#pragma unroll
                for (int o = 1; o < 8; o <<= 1) {
                    ebits = max(ebits, __shfl_xor_sync(0xffffffffu, ebits, o));
                    sm += __shfl_xor_sync(0xffffffffu, sm, o);
                }
                const bool finite = ebits != 255u;
                const uint32_t e = min(max(ebits, 30u), 254u);
                const float inv = __uint_as_float((283u - e) << 23);  // 2^(29 - exponent): |x| * inv < 2^30
                float sx = __uint_as_float((e - 29u) << 23);
                if (!finite) sx = __uint_as_float(0x7fc00000u);
                // the four s8 digits of an element are the bytes of this word
                // (features 1, 3, 5, 7 of a word enter divided by 16: their nibbles go to the tensor core as 16 n)
                const float inv_odd = inv * 0.0625f;
                uint32_t dg[8];
#pragma unroll
                for (int j = 0; j < 8; j++)
                    dg[j] = finite ? ((uint32_t)(__float2int_rn(v[j] * ((j & 1) ? inv_odd : inv)) + 0x00808080) ^ 0x00808080u) : 0u;
                // 4 x 4 byte transposes: digit c of features 0, 2, 4, 6 (the word's low nibbles) and of 1, 3, 5, 7
                uint32_t b0[4], b1[4];
                {
                    const uint32_t l01 = __byte_perm(dg[0], dg[2], 0x5140), h01 = __byte_perm(dg[0], dg[2], 0x7362);
                    const uint32_t l23 = __byte_perm(dg[4], dg[6], 0x5140), h23 = __byte_perm(dg[4], dg[6], 0x7362);
                    b0[0] = __byte_perm(l01, l23, 0x5410);
                    b0[1] = __byte_perm(l01, l23, 0x7632);
                    b0[2] = __byte_perm(h01, h23, 0x5410);
                    b0[3] = __byte_perm(h01, h23, 0x7632);
                }
                {
                    const uint32_t l01 = __byte_perm(dg[1], dg[3], 0x5140), h01 = __byte_perm(dg[1], dg[3], 0x7362);
                    const uint32_t l23 = __byte_perm(dg[5], dg[7], 0x5140), h23 = __byte_perm(dg[5], dg[7], 0x7362);
                    b1[0] = __byte_perm(l01, l23, 0x5410);
                    b1[1] = __byte_perm(l01, l23, 0x7632);
                    b1[2] = __byte_perm(h01, h23, 0x5410);
                    b1[3] = __byte_perm(h01, h23, 0x7632);
                }
                if (in) {
                    const int gi = wq >> 3, wl = wq & 7;
                    uint8_t *dst = xb_v + (size_t)gi * 256 + (wl >> 1) * 16 + (wl & 1) * 8;
#pragma unroll
                    for (int c = 0; c < 4; c++) *reinterpret_cast<uint2 *>(dst + c * 64) = make_uint2(b0[c], b1[c]);
                    if (wl == 0) xw_v[gi] = make_float4(sx, sx * 65536.0f, sm, 0.0f);
                }
            }
        }
    }
    if (tid == 0) sv_trace(mb, 2);
    asm volatile("bar.sync 1, %0;" ::"n"(CW * 32) : "memory");
    if (tid == 0) sv_trace(mb, 3);

    const int g = lane >> 2, t = lane & 3;
    const int my_sel = t >> 1, my_h = t & 1;  // which group of a pair, and which digit pair, this lane finishes
    const int b_sel = g >> 2, b_c = g & 3;    // which group and digit this lane's B column carries
    constexpr uint32_t NIB = 0x0f0f0f0fu;
    float tot0 = 0.0f, tot1 = 0.0f;           // rows g and g + 8 of the current tile
    int slot = 0, buf = 0;
    unsigned red_parity = 0;
    bool failed = false;

    auto flush = [&]() -> bool {
        // partial sums of `slot` tiles are in red[buf]: meet, then add the eight warps' parts in a fixed order
        __syncwarp();
        if (lane == 0) mbar_arrive(red_bar);
        if (!sv_wait(red_bar, red_parity, spins, abort_flag)) return false;
        red_parity ^= 1u;
        for (int idx = tid; idx < slot * NV * SV_ROWS; idx += CW * 32) {
            const int s = idx / (NV * SV_ROWS), vr = idx - s * (NV * SV_ROWS);  // vr = vector * 16 + row
            const int2 info = slot_info[buf * SV_BATCH + s];
            const float *src = red + ((size_t)(buf * BATCH + s) * CW) * (NV * SV_ROWS) + vr;
            float sum = 0.0f;
#pragma unroll
            for (int w = 0; w < CW; w++) sum += src[w * (NV * SV_ROWS)];
            const int out_dim = mb.out_dim[info.x], r = vr & (SV_ROWS - 1);
            if (info.y + r < out_dim) mb.out[info.x][(size_t)(vr >> 4) * out_dim + info.y + r] = sum;
        }
        buf ^= 1;
        slot = 0;
        return true;
    };

    // lane constants of the stage loop
    // Row g of the MMA is row rho(g) = (g >> 1) | (g & 1) << 2 of the tile (and g + 8 is rho(g) + 8): the eight lanes
    // that shared memory serves together (g = 2q, 2q + 1; t = 0..3) then read rows q and q + 4, whose 16-byte
    // chunks the 128-byte swizzle stores in opposite halves of the row: no bank is asked twice.
    const int rho = (g >> 1) | ((g & 1) << 2);
    // the box of a stage this warp works on, and which of its two pairs of groups (both, with eight consumer warps)
    const int box = CW == 16 ? warp >> 1 : warp;
    const int u_first = CW == 16 ? (warp & 1) : 0;
    constexpr int U_COUNT = CW == 16 ? 1 : 2;
    // Lane (g, t) reads chunk 4 u + t of row rho (16 bytes = four words = half a group) for pair u of the warp's box.
    // MMA j of the pair takes word j of every lane: its k slots of lanes t = 0, 1 are features of the pair's first
    // group, those of lanes t = 2, 3 features of the second; the B columns 0-3 hold the first group's digits of x and
    // are zero on the second group's k slots, columns 4-7 the other way round.
    int a_off[2];
#pragma unroll
    for (int uu = 0; uu < 2; uu++) a_off[uu] = box * SV_BOX_BYTES + rho * 128 + (((4 * (u_first + uu) + t) ^ rho) << 4);
    // B operand of lane (g, t): column g = digit b_c of group b_sel of the pair, on the k slots of lane t: real
    // for the lanes whose t belongs to that group, zero (never loaded) for the others
    const bool b_real = b_sel == (t >> 1);
    const uint8_t *xb_lane = xb + (4 * box + b_sel) * 256 + b_c * 64 + (t & 1) * 32;
    const int sb_lane = SV_W_BYTES + rho * SV_SB_ROW + 8 * box;  // scales of row rho, the box's four groups
    const float *xw_lane = reinterpret_cast<const float *>(xw + 4 * box + my_sel);
    uint4 bb[2][2];  // [pair][MMAs 0-1 | 2-3]: {b0, b1} of two MMAs each; stays zero in the lanes that never load
#pragma unroll
    for (int u = 0; u < 2; u++) bb[u][0] = bb[u][1] = make_uint4(0u, 0u, 0u, 0u);

    // ---- two to eight vectors: the B columns are (vector, digit), two vectors to an MMA, so the two groups of a pair
    // can no longer share an accumulator and every MMA must take its k slots from one group.  A lane holds four words
    // of one group (lanes t = 0, 1: the first group of the pair, t = 2, 3: the second); lanes t and t ^ 2 swap two
    // words each, after which every lane holds words base, base + 1 (base = 4 (t & 1) + 2 (t >> 1)) of both groups:
    // two MMAs per group and pair of vectors, the same loads and the same integer work per nibble as with one vector.
    constexpr int CB = (NV + 1) / 2;  // pairs of vectors
    float totv[CB][2];                // rows rho and rho + 8 of the tile, vector 2 cb + (t >> 1), digit pair t & 1
#pragma unroll
    for (int cb = 0; cb < CB; cb++) totv[cb][0] = totv[cb][1] = 0.0f;
    const bool upper = t >= 2;
    const int b_word = 4 * (t & 1) + 2 * (t >> 1);
    auto several_vectors = [&](const uint8_t *sbase, int m, int row0, int chunk, int groups_here) {
        // scales and biases of the box's four groups, rows rho and rho + 8: two bf16 per word (groups 0-1 | 2-3)
        uint2 sc_lo, sc_hi, bi_lo, bi_hi;
        if (mb.sb_bulk) {
            const uint8_t *sb = sbase + sb_lane;
            sc_lo = *reinterpret_cast<const uint2 *>(sb);
            sc_hi = *reinterpret_cast<const uint2 *>(sb + 8 * SV_SB_ROW);
            bi_lo = *reinterpret_cast<const uint2 *>(sb + SV_SB_BOX);
            bi_hi = *reinterpret_cast<const uint2 *>(sb + SV_SB_BOX + 8 * SV_SB_ROW);
        } else {
            const int out_dim = mb.out_dim[m];
            const int r_lo = min(row0 + rho, out_dim - 1), r_hi = min(row0 + rho + 8, out_dim - 1);
            uint32_t w4[4][4];
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const size_t cc = min((size_t)chunk * SV_CHUNK_GROUPS + 4 * box + q, (size_t)n_groups - 1);
                w4[0][q] = __ldg(mb.scales[m] + (size_t)r_lo * n_groups + cc);
                w4[1][q] = __ldg(mb.scales[m] + (size_t)r_hi * n_groups + cc);
                w4[2][q] = __ldg(mb.biases[m] + (size_t)r_lo * n_groups + cc);
                w4[3][q] = __ldg(mb.biases[m] + (size_t)r_hi * n_groups + cc);
            }
            sc_lo = make_uint2(w4[0][0] | (w4[0][1] << 16), w4[0][2] | (w4[0][3] << 16));
            sc_hi = make_uint2(w4[1][0] | (w4[1][1] << 16), w4[1][2] | (w4[1][3] << 16));
            bi_lo = make_uint2(w4[2][0] | (w4[2][1] << 16), w4[2][2] | (w4[2][3] << 16));
            bi_hi = make_uint2(w4[3][0] | (w4[3][1] << 16), w4[3][2] | (w4[3][3] << 16));
        }
        const size_t g_first = (size_t)chunk * SV_CHUNK_GROUPS + 4 * box;  // the box's first group
#pragma unroll
        for (int uu = 0; uu < U_COUNT; uu++) {
            const int u = u_first + uu;  // the pair of groups: both for a warp that has the box to itself
            const uint32_t p_sc_lo = u ? sc_lo.y : sc_lo.x, p_sc_hi = u ? sc_hi.y : sc_hi.x;  // the pair's two groups
            const uint32_t p_bi_lo = u ? bi_lo.y : bi_lo.x, p_bi_hi = u ? bi_hi.y : bi_hi.x;
            const uint4 wa = *reinterpret_cast<const uint4 *>(sbase + a_off[uu]);
            const uint4 wb = *reinterpret_cast<const uint4 *>(sbase + a_off[uu] + 8 * 128);
            // rows rho (wa) and rho + 8 (wb): words w0, w1 of the pair's first group (ga, gb) and of its second (ha, hb)
            const uint32_t ra0 = __shfl_xor_sync(0xffffffffu, upper ? wa.x : wa.z, 2);
            const uint32_t ra1 = __shfl_xor_sync(0xffffffffu, upper ? wa.y : wa.w, 2);
            const uint32_t rb0 = __shfl_xor_sync(0xffffffffu, upper ? wb.x : wb.z, 2);
            const uint32_t rb1 = __shfl_xor_sync(0xffffffffu, upper ? wb.y : wb.w, 2);
            const uint32_t ga0 = upper ? ra0 : wa.x, ga1 = upper ? ra1 : wa.y, gb0 = upper ? rb0 : wb.x, gb1 = upper ? rb1 : wb.y;
            const uint32_t ha0 = upper ? wa.z : ra0, ha1 = upper ? wa.w : ra1, hb0 = upper ? wb.z : rb0, hb1 = upper ? wb.w : rb1;
#pragma unroll
            for (int cb = 0; cb < CB; cb++) {
                // this lane's B column: digit g & 3 of vector 2 cb + (g >> 2), on this lane's k slots: words
                // b_word, b_word + 1 of the group
                const int vb = 2 * cb + (g >> 2);
                uint4 bg = make_uint4(0u, 0u, 0u, 0u), bh = bg;
                if (vb < NV) {
                    const uint8_t *pb = xb + ((size_t)vb * n_groups + g_first + 2 * u) * 256 + (g & 3) * 64 + b_word * 8;
                    bg = *reinterpret_cast<const uint4 *>(pb);
                    bh = *reinterpret_cast<const uint4 *>(pb + 256);
                }
                int da[4] = {0, 0, 0, 0}, db[4] = {0, 0, 0, 0};
                mma_u8s8_16832(da, ga0 & NIB, gb0 & NIB, ga0 & ~NIB, gb0 & ~NIB, bg.x, bg.y);
                mma_u8s8_16832(db, ha0 & NIB, hb0 & NIB, ha0 & ~NIB, hb0 & ~NIB, bh.x, bh.y);
                mma_u8s8_16832(da, ga1 & NIB, gb1 & NIB, ga1 & ~NIB, gb1 & ~NIB, bg.z, bg.w);
                mma_u8s8_16832(db, ha1 & NIB, hb1 & NIB, ha1 & ~NIB, hb1 & ~NIB, bh.z, bh.w);
                const int v = 2 * cb + (t >> 1);  // the accumulator columns of this lane: digit pair t & 1 of vector v
                if (v < NV) {
#pragma unroll
                    for (int grp = 0; grp < 2; grp++) {
                        const int q = 2 * u + grp;
                        if (4 * box + q < groups_here) {
                            const float4 wv = xw[(size_t)v * n_groups + g_first + q];
                            const float wgt = my_h ? wv.y : wv.x;
                            const int *d = grp ? db : da;
                            const float f0 = (float)(d[0] + d[1] * 256) * wgt;  // row rho
                            const float f1 = (float)(d[2] + d[3] * 256) * wgt;  // row rho + 8
                            totv[cb][0] = fmaf(bf16_bits_to_f32((uint16_t)(p_sc_lo >> (16 * grp))), f0, totv[cb][0]);
                            totv[cb][1] = fmaf(bf16_bits_to_f32((uint16_t)(p_sc_hi >> (16 * grp))), f1, totv[cb][1]);
                            if (my_h == 0) {
                                totv[cb][0] = fmaf(bf16_bits_to_f32((uint16_t)(p_bi_lo >> (16 * grp))), wv.z, totv[cb][0]);
                                totv[cb][1] = fmaf(bf16_bits_to_f32((uint16_t)(p_bi_hi >> (16 * grp))), wv.z, totv[cb][1]);
                            }
                        }
                    }
                }
            }
        }
    };

    int st = 0;
    unsigned phase = 0;
    long long wait_cycles = 0;
    for (bool first = true;; first = false) {
        const long long w0 = mb.trace ? clock64() : 0;
        if (!sv_wait(&full[st], phase, spins, abort_flag)) {
            failed = true;
            break;
        }
        if (mb.trace) wait_cycles += clock64() - w0;
        const int4 h = hdr[st];
        if (first && tid == 0) sv_trace(mb, 4);
        if (h.x < 0) break;
        const int m = h.y, row0 = h.z, chunk = h.w;
        const int groups_here = min(SV_CHUNK_GROUPS, n_groups - chunk * SV_CHUNK_GROUPS);
        const uint8_t *sbase = stages + (size_t)st * SV_STAGE_BYTES;
        if (NV > 1) {
            if (4 * box < groups_here)
                several_vectors(sbase, m, row0, chunk, groups_here);
        } else if (4 * box < groups_here) {  // the warp's box was loaded (bytes of it past the row's end arrived as zeros)
            // this lane's scale and bias of the two pairs
            uint16_t s_lo[2], s_hi[2], c_lo[2], c_hi[2];
            if (mb.sb_bulk) {
                // the warp's four groups are 8 bytes of a row: one read per row and array, then this lane's two
                const uint8_t *sb = sbase + sb_lane;
                const uint2 a = *reinterpret_cast<const uint2 *>(sb);
                const uint2 b = *reinterpret_cast<const uint2 *>(sb + 8 * SV_SB_ROW);
                const uint2 c = *reinterpret_cast<const uint2 *>(sb + SV_SB_BOX);
                const uint2 e8 = *reinterpret_cast<const uint2 *>(sb + SV_SB_BOX + 8 * SV_SB_ROW);
                const int sh = 16 * my_sel;  // groups 4w + my_sel (low word) and 4w + 2 + my_sel (high word)
                s_lo[0] = (uint16_t)(a.x >> sh);
                s_lo[1] = (uint16_t)(a.y >> sh);
                s_hi[0] = (uint16_t)(b.x >> sh);
                s_hi[1] = (uint16_t)(b.y >> sh);
                c_lo[0] = (uint16_t)(c.x >> sh);
                c_lo[1] = (uint16_t)(c.y >> sh);
                c_hi[0] = (uint16_t)(e8.x >> sh);
                c_hi[1] = (uint16_t)(e8.y >> sh);
            } else {
                const int out_dim = mb.out_dim[m];
                const int r_lo = min(row0 + rho, out_dim - 1), r_hi = min(row0 + rho + 8, out_dim - 1);
                const size_t col = (size_t)chunk * SV_CHUNK_GROUPS + 4 * box + my_sel;
#pragma unroll
                for (int u = 0; u < 2; u++) {
                    const size_t cc = min(col + 2 * u, (size_t)n_groups - 1);
                    s_lo[u] = __ldg(mb.scales[m] + (size_t)r_lo * n_groups + cc);
                    s_hi[u] = __ldg(mb.scales[m] + (size_t)r_hi * n_groups + cc);
                    c_lo[u] = __ldg(mb.biases[m] + (size_t)r_lo * n_groups + cc);
                    c_hi[u] = __ldg(mb.biases[m] + (size_t)r_hi * n_groups + cc);
                }
            }
            const uint8_t *xb_here = xb_lane + (size_t)chunk * (SV_CHUNK_GROUPS * 256);
            int d[2][4] = {{0, 0, 0, 0}, {0, 0, 0, 0}}, e[2][4] = {{0, 0, 0, 0}, {0, 0, 0, 0}};  // two chains per pair
#pragma unroll
            for (int u = 0; u < 2; u++) {
                const uint4 wa = *reinterpret_cast<const uint4 *>(sbase + a_off[u]);
                const uint4 wb = *reinterpret_cast<const uint4 *>(sbase + a_off[u] + 8 * 128);
                if (b_real) {
                    bb[u][0] = *reinterpret_cast<const uint4 *>(xb_here + u * 512);
                    bb[u][1] = *reinterpret_cast<const uint4 *>(xb_here + u * 512 + 16);
                }
                mma_u8s8_16832(d[u], wa.x & NIB, wb.x & NIB, wa.x & ~NIB, wb.x & ~NIB, bb[u][0].x, bb[u][0].y);
                mma_u8s8_16832(e[u], wa.y & NIB, wb.y & NIB, wa.y & ~NIB, wb.y & ~NIB, bb[u][0].z, bb[u][0].w);
                mma_u8s8_16832(d[u], wa.z & NIB, wb.z & NIB, wa.z & ~NIB, wb.z & ~NIB, bb[u][1].x, bb[u][1].y);
                mma_u8s8_16832(e[u], wa.w & NIB, wb.w & NIB, wa.w & ~NIB, wb.w & ~NIB, bb[u][1].z, bb[u][1].w);
            }
#pragma unroll
            for (int u = 0; u < 2; u++)
#pragma unroll
                for (int k = 0; k < 4; k++) d[u][k] += e[u][k];
            const float *xwv = xw_lane + (size_t)chunk * (SV_CHUNK_GROUPS * 4);
#pragma unroll
            for (int u = 0; u < 2; u++) {
                if (4 * box + 2 * u + my_sel < groups_here) {  // (always, but for a ragged last stage)
                    const float wgt = xwv[8 * u + my_h];
                    const float f0 = (float)(d[u][0] + d[u][1] * 256) * wgt;  // row rho:     digits (2h, 2h+1) of the group
                    const float f1 = (float)(d[u][2] + d[u][3] * 256) * wgt;  // row rho + 8
                    tot0 = fmaf(bf16_bits_to_f32(s_lo[u]), f0, tot0);
                    tot1 = fmaf(bf16_bits_to_f32(s_hi[u]), f1, tot1);
                    if (my_h == 0) {
                        const float xs = xwv[8 * u + 2];
                        tot0 = fmaf(bf16_bits_to_f32(c_lo[u]), xs, tot0);
                        tot1 = fmaf(bf16_bits_to_f32(c_hi[u]), xs, tot1);
                    }
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[st]);
        if (++st == n_stages) {
            st = 0;
            phase ^= 1u;
        }
        if (chunk == n_chunks - 1) {
            float *dst = red + ((size_t)(buf * BATCH + slot) * CW + warp) * (NV * SV_ROWS);
            if (NV == 1) {
                tot0 += __shfl_xor_sync(0xffffffffu, tot0, 1);
                tot1 += __shfl_xor_sync(0xffffffffu, tot1, 1);
                tot0 += __shfl_xor_sync(0xffffffffu, tot0, 2);
                tot1 += __shfl_xor_sync(0xffffffffu, tot1, 2);
                if (t == 0) {
                    dst[rho] = tot0;
                    dst[rho + 8] = tot1;
                }
                tot0 = tot1 = 0.0f;
            } else {
#pragma unroll
                for (int cb = 0; cb < CB; cb++) {  // lanes t and t ^ 1 hold the two digit pairs of the same vector
                    const float a0 = totv[cb][0] + __shfl_xor_sync(0xffffffffu, totv[cb][0], 1);
                    const float a1 = totv[cb][1] + __shfl_xor_sync(0xffffffffu, totv[cb][1], 1);
                    const int v = 2 * cb + (t >> 1);
                    if (my_h == 0 && v < NV) {
                        dst[v * SV_ROWS + rho] = a0;
                        dst[v * SV_ROWS + rho + 8] = a1;
                    }
                    totv[cb][0] = totv[cb][1] = 0.0f;
                }
            }
            if (tid == 0) slot_info[buf * SV_BATCH + slot] = make_int2(m, row0);
            if (++slot == BATCH && !flush()) {
                failed = true;
                break;
            }
        }
    }
    if (tid == 0) sv_trace(mb, 5);
    if (tid == 0 && mb.trace) mb.trace[(size_t)blockIdx.x * PHASE_TRACE_WORDS + 7] = (unsigned long long)wait_cycles;
    if (!failed && slot > 0 && !flush()) failed = true;
    if (tid == 0) sv_trace(mb, 6);
    if (failed && lane == 0) {
        *abort_flag = 1;
        atomicOr(mb.status, STATUS_TMA_TIMEOUT);
    }
}

// Stages of the ring and CTAs per SM for a given in_dim and number of vectors: two CTAs per SM when each can still
// hold three stages (and the kernel is built for two: one or two vectors).
void sv_plan(int in_dim, int n_vec, size_t smem_optin, int &n_stages, int &ctas_per_sm) {
    const size_t fixed = sv_fixed_bytes(in_dim, n_vec) + 1024;  // with the alignment slack
    const size_t half = smem_optin / 2 > 2048 ? smem_optin / 2 - 2048 : 0;  // room for the per-CTA reserve of the SM
    ctas_per_sm = 2;
    long long n = (n_vec <= 2 && half > fixed) ? (long long)((half - fixed) / SV_STAGE_BYTES) : 0;
    if (n < 3) {
        ctas_per_sm = 1;
        n = smem_optin > fixed ? (long long)((smem_optin - fixed) / SV_STAGE_BYTES) : 0;
    }
    n_stages = (int)(n > SV_MAX_STAGES ? SV_MAX_STAGES : n);
}

template <int NV>
cudaError_t launch_stream(MatvecBatch mb, const MatvecMaps *maps, const float *x, int in_dim, int n_sms, cudaStream_t stream,
                          int *grid_out) {
    if (!maps) return cudaErrorInvalidValue;
    static thread_local bool configured[64] = {false};  // per device: the opt-in is a host call of several microseconds
    static thread_local int optin[64];
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    if (!configured[dev]) {
        cudaError_t e = cudaDeviceGetAttribute(&optin[dev], cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
        if (e != cudaSuccess) return e;
        e = cudaFuncSetAttribute(dequant_matvec_4bit_stream_kernel<NV>, cudaFuncAttributeMaxDynamicSharedMemorySize, optin[dev]);
        if (e != cudaSuccess) return e;
        configured[dev] = true;
    }
    int n_stages = 0, ctas_per_sm = 1;
    sv_plan(in_dim, NV, (size_t)optin[dev], n_stages, ctas_per_sm);
    if (n_stages < 2 || !mb.sched || !mb.status) return cudaErrorInvalidValue;
    int tiles = 0;  // group_begin counts tiles of 16 rows per matrix
    for (int m = 0; m < mb.n_mat; m++) {
        mb.group_begin[m] = tiles;
        tiles += (mb.out_dim[m] + SV_ROWS - 1) / SV_ROWS;
    }
    mb.total_groups = tiles;
    mb.sb_bulk = in_dim % 512 == 0;  // rows of scales are then multiples of 16 bytes
    for (int m = 0; m < mb.n_mat; m++)
        if (((uintptr_t)mb.scales[m] | (uintptr_t)mb.biases[m]) & 15) mb.sb_bulk = 0;
    int grid = n_sms * ctas_per_sm;
    if (grid > tiles) grid = tiles;
    const size_t smem = 1024 + sv_fixed_bytes(in_dim, NV) + (size_t)n_stages * SV_STAGE_BYTES;  // 1 KiB: alignment slack
    if (grid_out) *grid_out = grid;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3((unsigned)((sv_warps(NV) + 1) * 32));
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr = {};
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;  // may start before the kernel ahead of it has drained
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = mb.overlap ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, dequant_matvec_4bit_stream_kernel<NV>, *maps, mb, x, in_dim, n_stages);
}

}  // namespace

size_t dequant_matvec_4bit_smem(int in_dim, int n_vec) {
    return 1024 + sv_fixed_bytes(in_dim, n_vec) + 2 * (size_t)SV_STAGE_BYTES;  // the least the ring works with
}

cudaError_t launch_dequant_matvec_4bit(MatvecBatch mb, const float *x, int in_dim, int n_vec, int n_sms,
                                       cudaStream_t stream, const MatvecMaps *maps, int *grid_out) {
    if (mb.n_mat < 1 || mb.n_mat > MATVEC_MAX_MATS) return cudaErrorInvalidValue;
    switch (n_vec) {
        case 1: return launch_stream<1>(mb, maps, x, in_dim, n_sms, stream, grid_out);
        case 2: return launch_stream<2>(mb, maps, x, in_dim, n_sms, stream, grid_out);
        case 3: return launch_stream<3>(mb, maps, x, in_dim, n_sms, stream, grid_out);
        case 4: return launch_stream<4>(mb, maps, x, in_dim, n_sms, stream, grid_out);
        case 5: return launch_stream<5>(mb, maps, x, in_dim, n_sms, stream, grid_out);
        case 6: return launch_stream<6>(mb, maps, x, in_dim, n_sms, stream, grid_out);
        case 7: return launch_stream<7>(mb, maps, x, in_dim, n_sms, stream, grid_out);
        case 8: return launch_stream<8>(mb, maps, x, in_dim, n_sms, stream, grid_out);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace mfc
