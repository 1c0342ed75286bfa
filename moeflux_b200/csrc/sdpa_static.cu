// Gated SDPA over a caller-held KV cache with NO allocation of any kind.
//
// Who needs this: code that may not call cudaMalloc at the point where it needs
// attention -- a plugin running inside another runtime's memory plan (every
// byte of device memory is accounted for by the host application and a hidden
// allocation can push it over its budget), a real-time or signal-handler-like
// path where a driver call that may block or fail on fragmentation is not
// acceptable, or a process that has already handed all free memory to its own
// pool allocator so that cudaMalloc would simply fail.  Such a caller owns the
// inputs and the output; the only thing the split-K decode kernel still needs
// is a place for its per-chunk partial results, its chunk counters and its item
// descriptor.  Here that place is a fixed array in the library's device image.
//
// The kernel is the same split-K flash-decoding kernel the contexts use
// (gqa_decode.cu / gqa_decode_f32.cu); only the scratch it is pointed at differs.
#include <math.h>
#include <stdio.h>
#include <string.h>

#include <mutex>
#include <string>

#include "../../include/moeflux_cuda.h"
#include "kernels.h"

using namespace mfc;

namespace {

// ---- fixed scratch -----------------------------------------------------------------
// Limits that size it (also declared in moeflux_cuda.h):
//   at most MFC_STATIC_MAX_KV_HEADS kv heads and MFC_STATIC_MAX_ROWS cached rows,
//   cut into at most STATIC_SLOTS (kv head, chunk) partials of 16 x 256 floats.
constexpr int STATIC_SLOTS = 256;
constexpr size_t OFF_TICKETS = 0;                                       // [MAX_KV_HEADS] unsigned
constexpr size_t OFF_STATUS = 256;                                      // 1 unsigned
constexpr size_t OFF_ITEM = 512;                                        // 1 GqaItem
constexpr size_t OFF_GROUP_TICKETS = 1024;                              // [SLOTS] unsigned
constexpr size_t OFF_M = 2048;                                          // [SLOTS][16] float
constexpr size_t OFF_L = OFF_M + sizeof(float) * STATIC_SLOTS * 16;     // [SLOTS][16] float
constexpr size_t OFF_O = OFF_L + sizeof(float) * STATIC_SLOTS * 16;     // [SLOTS][16][256] float
constexpr size_t SCRATCH_BYTES = OFF_O + sizeof(float) * STATIC_SLOTS * 16 * HEAD_DIM;  // ~4.03 MiB
static_assert(OFF_O % 256 == 0, "partials must stay 256-byte aligned");
static_assert(MFC_STATIC_MAX_KV_HEADS * sizeof(unsigned) <= 256, "ticket area too small");
static_assert(OFF_GROUP_TICKETS + STATIC_SLOTS * sizeof(unsigned) <= OFF_M, "group ticket area too small");

// Lives in the device image of every GPU that loads the library, until exit.
// In host code this name is only a handle for cudaGetSymbolAddress: it is NOT a
// device address and must never be handed to a kernel as one.
static __device__ __align__(256) unsigned char g_static_scratch[SCRATCH_BYTES];

// Start of a call, on the caller's stream: the item descriptor arrives by value (nothing is read from host memory
// when the kernel runs), the chunk counters start at zero, and the status word keeps only what earlier calls
// reported (mfc_sdpa_static_status reads and clears it).
__global__ void static_begin_kernel(unsigned char *scratch, GqaItem it) {
    unsigned *tickets = reinterpret_cast<unsigned *>(scratch + OFF_TICKETS);
    unsigned *group_tickets = reinterpret_cast<unsigned *>(scratch + OFF_GROUP_TICKETS);
    for (int i = threadIdx.x; i < MFC_STATIC_MAX_KV_HEADS; i += blockDim.x) tickets[i] = 0u;
    for (int i = threadIdx.x; i < STATIC_SLOTS; i += blockDim.x) group_tickets[i] = 0u;
    if (threadIdx.x == 0) *reinterpret_cast<GqaItem *>(scratch + OFF_ITEM) = it;
}

constexpr int MAX_DEVICES = 64;
std::mutex g_setup_mutex;
unsigned char *g_scratch_addr[MAX_DEVICES] = {nullptr};  // device address of the array, per device

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                  const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;

int fail(const std::string &msg) {
    no_ctx_error() = msg;  // read back with mfc_last_error(NULL)
    return -1;
}

// Once per device, with that device current: resolve the device address of the
// scratch array and raise the kernels' shared-memory limit.  Neither allocates.
int setup_device(int dev, unsigned char **addr_out) {
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (!g_scratch_addr[dev]) {
        unsigned char *ptr = nullptr;
        cudaError_t e = cudaGetSymbolAddress((void **)&ptr, g_static_scratch);
        if (e != cudaSuccess || !ptr)
            return fail(std::string("cudaGetSymbolAddress(scratch): ") + cudaGetErrorString(e));
        if ((e = gqa_decode_configure()) != cudaSuccess || (e = gqa_decode_f32_configure()) != cudaSuccess)
            return fail(std::string("cudaFuncSetAttribute: ") + cudaGetErrorString(e));
        if (!g_encode) {
            void *fn = nullptr;
            cudaDriverEntryPointQueryResult qres;
            e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
            if (e != cudaSuccess || !fn || qres != cudaDriverEntryPointSuccess)
                return fail("cuTensorMapEncodeTiled is not available from the driver");
            g_encode = (EncodeTiledFn)fn;
        }
        g_scratch_addr[dev] = ptr;
    }
    *addr_out = g_scratch_addr[dev];
    return 0;
}

int encode_map(CUtensorMap *map, const void *base, uint64_t rows, bool bf16) {
    cuuint64_t dims[2] = {(cuuint64_t)HEAD_DIM, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)(HEAD_DIM * (bf16 ? 2 : 4))};
    cuuint32_t box[2] = {(cuuint32_t)(bf16 ? 64 : 32), (cuuint32_t)(bf16 ? KV_TILE : KV_TILE_F32)};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = g_encode(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2,
                          const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail("cuTensorMapEncodeTiled failed, code " + std::to_string((int)r));
    return 0;
}

}  // namespace

#pragma GCC visibility push(default)
extern "C" {

int mfc_sdpa_static_dev(int32_t num_attn_heads, int32_t num_kv_heads, int32_t kv_dtype, int32_t kv_len,
                        int32_t cap_rows, const float *q, const float *gate, const void *k_cache,
                        const void *v_cache, float *out, void *stream_v) {
    if (!q || !k_cache || !v_cache || !out) return fail("NULL argument");
    if (num_attn_heads <= 0 || num_kv_heads <= 0 || num_attn_heads % num_kv_heads != 0 ||
        num_attn_heads / num_kv_heads > 16)
        return fail("bad head geometry: need num_attn_heads % num_kv_heads == 0 and a group of at most 16");
    if (num_kv_heads > MFC_STATIC_MAX_KV_HEADS)
        return fail("num_kv_heads " + std::to_string(num_kv_heads) + " exceeds the fixed scratch (at most " +
                    std::to_string(MFC_STATIC_MAX_KV_HEADS) + " kv heads); use a context instead");
    if (kv_dtype != MFC_KV_F32 && kv_dtype != MFC_KV_BF16) return fail("kv_dtype must be MFC_KV_F32 or MFC_KV_BF16");
    if (kv_len <= 0) return fail("kv_len must be > 0");
    if (kv_len > MFC_STATIC_MAX_ROWS)
        return fail("kv_len " + std::to_string(kv_len) + " exceeds the fixed scratch (at most " +
                    std::to_string(MFC_STATIC_MAX_ROWS) + " rows); use a context instead");
    if (cap_rows < kv_len) return fail("cap_rows is smaller than kv_len");
    if (((uintptr_t)k_cache & 15) || ((uintptr_t)v_cache & 15)) return fail("caches must be 16-byte aligned");
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return fail("no current CUDA device");
    unsigned char *scratch = nullptr;
    if (setup_device(dev, &scratch)) return -1;
    cudaStream_t stream = (cudaStream_t)stream_v;

    const bool bf16 = kv_dtype == MFC_KV_BF16;
    CUtensorMap kmap, vmap;
    const uint64_t rows = (uint64_t)num_kv_heads * cap_rows;
    if (encode_map(&kmap, k_cache, rows, bf16) || encode_map(&vmap, v_cache, rows, bf16)) return -1;

    // split: runs of equal tile counts over the heads' tiles, at most STATIC_SLOTS - num_kv_heads CTAs
    // (a slot per (head, CTA) pair) and at most MAX_UNIT_PARTS partials per head
    const int tile = bf16 ? KV_TILE : KV_TILE_F32;
    const int nt = (kv_len + tile - 1) / tile;
    const int total_tiles = nt * num_kv_heads;
    int w = (total_tiles + (STATIC_SLOTS - num_kv_heads) - 1) / (STATIC_SLOTS - num_kv_heads);
    if (w < 256 / tile) w = 256 / tile;
    const int w_split = (nt + (MAX_UNIT_PARTS - 2) - 1) / (MAX_UNIT_PARTS - 2);
    if (w < w_split) w = w_split;
    const int n_ctas = (total_tiles + w - 1) / w;
    GqaItem it;
    it.kv_slot = 0;
    it.local_len = kv_len;
    it.pos = 0;
    it.append_row = -1;
    it.tile_begin = 0;
    it.pad0 = it.pad1 = 0;
    it.in_idx = 0;
    if (n_ctas + num_kv_heads > STATIC_SLOTS) return fail("internal: split plan exceeds the fixed scratch");

    // The array keeps whatever the previous call left: the chunk counters and the
    // status word must start at zero.  (The partial slots are fully written before
    // they are read, so they need no clearing.)
    static_begin_kernel<<<1, 256, 0, stream>>>(scratch, it);
    e = cudaGetLastError();
    if (e != cudaSuccess) return fail(std::string("kernel launch: ") + cudaGetErrorString(e));

    GqaParams p;
    memset(&p, 0, sizeof(p));
    p.k_base = const_cast<void *>(k_cache);
    p.v_base = const_cast<void *>(v_cache);
    p.items = reinterpret_cast<const GqaItem *>(scratch + OFF_ITEM);
    p.n_items = 1;
    p.total_ctas = n_ctas;
    p.tiles_per_cta = w;
    p.total_tiles = total_tiles;
    p.q = q;
    p.gate = gate;
    p.k = nullptr;
    p.v = nullptr;
    p.out = out;
    p.sc_o = reinterpret_cast<float *>(scratch + OFF_O);
    p.sc_m = reinterpret_cast<float *>(scratch + OFF_M);
    p.sc_l = reinterpret_cast<float *>(scratch + OFF_L);
    p.tickets = reinterpret_cast<unsigned *>(scratch + OFF_TICKETS);
    p.group_tickets = reinterpret_cast<unsigned *>(scratch + OFF_GROUP_TICKETS);
    p.n_kv_slots = 1;
    p.inv_freq = nullptr;
    p.status = reinterpret_cast<unsigned *>(scratch + OFF_STATUS);
    p.H = num_attn_heads;
    p.Hkv = num_kv_heads;
    p.group = num_attn_heads / num_kv_heads;
    p.rotary_dim = 0;  // q and the cached K are already rotated
    p.cap_rows = cap_rows;
    p.partial_mode = 0;
    p.scale = 1.0f / sqrtf((float)HEAD_DIM);
    p.q_row_stride = HEAD_DIM;
    p.gate_row_stride = HEAD_DIM;
    p.po_item_stride = (size_t)num_attn_heads * HEAD_DIM;
    p.pml_item_stride = (size_t)num_attn_heads;
    p.n_seqs = 1;
    e = bf16 ? launch_gqa_decode_bf16(kmap, vmap, p, stream) : launch_gqa_decode_f32(kmap, vmap, p, stream);
    if (e != cudaSuccess) return fail(std::string("kernel launch: ") + cudaGetErrorString(e));
    return 0;
}

int mfc_sdpa_static_status(void *stream_v) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return fail("no current CUDA device");
    unsigned char *scratch = nullptr;
    if (setup_device(dev, &scratch)) return -1;
    cudaStream_t stream = (cudaStream_t)stream_v;
    unsigned st = 0;
    cudaError_t e = cudaMemcpyAsync(&st, scratch + OFF_STATUS, sizeof(st), cudaMemcpyDeviceToHost, stream);
    if (e == cudaSuccess) e = cudaMemsetAsync(scratch + OFF_STATUS, 0, sizeof(st), stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess) return fail(std::string("reading the status word: ") + cudaGetErrorString(e));
    if (st)
        return fail("a kernel of mfc_sdpa_static_dev gave up on a bounded wait or refused its work descriptor (device "
                    "status " + std::to_string(st) + "): outputs written since the last status call are not valid");
    return 0;
}

}  // extern "C"
#pragma GCC visibility pop
