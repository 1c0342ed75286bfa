// Context, state layer and C ABI of the attention backend.
//
// Owns what the reference keeps in `KvCache` / `LinearAttnState`
// (crates/moeflux/src/riir/state.rs:37-74, 336-362) and in the GPU mirrors of
// `LayerForwardBuffers` (crates/moeflux/src/riir/linear_attn_forward.rs:180-304),
// laid out for the sm_100a kernels:
//
//   K, V cache   [kv slot = full layer * n_seqs + seq][kv head][row][256]  bf16 or fp32
//                a (slot, head) is one contiguous run of rows, so a KV tile is a
//                2-D TMA box and a chunk of a head is a plain row range;
//   ssm state    [state slot = linear layer * n_seqs + seq][v head][128][128] fp32
//                (the reference's own order, value-major, key fastest);
//   conv ring    [state slot][4][conv_dim] fp32 (4-slot ring instead of a shifted
//                3-row history, see gdn_decode.cu).
//
// One extra slot of each kind at the end serves the stateless parity hooks.
// Lengths and ring positions live on the host; kernels receive them per item.
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <deque>
#include <map>
#include <string>
#include <vector>

#include "../../include/moeflux_cuda.h"
#include "kernels.h"

using namespace mfc;

namespace {

thread_local std::string g_open_error;

constexpr uint32_t SNAPSHOT_MAGIC = 0x4D464C58u;  // 'MFLX', state_snapshot.rs:55-57

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                  const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

}  // namespace

// Message slot of failures that have no context to attach to (mfc_open and the
// context-free entry points); read back through mfc_last_error(NULL).
namespace mfc {
std::string &no_ctx_error() { return g_open_error; }
}  // namespace mfc

struct mfc_ctx {
    mfc_config cfg;
    int n_full = 0, n_lin = 0;
    std::vector<int> layer_to_full, layer_to_lin;
    int group = 0;
    int cap_rows = 0;  // rows per (kv slot, kv head)
    int conv_dim = 0;
    int n_kv_slots = 0, n_state_slots = 0;
    size_t kv_esize = 4;
    cudaStream_t stream = nullptr;
    bool owns_stream = true;
    cudaStream_t side_stream = nullptr;  // second queue of mfc_eval_token_attn
    cudaEvent_t ev_fork = nullptr, ev_join = nullptr, ev_gate = nullptr;

    void *k_cache = nullptr, *v_cache = nullptr;
    CUtensorMap kmap, vmap;
    CUtensorMap kmap_pf, vmap_pf;  // same caches, 64-row boxes for the prefill kernel (bf16 cache only)
    float *pf_cos_sin = nullptr;   // [max_seq][32] (cos, sin) of the tokens of a prefill call
    // GatedDeltaNet prefill scratch, max_prefill tokens
    void *pf_q = nullptr, *pf_k = nullptr, *pf_wt = nullptr, *pf_wm = nullptr;
    float *pf_v = nullptr, *pf_lg = nullptr, *pf_beta = nullptr;
    float *ssm = nullptr, *conv = nullptr;
    uint16_t *conv_w = nullptr, *dt_bias = nullptr, *norm_w = nullptr;
    float *a_log = nullptr;
    float *inv_freq = nullptr;
    uint16_t *qnorm_w = nullptr, *knorm_w = nullptr;  // [n_full][256] bf16, optional per-head norm weights
    std::vector<uint8_t> full_norm_set;
    float *st_qproj = nullptr;                        // staging of interleaved q|gate rows

    std::vector<int32_t> kv_len;     // [n_full * n_seqs + 1] whole-sequence lengths
    std::vector<int64_t> conv_step;  // [n_state_slots]
    std::vector<uint8_t> lin_weights_set;

    GqaItem *d_gqa_items = nullptr;
    GdnItem *d_gdn_items = nullptr;
    std::vector<GqaItem> h_gqa_items;
    std::vector<GdnItem> h_gdn_items;
    // Item lists travel through a small ring of pinned host slots: a copy from pageable memory is staged by the
    // driver and blocks the calling thread, a copy from pinned memory is queued like a kernel.
    static constexpr int PIN_SLOTS = 8;
    uint8_t *pin_items = nullptr;
    size_t pin_slot_bytes = 0;
    cudaEvent_t pin_ev[PIN_SLOTS] = {};
    bool pin_used[PIN_SLOTS] = {};
    unsigned pin_next = 0;
    float *sc_o = nullptr, *sc_m = nullptr, *sc_l = nullptr;
    unsigned *tickets = nullptr, *group_tickets = nullptr, *status = nullptr;
    unsigned *mv_sched = nullptr;  // two pairs (tile counter, finished CTAs) of the one-vector projection kernel, used in turn
    unsigned mv_launches = 0;
    bool mv_overlap = true;        // tuning "matvec_overlap"
    struct MvMap {
        const uint32_t *w;
        const uint16_t *scales, *biases;
        int in_dim, out_dim;
        CUtensorMap map, sc_map, bi_map;
    };
    static constexpr size_t MV_MAP_CACHE = 256;
    std::vector<MvMap> mv_maps;  // tensor maps of the weight matrices seen last (one-vector projection kernel)
    int max_parts = 0;
    // every device allocation of the context, with a band of 0xFF bytes on either side (mfc_check_guards)
    struct Alloc {
        uint8_t *base;
        size_t bytes;  // user bytes between the bands
        const char *name;
        bool banded;   // false: a plain allocation (the exchange buffer, whose IPC handle names it from its base)
    };
    std::vector<Alloc> allocs;
    static constexpr size_t GUARD = 4096;
    // diagnostics
    unsigned gqa_wait_spins = 0;
    int gqa_inject_lost_load = 0;
    int mv_inject_lost_load = 0;
    unsigned long long *phase_trace = nullptr;  // [MAX_TRACE_CTAS][PHASE_TRACE_WORDS]
    static constexpr int MAX_TRACE_CTAS = 1024;
    bool phase_trace_on = false;
    int last_launch_ctas = 0;
    // fused exchange of the KV-sequence split (mfc_exchange_*)
    struct Exchange {
        uint8_t *base = nullptr;        // one allocation: [2][world][npr][item floats] receive blocks, then flags
        float *recv = nullptr;
        unsigned *flags = nullptr;      // [world], written by the peers
        size_t bytes = 0, recv_bytes = 0;
        int npr = 0;                    // items this rank finishes per step
        std::vector<uint8_t *> peer_base;   // this process's mapping of every rank's allocation
        std::vector<bool> peer_is_ipc;
        float **d_peer_recv = nullptr;      // device [2][world]
        unsigned **d_peer_flags = nullptr;  // device [world]
        unsigned *done_counter = nullptr;
        unsigned step = 0;              // steps issued so far (flag value of the latest one)
        bool connected = false;
        // gather of the query rows over the links (tuning "exchange_gather_q"): every rank receives from the host the
        // rows of the items it finishes only and stores them into every peer's copy of the step's row table
        float *q_rows = nullptr;            // [2][world * npr][q_dim], in the shared allocation after the flags
        unsigned *q_flags = nullptr;        // [world], written by the peers: rows of step n have landed
        float **d_peer_q = nullptr;         // device [2][world]: every rank's two row tables
        unsigned **d_peer_q_flags = nullptr;  // device [world]
        unsigned *q_done_counter = nullptr;
        bool gather_q = false;
        bool shares_device = false;         // a peer context lives on this context's GPU (tests in one process)
    } xc;
    static constexpr size_t XC_FLAG_BYTES = 512;  // one flag array: up to 128 ranks
    int plan_tiles_per_cta = 1, plan_total_tiles = 0;  // split of the launch being built
    int plan_max_parts = 1;                            // most CTAs that share one unit in it
    int coop_capacity = 0;                             // CTAs of the decode kernel the device holds at once
    bool gqa_coop = true;                              // merge widely shared units cooperatively when possible
    int gqa_coop_min_parts = 32;                       // ... when some unit is shared by more CTAs than this

    // device staging for the host-pointer entry points (max_batch items)
    float *st_q = nullptr, *st_gate = nullptr, *st_k = nullptr, *st_v = nullptr, *st_out = nullptr;
    float *st_qkv = nullptr, *st_z = nullptr, *st_alpha = nullptr, *st_beta = nullptr, *st_gout = nullptr;
    float *st_rows = nullptr;  // snapshot / hook staging, SNAP_ROWS wire rows
    static constexpr int SNAP_ROWS = 4096;

    // Per-sequence store of snapshots keyed by position (crates/moeflux/src/riir/mod.rs:2015-2087)
    std::vector<std::map<int32_t, std::vector<uint8_t>>> checkpoints;
    std::vector<std::deque<int32_t>> checkpoint_order;  // least recently stored first
    size_t max_checkpoints = 4;                         // DEFAULT_MAX_CHECKPOINTS, mod.rs:108

    bool gdn_side = false;  // issue GatedDeltaNet _dev launches on the side queue (joined by mfc_join)
    bool side_pending = false;
    int gdn_rows = 0;  // 0: chosen per launch from the item count
    int gqa_target_ctas = 0;  // 0: wave-aware plan; > 0: aim for this many CTAs per launch
    int gqa_slots = 296;      // CTAs resident at once (2 per SM)
    int n_sms = 148;
    size_t smem_optin = 227 * 1024;
    int gqa_forced_chunk = 0;
    int gqa_min_rows = 64;         // least cache rows per CTA
    bool gqa_unit_aligned = false;  // one CTA per unit when equal-length units nearly fill the wave (off: see the planner)
    bool gqa_align_units = true;    // few units on a full wave: whole CTA runs per unit (tuning "gqa_align_units")
    long long launches = 0;
    std::string err;
};

namespace {

bool fail(mfc_ctx *c, const std::string &msg) {
    if (c) c->err = msg;
    else g_open_error = msg;
    return false;
}
#define CK(call)                                                                          \
    do {                                                                                  \
        cudaError_t e_ = (call);                                                          \
        if (e_ != cudaSuccess) {                                                          \
            fail(c, std::string(#call) + ": " + cudaGetErrorString(e_));                  \
            return -1;                                                                    \
        }                                                                                 \
    } while (0)

inline bool is_full_layer(const mfc_config &g, int i) { return (i + 1) % g.full_attn_interval == 0; }

// rows of a sequence of whole length `len` stored by rank r of a block-cyclic split
int local_len_of(int len, int r, int W, int B) {
    if (W <= 1) return len;
    const int full_blocks = len / B, rem = len % B;
    int cnt = (full_blocks / W) * B;
    const int part = full_blocks % W;
    if (part > r) cnt += B;
    else if (part == r) cnt += rem;
    return cnt;
}
// local row of whole-sequence position p, or -1 when another rank owns it
int local_row_of(int p, int r, int W, int B) {
    if (W <= 1) return p;
    const int blk = p / B;
    if (blk % W != r) return -1;
    return (blk / W) * B + p % B;
}

// Device allocation with a band of GUARD bytes of 0xFF before and after the user range.  Kernels never write
// there; mfc_check_guards() verifies that they did not (evidence of in-bounds writes where no memory checker runs).
template <typename T>
bool dalloc(mfc_ctx *c, T **p, size_t n, bool zero, const char *name = "buffer") {
    if (n == 0) n = 1;
    const size_t bytes = (n * sizeof(T) + 255) & ~(size_t)255;
    uint8_t *base = nullptr;
    cudaError_t e = cudaMalloc((void **)&base, bytes + 2 * mfc_ctx::GUARD);
    if (e != cudaSuccess) return fail(c, std::string("cudaMalloc(") + name + "): " + cudaGetErrorString(e));
    c->allocs.push_back({base, bytes, name, true});
    e = cudaMemset(base, 0xFF, mfc_ctx::GUARD);
    if (e == cudaSuccess) e = cudaMemset(base + mfc_ctx::GUARD + bytes, 0xFF, mfc_ctx::GUARD);
    if (e == cudaSuccess && zero) e = cudaMemset(base + mfc_ctx::GUARD, 0, bytes);
    if (e != cudaSuccess) return fail(c, std::string("cudaMemset: ") + cudaGetErrorString(e));
    *p = reinterpret_cast<T *>(base + mfc_ctx::GUARD);
    return true;
}

// 2-D map over a row-major [rows][cols] array; with the 128-byte swizzle box_cols * esize must be 128.
bool make_map_2d(mfc_ctx *c, CUtensorMap *map, void *base, CUtensorMapDataType dtype, int esize, uint64_t cols,
                 uint64_t rows, int box_cols, int box_rows, bool swizzle128 = true) {
    void *fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
    if (e != cudaSuccess || !fn || qres != cudaDriverEntryPointSuccess)
        return fail(c, "cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)(cols * esize)};
    cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = ((EncodeTiledFn)fn)(map, dtype, 2, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                     swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(c, "cuTensorMapEncodeTiled failed, code " + std::to_string((int)r));
    return true;
}

bool make_tensor_map(mfc_ctx *c, CUtensorMap *map, void *base, uint64_t rows, int box_rows = 0) {
    void *fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
    if (e != cudaSuccess || !fn || qres != cudaDriverEntryPointSuccess)
        return fail(c, "cuTensorMapEncodeTiled is not available from the driver");
    const bool bf16 = c->cfg.kv_dtype == MFC_KV_BF16;
    cuuint64_t dims[2] = {(cuuint64_t)HEAD_DIM, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)(HEAD_DIM * c->kv_esize)};
    cuuint32_t box[2] = {(cuuint32_t)(bf16 ? 64 : 32), (cuuint32_t)(box_rows ? box_rows : (bf16 ? KV_TILE : KV_TILE_F32))};  // 128-byte inner extent
    cuuint32_t estr[2] = {1, 1};
    CUresult r = ((EncodeTiledFn)fn)(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32,
                                     2, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(c, "cuTensorMapEncodeTiled failed, code " + std::to_string((int)r));
    return true;
}

void free_all(mfc_ctx *c) {
    for (size_t r = 0; r < c->xc.peer_base.size(); r++)
        if (c->xc.peer_base[r] && c->xc.peer_is_ipc[r]) cudaIpcCloseMemHandle(c->xc.peer_base[r]);
    for (const mfc_ctx::Alloc &a : c->allocs) cudaFree(a.base);
    c->allocs.clear();
    if (c->pin_items) cudaFreeHost(c->pin_items);
    for (cudaEvent_t e : c->pin_ev)
        if (e) cudaEventDestroy(e);
    if (c->stream && c->owns_stream) cudaStreamDestroy(c->stream);
    if (c->side_stream) cudaStreamDestroy(c->side_stream);
    if (c->ev_fork) cudaEventDestroy(c->ev_fork);
    if (c->ev_join) cudaEventDestroy(c->ev_join);
    if (c->ev_gate) cudaEventDestroy(c->ev_gate);
}

// Queues the copy of an item list to the device through the next pinned slot.
int upload_items(mfc_ctx *c, void *dst, const void *src, size_t bytes, cudaStream_t stream) {
    if (bytes > c->pin_slot_bytes) {
        fail(c, "internal: item list larger than a staging slot");
        return -1;
    }
    const int slot = (int)(c->pin_next++ % mfc_ctx::PIN_SLOTS);
    if (c->pin_used[slot]) CK(cudaEventSynchronize(c->pin_ev[slot]));  // the copy that last read this slot
    uint8_t *h = c->pin_items + (size_t)slot * c->pin_slot_bytes;
    memcpy(h, src, bytes);
    CK(cudaMemcpyAsync(dst, h, bytes, cudaMemcpyHostToDevice, stream));
    CK(cudaEventRecord(c->pin_ev[slot], stream));
    c->pin_used[slot] = true;
    return 0;
}

int check_status(mfc_ctx *c) {
    unsigned st = 0;
    if (c->side_pending) {
        CK(cudaStreamWaitEvent(c->stream, c->ev_join, 0));
        c->side_pending = false;
    }
    CK(cudaMemcpyAsync(&st, c->status, sizeof(st), cudaMemcpyDeviceToHost, c->stream));
    CK(cudaStreamSynchronize(c->stream));
    if (st) {
        // the counters of the split-K merge return to zero by themselves (a CTA that gives up still takes its
        // tickets); they are cleared all the same, with the status word, so that the context stays usable
        cudaMemsetAsync(c->status, 0, sizeof(unsigned), c->stream);
        cudaMemsetAsync(c->tickets, 0, sizeof(unsigned) * (size_t)c->cfg.max_batch * c->cfg.num_kv_heads, c->stream);
        cudaMemsetAsync(c->group_tickets, 0, sizeof(unsigned) * (size_t)c->max_parts, c->stream);
        cudaMemsetAsync(c->mv_sched, 0, 4 * sizeof(unsigned), c->stream);
        if (c->xc.done_counter) cudaMemsetAsync(c->xc.done_counter, 0, sizeof(unsigned), c->stream);
        if (c->xc.q_done_counter) cudaMemsetAsync(c->xc.q_done_counter, 0, sizeof(unsigned), c->stream);
        cudaStreamSynchronize(c->stream);
        std::string what;
        if (st & 1u) what += " a load did not arrive within the wait limit;";
        if (st & 2u) what += " an item failed its range checks;";
        if (st & 4u) what += " a peer's partials did not arrive within the wait limit;";
        if (st & 8u) what += " the CTAs that share a unit did not all arrive within the wait limit;";
        fail(c, "a kernel gave up (device status " + std::to_string(st) + ":" + what +
                    ") the results since the last synchronisation are not valid");
        return -1;
    }
    return 0;
}

// ---- item list construction ---------------------------------------------------------

// Work split of one launch ("stream-K" over KV tiles).  The tiles of all (item, kv
// head) units form one sequence; it is cut into equal runs of `tiles_per_cta` tiles,
// one CTA each, across unit boundaries, so that one wave of CTAs (2 per SM) carries
// the whole launch with equal work per CTA.  A unit cut by a run boundary is merged
// from the partials of the CTAs that share it.  Constraints: at least gqa_min_rows
// rows per CTA, at most MAX_UNIT_PARTS partials per unit.
int plan_tiles_per_cta(const mfc_ctx *c, long long total_tiles, int max_unit_tiles, int min_unit_tiles = 0,
                       long long n_units = 0) {
    const int tile = c->cfg.kv_dtype == MFC_KV_BF16 ? KV_TILE : KV_TILE_F32;
    long long w;
    if (c->gqa_forced_chunk > 0) {
        w = (c->gqa_forced_chunk + tile - 1) / tile;
    } else {
        const long long ctas = c->gqa_target_ctas > 0 ? c->gqa_target_ctas : c->gqa_slots;
        w = (total_tiles + ctas - 1) / ctas;
        // A launch too small to give every CTA of the wave a long run (a single sequence, a few short ones) is bound
        // by latency, not by bandwidth: it is spread over as many SMs as runs of gqa_min_rows rows allow.
        const long long w_min = c->gqa_min_rows / tile;
        if (w < w_min) w = w_min;
        // Optional (tuning "gqa_unit_aligned", off by default): units of equal length that nearly fill the wave by
        // themselves get one CTA each.  No unit is shared, so nothing is parked or merged and every CTA builds its
        // query fragments once.  Measured: 2 % faster on short bursts of 0.6 ms launches, 7-15 % slower on sustained
        // 4.7 ms launches, where the SMs that hold two CTAs set the pace and fewer, longer runs lose.
        if (c->gqa_target_ctas == 0 && c->gqa_unit_aligned && n_units > 0 && min_unit_tiles == max_unit_tiles &&
            n_units <= ctas && n_units * 10 >= ctas * 7 && max_unit_tiles >= w)
            w = max_unit_tiles;
    }
    const long long w_split = (max_unit_tiles + (MAX_UNIT_PARTS - 2) - 1) / (MAX_UNIT_PARTS - 2);
    if (w < w_split) w = w_split;
    if (w < 1) w = 1;
    return (int)w;
}

// Validates the items, advances the lengths and fills c->h_gqa_items.
// kv_slot_override >= 0 selects the hook slot (no append, explicit length).
int build_gqa_items(mfc_ctx *c, int n, const int32_t *layers, const int32_t *seq_ids,
                    const int32_t *pos, int *total_ctas) {
    const mfc_config &g = c->cfg;
    if (n <= 0 || n > g.max_batch) {
        fail(c, "item count must be in [1, max_batch]");
        return -1;
    }
    if (!layers || !seq_ids || !pos) {
        fail(c, "NULL argument");
        return -1;
    }
    for (int i = 0; i < n; i++) {
        const int l = layers[i], s = seq_ids[i];
        if (l < 0 || l >= g.num_layers || !is_full_layer(g, l)) {
            fail(c, "layer " + std::to_string(l) + " is not a full-attention layer");
            return -1;
        }
        if (s < 0 || s >= g.n_seqs) {
            fail(c, "seq_id out of range");
            return -1;
        }
        const int slot = c->layer_to_full[l] * g.n_seqs + s;
        if (pos[i] < 0 || pos[i] != c->kv_len[slot]) {
            fail(c, "pos " + std::to_string(pos[i]) + " != current length " +
                        std::to_string(c->kv_len[slot]) + " of layer " + std::to_string(l));
            return -1;
        }
        if (pos[i] + 1 > g.max_seq) {
            fail(c, "kv cache overflow");
            return -1;
        }
    }
    c->h_gqa_items.resize(n);
    for (int i = 0; i < n; i++) {
        GqaItem &it = c->h_gqa_items[i];
        const int slot = c->layer_to_full[layers[i]] * g.n_seqs + seq_ids[i];
        it.kv_slot = slot;
        it.pos = pos[i];
        it.local_len = local_len_of(pos[i] + 1, g.kv_rank, g.kv_world, g.kv_block);
        it.append_row = local_row_of(pos[i], g.kv_rank, g.kv_world, g.kv_block);
        it.in_idx = i;
    }
    const int tile = g.kv_dtype == MFC_KV_BF16 ? KV_TILE : KV_TILE_F32;
    long long total_tiles = 0;
    int max_unit_tiles = 1, min_unit_tiles = 1 << 30;
    for (int i = 0; i < n; i++) {
        GqaItem &it = c->h_gqa_items[i];
        const int nt = it.local_len > 0 ? (it.local_len + tile - 1) / tile : 1;
        it.tile_begin = (int32_t)total_tiles;
        it.pad0 = it.pad1 = 0;
        total_tiles += (long long)nt * g.num_kv_heads;
        if (nt > max_unit_tiles) max_unit_tiles = nt;
        if (nt < min_unit_tiles) min_unit_tiles = nt;
    }
    if (total_tiles >= (1ll << 31)) {
        fail(c, "too many KV tiles in one launch");
        return -1;
    }
    c->plan_tiles_per_cta = plan_tiles_per_cta(c, total_tiles, max_unit_tiles, min_unit_tiles, (long long)n * g.num_kv_heads);
    c->plan_total_tiles = (int)total_tiles;
    c->plan_max_parts = (max_unit_tiles + c->plan_tiles_per_cta - 1) / c->plan_tiles_per_cta + 1;
    // A few long units on a full wave (a ragged batch of 8-32 sequences): runs that cross unit boundaries give one
    // CTA in ten a second segment -- a second prologue, a parked partial, a fence under full load -- and those CTAs
    // finish 30-45 us after the rest.  With few units it is cheaper to give every unit whole CTAs: the run length T
    // grows until sum ceil(tiles / T) fits the wave, every unit is padded to whole runs (half a run wasted per unit on
    // average) and no CTA has a second segment.  Taken when that waste costs less than the tail it removes.
    const long long n_units = (long long)n * g.num_kv_heads;
    if (c->gqa_align_units && c->gqa_target_ctas == 0 && c->gqa_forced_chunk == 0 && n_units * 4 <= c->gqa_slots) {
        const long long w_min = c->gqa_min_rows / tile;
        long long T = (total_tiles + c->gqa_slots - 1) / c->gqa_slots;
        if (T < w_min) T = w_min;
        const long long w_split = (max_unit_tiles + (MAX_UNIT_PARTS - 2) - 1) / (MAX_UNIT_PARTS - 2);
        if (T < w_split) T = w_split;
        long long runs = 0;
        for (;; T++) {
            runs = 0;
            for (int i = 0; i < n; i++) {
                const GqaItem &it = c->h_gqa_items[i];
                const long long nt = it.local_len > 0 ? (it.local_len + tile - 1) / tile : 1;
                runs += ((nt + T - 1) / T) * g.num_kv_heads;
            }
            if (runs <= c->gqa_slots) break;
        }
        const long long tile_bytes = 2ll * tile * HEAD_DIM * c->kv_esize;
        if (T * n_units * tile_bytes < 520000000ll) {  // waste (units / 2 runs) under 40 us of a CTA's stream at 22 GB/s
            long long tb = 0;
            for (int i = 0; i < n; i++) {
                GqaItem &it = c->h_gqa_items[i];
                const long long nt = it.local_len > 0 ? (it.local_len + tile - 1) / tile : 1;
                const long long padded = ((nt + T - 1) / T) * T;
                it.tile_begin = (int32_t)tb;
                it.pad0 = (int32_t)padded;
                tb += padded * g.num_kv_heads;
            }
            total_tiles = tb;
            c->plan_tiles_per_cta = (int)T;
            c->plan_total_tiles = (int)tb;
            c->plan_max_parts = (int)((max_unit_tiles + T - 1) / T);
        }
    }
    const int cta = (int)((total_tiles + c->plan_tiles_per_cta - 1) / c->plan_tiles_per_cta);
    if (cta + n * g.num_kv_heads > c->max_parts) {
        fail(c, "internal: split plan exceeds the scratch reserved at open");
        return -1;
    }
    for (int i = 0; i < n; i++) c->kv_len[c->layer_to_full[layers[i]] * g.n_seqs + seq_ids[i]] += 1;
    *total_ctas = cta;
    return 0;
}

void fill_gqa_params(mfc_ctx *c, GqaParams &p, int n, int total_ctas) {
    const mfc_config &g = c->cfg;
    memset(&p, 0, sizeof(p));
    p.k_base = c->k_cache;
    p.v_base = c->v_cache;
    p.items = c->d_gqa_items;
    p.n_items = n;
    p.total_ctas = total_ctas;
    p.tiles_per_cta = c->plan_tiles_per_cta;
    p.total_tiles = c->plan_total_tiles;
    p.sc_o = c->sc_o;
    p.sc_m = c->sc_m;
    p.sc_l = c->sc_l;
    p.tickets = c->tickets;
    p.group_tickets = c->group_tickets;
    p.n_kv_slots = c->n_kv_slots;
    // a unit shared by very many CTAs (a lone long sequence: the launch is at most four units' worth of CTAs) is merged
    // by its sharers together, which needs every CTA of the grid resident: a cooperative launch, when the grid fits
    // the device.  Moderately shared units (a ragged batch of several sequences) keep the ordinary launch and the
    // two-level merge: a cooperative launch cannot start
    // while another kernel (a collective, the GatedDeltaNet launch on the second queue) holds part of an SM.
    p.coop_merge = c->gqa_coop && c->plan_max_parts > c->gqa_coop_min_parts && c->plan_max_parts * 4 >= total_ctas &&
                   total_ctas <= c->coop_capacity;
    p.wait_spins = c->gqa_wait_spins;
    p.inject_lost_load = c->gqa_inject_lost_load;
    p.phase_trace = (c->phase_trace_on && total_ctas <= mfc_ctx::MAX_TRACE_CTAS) ? c->phase_trace : nullptr;
    c->last_launch_ctas = total_ctas;
    p.inv_freq = c->inv_freq;
    p.status = c->status;
    p.H = g.num_attn_heads;
    p.Hkv = g.num_kv_heads;
    p.group = c->group;
    p.rotary_dim = g.rotary_dim;
    p.cap_rows = c->cap_rows;
    p.scale = 1.0f / sqrtf((float)g.head_dim);
    p.q_row_stride = HEAD_DIM;
    p.gate_row_stride = HEAD_DIM;
    p.po_item_stride = (size_t)g.num_attn_heads * HEAD_DIM;
    p.pml_item_stride = (size_t)g.num_attn_heads;
    p.n_seqs = g.n_seqs;
    p.norm_eps = g.rms_norm_eps;
}

int launch_gqa(mfc_ctx *c, GqaParams &p) {
    if (p.n_items <= GQA_INLINE_ITEMS) {  // up to 128 items travel as kernel parameters: no copy before the launch
        p.items = nullptr;
        for (int i = 0; i < p.n_items; i++) p.inline_items[i] = c->h_gqa_items[i];
    } else if (upload_items(c, c->d_gqa_items, c->h_gqa_items.data(), sizeof(GqaItem) * p.n_items, c->stream)) {
        return -1;
    }
    if (c->cfg.kv_dtype == MFC_KV_BF16) CK(launch_gqa_decode_bf16(c->kmap, c->vmap, p, c->stream));
    else CK(launch_gqa_decode_f32(c->kmap, c->vmap, p, c->stream));
    c->launches += 1;
    return 0;
}

int build_gdn_items(mfc_ctx *c, int n, const int32_t *layers, const int32_t *seq_ids) {
    const mfc_config &g = c->cfg;
    if (n <= 0 || n > g.max_batch) {
        fail(c, "item count must be in [1, max_batch]");
        return -1;
    }
    if (!layers || !seq_ids) {
        fail(c, "NULL argument");
        return -1;
    }
    for (int i = 0; i < n; i++) {
        const int l = layers[i], s = seq_ids[i];
        if (l < 0 || l >= g.num_layers || is_full_layer(g, l)) {
            fail(c, "layer " + std::to_string(l) + " is not a linear-attention layer");
            return -1;
        }
        if (s < 0 || s >= g.n_seqs) {
            fail(c, "seq_id out of range");
            return -1;
        }
        if (!c->lin_weights_set[c->layer_to_lin[l]]) {
            fail(c, "mfc_set_linear_weights was not called for layer " + std::to_string(l));
            return -1;
        }
    }
    c->h_gdn_items.resize(n);
    for (int i = 0; i < n; i++) {
        const int ll = c->layer_to_lin[layers[i]];
        const int slot = ll * g.n_seqs + seq_ids[i];
        GdnItem &it = c->h_gdn_items[i];
        it.w_layer = ll;
        it.state_idx = slot;
        it.slot = (int)(c->conv_step[slot] & 3);
        it.pad = 0;
        c->conv_step[slot] += 1;
    }
    return 0;
}

int launch_gdn(mfc_ctx *c, int n, const float *qkv, const float *z, const float *alpha,
               const float *beta, float *out) {
    const mfc_config &g = c->cfg;
    GdnParams p;
    memset(&p, 0, sizeof(p));
    p.ssm_base = c->ssm;
    p.conv_base = c->conv;
    p.conv_w = c->conv_w;
    p.a_log = c->a_log;
    p.dt_bias = c->dt_bias;
    p.norm_w = c->norm_w;
    p.items = c->d_gdn_items;
    p.qkv = qkv;
    p.z = z;
    p.alpha = alpha;
    p.beta = beta;
    p.out = out;
    p.n_items = n;
    p.Hv = g.linear_num_v_heads;
    p.Hk = g.linear_num_k_heads;
    p.conv_dim = c->conv_dim;
    p.eps = g.rms_norm_eps;
    if (n <= INLINE_ITEMS) {  // up to 64 items travel as kernel parameters: no copy before the launch
        p.items = nullptr;
        for (int i = 0; i < n; i++) p.inline_items[i] = c->h_gdn_items[i];
    } else if (upload_items(c, c->d_gdn_items, c->h_gdn_items.data(), sizeof(GdnItem) * n, c->stream)) {
        return -1;
    }
    // Whole heads per CTA (128 rows) amortise the conv/norm prologue best; smaller
    // blocks only when the launch would otherwise leave SMs without work.
    int rows = c->gdn_rows;
    if (rows == 0) {
        const long long heads = (long long)n * g.linear_num_v_heads;
        rows = heads >= 2 * 592 ? 128 : (heads >= 592 ? 64 : 32);
    }
    CK(launch_gdn_decode(p, rows, c->stream));
    c->launches += 1;
    return 0;
}

// Validation of an 'MFLX' snapshot against a geometry without touching any
// state: header (crates/moeflux/src/riir/state_snapshot.rs:377-440) and the
// body walk (:445-507).  Returns the bytes the snapshot occupies, or -1 with
// the reason in `why`.
long long snapshot_preflight(const mfc_config &g, const uint8_t *in, size_t buf_len, size_t *hbytes_out,
                             std::string &why) {
    const int conv_dim = 2 * g.linear_num_k_heads * GDN_DIM + g.linear_num_v_heads * GDN_DIM;
    // header, crates/moeflux/src/riir/state_snapshot.rs:377-440
    if (buf_len < 8) {
        why = ("snapshot truncated: no header");
        return -1;
    }
    uint32_t w[10] = {0};
    memcpy(w, in, 8);
    if (w[0] != SNAPSHOT_MAGIC) {
        why = ("snapshot magic mismatch");
        return -1;
    }
    if (w[1] != 1 && w[1] != 2) {
        why = ("snapshot version " + std::to_string(w[1]) + " not understood");
        return -1;
    }
    const size_t hbytes = (w[1] == 1 ? 8 : 10) * sizeof(uint32_t);
    *hbytes_out = hbytes;
    if (buf_len < hbytes) {
        why = ("snapshot truncated: short header");
        return -1;
    }
    memcpy(w, in, hbytes);
    const uint32_t la_conv = (uint32_t)((CONV_TAPS - 1) * conv_dim * sizeof(float));
    const uint32_t la_ssm = (uint32_t)((size_t)g.linear_num_v_heads * GDN_DIM * GDN_DIM * sizeof(float));
    const uint32_t want[10] = {SNAPSHOT_MAGIC, w[1], (uint32_t)g.num_layers, (uint32_t)g.full_attn_interval,
                               (uint32_t)g.num_kv_heads, (uint32_t)g.head_dim, la_conv, la_ssm, 0u, 0u};
    static const char *names[10] = {"magic", "version", "num_layers", "full_attn_interval", "num_kv_heads",
                                    "head_dim", "linear_conv_bytes", "linear_ssm_bytes", "kv_lora_rank",
                                    "qk_rope_head_dim"};
    for (size_t i = 2; i < hbytes / 4; i++)
        if (w[i] != want[i]) {
            why = (std::string("snapshot shape mismatch on field '") + names[i] + "'");
            return -1;
        }
    // preflight: walk the body without touching any state (state_snapshot.rs:445-507)
    const size_t fa_stride = (size_t)g.num_kv_heads * HEAD_DIM * sizeof(float);
    {
        size_t q = hbytes;
        for (int i = 0; i < g.num_layers; i++) {
            if (is_full_layer(g, i)) {
                if (buf_len - q < 4) {
                    why = ("snapshot truncated at layer " + std::to_string(i));
                    return -1;
                }
                int32_t len;
                memcpy(&len, in + q, 4);
                q += 4;
                if (len < 0) {
                    why = ("snapshot layer " + std::to_string(i) + " has a negative KV length");
                    return -1;
                }
                if (len > g.max_seq) {
                    why = ("snapshot layer " + std::to_string(i) + " KV length exceeds max_seq");
                    return -1;
                }
                const size_t bytes = 2 * (size_t)len * fa_stride;
                if (buf_len - q < bytes) {
                    why = ("snapshot truncated at layer " + std::to_string(i));
                    return -1;
                }
                q += bytes;
            } else {
                const size_t bytes = (size_t)la_conv + la_ssm;
                if (buf_len - q < bytes) {
                    why = ("snapshot truncated at layer " + std::to_string(i));
                    return -1;
                }
                q += bytes;
            }
        }
        return (long long)q;
    }
}

void reset_state_slot(mfc_ctx *c, int slot) {
    const size_t ssm_elems = (size_t)c->cfg.linear_num_v_heads * GDN_DIM * GDN_DIM;
    cudaMemsetAsync(c->ssm + (size_t)slot * ssm_elems, 0, ssm_elems * sizeof(float), c->stream);
    cudaMemsetAsync(c->conv + (size_t)slot * CONV_TAPS * c->conv_dim, 0,
                    sizeof(float) * CONV_TAPS * c->conv_dim, c->stream);
    c->conv_step[slot] = 0;
}

}  // namespace

// =====================================================================================
#pragma GCC visibility push(default)
extern "C" {

void mfc_default_config(mfc_config *cfg) {
    if (!cfg) return;
    memset(cfg, 0, sizeof(*cfg));
    cfg->num_layers = 60;
    cfg->full_attn_interval = 4;
    cfg->num_attn_heads = 32;
    cfg->num_kv_heads = 2;
    cfg->head_dim = 256;
    cfg->rotary_dim = 64;
    cfg->rope_theta = 1.0e7f;
    cfg->linear_num_v_heads = 64;
    cfg->linear_num_k_heads = 16;
    cfg->linear_key_dim = 128;
    cfg->linear_value_dim = 128;
    cfg->conv_kernel_size = 4;
    cfg->rms_norm_eps = 1e-6f;
    cfg->kv_dtype = MFC_KV_F32;
    cfg->max_seq = 8192;
    cfg->n_seqs = 1;
    cfg->device = 0;
    cfg->kv_rank = 0;
    cfg->kv_world = 1;
    cfg->kv_block = 256;
    cfg->max_batch = 60;
    cfg->snapshot_version = 1;
    cfg->max_prefill = 0;
}

const char *mfc_last_error(const mfc_ctx *ctx) { return ctx ? ctx->err.c_str() : g_open_error.c_str(); }

mfc_ctx *mfc_open(const mfc_config *cfg) {
    mfc_ctx *c = nullptr;
    if (!cfg) {
        fail(c, "NULL config");
        return nullptr;
    }
    const mfc_config &g = *cfg;
    // invariants of the geometry (crates/moeflux/src/riir/variants.rs:546-610) and of the kernels
    if (g.num_layers <= 0 || g.full_attn_interval <= 0 || g.num_attn_heads <= 0 || g.num_kv_heads <= 0 ||
        g.num_attn_heads % g.num_kv_heads != 0 || g.num_attn_heads / g.num_kv_heads > 16) {
        fail(c, "bad head geometry: need num_attn_heads % num_kv_heads == 0 and a group of at most 16");
        return nullptr;
    }
    if (g.head_dim != HEAD_DIM || g.linear_key_dim != GDN_DIM || g.linear_value_dim != GDN_DIM ||
        g.conv_kernel_size != CONV_TAPS) {
        fail(c, "unsupported dims: head_dim must be 256, linear key/value dim 128, conv kernel 4");
        return nullptr;
    }
    if (g.rotary_dim < 0 || g.rotary_dim > HEAD_DIM || g.rotary_dim % 4 != 0) {
        fail(c, "rotary_dim must be a multiple of 4 in [0, 256]");
        return nullptr;
    }
    if (g.linear_num_v_heads <= 0 || g.linear_num_k_heads <= 0 ||
        g.linear_num_v_heads % g.linear_num_k_heads != 0) {
        fail(c, "linear_num_v_heads must be a positive multiple of linear_num_k_heads");
        return nullptr;
    }
    if (g.kv_dtype != MFC_KV_F32 && g.kv_dtype != MFC_KV_BF16) {
        fail(c, "kv_dtype must be MFC_KV_F32 or MFC_KV_BF16");
        return nullptr;
    }
    if (g.max_seq <= 0 || g.n_seqs <= 0 || g.max_batch <= 0) {
        fail(c, "max_seq, n_seqs and max_batch must be positive");
        return nullptr;
    }
    if (g.kv_world < 1 || g.kv_rank < 0 || g.kv_rank >= g.kv_world || g.kv_block <= 0 ||
        g.kv_block % KV_TILE != 0) {
        fail(c, "bad KV split: need 0 <= kv_rank < kv_world and kv_block a positive multiple of 32");
        return nullptr;
    }
    if (g.snapshot_version != 1 && g.snapshot_version != 2) {
        fail(c, "snapshot_version must be 1 or 2");
        return nullptr;
    }
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev <= 0) {
        cudaGetLastError();
        fail(c, "no CUDA device is usable; this library has no CPU path");
        return nullptr;
    }
    if (g.device < 0 || g.device >= ndev || cudaSetDevice(g.device) != cudaSuccess) {
        fail(c, "cannot select CUDA device " + std::to_string(g.device));
        return nullptr;
    }
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, g.device) != cudaSuccess || prop.major != 10) {
        fail(c, "device is not sm_100 (compute capability 10.x); the kernels are built for sm_100a only");
        return nullptr;
    }

    c = new mfc_ctx();
    c->cfg = g;
    if (c->cfg.max_prefill <= 0) c->cfg.max_prefill = g.max_seq < 8192 ? g.max_seq : 8192;
    if (c->cfg.max_prefill > g.max_seq) c->cfg.max_prefill = g.max_seq;
    c->group = g.num_attn_heads / g.num_kv_heads;
    c->kv_esize = g.kv_dtype == MFC_KV_BF16 ? 2 : 4;
    c->conv_dim = 2 * g.linear_num_k_heads * GDN_DIM + g.linear_num_v_heads * GDN_DIM;
    c->layer_to_full.assign(g.num_layers, -1);
    c->layer_to_lin.assign(g.num_layers, -1);
    for (int i = 0; i < g.num_layers; i++) {
        if (is_full_layer(g, i)) c->layer_to_full[i] = c->n_full++;
        else c->layer_to_lin[i] = c->n_lin++;
    }
    {
        const int blocks = (g.max_seq + g.kv_block - 1) / g.kv_block;
        const int my_blocks = (blocks + g.kv_world - 1) / g.kv_world;
        c->cap_rows = g.kv_world > 1 ? my_blocks * g.kv_block : (g.max_seq + KV_TILE - 1) / KV_TILE * KV_TILE;
    }
    c->n_kv_slots = c->n_full * g.n_seqs + 1;
    c->n_state_slots = c->n_lin * g.n_seqs + 1;
    c->kv_len.assign(c->n_kv_slots, 0);
    c->conv_step.assign(c->n_state_slots, 0);
    c->lin_weights_set.assign(c->n_lin > 0 ? c->n_lin : 1, 0);
    c->full_norm_set.assign(c->n_full > 0 ? c->n_full : 1, 0);
    c->checkpoints.resize(g.n_seqs);
    c->checkpoint_order.resize(g.n_seqs);
    if (const char *e = getenv("MFC_GDN_ROWS")) c->gdn_rows = atoi(e);
    if (const char *e = getenv("MFC_GQA_TARGET_CTAS")) c->gqa_target_ctas = atoi(e);
    if (c->gdn_rows != 32 && c->gdn_rows != 64 && c->gdn_rows != 128) c->gdn_rows = 0;
    if (c->gqa_target_ctas < 0) c->gqa_target_ctas = 0;
    if (c->gqa_target_ctas > 8192) c->gqa_target_ctas = 8192;
    c->gqa_slots = 2 * prop.multiProcessorCount;
    c->n_sms = prop.multiProcessorCount;
    c->smem_optin = prop.sharedMemPerBlockOptin;
    c->max_parts = 8192 + g.max_batch * g.num_kv_heads;  // one slot per (unit, CTA) pair: units + CTAs at most

    bool ok = cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking) == cudaSuccess &&
              cudaStreamCreateWithFlags(&c->side_stream, cudaStreamNonBlocking) == cudaSuccess &&
              cudaEventCreateWithFlags(&c->ev_fork, cudaEventDisableTiming) == cudaSuccess &&
              cudaEventCreateWithFlags(&c->ev_join, cudaEventDisableTiming) == cudaSuccess &&
              cudaEventCreateWithFlags(&c->ev_gate, cudaEventDisableTiming) == cudaSuccess;
    if (!ok) fail(c, "cudaStreamCreate failed");
    const uint64_t kv_rows = (uint64_t)c->n_kv_slots * g.num_kv_heads * c->cap_rows;
    if (ok && kv_rows >= (1ull << 32)) ok = fail(c, "KV cache has more rows than a tensor map can address");
    const size_t kv_bytes = (size_t)kv_rows * HEAD_DIM * c->kv_esize;
    const size_t ssm_elems = (size_t)g.linear_num_v_heads * GDN_DIM * GDN_DIM;
    const size_t qd = (size_t)g.num_attn_heads * HEAD_DIM, kvd = (size_t)g.num_kv_heads * HEAD_DIM;
    const size_t vd = (size_t)g.linear_num_v_heads * GDN_DIM;
    const size_t mb = (size_t)g.max_batch;
#define DA(field, count, zero) dalloc(c, &c->field, (size_t)(count), zero, #field)
#define DAV(field, type, count, zero) dalloc(c, (type **)&c->field, (size_t)(count), zero, #field)
    ok = ok && DAV(k_cache, uint8_t, kv_bytes, true) && DAV(v_cache, uint8_t, kv_bytes, true) &&
         DA(ssm, (size_t)c->n_state_slots * ssm_elems, true) &&
         DA(conv, (size_t)c->n_state_slots * CONV_TAPS * c->conv_dim, true) &&
         DA(conv_w, (size_t)(c->n_lin + 1) * c->conv_dim * 4, true) &&
         DA(a_log, (size_t)(c->n_lin + 1) * g.linear_num_v_heads, true) &&
         DA(dt_bias, (size_t)(c->n_lin + 1) * g.linear_num_v_heads, true) &&
         DA(norm_w, (size_t)(c->n_lin + 1) * GDN_DIM, true) && DA(inv_freq, HEAD_DIM / 2, true) &&
         DA(d_gqa_items, mb, false) && DA(d_gdn_items, mb, false) &&
         DA(sc_o, (size_t)c->max_parts * 16 * HEAD_DIM, false) && DA(sc_m, (size_t)c->max_parts * 16, false) &&
         DA(sc_l, (size_t)c->max_parts * 16, false) && DA(tickets, mb * g.num_kv_heads, true) &&
         DA(group_tickets, c->max_parts, true) && DA(status, 1, true) && DA(mv_sched, 4, true) &&
         DA(phase_trace, (size_t)mfc_ctx::MAX_TRACE_CTAS * PHASE_TRACE_WORDS, true) && DA(st_q, mb * qd, false) &&
         DA(st_gate, mb * qd, false) && DA(st_k, mb * kvd, false) && DA(st_v, mb * kvd, false) &&
         DA(st_out, mb * qd, false) && DA(st_qkv, mb * c->conv_dim, false) && DA(st_z, mb * vd, false) &&
         DA(st_alpha, mb * g.linear_num_v_heads, false) && DA(st_beta, mb * g.linear_num_v_heads, false) &&
         DA(st_gout, mb * vd, false) && DA(st_rows, (size_t)mfc_ctx::SNAP_ROWS * kvd, false) &&
         DA(pf_cos_sin, (size_t)g.max_seq * 64, false) && DA(qnorm_w, (size_t)(c->n_full + 1) * HEAD_DIM, true) &&
         DA(knorm_w, (size_t)(c->n_full + 1) * HEAD_DIM, true) && DA(st_qproj, mb * qd * 2, false) &&
         DAV(pf_q, uint16_t, (size_t)c->cfg.max_prefill * g.linear_num_k_heads * GDN_DIM, false) &&
         DAV(pf_k, uint16_t, (size_t)c->cfg.max_prefill * g.linear_num_k_heads * GDN_DIM, false) &&
         DAV(pf_wt, uint16_t, (size_t)c->cfg.max_prefill * vd, false) &&
         DAV(pf_wm, uint16_t, (size_t)c->cfg.max_prefill * g.linear_num_v_heads * 64, false) &&
         DA(pf_v, (size_t)c->cfg.max_prefill * vd, false) &&
         DA(pf_lg, (size_t)c->cfg.max_prefill * g.linear_num_v_heads, false) &&
         DA(pf_beta, (size_t)c->cfg.max_prefill * g.linear_num_v_heads, false);
    if (ok) {
        c->pin_slot_bytes = (mb * (sizeof(GqaItem) > sizeof(GdnItem) ? sizeof(GqaItem) : sizeof(GdnItem)) + 255) & ~(size_t)255;
        ok = cudaHostAlloc((void **)&c->pin_items, c->pin_slot_bytes * mfc_ctx::PIN_SLOTS, cudaHostAllocDefault) == cudaSuccess;
        for (int i = 0; ok && i < mfc_ctx::PIN_SLOTS; i++)
            ok = cudaEventCreateWithFlags(&c->pin_ev[i], cudaEventDisableTiming) == cudaSuccess;
        if (!ok) fail(c, "cannot allocate the pinned staging slots of the item lists");
    }
    if (ok) {
        // the host's libm evaluates the frequencies, exactly as the reference does
        // (crates/moeflux/src/riir/rope.rs:99-101); the device only multiplies by pos
        std::vector<float> f(HEAD_DIM / 2, 0.0f);
        const float rdim_f = (float)g.rotary_dim;
        for (int i = 0; i < g.rotary_dim / 2; i++) f[i] = 1.0f / powf(g.rope_theta, (float)(2 * i) / rdim_f);
        ok = cudaMemcpy(c->inv_freq, f.data(), sizeof(float) * f.size(), cudaMemcpyHostToDevice) == cudaSuccess;
        if (!ok) fail(c, "cudaMemcpy(inv_freq) failed");
    }
    ok = ok && make_tensor_map(c, &c->kmap, c->k_cache, kv_rows) && make_tensor_map(c, &c->vmap, c->v_cache, kv_rows);
    if (ok && g.kv_dtype == MFC_KV_BF16)
        ok = make_tensor_map(c, &c->kmap_pf, c->k_cache, kv_rows, 64) && make_tensor_map(c, &c->vmap_pf, c->v_cache, kv_rows, 64);
    if (ok && gdn_prefill_configure() != cudaSuccess) ok = fail(c, "cannot opt in to the prefill kernel's shared memory size");
    if (ok && gqa_prefill_configure() != cudaSuccess) ok = fail(c, "cannot opt in to the prefill kernel's shared memory size");
    if (ok && (gqa_decode_configure() != cudaSuccess || gqa_decode_f32_configure() != cudaSuccess ||
               mla_decode_configure() != cudaSuccess))
        ok = fail(c, "cannot opt in to the kernels' shared memory size");
    if (ok) c->coop_capacity = g.kv_dtype == MFC_KV_BF16 ? gqa_decode_bf16_coop_capacity() : gqa_decode_f32_coop_capacity();
    if (!ok) {
        g_open_error = c->err;
        free_all(c);
        delete c;
        cudaGetLastError();
        return nullptr;
    }
    return c;
}

void mfc_free(mfc_ctx *c) {
    if (!c) return;
    cudaSetDevice(c->cfg.device);
    cudaStreamSynchronize(c->stream);
    free_all(c);
    delete c;
}

int mfc_get_config(const mfc_ctx *c, mfc_config *out) {
    if (!c || !out) return -1;
    *out = c->cfg;
    return 0;
}

void *mfc_stream(mfc_ctx *c) { return c ? (void *)c->stream : nullptr; }
void *mfc_side_stream(mfc_ctx *c) { return c ? (void *)c->side_stream : nullptr; }

int mfc_set_stream(mfc_ctx *c, void *stream) {
    if (!c) return -1;
    cudaSetDevice(c->cfg.device);
    if (mfc_join(c)) return -1;
    if (cudaStreamSynchronize(c->stream) != cudaSuccess) {
        fail(c, "the context's previous stream is in a failed state");
        return -1;
    }
    if (c->owns_stream && c->stream) cudaStreamDestroy(c->stream);
    c->stream = (cudaStream_t)stream;
    c->owns_stream = false;
    return 0;
}

int mfc_synchronize(mfc_ctx *c) {
    if (!c) return -1;
    cudaSetDevice(c->cfg.device);
    return check_status(c);
}

long long mfc_launch_count(const mfc_ctx *c) { return c ? c->launches : 0; }

// ---------------------------------------------------------------- diagnostics

int mfc_check_guards(mfc_ctx *c) {
    if (!c) return -1;
    cudaSetDevice(c->cfg.device);
    if (mfc_join(c)) return -1;
    CK(cudaStreamSynchronize(c->stream));
    std::vector<uint8_t> band(2 * mfc_ctx::GUARD);
    for (const mfc_ctx::Alloc &a : c->allocs) {
        if (!a.banded) continue;
        CK(cudaMemcpy(band.data(), a.base, mfc_ctx::GUARD, cudaMemcpyDeviceToHost));
        CK(cudaMemcpy(band.data() + mfc_ctx::GUARD, a.base + mfc_ctx::GUARD + a.bytes, mfc_ctx::GUARD,
                      cudaMemcpyDeviceToHost));
        for (size_t i = 0; i < band.size(); i++)
            if (band[i] != 0xFF) {
                const bool before = i < mfc_ctx::GUARD;
                fail(c, std::string("guard band ") + (before ? "before" : "after") + " '" + a.name +
                            "' was written: byte " + std::to_string(before ? i : i - mfc_ctx::GUARD) + " of the band");
                return -1;
            }
    }
    return 0;
}

int mfc_read_phase_trace(mfc_ctx *c, unsigned long long *out, int32_t max_ctas) {
    if (!c || !out || max_ctas <= 0) return -1;
    cudaSetDevice(c->cfg.device);
    CK(cudaStreamSynchronize(c->stream));
    int n = c->last_launch_ctas < max_ctas ? c->last_launch_ctas : max_ctas;
    if (n > mfc_ctx::MAX_TRACE_CTAS) n = mfc_ctx::MAX_TRACE_CTAS;
    CK(cudaMemcpy(out, c->phase_trace, sizeof(unsigned long long) * PHASE_TRACE_WORDS * (size_t)n,
                  cudaMemcpyDeviceToHost));
    return n;
}

// ---------------------------------------------------------------- fused exchange of the KV-sequence split

namespace {
size_t xc_item_floats(const mfc_ctx *c) { return (size_t)c->cfg.num_attn_heads * (HEAD_DIM + 2); }

int xc_finish_connect(mfc_ctx *c) {
    const int W = c->cfg.kv_world;
    std::vector<float *> recv(2 * (size_t)W);
    std::vector<unsigned *> flags(W), q_flags(W);
    std::vector<float *> q_rows(2 * (size_t)W);
    const size_t half = (size_t)W * c->xc.npr * xc_item_floats(c);  // floats of one receive buffer
    const size_t q_half = (size_t)W * c->xc.npr * c->cfg.num_attn_heads * HEAD_DIM;  // floats of one row table
    for (int r = 0; r < W; r++) {
        uint8_t *b = c->xc.peer_base[r];
        recv[r] = reinterpret_cast<float *>(b);
        recv[W + r] = reinterpret_cast<float *>(b) + half;
        flags[r] = reinterpret_cast<unsigned *>(b + c->xc.recv_bytes);
        q_flags[r] = reinterpret_cast<unsigned *>(b + c->xc.recv_bytes + mfc_ctx::XC_FLAG_BYTES);
        q_rows[r] = reinterpret_cast<float *>(b + c->xc.recv_bytes + 2 * mfc_ctx::XC_FLAG_BYTES);
        q_rows[W + r] = q_rows[r] + q_half;
    }
    CK(cudaMemcpy(c->xc.d_peer_recv, recv.data(), sizeof(float *) * recv.size(), cudaMemcpyHostToDevice));
    CK(cudaMemcpy(c->xc.d_peer_flags, flags.data(), sizeof(unsigned *) * flags.size(), cudaMemcpyHostToDevice));
    CK(cudaMemcpy(c->xc.d_peer_q, q_rows.data(), sizeof(float *) * q_rows.size(), cudaMemcpyHostToDevice));
    CK(cudaMemcpy(c->xc.d_peer_q_flags, q_flags.data(), sizeof(unsigned *) * q_flags.size(), cudaMemcpyHostToDevice));
    c->xc.connected = true;
    return 0;
}
}  // namespace

int mfc_exchange_create(mfc_ctx *c, int32_t items_per_rank, void *ipc_handle_out) {
    if (!c) return -1;
    const mfc_config &g = c->cfg;
    if (g.kv_world < 2 || g.kv_world > 128) {
        fail(c, "the exchange needs a context of a KV split (2 <= kv_world <= 128)");
        return -1;
    }
    if (items_per_rank <= 0 || (long long)items_per_rank * g.kv_world > g.max_batch) {
        fail(c, "items_per_rank * kv_world must be in [kv_world, max_batch]");
        return -1;
    }
    if (c->xc.base) {
        fail(c, "the exchange was already created");
        return -1;
    }
    cudaSetDevice(g.device);
    c->xc.npr = items_per_rank;
    c->xc.recv_bytes = (2 * (size_t)g.kv_world * items_per_rank * xc_item_floats(c) * sizeof(float) + 255) & ~(size_t)255;
    const size_t q_bytes = 2 * sizeof(float) * (size_t)g.kv_world * items_per_rank * g.num_attn_heads * HEAD_DIM;
    c->xc.bytes = c->xc.recv_bytes + 2 * mfc_ctx::XC_FLAG_BYTES + q_bytes;
    // its own cudaMalloc (no guard bands): an IPC handle names a whole allocation, from its base
    CK(cudaMalloc((void **)&c->xc.base, c->xc.bytes));
    c->allocs.push_back({c->xc.base, c->xc.bytes, "exchange", false});  // freed with the rest; not band-checked
    CK(cudaMemset(c->xc.base, 0, c->xc.bytes));
    c->xc.recv = reinterpret_cast<float *>(c->xc.base);
    c->xc.flags = reinterpret_cast<unsigned *>(c->xc.base + c->xc.recv_bytes);
    c->xc.q_flags = reinterpret_cast<unsigned *>(c->xc.base + c->xc.recv_bytes + mfc_ctx::XC_FLAG_BYTES);
    c->xc.q_rows = reinterpret_cast<float *>(c->xc.base + c->xc.recv_bytes + 2 * mfc_ctx::XC_FLAG_BYTES);
    if (!dalloc(c, &c->xc.d_peer_recv, 2 * (size_t)g.kv_world, true, "xc.d_peer_recv") ||
        !dalloc(c, &c->xc.d_peer_flags, (size_t)g.kv_world, true, "xc.d_peer_flags") ||
        !dalloc(c, &c->xc.d_peer_q, 2 * (size_t)g.kv_world, true, "xc.d_peer_q") ||
        !dalloc(c, &c->xc.d_peer_q_flags, (size_t)g.kv_world, true, "xc.d_peer_q_flags") ||
        !dalloc(c, &c->xc.q_done_counter, 1, true, "xc.q_done_counter") ||
        !dalloc(c, &c->xc.done_counter, 1, true, "xc.done_counter"))
        return -1;
    c->xc.peer_base.assign(g.kv_world, nullptr);
    c->xc.peer_is_ipc.assign(g.kv_world, false);
    c->xc.peer_base[g.kv_rank] = c->xc.base;
    if (ipc_handle_out) {
        cudaIpcMemHandle_t h;
        CK(cudaIpcGetMemHandle(&h, c->xc.base));
        static_assert(sizeof(h) == MFC_IPC_HANDLE_BYTES, "handle size");
        memcpy(ipc_handle_out, &h, sizeof(h));
    }
    return 0;
}

int mfc_exchange_connect(mfc_ctx *c, const void *ipc_handles) {
    if (!c) return -1;
    if (!c->xc.base || !ipc_handles) {
        fail(c, "mfc_exchange_create first; handles must not be NULL");
        return -1;
    }
    cudaSetDevice(c->cfg.device);
    for (int r = 0; r < c->cfg.kv_world; r++) {
        if (r == c->cfg.kv_rank || c->xc.peer_base[r]) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, (const uint8_t *)ipc_handles + (size_t)r * sizeof(h), sizeof(h));
        void *ptr = nullptr;
        cudaError_t e = cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) {
            fail(c, "cudaIpcOpenMemHandle(rank " + std::to_string(r) + "): " + cudaGetErrorString(e));
            cudaGetLastError();
            return -1;
        }
        c->xc.peer_base[r] = (uint8_t *)ptr;
        c->xc.peer_is_ipc[r] = true;
    }
    return xc_finish_connect(c);
}

int mfc_exchange_connect_local(mfc_ctx *c, mfc_ctx *const *peers) {
    if (!c) return -1;
    if (!c->xc.base || !peers) {
        fail(c, "mfc_exchange_create first; peers must not be NULL");
        return -1;
    }
    cudaSetDevice(c->cfg.device);
    for (int r = 0; r < c->cfg.kv_world; r++) {
        if (r == c->cfg.kv_rank) continue;
        const mfc_ctx *o = peers[r];
        if (!o || !o->xc.base || o->cfg.kv_world != c->cfg.kv_world || o->cfg.kv_rank != r || o->xc.npr != c->xc.npr) {
            fail(c, "peer " + std::to_string(r) + " is not the matching context of this split with its exchange created");
            return -1;
        }
        if (o->cfg.device == c->cfg.device) c->xc.shares_device = true;
        if (o->cfg.device != c->cfg.device) {
            cudaError_t e = cudaDeviceEnablePeerAccess(o->cfg.device, 0);
            if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) {
                fail(c, std::string("cudaDeviceEnablePeerAccess: ") + cudaGetErrorString(e));
                cudaGetLastError();
                return -1;
            }
            cudaGetLastError();
        }
        c->xc.peer_base[r] = o->xc.base;
    }
    return xc_finish_connect(c);
}

int mfc_full_attn_partial_exchange_dev(mfc_ctx *c, int32_t n, const int32_t *layers, const int32_t *seq_ids,
                                       const int32_t *pos, const float *q, const float *k, const float *v) {
    if (!c) return -1;
    if (!q || !k || !v) {
        fail(c, "NULL argument");
        return -1;
    }
    if (!c->xc.connected) {
        fail(c, "the exchange is not connected (mfc_exchange_create, mfc_exchange_connect)");
        return -1;
    }
    if (n != c->xc.npr * c->cfg.kv_world) {
        fail(c, "n must be items_per_rank * kv_world, items sorted by the rank that finishes them");
        return -1;
    }
    cudaSetDevice(c->cfg.device);
    int total = 0;
    if (build_gqa_items(c, n, layers, seq_ids, pos, &total)) return -1;
    GqaParams p;
    fill_gqa_params(c, p, n, total);
    c->xc.step += 1;
    p.q = q;
    p.gate = nullptr;
    p.k = k;
    p.v = v;
    p.partial_mode = 1;
    p.po_item_stride = xc_item_floats(c);
    p.pml_item_stride = xc_item_floats(c);
    p.peer_recv = c->xc.d_peer_recv + (size_t)(c->xc.step & 1u) * c->cfg.kv_world;
    p.peer_flags = c->xc.d_peer_flags;
    p.done_counter = c->xc.done_counter;
    p.items_per_dest = c->xc.npr;
    p.my_rank = c->cfg.kv_rank;
    p.world = c->cfg.kv_world;
    p.flag_value = c->xc.step;
    return launch_gqa(c, p);
}

int mfc_lse_merge_gate_exchange_dev(mfc_ctx *c, const float *gate, float *out) {
    if (!c) return -1;
    if (!out) {
        fail(c, "NULL argument");
        return -1;
    }
    if (!c->xc.connected || c->xc.step == 0) {
        fail(c, "no exchanged step to merge");
        return -1;
    }
    cudaSetDevice(c->cfg.device);
    const size_t hd = (size_t)c->cfg.num_attn_heads * HEAD_DIM, hh = (size_t)c->cfg.num_attn_heads;
    const size_t item = xc_item_floats(c);
    const float *buf = c->xc.recv + (size_t)(c->xc.step & 1u) * c->cfg.kv_world * c->xc.npr * item;
    CK(launch_lse_merge_gate(c->cfg.kv_world, c->xc.npr, c->cfg.num_attn_heads, buf, buf + hd, buf + hd + hh,
                             (size_t)c->xc.npr * item, gate, out, c->stream, item, item, c->xc.flags, c->xc.step,
                             c->gqa_wait_spins, c->status));
    c->launches += 1;
    return 0;
}

// ---------------------------------------------------------------- projections: 4-bit dequant matvec

namespace {
// Tensor map of a weight matrix as bytes [out_dim][in_dim / 2], boxes of 16 rows x 128 bytes.  Encoding one is a
// driver call of a microsecond or two; the maps of the matrices seen last are kept (a model's projections recur every
// token).
bool matvec_map(mfc_ctx *c, const uint32_t *w, const uint16_t *scales, const uint16_t *biases, int in_dim, int out_dim,
                MatvecMaps *out, int m) {
    for (const mfc_ctx::MvMap &e : c->mv_maps)
        if (e.w == w && e.scales == scales && e.biases == biases && e.in_dim == in_dim && e.out_dim == out_dim) {
            out->w[m] = e.map;
            out->sc[m] = e.sc_map;
            out->bi[m] = e.bi_map;
            return true;
        }
    mfc_ctx::MvMap e;
    memset(&e, 0, sizeof(e));
    e.w = w;
    e.scales = scales;
    e.biases = biases;
    e.in_dim = in_dim;
    e.out_dim = out_dim;
    if (!make_map_2d(c, &e.map, const_cast<uint32_t *>(w), CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)in_dim / 2,
                     (uint64_t)out_dim, 128, 16))
        return false;
    // scales and biases travel as boxes only when their rows are multiples of 16 bytes and 16-byte aligned
    if (in_dim % 512 == 0 && !(((uintptr_t)scales | (uintptr_t)biases) & 15)) {
        if (!make_map_2d(c, &e.sc_map, const_cast<uint16_t *>(scales), CU_TENSOR_MAP_DATA_TYPE_UINT16, 2,
                         (uint64_t)in_dim / 64, (uint64_t)out_dim, 32, 16, false) ||
            !make_map_2d(c, &e.bi_map, const_cast<uint16_t *>(biases), CU_TENSOR_MAP_DATA_TYPE_UINT16, 2,
                         (uint64_t)in_dim / 64, (uint64_t)out_dim, 32, 16, false))
            return false;
    }
    if (c->mv_maps.size() >= mfc_ctx::MV_MAP_CACHE) c->mv_maps.erase(c->mv_maps.begin());
    c->mv_maps.push_back(e);
    out->w[m] = e.map;
    out->sc[m] = e.sc_map;
    out->bi[m] = e.bi_map;
    return true;
}

int check_matvec_args(mfc_ctx *c, const void *w, const void *s, const void *b, int32_t in_dim, int32_t out_dim,
                      const float *x, int32_t n_vec, const float *out) {
    if (!w || !s || !b || !x || !out) {
        fail(c, "NULL argument");
        return -1;
    }
    if (in_dim <= 0 || in_dim % MFC_MATVEC_GROUP_SIZE != 0) {  // CpuMatvecError::InDimNotMultiple
        fail(c, "in_dim " + std::to_string(in_dim) + " is not a positive multiple of the group size 64");
        return -1;
    }
    if (out_dim <= 0 || n_vec < 1 || n_vec > MFC_MATVEC_MAX_VECS) {
        fail(c, "out_dim must be positive and n_vec in [1, 8]");
        return -1;
    }
    if (dequant_matvec_4bit_smem(in_dim, 1) > c->smem_optin) {
        fail(c, "in_dim too large for the shared-memory staging of x (" +
                    std::to_string(dequant_matvec_4bit_smem(in_dim, 1)) + " bytes needed)");
        return -1;
    }
    if (((uintptr_t)w & 15) || ((uintptr_t)x & 15)) {
        fail(c, "w_packed and x must be 16-byte aligned");
        return -1;
    }
    return 0;
}
}  // namespace

int mfc_dequant_matvec_4bit_multi_dev(mfc_ctx *c, int32_t n_mat, const uint32_t *const *w_packed,
                                      const uint16_t *const *scales, const uint16_t *const *biases, int32_t in_dim,
                                      const int32_t *out_dims, const float *x, int32_t n_vec, float *const *outs) {
    if (!c) return -1;
    if (n_mat < 1 || n_mat > MATVEC_MAX_MATS || !w_packed || !scales || !biases || !out_dims || !outs) {
        fail(c, "n_mat must be in [1, 8] and the pointer tables non-NULL");
        return -1;
    }
    MatvecBatch mb;
    memset(&mb, 0, sizeof(mb));
    mb.n_mat = n_mat;
    mb.overlap = c->mv_overlap ? 1 : 0;
    mb.inject_lost_load = c->mv_inject_lost_load;
    mb.status = c->status;
    mb.spins = (unsigned)c->gqa_wait_spins;
    mb.trace = c->phase_trace_on ? c->phase_trace : nullptr;  // the grid never exceeds two CTAs per SM
    for (int m = 0; m < n_mat; m++) {
        if (check_matvec_args(c, w_packed[m], scales[m], biases[m], in_dim, out_dims[m], x, n_vec, outs[m])) return -1;
        mb.w[m] = w_packed[m];
        mb.scales[m] = scales[m];
        mb.biases[m] = biases[m];
        mb.out[m] = outs[m];
        mb.out_dim[m] = out_dims[m];
    }
    cudaSetDevice(c->cfg.device);
    // as many vectors per pass over the weights as the staging of x allows
    int per_pass = n_vec;
    MatvecMaps maps;
    for (int m = 0; m < n_mat; m++)
        if (!matvec_map(c, w_packed[m], scales[m], biases[m], in_dim, out_dims[m], &maps, m)) return -1;
    while (per_pass > 1 && dequant_matvec_4bit_smem(in_dim, per_pass) > c->smem_optin) per_pass--;
    for (int v0 = 0; v0 < n_vec; v0 += per_pass) {
        const int nv = n_vec - v0 < per_pass ? n_vec - v0 : per_pass;
        MatvecBatch pass = mb;
        for (int m = 0; m < n_mat; m++) pass.out[m] = outs[m] + (size_t)v0 * out_dims[m];
        int grid = 0;
        pass.sched = c->mv_sched + 2 * (c->mv_launches++ & 1u);  // a launch may overlap the one before it
        CK(launch_dequant_matvec_4bit(pass, x + (size_t)v0 * in_dim, in_dim, nv, c->n_sms, c->stream, &maps, &grid));
        if (pass.trace && grid > 0) c->last_launch_ctas = grid;
        c->launches += 1;
    }
    return 0;
}

int mfc_dequant_matvec_4bit_dev(mfc_ctx *c, const uint32_t *w_packed, const uint16_t *scales, const uint16_t *biases,
                                int32_t in_dim, int32_t out_dim, const float *x, int32_t n_vec, float *out) {
    return mfc_dequant_matvec_4bit_multi_dev(c, 1, &w_packed, &scales, &biases, in_dim, &out_dim, x, n_vec, &out);
}

int mfc_dequant_matvec_4bit(mfc_ctx *c, const uint32_t *w_packed, const uint16_t *scales, const uint16_t *biases,
                            int32_t in_dim, int32_t out_dim, const float *x, int32_t n_vec, float *out) {
    if (!c) return -1;
    if (!w_packed || !scales || !biases || !x || !out) {
        fail(c, "NULL argument");
        return -1;
    }
    if (in_dim <= 0 || in_dim % MFC_MATVEC_GROUP_SIZE != 0 || out_dim <= 0 || n_vec < 1 || n_vec > MFC_MATVEC_MAX_VECS) {
        fail(c, "in_dim must be a positive multiple of 64, out_dim positive, n_vec in [1, 8]");
        return -1;
    }
    cudaSetDevice(c->cfg.device);
    // a hook for tests and bring-up, not a hot path: the operands are staged in device memory for this call only
    const size_t wb = sizeof(uint32_t) * (size_t)out_dim * (in_dim / 8), sb = sizeof(uint16_t) * (size_t)out_dim * (in_dim / 64);
    const size_t xb = sizeof(float) * (size_t)n_vec * in_dim, ob = sizeof(float) * (size_t)n_vec * out_dim;
    uint8_t *d = nullptr;
    const size_t o_w = 0, o_s = (wb + 255) & ~(size_t)255, o_b = (o_s + sb + 255) & ~(size_t)255,
                 o_x = (o_b + sb + 255) & ~(size_t)255, o_o = (o_x + xb + 255) & ~(size_t)255;
    CK(cudaMalloc(&d, o_o + ob));
    int rc = -1;
    do {
        if (cudaMemcpyAsync(d + o_w, w_packed, wb, cudaMemcpyHostToDevice, c->stream) != cudaSuccess ||
            cudaMemcpyAsync(d + o_s, scales, sb, cudaMemcpyHostToDevice, c->stream) != cudaSuccess ||
            cudaMemcpyAsync(d + o_b, biases, sb, cudaMemcpyHostToDevice, c->stream) != cudaSuccess ||
            cudaMemcpyAsync(d + o_x, x, xb, cudaMemcpyHostToDevice, c->stream) != cudaSuccess) {
            fail(c, "host to device copy failed");
            break;
        }
        if (mfc_dequant_matvec_4bit_dev(c, (const uint32_t *)(d + o_w), (const uint16_t *)(d + o_s),
                                        (const uint16_t *)(d + o_b), in_dim, out_dim, (const float *)(d + o_x), n_vec,
                                        (float *)(d + o_o)))
            break;
        if (cudaMemcpyAsync(out, d + o_o, ob, cudaMemcpyDeviceToHost, c->stream) != cudaSuccess ||
            cudaStreamSynchronize(c->stream) != cudaSuccess) {
            fail(c, "device to host copy failed");
            break;
        }
        rc = check_status(c);  // a kernel that gave up on a bounded wait reports here
    } while (0);
    cudaStreamSynchronize(c->stream);
    cudaFree(d);
    return rc;
}

// ---------------------------------------------------------------- folded MLA attention

namespace {
int mla_sdpa_folded_dev(mfc_ctx *c, int32_t num_heads, int32_t cache_len, float softmax_scale, const float *q_prime,
                        const float *q_pe, const void *latent_cache, const void *rope_k_cache, float *v_combine,
                        bool cache_bf16) {
    if (!c) return -1;
    if (!q_prime || !q_pe || !latent_cache || !rope_k_cache || !v_combine) {
        fail(c, "NULL argument");
        return -1;
    }
    if (num_heads <= 0 || num_heads > 1024 || cache_len <= 0) {
        fail(c, "num_heads must be in [1, 1024] and cache_len positive");
        return -1;
    }
    if (((uintptr_t)latent_cache & 15) || ((uintptr_t)rope_k_cache & 15) || ((uintptr_t)q_prime & 15) ||
        ((uintptr_t)q_pe & 15) || ((uintptr_t)v_combine & 15)) {
        fail(c, "all arrays must be 16-byte aligned");
        return -1;
    }
    cudaSetDevice(c->cfg.device);
    MlaParams p;
    memset(&p, 0, sizeof(p));
    p.H = num_heads;
    p.cache_len = cache_len;
    p.n_head_blocks = (num_heads + 15) / 16;
    // chunks: one wave of CTAs (two per SM) over head blocks x chunks, at least 256 positions per chunk
    int n_chunks = c->gqa_slots / p.n_head_blocks;
    if (c->gqa_forced_chunk > 0) n_chunks = (cache_len + c->gqa_forced_chunk - 1) / c->gqa_forced_chunk;
    const int max_by_len = (cache_len + 255) / 256;
    if (n_chunks > max_by_len && c->gqa_forced_chunk <= 0) n_chunks = max_by_len;
    if (n_chunks < 1) n_chunks = 1;
    int rows = (cache_len + n_chunks - 1) / n_chunks;
    rows = (rows + 15) / 16 * 16;
    n_chunks = (cache_len + rows - 1) / rows;
    p.n_chunks = n_chunks;
    p.rows_per_chunk = rows;
    // partials in the split-K scratch: [n_chunks][H][512] floats, m and l behind them in their own arrays
    const size_t need_o = (size_t)n_chunks * num_heads * MLA_RANK;
    if (need_o > (size_t)c->max_parts * 16 * HEAD_DIM || (size_t)n_chunks * num_heads > (size_t)c->max_parts * 16) {
        fail(c, "split plan exceeds the scratch reserved at open");
        return -1;
    }
    p.q_prime = q_prime;
    p.q_pe = q_pe;
    p.out = v_combine;
    p.part_o = c->sc_o;
    p.part_m = c->sc_m;
    p.part_l = c->sc_l;
    p.status = c->status;
    p.scale = softmax_scale;
    p.wait_spins = c->gqa_wait_spins;
    p.cache_bf16 = cache_bf16 ? 1 : 0;
    CUtensorMap lat_map, rope_map;
    const CUtensorMapDataType dt = cache_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
    const int es = cache_bf16 ? 2 : 4, box_cols = cache_bf16 ? 64 : 32, box_rows = cache_bf16 ? 32 : 16;
    if (!make_map_2d(c, &lat_map, const_cast<void *>(latent_cache), dt, es, MLA_RANK, (uint64_t)cache_len, box_cols, box_rows) ||
        !make_map_2d(c, &rope_map, const_cast<void *>(rope_k_cache), dt, es, MLA_ROPE, (uint64_t)cache_len, box_cols, box_rows))
        return -1;
    CK(launch_mla_decode(lat_map, rope_map, p, c->stream));
    c->launches += n_chunks > 1 ? 2 : 1;
    return 0;
}
}  // namespace

int mfc_mla_sdpa_folded_dev(mfc_ctx *c, int32_t num_heads, int32_t cache_len, float softmax_scale, const float *q_prime,
                            const float *q_pe, const float *latent_cache, const float *rope_k_cache, float *v_combine) {
    return mla_sdpa_folded_dev(c, num_heads, cache_len, softmax_scale, q_prime, q_pe, latent_cache, rope_k_cache, v_combine,
                               false);
}

int mfc_mla_sdpa_folded_bf16_dev(mfc_ctx *c, int32_t num_heads, int32_t cache_len, float softmax_scale,
                                 const float *q_prime, const float *q_pe, const void *latent_cache_bf16,
                                 const void *rope_k_cache_bf16, float *v_combine) {
    return mla_sdpa_folded_dev(c, num_heads, cache_len, softmax_scale, q_prime, q_pe, latent_cache_bf16, rope_k_cache_bf16,
                               v_combine, true);
}

int mfc_mla_sdpa_folded(mfc_ctx *c, int32_t num_heads, int32_t cache_len, float softmax_scale, const float *q_prime,
                        const float *q_pe, const float *latent_cache, const float *rope_k_cache, float *v_combine) {
    if (!c) return -1;
    if (!q_prime || !q_pe || !latent_cache || !rope_k_cache || !v_combine || num_heads <= 0 || cache_len <= 0) {
        fail(c, "NULL argument, or num_heads / cache_len not positive");
        return -1;
    }
    cudaSetDevice(c->cfg.device);
    // a hook for tests and bring-up: the operands are staged in device memory for this call only
    const size_t qb = sizeof(float) * (size_t)num_heads * MLA_RANK, pb = sizeof(float) * (size_t)num_heads * MLA_ROPE;
    const size_t lb = sizeof(float) * (size_t)cache_len * MLA_RANK, rb = sizeof(float) * (size_t)cache_len * MLA_ROPE;
    const size_t al = 255;
    const size_t o_q = 0, o_p = (o_q + qb + al) & ~al, o_l = (o_p + pb + al) & ~al, o_r = (o_l + lb + al) & ~al,
                 o_o = (o_r + rb + al) & ~al;
    uint8_t *d = nullptr;
    CK(cudaMalloc(&d, o_o + qb));
    int rc = -1;
    do {
        if (cudaMemcpyAsync(d + o_q, q_prime, qb, cudaMemcpyHostToDevice, c->stream) != cudaSuccess ||
            cudaMemcpyAsync(d + o_p, q_pe, pb, cudaMemcpyHostToDevice, c->stream) != cudaSuccess ||
            cudaMemcpyAsync(d + o_l, latent_cache, lb, cudaMemcpyHostToDevice, c->stream) != cudaSuccess ||
            cudaMemcpyAsync(d + o_r, rope_k_cache, rb, cudaMemcpyHostToDevice, c->stream) != cudaSuccess) {
            fail(c, "host to device copy failed");
            break;
        }
        if (mfc_mla_sdpa_folded_dev(c, num_heads, cache_len, softmax_scale, (const float *)(d + o_q),
                                    (const float *)(d + o_p), (const float *)(d + o_l), (const float *)(d + o_r),
                                    (float *)(d + o_o)))
            break;
        if (cudaMemcpyAsync(v_combine, d + o_o, qb, cudaMemcpyDeviceToHost, c->stream) != cudaSuccess) {
            fail(c, "device to host copy failed");
            break;
        }
        rc = check_status(c);
    } while (0);
    cudaStreamSynchronize(c->stream);
    cudaFree(d);
    return rc;
}

int mfc_set_tuning(mfc_ctx *c, const char *key, int value) {
    if (!c || !key) return -1;
    if (!strcmp(key, "gdn_rows")) {
        if (value != 0 && value != 32 && value != 64 && value != 128) return -1;
        c->gdn_rows = value;
    } else if (!strcmp(key, "gqa_target_ctas")) {
        if (value < 0 || value > 8192) return -1;
        c->gqa_target_ctas = value;
    } else if (!strcmp(key, "gdn_side_queue")) {
        if (mfc_join(c)) return -1;
        c->gdn_side = value != 0;
    } else if (!strcmp(key, "gqa_chunk")) {
        if (value < 0) return -1;
        c->gqa_forced_chunk = value;
    } else if (!strcmp(key, "gqa_min_rows")) {
        if (value < 32 || value % 32) return -1;
        c->gqa_min_rows = value;
    } else if (!strcmp(key, "matvec_inject_lost_load")) {
        c->mv_inject_lost_load = value != 0;
    } else if (!strcmp(key, "matvec_overlap")) {
        c->mv_overlap = value != 0;
    } else if (!strcmp(key, "exchange_gather_q")) {
        c->xc.gather_q = value != 0;
    } else if (!strcmp(key, "gqa_align_units")) {
        c->gqa_align_units = value != 0;
    } else if (!strcmp(key, "gqa_coop_merge")) {
        c->gqa_coop = value != 0;
    } else if (!strcmp(key, "gqa_coop_min_parts")) {
        if (value < MERGE_GROUP) return -1;
        c->gqa_coop_min_parts = value;
    } else if (!strcmp(key, "gqa_unit_aligned")) {
        c->gqa_unit_aligned = value != 0;
    } else if (!strcmp(key, "gqa_wait_spins")) {
        if (value < 0) return -1;
        c->gqa_wait_spins = (unsigned)value;
    } else if (!strcmp(key, "gqa_inject_lost_load")) {
        c->gqa_inject_lost_load = value != 0;
    } else if (!strcmp(key, "gqa_phase_trace")) {
        c->phase_trace_on = value != 0;
    } else {
        return -1;
    }
    return 0;
}

int mfc_set_linear_weights(mfc_ctx *c, int32_t layer, const uint16_t *conv_w, const float *a_log,
                           const uint16_t *dt_bias, const uint16_t *norm_w) {
    if (!c) return -1;
    const mfc_config &g = c->cfg;
    // layer == -1 addresses the weight row used by the stateless hook slot only
    if (!conv_w || !a_log || !dt_bias) {
        fail(c, "NULL argument");
        return -1;
    }
    if (layer < 0 || layer >= g.num_layers || is_full_layer(g, layer)) {
        fail(c, "layer " + std::to_string(layer) + " is not a linear-attention layer");
        return -1;
    }
    cudaSetDevice(g.device);
    const int ll = c->layer_to_lin[layer];
    CK(cudaMemcpyAsync(c->conv_w + (size_t)ll * c->conv_dim * 4, conv_w, sizeof(uint16_t) * c->conv_dim * 4,
                       cudaMemcpyHostToDevice, c->stream));
    CK(cudaMemcpyAsync(c->a_log + (size_t)ll * g.linear_num_v_heads, a_log, sizeof(float) * g.linear_num_v_heads,
                       cudaMemcpyHostToDevice, c->stream));
    CK(cudaMemcpyAsync(c->dt_bias + (size_t)ll * g.linear_num_v_heads, dt_bias,
                       sizeof(uint16_t) * g.linear_num_v_heads, cudaMemcpyHostToDevice, c->stream));
    if (norm_w)
        CK(cudaMemcpyAsync(c->norm_w + (size_t)ll * GDN_DIM, norm_w, sizeof(uint16_t) * GDN_DIM,
                           cudaMemcpyHostToDevice, c->stream));
    CK(cudaStreamSynchronize(c->stream));
    c->lin_weights_set[ll] = norm_w ? 2 : 1;
    return 0;
}

// ---------------------------------------------------------------- full attention

int mfc_full_attn_step_batched_dev(mfc_ctx *c, int32_t n, const int32_t *layers, const int32_t *seq_ids,
                                   const int32_t *pos, const float *q, const float *gate, const float *k,
                                   const float *v, float *out) {
    if (!c) return -1;
    if (!q || !gate || !k || !v || !out) {
        fail(c, "NULL argument");
        return -1;
    }
    if (c->cfg.kv_world != 1) {
        fail(c, "this context holds a share of a KV split: use mfc_full_attn_partial_batched_dev");
        return -1;
    }
    cudaSetDevice(c->cfg.device);
    int total = 0;
    if (build_gqa_items(c, n, layers, seq_ids, pos, &total)) return -1;
    GqaParams p;
    fill_gqa_params(c, p, n, total);
    p.q = q;
    p.gate = gate;
    p.k = k;
    p.v = v;
    p.out = out;
    p.partial_mode = 0;
    return launch_gqa(c, p);
}

int mfc_full_attn_partial_batched_dev(mfc_ctx *c, int32_t n, const int32_t *layers, const int32_t *seq_ids,
                                      const int32_t *pos, const float *q, const float *k, const float *v,
                                      float *o_part, float *m_part, float *l_part) {
    if (!c) return -1;
    if (!q || !k || !v || !o_part || !m_part || !l_part) {
        fail(c, "NULL argument");
        return -1;
    }
    cudaSetDevice(c->cfg.device);
    int total = 0;
    if (build_gqa_items(c, n, layers, seq_ids, pos, &total)) return -1;
    GqaParams p;
    fill_gqa_params(c, p, n, total);
    p.q = q;
    p.gate = nullptr;
    p.k = k;
    p.v = v;
    p.po = o_part;
    p.pm = m_part;
    p.pl = l_part;
    p.partial_mode = 1;
    return launch_gqa(c, p);
}

int mfc_lse_merge_gate_dev(mfc_ctx *c, int32_t n_parts, int32_t n, const float *o_parts, const float *m_parts,
                           const float *l_parts, size_t part_stride, const float *gate, float *out) {
    if (!c) return -1;
    if (n_parts <= 0 || n <= 0 || !o_parts || !m_parts || !l_parts || !out) {
        fail(c, "bad argument");
        return -1;
    }
    cudaSetDevice(c->cfg.device);
    CK(launch_lse_merge_gate(n_parts, n, c->cfg.num_attn_heads, o_parts, m_parts, l_parts, part_stride, gate, out,
                             c->stream));
    c->launches += 1;
    return 0;
}

int mfc_full_attn_partial_packed_dev(mfc_ctx *c, int32_t n, const int32_t *layers, const int32_t *seq_ids,
                                     const int32_t *pos, const float *q, const float *k, const float *v,
                                     float *packed) {
    if (!c) return -1;
    if (!q || !k || !v || !packed) {
        fail(c, "NULL argument");
        return -1;
    }
    cudaSetDevice(c->cfg.device);
    int total = 0;
    if (build_gqa_items(c, n, layers, seq_ids, pos, &total)) return -1;
    const size_t hd = (size_t)c->cfg.num_attn_heads * HEAD_DIM, hh = (size_t)c->cfg.num_attn_heads;
    GqaParams p;
    fill_gqa_params(c, p, n, total);
    p.q = q;
    p.gate = nullptr;
    p.k = k;
    p.v = v;
    p.po = packed;  // item i: [o (H*256) | m (H) | l (H)]
    p.pm = packed + hd;
    p.pl = packed + hd + hh;
    p.po_item_stride = hd + 2 * hh;
    p.pml_item_stride = hd + 2 * hh;
    p.partial_mode = 1;
    return launch_gqa(c, p);
}

int mfc_lse_merge_gate_packed_dev(mfc_ctx *c, int32_t n_parts, int32_t n, const float *packed_parts,
                                  const float *gate, float *out) {
    if (!c) return -1;
    if (n_parts <= 0 || n <= 0 || !packed_parts || !out) {
        fail(c, "bad argument");
        return -1;
    }
    cudaSetDevice(c->cfg.device);
    const size_t hd = (size_t)c->cfg.num_attn_heads * HEAD_DIM, hh = (size_t)c->cfg.num_attn_heads;
    const size_t item = hd + 2 * hh;
    CK(launch_lse_merge_gate(n_parts, n, c->cfg.num_attn_heads, packed_parts, packed_parts + hd, packed_parts + hd + hh,
                             (size_t)n * item, gate, out, c->stream, item, item));
    c->launches += 1;
    return 0;
}

int mfc_full_attn_step_batched(mfc_ctx *c, int32_t n, const int32_t *layers, const int32_t *seq_ids,
                               const int32_t *pos, const float *q, const float *gate, const float *k,
                               const float *v, float *out) {
    if (!c) return -1;
    if (!q || !gate || !k || !v || !out) {
        fail(c, "NULL argument");
        return -1;
    }
    if (n <= 0 || n > c->cfg.max_batch) {
        fail(c, "item count must be in [1, max_batch]");
        return -1;
    }
    cudaSetDevice(c->cfg.device);
    const size_t qd = sizeof(float) * c->cfg.num_attn_heads * HEAD_DIM * (size_t)n;
    const size_t kd = sizeof(float) * c->cfg.num_kv_heads * HEAD_DIM * (size_t)n;
    CK(cudaMemcpyAsync(c->st_q, q, qd, cudaMemcpyHostToDevice, c->stream));
    CK(cudaMemcpyAsync(c->st_gate, gate, qd, cudaMemcpyHostToDevice, c->stream));
    CK(cudaMemcpyAsync(c->st_k, k, kd, cudaMemcpyHostToDevice, c->stream));
    CK(cudaMemcpyAsync(c->st_v, v, kd, cudaMemcpyHostToDevice, c->stream));
    if (mfc_full_attn_step_batched_dev(c, n, layers, seq_ids, pos, c->st_q, c->st_gate, c->st_k, c->st_v, c->st_out))
        return -1;
    CK(cudaMemcpyAsync(out, c->st_out, qd, cudaMemcpyDeviceToHost, c->stream));
    return check_status(c);
}

int mfc_full_attn_step(mfc_ctx *c, int32_t layer, int32_t seq_id, int32_t pos, const float *q, const float *gate,
                       const float *k, const float *v, float *out) {
    return mfc_full_attn_step_batched(c, 1, &layer, &seq_id, &pos, q, gate, k, v, out);
}

// ---------------------------------------------------------------- q projection layout + per-head norms

int mfc_set_full_attn_norm_weights(mfc_ctx *c, int32_t layer, const uint16_t *q_norm_bf16, const uint16_t *k_norm_bf16) {
    if (!c) return -1;
    const mfc_config &g = c->cfg;
    if (!q_norm_bf16 || !k_norm_bf16) {
        fail(c, "NULL argument");
        return -1;
    }
    if (layer < 0 || layer >= g.num_layers || !is_full_layer(g, layer)) {
        fail(c, "layer " + std::to_string(layer) + " is not a full-attention layer");
        return -1;
    }
    cudaSetDevice(g.device);
    const int fl = c->layer_to_full[layer];
    CK(cudaMemcpyAsync(c->qnorm_w + (size_t)fl * HEAD_DIM, q_norm_bf16, sizeof(uint16_t) * HEAD_DIM,
                       cudaMemcpyHostToDevice, c->stream));
    CK(cudaMemcpyAsync(c->knorm_w + (size_t)fl * HEAD_DIM, k_norm_bf16, sizeof(uint16_t) * HEAD_DIM,
                       cudaMemcpyHostToDevice, c->stream));
    CK(cudaStreamSynchronize(c->stream));
    c->full_norm_set[fl] = 1;
    return 0;
}

int mfc_full_attn_step_qproj_batched_dev(mfc_ctx *c, int32_t n, const int32_t *layers, const int32_t *seq_ids,
                                         const int32_t *pos, const float *q_proj, const float *k, const float *v,
                                         float *out) {
    if (!c) return -1;
    if (!q_proj || !k || !v || !out) {
        fail(c, "NULL argument");
        return -1;
    }
    if (c->cfg.kv_world != 1) {
        fail(c, "this context holds a share of a KV split");
        return -1;
    }
    cudaSetDevice(c->cfg.device);
    if (layers && n > 0 && n <= c->cfg.max_batch)
        for (int i = 0; i < n; i++) {
            const int l = layers[i];
            if (l < 0 || l >= c->cfg.num_layers || !is_full_layer(c->cfg, l) || !c->full_norm_set[c->layer_to_full[l]]) {
                fail(c, "mfc_set_full_attn_norm_weights was not called for layer " + std::to_string(l));
                return -1;
            }
        }
    int total = 0;
    if (build_gqa_items(c, n, layers, seq_ids, pos, &total)) return -1;
    GqaParams p;
    fill_gqa_params(c, p, n, total);
    p.q = q_proj;                    // head row h: [q (256) | gate (256)]
    p.gate = q_proj + HEAD_DIM;
    p.q_row_stride = 2 * HEAD_DIM;
    p.gate_row_stride = 2 * HEAD_DIM;
    p.qnorm_w = c->qnorm_w;
    p.knorm_w = c->knorm_w;
    p.k = k;
    p.v = v;
    p.out = out;
    p.partial_mode = 0;
    return launch_gqa(c, p);
}

int mfc_full_attn_step_qproj_batched(mfc_ctx *c, int32_t n, const int32_t *layers, const int32_t *seq_ids,
                                     const int32_t *pos, const float *q_proj, const float *k, const float *v,
                                     float *out) {
    if (!c) return -1;
    if (!q_proj || !k || !v || !out) {
        fail(c, "NULL argument");
        return -1;
    }
    if (n <= 0 || n > c->cfg.max_batch) {
        fail(c, "item count must be in [1, max_batch]");
        return -1;
    }
    cudaSetDevice(c->cfg.device);
    const size_t qd = sizeof(float) * c->cfg.num_attn_heads * HEAD_DIM * (size_t)n;
    const size_t kd = sizeof(float) * c->cfg.num_kv_heads * HEAD_DIM * (size_t)n;
    CK(cudaMemcpyAsync(c->st_qproj, q_proj, 2 * qd, cudaMemcpyHostToDevice, c->stream));
    CK(cudaMemcpyAsync(c->st_k, k, kd, cudaMemcpyHostToDevice, c->stream));
    CK(cudaMemcpyAsync(c->st_v, v, kd, cudaMemcpyHostToDevice, c->stream));
    if (mfc_full_attn_step_qproj_batched_dev(c, n, layers, seq_ids, pos, c->st_qproj, c->st_k, c->st_v, c->st_out))
        return -1;
    CK(cudaMemcpyAsync(out, c->st_out, qd, cudaMemcpyDeviceToHost, c->stream));
    return check_status(c);
}

// ---------------------------------------------------------------- GatedDeltaNet

int mfc_linear_attn_step_batched_dev(mfc_ctx *c, int32_t n, const int32_t *layers, const int32_t *seq_ids,
                                     const float *qkv, const float *z, const float *alpha, const float *beta,
                                     float *out) {
    if (!c) return -1;
    if (!qkv || !alpha || !beta || !out) {
        fail(c, "NULL argument");
        return -1;
    }
    cudaSetDevice(c->cfg.device);
    if (build_gdn_items(c, n, layers, seq_ids)) return -1;
    if (z) {
        for (int i = 0; i < n; i++)
            if (c->lin_weights_set[c->h_gdn_items[i].w_layer] != 2) {
                fail(c, "z given but no norm weight was set for layer " + std::to_string(layers[i]));
                return -1;
            }
    }
    if (!c->gdn_side) return launch_gdn(c, n, qkv, z, alpha, beta, out);
    // side queue: ordered after everything already on the main queue, runs beside what follows on it
    cudaStream_t main_stream = c->stream;
    CK(cudaEventRecord(c->ev_fork, main_stream));
    CK(cudaStreamWaitEvent(c->side_stream, c->ev_fork, 0));
    c->stream = c->side_stream;
    const int rc = launch_gdn(c, n, qkv, z, alpha, beta, out);
    c->stream = main_stream;
    if (rc) return -1;
    CK(cudaEventRecord(c->ev_join, c->side_stream));
    c->side_pending = true;
    return 0;
}

int mfc_join(mfc_ctx *c) {
    if (!c) return -1;
    if (c->side_pending) {
        cudaSetDevice(c->cfg.device);
        CK(cudaStreamWaitEvent(c->stream, c->ev_join, 0));
        c->side_pending = false;
    }
    return 0;
}

int mfc_linear_attn_step_batched(mfc_ctx *c, int32_t n, const int32_t *layers, const int32_t *seq_ids,
                                 const float *qkv, const float *z, const float *alpha, const float *beta,
                                 float *out) {
    if (!c) return -1;
    if (!qkv || !alpha || !beta || !out) {
        fail(c, "NULL argument");
        return -1;
    }
    if (n <= 0 || n > c->cfg.max_batch) {
        fail(c, "item count must be in [1, max_batch]");
        return -1;
    }
    cudaSetDevice(c->cfg.device);
    const mfc_config &g = c->cfg;
    const size_t vd = sizeof(float) * g.linear_num_v_heads * GDN_DIM * (size_t)n;
    const size_t hd = sizeof(float) * g.linear_num_v_heads * (size_t)n;
    CK(cudaMemcpyAsync(c->st_qkv, qkv, sizeof(float) * c->conv_dim * (size_t)n, cudaMemcpyHostToDevice, c->stream));
    if (z) CK(cudaMemcpyAsync(c->st_z, z, vd, cudaMemcpyHostToDevice, c->stream));
    CK(cudaMemcpyAsync(c->st_alpha, alpha, hd, cudaMemcpyHostToDevice, c->stream));
    CK(cudaMemcpyAsync(c->st_beta, beta, hd, cudaMemcpyHostToDevice, c->stream));
    if (mfc_linear_attn_step_batched_dev(c, n, layers, seq_ids, c->st_qkv, z ? c->st_z : nullptr, c->st_alpha,
                                         c->st_beta, c->st_gout))
        return -1;
    CK(cudaMemcpyAsync(out, c->st_gout, vd, cudaMemcpyDeviceToHost, c->stream));
    return check_status(c);
}

int mfc_linear_attn_step(mfc_ctx *c, int32_t layer, int32_t seq_id, const float *qkv, const float *z,
                         const float *alpha, const float *beta, float *out) {
    return mfc_linear_attn_step_batched(c, 1, &layer, &seq_id, qkv, z, alpha, beta, out);
}

// ---------------------------------------------------------------- whole-stack step

int mfc_eval_token_attn(mfc_ctx *c, int32_t n_full, const int32_t *full_layers, const int32_t *full_seqs,
                        const int32_t *pos, const float *q, const float *gate, const float *k, const float *v,
                        float *full_out, int32_t n_lin, const int32_t *lin_layers, const int32_t *lin_seqs,
                        const float *qkv, const float *z, const float *alpha, const float *beta, float *lin_out) {
    if (!c) return -1;
    const mfc_config &g = c->cfg;
    if (n_full < 0 || n_lin < 0 || n_full + n_lin == 0 || n_full > g.max_batch || n_lin > g.max_batch) {
        fail(c, "item counts must be in [0, max_batch] and not both zero");
        return -1;
    }
    if ((n_full && (!q || !gate || !k || !v || !full_out)) || (n_lin && (!qkv || !alpha || !beta || !lin_out))) {
        fail(c, "NULL argument");
        return -1;
    }
    const bool split = g.kv_world != 1;
    if (split && n_full && (!c->xc.connected || n_full != c->xc.npr * g.kv_world)) {
        fail(c, "this context holds a share of a KV split: connect the exchange (mfc_exchange_create / _connect) and "
                "pass items_per_rank * kv_world full-attention items sorted by the rank that finishes them");
        return -1;
    }
    if (split && n_full && c->xc.gather_q && c->xc.shares_device) {
        // its kernel waits for the peers' kernels, and kernels on one GPU are not guaranteed to run at the same time
        fail(c, "exchange_gather_q needs every rank of the split on a GPU of its own");
        return -1;
    }
    cudaSetDevice(g.device);
    cudaStream_t main_stream = c->stream;
    // Order of the host's work, chosen for the time until the attention kernel starts (the long one): the copies of
    // its inputs are queued first, the launches are planned under them (tens of microseconds for a hundred items),
    // its kernel is queued, and only then the gate logits, the GatedDeltaNet inputs (3.5x larger) and that group's
    // kernel, all of which travel under the attention kernel.  The early copies go to staging buffers and touch no
    // cache and no state: a validation failure still leaves every state as it was.
    const size_t qd = sizeof(float) * g.num_attn_heads * HEAD_DIM * (size_t)n_full;
    const size_t kd = sizeof(float) * g.num_kv_heads * HEAD_DIM * (size_t)n_full;
    // with a KV split, gate and full_out cover the items this rank finishes only
    const size_t own_qd = split ? sizeof(float) * g.num_attn_heads * HEAD_DIM * (size_t)c->xc.npr : qd;
    const size_t vd = sizeof(float) * g.linear_num_v_heads * GDN_DIM * (size_t)n_lin;
    const size_t hd = sizeof(float) * g.linear_num_v_heads * (size_t)n_lin;
    const bool gather = split && n_full && c->xc.gather_q;  // q: own rows only, the rest over the links
    const unsigned next_step = c->xc.step + 1;              // the exchange's step number of this call
    const float *q_dev = c->st_q;
    CK(cudaEventRecord(c->ev_fork, main_stream));
    CK(cudaStreamWaitEvent(c->side_stream, c->ev_fork, 0));
    if (n_full) {
        if (gather) {
            // q holds the rows of this rank's own items: they land in their slot of this step's row table; the other
            // slots arrive over the links
            const size_t own_floats = own_qd / sizeof(float);
            float *table = c->xc.q_rows + (size_t)(next_step & 1u) * g.kv_world * own_floats;
            CK(cudaMemcpyAsync(table + (size_t)g.kv_rank * own_floats, q, own_qd, cudaMemcpyHostToDevice, main_stream));
            q_dev = table;
        } else {
            CK(cudaMemcpyAsync(c->st_q, q, qd, cudaMemcpyHostToDevice, main_stream));
        }
        CK(cudaMemcpyAsync(c->st_k, k, kd, cudaMemcpyHostToDevice, main_stream));
        CK(cudaMemcpyAsync(c->st_v, v, kd, cudaMemcpyHostToDevice, main_stream));
    }
    // validate both groups before any kernel is queued; a refusal returns only after the queued copies have finished
    // reading the caller's buffers
    auto refuse = [&]() {
        cudaStreamSynchronize(main_stream);
        return -1;
    };
    if (n_lin) {
        if (build_gdn_items(c, n_lin, lin_layers, lin_seqs)) return refuse();
        if (z)
            for (int i = 0; i < n_lin; i++)
                if (c->lin_weights_set[c->h_gdn_items[i].w_layer] != 2) {
                    for (int j = 0; j < n_lin; j++) c->conv_step[c->h_gdn_items[j].state_idx] -= 1;
                    fail(c, "z given but no norm weight was set for layer " + std::to_string(lin_layers[i]));
                    return refuse();
                }
    }
    int total = 0;
    if (n_full && build_gqa_items(c, n_full, full_layers, full_seqs, pos, &total)) {
        for (int j = 0; j < n_lin; j++) c->conv_step[c->h_gdn_items[j].state_idx] -= 1;
        return refuse();
    }
    if (n_full) {
        GqaParams p;
        fill_gqa_params(c, p, n_full, total);
        p.q = q_dev;
        p.gate = nullptr;
        p.k = c->st_k;
        p.v = c->st_v;
        p.out = c->st_out;
        p.partial_mode = 0;
        if (split) {
            c->xc.step = next_step;
            if (gather) {
                CK(launch_q_rows_gather(c->xc.d_peer_q + (size_t)(next_step & 1u) * g.kv_world, c->xc.d_peer_q_flags,
                                        c->xc.q_flags, c->xc.q_done_counter, own_qd / sizeof(float), g.kv_rank,
                                        g.kv_world, next_step, c->gqa_wait_spins, c->status, main_stream));
                c->launches += 1;
            }
            // partials straight into the owners' receive buffers; the merge below waits for the peers' flags
            p.partial_mode = 1;
            p.po_item_stride = p.pml_item_stride = (size_t)g.num_attn_heads * (HEAD_DIM + 2);
            p.peer_recv = c->xc.d_peer_recv + (size_t)(c->xc.step & 1u) * g.kv_world;
            p.peer_flags = c->xc.d_peer_flags;
            p.done_counter = c->xc.done_counter;
            p.items_per_dest = c->xc.npr;
            p.my_rank = g.kv_rank;
            p.world = g.kv_world;
            p.flag_value = c->xc.step;
        }
        if (launch_gqa(c, p)) return -1;
        // the gate logits (as many bytes as q) are only needed after the attention kernel: they travel on the side
        // queue under it and are applied by a separate elementwise pass (or by the merge)
        CK(cudaMemcpyAsync(c->st_gate, gate, own_qd, cudaMemcpyHostToDevice, c->side_stream));
        CK(cudaEventRecord(c->ev_gate, c->side_stream));
    }
    if (n_lin) {
        // GatedDeltaNet group on the side queue: its copies and kernel overlap the attention kernel
        cudaStream_t s2 = c->side_stream;
        CK(cudaMemcpyAsync(c->st_qkv, qkv, sizeof(float) * c->conv_dim * (size_t)n_lin, cudaMemcpyHostToDevice, s2));
        if (z) CK(cudaMemcpyAsync(c->st_z, z, vd, cudaMemcpyHostToDevice, s2));
        CK(cudaMemcpyAsync(c->st_alpha, alpha, hd, cudaMemcpyHostToDevice, s2));
        CK(cudaMemcpyAsync(c->st_beta, beta, hd, cudaMemcpyHostToDevice, s2));
        c->stream = s2;
        const int rc = launch_gdn(c, n_lin, c->st_qkv, z ? c->st_z : nullptr, c->st_alpha, c->st_beta, c->st_gout);
        c->stream = main_stream;
        if (rc) return -1;
        CK(cudaMemcpyAsync(lin_out, c->st_gout, vd, cudaMemcpyDeviceToHost, s2));
        CK(cudaEventRecord(c->ev_join, s2));
    }
    if (n_full) {
        CK(cudaStreamWaitEvent(main_stream, c->ev_gate, 0));
        if (split) {
            if (mfc_lse_merge_gate_exchange_dev(c, c->st_gate, c->st_out)) return -1;
        } else {
            CK(launch_sigmoid_gate(c->st_out, c->st_gate, qd / sizeof(float), main_stream));
            c->launches += 1;
        }
        CK(cudaMemcpyAsync(full_out, c->st_out, own_qd, cudaMemcpyDeviceToHost, main_stream));
    }
    if (n_lin) CK(cudaStreamWaitEvent(main_stream, c->ev_join, 0));
    return check_status(c);
}

// ---------------------------------------------------------------- prefill

int mfc_full_attn_prefill_dev(mfc_ctx *c, int32_t layer, int32_t seq_id, int32_t start_pos, int32_t n_tokens,
                              const void *q_bf16, const void *gate_bf16, const void *k_bf16, const void *v_bf16,
                              void *out_bf16) {
    if (!c) return -1;
    const mfc_config &g = c->cfg;
    if (!q_bf16 || !k_bf16 || !v_bf16 || !out_bf16 || n_tokens <= 0) {
        fail(c, "NULL argument or n_tokens <= 0");
        return -1;
    }
    if (layer < 0 || layer >= g.num_layers || !is_full_layer(g, layer) || seq_id < 0 || seq_id >= g.n_seqs) {
        fail(c, "not a full-attention layer / seq_id out of range");
        return -1;
    }
    if (g.kv_dtype != MFC_KV_BF16 || g.kv_world != 1 || g.rotary_dim > 64) {
        fail(c, "prefill needs a bf16 KV cache held by one context and rotary_dim <= 64");
        return -1;
    }
    const int slot = c->layer_to_full[layer] * g.n_seqs + seq_id;
    if (start_pos != c->kv_len[slot]) {
        fail(c, "start_pos " + std::to_string(start_pos) + " != current length " + std::to_string(c->kv_len[slot]));
        return -1;
    }
    if ((long long)start_pos + n_tokens > g.max_seq) {
        fail(c, "kv cache overflow");
        return -1;
    }
    if (((uintptr_t)q_bf16 & 15) || ((uintptr_t)out_bf16 & 15) || ((uintptr_t)gate_bf16 & 15)) {
        fail(c, "q, gate and out must be 16-byte aligned");
        return -1;
    }
    cudaSetDevice(g.device);
    // 3-D map over q [T][H][256]: box = 64 dims x 1 head x 128 tokens
    CUtensorMap qmap;
    {
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess || !fn) {
            fail(c, "cuTensorMapEncodeTiled is not available from the driver");
            return -1;
        }
        cuuint64_t dims[3] = {(cuuint64_t)HEAD_DIM, (cuuint64_t)g.num_attn_heads, (cuuint64_t)n_tokens};
        cuuint64_t strides[2] = {(cuuint64_t)HEAD_DIM * 2, (cuuint64_t)HEAD_DIM * 2 * g.num_attn_heads};
        cuuint32_t box[3] = {64, 1, 128};
        cuuint32_t estr[3] = {1, 1, 1};
        CUresult r = ((EncodeTiledFn)fn)(&qmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void *>(q_bf16), dims,
                                         strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) {
            fail(c, "cuTensorMapEncodeTiled(q) failed, code " + std::to_string((int)r));
            return -1;
        }
    }
    const size_t slot_row0 = (size_t)slot * g.num_kv_heads * c->cap_rows;
    CK(launch_prefill_kv_append(k_bf16, v_bf16, c->k_cache, c->v_cache, 1, c->pf_cos_sin, c->inv_freq, n_tokens,
                                g.num_kv_heads, g.rotary_dim, start_pos, slot_row0, c->cap_rows, 0, 1, 1, c->stream));
    PrefillAttnParams p;
    memset(&p, 0, sizeof(p));
    p.gate = reinterpret_cast<const __nv_bfloat16 *>(gate_bf16);
    p.out = reinterpret_cast<__nv_bfloat16 *>(out_bf16);
    p.cos_sin = c->pf_cos_sin;
    p.T = n_tokens;
    p.H = g.num_attn_heads;
    p.Hkv = g.num_kv_heads;
    p.group = c->group;
    p.start_pos = start_pos;
    p.rotary_dim = g.rotary_dim;
    p.kv_slot = slot;
    p.cap_rows = c->cap_rows;
    p.scale = 1.0f / sqrtf((float)g.head_dim);
    p.status = c->status;
    CK(launch_gqa_prefill(qmap, c->kmap_pf, c->vmap_pf, p, c->stream));
    c->launches += 2;
    c->kv_len[slot] += n_tokens;
    return 0;
}

int mfc_linear_attn_prefill_dev(mfc_ctx *c, int32_t layer, int32_t seq_id, int32_t n_tokens, const void *qkv_bf16,
                                const void *z_bf16, const void *alpha_bf16, const void *beta_bf16, void *out_bf16) {
    if (!c) return -1;
    const mfc_config &g = c->cfg;
    if (!qkv_bf16 || !alpha_bf16 || !beta_bf16 || !out_bf16 || n_tokens <= 0) {
        fail(c, "NULL argument or n_tokens <= 0");
        return -1;
    }
    if (layer < 0 || layer >= g.num_layers || is_full_layer(g, layer) || seq_id < 0 || seq_id >= g.n_seqs) {
        fail(c, "not a linear-attention layer / seq_id out of range");
        return -1;
    }
    const int ll = c->layer_to_lin[layer];
    if (!c->lin_weights_set[ll] || (z_bf16 && c->lin_weights_set[ll] != 2)) {
        fail(c, "mfc_set_linear_weights was not called for layer " + std::to_string(layer) + " (or no norm weight for z)");
        return -1;
    }
    if (n_tokens > g.max_prefill) {
        fail(c, "n_tokens " + std::to_string(n_tokens) + " exceeds max_prefill " + std::to_string(g.max_prefill));
        return -1;
    }
    if ((g.linear_num_v_heads * GDN_DIM) % g.linear_num_k_heads != 0 || ((uintptr_t)qkv_bf16 & 15)) {
        fail(c, "unsupported head geometry or misaligned qkv");
        return -1;
    }
    cudaSetDevice(g.device);
    if (mfc_join(c)) return -1;  // a GatedDeltaNet launch may still be running on the side queue
    const int slot = ll * g.n_seqs + seq_id;
    GdnPrefillParams p;
    memset(&p, 0, sizeof(p));
    p.qkv = qkv_bf16;
    p.z = z_bf16;
    p.alpha = alpha_bf16;
    p.beta = beta_bf16;
    p.out = out_bf16;
    p.ssm = c->ssm + (size_t)slot * g.linear_num_v_heads * GDN_DIM * GDN_DIM;
    p.ring = c->conv + (size_t)slot * CONV_TAPS * c->conv_dim;
    p.slot0 = (int)(c->conv_step[slot] & 3);
    p.conv_w = c->conv_w + (size_t)ll * c->conv_dim * 4;
    p.a_log = c->a_log + (size_t)ll * g.linear_num_v_heads;
    p.dt_bias = c->dt_bias + (size_t)ll * g.linear_num_v_heads;
    p.norm_w = c->norm_w + (size_t)ll * GDN_DIM;
    p.q_hat = c->pf_q;
    p.k_hat = c->pf_k;
    p.v_io = c->pf_v;
    p.lg = c->pf_lg;
    p.beta_gate = c->pf_beta;
    p.w_tilde = c->pf_wt;
    p.w_mask = c->pf_wm;
    p.T = n_tokens;
    p.Hk = g.linear_num_k_heads;
    p.Hv = g.linear_num_v_heads;
    p.conv_dim = c->conv_dim;
    p.eps = g.rms_norm_eps;
    p.status = c->status;
    GdnPrefillMaps m;
    const uint64_t kd = (uint64_t)g.linear_num_k_heads * GDN_DIM, vd = (uint64_t)g.linear_num_v_heads * GDN_DIM;
    if (!make_map_2d(c, &m.wt, c->pf_wt, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, vd, n_tokens, 64, 64) ||
        !make_map_2d(c, &m.q, c->pf_q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, kd, n_tokens, 64, 64) ||
        !make_map_2d(c, &m.k, c->pf_k, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, kd, n_tokens, 64, 64) ||
        !make_map_2d(c, &m.wm, c->pf_wm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)g.linear_num_v_heads * 64, n_tokens,
                     64, 64) ||
        !make_map_2d(c, &m.ut, c->pf_v, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, vd, n_tokens, 32, 64))
        return -1;
    CK(launch_gdn_prefill(p, m, c->stream));
    c->launches += 5;
    c->conv_step[slot] += n_tokens;
    return 0;
}

// ---------------------------------------------------------------- bulk state import (device)

int mfc_kv_append_rows_dev(mfc_ctx *c, int32_t layer, int32_t seq_id, int32_t pos0, int32_t n_rows,
                           const float *k_rows, const float *v_rows) {
    if (!c) return -1;
    const mfc_config &g = c->cfg;
    if (!k_rows || !v_rows || n_rows <= 0) {
        fail(c, "bad argument");
        return -1;
    }
    if (layer < 0 || layer >= g.num_layers || !is_full_layer(g, layer) || seq_id < 0 || seq_id >= g.n_seqs) {
        fail(c, "not a full-attention layer / seq_id out of range");
        return -1;
    }
    const int slot = c->layer_to_full[layer] * g.n_seqs + seq_id;
    if (pos0 != c->kv_len[slot]) {
        fail(c, "pos0 " + std::to_string(pos0) + " != current length " + std::to_string(c->kv_len[slot]));
        return -1;
    }
    if ((long long)pos0 + n_rows > g.max_seq) {
        fail(c, "kv cache overflow");
        return -1;
    }
    cudaSetDevice(g.device);
    const size_t slot_off = (size_t)slot * g.num_kv_heads * c->cap_rows * HEAD_DIM * c->kv_esize;
    CK(launch_kv_pack(k_rows, (uint8_t *)c->k_cache + slot_off, n_rows, g.num_kv_heads, c->cap_rows,
                      g.kv_dtype == MFC_KV_BF16, pos0, g.kv_rank, g.kv_world, g.kv_block, c->stream));
    CK(launch_kv_pack(v_rows, (uint8_t *)c->v_cache + slot_off, n_rows, g.num_kv_heads, c->cap_rows,
                      g.kv_dtype == MFC_KV_BF16, pos0, g.kv_rank, g.kv_world, g.kv_block, c->stream));
    c->launches += 2;
    c->kv_len[slot] += n_rows;
    return 0;
}

int mfc_linear_state_set_dev(mfc_ctx *c, int32_t layer, int32_t seq_id, const float *conv_state,
                             const float *ssm_state) {
    if (!c) return -1;
    const mfc_config &g = c->cfg;
    if (!conv_state || !ssm_state) {
        fail(c, "NULL argument");
        return -1;
    }
    if (layer < 0 || layer >= g.num_layers || is_full_layer(g, layer) || seq_id < 0 || seq_id >= g.n_seqs) {
        fail(c, "not a linear-attention layer / seq_id out of range");
        return -1;
    }
    cudaSetDevice(g.device);
    if (mfc_join(c)) return -1;  // a GatedDeltaNet launch may still be running on the side queue
    const int slot = c->layer_to_lin[layer] * g.n_seqs + seq_id;
    const size_t ssm_elems = (size_t)g.linear_num_v_heads * GDN_DIM * GDN_DIM;
    float *ring = c->conv + (size_t)slot * CONV_TAPS * c->conv_dim;
    CK(cudaMemsetAsync(ring, 0, sizeof(float) * c->conv_dim, c->stream));
    CK(cudaMemcpyAsync(ring + c->conv_dim, conv_state, sizeof(float) * 3 * c->conv_dim, cudaMemcpyDeviceToDevice,
                       c->stream));
    CK(cudaMemcpyAsync(c->ssm + (size_t)slot * ssm_elems, ssm_state, sizeof(float) * ssm_elems,
                       cudaMemcpyDeviceToDevice, c->stream));
    c->conv_step[slot] = 0;
    return 0;
}

// ---------------------------------------------------------------- sequence state

void mfc_memory_clear(mfc_ctx *c, int32_t seq_id) {
    if (!c) return;
    mfc_memory_seq_rm(c, seq_id, 0, -1);
    // a full clear invalidates every stored position (mod.rs:1964-1968)
    if (seq_id >= -1 && seq_id < c->cfg.n_seqs)
        for (int s = (seq_id < 0 ? 0 : seq_id); s < (seq_id < 0 ? c->cfg.n_seqs : seq_id + 1); s++) {
            c->checkpoints[s].clear();
            c->checkpoint_order[s].clear();
        }
}

int mfc_memory_seq_rm(mfc_ctx *c, int32_t seq_id, int32_t p0, int32_t p1) {
    if (!c) return 0;
    const mfc_config &g = c->cfg;
    if (seq_id < -1 || seq_id >= g.n_seqs) return 0;
    cudaSetDevice(g.device);
    if (mfc_join(c)) return 0;  // a GatedDeltaNet launch may still be running on the side queue
    const int s0 = seq_id < 0 ? 0 : seq_id, s1 = seq_id < 0 ? g.n_seqs : seq_id + 1;
    const int new_len = p0 < 0 ? 0 : p0;
    for (int s = s0; s < s1; s++) {
        // crates/moeflux/src/riir/state.rs:431-458
        for (int f = 0; f < c->n_full; f++) {
            int32_t &len = c->kv_len[f * g.n_seqs + s];
            const int eff_end = (p1 < 0 || p1 > len) ? len : p1;
            const int to = new_len < eff_end ? new_len : eff_end;
            if (to <= len) len = to;
        }
        for (int l = 0; l < c->n_lin; l++) reset_state_slot(c, l * g.n_seqs + s);
    }
    return cudaStreamSynchronize(c->stream) == cudaSuccess ? 1 : 0;
}

int mfc_memory_seq_pos_max(mfc_ctx *c, int32_t seq_id) {
    if (!c || seq_id < 0 || seq_id >= c->cfg.n_seqs) return -1;
    int mx = -1;  // stays -1 only when the model has no full-attention layer (state.rs:460-473)
    for (int f = 0; f < c->n_full; f++) {
        const int len = c->kv_len[f * c->cfg.n_seqs + seq_id];
        if (len > mx) mx = len;
    }
    return mx;
}

// ---------------------------------------------------------------- snapshots ('MFLX')

size_t mfc_state_size(const mfc_ctx *c, int32_t seq_id) {
    if (!c || seq_id < 0 || seq_id >= c->cfg.n_seqs) return 0;
    const mfc_config &g = c->cfg;
    const size_t header = (g.snapshot_version == 1 ? 8 : 10) * sizeof(uint32_t);
    const size_t fa_stride = (size_t)g.num_kv_heads * HEAD_DIM * sizeof(float);
    const size_t la_conv = (size_t)(CONV_TAPS - 1) * c->conv_dim * sizeof(float);
    const size_t la_ssm = (size_t)g.linear_num_v_heads * GDN_DIM * GDN_DIM * sizeof(float);
    size_t nbytes = header;
    for (int i = 0; i < g.num_layers; i++) {
        if (is_full_layer(g, i)) nbytes += 4 + 2 * (size_t)c->kv_len[c->layer_to_full[i] * g.n_seqs + seq_id] * fa_stride;
        else nbytes += la_conv + la_ssm;
    }
    return nbytes;
}

long long mfc_state_save(mfc_ctx *c, int32_t seq_id, void *buf, size_t buf_len) {
    if (!c) return -1;
    const mfc_config &g = c->cfg;
    if (!buf || seq_id < 0 || seq_id >= g.n_seqs) {
        fail(c, "bad argument");
        return -1;
    }
    if (g.kv_world != 1) {
        fail(c, "snapshots need the whole cache in one context (kv_world == 1)");
        return -1;
    }
    const size_t need = mfc_state_size(c, seq_id);
    if (buf_len < need) {
        fail(c, "buffer too small: need " + std::to_string(need) + " bytes");
        return -1;
    }
    cudaSetDevice(g.device);
    if (mfc_join(c)) return -1;  // a GatedDeltaNet launch may still be running on the side queue
    uint8_t *out = (uint8_t *)buf;
    size_t off = 0;
    const uint32_t la_conv = (uint32_t)((CONV_TAPS - 1) * c->conv_dim * sizeof(float));
    const uint32_t la_ssm = (uint32_t)((size_t)g.linear_num_v_heads * GDN_DIM * GDN_DIM * sizeof(float));
    const uint32_t header[10] = {SNAPSHOT_MAGIC, (uint32_t)g.snapshot_version, (uint32_t)g.num_layers,
                                 (uint32_t)g.full_attn_interval, (uint32_t)g.num_kv_heads, (uint32_t)g.head_dim,
                                 la_conv, la_ssm, 0u, 0u};  // words 8, 9: kv_lora_rank, qk_rope_head_dim (0 for GQA)
    const size_t hbytes = (g.snapshot_version == 1 ? 8 : 10) * sizeof(uint32_t);
    memcpy(out, header, hbytes);
    off += hbytes;
    const size_t kvd = (size_t)g.num_kv_heads * HEAD_DIM;
    for (int i = 0; i < g.num_layers; i++) {
        if (is_full_layer(g, i)) {
            const int slot = c->layer_to_full[i] * g.n_seqs + seq_id;
            const int32_t len = c->kv_len[slot];
            memcpy(out + off, &len, 4);
            off += 4;
            for (int pass = 0; pass < 2; pass++) {
                const uint8_t *cache = (const uint8_t *)(pass == 0 ? c->k_cache : c->v_cache) +
                                       (size_t)slot * g.num_kv_heads * c->cap_rows * HEAD_DIM * c->kv_esize;
                for (int r0 = 0; r0 < len; r0 += mfc_ctx::SNAP_ROWS) {
                    const int nr = len - r0 < mfc_ctx::SNAP_ROWS ? len - r0 : mfc_ctx::SNAP_ROWS;
                    CK(launch_kv_unpack(cache + (size_t)r0 * HEAD_DIM * c->kv_esize, c->st_rows, nr, g.num_kv_heads,
                                        c->cap_rows, g.kv_dtype == MFC_KV_BF16, c->stream));
                    c->launches += 1;
                    CK(cudaMemcpyAsync(out + off, c->st_rows, sizeof(float) * kvd * nr, cudaMemcpyDeviceToHost,
                                       c->stream));
                    CK(cudaStreamSynchronize(c->stream));
                    off += sizeof(float) * kvd * nr;
                }
            }
        } else {
            const int slot = c->layer_to_lin[i] * g.n_seqs + seq_id;
            const float *ring = c->conv + (size_t)slot * CONV_TAPS * c->conv_dim;
            const int t = (int)(c->conv_step[slot] & 3);
            for (int k = 0; k < CONV_TAPS - 1; k++) {  // oldest first: slots t+1, t+2, t+3
                CK(cudaMemcpyAsync(out + off, ring + (size_t)((t + 1 + k) & 3) * c->conv_dim,
                                   sizeof(float) * c->conv_dim, cudaMemcpyDeviceToHost, c->stream));
                off += sizeof(float) * c->conv_dim;
            }
            CK(cudaMemcpyAsync(out + off, c->ssm + (size_t)slot * (la_ssm / 4), la_ssm, cudaMemcpyDeviceToHost,
                               c->stream));
            off += la_ssm;
        }
    }
    CK(cudaStreamSynchronize(c->stream));
    return (long long)off;
}

int mfc_state_load(mfc_ctx *c, int32_t seq_id, const void *buf, size_t buf_len) {
    if (!c) return -1;
    const mfc_config &g = c->cfg;
    if (!buf || seq_id < 0 || seq_id >= g.n_seqs) {
        fail(c, "bad argument");
        return -1;
    }
    if (g.kv_world != 1) {
        fail(c, "snapshots need the whole cache in one context (kv_world == 1)");
        return -1;
    }
    const uint8_t *in = (const uint8_t *)buf;
    size_t hbytes = 0;
    std::string why;
    if (snapshot_preflight(g, in, buf_len, &hbytes, why) < 0) {
        fail(c, why);
        return -1;
    }
    const uint32_t la_conv = (uint32_t)((CONV_TAPS - 1) * c->conv_dim * sizeof(float));
    const uint32_t la_ssm = (uint32_t)((size_t)g.linear_num_v_heads * GDN_DIM * GDN_DIM * sizeof(float));
    // restore
    cudaSetDevice(g.device);
    if (mfc_join(c)) return -1;  // a GatedDeltaNet launch may still be running on the side queue
    size_t off = hbytes;
    const size_t kvd = (size_t)g.num_kv_heads * HEAD_DIM;
    for (int i = 0; i < g.num_layers; i++) {
        if (is_full_layer(g, i)) {
            const int slot = c->layer_to_full[i] * g.n_seqs + seq_id;
            int32_t len;
            memcpy(&len, in + off, 4);
            off += 4;
            for (int pass = 0; pass < 2; pass++) {
                uint8_t *cache = (uint8_t *)(pass == 0 ? c->k_cache : c->v_cache) +
                                 (size_t)slot * g.num_kv_heads * c->cap_rows * HEAD_DIM * c->kv_esize;
                for (int r0 = 0; r0 < len; r0 += mfc_ctx::SNAP_ROWS) {
                    const int nr = len - r0 < mfc_ctx::SNAP_ROWS ? len - r0 : mfc_ctx::SNAP_ROWS;
                    CK(cudaMemcpyAsync(c->st_rows, in + off, sizeof(float) * kvd * nr, cudaMemcpyHostToDevice,
                                       c->stream));
                    CK(launch_kv_pack(c->st_rows, cache, nr, g.num_kv_heads, c->cap_rows,
                                      g.kv_dtype == MFC_KV_BF16, r0, 0, 1, 1, c->stream));
                    c->launches += 1;
                    CK(cudaStreamSynchronize(c->stream));
                    off += sizeof(float) * kvd * nr;
                }
            }
            c->kv_len[slot] = len;
        } else {
            const int slot = c->layer_to_lin[i] * g.n_seqs + seq_id;
            float *ring = c->conv + (size_t)slot * CONV_TAPS * c->conv_dim;
            // history rows go to slots 1..3; the next step writes slot 0
            CK(cudaMemsetAsync(ring, 0, sizeof(float) * c->conv_dim, c->stream));
            CK(cudaMemcpyAsync(ring + c->conv_dim, in + off, la_conv, cudaMemcpyHostToDevice, c->stream));
            off += la_conv;
            CK(cudaMemcpyAsync(c->ssm + (size_t)slot * (la_ssm / 4), in + off, la_ssm, cudaMemcpyHostToDevice,
                               c->stream));
            off += la_ssm;
            c->conv_step[slot] = 0;
        }
    }
    CK(cudaStreamSynchronize(c->stream));
    return 0;
}

// ---------------------------------------------------------------- checkpoints (mod.rs:2015-2087)

int mfc_checkpoint_pos(mfc_ctx *c, int32_t seq_id, int32_t pos) {
    if (!c) return -1;
    if (seq_id < 0 || seq_id >= c->cfg.n_seqs) {
        fail(c, "seq_id out of range");
        return -1;
    }
    std::vector<uint8_t> buf(mfc_state_size(c, seq_id));
    if (mfc_state_save(c, seq_id, buf.data(), buf.size()) < 0) return -1;
    auto &store = c->checkpoints[seq_id];
    auto &order = c->checkpoint_order[seq_id];
    if (store.count(pos)) {  // overwrite: refresh its place in the order
        for (auto it = order.begin(); it != order.end(); ++it)
            if (*it == pos) {
                order.erase(it);
                break;
            }
    }
    store[pos] = std::move(buf);
    order.push_back(pos);
    // evict the oldest entries, never position 0 nor the one just stored
    while (store.size() > c->max_checkpoints) {
        bool evicted = false;
        for (auto it = order.begin(); it != order.end(); ++it) {
            if (*it == 0 || *it == pos) continue;
            store.erase(*it);
            order.erase(it);
            evicted = true;
            break;
        }
        if (!evicted) break;
    }
    return 0;
}

int mfc_restore_to(mfc_ctx *c, int32_t seq_id, int32_t pos) {
    if (!c) return -1;
    if (seq_id < 0 || seq_id >= c->cfg.n_seqs) {
        fail(c, "seq_id out of range");
        return -1;
    }
    auto &store = c->checkpoints[seq_id];
    auto it = store.find(pos);
    if (it == store.end()) {
        fail(c, "no checkpoint stored at position " + std::to_string(pos));
        return -1;
    }
    if (mfc_state_load(c, seq_id, it->second.data(), it->second.size())) return -1;
    // positions after pos are about to be rewritten: their snapshots are void
    for (auto e = store.begin(); e != store.end();) e = (e->first > pos) ? store.erase(e) : std::next(e);
    auto &order = c->checkpoint_order[seq_id];
    for (auto e = order.begin(); e != order.end();) e = (*e > pos) ? order.erase(e) : std::next(e);
    return 0;
}

void mfc_set_max_checkpoints(mfc_ctx *c, int32_t n) {
    if (c && n >= 0) c->max_checkpoints = (size_t)n;
}

int mfc_checkpoint_count(const mfc_ctx *c, int32_t seq_id) {
    if (!c || seq_id < 0 || seq_id >= c->cfg.n_seqs) return -1;
    return (int)c->checkpoints[seq_id].size();
}

// ---------------------------------------------------------------- host-only helpers

int mfc_kv_local_len(int32_t len, int32_t rank, int32_t world, int32_t block) {
    if (len < 0 || world < 1 || rank < 0 || rank >= world || block <= 0) return -1;
    return local_len_of(len, rank, world, block);
}

int mfc_kv_local_row(int32_t pos, int32_t rank, int32_t world, int32_t block) {
    if (pos < 0 || world < 1 || rank < 0 || rank >= world || block <= 0) return -1;
    return local_row_of(pos, rank, world, block);
}

long long mfc_snapshot_validate(const mfc_config *cfg, const void *buf, size_t buf_len) {
    if (!cfg || !buf) return -1;
    size_t hb = 0;
    std::string why;
    const long long r = snapshot_preflight(*cfg, (const uint8_t *)buf, buf_len, &hb, why);
    if (r < 0) g_open_error = why;
    return r;
}

// ---------------------------------------------------------------- parity hooks

int mfc_apply_rotary_emb(mfc_ctx *c, int32_t pos, float *q, float *k) {
    if (!c) return -1;
    if (!q || !k || pos < 0) {
        fail(c, "NULL argument or pos < 0");
        return -1;
    }
    const mfc_config &g = c->cfg;
    cudaSetDevice(g.device);
    const size_t qd = sizeof(float) * g.num_attn_heads * HEAD_DIM, kd = sizeof(float) * g.num_kv_heads * HEAD_DIM;
    CK(cudaMemcpyAsync(c->st_q, q, qd, cudaMemcpyHostToDevice, c->stream));
    CK(cudaMemcpyAsync(c->st_k, k, kd, cudaMemcpyHostToDevice, c->stream));
    CK(launch_rope(c->st_q, c->st_k, g.num_attn_heads, g.num_kv_heads, g.rotary_dim, pos, c->inv_freq, c->stream));
    c->launches += 1;
    CK(cudaMemcpyAsync(q, c->st_q, qd, cudaMemcpyDeviceToHost, c->stream));
    CK(cudaMemcpyAsync(k, c->st_k, kd, cudaMemcpyDeviceToHost, c->stream));
    CK(cudaStreamSynchronize(c->stream));
    return 0;
}

int mfc_sdpa(mfc_ctx *c, int32_t kv_len, const float *q, const float *q_gate, const float *k_cache,
             const float *v_cache, float *out) {
    if (!c) return -1;
    if (!q || !q_gate || !k_cache || !v_cache || !out || kv_len <= 0) {
        fail(c, "NULL argument or kv_len <= 0");
        return -1;
    }
    const mfc_config &g = c->cfg;
    if (kv_len > c->cap_rows) {
        fail(c, "kv_len exceeds the rows reserved per sequence");
        return -1;
    }
    cudaSetDevice(g.device);
    const int slot = c->n_kv_slots - 1;  // hook slot
    const size_t kvd = (size_t)g.num_kv_heads * HEAD_DIM;
    for (int pass = 0; pass < 2; pass++) {
        uint8_t *cache = (uint8_t *)(pass == 0 ? c->k_cache : c->v_cache) +
                         (size_t)slot * g.num_kv_heads * c->cap_rows * HEAD_DIM * c->kv_esize;
        const float *src = pass == 0 ? k_cache : v_cache;
        for (int r0 = 0; r0 < kv_len; r0 += mfc_ctx::SNAP_ROWS) {
            const int nr = kv_len - r0 < mfc_ctx::SNAP_ROWS ? kv_len - r0 : mfc_ctx::SNAP_ROWS;
            CK(cudaMemcpyAsync(c->st_rows, src + (size_t)r0 * kvd, sizeof(float) * kvd * nr, cudaMemcpyHostToDevice,
                               c->stream));
            CK(launch_kv_pack(c->st_rows, cache, nr, g.num_kv_heads, c->cap_rows, g.kv_dtype == MFC_KV_BF16, r0,
                              0, 1, 1, c->stream));
            c->launches += 1;
            CK(cudaStreamSynchronize(c->stream));
        }
    }
    const size_t qd = sizeof(float) * g.num_attn_heads * HEAD_DIM;
    CK(cudaMemcpyAsync(c->st_q, q, qd, cudaMemcpyHostToDevice, c->stream));
    CK(cudaMemcpyAsync(c->st_gate, q_gate, qd, cudaMemcpyHostToDevice, c->stream));
    c->h_gqa_items.resize(1);
    GqaItem &it = c->h_gqa_items[0];
    it.kv_slot = slot;
    it.local_len = kv_len;
    it.pos = 0;
    it.append_row = -1;
    it.in_idx = 0;
    it.tile_begin = 0;
    it.pad0 = it.pad1 = 0;
    {
        const int tile = g.kv_dtype == MFC_KV_BF16 ? KV_TILE : KV_TILE_F32;
        const int nt = (kv_len + tile - 1) / tile;
        c->plan_total_tiles = nt * g.num_kv_heads;
        c->plan_tiles_per_cta = plan_tiles_per_cta(c, c->plan_total_tiles, nt);
        c->plan_max_parts = (nt + c->plan_tiles_per_cta - 1) / c->plan_tiles_per_cta + 1;
    }
    GqaParams p;
    fill_gqa_params(c, p, 1, (c->plan_total_tiles + c->plan_tiles_per_cta - 1) / c->plan_tiles_per_cta);
    p.q = c->st_q;
    p.gate = c->st_gate;
    p.k = c->st_k;
    p.v = c->st_v;
    p.out = c->st_out;
    p.rotary_dim = 0;  // q and the cached K are already rotated
    if (launch_gqa(c, p)) return -1;
    CK(cudaMemcpyAsync(out, c->st_out, qd, cudaMemcpyDeviceToHost, c->stream));
    return check_status(c);
}

int mfc_linear_attn_step_stateless(mfc_ctx *c, int32_t layer, const float *qkv, const float *z, const float *alpha,
                                   const float *beta, float *conv_state, float *ssm_state, float *out) {
    if (!c) return -1;
    const mfc_config &g = c->cfg;
    if (!qkv || !alpha || !beta || !conv_state || !ssm_state || !out) {
        fail(c, "NULL argument");
        return -1;
    }
    if (layer < 0 || layer >= g.num_layers || is_full_layer(g, layer) || !c->lin_weights_set[c->layer_to_lin[layer]]) {
        fail(c, "layer is not a linear-attention layer with weights set");
        return -1;
    }
    if (z && c->lin_weights_set[c->layer_to_lin[layer]] != 2) {
        fail(c, "z given but no norm weight was set for the layer");
        return -1;
    }
    cudaSetDevice(g.device);
    if (mfc_join(c)) return -1;  // a GatedDeltaNet launch may still be running on the side queue
    const int slot = c->n_state_slots - 1;  // hook slot
    const size_t ssm_elems = (size_t)g.linear_num_v_heads * GDN_DIM * GDN_DIM;
    float *ring = c->conv + (size_t)slot * CONV_TAPS * c->conv_dim;
    const size_t row = sizeof(float) * c->conv_dim;
    CK(cudaMemcpyAsync(ring + c->conv_dim, conv_state, 3 * row, cudaMemcpyHostToDevice, c->stream));
    CK(cudaMemcpyAsync(c->ssm + (size_t)slot * ssm_elems, ssm_state, sizeof(float) * ssm_elems,
                       cudaMemcpyHostToDevice, c->stream));
    const size_t vd = sizeof(float) * g.linear_num_v_heads * GDN_DIM;
    const size_t hd = sizeof(float) * g.linear_num_v_heads;
    CK(cudaMemcpyAsync(c->st_qkv, qkv, row, cudaMemcpyHostToDevice, c->stream));
    if (z) CK(cudaMemcpyAsync(c->st_z, z, vd, cudaMemcpyHostToDevice, c->stream));
    CK(cudaMemcpyAsync(c->st_alpha, alpha, hd, cudaMemcpyHostToDevice, c->stream));
    CK(cudaMemcpyAsync(c->st_beta, beta, hd, cudaMemcpyHostToDevice, c->stream));
    c->h_gdn_items.resize(1);
    c->h_gdn_items[0].w_layer = c->layer_to_lin[layer];
    c->h_gdn_items[0].state_idx = slot;
    c->h_gdn_items[0].slot = 0;  // history sits in slots 1..3
    c->h_gdn_items[0].pad = 0;
    if (launch_gdn(c, 1, c->st_qkv, z ? c->st_z : nullptr, c->st_alpha, c->st_beta, c->st_gout)) return -1;
    // advanced history = old rows 1, 2 and the new input = slots 2, 3, 0
    CK(cudaMemcpyAsync(conv_state, ring + 2 * (size_t)c->conv_dim, 2 * row, cudaMemcpyDeviceToHost, c->stream));
    CK(cudaMemcpyAsync(conv_state + 2 * (size_t)c->conv_dim, ring, row, cudaMemcpyDeviceToHost, c->stream));
    CK(cudaMemcpyAsync(ssm_state, c->ssm + (size_t)slot * ssm_elems, sizeof(float) * ssm_elems,
                       cudaMemcpyDeviceToHost, c->stream));
    CK(cudaMemcpyAsync(out, c->st_gout, vd, cudaMemcpyDeviceToHost, c->stream));
    return check_status(c);
}

}  // extern "C"
#pragma GCC visibility pop
