// Host-visible launch interface of the sm_100a kernels.  The context layer
// (ctx.cu) builds the item lists; the kernels know nothing about sequences or
// layers beyond the indices stored in an item.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

namespace mfc {

constexpr int HEAD_DIM = 256;      // full-attention head dim
constexpr int GDN_DIM = 128;       // GatedDeltaNet key dim == value dim
constexpr int KV_TILE = 32;        // cache rows per pipeline stage (bf16 cache)
constexpr int KV_TILE_F32 = 16;    // same for the fp32 cache
constexpr int MERGE_GROUP = 8;     // partials merged by one CTA at the first level of a unit's merge
constexpr int MAX_SPLITS = 64;     // most first-level groups of one unit (second-level fan-in)
constexpr int MAX_UNIT_PARTS = MERGE_GROUP * MAX_SPLITS;  // most CTAs that may share one (item, kv head) unit
constexpr int PHASE_TRACE_WORDS = 8;  // timestamps per CTA of the optional phase trace
constexpr int CONV_TAPS = 4;

// ---------------------------------------------------------------- GatedDeltaNet
struct GdnItem {
    int32_t w_layer;    // index into the per-layer weight arrays
    int32_t state_idx;  // index of the (layer, sequence) state slot
    int32_t slot;       // ring slot the new conv input is written to (step % 4)
    int32_t pad;
};

constexpr int INLINE_ITEMS = 64;       // GatedDeltaNet launches of at most this many items carry them in the kernel's parameters (1 KiB)
constexpr int GQA_INLINE_ITEMS = 128;  // the same for the full-attention launches (4 KiB: the benchmark's 120 items; a
                                       // table in device memory costs every CTA two more dependent reads at its start)

struct GdnParams {
    float *ssm_base;          // [state][Hv][128 value][128 key]
    float *conv_base;         // [state][4 slots][conv_dim]
    const uint16_t *conv_w;   // [w_layer][conv_dim][4] bf16
    const float *a_log;       // [w_layer][Hv]
    const uint16_t *dt_bias;  // [w_layer][Hv] bf16
    const uint16_t *norm_w;   // [w_layer][128] bf16
    const GdnItem *items;     // device; nullptr: the items are `inline_items` (no copy precedes the launch)
    GdnItem inline_items[INLINE_ITEMS];
    const float *qkv;         // [n][conv_dim]
    const float *z;           // [n][Hv*128] or nullptr
    const float *alpha;       // [n][Hv]
    const float *beta;        // [n][Hv]
    float *out;               // [n][Hv*128]
    int n_items, Hv, Hk, conv_dim;
    float eps;
};

// rows_per_cta in {32, 64, 128}: value rows of one head handled by one CTA;
// 128 / rows_per_cta CTAs form a thread-block cluster per (item, head).
cudaError_t launch_gdn_decode(const GdnParams &p, int rows_per_cta, cudaStream_t stream);

// ---------------------------------------------------------------- full attention
struct GqaItem {
    int32_t kv_slot;     // (full layer index * n_seqs + seq): selects the cache rows
    int32_t local_len;   // rows held locally, the row appended by this step included
    int32_t pos;         // absolute position of the token (RoPE angle)
    int32_t append_row;  // local row that receives k,v, or -1 when another context owns it
    int32_t tile_begin;  // index, in the launch-wide tile sequence, of the first tile of kv head 0;
                         //   every kv head of the item has max(1, ceil(local_len / tile rows)) tiles
    int32_t pad0;        // 0, or the tiles every kv head of the item occupies in the tile sequence when the plan pads
                         //   units to whole CTA runs (a multiple of tiles_per_cta, >= the head's own tiles)
    int32_t pad1;
    int32_t in_idx;      // index of the item's q/gate/k/v/out rows
};

struct GqaParams {
    void *k_base;            // cache base pointers (for the append)
    void *v_base;
    const GqaItem *items;    // device; nullptr: the items are `inline_items` (no copy precedes the launch)
    GqaItem inline_items[GQA_INLINE_ITEMS];
    int n_items;
    int total_ctas;
    // The tiles of all (item, kv head) units form one sequence; CTA c works on tiles
    // [c * tiles_per_cta, (c+1) * tiles_per_cta) of it, across unit boundaries.
    int tiles_per_cta;
    int total_tiles;
    const float *q;          // [n][H][256]
    const float *gate;       // [n][H][256] or nullptr
    const float *k;          // [n][Hkv][256]
    const float *v;          // [n][Hkv][256]
    float *out;              // final mode: [n][H][256]
    float *po, *pm, *pl;     // partial mode outputs: item i at po + i*po_item_stride ([H][256]) and
    size_t po_item_stride;   //   pm/pl + i*pml_item_stride ([H]); dense = H*256 and H, packed per item
    size_t pml_item_stride;  //   [o | m | l] = H*256 + 2H for both
    float *sc_o, *sc_m, *sc_l;  // split-K scratch, one slot per CTA
    unsigned *tickets;       // [n][Hkv], zero between launches
    unsigned *group_tickets; // one per scratch slot, zero between launches: arrivals of a first-level merge group
    const float *inv_freq;   // [rotary_dim/2]
    unsigned *status;
    int H, Hkv, group;       // group = H / Hkv <= 16
    int rotary_dim;
    int cap_rows;            // cache rows reserved per (kv_slot, kv head)
    int partial_mode;        // 0: gated final output, 1: un-normalised partials
    float scale;             // 1/sqrt(head_dim)
    // Fused prologue of the projection outputs (all optional):
    int q_row_stride;        // floats between consecutive head rows of q (256 packed; 512 when q and gate
    int gate_row_stride;     //   are interleaved per head as the q projection emits them), same for gate
    const uint16_t *qnorm_w; // [full layer][256] bf16 per-head RMSNorm weights of q, or nullptr
    const uint16_t *knorm_w; // same for k
    int n_seqs;              // kv_slot / n_seqs = full-layer index of an item
    float norm_eps;
    int n_kv_slots;          // items are checked against it (kv_slot) and against cap_rows (local_len, append_row)
    int coop_merge;          // 1: the launch is cooperative (every CTA resident): units shared by more than
                             //    MERGE_GROUP CTAs are merged by their sharers together (they wait for one another)
    // Diagnostics (all off by default):
    unsigned wait_spins;     // poll limit of the bounded mbarrier waits; 0 = default
    int inject_lost_load;    // 1: CTA 0 arms the barrier of its first tile and issues no load for it, so that its
                             //    bounded wait runs out with nothing in flight (exercises the failure path)
    unsigned long long *phase_trace;  // [total_ctas][PHASE_TRACE_WORDS] globaltimer stamps, or nullptr
    // Fused exchange of the KV-sequence split (partial_mode only): when peer_recv != nullptr the merged partial of
    // item i goes, instead of po/pm/pl, to the receive buffer of the rank that finishes the item,
    //   peer_recv[i / items_per_dest] + ((size_t)my_rank * items_per_dest + i % items_per_dest) * po_item_stride
    // as one block [o | m | l], through peer-mapped pointers (plain stores over NVLink); the last CTA
    // of the launch then publishes `flag_value` in slot my_rank of every peer's flag array.
    float *const *peer_recv;             // device array [world] of device pointers
    unsigned *const *peer_flags;         // device array [world] of device pointers to [world] flags
    unsigned *done_counter;              // zero between launches
    int items_per_dest, my_rank, world;
    unsigned flag_value;
};

cudaError_t launch_gqa_decode_bf16(const CUtensorMap &kmap, const CUtensorMap &vmap,
                                   const GqaParams &p, cudaStream_t stream);
cudaError_t launch_gqa_decode_f32(const CUtensorMap &kmap, const CUtensorMap &vmap,
                                  const GqaParams &p, cudaStream_t stream);
// one-time opt-in to large dynamic shared memory
cudaError_t gqa_decode_configure();
cudaError_t gqa_decode_f32_configure();
// CTAs of the decode kernel that the current device holds at once (0 when it cannot launch cooperatively): the
// largest grid that may be launched with GqaParams::coop_merge.  Call after the configure function.
int gqa_decode_bf16_coop_capacity();
int gqa_decode_f32_coop_capacity();

// Merge of gathered partials.  Part r of o/m/l starts part_stride floats after
// part r-1; part_stride 0 means densely packed [n_parts][n][H][256] / [n_parts][n][H].
// flags != nullptr (n_parts <= 128): every CTA first waits, bounded by `spins` polls of about a microsecond each (0: about
// two seconds, enough for ranks that are out of step by a host hiccup), until flags[r] has reached
// flag_value for every part r (the fused exchange's "rank r's stores have landed"); a wait that runs out sets
// STATUS_PEER_TIMEOUT in *status.
cudaError_t launch_lse_merge_gate(int n_parts, int n, int H, const float *o_parts,
                                  const float *m_parts, const float *l_parts, size_t part_stride,
                                  const float *gate, float *out, cudaStream_t stream,
                                  size_t o_item_stride = 0, size_t ml_item_stride = 0,
                                  const unsigned *flags = nullptr, unsigned flag_value = 0, unsigned spins = 0,
                                  unsigned *status = nullptr);

// Gather of a step's query rows across the ranks of a KV split: rank my_rank's own_floats floats, at offset
// my_rank * own_floats of its table peer_rows[my_rank], are stored at the same offset of every peer's table
// peer_rows[r]; then flags are exchanged (peer_flags[r][my_rank] = flag_value; wait, at most `spins` polls of half a
// microsecond, two seconds by default, for my_flags[r] >= flag_value from every peer).  When the kernel has ended the
// whole table is in this GPU's memory.  A wait that runs out sets STATUS_PEER_TIMEOUT in *status.
cudaError_t launch_q_rows_gather(float *const *peer_rows, unsigned *const *peer_flags, const unsigned *my_flags,
                                 unsigned *done_counter, size_t own_floats, int my_rank, int world,
                                 unsigned flag_value, unsigned spins, unsigned *status, cudaStream_t stream);

// RoPE on packed q [H][256], k [Hkv][256] in place (parity hook).
// out[i] *= sigmoid(gate[i]) for n floats (n a multiple of 4): the gate applied after the fact, with the arithmetic
// of the fused epilogue, when the gate logits arrive later than q, k and v.
cudaError_t launch_sigmoid_gate(float *out, const float *gate, size_t n, cudaStream_t stream);
cudaError_t launch_rope(float *q, float *k, int H, int Hkv, int rotary_dim, int pos,
                        const float *inv_freq, cudaStream_t stream);

// Layout conversions between the wire/reference layout [pos][kv_head][256] fp32
// and the cache layout [kv_head][row][256] of the context's storage type.
// Wire row i is whole-sequence position pos0 + i; with world > 1 only the rows
// of this rank's blocks are stored (block-cyclic split).
cudaError_t launch_kv_pack(const float *src_rows, void *dst_cache, int n_rows, int Hkv,
                           int cap_rows, int kv_bf16, int pos0, int rank, int world, int block,
                           cudaStream_t stream);
cudaError_t launch_kv_unpack(const void *src_cache, float *dst_rows, int n_rows, int Hkv,
                             int cap_rows, int kv_bf16, cudaStream_t stream);

// ---------------------------------------------------------------- prefill
struct PrefillAttnParams {
    const __nv_bfloat16 *gate;  // [T][H][256] bf16, or nullptr
    __nv_bfloat16 *out;         // [T][H][256] bf16
    const float *cos_sin;       // [T][32] (cos, sin) pairs written by the append kernel
    int T, H, Hkv, group;
    int start_pos;              // absolute position of token 0
    int rotary_dim;             // <= 64
    int kv_slot, cap_rows;
    float scale;
    unsigned *status;
};
cudaError_t gqa_prefill_configure();
// RoPE table, rotated K and V of T tokens stored into the cache (bf16 inputs).
cudaError_t launch_prefill_kv_append(const void *k_bf16, const void *v_bf16, void *k_cache, void *v_cache,
                                     int kv_bf16, float *cos_sin, const float *inv_freq, int T, int Hkv,
                                     int rotary_dim, int start_pos, size_t slot_row0, int cap_rows, int rank,
                                     int world, int block, cudaStream_t stream);
// qmap: 3-D map over q [T][H][256] bf16 with box {64, 1, 128}; kmap/vmap: cache maps with box {64, 64}.
cudaError_t launch_gqa_prefill(const CUtensorMap &qmap, const CUtensorMap &kmap, const CUtensorMap &vmap,
                               const PrefillAttnParams &p, cudaStream_t stream);

struct GdnPrefillParams {
    const void *qkv;          // [T][conv_dim] bf16
    const void *z;            // [T][Hv*128] bf16 or nullptr
    const void *alpha, *beta; // [T][Hv] bf16
    void *out;                // [T][Hv*128] bf16
    float *ssm;               // this (layer, sequence)'s state [Hv][128][128]
    float *ring;              // its conv ring [4][conv_dim]
    int slot0;                // ring slot of token 0 (conv step & 3)
    const uint16_t *conv_w;   // the layer's weights
    const float *a_log;
    const uint16_t *dt_bias, *norm_w;
    void *q_hat, *k_hat;      // scratch [T][Hk*128] bf16
    float *v_io;              // scratch [T][Hv*128] fp32 (v in, raw read-out out)
    float *lg, *beta_gate;    // scratch [T][Hv]
    void *w_tilde;            // scratch [T][Hv*128] bf16
    void *w_mask;             // scratch [T][Hv*64] bf16
    unsigned *status;         // device status word (bounded waits that expired)
    int T, Hk, Hv, conv_dim;
    float eps;
};
cudaError_t gdn_prefill_configure();
// Tensor maps over the first T rows of the scratch arrays (128-byte swizzle, 64-row boxes):
// w_tilde, q^, k^ and w_mask with 64 bf16 columns per box, v_io with 32 fp32 columns per box.
struct GdnPrefillMaps {
    CUtensorMap wt, q, k, wm, ut;
};
cudaError_t launch_gdn_prefill(const GdnPrefillParams &p, const GdnPrefillMaps &m, cudaStream_t stream);

// ---------------------------------------------------------------- folded MLA attention (mla_decode.cu)
constexpr int MLA_RANK = 512;  // kv_lora_rank: latent dims of a cached row, and dims of an output row
constexpr int MLA_ROPE = 64;   // qk_rope_head_dim
struct MlaParams {
    const float *q_prime;   // [H][512]
    const float *q_pe;      // [H][64]
    float *out;             // [H][512]
    float *part_o;          // [n_chunks][H][512] un-normalised partials (n_chunks > 1)
    float *part_m, *part_l; // [n_chunks][H]
    unsigned *status;
    int H, cache_len;
    int n_head_blocks;      // ceil(H / 16)
    int n_chunks;           // chunks of rows_per_chunk positions (a multiple of 16)
    int rows_per_chunk;
    int cache_bf16;         // 0: fp32 cache (the reference's storage), 1: bf16 cache
    float scale;            // softmax scale
    unsigned wait_spins;    // poll limit of the bounded waits; 0 = default
};
cudaError_t mla_decode_configure();
// fp32 cache: lat_map [cache_len][512], rope_map [cache_len][64], boxes of 32 floats x 16 rows, 128-byte swizzle;
// bf16 cache (p.cache_bf16): the same arrays as bf16, boxes of 64 elements x 32 rows.
cudaError_t launch_mla_decode(const CUtensorMap &lat_map, const CUtensorMap &rope_map, const MlaParams &p,
                              cudaStream_t stream);

// 4-bit group-64 dequant matvec (matvec.cu): for every matrix m of the batch and vector v,
// out[m][v][r] = sum_c (nibble * scale + bias)(m; r, c) * x[v][c]; the matrices share in_dim and x; n_vec in 1..8.
constexpr int MATVEC_MAX_MATS = 8;
struct MatvecBatch {
    int n_mat;
    const uint32_t *w[MATVEC_MAX_MATS];
    const uint16_t *scales[MATVEC_MAX_MATS], *biases[MATVEC_MAX_MATS];
    float *out[MATVEC_MAX_MATS];
    int out_dim[MATVEC_MAX_MATS];
    int group_begin[MATVEC_MAX_MATS];  // filled by the launcher: first row tile of each matrix
    int total_groups;                  // filled by the launcher: row tiles in all
    unsigned *sched;                   // two zeroed words in device memory: next tile, finished CTAs (one-vector kernel);
                                       // consecutive launches must not share them (they may overlap)
    unsigned *status;                  // the context's status word
    unsigned spins;                    // poll limit of the kernel's bounded waits
    int sb_bulk;                       // filled by the launcher: scales and biases travel with the weight stages
    unsigned long long *trace;         // optional [CTA][PHASE_TRACE_WORDS] nanosecond stamps of the one-vector kernel
    int overlap;                       // launch as a programmatic dependent launch (the kernel waits by itself)
    int inject_lost_load;              // test hook: CTA 0 arms its first stage and requests nothing for it
};
// Tensor maps of the batch's matrices for the one-vector kernel: the weights of matrix m as a 2-D byte array
// [out_dim][in_dim / 2], boxes of 16 rows x 128 bytes, 128-byte swizzle; its scales and its biases as
// [out_dim][in_dim / 64] 16-bit arrays, boxes of 16 rows x 32 groups, no swizzle (only when in_dim is a multiple of
// 512: rows of 16-byte multiples).
struct alignas(64) MatvecMaps {
    CUtensorMap w[MATVEC_MAX_MATS], sc[MATVEC_MAX_MATS], bi[MATVEC_MAX_MATS];
};
size_t dequant_matvec_4bit_smem(int in_dim, int n_vec);
// maps: needed when n_vec == 1; grid_out (optional): the grid of the one-vector kernel, for readers of its phase trace
cudaError_t launch_dequant_matvec_4bit(MatvecBatch mb, const float *x, int in_dim, int n_vec, int n_sms,
                                       cudaStream_t stream, const MatvecMaps *maps = nullptr, int *grid_out = nullptr);

// Per-thread message of the last failure that had no context (ctx.cu).
std::string &no_ctx_error();

}  // namespace mfc
