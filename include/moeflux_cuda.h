/*
 * moeflux_cuda.h - C ABI of the B200 (sm_100a) attention backend for moeflux.
 *
 * The library replaces the attention sub-block of moeflux's per-layer forward:
 * what `full_attn_layer_forward` does between "q/k/v projections are ready"
 * and "o_proj input is ready" (crates/moeflux/src/riir/full_attn_forward.rs:
 * 278-389: RoPE, KV append, SDPA, sigmoid gate) and what
 * `linear_attn_layer_forward` does with its five GatedDeltaNet kernels
 * (crates/moeflux/src/riir/linear_attn_forward.rs:607-664: conv1d_step,
 * rms_norm_qk, compute_decay_beta, gated_delta_net_step, gated_rms_norm),
 * together with the per-layer state those steps own and the state calls of the
 * public surface (crates/moeflux-sys/metal_infer/moeflux.h:88-104, 627-639).
 *
 * Conventions follow moeflux.h: opaque context, NULL on construction failure;
 * `int` results are 0 on success and -1 on error unless stated; every buffer is
 * caller-allocated and caller-owned; outputs are fully overwritten.  All
 * pointers are HOST pointers unless the function name ends in `_dev`, in which
 * case they are device pointers on the context's device and the call is
 * asynchronous on the context's stream.  One thread per context at a time;
 * several contexts may be used from different threads.
 *
 * There is no CPU fallback: every entry point that computes runs CUDA kernels
 * and fails (-1, message in mfc_last_error) when no sm_100 device is usable.
 */
#ifndef MOEFLUX_CUDA_H
#define MOEFLUX_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct mfc_ctx mfc_ctx;

enum { MFC_KV_F32 = 0, MFC_KV_BF16 = 1 };

/* Geometry and placement.  The geometry fields mirror `Variant`
 * (crates/moeflux/src/riir/variants.rs:132-250); mfc_default_config() fills
 * them with the Qwen3.5-397B-A17B values (variants.rs:383-423). */
typedef struct mfc_config {
    int32_t num_layers;          /* 60 */
    int32_t full_attn_interval;  /* 4: layer i is full attention iff (i+1) % interval == 0 */
    int32_t num_attn_heads;      /* 32 */
    int32_t num_kv_heads;        /* 2;  num_attn_heads / num_kv_heads must be <= 16 */
    int32_t head_dim;            /* 256 (the only supported value) */
    int32_t rotary_dim;          /* 64 (multiple of 4, <= head_dim) */
    float   rope_theta;          /* 1e7 */
    int32_t linear_num_v_heads;  /* 64 */
    int32_t linear_num_k_heads;  /* 16 */
    int32_t linear_key_dim;      /* 128 (only) */
    int32_t linear_value_dim;    /* 128 (only) */
    int32_t conv_kernel_size;    /* 4 (only) */
    float   rms_norm_eps;        /* 1e-6 */
    int32_t kv_dtype;            /* MFC_KV_F32 | MFC_KV_BF16: storage type of the KV cache */
    int32_t max_seq;             /* positions per sequence (whole sequence, before any split) */
    int32_t n_seqs;              /* independent sequences (seq_id in [0, n_seqs)) */
    int32_t device;              /* CUDA device ordinal */
    /* KV-sequence split across contexts (one per GPU): this context stores the
     * positions p with (p / kv_block) % kv_world == kv_rank.  kv_world = 1
     * keeps everything here. */
    int32_t kv_rank;
    int32_t kv_world;
    int32_t kv_block;            /* positions per block of the cyclic split (multiple of 32) */
    int32_t max_batch;           /* most (layer, sequence) items one batched call may carry */
    int32_t snapshot_version;    /* 1 (C engine's header, 8 words) or 2 (Rust port's, 10 words) */
    int32_t max_prefill;         /* most tokens one mfc_linear_attn_prefill_dev call may carry
                                    (sizes its scratch); 0 = min(max_seq, 8192) */
} mfc_config;

/* Fills *cfg with the A17B geometry, bf16 KV off (fp32), max_seq 8192,
 * n_seqs 1, device 0, no KV split, max_batch = num_layers * n_seqs. */
void mfc_default_config(mfc_config *cfg);

/* Replaces mf_init_model / RsCtx::open for this path (moeflux.h:55,
 * crates/moeflux/src/riir/mod.rs:270).  Allocates the KV caches, the
 * GatedDeltaNet states (zeroed) and all working memory up front.  No entry
 * point of the hot path allocates device memory afterwards; the exceptions are
 * mfc_exchange_create (once, at set-up) and the host-pointer test hooks
 * mfc_dequant_matvec_4bit and mfc_mla_sdpa_folded (a temporary allocation per call).  Every allocation
 * of the context sits between two bands of 0xFF bytes that no kernel may touch
 * (mfc_check_guards).  NULL on failure (mfc_last_error(NULL)). */
mfc_ctx *mfc_open(const mfc_config *cfg);
/* mf_free_model (moeflux.h:66).  No-op on NULL. */
void mfc_free(mfc_ctx *ctx);
/* Message of the last failure on this context (or of mfc_open when ctx is
 * NULL).  Points to storage owned by the library. */
const char *mfc_last_error(const mfc_ctx *ctx);
/* The geometry the context was opened with. */
int mfc_get_config(const mfc_ctx *ctx, mfc_config *out);
/* cudaStream_t of the context, as void*; `_dev` calls are ordered on it. */
void *mfc_stream(mfc_ctx *ctx);
/* The context's second queue (see mfc_join), as void*: for recording events around what runs there. */
void *mfc_side_stream(mfc_ctx *ctx);
/* Makes the context issue all further work on the caller's stream (a
 * cudaStream_t on the context's device; NULL = the legacy default stream).  The
 * caller keeps ownership and must keep the stream alive while the context uses
 * it.  Waits for the work already queued on the previous stream. */
int mfc_set_stream(mfc_ctx *ctx, void *stream);
/* Blocks until the context's stream is idle; -1 if a kernel gave up since the
 * last call (a bounded wait ran out, or an item failed the kernel's range
 * checks): the message names which.  The report is cleared and the context
 * stays usable. */
int mfc_synchronize(mfc_ctx *ctx);

/* Per-layer constant tensors of a GatedDeltaNet layer, read where the reference
 * reads them from the weight file (linear_attn_forward.rs:507-510):
 * conv1d.weight bf16 [conv_dim][4], A_log f32 [v_heads], dt_bias bf16 [v_heads],
 * norm.weight bf16 [value_dim] (may be NULL when the gated norm is never used). */
int mfc_set_linear_weights(mfc_ctx *ctx, int32_t layer, const uint16_t *conv_w_bf16,
                           const float *a_log, const uint16_t *dt_bias_bf16,
                           const uint16_t *norm_w_bf16);
/* q_norm / k_norm weights (bf16 [head_dim] each) of a full-attention layer, as
 * read at crates/moeflux/src/riir/full_attn_forward.rs:257-276. */
int mfc_set_full_attn_norm_weights(mfc_ctx *ctx, int32_t layer, const uint16_t *q_norm_bf16,
                                   const uint16_t *k_norm_bf16);

/* ------------------------------------------------------------------------
 * The hot path, one (layer, sequence) item per call.
 * ---------------------------------------------------------------------- */

/* Full-attention decode step of layer `layer` for sequence `seq_id` at absolute
 * position `pos`: RoPE(q,k) -> append k,v -> SDPA over the pos+1 cached rows ->
 * sigmoid gate.  Replaces full_attn_forward.rs:278-389 (apply_rotary_emb, the
 * KV append, encode_attn_scores/softmax/values_batched + encode_sigmoid_gate of
 * crates/moeflux/src/riir/gpu_attn.rs:119-235, and the sdpa_cpu fallback).
 *   q, gate, out: [num_attn_heads * head_dim];  k, v: [num_kv_heads * head_dim].
 * `pos` must equal the layer's current length (full_attn_forward.rs:73-78);
 * -1 on mismatch, on overflow of max_seq, on a linear layer index, NULL args. */
int mfc_full_attn_step(mfc_ctx *ctx, int32_t layer, int32_t seq_id, int32_t pos, const float *q,
                       const float *gate, const float *k, const float *v, float *out);

/* GatedDeltaNet decode step of layer `layer` for sequence `seq_id`:
 * conv1d+SiLU (history advanced) -> q/k norm -> decay/beta -> delta-rule state
 * update and read-out -> gated RMSNorm when z != NULL.  Replaces the five
 * encoders of crates/moeflux/src/riir/gpu_linear_attn.rs:54-202 as sequenced at
 * linear_attn_forward.rs:607-664.
 *   qkv: [conv_dim] (q | k | v);  z: [v_heads*value_dim] or NULL;
 *   alpha, beta: [v_heads];  out: [v_heads*value_dim]. */
int mfc_linear_attn_step(mfc_ctx *ctx, int32_t layer, int32_t seq_id, const float *qkv,
                         const float *z, const float *alpha, const float *beta, float *out);

/* ------------------------------------------------------------------------
 * Batched forms: n items, item i = (layers[i], seq_ids[i]); inputs and outputs
 * are packed [n][...] in item order.  An item pair may appear once per call.
 * The reference runs one sequence (seq_id ignored, moeflux.h:15-17); these are
 * the same step applied to n independent (layer, sequence) states in one
 * launch.  n <= max_batch.
 * ---------------------------------------------------------------------- */
int mfc_full_attn_step_batched(mfc_ctx *ctx, int32_t n, const int32_t *layers,
                               const int32_t *seq_ids, const int32_t *pos, const float *q,
                               const float *gate, const float *k, const float *v, float *out);
int mfc_linear_attn_step_batched(mfc_ctx *ctx, int32_t n, const int32_t *layers,
                                 const int32_t *seq_ids, const float *qkv, const float *z,
                                 const float *alpha, const float *beta, float *out);

/* Full-attention step taken from the projection outputs as the reference has
 * them right after its q/k/v matvecs (full_attn_forward.rs:233-236): q_proj is
 * [n][num_attn_heads][q (head_dim) | gate (head_dim)] interleaved per head.  The
 * kernel de-interleaves (full_attn_forward.rs:238-254), applies the per-head
 * RMSNorm of q and k with the weights of mfc_set_full_attn_norm_weights
 * (:256-276), then RoPE, append, SDPA and the sigmoid gate as
 * mfc_full_attn_step does.  k, v: [n][num_kv_heads*head_dim]; out:
 * [n][num_attn_heads*head_dim].  Host pointers; the _dev form takes device
 * pointers and is asynchronous. */
int mfc_full_attn_step_qproj_batched(mfc_ctx *ctx, int32_t n, const int32_t *layers,
                                     const int32_t *seq_ids, const int32_t *pos,
                                     const float *q_proj, const float *k, const float *v,
                                     float *out);
int mfc_full_attn_step_qproj_batched_dev(mfc_ctx *ctx, int32_t n, const int32_t *layers,
                                         const int32_t *seq_ids, const int32_t *pos,
                                         const float *q_proj, const float *k, const float *v,
                                         float *out);

/* One token step of the attention sub-blocks of a whole layer stack, host
 * pointers: n_full full-attention items and n_lin GatedDeltaNet items (either
 * may be 0), arguments as in the two batched calls above.  It is what
 * RsCtx::eval_token (crates/moeflux/src/riir/mod.rs:1218) does across its layer
 * loop for this path, for layers whose inputs do not depend on one another's
 * outputs; the two groups run on two queues so that the host<->device copies of
 * one overlap the kernel of the other.  The input copies into staging buffers
 * are queued first and the arguments validated under them, before any kernel:
 * on -1 no cache or state has changed.  On a context of a KV split
 * (kv_world > 1, exchange connected) the full-attention group is the whole
 * step's item list sorted by finishing rank, and gate / full_out cover the
 * items_per_rank items this rank finishes (see mfc_exchange_create).  With the
 * tuning "exchange_gather_q" 1 (set alike on every rank) q, too, holds only the
 * rows of the items this rank finishes, [items_per_rank][num_attn_heads*head_dim]:
 * every rank stores its rows into the peers' memory over the links instead of
 * every rank's host sending all rows over PCIe (an eighth of the bytes at
 * kv_world 8); the flags that order it are step numbers, and the waits bounded
 * like the merge's. */
int mfc_eval_token_attn(mfc_ctx *ctx, int32_t n_full, const int32_t *full_layers,
                        const int32_t *full_seqs, const int32_t *pos, const float *q,
                        const float *gate, const float *k, const float *v, float *full_out,
                        int32_t n_lin, const int32_t *lin_layers, const int32_t *lin_seqs,
                        const float *qkv, const float *z, const float *alpha, const float *beta,
                        float *lin_out);

/* Device-pointer forms: same meaning, q/gate/k/v/out (qkv/z/alpha/beta/out) are
 * device pointers, layers/seq_ids/pos stay host arrays.  Asynchronous on
 * mfc_stream(ctx); the per-sequence lengths advance at call time. */
int mfc_full_attn_step_batched_dev(mfc_ctx *ctx, int32_t n, const int32_t *layers,
                                   const int32_t *seq_ids, const int32_t *pos, const float *q,
                                   const float *gate, const float *k, const float *v, float *out);
int mfc_linear_attn_step_batched_dev(mfc_ctx *ctx, int32_t n, const int32_t *layers,
                                     const int32_t *seq_ids, const float *qkv, const float *z,
                                     const float *alpha, const float *beta, float *out);

/* KV-sequence split (kv_world > 1): same as mfc_full_attn_step_batched_dev but
 * the context attends over the positions it stores only and writes, per item,
 * the un-normalised partial of every head: o_part [n][heads][head_dim],
 * m_part [n][heads] (max scaled score, -inf if no row), l_part [n][heads]
 * (sum of exp(s - m)).  The row at `pos` is appended by the context that owns
 * it.  Gather the partials of all contexts (NCCL all-gather) and finish with
 * mfc_lse_merge_gate_dev. */
int mfc_full_attn_partial_batched_dev(mfc_ctx *ctx, int32_t n, const int32_t *layers,
                                      const int32_t *seq_ids, const int32_t *pos, const float *q,
                                      const float *k, const float *v, float *o_part,
                                      float *m_part, float *l_part);
/* out[i,h,:] = (sum_r e^{m_r-M} o_r / sum_r e^{m_r-M} l_r) * sigmoid(gate[i,h,:]),
 * part r of o/m/l starts part_stride floats after part r-1 (so one gathered
 * buffer [n_parts][o | m | l] works); part_stride 0 = densely packed
 * [n_parts][n][heads][...].  gate may be NULL (no gate). */
int mfc_lse_merge_gate_dev(mfc_ctx *ctx, int32_t n_parts, int32_t n, const float *o_parts,
                           const float *m_parts, const float *l_parts, size_t part_stride,
                           const float *gate, float *out);

/* Prefill of n_tokens tokens of one full-attention layer in one call, device
 * pointers, bf16 activations: token t (absolute position start_pos + t) gets
 * exactly what mfc_full_attn_step computes for it -- RoPE, append, causal SDPA
 * over rows [0, start_pos + t], sigmoid gate.  The reference prefills by
 * running its decode step per token (RsCtx::eval_prompt,
 * crates/moeflux/src/riir/mod.rs:1196-1214); this is the batched form on the
 * tcgen05 tensor cores.  q, gate, out: [n_tokens][num_attn_heads][256] bf16
 * (gate may be NULL); k, v: [n_tokens][num_kv_heads][256] bf16.  start_pos must
 * equal the layer's current length.  Needs a bf16 KV cache and kv_world == 1.
 * Asynchronous on mfc_stream(ctx). */
int mfc_full_attn_prefill_dev(mfc_ctx *ctx, int32_t layer, int32_t seq_id, int32_t start_pos,
                              int32_t n_tokens, const void *q_bf16, const void *gate_bf16,
                              const void *k_bf16, const void *v_bf16, void *out_bf16);

/* Prefill of n_tokens tokens of one GatedDeltaNet layer in one call, device
 * pointers, bf16 activations: equal to n_tokens calls of mfc_linear_attn_step
 * (which is how the reference prefills, mod.rs:1206-1212), computed as a causal
 * conv over the tokens followed by the delta rule in chunks of 64 tokens on the
 * tensor cores.  qkv: [n_tokens][conv_dim] bf16; z: [n_tokens][v_heads*128] bf16
 * or NULL; alpha, beta: [n_tokens][v_heads] bf16; out: [n_tokens][v_heads*128]
 * bf16.  n_tokens <= max_prefill.  Asynchronous on mfc_stream(ctx). */
int mfc_linear_attn_prefill_dev(mfc_ctx *ctx, int32_t layer, int32_t seq_id, int32_t n_tokens,
                                const void *qkv_bf16, const void *z_bf16, const void *alpha_bf16,
                                const void *beta_bf16, void *out_bf16);

/* Packed forms for an exchange that sends every item to one destination
 * (all-to-all by sequence): the partial of item i is one block
 * [o (heads*256) | m (heads) | l (heads)] at packed + i*(heads*258), so items
 * sorted by destination form contiguous, equal-sized send segments.  The merge
 * takes [n_parts][n] such blocks (what the all-to-all delivers for the n items
 * this context finishes) and writes the gated outputs of those n items. */
int mfc_full_attn_partial_packed_dev(mfc_ctx *ctx, int32_t n, const int32_t *layers,
                                     const int32_t *seq_ids, const int32_t *pos, const float *q,
                                     const float *k, const float *v, float *packed);
int mfc_lse_merge_gate_packed_dev(mfc_ctx *ctx, int32_t n_parts, int32_t n,
                                  const float *packed_parts, const float *gate, float *out);

/* Bulk import of state that already exists on the device (what a prefill, or a
 * prefix cache, hands over; the reference fills the same state token by token,
 * crates/moeflux/src/riir/mod.rs:1206-1212).  Asynchronous on mfc_stream(ctx).
 * kv_append_rows: rows [pos0, pos0+n_rows) of a full-attention layer, post-RoPE
 * K and V as [n_rows][num_kv_heads*head_dim] fp32; pos0 must equal the current
 * length; a context of a KV split keeps only the rows it owns.
 * linear_state_set: conv history [3][conv_dim] (oldest first) and ssm state
 * [v_heads][value][key] of a GatedDeltaNet layer. */
int mfc_kv_append_rows_dev(mfc_ctx *ctx, int32_t layer, int32_t seq_id, int32_t pos0,
                           int32_t n_rows, const float *k_rows, const float *v_rows);
int mfc_linear_state_set_dev(mfc_ctx *ctx, int32_t layer, int32_t seq_id,
                             const float *conv_state, const float *ssm_state);

/* ------------------------------------------------------------------------
 * Sequence state: mf_memory_clear / mf_memory_seq_rm / mf_memory_seq_pos_max
 * (moeflux.h:88-104; crates/moeflux/src/riir/state.rs:417-473) with seq_id
 * honoured.  seq_id = -1 applies to every sequence.
 * ---------------------------------------------------------------------- */
void mfc_memory_clear(mfc_ctx *ctx, int32_t seq_id);
/* Truncate to [0, p0); GatedDeltaNet layers are reset to the empty state.
 * p0 < 0 is 0; p1 < 0 or beyond the length means "to end".  Returns NONZERO on
 * success, 0 on failure (moeflux.h:98). */
int mfc_memory_seq_rm(mfc_ctx *ctx, int32_t seq_id, int32_t p0, int32_t p1);
/* Largest length over the sequence's full-attention layers (state.rs:460-473:
 * the reference returns the length, not length-1); -1 on NULL/bad seq_id. */
int mfc_memory_seq_pos_max(mfc_ctx *ctx, int32_t seq_id);

/* mf_state_size / mf_state_save / mf_state_load (moeflux.h:627-639;
 * crates/moeflux/src/riir/state_snapshot.rs:195-663), per sequence, in the
 * 'MFLX' wire format: KV rows fp32 [pos][kv_head][d], conv state [3][conv_dim],
 * ssm state [v_head][value][key].  A bf16 cache is widened on save and rounded
 * on load.  Only valid on a context with kv_world == 1.
 * size: 0 on NULL.  save: bytes written or -1.  load: 0 or -1, and on -1 the
 * state is unchanged (the buffer is validated before anything is written). */
size_t mfc_state_size(const mfc_ctx *ctx, int32_t seq_id);
long long mfc_state_save(mfc_ctx *ctx, int32_t seq_id, void *buf, size_t buf_len);
int mfc_state_load(mfc_ctx *ctx, int32_t seq_id, const void *buf, size_t buf_len);

/* Position-keyed snapshots of one sequence kept inside the context:
 * RsCtx::checkpoint_pos / restore_to / set_max_checkpoints / checkpoint_count
 * (crates/moeflux/src/riir/mod.rs:2015-2100).  checkpoint_pos stores the current
 * state under `pos` (overwriting an entry at the same pos) and, above the cap
 * (default 4), evicts the least recently stored entry that is neither pos 0 nor
 * the one just stored.  restore_to reloads the state stored under exactly `pos`
 * (-1 with "no checkpoint stored at position ..." otherwise) and drops every
 * entry with a larger position.  mfc_memory_clear drops them all;
 * mfc_memory_seq_rm leaves them.  0 on success, -1 on error. */
int mfc_checkpoint_pos(mfc_ctx *ctx, int32_t seq_id, int32_t pos);
int mfc_restore_to(mfc_ctx *ctx, int32_t seq_id, int32_t pos);
void mfc_set_max_checkpoints(mfc_ctx *ctx, int32_t n);
int mfc_checkpoint_count(const mfc_ctx *ctx, int32_t seq_id);

/* Host-only helpers (no GPU needed).
 * Block-cyclic KV split: rows of a sequence of whole length `len` that rank
 * `rank` of `world` stores, and the local row of position `pos` (-1 when
 * another rank owns it).  -1 on bad arguments. */
int mfc_kv_local_len(int32_t len, int32_t rank, int32_t world, int32_t block);
int mfc_kv_local_row(int32_t pos, int32_t rank, int32_t world, int32_t block);
/* The checks mfc_state_load runs before it writes anything (header fields, per
 * layer lengths, truncation; state_snapshot.rs:377-507) against a geometry.
 * Returns the snapshot's size in bytes, or -1 (reason in mfc_last_error(NULL)). */
long long mfc_snapshot_validate(const mfc_config *cfg, const void *buf, size_t buf_len);

/* ------------------------------------------------------------------------
 * Stateless parity hooks, GPU twins of the reference's diff-oracle hooks with
 * the same argument meaning.  Each stages its host arguments on the device,
 * runs the production kernel, and copies the result back.
 * ---------------------------------------------------------------------- */

/* mf_apply_rotary_emb (moeflux.h:151): q, k rotated in place at `pos`. */
int mfc_apply_rotary_emb(mfc_ctx *ctx, int32_t pos, float *q, float *k);
/* mf_sdpa_cpu (moeflux.h:179-182) on the GPU decode kernel: caches are
 * [kv_len][num_kv_heads*head_dim] fp32 host rows (post-RoPE K). Stored in the
 * context's kv_dtype before the kernel runs. */
int mfc_sdpa(mfc_ctx *ctx, int32_t kv_len, const float *q, const float *q_gate,
             const float *k_cache, const float *v_cache, float *out);
/* One GatedDeltaNet step on caller-held state: conv_state [3][conv_dim] and
 * ssm_state [v_heads][value_dim][key_dim] are read, advanced and written back
 * (mf_conv1d_step_cpu + state shift, mf_gated_delta_recurrence_cpu,
 * mf_rms_norm_gated_cpu in one call; moeflux.h:224-272). Uses the weights set
 * for `layer`. */
int mfc_linear_attn_step_stateless(mfc_ctx *ctx, int32_t layer, const float *qkv, const float *z,
                                   const float *alpha, const float *beta, float *conv_state,
                                   float *ssm_state, float *out);

/* Gated SDPA over a caller-held KV cache that allocates nothing.  It has no
 * counterpart in the reference.  It is for callers that cannot call cudaMalloc
 * where they need attention: a plugin inside a host application that budgets
 * every byte of device memory, a latency-critical path that must not enter the
 * driver's allocator, or a process whose own pool already owns all free memory.
 * Such a caller cannot open an mfc_ctx (mfc_open allocates caches and scratch).
 *
 * The caller passes every input and the output as device pointers on the
 * CURRENT device; the call is asynchronous on `stream` (a cudaStream_t):
 *   q, gate, out : [num_attn_heads][256] fp32; q is post-RoPE; gate may be NULL;
 *   k_cache, v_cache : [num_kv_heads][cap_rows][256] of kv_dtype (bf16 or fp32),
 *                      16-byte aligned, post-RoPE K; rows [0, kv_len) are used.
 * The split-K partials, chunk counters and work descriptor of the kernel live in
 * one fixed array inside the library's device image (about 4 MiB, held by every
 * GPU that loads the library until the process exits).  Limits that follow from
 * its size: num_kv_heads <= MFC_STATIC_MAX_KV_HEADS and
 * kv_len <= MFC_STATIC_MAX_ROWS; larger requests are refused with -1 and a
 * message (mfc_last_error(NULL)).  It calls no cudaMalloc / cudaFree and no
 * allocating library routine.
 *
 * All calls on a device share that array, and the array keeps the previous
 * call's contents (the entry point clears the counters it needs at zero on
 * `stream` before the kernel).  Two calls whose kernels may overlap on the GPU
 * (different streams, different threads) therefore race: serialise them.
 * The first call on each device resolves the array's device address and raises
 * the kernel's shared-memory limit; make that first call before any stream
 * capture begins.  Nothing is read from host memory after the call returns (the
 * work descriptor travels as a kernel argument).  The cache rows past kv_len
 * are never used, whatever they hold.  Returns 0 on success, -1 on error.
 *
 * mfc_sdpa_static_status(stream) waits for `stream` and reports what the kernels
 * of the calls since the previous status call found: 0, or -1 (a bounded wait on
 * a load ran out; message in mfc_last_error(NULL)).  It allocates nothing and
 * clears the report. */
#define MFC_STATIC_MAX_KV_HEADS 8
#define MFC_STATIC_MAX_ROWS 262144
int mfc_sdpa_static_dev(int32_t num_attn_heads, int32_t num_kv_heads, int32_t kv_dtype,
                        int32_t kv_len, int32_t cap_rows, const float *q, const float *gate,
                        const void *k_cache, const void *v_cache, float *out, void *stream);
int mfc_sdpa_static_status(void *stream);

/* ---- The step either side of the path: 4-bit affine-quantised projections ----
 * Replaces dequant_matvec_4bit_cpu (crates/moeflux/src/riir/cpu_matvec.rs:83-171) and the
 * GPU dispatch encode_matvec (riir/gpu_matvec.rs:84-129; kernels dequant_matvec_4bit_v3 /
 * _fast, shaders/shaders.metal:251-340, and the batched form :667) for the q/k/v/o_proj,
 * in_proj_qkv/z/a/b and out_proj products around the attention sub-block.
 *   w_packed [out_dim][in_dim/8] u32: eight nibbles per word, least significant nibble =
 *            lowest input feature;  scales, biases [out_dim][in_dim/64] bf16 bit patterns;
 *   out[v][r] = sum_c (nibble(r,c) * scale[r][c/64] + bias[r][c/64]) * x[v][c]
 * for n_vec (1..8) input vectors x [n_vec][in_dim] -> out [n_vec][out_dim], fp32, the
 * weights read once per pass.  in_dim must be a positive multiple of 64 (the reference's
 * InDimNotMultiple error).  One pass takes as many vectors as fit in shared memory
 * (n_vec * in_dim * 4.25 bytes beside 45 KB of staging: all 8 at in_dim 4096, 4 at 8192, 2 at
 * 16384); more vectors take further passes; in_dim itself is limited to 40,000 or so.
 * Arithmetic: the nibbles and a per-group integer form of x (31 bits relative to the group's
 * largest |x|) are multiplied exactly on the integer tensor cores; scales, biases and the sums
 * over groups are fp32.  Against the reference's fp32 product: 3e-6 (max-norm relative) on
 * N(0,1) inputs; a NaN or an infinity in x makes every output NaN.
 * _dev: device pointers (w_packed and x 16-byte aligned), asynchronous on mfc_stream(ctx).
 * The kernel is launched so that it may begin (fetching weights, scales and biases) before the
 * kernel queued ahead of it on the stream has finished; it waits for that kernel by itself
 * before it reads x or writes out.  The weights, scales and biases must therefore be complete
 * when the call is made if a kernel produces them (data copied or loaded earlier, the usual
 * case for model weights, needs nothing); the tuning "matvec_overlap" 0 restores plain
 * stream order.
 * The host-pointer form stages the operands in device memory for the call (a hook for
 * tests and bring-up, like mfc_sdpa).  Return 0 on success, -1 on error. */
#define MFC_MATVEC_GROUP_SIZE 64
#define MFC_MATVEC_MAX_VECS 8
int mfc_dequant_matvec_4bit_dev(mfc_ctx *ctx, const uint32_t *w_packed, const uint16_t *scales,
                                const uint16_t *biases, int32_t in_dim, int32_t out_dim, const float *x,
                                int32_t n_vec, float *out);
int mfc_dequant_matvec_4bit(mfc_ctx *ctx, const uint32_t *w_packed, const uint16_t *scales,
                            const uint16_t *biases, int32_t in_dim, int32_t out_dim, const float *x,
                            int32_t n_vec, float *out);
/* Several matrices applied to the same input in one launch (the reference encodes such a
 * batch of MatvecSpec into one command buffer: gpu_encode_batch_matvec, infer.m:1534-1542,
 * riir/gpu_matvec.rs:84; e.g. q/k/v_proj of a full-attention layer, or in_proj_qkv/z/a/b of
 * a GatedDeltaNet layer).  n_mat in 1..8 matrices of the same in_dim; the four tables are
 * host arrays of n_mat device pointers, out_dims a host array; outs[m] is [n_vec][out_dims[m]].
 * A launch has a fixed cost of several microseconds, more than streaming a 20 MB matrix takes. */
#define MFC_MATVEC_MAX_MATS 8
int mfc_dequant_matvec_4bit_multi_dev(mfc_ctx *ctx, int32_t n_mat, const uint32_t *const *w_packed,
                                      const uint16_t *const *scales, const uint16_t *const *biases,
                                      int32_t in_dim, const int32_t *out_dims, const float *x, int32_t n_vec,
                                      float *const *outs);

/* ---- Folded MLA attention (the third attention flavour: Cogito-V2 / DeepSeek-V3 style latent KV) ----
 * Replaces mla_sdpa_folded and its tiled form mla_sdpa_tile_accumulate / _finalize
 * (crates/moeflux/shaders/shaders.metal:1717-1987) as dispatched by encode_mla_sdpa_folded[_tiled]
 * (crates/moeflux/src/riir/gpu_mla.rs:146-274; CPU statement crates/moeflux/src/riir/mla_attn_cpu.rs:297-340):
 *   s[h][t] = (q_prime[h] . latent[t] + q_pe[h] . rope_k[t]) * softmax_scale;  p = softmax_t(s[h]);
 *   v_combine[h] = sum_t p[t] * latent[t]
 * for num_heads heads over a caller-held compressed cache of cache_len positions:
 *   q_prime [num_heads][512] (the query folded through kv_b_proj), q_pe [num_heads][64] (post-RoPE),
 *   latent_cache [cache_len][512], rope_k_cache [cache_len][64], v_combine [num_heads][512], all fp32.
 * kv_lora_rank 512 and qk_rope_head_dim 64 are the only supported sizes (MFC_MLA_RANK, MFC_MLA_ROPE).  The
 * reference caps its single-dispatch kernel at 4096 positions and tiles beyond that; here every length is one call
 * (split over the positions, merged by log-sum-exp: the algebra of the reference's tile merge).
 * _dev: device pointers, 16-byte aligned, asynchronous on mfc_stream(ctx); the split's partials live in the
 * context's scratch.  The host-pointer form stages its operands in device memory for the call (a test hook, like
 * mfc_sdpa).  0 on success, -1 on error. */
#define MFC_MLA_RANK 512
#define MFC_MLA_ROPE 64
int mfc_mla_sdpa_folded_dev(mfc_ctx *ctx, int32_t num_heads, int32_t cache_len, float softmax_scale,
                            const float *q_prime, const float *q_pe, const float *latent_cache,
                            const float *rope_k_cache, float *v_combine);
int mfc_mla_sdpa_folded(mfc_ctx *ctx, int32_t num_heads, int32_t cache_len, float softmax_scale, const float *q_prime,
                        const float *q_pe, const float *latent_cache, const float *rope_k_cache, float *v_combine);
/* The same for a cache stored as bf16 (latent [cache_len][512], rope_k [cache_len][64] bf16 bit patterns; not a format
 * of the reference, which stores fp32): half the HBM bytes per position and single bf16 products, like the bf16 KV
 * cache of the GQA path; results within 2e-2 of the fp32 statement on the rounded cache.  Device pointers. */
int mfc_mla_sdpa_folded_bf16_dev(mfc_ctx *ctx, int32_t num_heads, int32_t cache_len, float softmax_scale,
                                 const float *q_prime, const float *q_pe, const void *latent_cache_bf16,
                                 const void *rope_k_cache_bf16, float *v_combine);

/* Tuning knobs (tests and sweeps): "gdn_rows" in {0,32,64,128} state rows per
 * CTA (0 = chosen per launch); "gqa_target_ctas" CTAs a decode launch aims for when it cuts the launch's
 * KV tiles into equal runs (0 = one wave: two CTAs per SM); "gqa_chunk" forces the rows per CTA (0 = automatic); "gqa_min_rows" least rows per CTA under the automatic
 * plan (a multiple of 32, default 64); "gqa_unit_aligned" 1 = give every (item, kv head) unit a CTA of its own when
 * equal-length units nearly fill the wave (default 0); "gqa_align_units" 0 = never pad units to whole CTA runs (default 1:
 * a launch of few long units on a full wave, e.g. a ragged batch of 8-32 sequences, gives every unit whole CTAs, so
 * that no CTA works on two units); "gqa_coop_merge" 0 = never launch cooperatively (default 1: a
 * launch in which more than "gqa_coop_min_parts" (default 32, at least 8) CTAs share a unit and that
 * unit has at least a quarter of the launch's CTAs, i.e. a lone long sequence or two, is launched cooperatively when
 * it fits the device, and the CTAs that share a unit merge it together);
 * "exchange_gather_q" (see mfc_eval_token_attn; default 0);
 * "gdn_side_queue" (see mfc_join); "gqa_wait_spins" poll limit of the kernels' bounded waits (0 = default);
 * "gqa_inject_lost_load" 1 = the first CTA of the next decode launches arms the barrier of its first KV tile and
 * issues no load for it, so that its bounded wait runs out with nothing in flight (exercises the failure path
 * without faulting the GPU: the kernel returns, mfc_synchronize reports -1, the context stays usable);
 * "gqa_phase_trace" 1 = decode launches of at most 1024 CTAs, and the projection launches, record per-CTA time
 * stamps (mfc_read_phase_trace); "matvec_overlap" 0 = projection kernels start only when the kernel ahead of them on
 * the stream has finished (default 1, see mfc_dequant_matvec_4bit_dev); "matvec_inject_lost_load" 1 = the same
 * exercise as "gqa_inject_lost_load" for the projection kernel (its first CTA arms its first stage of weights and
 * requests nothing for it). */
int mfc_set_tuning(mfc_ctx *ctx, const char *key, int value);
/* With the tuning "gdn_side_queue" = 1, mfc_linear_attn_step_batched_dev issues
 * its kernel on a second queue of the context: it starts after everything
 * already queued on mfc_stream(ctx) and runs beside whatever is queued there
 * next (a bandwidth-bound attention launch leaves room for it).  mfc_join makes
 * mfc_stream(ctx) wait for that kernel; mfc_synchronize, every host-pointer
 * entry point and every call that reads or writes GatedDeltaNet state outside
 * the step (snapshots, checkpoints, truncation, bulk import, prefill) join
 * implicitly. */
int mfc_join(mfc_ctx *ctx);

/* Number of kernels this library has launched on the context so far. */
long long mfc_launch_count(const mfc_ctx *ctx);

/* Waits for the context's work and verifies the bands of 0xFF bytes that surround every device allocation of the
 * context (KV caches, states, weights, split-K scratch, counters, staging).  0 when all are intact; -1 and the name
 * of the allocation in mfc_last_error when a kernel wrote outside its buffer.  Stands in for a memory checker (the
 * reference relies on Rust ownership, crates/moeflux/src/lib.rs:37); the GPU tests call it after every test. */
int mfc_check_guards(mfc_ctx *ctx);
/* Time stamps (nanoseconds, %globaltimer) of the CTAs of the last decode launch made with the tuning
 * "gqa_phase_trace" on: out[cta][8] = {start, first segment's Q fragments ready, its last KV tile consumed, its
 * epilogue done, CTA done, (bf16 cache only:) query rows staged, query rows rotated, 0}.  After a projection launch
 * (mfc_dequant_matvec_4bit*): {start, barriers set up, x staged by thread 0, x staged by all, first stage of weights
 * arrived, last stage consumed, results stored, cycles warp 0 spent waiting for weights}.  Returns the number of CTAs
 * written (at most max_ctas), or -1. */
int mfc_read_phase_trace(mfc_ctx *ctx, unsigned long long *out, int32_t max_ctas);

/* ---- KV-sequence split: the exchange fused into the decode kernel ----
 * New (the reference is single-device).  With the KV positions of every sequence split over kv_world contexts, one
 * per GPU, each context computes un-normalised partials for all items and every item is finished on one rank (the
 * owner of its sequence).  Instead of writing the partials locally and handing them to a collective, the decode
 * kernel stores each merged partial block [o | m | l] straight into the receive buffer of the owner through a
 * peer-mapped pointer (plain stores over NVLink: nothing else touches peer memory), and its last CTA
 * publishes a step number in every peer's flag array once the stores are visible.  The owner's merge kernel waits
 * (bounded) for the step number of every rank, merges by log-sum-exp and applies the gate.  Receive buffers are
 * double-buffered by step parity, which is enough: a rank cannot start step s+2 before every peer has merged step s.
 *
 * Set-up, once: every rank calls mfc_exchange_create (allocates its receive buffers and flags, returns a CUDA IPC
 * handle of MFC_IPC_HANDLE_BYTES bytes), the ranks exchange the handles by any means (e.g. an all-gather), and each
 * calls mfc_exchange_connect with the kv_world handles in rank order.  Contexts that live in ONE process (tests)
 * call mfc_exchange_connect_local with the kv_world context pointers instead (ipc_handle_out may be NULL).
 * items_per_rank: full-attention items each rank finishes per step; a step carries items_per_rank * kv_world items
 * sorted by finishing rank (item i is finished by rank i / items_per_rank).
 *
 * Per step: mfc_full_attn_partial_exchange_dev (arguments as mfc_full_attn_partial_packed_dev, no output pointer),
 * then mfc_lse_merge_gate_exchange_dev: gate [items_per_rank][heads*256] (may be NULL) and out of the same shape
 * for the items this rank finishes, in item order.  Every rank must issue the same steps.  mfc_eval_token_attn on
 * such a context does both, with gate and full_out covering this rank's items only. */
#define MFC_IPC_HANDLE_BYTES 64
int mfc_exchange_create(mfc_ctx *ctx, int32_t items_per_rank, void *ipc_handle_out);
int mfc_exchange_connect(mfc_ctx *ctx, const void *ipc_handles);
int mfc_exchange_connect_local(mfc_ctx *ctx, mfc_ctx *const *peers);
int mfc_full_attn_partial_exchange_dev(mfc_ctx *ctx, int32_t n, const int32_t *layers, const int32_t *seq_ids,
                                       const int32_t *pos, const float *q, const float *k, const float *v);
int mfc_lse_merge_gate_exchange_dev(mfc_ctx *ctx, const float *gate, float *out);

#ifdef __cplusplus
}
#endif
#endif /* MOEFLUX_CUDA_H */
