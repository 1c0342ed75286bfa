/*
 * CPU oracle for the moeflux attention hot path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file restates, in plain C, the arithmetic of
 * the reference's attention sub-block (full-attention GQA SDPA with sigmoid
 * output gate; GatedDeltaNet conv1d + delta-rule step) in the reference's own
 * operation order.  It is the checker that the CUDA path is compared with and
 * the timed CPU baseline.  Nothing the library ships may call into it.
 *
 * PARITY PINNED against the reference's own C code: oracle/ref.py compiles the
 * plain-C CPU twins of this path out of the reference's
 * crates/moeflux-sys/metal_infer/infer.m (cpu_sdpa, apply_rotary_emb,
 * cpu_conv1d_step, cpu_rms_norm_bare/_gated/_per_head,
 * cpu_gated_delta_recurrence, cpu_dequant_matvec) into oracle/_ref/, and
 * tests/test_oracle_ref.py holds every function below to them on the inputs and
 * at the bounds of the reference's differential tests (128 ULP; cosine 0.9999
 * and 1e-3 for SDPA).  The reference stores no golden vectors for this path;
 * closed-form known answers derived from its formulas (tests/test_oracle_kat.py)
 * and the known answers of its unit tests of the 4-bit matvec
 * (crates/moeflux/src/riir/cpu_matvec.rs:370-451) are checked as well.
 *
 * Every function cites the reference source it follows, by path inside the
 * reference project.  Rust `mul_add` call sites are kept as fmaf(); all other
 * products and sums are left un-contracted (build with -ffp-contract=off).
 * Threads (OpenMP) split independent heads only; the order of operations inside
 * one head is the reference's sequential order.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define MFO_API __attribute__((visibility("default")))

/* bf16 -> f32: bits << 16.  crates/moeflux/src/riir/embedding.rs:153-155,
 * crates/moeflux/shaders/shaders.metal:35-37. */
static inline float bf16_to_f32(uint16_t b) {
    uint32_t u = ((uint32_t)b) << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* f32 -> bf16, round to nearest even (the storage rounding of the new bf16 KV
 * cache; no reference counterpart, the reference stores fp32 only). */
MFO_API uint16_t mfo_f32_to_bf16(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40); /* NaN */
    uint32_t lsb = (u >> 16) & 1u;
    u += 0x7fffu + lsb;
    return (uint16_t)(u >> 16);
}

MFO_API void mfo_round_bf16(const float *x, float *out, size_t n) {
    for (size_t i = 0; i < n; i++) out[i] = bf16_to_f32(mfo_f32_to_bf16(x[i]));
}

/* Launchers such as torchrun export OMP_NUM_THREADS=1; the timed CPU baseline asks
 * for all the host's cores explicitly. */
MFO_API void mfo_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

MFO_API int mfo_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* ------------------------------------------------------------------------
 * RoPE, MLX half-split pairing over the first rotary_dim channels of each
 * head.  crates/moeflux/src/riir/rope.rs:65-131 (C twin:
 * crates/moeflux-sys/metal_infer/infer.m:2138-2172).
 * freq_i = 1/powf(theta, 2i/rotary_dim); angle = float(pos)*freq_i;
 * (x[i], x[i+half]) <- (x0 cos - x1 sin, x0 sin + x1 cos).
 * Returns -1 on NULL args or pos < 0 (moeflux.h:151).
 * ---------------------------------------------------------------------- */
MFO_API void mfo_rope_inv_freq(float theta, int rotary_dim, float *inv_freq) {
    int half = rotary_dim / 2;
    float rdim_f = (float)rotary_dim;
    for (int i = 0; i < half; i++)
        inv_freq[i] = 1.0f / powf(theta, (float)(2 * i) / rdim_f);
}

MFO_API int mfo_apply_rotary_emb(int32_t pos, float *q, float *k, int num_heads,
                                 int num_kv_heads, int head_dim, int rotary_dim,
                                 float theta) {
    if (!q || !k || pos < 0) return -1;
    int half = rotary_dim / 2;
    float pos_f = (float)pos;
    float rdim_f = (float)rotary_dim;
    for (int pass = 0; pass < 2; pass++) {
        float *x = pass == 0 ? q : k;
        int nh = pass == 0 ? num_heads : num_kv_heads;
        for (int h = 0; h < nh; h++) {
            float *xh = x + (size_t)h * head_dim;
            for (int i = 0; i < half; i++) {
                float freq = 1.0f / powf(theta, (float)(2 * i) / rdim_f);
                float angle = pos_f * freq;
                float c = cosf(angle), s = sinf(angle);
                float x0 = xh[i], x1 = xh[i + half];
                xh[i] = x0 * c - x1 * s;
                xh[i + half] = x0 * s + x1 * c;
            }
        }
    }
    return 0;
}

/* ------------------------------------------------------------------------
 * Per-head weighted RMSNorm, in place.
 * crates/moeflux/src/riir/rms_norm.rs:104-153 (called for q and k at
 * crates/moeflux/src/riir/full_attn_forward.rs:256-276).
 * ---------------------------------------------------------------------- */
MFO_API int mfo_rms_norm_per_head(const uint16_t *w_bf16, int num_heads, int head_dim,
                                  float eps, float *x) {
    if (!w_bf16 || !x || num_heads <= 0 || head_dim <= 0) return -1;
    for (int h = 0; h < num_heads; h++) {
        float *xh = x + (size_t)h * head_dim;
        float sum_sq = 0.0f;
        for (int i = 0; i < head_dim; i++) sum_sq += xh[i] * xh[i];
        float inv_rms = 1.0f / sqrtf(sum_sq / (float)head_dim + eps);
        for (int i = 0; i < head_dim; i++) xh[i] = xh[i] * inv_rms * bf16_to_f32(w_bf16[i]);
    }
    return 0;
}

/* ------------------------------------------------------------------------
 * 4-bit group-64 affine dequant matvec.  crates/moeflux/src/riir/cpu_matvec.rs:83-171
 * (GPU twin: crates/moeflux/shaders/shaders.metal:48-91): per row, groups in order,
 * words in order, nibbles least significant first; w = nibble.mul_add(scale, bias),
 * acc = w.mul_add(x, acc).  Rows are independent (rayon there, OpenMP here).
 * Returns -1 for the reference's InDimNotMultiple / bad-argument errors.
 * ---------------------------------------------------------------------- */
#define MFO_GROUP_SIZE 64
MFO_API int mfo_dequant_matvec_4bit(const uint32_t *packed, const uint16_t *scales, const uint16_t *biases,
                                    int in_dim, int out_dim, const float *x, float *out) {
    if (!packed || !scales || !biases || !x || !out || in_dim <= 0 || out_dim <= 0) return -1;
    if (in_dim % MFO_GROUP_SIZE != 0) return -1;
    const int in_packed = in_dim / 8, in_groups = in_dim / MFO_GROUP_SIZE, packed_per_group = MFO_GROUP_SIZE / 8;
#pragma omp parallel for schedule(static)
    for (int r = 0; r < out_dim; r++) {
        const uint32_t *packed_row = packed + (size_t)r * in_packed;
        const uint16_t *scale_row = scales + (size_t)r * in_groups;
        const uint16_t *bias_row = biases + (size_t)r * in_groups;
        float acc = 0.0f;
        for (int g = 0; g < in_groups; g++) {
            const float scale = bf16_to_f32(scale_row[g]);
            const float bias = bf16_to_f32(bias_row[g]);
            for (int p = 0; p < packed_per_group; p++) {
                const uint32_t word = packed_row[g * packed_per_group + p];
                const float *x_chunk = x + (size_t)g * MFO_GROUP_SIZE + p * 8;
                for (int n = 0; n < 8; n++) {
                    const float nibble = (float)((word >> (n * 4)) & 0xFu);
                    const float w = fmaf(nibble, scale, bias);
                    acc = fmaf(w, x_chunk[n], acc);
                }
            }
        }
        out[r] = acc;
    }
    return 0;
}

/* ------------------------------------------------------------------------
 * q|gate de-interleave.  crates/moeflux/src/riir/full_attn_forward.rs:238-254:
 * q_proj_out is [head][q(head_dim) | gate(head_dim)].
 * ---------------------------------------------------------------------- */
MFO_API void mfo_split_q_gate(const float *q_proj, int num_heads, int head_dim, float *q,
                              float *gate) {
    for (int h = 0; h < num_heads; h++) {
        memcpy(q + (size_t)h * head_dim, q_proj + (size_t)h * 2 * head_dim,
               sizeof(float) * head_dim);
        memcpy(gate + (size_t)h * head_dim, q_proj + (size_t)h * 2 * head_dim + head_dim,
               sizeof(float) * head_dim);
    }
}

/* ------------------------------------------------------------------------
 * SDPA with sigmoid output gate over a [kv_len][num_kv_heads][head_dim] cache.
 * crates/moeflux/src/riir/sdpa.rs:63-172 (C twin infer.m:762-804):
 * sequential dot * scale -> max -> expf/sum -> normalise -> sum_p w*V -> gate.
 * Returns -1 on NULL args or kv_len <= 0 (moeflux.h:179-182).
 * ---------------------------------------------------------------------- */
MFO_API int mfo_sdpa(int32_t kv_len, const float *q, const float *q_gate, const float *k_cache,
                     const float *v_cache, float *out, int num_heads, int num_kv_heads,
                     int head_dim) {
    if (!q || !q_gate || !k_cache || !v_cache || !out || kv_len <= 0) return -1;
    size_t kv_dim = (size_t)num_kv_heads * head_dim;
    int heads_per_kv = num_heads / num_kv_heads;
    float scale = 1.0f / sqrtf((float)head_dim);
    int failed = 0;
#pragma omp parallel for schedule(dynamic, 1)
    for (int h = 0; h < num_heads; h++) {
        float *scores = (float *)malloc(sizeof(float) * (size_t)kv_len);
        if (!scores) {
            failed = 1;
            continue;
        }
        int kv_h = h / heads_per_kv;
        const float *qh = q + (size_t)h * head_dim;
        for (int p = 0; p < kv_len; p++) {
            const float *kp = k_cache + (size_t)p * kv_dim + (size_t)kv_h * head_dim;
            float dot = 0.0f;
            for (int d = 0; d < head_dim; d++) dot += qh[d] * kp[d];
            scores[p] = dot * scale;
        }
        float max_val = scores[0];
        for (int p = 1; p < kv_len; p++)
            if (scores[p] > max_val) max_val = scores[p];
        float sum = 0.0f;
        for (int p = 0; p < kv_len; p++) {
            scores[p] = expf(scores[p] - max_val);
            sum += scores[p];
        }
        float inv_sum = 1.0f / sum;
        for (int p = 0; p < kv_len; p++) scores[p] *= inv_sum;
        float *oh = out + (size_t)h * head_dim;
        for (int d = 0; d < head_dim; d++) oh[d] = 0.0f;
        for (int p = 0; p < kv_len; p++) {
            const float *vp = v_cache + (size_t)p * kv_dim + (size_t)kv_h * head_dim;
            float w = scores[p];
            for (int d = 0; d < head_dim; d++) oh[d] += w * vp[d];
        }
        for (int d = 0; d < head_dim; d++) {
            float g = 1.0f / (1.0f + expf(-q_gate[(size_t)h * head_dim + d]));
            oh[d] *= g;
        }
        free(scores);
    }
    return failed ? -1 : 0;
}

/* ------------------------------------------------------------------------
 * The four GPU attention kernels, one function each, tight stride
 * (seq_stride = seq_len as in the reference's test hooks, moeflux.h:475-527).
 * crates/moeflux/shaders/shaders.metal:976-1019 (scores), :1026-1084 (softmax),
 * :1095-1117 (values), :1125-1134 (sigmoid gate).  The in-threadgroup tree
 * reductions of the shader are replaced with sequential sums.
 * ---------------------------------------------------------------------- */
MFO_API int mfo_attn_scores_batched(int num_heads, int num_kv_heads, int head_dim, int seq_len,
                                    const float *q, const float *k_cache, float scale,
                                    float *scores_out) {
    if (!q || !k_cache || !scores_out || num_heads <= 0 || num_kv_heads <= 0 || head_dim <= 0 ||
        seq_len <= 0 || num_heads % num_kv_heads)
        return -1;
    int heads_per_kv = num_heads / num_kv_heads;
    size_t kv_dim = (size_t)num_kv_heads * head_dim;
#pragma omp parallel for
    for (int h = 0; h < num_heads; h++) {
        int kv_h = h / heads_per_kv;
        for (int p = 0; p < seq_len; p++) {
            const float *qh = q + (size_t)h * head_dim;
            const float *kp = k_cache + (size_t)p * kv_dim + (size_t)kv_h * head_dim;
            float acc = 0.0f;
            for (int d = 0; d < head_dim; d++) acc += qh[d] * kp[d];
            scores_out[(size_t)h * seq_len + p] = acc * scale;
        }
    }
    return 0;
}

MFO_API int mfo_attn_softmax_batched(int num_heads, int seq_len, float *scores) {
    if (!scores || num_heads <= 0 || seq_len <= 0) return -1;
    for (int h = 0; h < num_heads; h++) {
        float *s = scores + (size_t)h * seq_len;
        float m = -1e30f;
        for (int i = 0; i < seq_len; i++) m = fmaxf(m, s[i]);
        float sum = 0.0f;
        for (int i = 0; i < seq_len; i++) {
            s[i] = expf(s[i] - m);
            sum += s[i];
        }
        float inv = 1.0f / sum;
        for (int i = 0; i < seq_len; i++) s[i] *= inv;
    }
    return 0;
}

MFO_API int mfo_attn_values_batched(int num_heads, int num_kv_heads, int head_dim, int seq_len,
                                    const float *scores, const float *v_cache, float *out) {
    if (!scores || !v_cache || !out || num_heads <= 0 || num_kv_heads <= 0 || head_dim <= 0 ||
        seq_len <= 0 || num_heads % num_kv_heads)
        return -1;
    int heads_per_kv = num_heads / num_kv_heads;
    size_t kv_dim = (size_t)num_kv_heads * head_dim;
#pragma omp parallel for
    for (int h = 0; h < num_heads; h++) {
        int kv_h = h / heads_per_kv;
        const float *s = scores + (size_t)h * seq_len;
        for (int d = 0; d < head_dim; d++) {
            float acc = 0.0f;
            for (int p = 0; p < seq_len; p++)
                acc += s[p] * v_cache[(size_t)p * kv_dim + (size_t)kv_h * head_dim + d];
            out[(size_t)h * head_dim + d] = acc;
        }
    }
    return 0;
}

MFO_API int mfo_sigmoid_gate(int dim, const float *gate, float *x) {
    if (!gate || !x || dim <= 0) return -1;
    for (int i = 0; i < dim; i++) {
        float g = 1.0f / (1.0f + expf(-gate[i]));
        x[i] = x[i] * g;
    }
    return 0;
}

/* ------------------------------------------------------------------------
 * Depthwise conv1d step + SiLU; the state is read, not advanced.
 * crates/moeflux/src/riir/linear_attn.rs:89-156: acc = fma(state[k][c], w[c][k],
 * acc) for the history taps in order, then fma(x[c], w[c][K-1], acc), then
 * silu(acc) = acc / (1 + exp(-acc)).
 * ---------------------------------------------------------------------- */
MFO_API int mfo_conv1d_step(const float *conv_state, const float *new_input,
                            const uint16_t *w_bf16, int channels, int kernel_size, float *out) {
    if (!conv_state || !new_input || !w_bf16 || !out || channels <= 0 || kernel_size <= 0)
        return -1;
    for (int c = 0; c < channels; c++) {
        float acc = 0.0f;
        for (int k = 0; k < kernel_size - 1; k++) {
            float w = bf16_to_f32(w_bf16[(size_t)c * kernel_size + k]);
            float s = conv_state[(size_t)k * channels + c];
            acc = fmaf(s, w, acc);
        }
        float w = bf16_to_f32(w_bf16[(size_t)c * kernel_size + kernel_size - 1]);
        acc = fmaf(new_input[c], w, acc);
        out[c] = acc;
    }
    for (int c = 0; c < channels; c++) out[c] = out[c] / (1.0f + expf(-out[c]));
    return 0;
}

/* State advance that follows every conv step: drop the oldest row, append the
 * pre-activation input.  crates/moeflux-sys/metal_infer/infer.m:4874-4877,
 * crates/moeflux/shaders/shaders.metal:1240-1243. */
MFO_API void mfo_conv_state_shift(float *conv_state, const float *new_input, int channels,
                                  int kernel_size) {
    if (kernel_size > 2)
        memmove(conv_state, conv_state + channels,
                sizeof(float) * (size_t)(kernel_size - 2) * channels);
    if (kernel_size > 1)
        memcpy(conv_state + (size_t)(kernel_size - 2) * channels, new_input,
               sizeof(float) * channels);
}

/* Bare RMSNorm.  crates/moeflux/src/riir/linear_attn.rs:160-185. */
MFO_API int mfo_rms_norm_bare(int dim, float eps, const float *x, float *out) {
    if (!x || !out || dim <= 0) return -1;
    float sum_sq = 0.0f;
    for (int i = 0; i < dim; i++) sum_sq += x[i] * x[i];
    float inv_rms = 1.0f / sqrtf(sum_sq / (float)dim + eps);
    for (int i = 0; i < dim; i++) out[i] = x[i] * inv_rms;
    return 0;
}

/* Gated RMSNorm: out = x * inv_rms * w * silu(z).
 * crates/moeflux/src/riir/linear_attn.rs:190-242 (GPU twin shaders.metal:1337-1370). */
MFO_API int mfo_rms_norm_gated(const uint16_t *w_bf16, int dim, float eps, const float *x,
                               const float *z, float *out) {
    if (!w_bf16 || !x || !z || !out || dim <= 0) return -1;
    float sum_sq = 0.0f;
    for (int i = 0; i < dim; i++) sum_sq += x[i] * x[i];
    float inv_rms = 1.0f / sqrtf(sum_sq / (float)dim + eps);
    for (int i = 0; i < dim; i++) {
        float w = bf16_to_f32(w_bf16[i]);
        float silu_z = z[i] / (1.0f + expf(-z[i]));
        out[i] = x[i] * inv_rms * w * silu_z;
    }
    return 0;
}

/* q/k normalisation of the GatedDeltaNet layer, in place, per k-head:
 * q <- q * rsqrt(mean q^2 + 1e-6) * inv_scale^2, k <- k * rsqrt(mean k^2 + 1e-6) * inv_scale,
 * inv_scale = 1/sqrt(key_dim).  crates/moeflux/shaders/shaders.metal:1254-1303
 * (C twin infer.m:4885-4896).  rsqrt is evaluated as 1/sqrtf. */
MFO_API int mfo_rms_norm_qk(float *q, float *k, int num_k_heads, int key_dim) {
    if (!q || !k || num_k_heads <= 0 || key_dim <= 0) return -1;
    float inv_scale = 1.0f / sqrtf((float)key_dim);
    for (int h = 0; h < num_k_heads; h++) {
        float *qh = q + (size_t)h * key_dim, *kh = k + (size_t)h * key_dim;
        float qs = 0.0f, ks = 0.0f;
        for (int i = 0; i < key_dim; i++) qs += qh[i] * qh[i];
        float q_inv = 1.0f / sqrtf(qs / (float)key_dim + 1e-6f);
        for (int i = 0; i < key_dim; i++) qh[i] = qh[i] * q_inv * inv_scale * inv_scale;
        for (int i = 0; i < key_dim; i++) ks += kh[i] * kh[i];
        float k_inv = 1.0f / sqrtf(ks / (float)key_dim + 1e-6f);
        for (int i = 0; i < key_dim; i++) kh[i] = kh[i] * k_inv * inv_scale;
    }
    return 0;
}

/* Per v-head decay and beta gate.  crates/moeflux/src/riir/linear_attn.rs:357-370
 * (GPU twin shaders.metal:1312-1327). */
MFO_API int mfo_decay_beta(const float *alpha, const float *beta, const float *a_log,
                           const uint16_t *dt_bias_bf16, int v_heads, float *g_decay,
                           float *beta_gate) {
    if (!alpha || !beta || !a_log || !dt_bias_bf16 || !g_decay || !beta_gate || v_heads <= 0)
        return -1;
    for (int vh = 0; vh < v_heads; vh++) {
        float a_val = alpha[vh];
        float dt_b = bf16_to_f32(dt_bias_bf16[vh]);
        float a_capital = expf(a_log[vh]);
        float softplus_val = logf(1.0f + expf(a_val + dt_b));
        g_decay[vh] = expf(-a_capital * softplus_val);
        beta_gate[vh] = 1.0f / (1.0f + expf(-beta[vh]));
    }
    return 0;
}

/* Gated delta-rule recurrence, one token.  crates/moeflux/src/riir/linear_attn.rs:288-414
 * (C twin infer.m:7931-7988, GPU twin shaders.metal:1154-1194): decay the whole
 * head state, then per row kv_mem / delta / update, then read-out. */
MFO_API int mfo_gated_delta_recurrence(const float *a_log, const uint16_t *dt_bias_bf16,
                                       const float *alpha, const float *beta, const float *q,
                                       const float *k, const float *v, int v_heads, int k_heads,
                                       int key_dim, int value_dim, float *ssm_state,
                                       float *out_values) {
    if (!a_log || !dt_bias_bf16 || !alpha || !beta || !q || !k || !v || !ssm_state ||
        !out_values || v_heads <= 0 || k_heads <= 0 || key_dim <= 0 || value_dim <= 0 ||
        v_heads % k_heads)
        return -1;
    int k_heads_per_v = v_heads / k_heads;
    float *g_decay = (float *)malloc(sizeof(float) * 2 * (size_t)v_heads);
    if (!g_decay) return -1;
    float *beta_gate = g_decay + v_heads;
    mfo_decay_beta(alpha, beta, a_log, dt_bias_bf16, v_heads, g_decay, beta_gate);
    size_t head_state_stride = (size_t)value_dim * key_dim;
#pragma omp parallel for schedule(static)
    for (int vh = 0; vh < v_heads; vh++) {
        int kh = vh / k_heads_per_v;
        float g = g_decay[vh], b_gate = beta_gate[vh];
        float *S = ssm_state + (size_t)vh * head_state_stride;
        const float *vv = v + (size_t)vh * value_dim;
        const float *kk = k + (size_t)kh * key_dim;
        const float *qq = q + (size_t)kh * key_dim;
        float *oo = out_values + (size_t)vh * value_dim;
        for (size_t i = 0; i < head_state_stride; i++) S[i] *= g;
        for (int vi = 0; vi < value_dim; vi++) {
            float *row = S + (size_t)vi * key_dim;
            float kv_mem = 0.0f;
            for (int ki = 0; ki < key_dim; ki++) kv_mem = fmaf(row[ki], kk[ki], kv_mem);
            float delta = (vv[vi] - kv_mem) * b_gate;
            for (int ki = 0; ki < key_dim; ki++) row[ki] = fmaf(kk[ki], delta, row[ki]);
        }
        for (int vi = 0; vi < value_dim; vi++) {
            const float *row = S + (size_t)vi * key_dim;
            float sum = 0.0f;
            for (int ki = 0; ki < key_dim; ki++) sum = fmaf(row[ki], qq[ki], sum);
            oo[vi] = sum;
        }
    }
    free(g_decay);
    return 0;
}

/* ------------------------------------------------------------------------
 * Composite: one full-attention decode step on a host cache, in the order of
 * crates/moeflux/src/riir/full_attn_forward.rs:278-389: RoPE(q,k) at pos ->
 * append k,v at row kv_len -> SDPA over kv_len+1 rows -> sigmoid gate.
 * kv_bf16 != 0 rounds the appended K/V rows to bf16 (new storage mode; the
 * reference stores fp32).  q and k are rotated in place.  k_cache/v_cache must
 * hold at least kv_len+1 rows.  Returns -1 if pos != kv_len (the caller
 * contract stated at full_attn_forward.rs:73-78).
 * ---------------------------------------------------------------------- */
MFO_API int mfo_full_attn_step(int32_t pos, int32_t kv_len, float *q, const float *gate, float *k,
                               const float *v, float *k_cache, float *v_cache, float *out,
                               int num_heads, int num_kv_heads, int head_dim, int rotary_dim,
                               float theta, int kv_bf16) {
    if (pos < 0 || pos != kv_len) return -1;
    if (mfo_apply_rotary_emb(pos, q, k, num_heads, num_kv_heads, head_dim, rotary_dim, theta))
        return -1;
    size_t kv_dim = (size_t)num_kv_heads * head_dim;
    float *krow = k_cache + (size_t)kv_len * kv_dim, *vrow = v_cache + (size_t)kv_len * kv_dim;
    if (kv_bf16) {
        mfo_round_bf16(k, krow, kv_dim);
        mfo_round_bf16(v, vrow, kv_dim);
    } else {
        memcpy(krow, k, sizeof(float) * kv_dim);
        memcpy(vrow, v, sizeof(float) * kv_dim);
    }
    return mfo_sdpa(kv_len + 1, q, gate, k_cache, v_cache, out, num_heads, num_kv_heads, head_dim);
}

/* ------------------------------------------------------------------------
 * Composite: one GatedDeltaNet decode step, the five kernels in the order of
 * crates/moeflux/src/riir/linear_attn_forward.rs:607-664: conv1d+SiLU (then the
 * state shift) -> q/k norm -> decay/beta -> delta recurrence -> gated RMSNorm
 * (skipped when z or norm_w is NULL).  qkv is [q(k_heads*key_dim) |
 * k(k_heads*key_dim) | v(v_heads*value_dim)].
 * ---------------------------------------------------------------------- */
MFO_API int mfo_linear_attn_step(const float *qkv, const float *z, const float *alpha,
                                 const float *beta, const uint16_t *conv_w_bf16,
                                 const float *a_log, const uint16_t *dt_bias_bf16,
                                 const uint16_t *norm_w_bf16, float *conv_state, float *ssm_state,
                                 float *out, int v_heads, int k_heads, int key_dim, int value_dim,
                                 int kernel_size, float eps) {
    int total_key = k_heads * key_dim;
    int conv_dim = 2 * total_key + v_heads * value_dim;
    float *y = (float *)malloc(sizeof(float) * (size_t)(conv_dim + v_heads * value_dim));
    if (!y) return -1;
    float *rec = y + conv_dim;
    int rc = mfo_conv1d_step(conv_state, qkv, conv_w_bf16, conv_dim, kernel_size, y);
    if (!rc) {
        mfo_conv_state_shift(conv_state, qkv, conv_dim, kernel_size);
        rc = mfo_rms_norm_qk(y, y + total_key, k_heads, key_dim);
    }
    if (!rc)
        rc = mfo_gated_delta_recurrence(a_log, dt_bias_bf16, alpha, beta, y, y + total_key,
                                        y + 2 * total_key, v_heads, k_heads, key_dim, value_dim,
                                        ssm_state, rec);
    if (!rc) {
        if (z && norm_w_bf16) {
            for (int h = 0; h < v_heads && !rc; h++)
                rc = mfo_rms_norm_gated(norm_w_bf16, value_dim, eps, rec + (size_t)h * value_dim,
                                        z + (size_t)h * value_dim, out + (size_t)h * value_dim);
        } else {
            memcpy(out, rec, sizeof(float) * (size_t)v_heads * value_dim);
        }
    }
    free(y);
    return rc;
}

/* ------------------------------------------------------------------------
 * Split-softmax algebra used to check the split-K and cross-GPU KV-split
 * merges.  No reference counterpart for GQA; the algebra is that of the
 * reference's MLA tile merge, crates/moeflux/shaders/shaders.metal:1933-1968.
 * Partial over cache rows [p0, p1): m = max s, l = sum exp(s-m),
 * o = sum exp(s-m) V (un-normalised).  An empty range gives m=-inf, l=0, o=0.
 * ---------------------------------------------------------------------- */
MFO_API int mfo_sdpa_partial(int32_t p0, int32_t p1, const float *q, const float *k_cache,
                             const float *v_cache, float *o_part, float *m_part, float *l_part,
                             int num_heads, int num_kv_heads, int head_dim) {
    if (!q || !k_cache || !v_cache || !o_part || !m_part || !l_part || p0 < 0 || p1 < p0)
        return -1;
    size_t kv_dim = (size_t)num_kv_heads * head_dim;
    int heads_per_kv = num_heads / num_kv_heads;
    float scale = 1.0f / sqrtf((float)head_dim);
#pragma omp parallel for schedule(dynamic, 1)
    for (int h = 0; h < num_heads; h++) {
        int kv_h = h / heads_per_kv;
        const float *qh = q + (size_t)h * head_dim;
        float *oh = o_part + (size_t)h * head_dim;
        for (int d = 0; d < head_dim; d++) oh[d] = 0.0f;
        float m = -INFINITY, l = 0.0f;
        for (int p = p0; p < p1; p++) {
            const float *kp = k_cache + (size_t)p * kv_dim + (size_t)kv_h * head_dim;
            float dot = 0.0f;
            for (int d = 0; d < head_dim; d++) dot += qh[d] * kp[d];
            float s = dot * scale;
            if (s > m) m = s;
        }
        for (int p = p0; p < p1; p++) {
            const float *kp = k_cache + (size_t)p * kv_dim + (size_t)kv_h * head_dim;
            const float *vp = v_cache + (size_t)p * kv_dim + (size_t)kv_h * head_dim;
            float dot = 0.0f;
            for (int d = 0; d < head_dim; d++) dot += qh[d] * kp[d];
            float e = expf(dot * scale - m);
            l += e;
            for (int d = 0; d < head_dim; d++) oh[d] += e * vp[d];
        }
        m_part[h] = m;
        l_part[h] = l;
    }
    return 0;
}

/* Merge R partials [r][head][...] and apply the sigmoid gate:
 * M = max_r m_r; out = (sum_r e^{m_r-M} o_r / sum_r e^{m_r-M} l_r) * sigmoid(gate). */
MFO_API int mfo_lse_merge_gate(int n_parts, const float *o_parts, const float *m_parts,
                               const float *l_parts, const float *gate, float *out,
                               int num_heads, int head_dim) {
    if (!o_parts || !m_parts || !l_parts || !out || n_parts <= 0) return -1;
    for (int h = 0; h < num_heads; h++) {
        float M = -INFINITY;
        for (int r = 0; r < n_parts; r++) M = fmaxf(M, m_parts[(size_t)r * num_heads + h]);
        float L = 0.0f;
        for (int d = 0; d < head_dim; d++) out[(size_t)h * head_dim + d] = 0.0f;
        for (int r = 0; r < n_parts; r++) {
            float mr = m_parts[(size_t)r * num_heads + h];
            float w = (mr == -INFINITY) ? 0.0f : expf(mr - M);
            L += w * l_parts[(size_t)r * num_heads + h];
            const float *o = o_parts + ((size_t)r * num_heads + h) * head_dim;
            for (int d = 0; d < head_dim; d++) out[(size_t)h * head_dim + d] += w * o[d];
        }
        for (int d = 0; d < head_dim; d++) {
            float val = out[(size_t)h * head_dim + d] / L;
            if (gate) val *= 1.0f / (1.0f + expf(-gate[(size_t)h * head_dim + d]));
            out[(size_t)h * head_dim + d] = val;
        }
    }
    return 0;
}

/* ------------------------------------------------------------------------
 * Folded MLA attention.  crates/moeflux/shaders/shaders.metal:1717-1822
 * (mla_sdpa_folded; the same sums per head as the CPU layer's SDPA loop,
 * crates/moeflux/src/riir/mla_attn_cpu.rs:297-340, with K and V folded into the
 * latent): scores by an fma chain over the latent then the rope dims, scaled;
 * softmax as max / exp / sum / normalise; v_combine by an fma chain over the
 * positions.  Threads split heads only.
 * ---------------------------------------------------------------------- */
MFO_API int mfo_mla_sdpa_folded(int num_heads, int kv_lora_rank, int rope_dim, int cache_len, float softmax_scale,
                                const float *q_prime, const float *q_pe, const float *latent,
                                const float *rope_k, float *v_combine) {
    if (num_heads <= 0 || kv_lora_rank <= 0 || rope_dim < 0 || cache_len <= 0) return -1;
    int err = 0;
#pragma omp parallel for schedule(static)
    for (int h = 0; h < num_heads; h++) {
        float *scores = (float *)malloc(sizeof(float) * (size_t)cache_len);
        if (!scores) {
            err = 1;
            continue;
        }
        const float *qh = q_prime + (size_t)h * kv_lora_rank, *ph = q_pe + (size_t)h * rope_dim;
        for (int t = 0; t < cache_len; t++) {
            const float *lt = latent + (size_t)t * kv_lora_rank, *rt = rope_k + (size_t)t * rope_dim;
            float s = 0.0f;
            for (int c = 0; c < kv_lora_rank; c++) s = fmaf(qh[c], lt[c], s);
            for (int r = 0; r < rope_dim; r++) s = fmaf(ph[r], rt[r], s);
            scores[t] = s * softmax_scale;
        }
        float mx = -INFINITY;
        for (int t = 0; t < cache_len; t++) mx = scores[t] > mx ? scores[t] : mx;
        float sum = 0.0f;
        for (int t = 0; t < cache_len; t++) {
            scores[t] = expf(scores[t] - mx);
            sum += scores[t];
        }
        const float inv = 1.0f / sum;
        for (int t = 0; t < cache_len; t++) scores[t] *= inv;
        float *out = v_combine + (size_t)h * kv_lora_rank;
        for (int c = 0; c < kv_lora_rank; c++) {
            float acc = 0.0f;
            for (int t = 0; t < cache_len; t++) acc = fmaf(scores[t], latent[(size_t)t * kv_lora_rank + c], acc);
            out[c] = acc;
        }
        free(scores);
    }
    return err ? -1 : 0;
}

/* The tiled form: tiles of `tile` positions merged by the online softmax of
 * mla_sdpa_tile_accumulate (shaders.metal:1845-1966), finished by
 * mla_sdpa_tile_finalize (:1971-1987); the tile loop of
 * encode_mla_sdpa_folded_tiled (crates/moeflux/src/riir/gpu_mla.rs:226-274). */
MFO_API int mfo_mla_sdpa_folded_tiled(int num_heads, int kv_lora_rank, int rope_dim, int cache_len, int tile,
                                      float softmax_scale, const float *q_prime, const float *q_pe,
                                      const float *latent, const float *rope_k, float *v_combine) {
    if (num_heads <= 0 || kv_lora_rank <= 0 || rope_dim < 0 || cache_len <= 0 || tile <= 0) return -1;
    int err = 0;
#pragma omp parallel for schedule(static)
    for (int h = 0; h < num_heads; h++) {
        float *scores = (float *)malloc(sizeof(float) * (size_t)tile);
        float *vp = (float *)calloc((size_t)kv_lora_rank, sizeof(float));
        if (!scores || !vp) {
            err = 1;
            free(scores);
            free(vp);
            continue;
        }
        const float *qh = q_prime + (size_t)h * kv_lora_rank, *ph = q_pe + (size_t)h * rope_dim;
        float run_max = -INFINITY, run_den = 0.0f;
        for (int t0 = 0; t0 < cache_len; t0 += tile) {
            const int n = cache_len - t0 < tile ? cache_len - t0 : tile;
            float tmax = -INFINITY;
            for (int i = 0; i < n; i++) {
                const float *lt = latent + (size_t)(t0 + i) * kv_lora_rank, *rt = rope_k + (size_t)(t0 + i) * rope_dim;
                float s = 0.0f;
                for (int c = 0; c < kv_lora_rank; c++) s = fmaf(qh[c], lt[c], s);
                for (int r = 0; r < rope_dim; r++) s = fmaf(ph[r], rt[r], s);
                scores[i] = s * softmax_scale;
                tmax = scores[i] > tmax ? scores[i] : tmax;
            }
            float tsum = 0.0f;
            for (int i = 0; i < n; i++) {
                scores[i] = expf(scores[i] - tmax);
                tsum += scores[i];
            }
            const float new_max = run_max > tmax ? run_max : tmax;
            const float scale_old = expf(run_max - new_max), scale_new = expf(tmax - new_max);
            run_den = run_den * scale_old + tsum * scale_new;
            for (int c = 0; c < kv_lora_rank; c++) {
                float part = 0.0f;
                for (int i = 0; i < n; i++) part = fmaf(scores[i], latent[(size_t)(t0 + i) * kv_lora_rank + c], part);
                vp[c] = vp[c] * scale_old + part * scale_new;
            }
            run_max = new_max;
        }
        const float inv = run_den > 0.0f ? 1.0f / run_den : 0.0f;
        for (int c = 0; c < kv_lora_rank; c++) v_combine[(size_t)h * kv_lora_rank + c] = vp[c] * inv;
        free(scores);
        free(vp);
    }
    return err ? -1 : 0;
}
