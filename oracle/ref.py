"""Builds and binds ``oracle/_ref/libmf_ref.so``: the reference's OWN plain-C CPU
statements of this path, compiled from the reference tree where it lies.

TEST INFRASTRUCTURE ONLY (like everything under ``oracle/``).

The reference's C engine is one Objective-C file
(crates/moeflux-sys/metal_infer/infer.m) that imports Metal, Foundation and
Accelerate, so it cannot be compiled as a whole outside macOS.  Its CPU twins of
the kernels on this path are however self-contained static C functions of that
file:

    bf16_to_f32 (:324)             cpu_dequant_matvec (:671)
    cpu_rms_norm_per_head (:729)   cpu_sdpa (:762)          cpu_sigmoid (:816)
    cpu_softmax (:821)             cpu_silu (:911)          cpu_conv1d_step (:922)
    apply_rotary_emb (:2138)       cpu_rms_norm_bare (:2521)
    cpu_rms_norm_gated (:2529)     cpu_gated_delta_recurrence (:7931)

``build()`` reads that file, cuts exactly those definitions out of it by name
(signature at the start of a line, body by brace matching), prepends libc
includes and ``ROPE_THETA`` as model_variant.h defines it, appends the exported
wrappers below, and hands the translation unit to gcc on standard input.  Only
the shared object is written, into the git-ignored ``oracle/_ref/``: no reference
source text is stored in this repository.  The shared object travels to
machines that do not have the reference tree; ``available()`` says whether it
can be used.

The wrappers add nothing but an exported name, except the two composite steps,
whose glue restates inline code of the reference's layer functions (the conv
history shift, infer.m:4874-4877; the q/k normalisation loop, :4885-4896; the
per-head gated norm, the RoPE -> append -> SDPA order of the full-attention
layer), so that the reference arm of the benchmark times a whole layer-step
made of the reference's own functions.
"""
from __future__ import annotations

import ctypes as C
import os
import re
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_DIR = os.path.join(_HERE, "_ref")
_SO = os.path.join(_DIR, "libmf_ref.so")

FUNCTIONS = ["bf16_to_f32", "cpu_dequant_matvec", "cpu_rms_norm_per_head", "cpu_sdpa", "cpu_sigmoid", "cpu_softmax",
             "cpu_silu", "cpu_conv1d_step", "apply_rotary_emb", "cpu_rms_norm_bare", "cpu_rms_norm_gated",
             "cpu_gated_delta_recurrence"]

_PRELUDE = """
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#define REF_API __attribute__((visibility("default")))
"""

# Exported names over the static functions, and the two composite layer-steps.
_WRAPPERS = r"""
REF_API float ref_rope_theta(void) { return ROPE_THETA; }
REF_API void ref_apply_rotary_emb(float *q, float *k, int pos, int nh, int nkv, int hd, int rd) {
    apply_rotary_emb(q, k, pos, nh, nkv, hd, rd);
}
REF_API void ref_sdpa(int kv_len, const float *q, const float *gate, const float *kc, const float *vc, int nh, int nkv,
                      int hd, float *out) {
    cpu_sdpa(kv_len, q, gate, kc, vc, nh, nkv, hd, out);
}
REF_API void ref_rms_norm_per_head(float *x, const uint16_t *w, int nh, int hd, float eps) {
    cpu_rms_norm_per_head(x, w, nh, hd, eps);
}
REF_API void ref_conv1d_step(const float *st, const float *x, const uint16_t *w, float *out, int ch, int ks) {
    cpu_conv1d_step(st, x, w, out, ch, ks);
}
REF_API void ref_rms_norm_bare(const float *x, float *out, int dim, float eps) { cpu_rms_norm_bare(x, out, dim, eps); }
REF_API void ref_rms_norm_gated(const float *x, const float *z, const uint16_t *w, float *out, int dim, float eps) {
    cpu_rms_norm_gated(x, z, w, out, dim, eps);
}
REF_API void ref_gated_delta_recurrence(const float *a_log, const uint16_t *dt_bias, const float *alpha,
                                        const float *beta, const float *q, const float *k, const float *v, int vh,
                                        int kh, int kd, int vd, float *ssm, float *out) {
    cpu_gated_delta_recurrence(a_log, dt_bias, alpha, beta, q, k, v, vh, kh, kd, vd, ssm, out);
}
REF_API void ref_dequant_matvec(const uint32_t *W, const uint16_t *s, const uint16_t *b, const float *x, float *out,
                                int out_dim, int in_dim, int group, int bits) {
    cpu_dequant_matvec(W, s, b, x, out, out_dim, in_dim, group, bits);
}
/* Full-attention layer-step from the reference's functions: RoPE(q, k) at pos, rows appended at kv_len, SDPA over
 * kv_len + 1 rows with the sigmoid gate.  q and k are rotated in place; the caches hold fp32 rows [pos][nkv*hd]. */
REF_API void ref_full_attn_step(int pos, int kv_len, float *q, const float *gate, float *k, const float *v,
                                float *kc, float *vc, float *out, int nh, int nkv, int hd, int rd) {
    apply_rotary_emb(q, k, pos, nh, nkv, hd, rd);
    memcpy(kc + (size_t)kv_len * nkv * hd, k, sizeof(float) * nkv * hd);
    memcpy(vc + (size_t)kv_len * nkv * hd, v, sizeof(float) * nkv * hd);
    cpu_sdpa(kv_len + 1, q, gate, kc, vc, nh, nkv, hd, out);
}
/* GatedDeltaNet layer-step from the reference's functions, sequenced as its layer function sequences them.
 * work: conv_dim floats of scratch. */
REF_API void ref_linear_attn_step(const float *qkv, const float *z, const float *alpha, const float *beta,
                                  const uint16_t *conv_w, const float *a_log, const uint16_t *dt_bias,
                                  const uint16_t *norm_w, float *conv_state, float *ssm, float *out, float *work,
                                  int vh, int kh, int kd, int vd, int ks, float eps) {
    const int total_key = kh * kd, conv_dim = 2 * total_key + vh * vd;
    cpu_conv1d_step(conv_state, qkv, conv_w, work, conv_dim, ks);
    memmove(conv_state, conv_state + conv_dim, (size_t)(ks - 2) * conv_dim * sizeof(float));
    memcpy(conv_state + (size_t)(ks - 2) * conv_dim, qkv, (size_t)conv_dim * sizeof(float));
    float *lq = work, *lk = work + total_key, *lv = work + 2 * total_key;
    const float inv_scale = 1.0f / sqrtf((float)kd);
    for (int h = 0; h < kh; h++) {
        float *qh = lq + h * kd;
        cpu_rms_norm_bare(qh, qh, kd, 1e-6f);
        const float q_scale = inv_scale * inv_scale;
        for (int d = 0; d < kd; d++) qh[d] *= q_scale;
    }
    for (int h = 0; h < kh; h++) {
        float *kh_ = lk + h * kd;
        cpu_rms_norm_bare(kh_, kh_, kd, 1e-6f);
        for (int d = 0; d < kd; d++) kh_[d] *= inv_scale;
    }
    if (z) {
        float *raw = (float *)malloc(sizeof(float) * (size_t)vh * vd);
        cpu_gated_delta_recurrence(a_log, dt_bias, alpha, beta, lq, lk, lv, vh, kh, kd, vd, ssm, raw);
        for (int h = 0; h < vh; h++)
            cpu_rms_norm_gated(raw + (size_t)h * vd, z + (size_t)h * vd, norm_w, out + (size_t)h * vd, vd, eps);
        free(raw);
    } else {
        cpu_gated_delta_recurrence(a_log, dt_bias, alpha, beta, lq, lk, lv, vh, kh, kd, vd, ssm, out);
    }
}
"""


def reference_root() -> str | None:
    """Root of the reference tree on this machine, or None."""
    for cand in (os.environ.get("MOEFLUX_REFERENCE"), "/root/reference"):
        if cand and os.path.exists(os.path.join(cand, "crates", "moeflux-sys", "metal_infer", "infer.m")):
            return cand
    return None


def _cut_function(text: str, name: str) -> str:
    """The definition of static function ``name``: from its signature line to the matching closing brace."""
    sig = re.compile(r"^static\s+(?:inline\s+)?[A-Za-z_][\w \t\*]*?\b" + re.escape(name) + r"\s*\(", re.M)
    m = None
    for cand in sig.finditer(text):
        # a prototype (a ';' before any '{') is not the definition
        brace, semi = text.find("{", cand.end()), text.find(";", cand.end())
        if brace != -1 and (semi == -1 or brace < semi):
            m = cand
            break
    if m is None:
        raise RuntimeError(f"reference function {name} not found")
    depth, i = 0, text.find("{", m.end())
    start = i
    while i < len(text):
        ch = text[i]
        if ch == "{":
            depth += 1
        elif ch == "}":
            depth -= 1
            if depth == 0:
                return text[m.start():i + 1]
        i += 1
    raise RuntimeError(f"unbalanced braces in reference function {name} (from offset {start})")


def translation_unit(root: str) -> str:
    mi = os.path.join(root, "crates", "moeflux-sys", "metal_infer")
    text = open(os.path.join(mi, "infer.m"), encoding="utf-8", errors="replace").read()
    variant = open(os.path.join(mi, "model_variant.h"), encoding="utf-8", errors="replace").read()
    m = re.search(r"^#define\s+ROPE_THETA\s+(\S+)", variant, re.M)
    if not m:
        raise RuntimeError("ROPE_THETA not found in model_variant.h")
    defs = [_cut_function(text, n) for n in FUNCTIONS]
    protos = [d[:d.find("{")].strip() + ";" for d in defs]
    return "\n".join([_PRELUDE, f"#define ROPE_THETA {m.group(1)}", *protos, *defs, _WRAPPERS])


def build(force: bool = False) -> str | None:
    """Compiles the shared object when the reference tree is present; returns its path, or None when neither the
    tree nor a previously built object exists."""
    root = reference_root()
    if root is None:
        return _SO if os.path.exists(_SO) else None
    src = os.path.join(root, "crates", "moeflux-sys", "metal_infer", "infer.m")
    if not force and os.path.exists(_SO) and os.path.getmtime(_SO) >= max(os.path.getmtime(src),
                                                                        os.path.getmtime(os.path.abspath(__file__))):
        return _SO
    os.makedirs(_DIR, exist_ok=True)
    gcc = "/usr/bin/gcc" if os.access("/usr/bin/gcc", os.X_OK) else "gcc"
    cmd = [gcc, "-O2", "-ffp-contract=off", "-fPIC", "-fvisibility=hidden", "-shared", "-x", "c", "-", "-o", _SO, "-lm"]
    r = subprocess.run(cmd, input=translation_unit(root), capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("gcc failed on the lifted reference functions:\n" + r.stderr)
    return _SO


def available() -> bool:
    return os.path.exists(_SO) or reference_root() is not None


_lib = None
_F = C.POINTER(C.c_float)
_U16 = C.POINTER(C.c_uint16)


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        path = build()
        if path is None:
            raise RuntimeError("oracle/_ref is not built and the reference tree is not on this machine")
        L = C.CDLL(path)
        L.ref_rope_theta.restype = C.c_float
        for name in ("ref_apply_rotary_emb", "ref_sdpa", "ref_rms_norm_per_head", "ref_conv1d_step", "ref_rms_norm_bare",
                     "ref_rms_norm_gated", "ref_gated_delta_recurrence", "ref_dequant_matvec", "ref_full_attn_step",
                     "ref_linear_attn_step"):
            getattr(L, name).restype = None
        _lib = L
    return _lib


def _f(a, copy=False):
    a = np.array(a, np.float32, copy=True) if copy else np.ascontiguousarray(a, dtype=np.float32)
    return a, a.ctypes.data_as(_F)


def _u(a):
    a = np.ascontiguousarray(a, dtype=np.uint16)
    return a, a.ctypes.data_as(_U16)


def rope_theta() -> float:
    return float(lib().ref_rope_theta())


def apply_rotary_emb(pos, q, k, num_heads, num_kv_heads, head_dim, rotary_dim):
    q, qp = _f(q, copy=True)
    k, kp = _f(k, copy=True)
    lib().ref_apply_rotary_emb(qp, kp, int(pos), int(num_heads), int(num_kv_heads), int(head_dim), int(rotary_dim))
    return q, k


def sdpa(kv_len, q, gate, k_cache, v_cache, num_heads, num_kv_heads, head_dim):
    q, qp = _f(q)
    gate, gp = _f(gate)
    kc, kp = _f(k_cache)
    vc, vp = _f(v_cache)
    out = np.zeros(num_heads * head_dim, np.float32)
    lib().ref_sdpa(int(kv_len), qp, gp, kp, vp, int(num_heads), int(num_kv_heads), int(head_dim), out.ctypes.data_as(_F))
    return out


def rms_norm_per_head(w_bits, num_heads, head_dim, x, eps=1e-6):
    x, xp = _f(x, copy=True)
    w, wp = _u(w_bits)
    lib().ref_rms_norm_per_head(xp, wp, int(num_heads), int(head_dim), C.c_float(eps))
    return x


def conv1d_step(conv_state, new_input, w_bits, channels, kernel_size=4):
    st, sp = _f(conv_state)
    x, xp = _f(new_input)
    w, wp = _u(w_bits)
    out = np.zeros(channels, np.float32)
    lib().ref_conv1d_step(sp, xp, wp, out.ctypes.data_as(_F), int(channels), int(kernel_size))
    return out


def rms_norm_bare(x, eps=1e-6):
    x, xp = _f(x)
    out = np.zeros_like(x)
    lib().ref_rms_norm_bare(xp, out.ctypes.data_as(_F), int(x.size), C.c_float(eps))
    return out


def rms_norm_gated(w_bits, x, z, eps=1e-6):
    x, xp = _f(x)
    z, zp = _f(z)
    w, wp = _u(w_bits)
    out = np.zeros_like(x)
    lib().ref_rms_norm_gated(xp, zp, wp, out.ctypes.data_as(_F), int(x.size), C.c_float(eps))
    return out


def gated_delta_recurrence(a_log, dt_bias_bits, alpha, beta, q, k, v, v_heads, k_heads, key_dim, value_dim, ssm_state):
    """Returns (new_state, out_values); the input state is not modified."""
    al, alp = _f(a_log)
    dt, dtp = _u(dt_bias_bits)
    a, ap = _f(alpha)
    b, bp = _f(beta)
    q, qp = _f(q)
    k, kp = _f(k)
    v, vp = _f(v)
    st, sp = _f(ssm_state, copy=True)
    out = np.zeros(v_heads * value_dim, np.float32)
    lib().ref_gated_delta_recurrence(alp, dtp, ap, bp, qp, kp, vp, int(v_heads), int(k_heads), int(key_dim),
                                     int(value_dim), sp, out.ctypes.data_as(_F))
    return st, out


def dequant_matvec(packed, scales, biases, in_dim, out_dim, x, group=64, bits=4):
    pk = np.ascontiguousarray(packed, dtype=np.uint32).reshape(-1)
    sc, scp = _u(np.asarray(scales).reshape(-1))
    bi, bip = _u(np.asarray(biases).reshape(-1))
    xv, xp = _f(np.asarray(x).reshape(-1))
    out = np.zeros(out_dim, np.float32)
    lib().ref_dequant_matvec(pk.ctypes.data_as(C.POINTER(C.c_uint32)), scp, bip, xp, out.ctypes.data_as(_F), int(out_dim),
                             int(in_dim), int(group), int(bits))
    return out


def full_attn_step(pos, kv_len, q, gate, k, v, k_cache, v_cache, num_heads, num_kv_heads, head_dim, rotary_dim):
    """One full-attention layer-step on fp32 host caches (row kv_len is appended in place)."""
    q, qp = _f(q, copy=True)
    k, kp = _f(k, copy=True)
    gate, gp = _f(gate)
    v, vp = _f(v)
    assert k_cache.dtype == np.float32 and k_cache.flags.c_contiguous and v_cache.dtype == np.float32
    out = np.zeros(num_heads * head_dim, np.float32)
    lib().ref_full_attn_step(int(pos), int(kv_len), qp, gp, kp, vp, k_cache.ctypes.data_as(_F),
                             v_cache.ctypes.data_as(_F), out.ctypes.data_as(_F), int(num_heads), int(num_kv_heads),
                             int(head_dim), int(rotary_dim))
    return out


def linear_attn_step(qkv, z, alpha, beta, conv_w_bits, a_log, dt_bias_bits, norm_w_bits, conv_state, ssm_state, g):
    """One GatedDeltaNet layer-step; conv_state [3][conv_dim] and ssm_state are fp32 arrays modified in place."""
    qkv, qp = _f(qkv)
    a, ap = _f(alpha)
    b, bp = _f(beta)
    cw, cwp = _u(conv_w_bits)
    al, alp = _f(a_log)
    dt, dtp = _u(dt_bias_bits)
    zp = nwp = None
    if z is not None:
        z, zp = _f(z)
        nw, nwp = _u(norm_w_bits)
    work = np.zeros(g.conv_dim, np.float32)
    out = np.zeros(g.total_value, np.float32)
    lib().ref_linear_attn_step(qp, zp, ap, bp, cwp, alp, dtp, nwp, conv_state.ctypes.data_as(_F),
                               ssm_state.ctypes.data_as(_F), out.ctypes.data_as(_F), work.ctypes.data_as(_F),
                               int(g.linear_num_v_heads), int(g.linear_num_k_heads), int(g.linear_key_dim),
                               int(g.linear_value_dim), int(g.conv_kernel_size), C.c_float(g.rms_norm_eps))
    return out


if __name__ == "__main__":
    print(build(force=True))
