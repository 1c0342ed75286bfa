"""ctypes wrapper over the CPU oracle (``libmf_oracle.so``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by ``__graft_entry__.smoke()``
and by ``bench.py``'s CPU-baseline leg, as the checker.  The library in
``moeflux_b200`` never imports this package.

Parity pinned against the reference's own C functions (``oracle/ref.py``,
``tests/test_oracle_ref.py``): see the header of ``mf_oracle.c``.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from dataclasses import dataclass

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libmf_oracle.so")


def build(force: bool = False) -> str:
    """Compile the oracle with the Makefile beside it (gcc + OpenMP)."""
    src = os.path.join(_HERE, "mf_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "libmf_oracle.so"], stdout=subprocess.DEVNULL)
    return _SO


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        _lib = C.CDLL(_SO)
        _lib.mfo_f32_to_bf16.restype = C.c_uint16
        _lib.mfo_f32_to_bf16.argtypes = [C.c_float]
    return _lib


@dataclass(frozen=True)
class Geometry:
    """Model geometry of the path (crates/moeflux/src/riir/variants.rs:383-423,
    derived dims :219-250; constants :358-379)."""

    num_layers: int = 60
    full_attn_interval: int = 4
    num_attn_heads: int = 32
    num_kv_heads: int = 2
    head_dim: int = 256
    rotary_dim: int = 64
    rope_theta: float = 1.0e7
    linear_num_v_heads: int = 64
    linear_num_k_heads: int = 16
    linear_key_dim: int = 128
    linear_value_dim: int = 128
    conv_kernel_size: int = 4
    rms_norm_eps: float = 1e-6

    @property
    def q_dim(self) -> int:
        return self.num_attn_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_kv_heads * self.head_dim

    @property
    def total_key(self) -> int:
        return self.linear_num_k_heads * self.linear_key_dim

    @property
    def total_value(self) -> int:
        return self.linear_num_v_heads * self.linear_value_dim

    @property
    def conv_dim(self) -> int:
        return 2 * self.total_key + self.total_value

    @property
    def ssm_elems(self) -> int:
        return self.linear_num_v_heads * self.linear_value_dim * self.linear_key_dim

    def is_full_layer(self, i: int) -> bool:
        return (i + 1) % self.full_attn_interval == 0

    @property
    def num_full_layers(self) -> int:
        return sum(self.is_full_layer(i) for i in range(self.num_layers))

    @property
    def num_linear_layers(self) -> int:
        return self.num_layers - self.num_full_layers


A17B = Geometry()


def _f(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a, a.ctypes.data_as(C.POINTER(C.c_float))


def _u16(a):
    a = np.ascontiguousarray(a, dtype=np.uint16)
    return a, a.ctypes.data_as(C.POINTER(C.c_uint16))


def num_threads() -> int:
    return int(lib().mfo_num_threads())


def use_all_cores() -> int:
    """Let the OpenMP loops use every core this process may run on (launchers
    such as torchrun export OMP_NUM_THREADS=1).  Returns the thread count."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    lib().mfo_set_num_threads(int(n))
    return num_threads()


def f32_to_bf16_bits(x) -> np.ndarray:
    """Round-to-nearest-even f32 -> bf16 bit patterns (vectorised twin of
    ``mfo_f32_to_bf16``; inputs must be finite)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    u = u + 0x7FFF + ((u >> 16) & 1)
    return (u >> 16).astype(np.uint16)


def bf16_bits_to_f32(b) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def round_bf16(x) -> np.ndarray:
    return bf16_bits_to_f32(f32_to_bf16_bits(x)).reshape(np.shape(x))


def rope_inv_freq(g: Geometry = A17B) -> np.ndarray:
    out = np.zeros(g.rotary_dim // 2, np.float32)
    lib().mfo_rope_inv_freq(C.c_float(g.rope_theta), g.rotary_dim, out.ctypes.data_as(C.POINTER(C.c_float)))
    return out


def apply_rotary_emb(pos: int, q, k, g: Geometry = A17B):
    """Returns rotated copies (q, k); raises ValueError where the reference
    returns an error (pos < 0)."""
    q, qp = _f(np.array(q, np.float32, copy=True))
    k, kp = _f(np.array(k, np.float32, copy=True))
    rc = lib().mfo_apply_rotary_emb(int(pos), qp, kp, g.num_attn_heads, g.num_kv_heads, g.head_dim,
                                    g.rotary_dim, C.c_float(g.rope_theta))
    if rc:
        raise ValueError("apply_rotary_emb: bad arguments")
    return q, k


def rms_norm_per_head(w_bits, num_heads: int, head_dim: int, x, eps: float = 1e-6):
    x, xp = _f(np.array(x, np.float32, copy=True))
    w, wp = _u16(w_bits)
    if lib().mfo_rms_norm_per_head(wp, num_heads, head_dim, C.c_float(eps), xp):
        raise ValueError("rms_norm_per_head: bad arguments")
    return x


def dequant_matvec_4bit(packed, scales, biases, in_dim: int, out_dim: int, x) -> np.ndarray:
    """cpu_matvec.rs:83-171.  Raises ValueError where the reference returns an error
    (in_dim not a multiple of 64, slice lengths that do not match the shape)."""
    pk = np.ascontiguousarray(packed, dtype=np.uint32).reshape(-1)
    sc, scp = _u16(np.asarray(scales).reshape(-1))
    bi, bip = _u16(np.asarray(biases).reshape(-1))
    xv, xp = _f(np.asarray(x).reshape(-1))
    if in_dim <= 0 or in_dim % 64 != 0:
        raise ValueError(f"in_dim {in_dim} is not a multiple of GROUP_SIZE=64")
    for name, got, exp in (("packed", pk.size, out_dim * in_dim // 8), ("scales", sc.size, out_dim * in_dim // 64),
                           ("biases", bi.size, out_dim * in_dim // 64), ("x", xv.size, in_dim)):
        if got != exp:
            raise ValueError(f"slice length mismatch on '{name}': got {got} elements, expected {exp}")
    out = np.zeros(out_dim, np.float32)
    if lib().mfo_dequant_matvec_4bit(pk.ctypes.data_as(C.POINTER(C.c_uint32)), scp, bip, int(in_dim), int(out_dim), xp,
                                     out.ctypes.data_as(C.POINTER(C.c_float))):
        raise ValueError("dequant_matvec_4bit: bad arguments")
    return out


def split_q_gate(q_proj, g: Geometry = A17B):
    qp_, p = _f(q_proj)
    q = np.zeros(g.q_dim, np.float32)
    gate = np.zeros(g.q_dim, np.float32)
    lib().mfo_split_q_gate(p, g.num_attn_heads, g.head_dim, q.ctypes.data_as(C.POINTER(C.c_float)),
                           gate.ctypes.data_as(C.POINTER(C.c_float)))
    return q, gate


def sdpa(kv_len: int, q, gate, k_cache, v_cache, g: Geometry = A17B) -> np.ndarray:
    q, qp = _f(q)
    gate, gp = _f(gate)
    kc, kp = _f(k_cache)
    vc, vp = _f(v_cache)
    out = np.zeros(g.q_dim, np.float32)
    rc = lib().mfo_sdpa(int(kv_len), qp, gp, kp, vp, out.ctypes.data_as(C.POINTER(C.c_float)),
                        g.num_attn_heads, g.num_kv_heads, g.head_dim)
    if rc:
        raise ValueError("sdpa: bad arguments (kv_len must be > 0)")
    return out


def attn_scores_batched(num_heads, num_kv_heads, head_dim, seq_len, q, k_cache, scale):
    q, qp = _f(q)
    kc, kp = _f(k_cache)
    out = np.zeros(num_heads * seq_len, np.float32)
    if lib().mfo_attn_scores_batched(num_heads, num_kv_heads, head_dim, seq_len, qp, kp,
                                     C.c_float(scale), out.ctypes.data_as(C.POINTER(C.c_float))):
        raise ValueError("attn_scores_batched: bad arguments")
    return out


def attn_softmax_batched(num_heads, seq_len, scores):
    s, sp = _f(np.array(scores, np.float32, copy=True))
    if lib().mfo_attn_softmax_batched(num_heads, seq_len, sp):
        raise ValueError("attn_softmax_batched: bad arguments")
    return s


def attn_values_batched(num_heads, num_kv_heads, head_dim, seq_len, scores, v_cache):
    s, sp = _f(scores)
    vc, vp = _f(v_cache)
    out = np.zeros(num_heads * head_dim, np.float32)
    if lib().mfo_attn_values_batched(num_heads, num_kv_heads, head_dim, seq_len, sp, vp,
                                     out.ctypes.data_as(C.POINTER(C.c_float))):
        raise ValueError("attn_values_batched: bad arguments")
    return out


def sigmoid_gate(gate, x):
    gt, gp = _f(gate)
    x, xp = _f(np.array(x, np.float32, copy=True))
    if lib().mfo_sigmoid_gate(int(x.size), gp, xp):
        raise ValueError("sigmoid_gate: bad arguments")
    return x


def conv1d_step(conv_state, new_input, w_bits, channels: int, kernel_size: int = 4):
    st, sp = _f(conv_state)
    x, xp = _f(new_input)
    w, wp = _u16(w_bits)
    out = np.zeros(channels, np.float32)
    if lib().mfo_conv1d_step(sp, xp, wp, channels, kernel_size, out.ctypes.data_as(C.POINTER(C.c_float))):
        raise ValueError("conv1d_step: bad arguments")
    return out


def conv_state_shift(conv_state, new_input, channels: int, kernel_size: int = 4):
    st, sp = _f(np.array(conv_state, np.float32, copy=True))
    x, xp = _f(new_input)
    lib().mfo_conv_state_shift(sp, xp, channels, kernel_size)
    return st


def rms_norm_bare(x, eps: float = 1e-6):
    x, xp = _f(x)
    out = np.zeros_like(x)
    if lib().mfo_rms_norm_bare(int(x.size), C.c_float(eps), xp, out.ctypes.data_as(C.POINTER(C.c_float))):
        raise ValueError("rms_norm_bare: bad arguments")
    return out


def rms_norm_gated(w_bits, x, z, eps: float = 1e-6):
    x, xp = _f(x)
    z, zp = _f(z)
    w, wp = _u16(w_bits)
    out = np.zeros_like(x)
    if lib().mfo_rms_norm_gated(wp, int(x.size), C.c_float(eps), xp, zp,
                                out.ctypes.data_as(C.POINTER(C.c_float))):
        raise ValueError("rms_norm_gated: bad arguments")
    return out


def rms_norm_qk(q, k, num_k_heads: int, key_dim: int):
    q, qp = _f(np.array(q, np.float32, copy=True))
    k, kp = _f(np.array(k, np.float32, copy=True))
    if lib().mfo_rms_norm_qk(qp, kp, num_k_heads, key_dim):
        raise ValueError("rms_norm_qk: bad arguments")
    return q, k


def decay_beta(alpha, beta, a_log, dt_bias_bits):
    a, ap = _f(alpha)
    b, bp = _f(beta)
    al, alp = _f(a_log)
    dt, dtp = _u16(dt_bias_bits)
    n = int(a.size)
    gd = np.zeros(n, np.float32)
    bg = np.zeros(n, np.float32)
    if lib().mfo_decay_beta(ap, bp, alp, dtp, n, gd.ctypes.data_as(C.POINTER(C.c_float)),
                            bg.ctypes.data_as(C.POINTER(C.c_float))):
        raise ValueError("decay_beta: bad arguments")
    return gd, bg


def gated_delta_recurrence(a_log, dt_bias_bits, alpha, beta, q, k, v, v_heads, k_heads, key_dim,
                           value_dim, ssm_state):
    """Returns (new_state, out_values); the input state is not modified."""
    al, alp = _f(a_log)
    dt, dtp = _u16(dt_bias_bits)
    a, ap = _f(alpha)
    b, bp = _f(beta)
    q, qp = _f(q)
    k, kp = _f(k)
    v, vp = _f(v)
    st, sp = _f(np.array(ssm_state, np.float32, copy=True))
    out = np.zeros(v_heads * value_dim, np.float32)
    if lib().mfo_gated_delta_recurrence(alp, dtp, ap, bp, qp, kp, vp, v_heads, k_heads, key_dim,
                                        value_dim, sp, out.ctypes.data_as(C.POINTER(C.c_float))):
        raise ValueError("gated_delta_recurrence: bad arguments")
    return st, out


def full_attn_step(pos, kv_len, q, gate, k, v, k_cache, v_cache, g: Geometry = A17B, kv_bf16=False):
    """One decode step on host caches (modified in place: row kv_len is appended).
    k_cache/v_cache: float32 arrays with at least kv_len+1 rows of kv_dim."""
    q, qp = _f(np.array(q, np.float32, copy=True))
    k, kp = _f(np.array(k, np.float32, copy=True))
    gate, gp = _f(gate)
    v, vp = _f(v)
    assert k_cache.dtype == np.float32 and k_cache.flags.c_contiguous
    assert v_cache.dtype == np.float32 and v_cache.flags.c_contiguous
    assert k_cache.size >= (kv_len + 1) * g.kv_dim
    out = np.zeros(g.q_dim, np.float32)
    rc = lib().mfo_full_attn_step(int(pos), int(kv_len), qp, gp, kp, vp,
                                  k_cache.ctypes.data_as(C.POINTER(C.c_float)),
                                  v_cache.ctypes.data_as(C.POINTER(C.c_float)),
                                  out.ctypes.data_as(C.POINTER(C.c_float)), g.num_attn_heads,
                                  g.num_kv_heads, g.head_dim, g.rotary_dim, C.c_float(g.rope_theta),
                                  int(bool(kv_bf16)))
    if rc:
        raise ValueError("full_attn_step: pos must equal kv_len and be >= 0")
    return out


def linear_attn_step(qkv, z, alpha, beta, conv_w_bits, a_log, dt_bias_bits, norm_w_bits, conv_state,
                     ssm_state, g: Geometry = A17B):
    """One GatedDeltaNet decode step; conv_state [K-1][conv_dim] and ssm_state
    are float32 arrays modified in place.  z=None skips the gated norm."""
    qkv, qp = _f(qkv)
    a, ap = _f(alpha)
    b, bp = _f(beta)
    cw, cwp = _u16(conv_w_bits)
    al, alp = _f(a_log)
    dt, dtp = _u16(dt_bias_bits)
    assert conv_state.dtype == np.float32 and conv_state.flags.c_contiguous
    assert ssm_state.dtype == np.float32 and ssm_state.flags.c_contiguous
    if z is not None:
        z, zp = _f(z)
        nw, nwp = _u16(norm_w_bits)
    else:
        zp = None
        nwp = None
    out = np.zeros(g.total_value, np.float32)
    rc = lib().mfo_linear_attn_step(qp, zp, ap, bp, cwp, alp, dtp, nwp,
                                    conv_state.ctypes.data_as(C.POINTER(C.c_float)),
                                    ssm_state.ctypes.data_as(C.POINTER(C.c_float)),
                                    out.ctypes.data_as(C.POINTER(C.c_float)), g.linear_num_v_heads,
                                    g.linear_num_k_heads, g.linear_key_dim, g.linear_value_dim,
                                    g.conv_kernel_size, C.c_float(g.rms_norm_eps))
    if rc:
        raise ValueError("linear_attn_step: bad arguments")
    return out


def sdpa_partial(p0, p1, q, k_cache, v_cache, g: Geometry = A17B):
    q, qp = _f(q)
    kc, kp = _f(k_cache)
    vc, vp = _f(v_cache)
    o = np.zeros((g.num_attn_heads, g.head_dim), np.float32)
    m = np.zeros(g.num_attn_heads, np.float32)
    l = np.zeros(g.num_attn_heads, np.float32)
    P = C.POINTER(C.c_float)
    if lib().mfo_sdpa_partial(int(p0), int(p1), qp, kp, vp, o.ctypes.data_as(P), m.ctypes.data_as(P),
                              l.ctypes.data_as(P), g.num_attn_heads, g.num_kv_heads, g.head_dim):
        raise ValueError("sdpa_partial: bad arguments")
    return o, m, l


def lse_merge_gate(o_parts, m_parts, l_parts, gate, g: Geometry = A17B):
    o, op = _f(o_parts)
    m, mp = _f(m_parts)
    l, lp = _f(l_parts)
    n = int(m.size // g.num_attn_heads)
    if gate is not None:
        gate, gp = _f(gate)
    else:
        gp = None
    out = np.zeros(g.q_dim, np.float32)
    if lib().mfo_lse_merge_gate(n, op, mp, lp, gp, out.ctypes.data_as(C.POINTER(C.c_float)),
                                g.num_attn_heads, g.head_dim):
        raise ValueError("lse_merge_gate: bad arguments")
    return out


def mla_sdpa_folded(cache_len: int, softmax_scale: float, q_prime, q_pe, latent, rope_k, kv_lora_rank: int = 512,
                    rope_dim: int = 64, tile: int = 0) -> np.ndarray:
    """shaders.metal:1717-1822 (tile == 0) or the tiled online-softmax form :1845-1987 with tiles of `tile` positions.
    Returns v_combine [num_heads, kv_lora_rank]."""
    qp, qpp = _f(q_prime)
    pe, pep = _f(q_pe)
    lat, lp = _f(latent)
    rk, rp = _f(rope_k)
    H = qp.size // kv_lora_rank
    out = np.zeros((H, kv_lora_rank), np.float32)
    op = out.ctypes.data_as(C.POINTER(C.c_float))
    if tile:
        rc = lib().mfo_mla_sdpa_folded_tiled(H, kv_lora_rank, rope_dim, int(cache_len), int(tile), C.c_float(softmax_scale),
                                             qpp, pep, lp, rp, op)
    else:
        rc = lib().mfo_mla_sdpa_folded(H, kv_lora_rank, rope_dim, int(cache_len), C.c_float(softmax_scale), qpp, pep, lp,
                                       rp, op)
    if rc:
        raise ValueError("mla_sdpa_folded: bad arguments")
    return out
