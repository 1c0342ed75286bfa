"""Pins the CPU oracle (oracle/mf_oracle.c) to the reference's own C code.

oracle/ref.py compiles the plain-C CPU twins of this path out of the reference's
crates/moeflux-sys/metal_infer/infer.m (cpu_sdpa, apply_rotary_emb,
cpu_conv1d_step, cpu_rms_norm_bare/_gated/_per_head, cpu_gated_delta_recurrence,
cpu_dequant_matvec).  These tests hold the restatement to that code on the input
formulas, probe points and bounds of the reference's own differential tests
(crates/moeflux/tests/diff_oracle.rs): <= 128 ULP for RoPE (:1357, :1379-1442),
conv1d (:2079-2133), gated norm (:2146-2196) and the recurrence from a zero
state (:2229-2327); cosine >= 0.9999 and max|d| <= 1e-3 * max|out| for SDPA
(:1541-1615).  No GPU.
"""
import numpy as np
import pytest

import oracle as O
import oracle.ref as R
from oracle import A17B as G
from tests import inputs as I

pytestmark = pytest.mark.skipif(not R.available(), reason="neither the reference tree nor a built oracle/_ref is here")

ULP_BOUND = 128  # diff_oracle.rs:1357


def ulp_diff(a, b):
    """Largest distance in units of last place between two float32 arrays (sign-magnitude ordered ints)."""
    def key(x):
        u = np.ascontiguousarray(x, np.float32).view(np.int32).astype(np.int64)
        return np.where(u < 0, -(u & 0x7FFFFFFF), u)
    return int(np.max(np.abs(key(a) - key(b))))


def test_reference_constants_match_the_geometry():
    assert R.rope_theta() == G.rope_theta


@pytest.mark.parametrize("pos", [0, 1, 17, 1024, 65535])
def test_rope(pos):
    q = I.ramp_sin(G.q_dim, 0.013, 0.7, 0.1)
    k = I.ramp_cos(G.kv_dim, 0.019, 0.5, -0.2)
    q1, k1 = O.apply_rotary_emb(pos, q, k)
    q2, k2 = R.apply_rotary_emb(pos, q, k, G.num_attn_heads, G.num_kv_heads, G.head_dim, G.rotary_dim)
    assert ulp_diff(q1, q2) <= ULP_BOUND and ulp_diff(k1, k2) <= ULP_BOUND


@pytest.mark.parametrize("kv_len", [1, 8, 32, 33, 64, 512, 4096])
def test_sdpa(kv_len):
    q = I.ramp_sin(G.q_dim, 0.011, 0.6, 0.05)
    gate = I.ramp_cos(G.q_dim, 0.007, 1.2, -0.1)
    K = I.ramp_sin(kv_len * G.kv_dim, 0.013, 0.5, 0.02).reshape(kv_len, G.kv_dim)
    V = I.ramp_cos(kv_len * G.kv_dim, 0.017, 0.4, -0.05).reshape(kv_len, G.kv_dim)
    got = O.sdpa(kv_len, q, gate, K, V)
    ref = R.sdpa(kv_len, q, gate, K, V, G.num_attn_heads, G.num_kv_heads, G.head_dim)
    assert I.cosine(got, ref) >= 0.9999
    assert np.max(np.abs(got - ref)) <= 1e-3 * np.max(np.abs(ref))
    # the two are the same arithmetic up to the order of the normalisation: far inside the reference's floor
    assert I.rel_err(got, ref) <= 2e-6


def test_sdpa_seeded_normal_inputs():
    r = I.rng(0)
    kv_len = 1000
    q, gate, _, _ = I.gqa_step_inputs(r)
    K, V = I.normal(r, (kv_len, G.kv_dim)), I.normal(r, (kv_len, G.kv_dim))
    got = O.sdpa(kv_len, q, gate, K, V)
    ref = R.sdpa(kv_len, q, gate, K, V, G.num_attn_heads, G.num_kv_heads, G.head_dim)
    assert I.rel_err(got, ref) <= 2e-6


def test_per_head_rms_norm():
    r = I.rng(3)
    w = O.f32_to_bf16_bits(1.0 + I.normal(r, G.head_dim, 0.1))
    x = I.normal(r, G.q_dim)
    assert ulp_diff(O.rms_norm_per_head(w, G.num_attn_heads, G.head_dim, x),
                    R.rms_norm_per_head(w, G.num_attn_heads, G.head_dim, x)) <= ULP_BOUND


def test_conv1d_step():
    # state and input formulas of conv1d_step_cpu_close_c_vs_rust (diff_oracle.rs:2091-2097); the reference reads
    # the weights from the model file, here they are seeded N(0, 0.5) bf16
    ch = G.conv_dim
    st = I.ramp_sin(3 * ch, 0.013, 0.4, 0.02)
    x = I.ramp_cos(ch, 0.019, 0.5, -0.1)
    w = O.f32_to_bf16_bits(I.normal(I.rng(9), 4 * ch, 0.5))
    got, ref = O.conv1d_step(st, x, w, ch), R.conv1d_step(st, x, w, ch)
    # The oracle follows the Rust port (fused multiply-adds), the C twin rounds every product: a four-term sum that
    # nearly cancels differs by many ULPs of its small result, so the ULP bound is taken where the result is not a
    # cancellation (|y| >= 1% of the largest output) and a tensor-wide bound covers the rest.
    big = np.abs(ref) >= 1e-2 * np.max(np.abs(ref))
    assert ulp_diff(got[big], ref[big]) <= ULP_BOUND
    assert I.rel_err(got, ref) <= 1e-6


def test_rms_norm_bare_and_gated():
    r = I.rng(4)
    x, z = I.normal(r, 128), I.normal(r, 128)
    w = O.f32_to_bf16_bits(1.0 + I.normal(r, 128, 0.1))
    assert ulp_diff(O.rms_norm_bare(x), R.rms_norm_bare(x)) <= ULP_BOUND
    assert ulp_diff(O.rms_norm_gated(w, x, z), R.rms_norm_gated(w, x, z)) <= ULP_BOUND


def _recurrence_inputs(r):
    a_log = r.uniform(0.0, 2.7, G.linear_num_v_heads).astype(np.float32)
    dt = O.f32_to_bf16_bits(I.normal(r, G.linear_num_v_heads))
    alpha, beta = I.normal(r, G.linear_num_v_heads), I.normal(r, G.linear_num_v_heads)
    q, k = I.normal(r, G.total_key, 0.1), I.normal(r, G.total_key, 0.1)
    v = I.normal(r, G.total_value)
    return a_log, dt, alpha, beta, q, k, v


def test_recurrence_from_zero_state():
    # the reference's own inputs (diff_oracle.rs:2245-2260); A_log and dt_bias come from the model file there and are
    # seeded here
    r = I.rng(5)
    a_log = r.uniform(0.0, 2.7, G.linear_num_v_heads).astype(np.float32)
    dt = O.f32_to_bf16_bits(I.normal(r, G.linear_num_v_heads))
    alpha = I.ramp_sin(G.linear_num_v_heads, 0.013, 0.3, 0.0)
    beta = I.ramp_cos(G.linear_num_v_heads, 0.017, 0.5, 0.0)
    q = I.ramp_sin(G.total_key, 0.011, 0.4, 0.05)
    k = I.ramp_cos(G.total_key, 0.019, 0.5, -0.1)
    v = I.ramp_sin(G.total_value, 0.023, 0.6, 0.02)
    args = (a_log, dt, alpha, beta, q, k, v)
    dims = (G.linear_num_v_heads, G.linear_num_k_heads, G.linear_key_dim, G.linear_value_dim)
    zero = np.zeros(G.ssm_elems, np.float32)
    s1, o1 = O.gated_delta_recurrence(*args, *dims, zero)
    s2, o2 = R.gated_delta_recurrence(*args, *dims, zero)
    assert ulp_diff(s1, s2) <= ULP_BOUND and ulp_diff(o1, o2) <= ULP_BOUND
    # seeded N(0, .) inputs: the read-out is a 128-term signed sum, so the ULP bound holds where it did not cancel
    args = _recurrence_inputs(I.rng(5))
    s1, o1 = O.gated_delta_recurrence(*args, *dims, zero)
    s2, o2 = R.gated_delta_recurrence(*args, *dims, zero)
    big = np.abs(o2) >= 1e-2 * np.max(np.abs(o2))
    assert ulp_diff(s1, s2) <= ULP_BOUND and ulp_diff(o1[big], o2[big]) <= ULP_BOUND and I.rel_err(o1, o2) <= 1e-6


def test_recurrence_from_seeded_state():
    r = I.rng(6)
    args = _recurrence_inputs(r)
    dims = (G.linear_num_v_heads, G.linear_num_k_heads, G.linear_key_dim, G.linear_value_dim)
    st = I.normal(r, G.ssm_elems, 0.02)
    s1, o1 = O.gated_delta_recurrence(*args, *dims, st)
    s2, o2 = R.gated_delta_recurrence(*args, *dims, st)
    # sums of 128 signed terms: ULPs of a near-cancelled element are not meaningful, the tensor-wide bound is
    assert I.rel_err(s1, s2) <= 1e-6 and I.rel_err(o1, o2) <= 1e-5


def test_whole_layer_steps_chain():
    """Ten chained steps of both layer kinds: the oracle's composites against the composites made of the reference's
    functions (state carried by each side on its own)."""
    r = I.rng(7)
    conv_w, a_log, dt, nw = I.gdn_weights(r)
    c1 = I.normal(r, (3, G.conv_dim))
    s1 = I.normal(r, G.ssm_elems, 0.02)
    c2, s2 = c1.copy(), s1.copy()
    n = 10
    K1 = np.zeros((n, G.kv_dim), np.float32)
    V1 = np.zeros((n, G.kv_dim), np.float32)
    K2, V2 = K1.copy(), V1.copy()
    for pos in range(n):
        qkv, z, alpha, beta = I.gdn_step_inputs(r)
        o1 = O.linear_attn_step(qkv, z, alpha, beta, conv_w, a_log, dt, nw, c1, s1)
        o2 = R.linear_attn_step(qkv, z, alpha, beta, conv_w, a_log, dt, nw, c2, s2, G)
        assert I.rel_err(o1, o2) <= 1e-5, pos
        q, gate, k, v = I.gqa_step_inputs(r)
        f1 = O.full_attn_step(pos, pos, q, gate, k, v, K1, V1)
        f2 = R.full_attn_step(pos, pos, q, gate, k, v, K2, V2, G.num_attn_heads, G.num_kv_heads, G.head_dim,
                              G.rotary_dim)
        assert I.rel_err(f1, f2) <= 2e-6, pos
    assert np.array_equal(c1, c2)
    assert I.rel_err(s1, s2) <= 1e-5
    assert ulp_diff(K1, K2) <= ULP_BOUND and np.array_equal(V1, V2)


@pytest.mark.parametrize("shape", [(64, 3), (256, 17), (4096, 8)])
def test_dequant_matvec_random_nibbles(shape):
    """Random nibbles, scales and biases: pins nibble order within a word, the word order within a group and the
    group stride, which the reference's three uniform-nibble known answers cannot tell apart."""
    in_dim, out_dim = shape
    r = I.rng(8 + in_dim)
    packed, sc, bi = I.quant_weights(r, in_dim, out_dim)
    x = I.normal(r, in_dim)
    got = O.dequant_matvec_4bit(packed, sc, bi, in_dim, out_dim, x)
    ref = R.dequant_matvec(packed, sc, bi, in_dim, out_dim, x)
    assert I.rel_err(got, ref) <= 1e-5
    # and the nibble order explicitly, in float64
    w = np.zeros((out_dim, in_dim))
    pk = packed.reshape(out_dim, in_dim // 8).astype(np.uint64)
    for n in range(8):
        w[:, n::8] = ((pk >> np.uint64(4 * n)) & np.uint64(15)).astype(np.float64)
    s = np.repeat(O.bf16_bits_to_f32(sc).reshape(out_dim, in_dim // 64).astype(np.float64), 64, axis=1)
    b = np.repeat(O.bf16_bits_to_f32(bi).reshape(out_dim, in_dim // 64).astype(np.float64), 64, axis=1)
    assert I.rel_err(ref, (w * s + b) @ x.astype(np.float64)) <= 1e-5
