"""Pins the CPU oracle: closed-form known answers derived from the reference's
formulas, the reference's own unit-test facts (RoPE identity at pos 0, SiLU and
bare-norm values, state ops), and an independent float64 numpy restatement on
the reference's differential-test inputs.  No GPU."""
import numpy as np
import pytest

import oracle as O
from oracle import A17B as G
from tests import inputs as I


def test_bf16_roundtrip_and_rne():
    x = np.array([1.0, 1.00390625, 1.005859375, -2.5, 3.1415927], np.float32)
    bits = O.f32_to_bf16_bits(x)
    scalar = np.array([O.lib().mfo_f32_to_bf16(float(v)) for v in x], np.uint16)
    assert np.array_equal(bits, scalar)
    # 1.00390625 = 1 + 2^-8 is a tie between 1.0 and 1.0078125: even mantissa wins
    assert O.bf16_bits_to_f32(bits)[1] == 1.0
    assert O.bf16_bits_to_f32(bits)[0] == 1.0 and O.bf16_bits_to_f32(bits)[3] == -2.5


def test_rope_pos0_is_identity():
    # crates/moeflux/src/riir/rope.rs:352-381
    q = I.ramp_sin(G.q_dim, 0.013, 0.7, 0.1)
    k = I.ramp_cos(G.kv_dim, 0.019, 0.5, -0.2)
    q2, k2 = O.apply_rotary_emb(0, q, k)
    assert np.array_equal(q, q2) and np.array_equal(k, k2)


def test_rope_negative_pos_is_error():
    with pytest.raises(ValueError):
        O.apply_rotary_emb(-1, np.zeros(G.q_dim, np.float32), np.zeros(G.kv_dim, np.float32))


@pytest.mark.parametrize("pos", [1, 17, 1024, 65535])
def test_rope_matches_float64_formula(pos):
    q = I.ramp_sin(G.q_dim, 0.013, 0.7, 0.1)
    k = I.ramp_cos(G.kv_dim, 0.019, 0.5, -0.2)
    q2, k2 = O.apply_rotary_emb(pos, q, k)
    inv = O.rope_inv_freq(G).astype(np.float64)
    ang = (np.float32(pos) * O.rope_inv_freq(G)).astype(np.float64)  # angle is formed in f32
    for x, y, nh in ((q, q2, G.num_attn_heads), (k, k2, G.num_kv_heads)):
        x = x.reshape(nh, G.head_dim).astype(np.float64)
        ref = x.copy()
        ref[:, :32] = x[:, :32] * np.cos(ang) - x[:, 32:64] * np.sin(ang)
        ref[:, 32:64] = x[:, :32] * np.sin(ang) + x[:, 32:64] * np.cos(ang)
        assert np.max(np.abs(ref - y.reshape(nh, G.head_dim))) < 2e-6
        # untouched tail, norm preserved per rotated pair
        assert np.array_equal(y.reshape(nh, G.head_dim)[:, 64:], x[:, 64:].astype(np.float32))
    assert inv[0] == 1.0 and abs(inv[1] - 1e7 ** (-2 / 64)) < 1e-7


def test_sdpa_kv_len_1_is_v_times_sigmoid_gate():
    r = I.rng(1)
    q, gate, k, v = I.gqa_step_inputs(r)
    out = O.sdpa(1, q, gate, k, v).reshape(G.num_attn_heads, G.head_dim)
    sig = 1.0 / (1.0 + np.exp(-gate.astype(np.float64))).reshape(G.num_attn_heads, G.head_dim)
    for h in range(G.num_attn_heads):
        ref = v.reshape(G.num_kv_heads, G.head_dim)[h // 16] * sig[h]
        assert np.max(np.abs(out[h] - ref)) < 1e-6


def test_sdpa_uniform_keys_give_mean_of_values():
    r = I.rng(2)
    n = 37
    q, gate, k, _ = I.gqa_step_inputs(r)
    K = np.tile(k, (n, 1))
    V = I.normal(r, (n, G.kv_dim))
    out = O.sdpa(n, q, gate, K, V).reshape(G.num_attn_heads, G.head_dim)
    sig = 1.0 / (1.0 + np.exp(-gate.astype(np.float64))).reshape(G.num_attn_heads, G.head_dim)
    mean_v = V.astype(np.float64).mean(0).reshape(G.num_kv_heads, G.head_dim)
    for h in range(G.num_attn_heads):
        assert np.max(np.abs(out[h] - mean_v[h // 16] * sig[h])) < 1e-5


def test_sdpa_rejects_empty_cache():
    z = np.zeros(G.q_dim, np.float32)
    with pytest.raises(ValueError):
        O.sdpa(0, z, z, np.zeros(G.kv_dim, np.float32), np.zeros(G.kv_dim, np.float32))


@pytest.mark.parametrize("kv_len", [1, 8, 64, 512])
def test_sdpa_matches_float64_on_reference_inputs(kv_len):
    # inputs of sdpa_cpu_close_c_vs_rust (diff_oracle.rs:1555-1571); its floors: cosine >= 0.9999, rel <= 1e-3
    q = I.ramp_sin(G.q_dim, 0.011, 0.6, 0.05)
    gate = I.ramp_cos(G.q_dim, 0.007, 1.2, -0.1)
    K = I.ramp_sin(kv_len * G.kv_dim, 0.013, 0.5, 0.02).reshape(kv_len, G.kv_dim)
    V = I.ramp_cos(kv_len * G.kv_dim, 0.017, 0.4, -0.05).reshape(kv_len, G.kv_dim)
    out = O.sdpa(kv_len, q, gate, K, V)
    qd = q.astype(np.float64).reshape(G.num_attn_heads, G.head_dim)
    Kd = K.astype(np.float64).reshape(kv_len, G.num_kv_heads, G.head_dim)
    Vd = V.astype(np.float64).reshape(kv_len, G.num_kv_heads, G.head_dim)
    ref = np.zeros_like(qd)
    for h in range(G.num_attn_heads):
        s = Kd[:, h // 16] @ qd[h] / 16.0
        w = np.exp(s - s.max())
        w /= w.sum()
        ref[h] = w @ Vd[:, h // 16]
    ref *= 1.0 / (1.0 + np.exp(-gate.astype(np.float64))).reshape(ref.shape)
    assert I.cosine(out, ref) >= 0.9999
    assert I.rel_err(out, ref) <= 1e-5


def test_three_kernel_split_equals_sdpa():
    # attn_scores -> softmax -> values -> sigmoid_gate == sdpa (shaders.metal:976-1134 vs sdpa.rs:63-172)
    n = 64
    q = I.synth_floats(n, G.q_dim, 0.4)
    K = I.synth_floats(n + 1, n * G.kv_dim, 0.3)
    V = I.synth_floats(n + 2, n * G.kv_dim, 0.5)
    gate = I.synth_floats(n + 3, G.q_dim, 1.0)
    s = O.attn_scores_batched(G.num_attn_heads, G.num_kv_heads, G.head_dim, n, q, K, 1 / 16.0)
    p = O.attn_softmax_batched(G.num_attn_heads, n, s)
    assert np.allclose(p.reshape(G.num_attn_heads, n).sum(1), 1.0, atol=1e-3)  # diff_oracle.rs floor
    o = O.attn_values_batched(G.num_attn_heads, G.num_kv_heads, G.head_dim, n, p, V)
    o = O.sigmoid_gate(gate, o)
    assert I.rel_err(o, O.sdpa(n, q, gate, K, V)) < 1e-6


def test_partial_merge_equals_unsplit():
    r = I.rng(3)
    n = 200
    q, gate, _, _ = I.gqa_step_inputs(r)
    K, V = I.normal(r, (n, G.kv_dim)), I.normal(r, (n, G.kv_dim))
    ref = O.sdpa(n, q, gate, K, V)
    cuts = [0, 0, 33, 64, 64, 150, 200]  # empty ranges included
    parts = [O.sdpa_partial(a, b, q, K, V) for a, b in zip(cuts[:-1], cuts[1:])]
    o = np.stack([p[0] for p in parts])
    m = np.stack([p[1] for p in parts])
    l = np.stack([p[2] for p in parts])
    assert np.isneginf(m[0]).all() and (l[0] == 0).all()
    got = O.lse_merge_gate(o, m, l, gate)
    assert I.rel_err(got, ref) < 1e-6


def test_silu_and_bare_norm_facts():
    # crates/moeflux/src/riir/linear_attn.rs:420-445
    assert np.allclose(O.rms_norm_bare(np.ones(16, np.float32)), 1.0, atol=1e-3)
    w1 = O.f32_to_bf16_bits(np.array([[0, 0, 0, 1.0]], np.float32))
    assert O.conv1d_step(np.zeros(3, np.float32), np.array([0.0], np.float32), w1, 1)[0] == 0.0
    y = O.conv1d_step(np.zeros(3, np.float32), np.array([10.0], np.float32), w1, 1)[0]
    assert abs(y - 10.0) < 1e-3


def test_conv_zero_history_is_silu_of_last_tap():
    r = I.rng(4)
    cw, _, _, _ = I.gdn_weights(r)
    x = I.normal(r, G.conv_dim)
    y = O.conv1d_step(np.zeros((3, G.conv_dim), np.float32), x, cw, G.conv_dim)
    a = x.astype(np.float64) * O.bf16_bits_to_f32(cw.reshape(G.conv_dim, 4)[:, 3]).astype(np.float64)
    assert np.max(np.abs(y - a / (1 + np.exp(-a)))) < 1e-6


def test_conv_matches_float64_on_reference_inputs():
    # inputs of conv1d_step_cpu_close_c_vs_rust (diff_oracle.rs:2092-2097); weights are seeded here
    cw, _, _, _ = I.gdn_weights(I.rng(5))
    st = I.ramp_sin(3 * G.conv_dim, 0.013, 0.4, 0.02).reshape(3, G.conv_dim)
    x = I.ramp_cos(G.conv_dim, 0.019, 0.5, -0.1)
    y = O.conv1d_step(st, x, cw, G.conv_dim)
    w = O.bf16_bits_to_f32(cw).reshape(G.conv_dim, 4).astype(np.float64)
    a = (st.astype(np.float64).T * w[:, :3]).sum(1) + x * w[:, 3]
    assert np.max(np.abs(y - a / (1 + np.exp(-a)))) < 1e-6
    st2 = O.conv_state_shift(st, x, G.conv_dim)
    assert np.array_equal(st2[0], st[1]) and np.array_equal(st2[1], st[2]) and np.array_equal(st2[2], x)


def test_qk_norm_is_l2_normalisation():
    r = I.rng(6)
    q, k = I.normal(r, G.total_key), I.normal(r, G.total_key)
    qn, kn = O.rms_norm_qk(q, k, G.linear_num_k_heads, 128)
    qn, kn = qn.reshape(-1, 128), kn.reshape(-1, 128)
    assert np.allclose(np.linalg.norm(kn, axis=1), 1.0, atol=1e-4)
    assert np.allclose(np.linalg.norm(qn, axis=1), 1 / np.sqrt(128), atol=1e-5)


def test_recurrence_zero_state_single_step_closed_form():
    # zero state + one step: S[vi,:] = beta*v[vi]*k, o[vi] = beta*v[vi]*(k.q); inputs of diff_oracle.rs:2245-2260
    vh, kh, d = G.linear_num_v_heads, G.linear_num_k_heads, 128
    alpha = I.ramp_sin(vh, 0.013, 0.3, 0.0)
    beta = I.ramp_cos(vh, 0.017, 0.5, 0.0)
    q = I.ramp_sin(kh * d, 0.011, 0.4, 0.05)
    k = I.ramp_cos(kh * d, 0.019, 0.5, -0.1)
    v = I.ramp_sin(vh * d, 0.023, 0.6, 0.02)
    _, a_log, dt, _ = I.gdn_weights(I.rng(7))
    S, o = O.gated_delta_recurrence(a_log, dt, alpha, beta, q, k, v, vh, kh, d, d, np.zeros(vh * d * d, np.float32))
    bg = 1 / (1 + np.exp(-beta.astype(np.float64)))
    S = S.reshape(vh, d, d)
    for h in (0, 5, 63):
        kk, qq = k.reshape(kh, d)[h // 4].astype(np.float64), q.reshape(kh, d)[h // 4].astype(np.float64)
        vv = v.reshape(vh, d)[h].astype(np.float64)
        assert np.max(np.abs(S[h] - bg[h] * np.outer(vv, kk))) < 1e-6
        assert np.max(np.abs(o.reshape(vh, d)[h] - bg[h] * vv * (kk @ qq))) < 1e-5


def test_recurrence_g1_beta0_leaves_state_unchanged():
    vh, kh, d = G.linear_num_v_heads, G.linear_num_k_heads, 128
    r = I.rng(8)
    S0 = I.normal(r, vh * d * d, 0.02)
    a_log = np.full(vh, -1e9, np.float32)  # exp(A_log) = 0 -> g = exp(0) = 1
    dt = O.f32_to_bf16_bits(np.zeros(vh, np.float32))
    beta = np.full(vh, -1e9, np.float32)   # sigmoid -> 0
    q, k, v = I.normal(r, kh * d), I.normal(r, kh * d), I.normal(r, vh * d)
    S, o = O.gated_delta_recurrence(a_log, dt, np.zeros(vh, np.float32), beta, q, k, v, vh, kh, d, d, S0)
    assert np.array_equal(S, S0)
    ref = S0.reshape(vh, d, d).astype(np.float64)  # read-out only
    for h in (0, 17):
        assert np.max(np.abs(o.reshape(vh, d)[h] - ref[h] @ q.reshape(kh, d)[h // 4])) < 1e-5


def test_decay_beta_formula():
    r = I.rng(9)
    _, a_log, dt, _ = I.gdn_weights(r)
    alpha, beta = I.normal(r, 64), I.normal(r, 64)
    g, b = O.decay_beta(alpha, beta, a_log, dt)
    x = alpha.astype(np.float64) + O.bf16_bits_to_f32(dt)
    ref = np.exp(-np.exp(a_log.astype(np.float64)) * np.log1p(np.exp(x)))
    assert np.max(np.abs(g - ref)) < 1e-6 and ((g > 0) & (g <= 1)).all()
    assert np.max(np.abs(b - 1 / (1 + np.exp(-beta.astype(np.float64))))) < 1e-6


def test_gated_norm_matches_float64():
    r = I.rng(10)
    _, _, _, nw = I.gdn_weights(r)
    x, z = I.normal(r, 128), I.normal(r, 128)
    y = O.rms_norm_gated(nw, x, z)
    xd, zd = x.astype(np.float64), z.astype(np.float64)
    ref = xd / np.sqrt((xd * xd).mean() + 1e-6) * O.bf16_bits_to_f32(nw) * (zd / (1 + np.exp(-zd)))
    assert np.max(np.abs(y - ref)) < 1e-5


def test_linear_step_composite_equals_pieces():
    r = I.rng(11)
    cw, a_log, dt, nw = I.gdn_weights(r)
    qkv, z, alpha, beta = I.gdn_step_inputs(r)
    conv = I.normal(r, (3, G.conv_dim))
    ssm = I.normal(r, G.ssm_elems, 0.02)
    conv2, ssm2 = conv.copy(), ssm.copy()
    out = O.linear_attn_step(qkv, z, alpha, beta, cw, a_log, dt, nw, conv2, ssm2)
    y = O.conv1d_step(conv, qkv, cw, G.conv_dim)
    qn, kn = O.rms_norm_qk(y[:2048], y[2048:4096], 16, 128)
    S, o = O.gated_delta_recurrence(a_log, dt, alpha, beta, qn, kn, y[4096:], 64, 16, 128, 128, ssm)
    ref = np.concatenate([O.rms_norm_gated(nw, o[h * 128:(h + 1) * 128], z[h * 128:(h + 1) * 128]) for h in range(64)])
    assert np.array_equal(out, ref) and np.array_equal(ssm2, S)
    assert np.array_equal(conv2, O.conv_state_shift(conv, qkv, G.conv_dim))


def test_split_q_gate_and_per_head_norm():
    r = I.rng(12)
    qp = I.normal(r, 2 * G.q_dim)
    q, gate = O.split_q_gate(qp)
    v = qp.reshape(G.num_attn_heads, 2, G.head_dim)
    assert np.array_equal(q, v[:, 0].reshape(-1)) and np.array_equal(gate, v[:, 1].reshape(-1))
    w = O.f32_to_bf16_bits(1.0 + I.normal(r, G.head_dim, 0.1))
    y = O.rms_norm_per_head(w, G.num_attn_heads, G.head_dim, q).reshape(G.num_attn_heads, -1)
    xd = q.reshape(G.num_attn_heads, -1).astype(np.float64)
    ref = xd / np.sqrt((xd * xd).mean(1, keepdims=True) + 1e-6) * O.bf16_bits_to_f32(w)
    assert np.max(np.abs(y - ref)) < 1e-5


# ---- 4-bit dequant matvec: the reference's own known answers (crates/moeflux/src/riir/cpu_matvec.rs:370-451) ----
def test_dequant_matvec_all_ones():
    # every nibble 1, scale 1.0 (bf16 0x3F80), bias 0: an all-ones row against x = ones gives 64
    out = O.dequant_matvec_4bit(np.full(8, 0x11111111, np.uint32), [0x3F80], [0x0000], 64, 1, np.ones(64, np.float32))
    assert out.tolist() == [64.0]


def test_dequant_matvec_zero_input_yields_zero_output():
    out = O.dequant_matvec_4bit(np.full(16, 0xFFFFFFFF, np.uint32), [0x3F80] * 2, [0x3F80] * 2, 64, 2,
                                np.zeros(64, np.float32))
    assert out.tolist() == [0.0, 0.0]


def test_dequant_matvec_bias_only_path():
    # nibble 0, scale 5.0 (0x40A0), bias 2.0 (0x4000): every weight is 2, the sum is 128
    out = O.dequant_matvec_4bit(np.zeros(8, np.uint32), [0x40A0], [0x4000], 64, 1, np.ones(64, np.float32))
    assert out.tolist() == [128.0]


def test_dequant_matvec_errors_like_the_reference():
    with pytest.raises(ValueError, match="packed"):  # SliceLen { field: "packed", got: 7, expected: 8 }
        O.dequant_matvec_4bit(np.zeros(7, np.uint32), [0x3F80], [0x0000], 64, 1, np.ones(64, np.float32))
    with pytest.raises(ValueError, match="multiple"):  # InDimNotMultiple
        O.dequant_matvec_4bit(np.zeros(12, np.uint32), [0x3F80], [0x0000], 96, 1, np.ones(96, np.float32))


def test_dequant_matvec_against_float64_restatement():
    r = I.rng(31)
    in_dim, out_dim = 256, 37
    packed, scales, biases = I.quant_weights(r, in_dim, out_dim)
    x = I.normal(r, in_dim)
    out = O.dequant_matvec_4bit(packed, scales, biases, in_dim, out_dim, x)
    nib = ((packed.reshape(out_dim, in_dim // 8, 1) >> (4 * np.arange(8, dtype=np.uint32))) & 0xF).reshape(out_dim, in_dim)
    s = np.repeat(O.bf16_bits_to_f32(scales).reshape(out_dim, -1), 64, axis=1).astype(np.float64)
    b = np.repeat(O.bf16_bits_to_f32(biases).reshape(out_dim, -1), 64, axis=1).astype(np.float64)
    ref = ((nib * s + b) * x.astype(np.float64)).sum(1)
    assert np.max(np.abs(out - ref)) <= 1e-5 * max(1.0, np.max(np.abs(ref)))
