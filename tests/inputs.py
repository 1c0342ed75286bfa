"""Seeded and closed-form test inputs.

The closed-form ramps are the input formulas of the reference's differential
tests (crates/moeflux/tests/diff_oracle.rs: RoPE :1390-1395, SDPA :1555-1571,
conv1d :2092-2097, recurrence :2245-2260, synth_floats :2698-2705); the seeded
generators follow the value distributions the benchmark configurations state.
"""
import numpy as np

from oracle import A17B, Geometry, f32_to_bf16_bits


def ramp_sin(n, step, scale, offset):
    i = np.arange(n, dtype=np.float32)
    return (np.sin(i * np.float32(step)) * np.float32(scale) + np.float32(offset)).astype(np.float32)


def ramp_cos(n, step, scale, offset):
    i = np.arange(n, dtype=np.float32)
    return (np.cos(i * np.float32(step)) * np.float32(scale) + np.float32(offset)).astype(np.float32)


def synth_floats(seed, n, scale):
    i = np.arange(n, dtype=np.float32)
    phase = np.float32(seed) * np.float32(0.13) + i * np.float32(0.017)
    return (np.sin(phase) * np.float32(scale) + np.cos(phase * np.float32(1.7)) * np.float32(scale * 0.5)).astype(
        np.float32)


def rng(seed):
    return np.random.Generator(np.random.Philox(seed))


def normal(r, shape, std=1.0):
    return (r.standard_normal(shape, dtype=np.float32) * np.float32(std)).astype(np.float32)


def quant_weights(r, in_dim: int, out_dim: int):
    """A 4-bit group-64 affine-quantised matrix as the reference's converter lays it out: packed words of eight
    random nibbles, per-group scale ~ |N(0, 0.02)| + 1e-3 and bias = -8 * scale + N(0, 0.01), both bf16."""
    packed = r.integers(0, 1 << 32, size=out_dim * in_dim // 8, dtype=np.uint64).astype(np.uint32)
    sc = np.abs(normal(r, out_dim * in_dim // 64, 0.02)) + np.float32(1e-3)
    bi = -8.0 * sc + normal(r, out_dim * in_dim // 64, 0.01)
    return packed, f32_to_bf16_bits(sc), f32_to_bf16_bits(bi)


def gdn_weights(r, g: Geometry = A17B):
    """conv_w ~ N(0, 0.5) bf16, A_log ~ U(0, 2.7), dt_bias ~ N(0,1) bf16, norm_w ~ 1 + N(0, 0.1) bf16."""
    conv_w = f32_to_bf16_bits(normal(r, (g.conv_dim, g.conv_kernel_size), 0.5))
    a_log = r.uniform(0.0, 2.7, g.linear_num_v_heads).astype(np.float32)
    dt_bias = f32_to_bf16_bits(normal(r, g.linear_num_v_heads))
    norm_w = f32_to_bf16_bits(1.0 + normal(r, g.linear_value_dim, 0.1))
    return conv_w, a_log, dt_bias, norm_w


def gdn_step_inputs(r, g: Geometry = A17B):
    qkv = normal(r, g.conv_dim)
    z = normal(r, g.total_value)
    alpha = normal(r, g.linear_num_v_heads)
    beta = normal(r, g.linear_num_v_heads)
    return qkv, z, alpha, beta


def gqa_step_inputs(r, g: Geometry = A17B):
    return normal(r, g.q_dim), normal(r, g.q_dim), normal(r, g.kv_dim), normal(r, g.kv_dim)


def rel_err(got, ref):
    """max|got-ref| / max|ref|: the reference's own relative-error convention
    (crates/moeflux/tests/diff_oracle.rs:1609-1613)."""
    got = np.asarray(got, np.float64).reshape(-1)
    ref = np.asarray(ref, np.float64).reshape(-1)
    return float(np.max(np.abs(got - ref)) / max(np.max(np.abs(ref)), 1e-30))


def cosine(a, b):
    a = np.asarray(a, np.float64).reshape(-1)
    b = np.asarray(b, np.float64).reshape(-1)
    return float(np.dot(a, b) / max(np.linalg.norm(a) * np.linalg.norm(b), 1e-30))
