"""GPU parity of the fused GatedDeltaNet decode step (conv1d+SiLU, q/k norm,
decay/beta, delta rule, gated RMSNorm) against the CPU oracle, through the C
ABI.  Test shapes follow crates/moeflux/tests/diff_oracle.rs:2079-2327 (conv1d,
gated norm, recurrence from a zero state) and :3249 (linear layer dump)."""
import numpy as np
import pytest

import moeflux_b200 as M
import oracle as O
from oracle import A17B as G
from oracle import Geometry
from tests import inputs as I
from tests.gpu_common import TOL_F32, make_pair

pytestmark = pytest.mark.gpu

LIN = [0, 1, 2]


@pytest.fixture(scope="module")
def pair():
    ctx, orc = make_pair(max_seq=64, n_seqs=2, linear_layers=LIN)
    yield ctx, orc
    ctx.close()


@pytest.mark.parametrize("with_z", [True, False])
def test_single_step_seeded_state(pair, with_z):
    """The single-step configuration: N(0,1) inputs, 3-row conv history, N(0,0.02) state."""
    ctx, orc = pair
    r = I.rng(100)
    qkv, z, alpha, beta = I.gdn_step_inputs(r)
    conv = I.normal(r, (3, G.conv_dim))
    ssm = I.normal(r, G.ssm_elems, 0.02)
    out, conv2, ssm2 = ctx.linear_attn_step_stateless(0, qkv, z if with_z else None, alpha, beta, conv, ssm)
    rconv, rssm = conv.copy(), ssm.copy()
    cw, al, dt, nw = orc.weights[0]
    ref = O.linear_attn_step(qkv, z if with_z else None, alpha, beta, cw, al, dt, nw, rconv, rssm)
    assert I.rel_err(out, ref) <= TOL_F32
    assert I.rel_err(ssm2, rssm) <= TOL_F32
    assert np.array_equal(conv2.reshape(3, -1), rconv)  # the history is moved, not computed: exact


def test_zero_state_closed_form(pair):
    ctx, orc = pair
    r = I.rng(101)
    qkv, _, alpha, beta = I.gdn_step_inputs(r)
    zero_conv = np.zeros((3, G.conv_dim), np.float32)
    out, _, ssm = ctx.linear_attn_step_stateless(1, qkv, None, alpha, beta, zero_conv, np.zeros(G.ssm_elems, np.float32))
    cw, al, dt, nw = orc.weights[1]
    a = qkv.astype(np.float64) * O.bf16_bits_to_f32(cw.reshape(-1, 4)[:, 3])
    y = a / (1 + np.exp(-a))  # conv with zero history = silu(x * w[:,3])
    q, k, v = y[:2048].reshape(16, 128), y[2048:4096].reshape(16, 128), y[4096:].reshape(64, 128)
    qn = q / np.sqrt((q * q).mean(1, keepdims=True) + 1e-6) / 128.0
    kn = k / np.sqrt((k * k).mean(1, keepdims=True) + 1e-6) / np.sqrt(128.0)
    bg = 1 / (1 + np.exp(-beta.astype(np.float64)))
    ref_o = np.stack([bg[h] * v[h] * (kn[h // 4] @ qn[h // 4]) for h in range(64)])
    ref_S = np.stack([bg[h] * np.outer(v[h], kn[h // 4]) for h in range(64)])
    assert I.rel_err(out, ref_o) <= TOL_F32
    assert I.rel_err(ssm, ref_S) <= TOL_F32


def test_reference_test_inputs_from_zero_state(pair):
    # gated_delta_recurrence_cpu_close_c_vs_rust inputs (diff_oracle.rs:2245-2260) fed through the conv
    ctx, orc = pair
    qkv = np.concatenate([I.ramp_sin(2048, 0.011, 0.4, 0.05), I.ramp_cos(2048, 0.019, 0.5, -0.1),
                          I.ramp_sin(8192, 0.023, 0.6, 0.02)])
    alpha = I.ramp_sin(64, 0.013, 0.3, 0.0)
    beta = I.ramp_cos(64, 0.017, 0.5, 0.0)
    z = I.ramp_cos(8192, 0.007, 1.2, -0.1)
    conv = I.ramp_sin(3 * G.conv_dim, 0.013, 0.4, 0.02).reshape(3, -1)
    out, conv2, ssm2 = ctx.linear_attn_step_stateless(2, qkv, z, alpha, beta, conv, np.zeros(G.ssm_elems, np.float32))
    rconv, rssm = conv.copy(), np.zeros(G.ssm_elems, np.float32)
    ref = O.linear_attn_step(qkv, z, alpha, beta, *orc.weights[2], rconv, rssm)
    assert I.rel_err(out, ref) <= TOL_F32 and I.rel_err(ssm2, rssm) <= TOL_F32


@pytest.mark.parametrize("rows", [32, 64, 128])
def test_multi_step_batched_sequences(pair, rows):
    """Ten chained steps on 3 layers x 2 sequences in one launch per step: the
    conv ring wraps twice, states stay separate, every block size agrees."""
    ctx, orc = pair
    ctx.set_tuning("gdn_rows", rows)
    ctx.memory_clear(-1)
    orc.memory_clear(-1)
    r = I.rng(102)
    items = [(l, s) for l in LIN for s in range(2)]
    for step in range(10):
        ins = [I.gdn_step_inputs(r) for _ in items]
        use_z = step % 2 == 0
        got = ctx.linear_attn_step_batched([l for l, _ in items], [s for _, s in items],
                                           np.stack([i[0] for i in ins]),
                                           np.stack([i[1] for i in ins]) if use_z else None,
                                           np.stack([i[2] for i in ins]), np.stack([i[3] for i in ins]))
        for j, (l, s) in enumerate(items):
            ref = orc.linear_attn_step(l, s, ins[j][0], ins[j][1] if use_z else None, ins[j][2], ins[j][3])
            assert I.rel_err(got[j], ref) <= TOL_F32, (step, l, s)
    ctx.set_tuning("gdn_rows", 0)


def test_argument_errors(pair):
    ctx, _ = pair
    x = np.zeros(ctx.conv_dim, np.float32)
    h = np.zeros(64, np.float32)
    with pytest.raises(M.MfcError, match="not a linear-attention layer"):
        ctx.linear_attn_step(3, 0, x, None, h, h)
    with pytest.raises(M.MfcError, match="mfc_set_linear_weights"):
        ctx.linear_attn_step(4, 0, x, None, h, h)  # weights never set for layer 4
    with pytest.raises(M.MfcError):
        ctx.linear_attn_step(0, 2, x, None, h, h)  # seq_id out of range


def test_a3b_head_geometry():
    """Qwen3.6-35B-A3B heads (crates/moeflux/src/riir/variants.rs:426-440):
    16 query heads (group of 8 per kv head), 32 v-heads (2 per k-head)."""
    g = Geometry(num_layers=8, num_attn_heads=16, linear_num_v_heads=32)
    ctx, orc = make_pair(g, max_seq=128, linear_layers=[0, 1])
    r = I.rng(103)
    for step in range(5):
        qkv, z, alpha, beta = I.gdn_step_inputs(r, g)
        got = ctx.linear_attn_step(1, 0, qkv, z, alpha, beta)
        assert I.rel_err(got, orc.linear_attn_step(1, 0, qkv, z, alpha, beta)) <= TOL_F32
    for pos in range(40):
        ins = I.gqa_step_inputs(r, g)
        got = ctx.full_attn_step(3, 0, pos, *ins)
        assert I.rel_err(got, orc.full_attn_step(3, 0, pos, *ins)) <= TOL_F32
    ctx.close()


def test_side_queue_step_then_snapshot_without_join():
    """With the tuning "gdn_side_queue" the step's kernel runs on the context's second queue; a snapshot taken right
    after it, with no explicit mfc_join, still sees the finished step (every call that reads or writes the
    GatedDeltaNet state joins first)."""
    import torch

    from oracle import snapshot as snap

    dev = torch.device("cuda:0")
    ctx, orc = make_pair(max_seq=64, n_seqs=2, linear_layers=[0, 1, 2])
    ctx.set_tuning("gdn_side_queue", 1)
    r = I.rng(140)
    items = [(0, 0), (1, 0), (2, 1)]
    for step in range(5):
        ins = [I.gdn_step_inputs(r) for _ in items]
        d = [torch.tensor(np.stack([i[k] for i in ins]), device=dev) for k in range(4)]
        out = torch.empty(len(items), G.total_value, device=dev)
        torch.cuda.synchronize()
        ctx.linear_attn_step_batched_dev([l for l, _ in items], [s for _, s in items], d[0].data_ptr(), d[1].data_ptr(),
                                         d[2].data_ptr(), d[3].data_ptr(), out.data_ptr())
        blob = ctx.state_save(0)  # no join in between
        for j, (l, s) in enumerate(items):
            orc.linear_attn_step(l, s, *ins[j])
        a, b = snap.state_load(G, blob), snap.state_load(G, orc.state_save(0))
        for layer in (0, 1):
            assert np.array_equal(a[layer][1], b[layer][1]), step       # conv history
            assert I.rel_err(a[layer][2], b[layer][2]) <= TOL_F32, step  # ssm state
    # truncation resets the states: it must not race the step either
    ins = [I.gdn_step_inputs(r) for _ in items]
    d = [torch.tensor(np.stack([i[k] for i in ins]), device=dev) for k in range(4)]
    torch.cuda.synchronize()
    ctx.linear_attn_step_batched_dev([l for l, _ in items], [s for _, s in items], d[0].data_ptr(), d[1].data_ptr(),
                                     d[2].data_ptr(), d[3].data_ptr(), out.data_ptr())
    assert ctx.memory_seq_rm(0, 0, -1)
    z = snap.state_load(G, ctx.state_save(0))
    assert not z[0][2].any() and not z[1][1].any()
    ctx.close()
