"""GPU parity of the full-attention path (RoPE, append, split-K SDPA, sigmoid
gate) against the CPU oracle, through the C ABI.  Probe points follow the
reference's tests: kv_len {1, 8, 32, 33, 64, 128, 512}, pos {0, 1, 17, 1024,
65535} (crates/moeflux/tests/diff_oracle.rs:1379-1442, 1541-1615, 2712-2955,
3505-3654)."""
import numpy as np
import pytest

import moeflux_b200 as M
import oracle as O
from oracle import A17B as G
from tests import inputs as I
from tests.gpu_common import TOL_BF16, TOL_F32, make_pair

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def f32_pair():
    ctx, orc = make_pair(max_seq=1024, n_seqs=2, linear_layers=[])
    yield ctx, orc
    ctx.close()


@pytest.fixture(scope="module")
def bf16_pair():
    ctx, orc = make_pair(max_seq=4096, n_seqs=2, kv_bf16=True, linear_layers=[])
    yield ctx, orc
    ctx.close()


@pytest.mark.parametrize("pos", [0, 1, 17, 1024, 65535])
def test_rope_hook(f32_pair, pos):
    ctx, _ = f32_pair
    q = I.ramp_sin(G.q_dim, 0.013, 0.7, 0.1)
    k = I.ramp_cos(G.kv_dim, 0.019, 0.5, -0.2)
    gq, gk = ctx.apply_rotary_emb(pos, q, k)
    rq, rk = O.apply_rotary_emb(pos, q, k)
    if pos == 0:
        assert np.array_equal(gq, q) and np.array_equal(gk, k)
    # the reference's own bound is 128 ULP; near 1.0 that is 1.5e-5
    assert np.max(np.abs(gq - rq)) <= 2e-6 and np.max(np.abs(gk - rk)) <= 2e-6


def test_rope_hook_rejects_negative_pos(f32_pair):
    ctx, _ = f32_pair
    with pytest.raises(M.MfcError):
        ctx.apply_rotary_emb(-1, np.zeros(G.q_dim, np.float32), np.zeros(G.kv_dim, np.float32))


@pytest.mark.parametrize("kv_len", [1, 8, 32, 33, 64, 128, 512])
def test_sdpa_hook_fp32_reference_inputs(f32_pair, kv_len):
    ctx, _ = f32_pair
    q = I.ramp_sin(G.q_dim, 0.011, 0.6, 0.05)
    gate = I.ramp_cos(G.q_dim, 0.007, 1.2, -0.1)
    K = I.ramp_sin(kv_len * G.kv_dim, 0.013, 0.5, 0.02)
    V = I.ramp_cos(kv_len * G.kv_dim, 0.017, 0.4, -0.05)
    got = ctx.sdpa(kv_len, q, gate, K, V)
    ref = O.sdpa(kv_len, q, gate, K, V)
    assert np.isfinite(got).all()
    assert I.cosine(got, ref) >= 0.9999
    assert I.rel_err(got, ref) <= TOL_F32


def test_sdpa_hook_known_answers(f32_pair):
    ctx, _ = f32_pair
    r = I.rng(21)
    q, gate, k, v = I.gqa_step_inputs(r)
    got = ctx.sdpa(1, q, gate, k, v).reshape(G.num_attn_heads, -1)
    sig = 1 / (1 + np.exp(-gate.astype(np.float64))).reshape(G.num_attn_heads, -1)
    ref = np.repeat(v.reshape(G.num_kv_heads, -1), 16, axis=0) * sig
    assert I.rel_err(got, ref) <= 1e-5
    n = 100
    K = np.tile(k, (n, 1))
    V = I.normal(r, (n, G.kv_dim))
    got = ctx.sdpa(n, q, gate, K, V).reshape(G.num_attn_heads, -1)
    ref = np.repeat(V.astype(np.float64).mean(0).reshape(G.num_kv_heads, -1), 16, axis=0) * sig
    assert I.rel_err(got, ref) <= 1e-4
    with pytest.raises(M.MfcError):
        ctx.sdpa(0, q, gate, k, v)


@pytest.mark.parametrize("kv_len", [1, 33, 512, 1000])
def test_sdpa_hook_fp32_seeded_normal(f32_pair, kv_len):
    ctx, _ = f32_pair
    r = I.rng(30 + kv_len)
    q, gate, _, _ = I.gqa_step_inputs(r)
    K, V = I.normal(r, (kv_len, G.kv_dim)), I.normal(r, (kv_len, G.kv_dim))
    assert I.rel_err(ctx.sdpa(kv_len, q, gate, K, V), O.sdpa(kv_len, q, gate, K, V)) <= TOL_F32


@pytest.mark.parametrize("kv_len", [1, 31, 33, 512, 3000])
def test_sdpa_hook_bf16_cache(bf16_pair, kv_len):
    ctx, _ = bf16_pair
    r = I.rng(40 + kv_len)
    q, gate, _, _ = I.gqa_step_inputs(r)
    K, V = I.normal(r, (kv_len, G.kv_dim)), I.normal(r, (kv_len, G.kv_dim))
    ref = O.sdpa(kv_len, q, gate, O.round_bf16(K), O.round_bf16(V))
    got = ctx.sdpa(kv_len, q, gate, K, V)
    assert np.isfinite(got).all()
    assert I.rel_err(got, ref) <= TOL_BF16


@pytest.mark.parametrize("bf16", [False, True])
def test_split_k_merge_equals_unsplit(f32_pair, bf16_pair, bf16):
    ctx, _ = bf16_pair if bf16 else f32_pair
    r = I.rng(50)
    n = 1000
    q, gate, _, _ = I.gqa_step_inputs(r)
    K, V = I.normal(r, (n, G.kv_dim)), I.normal(r, (n, G.kv_dim))
    ctx.set_tuning("gqa_chunk", 1024)
    one = ctx.sdpa(n, q, gate, K, V)
    outs = []
    for chunk in (32, 96, 512):
        ctx.set_tuning("gqa_chunk", chunk)
        outs.append(ctx.sdpa(n, q, gate, K, V))
    ctx.set_tuning("gqa_chunk", 0)
    for o in outs:
        # the split reorders fp32 sums and moves the rounding points of P (bf16, or the tf32 hi/lo split)
        assert I.rel_err(o, one) <= (2e-3 if bf16 else 2e-5)


@pytest.mark.parametrize("bf16", [False, True])
def test_decode_steps_from_empty_cache(f32_pair, bf16_pair, bf16):
    ctx, orc = bf16_pair if bf16 else f32_pair
    ctx.memory_clear(-1)
    orc.memory_clear(-1)
    r = I.rng(60)
    tol = TOL_BF16 if bf16 else TOL_F32
    for pos in range(70):  # crosses the 32/64-row tile boundaries
        for layer, seq in ((3, 0), (59, 1)):
            q, gate, k, v = I.gqa_step_inputs(r)
            got = ctx.full_attn_step(layer, seq, pos, q, gate, k, v)
            ref = orc.full_attn_step(layer, seq, pos, q, gate, k, v)
            assert I.rel_err(got, ref) <= tol, (pos, layer)
    assert ctx.memory_seq_pos_max(0) == orc.memory_seq_pos_max(0) == 70
    assert ctx.memory_seq_pos_max(1) == 70


def test_step_argument_errors(f32_pair):
    ctx, _ = f32_pair
    ctx.memory_clear(-1)
    z = np.zeros(G.q_dim, np.float32)
    kz = np.zeros(G.kv_dim, np.float32)
    with pytest.raises(M.MfcError, match="not a full-attention layer"):
        ctx.full_attn_step(0, 0, 0, z, z, kz, kz)
    with pytest.raises(M.MfcError, match="current length"):
        ctx.full_attn_step(3, 0, 5, z, z, kz, kz)  # pos must equal the length (full_attn_forward.rs:73-78)
    with pytest.raises(M.MfcError):
        ctx.full_attn_step(3, 7, 0, z, z, kz, kz)  # seq_id out of range
    with pytest.raises(M.MfcError):
        ctx.linear_attn_step(3, 0, np.zeros(ctx.conv_dim, np.float32), None, np.zeros(64, np.float32),
                             np.zeros(64, np.float32))  # full layer given to the linear step
    assert ctx.memory_seq_pos_max(0) == 0  # failed calls changed nothing


def test_caller_owned_stream(f32_pair):
    """mfc_set_stream: the context works on a stream the caller owns (here torch's)."""
    import torch

    ctx, orc = make_pair(max_seq=128, linear_layers=[])
    s = torch.cuda.Stream()
    ctx.set_stream(s.cuda_stream)
    assert ctx.stream == s.cuda_stream
    r = I.rng(62)
    for pos in range(3):
        ins = I.gqa_step_inputs(r)
        assert I.rel_err(ctx.full_attn_step(3, 0, pos, *ins), orc.full_attn_step(3, 0, pos, *ins)) <= TOL_F32
    ctx.close()
    s.synchronize()  # still alive after the context is gone


def test_cache_overflow_is_an_error():
    ctx, _ = make_pair(max_seq=33, linear_layers=[])
    r = I.rng(61)
    for pos in range(33):
        ctx.full_attn_step(3, 0, pos, *I.gqa_step_inputs(r))
    with pytest.raises(M.MfcError, match="overflow"):
        ctx.full_attn_step(3, 0, 33, *I.gqa_step_inputs(r))
    ctx.close()


def test_ragged_batched_decode_bf16():
    """Batched step over sequences of unequal length (the shape of the ragged
    64-sequence configuration, scaled down), contexts installed through
    state_load, several chunks per sequence."""
    n_seqs = 6
    ctx, orc = make_pair(max_seq=2048, n_seqs=n_seqs, kv_bf16=True, linear_layers=[])
    r = I.rng(70)
    lens = [1, 31, 257, 1024, 1500, 2046]
    layers = [3, 7]
    for s, ln in enumerate(lens):
        for layer in layers:
            orc.load_kv(layer, s, I.normal(r, (ln, G.kv_dim)), I.normal(r, (ln, G.kv_dim)))
        ctx.state_load(s, orc.state_save(s))
    ctx.set_tuning("gqa_target_ctas", 64)  # forces several chunks for the long sequences
    items = [(l, s) for s in range(n_seqs) for l in layers]
    for step in range(2):
        ins = [I.gqa_step_inputs(r) for _ in items]
        pos = [orc.len[(l, s)] for l, s in items]
        got = ctx.full_attn_step_batched([l for l, _ in items], [s for _, s in items], pos,
                                         np.stack([i[0] for i in ins]), np.stack([i[1] for i in ins]),
                                         np.stack([i[2] for i in ins]), np.stack([i[3] for i in ins]))
        for j, (l, s) in enumerate(items):
            ref = orc.full_attn_step(l, s, pos[j], *ins[j])
            assert I.rel_err(got[j], ref) <= TOL_BF16, (step, l, s)
    ctx.close()


def test_kv_split_partials_merge_to_the_whole():
    """Two contexts hold the block-cyclic halves of every sequence; their
    partials merged by log-sum-exp equal the single-context result."""
    import torch

    dev = torch.device("cuda:0")
    kw = dict(max_seq=512, n_seqs=2, linear_layers=[])
    whole, orc = make_pair(**kw)
    parts = [make_pair(kv_rank=rk, kv_world=2, kv_block=32, **kw)[0] for rk in range(2)]
    packed_parts = [make_pair(kv_rank=rk, kv_world=2, kv_block=32, **kw)[0] for rk in range(2)]
    r = I.rng(80)
    items = [(3, 0), (3, 1), (11, 1)]
    layers, seqs = [i[0] for i in items], [i[1] for i in items]
    n = len(items)
    H, D = G.num_attn_heads, G.head_dim
    for pos in range(100):
        ins = [I.gqa_step_inputs(r) for _ in items]
        q = torch.tensor(np.stack([i[0] for i in ins]), device=dev)
        gate = torch.tensor(np.stack([i[1] for i in ins]), device=dev)
        k = torch.tensor(np.stack([i[2] for i in ins]), device=dev)
        v = torch.tensor(np.stack([i[3] for i in ins]), device=dev)
        o = torch.empty(2, n, H, D, device=dev)
        m = torch.empty(2, n, H, device=dev)
        l = torch.empty(2, n, H, device=dev)
        torch.cuda.synchronize()
        for rk, c in enumerate(parts):
            c.full_attn_partial_batched_dev(layers, seqs, [pos] * n, q.data_ptr(), k.data_ptr(), v.data_ptr(),
                                            o[rk].data_ptr(), m[rk].data_ptr(), l[rk].data_ptr())
            c.synchronize()
        out = torch.empty(n, H * D, device=dev)
        parts[0].lse_merge_gate_dev(2, n, o.data_ptr(), m.data_ptr(), l.data_ptr(), gate.data_ptr(), out.data_ptr())
        parts[0].synchronize()
        out = out.cpu().numpy()
        refs = [orc.full_attn_step(layer, seq, pos, *ins[j]) for j, (layer, seq) in enumerate(items)]
        for j in range(n):
            assert I.rel_err(out[j], refs[j]) <= TOL_F32, (pos, j)
        # packed form on a second pair of contexts: one [o | m | l] block per item, the
        # layout an all-to-all by destination delivers
        item = H * D + 2 * H
        packed = torch.empty(2, n, item, device=dev)
        for rk, c in enumerate(packed_parts):
            c.full_attn_partial_packed_dev(layers, seqs, [pos] * n, q.data_ptr(), k.data_ptr(), v.data_ptr(),
                                           packed[rk].data_ptr())
            c.synchronize()
        out2 = torch.empty(n, H * D, device=dev)
        packed_parts[0].lse_merge_gate_packed_dev(2, n, packed.data_ptr(), gate.data_ptr(), out2.data_ptr())
        packed_parts[0].synchronize()
        out2 = out2.cpu().numpy()
        for j in range(n):
            assert I.rel_err(out2[j], refs[j]) <= TOL_F32, ("packed", pos, j)
        if pos < 40:  # early steps: rank 1 owns no row yet -> empty partial (m = -inf, l = 0)
            if pos < 32:
                assert torch.isinf(m[1]).all() and (l[1] == 0).all()
    for c in parts + packed_parts + [whole]:
        c.close()


@pytest.mark.parametrize("bf16", [False, True])
def test_step_from_projection_outputs(bf16):
    """q|gate de-interleave and per-head q/k RMSNorm fused into the kernel
    (crates/moeflux/src/riir/full_attn_forward.rs:238-276), then the usual step."""
    ctx, orc = make_pair(max_seq=128, n_seqs=2, kv_bf16=bf16, linear_layers=[])
    r = I.rng(90)
    qw = O.f32_to_bf16_bits(1.0 + I.normal(r, G.head_dim, 0.1))
    kw = O.f32_to_bf16_bits(1.0 + I.normal(r, G.head_dim, 0.1))
    with pytest.raises(M.MfcError, match="mfc_set_full_attn_norm_weights"):
        ctx.full_attn_step_qproj_batched([3], [0], [0], np.zeros(2 * G.q_dim, np.float32), np.zeros(G.kv_dim, np.float32),
                                         np.zeros(G.kv_dim, np.float32))
    for layer in (3, 7):
        ctx.set_full_attn_norm_weights(layer, qw, kw)
    items = [(3, 0), (3, 1), (7, 1)]
    tol = TOL_BF16 if bf16 else TOL_F32
    for pos in range(40):
        qp = [I.normal(r, 2 * G.q_dim) * 3.0 for _ in items]   # un-normalised projection outputs
        k = [I.normal(r, G.kv_dim) * 2.0 for _ in items]
        v = [I.normal(r, G.kv_dim) for _ in items]
        got = ctx.full_attn_step_qproj_batched([l for l, _ in items], [s for _, s in items], [pos] * 3, np.stack(qp),
                                               np.stack(k), np.stack(v))
        for j, (l, s) in enumerate(items):
            q, gate = O.split_q_gate(qp[j])
            qn = O.rms_norm_per_head(qw, G.num_attn_heads, G.head_dim, q)
            kn = O.rms_norm_per_head(kw, G.num_kv_heads, G.head_dim, k[j])
            ref = orc.full_attn_step(l, s, pos, qn, gate, kn, v[j])
            assert I.rel_err(got[j], ref) <= tol, (pos, j)
    ctx.close()


@pytest.mark.parametrize("bf16", [False, True])
def test_kv_split_fused_exchange_on_one_gpu(bf16):
    """The exchange fused into the decode kernel: two contexts hold the block-cyclic halves of every sequence, each
    stores the partial blocks of an item straight into the receive buffer of the context that finishes it and
    publishes its step number; the finishing context's merge checks the step numbers, merges and gates.  Both
    contexts live on one GPU here, so the two decode launches of a step are complete before the merges are issued
    (kernels that wait on one another must not share a GPU); the receive buffers alternate by step parity."""
    import torch

    dev = torch.device("cuda:0")
    kw = dict(max_seq=512, n_seqs=2, kv_bf16=bf16, linear_layers=[])
    _, orc = make_pair(**kw)
    parts = [make_pair(kv_rank=rk, kv_world=2, kv_block=32, **kw)[0] for rk in range(2)]
    npr = 2
    for c in parts:
        c.exchange_create(npr)
    for c in parts:
        c.exchange_connect_local(parts)
    r = I.rng(81)
    items = [(3, 0), (7, 0), (3, 1), (7, 1)]  # sorted by finishing rank: sequence 0 on rank 0, sequence 1 on rank 1
    layers, seqs = [i[0] for i in items], [i[1] for i in items]
    n = len(items)
    tol = TOL_BF16 if bf16 else TOL_F32
    for pos in range(70):
        ins = [I.gqa_step_inputs(r) for _ in items]
        q = torch.tensor(np.stack([i[0] for i in ins]), device=dev)
        gate = torch.tensor(np.stack([i[1] for i in ins]), device=dev)
        k = torch.tensor(np.stack([i[2] for i in ins]), device=dev)
        v = torch.tensor(np.stack([i[3] for i in ins]), device=dev)
        torch.cuda.synchronize()
        for c in parts:
            c.full_attn_partial_exchange_dev(layers, seqs, [pos] * n, q.data_ptr(), k.data_ptr(), v.data_ptr())
        for c in parts:
            c.synchronize()
        outs = []
        for rk, c in enumerate(parts):
            out = torch.empty(npr, G.q_dim, device=dev)
            c.lse_merge_gate_exchange_dev(gate[rk * npr:(rk + 1) * npr].data_ptr(), out.data_ptr())
            c.synchronize()
            outs.append(out.cpu().numpy())
        got = np.concatenate(outs)
        for j, (layer, seq) in enumerate(items):
            ref = orc.full_attn_step(layer, seq, pos, *ins[j])
            assert I.rel_err(got[j], ref) <= tol, (pos, j)
    # a merge whose peers never published the step: the bounded wait runs out and the call reports it
    parts[0].set_tuning("gqa_wait_spins", 200)
    parts[0].full_attn_partial_exchange_dev(layers, seqs, [70] * n, q.data_ptr(), k.data_ptr(), v.data_ptr())
    out = torch.empty(npr, G.q_dim, device=dev)
    parts[0].lse_merge_gate_exchange_dev(gate.data_ptr(), out.data_ptr())
    with pytest.raises(M.MfcError, match="peer's partials did not arrive"):
        parts[0].synchronize()
    with pytest.raises(M.MfcError, match="exchange"):
        parts[0].exchange_create(npr)  # already created
    # the gather of the query rows over the links waits for the peers' kernels: with a peer on the same GPU the
    # host-pointer step refuses it before anything is queued
    parts[1].set_tuning("exchange_gather_q", 1)
    zq, zk = np.zeros((npr, G.q_dim), np.float32), np.zeros((n, G.kv_dim), np.float32)
    with pytest.raises(M.MfcError, match="GPU of its own"):
        parts[1].eval_token_attn_split(items, [0] * n, zq, zq, zk, zk, [], None, None, None, None, npr, q_own=True)
    parts[1].set_tuning("exchange_gather_q", 0)
    for c in parts:
        c.check_guards()
        c.close()
