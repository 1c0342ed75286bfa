"""GPU parity of the full-attention decode step at the contexts the benchmark and the
configurations quote: the reference hands everything outside 32 <= kv_len < 8192 to its
CPU SDPA (crates/moeflux/src/riir/full_attn_forward.rs:331-334, 357-389); here every
length runs on the GPU, so every length is compared with the CPU oracle.  Also the code
that only large launches reach: units cut by run boundaries into many partials (one- and
two-level merges), and launches of more than 512 items (the work lookup in device memory).
"""
import numpy as np
import pytest

import moeflux_b200 as M
import oracle as O
from oracle import Geometry
from tests import inputs as I
from tests.gpu_common import TOL_BF16, TOL_F32, make_pair

pytestmark = pytest.mark.gpu

G4 = Geometry(num_layers=4)  # three GatedDeltaNet layers and one full-attention layer (index 3), full-size heads
FULL = 3


def install_kv(ctx, orc, layer, seq, K, V):
    """Same cache rows on both sides: the oracle's host arrays and, through the bulk import, the GPU context."""
    import torch

    orc.load_kv(layer, seq, K, V)
    n = K.shape[0]
    for p0 in range(0, n, 16384):
        k = torch.tensor(K[p0:p0 + 16384], device="cuda:0")
        v = torch.tensor(V[p0:p0 + 16384], device="cuda:0")
        ctx.kv_append_rows_dev(layer, seq, p0, k.shape[0], k.data_ptr(), v.data_ptr())
        ctx.synchronize()


def one_step(ctx, orc, seq, ctx_len, r, tol):
    """The step that appends row ctx_len - 1 and attends over ctx_len rows."""
    q, gate, k, v = I.gqa_step_inputs(r, G4)
    got = ctx.full_attn_step(FULL, seq, ctx_len - 1, q, gate, k, v)
    ref = orc.full_attn_step(FULL, seq, ctx_len - 1, q, gate, k, v)
    assert np.isfinite(got).all()
    err = I.rel_err(got, ref)
    assert err <= tol, err
    return err


def test_config0_fp32_ctx4096_single_step():
    """Configuration 0 as stated: batch 1, 32 query / 2 kv heads of 256, context 4096, fp32 q/K/V ~ N(0,1) from seed
    0, RoPE on the first 64 dims (theta 1e7), gate logits N(0,1), scale 1/16.  (The cached rows are drawn N(0,1)
    directly: a rotation does not change their distribution.)"""
    ctx, orc = make_pair(G4, max_seq=4096, linear_layers=[])
    r = I.rng(0)
    install_kv(ctx, orc, FULL, 0, I.normal(r, (4095, G4.kv_dim)), I.normal(r, (4095, G4.kv_dim)))
    one_step(ctx, orc, 0, 4096, r, TOL_F32)
    ctx.check_guards()
    ctx.close()


@pytest.mark.parametrize("coop", [1, 0])
@pytest.mark.parametrize("bf16", [False, True])
def test_ctx32768_single_step(bf16, coop):
    """The target shape: one sequence at context 32768.  A lone sequence is cut into well over a hundred partials per
    kv head: merged by the CTAs that share the unit together in a cooperative launch (coop=1), or in two levels of
    last-arriver merges in an ordinary one (coop=0)."""
    ctx, orc = make_pair(G4, max_seq=32768 + 4, kv_bf16=bf16, linear_layers=[])
    ctx.set_tuning("gqa_coop_merge", coop)
    r = I.rng(32768 + bf16)
    install_kv(ctx, orc, FULL, 0, I.normal(r, (32767, G4.kv_dim)), I.normal(r, (32767, G4.kv_dim)))
    for step in range(3):  # three launches in a row: the merge counters of one are back at zero for the next
        one_step(ctx, orc, 0, 32768 + step, r, TOL_BF16 if bf16 else TOL_F32)
    ctx.check_guards()
    ctx.close()


def test_fp32_long_run_per_cta_keeps_fp32_accuracy():
    """A CTA that streams 16384 rows by itself (the benchmark's launches of 120 items give every CTA runs of this
    length; here one sequence with the least run length raised to 16384 rows).  An output accumulator that lives in
    the tensor core is truncated after each of its 3072 instructions and ends 1e-4 below the true sum; the kernel
    joins each tile's products to the running output with a rounded fused multiply-add instead.  Checked against a
    float64 evaluation of the definition: 2e-5, five times inside the fp32 contract."""
    ctx, _ = make_pair(G4, max_seq=32768, linear_layers=[])
    ctx.set_tuning("gqa_min_rows", 16384)
    r = I.rng(777)
    n = 32768
    q, gate, _, _ = I.gqa_step_inputs(r, G4)
    K, V = I.normal(r, (n, G4.kv_dim)), I.normal(r, (n, G4.kv_dim))
    got = ctx.sdpa(n, q, gate, K, V)
    H, Hkv, D = G4.num_attn_heads, G4.num_kv_heads, G4.head_dim
    ref = np.empty(H * D)
    for h in range(H):
        kv = h // (H // Hkv)
        s = K[:, kv * D:(kv + 1) * D].astype(np.float64) @ q[h * D:(h + 1) * D].astype(np.float64) / np.sqrt(D)
        p = np.exp(s - s.max())
        o = (p / p.sum()) @ V[:, kv * D:(kv + 1) * D].astype(np.float64)
        ref[h * D:(h + 1) * D] = o / (1.0 + np.exp(-gate[h * D:(h + 1) * D].astype(np.float64)))
    err = float(np.max(np.abs(got - ref)) / np.max(np.abs(ref)))
    assert err <= 2e-5, err
    assert I.rel_err(got, O.sdpa(n, q, gate, K, V)) <= TOL_F32
    ctx.close()


def test_ctx131072_bf16_single_step():
    """The benchmark's context: 131072 rows, bf16 cache."""
    ctx, orc = make_pair(G4, max_seq=131072, kv_bf16=True, linear_layers=[])
    r = I.rng(131072)
    install_kv(ctx, orc, FULL, 0, I.normal(r, (131071, G4.kv_dim)), I.normal(r, (131071, G4.kv_dim)))
    one_step(ctx, orc, 0, 131072, r, TOL_BF16)
    ctx.check_guards()
    ctx.close()


@pytest.mark.parametrize("bf16", [False, True])
def test_ragged_batch_of_16_automatic_plan(bf16):
    """Sixteen sequences with ragged contexts between 8k and 32k in one launch under the automatic plan: one wave of
    CTAs with equal tile runs that cross unit boundaries, every unit shared by several CTAs."""
    n = 16
    ctx, orc = make_pair(G4, max_seq=32768 + 8, n_seqs=n, kv_bf16=bf16, linear_layers=[])
    r = I.rng(1600 + bf16)
    lens = [int(x) for x in r.integers(8192, 32768, n)]
    lens[0], lens[1] = 32767, 8192
    for s, ln in enumerate(lens):
        install_kv(ctx, orc, FULL, s, I.normal(r, (ln, G4.kv_dim)), I.normal(r, (ln, G4.kv_dim)))
    tol = TOL_BF16 if bf16 else TOL_F32
    for step in range(2):
        ins = [I.gqa_step_inputs(r, G4) for _ in range(n)]
        pos = [ln + step for ln in lens]
        got = ctx.full_attn_step_batched([FULL] * n, list(range(n)), pos, np.stack([i[0] for i in ins]),
                                         np.stack([i[1] for i in ins]), np.stack([i[2] for i in ins]),
                                         np.stack([i[3] for i in ins]))
        for s in range(n):
            ref = orc.full_attn_step(FULL, s, pos[s], *ins[s])
            assert I.rel_err(got[s], ref) <= tol, (step, s, lens[s])
    ctx.check_guards()
    ctx.close()


@pytest.mark.parametrize("coop", [1, 0])
@pytest.mark.parametrize("lens", [(20000, 9000, 31000), (5000,), (300, 32000), (2500, 40, 2500, 7)])
def test_units_shared_by_many_ctas(lens, coop):
    """Few long sequences: every (item, kv head) unit is shared by far more than sixteen CTAs, run boundaries fall
    inside units (a unit's last sharer goes on to the next unit and takes no part in a cooperative merge), short
    units sit between long ones, and the last merge group of a unit is partly filled."""
    n = len(lens)
    ctx, orc = make_pair(G4, max_seq=32768 + 8, n_seqs=n, kv_bf16=True, linear_layers=[])
    ctx.set_tuning("gqa_coop_merge", coop)
    ctx.set_tuning("gqa_coop_min_parts", 8)  # also the moderately shared units of these launches
    r = I.rng(1700 + n)
    for s, ln in enumerate(lens):
        install_kv(ctx, orc, FULL, s, I.normal(r, (ln, G4.kv_dim)), I.normal(r, (ln, G4.kv_dim)))
    for step in range(3):
        ins = [I.gqa_step_inputs(r, G4) for _ in range(n)]
        pos = [ln + step for ln in lens]
        got = ctx.full_attn_step_batched([FULL] * n, list(range(n)), pos, np.stack([i[0] for i in ins]),
                                         np.stack([i[1] for i in ins]), np.stack([i[2] for i in ins]),
                                         np.stack([i[3] for i in ins]))
        for s in range(n):
            ref = orc.full_attn_step(FULL, s, pos[s], *ins[s])
            assert I.rel_err(got[s], ref) <= TOL_BF16, (step, s)
    ctx.check_guards()
    ctx.close()


@pytest.mark.parametrize("bf16", [False, True])
def test_launch_of_more_than_512_items(bf16):
    """600 short sequences in one launch: beyond the 512 items whose tile offsets a CTA stages in shared memory, the
    work lookup reads the item list in device memory."""
    n = 600
    ctx, orc = make_pair(G4, max_seq=64, n_seqs=n, kv_bf16=bf16, linear_layers=[], max_batch=n)
    r = I.rng(1800 + bf16)
    lens = [int(x) for x in r.integers(0, 41, n)]
    for s, ln in enumerate(lens):
        if ln:
            install_kv(ctx, orc, FULL, s, I.normal(r, (ln, G4.kv_dim)), I.normal(r, (ln, G4.kv_dim)))
    tol = TOL_BF16 if bf16 else TOL_F32
    for step in range(2):
        ins = [I.gqa_step_inputs(r, G4) for _ in range(n)]
        pos = [ln + step for ln in lens]
        got = ctx.full_attn_step_batched([FULL] * n, list(range(n)), pos, np.stack([i[0] for i in ins]),
                                         np.stack([i[1] for i in ins]), np.stack([i[2] for i in ins]),
                                         np.stack([i[3] for i in ins]))
        worst = max(I.rel_err(got[s], orc.full_attn_step(FULL, s, pos[s], *ins[s])) for s in range(n))
        assert worst <= tol, (step, worst)
    ctx.check_guards()
    ctx.close()


def test_bounded_wait_runs_out_and_the_context_survives():
    """A load that never arrives: the first CTA arms the barrier of its first KV tile and issues no load for it, with
    a low poll limit.  Nothing is in flight for that barrier, so the wait simply runs out: the kernel returns, the
    call reports the failure, the merge counters are back at zero and the same context goes on to compute correct
    steps.  (No fault, trap or hang is involved anywhere.)"""
    ctx, orc = make_pair(G4, max_seq=4096, n_seqs=2, kv_bf16=True, linear_layers=[])
    r = I.rng(1900)
    for s in range(2):
        install_kv(ctx, orc, FULL, s, I.normal(r, (3000, G4.kv_dim)), I.normal(r, (3000, G4.kv_dim)))
    ctx.set_tuning("gqa_wait_spins", 2000)
    ctx.set_tuning("gqa_inject_lost_load", 1)
    ins = [I.gqa_step_inputs(r, G4) for _ in range(2)]
    with pytest.raises(M.MfcError, match="did not arrive within the wait limit"):
        ctx.full_attn_step_batched([FULL] * 2, [0, 1], [3000, 3000], np.stack([i[0] for i in ins]),
                                   np.stack([i[1] for i in ins]), np.stack([i[2] for i in ins]),
                                   np.stack([i[3] for i in ins]))
    ctx.set_tuning("gqa_inject_lost_load", 0)
    ctx.set_tuning("gqa_wait_spins", 0)
    ctx.synchronize()  # the report was cleared with the failed call
    # the failed step did append its rows (lengths advance when the call is issued): mirror that on the oracle
    for s in range(2):
        orc.full_attn_step(FULL, s, 3000, *ins[s])
    for step in range(3):
        ins = [I.gqa_step_inputs(r, G4) for _ in range(2)]
        pos = [3001 + step] * 2
        got = ctx.full_attn_step_batched([FULL] * 2, [0, 1], pos, np.stack([i[0] for i in ins]),
                                         np.stack([i[1] for i in ins]), np.stack([i[2] for i in ins]),
                                         np.stack([i[3] for i in ins]))
        for s in range(2):
            assert I.rel_err(got[s], orc.full_attn_step(FULL, s, pos[s], *ins[s])) <= TOL_BF16, (step, s)
    ctx.check_guards()
    ctx.close()


def test_one_cta_per_unit_plan():
    """Tuning "gqa_unit_aligned": 120 sequences of equal length give 240 equal units, which nearly fill the wave of 296
    CTAs, so every unit gets a CTA of its own (no shared units, nothing parked or merged).  Off, the same launch is
    cut into equal runs across unit boundaries; both must agree with the oracle."""
    n = 120
    ctx, orc = make_pair(G4, max_seq=512, n_seqs=n, kv_bf16=True, linear_layers=[], max_batch=n)
    r = I.rng(2000)
    for s in range(n):
        install_kv(ctx, orc, FULL, s, I.normal(r, (300, G4.kv_dim)), I.normal(r, (300, G4.kv_dim)))
    for step, aligned in enumerate((1, 0, 1)):
        ctx.set_tuning("gqa_unit_aligned", aligned)
        ins = [I.gqa_step_inputs(r, G4) for _ in range(n)]
        pos = [300 + step] * n
        got = ctx.full_attn_step_batched([FULL] * n, list(range(n)), pos, np.stack([i[0] for i in ins]),
                                         np.stack([i[1] for i in ins]), np.stack([i[2] for i in ins]),
                                         np.stack([i[3] for i in ins]))
        worst = max(I.rel_err(got[s], orc.full_attn_step(FULL, s, pos[s], *ins[s])) for s in range(n))
        assert worst <= TOL_BF16, (step, worst)
    ctx.check_guards()
    ctx.close()
