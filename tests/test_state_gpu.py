"""Sequence-state calls on the GPU context against the host-memory oracle:
memory_clear / memory_seq_rm / memory_seq_pos_max (crates/moeflux/src/riir/
state.rs:417-473) and the 'MFLX' snapshot (state_snapshot.rs), including wire
compatibility in both directions and the no-mutation-on-failure contract
(crates/moeflux/tests/diff_oracle.rs:3902-4051)."""
import struct

import numpy as np
import pytest

import moeflux_b200 as M
from oracle import Geometry
from oracle import snapshot as snap
from tests import inputs as I
from tests.gpu_common import TOL_F32, make_pair

pytestmark = pytest.mark.gpu

G8 = Geometry(num_layers=8)  # 6 linear + 2 full layers, full-size heads


def _run_steps(ctx, orc, r, n_steps, seq=0, start=0):
    for pos in range(start, start + n_steps):
        for layer in range(G8.num_layers):
            if G8.is_full_layer(layer):
                ins = I.gqa_step_inputs(r, G8)
                a = ctx.full_attn_step(layer, seq, pos, *ins)
                b = orc.full_attn_step(layer, seq, pos, *ins)
            else:
                ins = I.gdn_step_inputs(r, G8)
                a = ctx.linear_attn_step(layer, seq, *ins)
                b = orc.linear_attn_step(layer, seq, *ins)
            assert I.rel_err(a, b) <= TOL_F32


@pytest.mark.parametrize("version", [1, 2])
def test_snapshot_matches_oracle_and_round_trips(version):
    ctx, orc = make_pair(G8, max_seq=64, n_seqs=2, snapshot_version=version)
    r = I.rng(200)
    _run_steps(ctx, orc, r, 7)           # 7 steps: the conv ring is mid-cycle
    _run_steps(ctx, orc, r, 3, seq=1)
    for seq, ln in ((0, 7), (1, 3)):
        assert ctx.state_size(seq) == orc.state_size(seq) == snap.state_size(G8, [ln, ln], version)
        blob, ref = ctx.state_save(seq), orc.state_save(seq)
        assert len(blob) == len(ref)
        hb = (8 if version == 1 else 10) * 4
        assert blob[:hb] == ref[:hb]
        got_layers, ref_layers = snap.state_load(G8, blob), snap.state_load(G8, ref)
        for a, b in zip(got_layers, ref_layers):
            for x, y in zip(a[1:], b[1:]):
                assert x.shape == y.shape
                if x.size:
                    assert I.rel_err(x, y) <= TOL_F32
        # conv history and V rows are moved, never computed: bit-exact
        assert np.array_equal(got_layers[0][1], ref_layers[0][1])
        assert np.array_equal(got_layers[3][2], ref_layers[3][2])
    # save -> clear -> load -> save is byte-identical, and decoding continues identically
    blob = ctx.state_save(0)
    ctx.memory_clear(0)
    assert ctx.memory_seq_pos_max(0) == 0 and ctx.memory_seq_pos_max(1) == 3
    ctx.state_load(0, blob)
    assert ctx.state_save(0) == blob
    orc.state_load(0, blob)
    _run_steps(ctx, orc, r, 3, start=7)
    ctx.close()


def test_wire_compat_oracle_to_gpu_and_back():
    ctx, orc = make_pair(G8, max_seq=64)
    r = I.rng(201)
    _run_steps(ctx, orc, r, 5)
    ref = orc.state_save(0)
    ctx.memory_clear(0)
    ctx.state_load(0, ref)            # host-written snapshot into the GPU context
    assert ctx.state_save(0) == ref   # fp32 cache: nothing is recomputed, bytes must survive
    v2 = snap.state_save(G8, snap.state_load(G8, ref), 2)
    ctx.state_load(0, v2)             # the loader accepts both header versions
    assert ctx.state_save(0) == ref
    ctx.close()


def test_bf16_cache_widens_and_rounds():
    ctx, orc = make_pair(G8, max_seq=64, kv_bf16=True)
    r = I.rng(202)
    for layer in (3, 7):
        orc.load_kv(layer, 0, I.normal(r, (9, G8.kv_dim)), I.normal(r, (9, G8.kv_dim)))
    ref = orc.state_save(0)           # rows already rounded to bf16 values
    ctx.state_load(0, ref)
    assert ctx.state_save(0) == ref
    ctx.close()


def test_failed_load_leaves_state_unchanged():
    ctx, orc = make_pair(G8, max_seq=16)
    r = I.rng(203)
    _run_steps(ctx, orc, r, 4)
    good = ctx.state_save(0)
    hb = 32
    lin = 3 * G8.conv_dim * 4 + G8.ssm_elems * 4
    off = hb + 3 * lin
    bads = [good[:7], b"XXXX" + good[4:], good[:4] + struct.pack("<I", 9) + good[8:],
            good[:8] + struct.pack("<I", 60) + good[12:], good[:-5],
            good[:off] + struct.pack("<i", -2) + good[off + 4:],
            good[:off] + struct.pack("<i", 17) + good[off + 4:]]  # 17 > max_seq
    for b in bads:
        with pytest.raises(M.MfcError):
            ctx.state_load(0, b)
        assert ctx.state_save(0) == good
        assert ctx.memory_seq_pos_max(0) == 4
    small = np.empty(ctx.state_size(0) - 1, np.uint8)
    assert ctx.state_save_into(0, small) == -1   # buffer too small (moeflux.h:629-633)
    ctx.close()


def test_memory_seq_rm_and_pos_max_semantics():
    ctx, orc = make_pair(G8, max_seq=64, n_seqs=2)
    r = I.rng(204)
    assert ctx.memory_seq_pos_max(0) == 0   # empty sequence: the reference returns the length, 0
    assert ctx.memory_seq_pos_max(5) == -1
    _run_steps(ctx, orc, r, 6)
    _run_steps(ctx, orc, r, 2, seq=1)
    for p0, p1 in ((8, -1), (4, 5), (5, 2), (-3, -1)):
        assert ctx.memory_seq_rm(0, p0, p1) and orc.memory_seq_rm(0, p0, p1)
        assert ctx.memory_seq_pos_max(0) == orc.memory_seq_pos_max(0)
        assert ctx.memory_seq_pos_max(1) == 2      # the other sequence is untouched
        # linear layers were reset (lossy by specification) on both sides; KV prefix kept
        a, b = snap.state_load(G8, ctx.state_save(0)), snap.state_load(G8, orc.state_save(0))
        for x, y in zip(a, b):
            assert all(np.allclose(u, w, rtol=0, atol=1e-4) for u, w in zip(x[1:], y[1:]))
        assert not np.any(a[0][2])
    assert not ctx.memory_seq_rm(9, 0, -1)
    # decoding resumes at the truncated length
    _run_steps(ctx, orc, r, 2, start=ctx.memory_seq_pos_max(0))
    ctx.close()


def test_checkpoint_restore_lru():
    """checkpoint_pos / restore_to, the shapes of crates/moeflux/tests/checkpoint_restore.rs:
    round trip, unknown position, memory_clear drops snapshots, LRU keeps the last n,
    position 0 is protected."""
    ctx, orc = make_pair(G8, max_seq=64)
    r = I.rng(205)
    ctx.checkpoint_pos(0)
    _run_steps(ctx, orc, r, 3)
    ctx.checkpoint_pos(3)
    at3 = ctx.state_save(0)
    orc3 = orc.state_save(0)
    _run_steps(ctx, orc, r, 4, start=3)           # mutate by decoding
    assert ctx.state_save(0) != at3
    ctx.restore_to(3)
    assert ctx.state_save(0) == at3 and ctx.memory_seq_pos_max(0) == 3
    orc.state_load(0, orc3)
    _run_steps(ctx, orc, r, 2, start=3)           # decoding resumes identically after the rewind
    with pytest.raises(M.MfcError, match="no checkpoint stored at position 17"):
        ctx.restore_to(17)
    # LRU: cap 4, position 0 protected, the oldest other entry goes first
    assert ctx.checkpoint_count() == 2
    for p in (5, 6, 7, 8):
        ctx.checkpoint_pos(p)
    assert ctx.checkpoint_count() == 4
    ctx.restore_to(0)                              # 0 survived; entries > 0 are dropped by the restore
    assert ctx.checkpoint_count() == 1 and ctx.memory_seq_pos_max(0) == 0
    with pytest.raises(M.MfcError):
        ctx.restore_to(8)
    ctx.checkpoint_pos(2)
    ctx.checkpoint_pos(2)                          # overwrite keeps one entry
    assert ctx.checkpoint_count() == 2
    ctx.set_max_checkpoints(2)
    ctx.checkpoint_pos(9)
    assert ctx.checkpoint_count() == 2             # 2 evicted, 0 and 9 kept
    with pytest.raises(M.MfcError):
        ctx.restore_to(2)
    ctx.memory_seq_rm(0, 1, -1)
    assert ctx.checkpoint_count() == 2             # truncation keeps snapshots
    ctx.memory_clear(0)
    assert ctx.checkpoint_count() == 0             # a full clear drops them
    ctx.close()
