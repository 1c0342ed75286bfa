"""One-call token step over a layer stack (mfc_eval_token_attn) against the
oracle driven layer by layer, as RsCtx::eval_token walks its layers
(crates/moeflux/src/riir/mod.rs:1769-1876)."""
import numpy as np
import pytest

import moeflux_b200 as M
from oracle import Geometry
from tests import inputs as I
from tests.gpu_common import TOL_BF16, TOL_F32, make_pair

pytestmark = pytest.mark.gpu

G8 = Geometry(num_layers=8)


@pytest.mark.parametrize("bf16", [False, True])
def test_stack_step_matches_layerwise_oracle(bf16):
    n_seqs = 3
    ctx, orc = make_pair(G8, max_seq=96, n_seqs=n_seqs, kv_bf16=bf16)
    r = I.rng(400)
    full_items = [(l, s) for l in range(8) if G8.is_full_layer(l) for s in range(n_seqs)]
    lin_items = [(l, s) for l in range(8) if not G8.is_full_layer(l) for s in range(n_seqs)]
    tol = TOL_BF16 if bf16 else TOL_F32
    for pos in range(40):
        fin = [I.gqa_step_inputs(r, G8) for _ in full_items]
        lin = [I.gdn_step_inputs(r, G8) for _ in lin_items]
        fo, lo = ctx.eval_token_attn(
            full_items, [pos] * len(full_items), np.stack([i[0] for i in fin]), np.stack([i[1] for i in fin]),
            np.stack([i[2] for i in fin]), np.stack([i[3] for i in fin]), lin_items, np.stack([i[0] for i in lin]),
            np.stack([i[1] for i in lin]), np.stack([i[2] for i in lin]), np.stack([i[3] for i in lin]))
        for j, (l, s) in enumerate(full_items):
            assert I.rel_err(fo[j], orc.full_attn_step(l, s, pos, *fin[j])) <= tol, (pos, l, s)
        for j, (l, s) in enumerate(lin_items):
            assert I.rel_err(lo[j], orc.linear_attn_step(l, s, *lin[j])) <= TOL_F32, (pos, l, s)
    # either group may be empty
    fin = [I.gqa_step_inputs(r, G8) for _ in full_items]
    fo, lo = ctx.eval_token_attn(full_items, [40] * len(full_items), np.stack([i[0] for i in fin]),
                                 np.stack([i[1] for i in fin]), np.stack([i[2] for i in fin]),
                                 np.stack([i[3] for i in fin]), [], None, None, None, None)
    assert lo.shape[0] == 0
    for j, (l, s) in enumerate(full_items):
        assert I.rel_err(fo[j], orc.full_attn_step(l, s, 40, *fin[j])) <= tol
    ctx.close()


def test_stack_step_failure_changes_nothing():
    ctx, orc = make_pair(G8, max_seq=32)
    r = I.rng(401)
    full_items, lin_items = [(3, 0), (7, 0)], [(0, 0), (1, 0)]
    fin = [I.gqa_step_inputs(r, G8) for _ in full_items]
    lin = [I.gdn_step_inputs(r, G8) for _ in lin_items]
    args = lambda pos: (full_items, pos, np.stack([i[0] for i in fin]), np.stack([i[1] for i in fin]),
                        np.stack([i[2] for i in fin]), np.stack([i[3] for i in fin]), lin_items,
                        np.stack([i[0] for i in lin]), np.stack([i[1] for i in lin]), np.stack([i[2] for i in lin]),
                        np.stack([i[3] for i in lin]))
    ctx.eval_token_attn(*args([0, 0]))
    before = ctx.state_save(0)
    with pytest.raises(M.MfcError, match="current length"):
        ctx.eval_token_attn(*args([1, 5]))  # second position is wrong: nothing may advance, not even the conv ring
    assert ctx.state_save(0) == before
    fo, lo = ctx.eval_token_attn(*args([1, 1]))
    for l, s in full_items:
        orc.full_attn_step(l, s, 0, *fin[full_items.index((l, s))])
    for j, (l, s) in enumerate(lin_items):
        orc.linear_attn_step(l, s, *lin[j])
    for j, (l, s) in enumerate(lin_items):
        assert I.rel_err(lo[j], orc.linear_attn_step(l, s, *lin[j])) <= TOL_F32
    ctx.close()
