"""The allocation-free SDPA entry point against the context's own SDPA.

``mfc_sdpa_static_dev`` serves callers that must not allocate device memory
(see include/moeflux_cuda.h): its split-K scratch is a fixed array inside the
library.  This file is collected last on purpose, so that a run that stops at
the first failure has already run every other test.  The entry point is called
twice in a row on different inputs: the second call finds the first call's
leftovers in the shared array and must not be disturbed by them.
"""
import numpy as np
import pytest

import moeflux_b200 as M
from oracle import A17B as G
from tests import inputs as I

pytestmark = pytest.mark.gpu


def _cache_layout(rows_f32, cap_rows, bf16, dev):
    """[n][Hkv*256] fp32 host rows -> device tensor [Hkv][cap_rows][256] of the cache type."""
    import torch

    n = rows_f32.shape[0]
    t = torch.zeros(G.num_kv_heads, cap_rows, G.head_dim, dtype=torch.bfloat16 if bf16 else torch.float32, device=dev)
    src = torch.tensor(rows_f32.reshape(n, G.num_kv_heads, G.head_dim)).permute(1, 0, 2)
    t[:, :n] = src.to(dev).to(t.dtype)
    return t


@pytest.mark.parametrize("bf16", [False, True])
def test_static_sdpa_matches_context_sdpa_twice_in_a_row(bf16):
    import torch

    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    ctx = M.Ctx(max_seq=4096, kv_dtype=M.KV_BF16 if bf16 else M.KV_F32)
    dtype = M.KV_BF16 if bf16 else M.KV_F32
    # same kernel, same stored values: only the chunking (hence summation order) differs
    tol = 2e-3 if bf16 else 2e-5
    r = I.rng(300)
    for call, kv_len in enumerate((3000, 700)):  # several chunks, then fewer: stale partials stay behind
        q, gate, _, _ = I.gqa_step_inputs(r)
        K, V = I.normal(r, (kv_len, G.kv_dim)), I.normal(r, (kv_len, G.kv_dim))
        want = ctx.sdpa(kv_len, q, gate, K, V)
        cap = 4096
        kc, vc = _cache_layout(K, cap, bf16, dev), _cache_layout(V, cap, bf16, dev)
        dq, dg = torch.tensor(q, device=dev), torch.tensor(gate, device=dev)
        out = torch.full((G.q_dim,), float("nan"), device=dev)
        torch.cuda.synchronize()
        M.sdpa_static_dev(G.num_attn_heads, G.num_kv_heads, dtype, kv_len, cap, dq.data_ptr(), dg.data_ptr(),
                          kc.data_ptr(), vc.data_ptr(), out.data_ptr(), torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        got = out.cpu().numpy()
        assert np.isfinite(got).all(), f"call {call}"
        assert I.rel_err(got, want) <= tol, f"call {call}"
    ctx.close()


def test_static_sdpa_refuses_sizes_beyond_its_scratch():
    import torch

    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    x = torch.zeros(G.num_kv_heads * 64 * G.head_dim, device=dev)
    q = torch.zeros(G.q_dim, device=dev)
    args = (q.data_ptr(), 0, x.data_ptr(), x.data_ptr(), q.data_ptr(), 0)
    with pytest.raises(M.MfcError, match="at most 262144 rows"):
        M.sdpa_static_dev(32, 2, M.KV_F32, 262145, 262145, *args)
    with pytest.raises(M.MfcError, match="at most 8 kv heads"):
        M.sdpa_static_dev(32, 16, M.KV_F32, 64, 64, *args)
    with pytest.raises(M.MfcError, match="kv_len must be > 0"):
        M.sdpa_static_dev(32, 2, M.KV_F32, 0, 64, *args)
