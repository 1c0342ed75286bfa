"""The allocation-free SDPA entry point against the CPU oracle and the context's own SDPA.

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
import oracle as O
from oracle import A17B as G
from tests import inputs as I
from tests.gpu_common import TOL_BF16, TOL_F32

pytestmark = pytest.mark.gpu


def _cache_layout(rows_f32, cap_rows, bf16, dev, fill=0.0):
    """[n][Hkv*256] fp32 host rows -> device tensor [Hkv][cap_rows][256] of the cache type; rows past n hold `fill`."""
    import torch

    n = rows_f32.shape[0]
    t = torch.full((G.num_kv_heads, cap_rows, G.head_dim), fill, dtype=torch.bfloat16 if bf16 else torch.float32,
                   device=dev)
    src = torch.tensor(rows_f32.reshape(n, G.num_kv_heads, G.head_dim)).permute(1, 0, 2)
    t[:, :n] = src.to(dev).to(t.dtype)
    return t


@pytest.mark.parametrize("bf16", [False, True])
def test_static_sdpa_matches_oracle_and_context_twice_in_a_row(bf16):
    import torch

    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    ctx = M.Ctx(max_seq=4096, kv_dtype=M.KV_BF16 if bf16 else M.KV_F32)
    dtype = M.KV_BF16 if bf16 else M.KV_F32
    r = I.rng(300)
    stream = torch.cuda.current_stream().cuda_stream
    for call, kv_len in enumerate((3000, 700)):  # several chunks, then fewer: stale partials stay behind
        q, gate, _, _ = I.gqa_step_inputs(r)
        K, V = I.normal(r, (kv_len, G.kv_dim)), I.normal(r, (kv_len, G.kv_dim))
        want_ctx = ctx.sdpa(kv_len, q, gate, K, V)
        want = O.sdpa(kv_len, q, gate, O.round_bf16(K) if bf16 else K, O.round_bf16(V) if bf16 else V)
        cap = 4096
        kc, vc = _cache_layout(K, cap, bf16, dev), _cache_layout(V, cap, bf16, dev)
        dq, dg = torch.tensor(q, device=dev), torch.tensor(gate, device=dev)
        out = torch.full((G.q_dim,), float("nan"), device=dev)
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info(dev)[0]
        M.sdpa_static_dev(G.num_attn_heads, G.num_kv_heads, dtype, kv_len, cap, dq.data_ptr(), dg.data_ptr(),
                          kc.data_ptr(), vc.data_ptr(), out.data_ptr(), stream)
        M.sdpa_static_status(stream)  # waits, and raises if a kernel gave up
        if call > 0:  # (the very first call on a device loads the kernels' code, which the driver accounts for)
            assert torch.cuda.mem_get_info(dev)[0] == free_before, "the call changed the free device memory"
        got = out.cpu().numpy()
        assert np.isfinite(got).all(), f"call {call}"
        assert I.rel_err(got, want) <= (TOL_BF16 if bf16 else TOL_F32), f"call {call}"
        # same kernel, same stored values as the context's hook: only the chunking (summation order) differs
        assert I.rel_err(got, want_ctx) <= (2e-3 if bf16 else 2e-5), f"call {call}"
    ctx.close()


@pytest.mark.parametrize("bf16", [False, True])
@pytest.mark.parametrize("kv_len", [1, 45, 1001])
def test_static_sdpa_never_uses_rows_past_kv_len(bf16, kv_len):
    """A caller's cache is whatever memory the caller had: the rows past kv_len hold NaN here, and kv_len is not a
    multiple of the kernel's tile.  The output must be finite and equal to the oracle's."""
    import torch

    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    r = I.rng(310 + kv_len)
    q, gate, _, _ = I.gqa_step_inputs(r)
    K, V = I.normal(r, (kv_len, G.kv_dim)), I.normal(r, (kv_len, G.kv_dim))
    want = O.sdpa(kv_len, q, gate, O.round_bf16(K) if bf16 else K, O.round_bf16(V) if bf16 else V)
    cap = 1024 + 64
    kc, vc = _cache_layout(K, cap, bf16, dev, float("nan")), _cache_layout(V, cap, bf16, dev, float("nan"))
    dq, dg = torch.tensor(q, device=dev), torch.tensor(gate, device=dev)
    out = torch.full((G.q_dim,), float("nan"), device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    M.sdpa_static_dev(G.num_attn_heads, G.num_kv_heads, M.KV_BF16 if bf16 else M.KV_F32, kv_len, cap, dq.data_ptr(),
                      dg.data_ptr(), kc.data_ptr(), vc.data_ptr(), out.data_ptr(), stream)
    M.sdpa_static_status(stream)
    got = out.cpu().numpy()
    assert np.isfinite(got).all()
    assert I.rel_err(got, want) <= (TOL_BF16 if bf16 else TOL_F32)


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
