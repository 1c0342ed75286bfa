"""Folded MLA attention (crates/moeflux/shaders/shaders.metal:1717-1987): the oracle against a float64 statement and
its own tiled form at the reference's bound (cosine >= 0.99999, max |d| < 1e-2: tests/mla_sdpa_tiled.rs:176-186), and
the CUDA kernel against the oracle through the C ABI.  Inputs: the sin ramps of the reference's test
(tests/mla_sdpa_tiled.rs:92-105) and seeded normals; geometry of the MLA variant (128 heads, rank 512, rope 64,
scale 1/sqrt(192): crates/moeflux/src/riir/variants.rs:475-526)."""
import numpy as np
import pytest

import oracle as O
from tests import inputs as I

H, RANK, ROPE = 128, 512, 64
SCALE = 1.0 / np.sqrt(np.float32(192.0))


def ramp_inputs(cache_len, heads=H):
    f = lambda n, step, amp: (np.sin(np.arange(n, dtype=np.float32) * np.float32(step)) * np.float32(amp)).astype(np.float32)
    return (f(heads * RANK, 0.0007, 0.1), f(heads * ROPE, 0.0011, 0.1), f(cache_len * RANK, 0.00013, 0.05),
            f(cache_len * ROPE, 0.00017, 0.05))


def normal_inputs(cache_len, seed, heads=H, qs=1.0):
    r = I.rng(seed)
    return (I.normal(r, heads * RANK, qs), I.normal(r, heads * ROPE, qs), I.normal(r, cache_len * RANK),
            I.normal(r, cache_len * ROPE))


def f64_reference(cache_len, scale, qp, pe, lat, rk, heads=H):
    q = np.concatenate([qp.reshape(heads, RANK), pe.reshape(heads, ROPE)], axis=1).astype(np.float64)
    k = np.concatenate([lat.reshape(cache_len, RANK), rk.reshape(cache_len, ROPE)], axis=1).astype(np.float64)
    s = q @ k.T * float(scale)
    w = np.exp(s - s.max(axis=1, keepdims=True))
    w /= w.sum(axis=1, keepdims=True)
    return w @ lat.reshape(cache_len, RANK).astype(np.float64)


@pytest.mark.parametrize("cache_len", [1, 17, 300])
def test_oracle_matches_float64(cache_len):
    ins = normal_inputs(cache_len, 600 + cache_len, heads=16, qs=0.2)
    got = O.mla_sdpa_folded(cache_len, SCALE, *ins)
    assert I.rel_err(got, f64_reference(cache_len, SCALE, *ins, heads=16)) <= 1e-5
    if cache_len == 1:  # one position: the output is that latent row, for every head
        assert np.allclose(got, np.tile(ins[2].reshape(1, RANK), (16, 1)), atol=1e-6)


@pytest.mark.parametrize("cache_len,tile", [(4096, 4096), (8192, 4096), (1000, 64)])
def test_oracle_tiled_merge_matches_single_shot(cache_len, tile):
    ins = ramp_inputs(cache_len, heads=16)
    one = O.mla_sdpa_folded(cache_len, SCALE, *ins)
    tiled = O.mla_sdpa_folded(cache_len, SCALE, *ins, tile=tile)
    assert I.cosine(one, tiled) >= 0.99999
    assert np.max(np.abs(one - tiled)) < 1e-2
    assert I.rel_err(tiled, one) <= 1e-5  # far inside the reference's floor


@pytest.mark.gpu
@pytest.mark.parametrize("cache_len", [1, 15, 16, 17, 255, 256, 1000, 4096, 4097, 20000])
def test_gpu_matches_oracle_on_reference_ramps(cache_len):
    import moeflux_b200 as M

    ctx = M.Ctx(num_layers=4, max_seq=64)
    ins = ramp_inputs(cache_len)
    got = ctx.mla_sdpa_folded(cache_len, float(SCALE), *ins)
    ref = O.mla_sdpa_folded(cache_len, SCALE, *ins)
    assert np.isfinite(got).all()
    assert I.cosine(got, ref) >= 0.99999 and np.max(np.abs(got - ref)) < 1e-2  # the reference's own bound
    assert I.rel_err(got, ref) <= 1e-3                                         # its GPU-vs-CPU bound
    ctx.check_guards()
    ctx.close()


@pytest.mark.gpu
@pytest.mark.parametrize("cache_len,heads", [(333, 128), (5000, 128), (2048, 16), (700, 40), (32768, 128)])
def test_gpu_matches_oracle_on_seeded_normals(cache_len, heads):
    import moeflux_b200 as M

    ctx = M.Ctx(num_layers=4, max_seq=64)
    ins = normal_inputs(cache_len, 700 + cache_len, heads=heads, qs=0.3)
    got = ctx.mla_sdpa_folded(cache_len, float(SCALE), *ins)
    ref = O.mla_sdpa_folded(cache_len, SCALE, *ins)
    assert np.isfinite(got).all()
    assert I.rel_err(got, ref) <= 1e-4
    # forced small chunks: many partials per head through the merge kernel
    ctx.set_tuning("gqa_chunk", 64)
    got2 = ctx.mla_sdpa_folded(min(cache_len, 3000), float(SCALE), *ins)
    ref2 = ref if cache_len <= 3000 else O.mla_sdpa_folded(3000, SCALE, *ins)
    assert I.rel_err(got2, ref2) <= 1e-4
    ctx.check_guards()
    ctx.close()


@pytest.mark.gpu
def test_gpu_argument_errors():
    import moeflux_b200 as M

    ctx = M.Ctx(num_layers=4, max_seq=64)
    z = np.zeros(16 * RANK, np.float32)
    with pytest.raises(M.MfcError):
        ctx.mla_sdpa_folded(0, 1.0, z, np.zeros(16 * ROPE, np.float32), np.zeros(RANK, np.float32), np.zeros(ROPE, np.float32))
    ctx.close()


@pytest.mark.gpu
@pytest.mark.parametrize("cache_len,heads", [(1, 128), (31, 16), (32, 128), (33, 128), (1000, 128), (5000, 40), (32768, 128)])
def test_gpu_bf16_cache_matches_oracle_on_the_rounded_cache(cache_len, heads):
    """The bf16 latent cache (not a reference format; the counterpart of the GQA path's bf16 KV cache): the oracle
    runs in fp32 on the rounded cache values, tolerance 2e-2."""
    import torch

    import moeflux_b200 as M

    dev = torch.device("cuda:0")
    ctx = M.Ctx(num_layers=4, max_seq=64)
    qp, pe, lat, rk = normal_inputs(cache_len, 800 + cache_len, heads=heads, qs=0.3)
    ref = O.mla_sdpa_folded(cache_len, SCALE, qp, pe, O.round_bf16(lat), O.round_bf16(rk))
    dq, dp = torch.tensor(qp, device=dev), torch.tensor(pe, device=dev)
    dl = torch.tensor(lat, device=dev).to(torch.bfloat16).contiguous()
    dr = torch.tensor(rk, device=dev).to(torch.bfloat16).contiguous()
    out = torch.full((heads, RANK), float("nan"), device=dev)
    torch.cuda.synchronize()
    for chunk in (0, 64):  # the automatic split, then many small chunks through the merge kernel
        ctx.set_tuning("gqa_chunk", chunk)
        ctx.mla_sdpa_folded_bf16_dev(heads, cache_len, float(SCALE), dq.data_ptr(), dp.data_ptr(), dl.data_ptr(),
                                     dr.data_ptr(), out.data_ptr())
        ctx.synchronize()
        got = out.cpu().numpy()
        assert np.isfinite(got).all()
        assert I.rel_err(got, ref) <= 2e-2, chunk
    ctx.check_guards()
    ctx.close()
