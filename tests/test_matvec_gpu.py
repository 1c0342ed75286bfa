"""GPU parity of the 4-bit group-64 dequant matvec (the projections either side of the attention
sub-block) against the CPU oracle, through the C ABI.  The first three cases are the reference's own
known answers (crates/moeflux/src/riir/cpu_matvec.rs:370-451); shapes are the A17B projections
(hidden 4096: q_proj 16384, k/v_proj 512, in_proj_qkv 12288, z 8192, a/b 64; o_proj / out_proj
8192 -> 4096).  fp32 throughout, tolerance 1e-4 as max|d| / max|ref|."""
import numpy as np
import pytest

import moeflux_b200 as M
import oracle as O
from tests import inputs as I
from tests.gpu_common import TOL_F32, make_pair

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    c, _ = make_pair(max_seq=64, n_seqs=1, linear_layers=[])
    yield c
    c.close()


def test_reference_known_answers(ctx):
    ones = np.ones(64, np.float32)
    assert ctx.dequant_matvec_4bit(np.full(8, 0x11111111, np.uint32), [0x3F80], [0x0000], 64, 1, ones).tolist() == [64.0]
    out = ctx.dequant_matvec_4bit(np.full(16, 0xFFFFFFFF, np.uint32), [0x3F80] * 2, [0x3F80] * 2, 64, 2,
                                  np.zeros(64, np.float32))
    assert out.tolist() == [0.0, 0.0]
    assert ctx.dequant_matvec_4bit(np.zeros(8, np.uint32), [0x40A0], [0x4000], 64, 1, ones).tolist() == [128.0]


@pytest.mark.parametrize("in_dim,out_dim", [(64, 1), (128, 5), (4096, 512), (4096, 64), (4096, 1000), (8192, 4096),
                                            (16384, 33)])
def test_single_vector_parity(ctx, in_dim, out_dim):
    r = I.rng(in_dim + out_dim)
    packed, scales, biases = I.quant_weights(r, in_dim, out_dim)
    x = I.normal(r, in_dim)
    got = ctx.dequant_matvec_4bit(packed, scales, biases, in_dim, out_dim, x)
    ref = O.dequant_matvec_4bit(packed, scales, biases, in_dim, out_dim, x)
    assert np.isfinite(got).all()
    assert I.rel_err(got, ref) <= TOL_F32


@pytest.mark.parametrize("in_dim,out_dim", [(192, 40), (2112, 100), (4096, 12288), (4160, 4100)])
def test_single_vector_ragged_stages_and_many_tiles(ctx, in_dim, out_dim):
    """Shapes that exercise the one-vector kernel's edges: an odd number of groups (the last pair of groups is half
    empty), a last stage of one group (2112 = 33 groups), more tiles than CTAs (every CTA takes several, in batches of
    four behind one rendezvous), a last tile of 4 rows.  Twice in a row: the tile counter is back at zero for the
    second launch, and the result is the same to the bit (fixed summation order)."""
    r = I.rng(3 * in_dim + out_dim)
    packed, scales, biases = I.quant_weights(r, in_dim, out_dim)
    x = I.normal(r, in_dim)
    ref = O.dequant_matvec_4bit(packed, scales, biases, in_dim, out_dim, x)
    got = ctx.dequant_matvec_4bit(packed, scales, biases, in_dim, out_dim, x)
    assert I.rel_err(got, ref) <= 1e-5, I.rel_err(got, ref)  # integer products: ten times inside the 1e-4 contract
    again = ctx.dequant_matvec_4bit(packed, scales, biases, in_dim, out_dim, x)
    assert np.array_equal(got, again)


def test_single_vector_wide_dynamic_range_and_nonfinite_inputs(ctx):
    """x is turned into integers per group of 64 features, relative to the group's largest element: elements 2^20
    times smaller than their neighbours keep their leading bits, a zero group stays zero, and a NaN or an infinity in
    x makes every output NaN (every row multiplies every feature), as in the reference's product."""
    r = I.rng(4242)
    in_dim, out_dim = 4096, 300
    packed, scales, biases = I.quant_weights(r, in_dim, out_dim)
    x = I.normal(r, in_dim)
    x[::7] *= 2.0 ** 20
    x[64:128] = 0.0
    x[130] = 1e-30
    ref = O.dequant_matvec_4bit(packed, scales, biases, in_dim, out_dim, x)
    got = ctx.dequant_matvec_4bit(packed, scales, biases, in_dim, out_dim, x)
    assert I.rel_err(got, ref) <= 1e-5, I.rel_err(got, ref)
    small = np.zeros(in_dim, np.float32)
    small[5] = 3e-39  # a denormal on its own: below what the integer scale reaches, contributes nothing or its value
    got = ctx.dequant_matvec_4bit(packed, scales, biases, in_dim, out_dim, small)
    assert np.all(np.abs(got) <= 3e-39 * 16 * 0.2)
    for bad in (np.nan, np.inf):
        xb = I.normal(r, in_dim)
        xb[1000] = bad
        got = ctx.dequant_matvec_4bit(packed, scales, biases, in_dim, out_dim, xb)
        assert np.isnan(got).all() or (bad == np.inf and not np.isfinite(got).any())


@pytest.mark.parametrize("n_vec", [2, 3, 5, 8])
def test_several_vectors_share_the_weights(ctx, n_vec):
    r = I.rng(70 + n_vec)
    in_dim, out_dim = 4096, 777
    packed, scales, biases = I.quant_weights(r, in_dim, out_dim)
    x = I.normal(r, (n_vec, in_dim))
    got = ctx.dequant_matvec_4bit(packed, scales, biases, in_dim, out_dim, x)
    assert got.shape == (n_vec, out_dim)
    for v in range(n_vec):
        ref = O.dequant_matvec_4bit(packed, scales, biases, in_dim, out_dim, x[v])
        assert I.rel_err(got[v], ref) <= TOL_F32
    # each vector's result does not depend on its neighbours or on its place in the batch
    rev = ctx.dequant_matvec_4bit(packed, scales, biases, in_dim, out_dim, x[::-1].copy())
    assert np.array_equal(rev[::-1], got)
    alone = ctx.dequant_matvec_4bit(packed, scales, biases, in_dim, out_dim, x[n_vec - 1])  # another kernel: tolerance
    assert I.rel_err(alone, got[n_vec - 1]) <= TOL_F32


@pytest.mark.parametrize("n_vec,in_dim,out_dim", [(3, 2112, 100), (5, 192, 40), (2, 4160, 530), (8, 8192, 300), (7, 64, 3)])
def test_several_vectors_ragged_shapes(ctx, n_vec, in_dim, out_dim):
    """The several-vector form of the kernel at the shapes that take its other branches: scales and biases read from
    global memory (in_dim not a multiple of 512), a last stage of one group, an odd number of groups, a last tile of a
    few rows, an odd number of vectors (the last pair of columns half empty), 8192-wide rows (four passes' worth of
    staging for 8 vectors)."""
    r = I.rng(100 * n_vec + in_dim + out_dim)
    packed, scales, biases = I.quant_weights(r, in_dim, out_dim)
    x = I.normal(r, (n_vec, in_dim))
    got = ctx.dequant_matvec_4bit(packed, scales, biases, in_dim, out_dim, x)
    assert got.shape == (n_vec, out_dim)
    for v in range(n_vec):
        ref = O.dequant_matvec_4bit(packed, scales, biases, in_dim, out_dim, x[v])
        assert I.rel_err(got[v], ref) <= 1e-5, (v, I.rel_err(got[v], ref))


def test_device_pointer_entry_point(ctx):
    import torch
    r = I.rng(5)
    in_dim, out_dim, n_vec = 4096, 12288, 4
    packed, scales, biases = I.quant_weights(r, in_dim, out_dim)
    x = I.normal(r, (n_vec, in_dim))
    dev = torch.device("cuda:0")
    d_w = torch.from_numpy(packed.view(np.int32)).to(dev)
    d_s = torch.from_numpy(scales.view(np.int16)).to(dev)
    d_b = torch.from_numpy(biases.view(np.int16)).to(dev)
    d_x = torch.from_numpy(x).to(dev)
    d_o = torch.empty(n_vec, out_dim, device=dev)
    torch.cuda.synchronize(dev)  # the operands are in place before the context's own stream reads them
    ctx.dequant_matvec_4bit_dev(d_w.data_ptr(), d_s.data_ptr(), d_b.data_ptr(), in_dim, out_dim, d_x.data_ptr(), n_vec,
                                d_o.data_ptr())
    ctx.synchronize()
    got = d_o.cpu().numpy()
    for v in range(n_vec):
        assert I.rel_err(got[v], O.dequant_matvec_4bit(packed, scales, biases, in_dim, out_dim, x[v])) <= TOL_F32


def test_errors_like_the_reference(ctx):
    ones = np.ones(96, np.float32)
    with pytest.raises(M.MfcError, match="multiple"):  # InDimNotMultiple
        ctx.dequant_matvec_4bit(np.zeros(12, np.uint32), [0x3F80], [0x0000], 96, 1, ones)
    with pytest.raises(ValueError, match="packed"):  # SliceLen
        ctx.dequant_matvec_4bit(np.zeros(7, np.uint32), [0x3F80], [0x0000], 64, 1, np.ones(64, np.float32))
    with pytest.raises(M.MfcError):  # more vectors than one launch takes
        ctx.dequant_matvec_4bit(np.zeros(8, np.uint32), [0x3F80], [0x0000], 64, 1, np.ones((9, 64), np.float32))


def test_more_vectors_than_one_pass_holds(ctx):
    # 8 vectors of 16384 features do not fit the staging area at once: the call makes several passes
    r = I.rng(9)
    packed, scales, biases = I.quant_weights(r, 16384, 40)
    x = I.normal(r, (8, 16384))
    got = ctx.dequant_matvec_4bit(packed, scales, biases, 16384, 40, x)
    for v in range(8):
        assert I.rel_err(got[v], O.dequant_matvec_4bit(packed, scales, biases, 16384, 40, x[v])) <= TOL_F32


def test_several_matrices_in_one_launch(ctx):
    # q/k/v_proj-like batch: three matrices of the same in_dim on the same input, odd row counts
    import torch
    r = I.rng(21)
    in_dim, n_vec, out_dims = 4096, 2, [1030, 513, 7]
    dev = torch.device("cuda:0")
    mats = [I.quant_weights(r, in_dim, o) for o in out_dims]
    x = I.normal(r, (n_vec, in_dim))
    d_w = [torch.from_numpy(m[0].view(np.int32)).to(dev) for m in mats]
    d_s = [torch.from_numpy(m[1].view(np.int16)).to(dev) for m in mats]
    d_b = [torch.from_numpy(m[2].view(np.int16)).to(dev) for m in mats]
    d_x = torch.from_numpy(x).to(dev)
    d_o = [torch.full((n_vec, o), float("nan"), device=dev) for o in out_dims]
    torch.cuda.synchronize(dev)
    ctx.dequant_matvec_4bit_multi_dev([t.data_ptr() for t in d_w], [t.data_ptr() for t in d_s], [t.data_ptr() for t in d_b],
                                      in_dim, out_dims, d_x.data_ptr(), n_vec, [t.data_ptr() for t in d_o])
    ctx.synchronize()
    for m, o in zip(mats, d_o):
        got = o.cpu().numpy()
        for v in range(n_vec):
            assert I.rel_err(got[v], O.dequant_matvec_4bit(m[0], m[1], m[2], in_dim, got.shape[1], x[v])) <= TOL_F32
    with pytest.raises(M.MfcError):
        ctx.dequant_matvec_4bit_multi_dev([0] * 9, [0] * 9, [0] * 9, in_dim, [1] * 9, d_x.data_ptr(), 1, [0] * 9)


def test_bounded_wait_runs_out_and_the_context_survives():
    """The projection kernel's failure path: its first CTA arms the barrier of its first stage of weights and requests
    nothing for it, with a low poll limit.  Nothing is in flight for that barrier, so the consumers' wait runs out:
    the CTA gives up, the others finish, the call reports the failure, the tile counters are back at zero and the
    same context goes on to compute correct products.  (No fault, trap or hang is involved anywhere.)"""
    c, _ = make_pair(max_seq=64, n_seqs=1, linear_layers=[])
    r = I.rng(31337)
    in_dim, out_dim = 4096, 5000  # more tiles than CTAs: the other CTAs take over the tile counter meanwhile
    packed, scales, biases = I.quant_weights(r, in_dim, out_dim)
    x = I.normal(r, in_dim)
    c.set_tuning("gqa_wait_spins", 200)
    c.set_tuning("matvec_inject_lost_load", 1)
    with pytest.raises(M.MfcError, match="did not arrive within the wait limit"):
        c.dequant_matvec_4bit(packed, scales, biases, in_dim, out_dim, x)
    c.set_tuning("matvec_inject_lost_load", 0)
    c.set_tuning("gqa_wait_spins", 0)
    c.synchronize()  # the report was cleared with the failed call
    ref = O.dequant_matvec_4bit(packed, scales, biases, in_dim, out_dim, x)
    for _ in range(2):
        assert I.rel_err(c.dequant_matvec_4bit(packed, scales, biases, in_dim, out_dim, x), ref) <= 1e-5
    x2 = I.normal(r, (3, in_dim))
    got = c.dequant_matvec_4bit(packed, scales, biases, in_dim, out_dim, x2)
    for v in range(3):
        assert I.rel_err(got[v], O.dequant_matvec_4bit(packed, scales, biases, in_dim, out_dim, x2[v])) <= 1e-5
    c.check_guards()
    c.close()
