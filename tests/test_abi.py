"""The C-ABI library loads without a GPU, exports every symbol the header
declares, and refuses to compute without a device.  Host-only helpers (KV
split arithmetic, snapshot validation) are checked against the oracle."""
import ctypes as C
import os
import re
import struct

import numpy as np
import pytest

import moeflux_b200 as M
from moeflux_b200._lib import SIGNATURES, Config
from oracle import A17B as G
from oracle import snapshot as snap

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _header_symbols():
    text = open(os.path.join(ROOT, "include", "moeflux_cuda.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(mfc_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    L = M.lib()
    names = _header_symbols()
    assert len(names) >= 25
    for n in names:
        assert hasattr(L, n), f"{n} declared in moeflux_cuda.h but not exported"
    assert sorted(SIGNATURES) == names, "python binding and header disagree"


def test_default_config_is_a17b():
    cfg = Config()
    M.lib().mfc_default_config(C.byref(cfg))
    assert (cfg.num_layers, cfg.full_attn_interval, cfg.num_attn_heads, cfg.num_kv_heads, cfg.head_dim) == (
        G.num_layers, G.full_attn_interval, G.num_attn_heads, G.num_kv_heads, G.head_dim)
    assert (cfg.linear_num_v_heads, cfg.linear_num_k_heads, cfg.rotary_dim) == (64, 16, 64)
    assert cfg.rope_theta == 1.0e7 and abs(cfg.rms_norm_eps - 1e-6) < 1e-12


def test_open_fails_loudly_without_gpu_or_on_bad_geometry():
    import torch

    if not torch.cuda.is_available():
        with pytest.raises(M.MfcError, match="no CUDA device"):
            M.Ctx()
    L = M.lib()
    cfg = Config()
    L.mfc_default_config(C.byref(cfg))
    cfg.head_dim = 128
    assert not L.mfc_open(C.byref(cfg))
    assert b"head" in L.mfc_last_error(None) or b"CUDA" in L.mfc_last_error(None)
    assert not L.mfc_open(None)


def test_null_context_conventions():
    # moeflux.h: state_size 0 on NULL, seq_rm 0 (= failure), pos_max -1, save -1
    L = M.lib()
    assert L.mfc_state_size(None, 0) == 0
    assert L.mfc_memory_seq_rm(None, 0, 0, -1) == 0
    assert L.mfc_memory_seq_pos_max(None, 0) == -1
    assert L.mfc_state_save(None, 0, None, 0) == -1
    assert L.mfc_state_load(None, 0, None, 0) == -1
    assert L.mfc_full_attn_step(None, 3, 0, 0, None, None, None, None, None) == -1
    L.mfc_memory_clear(None, 0)
    L.mfc_free(None)


@pytest.mark.parametrize("world,block", [(1, 256), (2, 256), (8, 256), (4, 32), (3, 64)])
def test_block_cyclic_split_partitions_every_position_once(world, block):
    L = M.lib()
    n = 5 * world * block + 77
    owner = np.full(n, -1)
    for r in range(world):
        rows = []
        for p in range(n):
            row = L.mfc_kv_local_row(p, r, world, block)
            if row >= 0:
                assert owner[p] == -1
                owner[p] = r
                rows.append(row)
        assert rows == list(range(len(rows))), "a rank's rows must be dense and in position order"
        for ln in (0, 1, block - 1, block, block + 1, n // 2, n):
            assert L.mfc_kv_local_len(ln, r, world, block) == int(np.sum(owner[:ln] == r))
    assert (owner >= 0).all()
    assert L.mfc_kv_local_len(10, 2, 2, 32) == -1 and L.mfc_kv_local_row(-1, 0, 1, 32) == -1


def _tiny_geometry():
    from oracle import Geometry

    return Geometry(num_layers=4, linear_num_v_heads=4, linear_num_k_heads=2)


def _cfg_for(g, max_seq=64, version=1):
    cfg = Config()
    M.lib().mfc_default_config(C.byref(cfg))
    cfg.num_layers = g.num_layers
    cfg.linear_num_v_heads = g.linear_num_v_heads
    cfg.linear_num_k_heads = g.linear_num_k_heads
    cfg.max_seq = max_seq
    cfg.snapshot_version = version
    return cfg


def _tiny_snapshot(g, ln=5, version=1):
    r = np.random.default_rng(0)
    layers = []
    for i in range(g.num_layers):
        if g.is_full_layer(i):
            layers.append(("full", r.standard_normal((ln, g.kv_dim), dtype=np.float32),
                           r.standard_normal((ln, g.kv_dim), dtype=np.float32)))
        else:
            layers.append(("linear", r.standard_normal((3, g.conv_dim), dtype=np.float32),
                           r.standard_normal(g.ssm_elems, dtype=np.float32)))
    return snap.state_save(g, layers, version), layers


@pytest.mark.parametrize("version", [1, 2])
def test_snapshot_validate_agrees_with_oracle_loader(version):
    g = _tiny_geometry()
    cfg = _cfg_for(g)
    data, layers = _tiny_snapshot(g, version=version)
    L = M.lib()
    assert len(data) == snap.state_size(g, [5], version)
    assert L.mfc_snapshot_validate(C.byref(cfg), data, len(data)) == len(data)
    back = snap.state_load(g, data)
    for a, b in zip(layers, back):
        assert all(np.array_equal(x, y) for x, y in zip(a[1:], b[1:]))

    def bad(buf):
        with pytest.raises(snap.SnapshotError):
            snap.state_load(g, buf, max_seq=64)
        assert L.mfc_snapshot_validate(C.byref(cfg), buf, len(buf)) == -1

    bad(data[:7])                                         # no header
    bad(data[:20])                                        # short header
    bad(b"XXXX" + data[4:])                               # magic
    bad(data[:4] + struct.pack("<I", 3) + data[8:])       # version
    bad(data[:8] + struct.pack("<I", 5) + data[12:])      # num_layers
    bad(data[:20] + struct.pack("<I", 128) + data[24:])   # head_dim
    bad(data[:-1])                                        # short body
    hb = (8 if version == 1 else 10) * 4
    off = hb + 3 * ((g.conv_kernel_size - 1) * g.conv_dim * 4 + g.ssm_elems * 4)
    bad(data[:off] + struct.pack("<i", -1) + data[off + 4:])   # negative length
    bad(data[:off] + struct.pack("<i", 65) + data[off + 4:])   # beyond max_seq
    bad(data[:off] + struct.pack("<i", 6) + data[off + 4:])    # length larger than the body holds
