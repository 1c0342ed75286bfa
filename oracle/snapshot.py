"""'MFLX' snapshot wire format, restated from
crates/moeflux/src/riir/state_snapshot.rs:1-73 (layout), :195-232 (size),
:236-365 (save), :367-663 (load: header checks, preflight walk, restore).

TEST INFRASTRUCTURE ONLY (see oracle/__init__.py).  Byte work in numpy/struct.
"""
from __future__ import annotations

import struct

import numpy as np

from . import Geometry, A17B

MAGIC = 0x4D464C58
MAX_SEQ_LEN = 1_048_576  # crates/moeflux/src/riir/variants.rs:377


class SnapshotError(ValueError):
    pass


def _conv_bytes(g: Geometry) -> int:
    return (g.conv_kernel_size - 1) * g.conv_dim * 4


def _ssm_bytes(g: Geometry) -> int:
    return g.ssm_elems * 4


def header(g: Geometry, version: int) -> bytes:
    words = [MAGIC, version, g.num_layers, g.full_attn_interval, g.num_kv_heads, g.head_dim,
             _conv_bytes(g), _ssm_bytes(g)]
    if version == 2:
        words += [0, 0]  # kv_lora_rank, qk_rope_head_dim: 0 for GQA variants
    return struct.pack("<%dI" % len(words), *words)


def state_size(g: Geometry, kv_lens, version: int = 1) -> int:
    """kv_lens: length of every full-attention layer, in layer order."""
    n = (8 if version == 1 else 10) * 4
    it = iter(kv_lens)
    for i in range(g.num_layers):
        if g.is_full_layer(i):
            n += 4 + 2 * max(int(next(it)), 0) * g.kv_dim * 4
        else:
            n += _conv_bytes(g) + _ssm_bytes(g)
    return n


def state_save(g: Geometry, layers, version: int = 1) -> bytes:
    """layers[i] is ("full", K[len, kv_dim], V[len, kv_dim]) or
    ("linear", conv_state[3, conv_dim], ssm_state[v_heads, value, key])."""
    out = [header(g, version)]
    for i in range(g.num_layers):
        kind = layers[i][0]
        if g.is_full_layer(i):
            assert kind == "full"
            K = np.ascontiguousarray(layers[i][1], np.float32).reshape(-1, g.kv_dim)
            V = np.ascontiguousarray(layers[i][2], np.float32).reshape(-1, g.kv_dim)
            out.append(struct.pack("<i", K.shape[0]))
            out.append(K.tobytes())
            out.append(V.tobytes())
        else:
            assert kind == "linear"
            out.append(np.ascontiguousarray(layers[i][1], np.float32).reshape(3, g.conv_dim).tobytes())
            out.append(np.ascontiguousarray(layers[i][2], np.float32).reshape(-1).tobytes())
    return b"".join(out)


def state_load(g: Geometry, data: bytes, max_seq: int = MAX_SEQ_LEN):
    """Returns the layers list of state_save.  Raises SnapshotError exactly where
    the reference's loader rejects (before it mutates anything)."""
    if len(data) < 8:
        raise SnapshotError("truncated: no header")
    magic, version = struct.unpack_from("<II", data, 0)
    if magic != MAGIC:
        raise SnapshotError("bad magic")
    if version not in (1, 2):
        raise SnapshotError("bad version")
    hwords = 8 if version == 1 else 10
    if len(data) < hwords * 4:
        raise SnapshotError("truncated: short header")
    words = struct.unpack_from("<%dI" % hwords, data, 0)
    want = struct.unpack("<%dI" % hwords, header(g, version))
    if words[2:] != want[2:]:
        raise SnapshotError("shape mismatch")
    q = hwords * 4
    for i in range(g.num_layers):  # preflight
        if g.is_full_layer(i):
            if len(data) - q < 4:
                raise SnapshotError("truncated at layer %d" % i)
            (ln,) = struct.unpack_from("<i", data, q)
            q += 4
            if ln < 0:
                raise SnapshotError("negative length")
            if ln > max_seq:
                raise SnapshotError("length overflow")
            need = 2 * ln * g.kv_dim * 4
        else:
            need = _conv_bytes(g) + _ssm_bytes(g)
        if len(data) - q < need:
            raise SnapshotError("truncated at layer %d" % i)
        q += need
    layers = []
    off = hwords * 4
    for i in range(g.num_layers):
        if g.is_full_layer(i):
            (ln,) = struct.unpack_from("<i", data, off)
            off += 4
            nb = ln * g.kv_dim * 4
            K = np.frombuffer(data, np.float32, ln * g.kv_dim, off).reshape(ln, g.kv_dim).copy()
            off += nb
            V = np.frombuffer(data, np.float32, ln * g.kv_dim, off).reshape(ln, g.kv_dim).copy()
            off += nb
            layers.append(("full", K, V))
        else:
            cs = np.frombuffer(data, np.float32, 3 * g.conv_dim, off).reshape(3, g.conv_dim).copy()
            off += _conv_bytes(g)
            ss = np.frombuffer(data, np.float32, g.ssm_elems, off).copy()
            off += _ssm_bytes(g)
            layers.append(("linear", cs, ss))
    return layers
