"""Host-memory twin of the attention slice of ``RsCtx``, built from the oracle
functions: the checker that the GPU context is driven against, call for call.

TEST INFRASTRUCTURE ONLY (see oracle/__init__.py).
State semantics: crates/moeflux/src/riir/state.rs:37-74 (KvCache), :336-362
(LinearAttnState), :417-473 (clear_all / truncate / pos_max).
"""
from __future__ import annotations

import numpy as np

from . import (A17B, Geometry, full_attn_step, linear_attn_step, round_bf16)
from . import snapshot as snap


class OracleCtx:
    def __init__(self, g: Geometry = A17B, max_seq: int = 8192, n_seqs: int = 1, kv_bf16: bool = False,
                 snapshot_version: int = 1):
        self.g = g
        self.max_seq = max_seq
        self.n_seqs = n_seqs
        self.kv_bf16 = kv_bf16
        self.snapshot_version = snapshot_version
        self.weights = {}
        self.k = {}
        self.v = {}
        self.len = {}
        self.conv = {}
        self.ssm = {}
        for s in range(n_seqs):
            for i in range(g.num_layers):
                if g.is_full_layer(i):
                    self.len[(i, s)] = 0
                else:
                    self.conv[(i, s)] = np.zeros((3, g.conv_dim), np.float32)
                    self.ssm[(i, s)] = np.zeros(g.ssm_elems, np.float32)

    def _kv(self, layer, seq):
        key = (layer, seq)
        if key not in self.k:  # allocated lazily: host memory only for layers that are used
            self.k[key] = np.zeros((self.max_seq, self.g.kv_dim), np.float32)
            self.v[key] = np.zeros((self.max_seq, self.g.kv_dim), np.float32)
        return self.k[key], self.v[key]

    def set_linear_weights(self, layer, conv_w_bits, a_log, dt_bias_bits, norm_w_bits=None):
        self.weights[layer] = (np.array(conv_w_bits, np.uint16), np.array(a_log, np.float32),
                               np.array(dt_bias_bits, np.uint16),
                               None if norm_w_bits is None else np.array(norm_w_bits, np.uint16))

    def full_attn_step(self, layer, seq, pos, q, gate, k, v):
        if not self.g.is_full_layer(layer):
            raise ValueError("not a full-attention layer")
        ln = self.len[(layer, seq)]
        if pos != ln or pos + 1 > self.max_seq:
            raise ValueError("pos must equal the current length")
        kc, vc = self._kv(layer, seq)
        out = full_attn_step(pos, ln, q, gate, k, v, kc, vc, self.g, self.kv_bf16)
        self.len[(layer, seq)] = ln + 1
        return out

    def load_kv(self, layer, seq, K, V):
        """Test helper: install cache contents directly (rows already post-RoPE)."""
        kc, vc = self._kv(layer, seq)
        n = K.shape[0]
        kc[:n] = round_bf16(K) if self.kv_bf16 else K
        vc[:n] = round_bf16(V) if self.kv_bf16 else V
        self.len[(layer, seq)] = n

    def linear_attn_step(self, layer, seq, qkv, z, alpha, beta):
        if self.g.is_full_layer(layer):
            raise ValueError("not a linear-attention layer")
        cw, al, dt, nw = self.weights[layer]
        return linear_attn_step(qkv, z, alpha, beta, cw, al, dt, nw, self.conv[(layer, seq)],
                                self.ssm[(layer, seq)], self.g)

    # ---- state.rs:417-473 -------------------------------------------------
    def memory_clear(self, seq=-1):
        self.memory_seq_rm(seq, 0, -1)

    def memory_seq_rm(self, seq, p0, p1):
        seqs = range(self.n_seqs) if seq < 0 else [seq]
        new_len = max(p0, 0)
        for s in seqs:
            for i in range(self.g.num_layers):
                if self.g.is_full_layer(i):
                    ln = self.len[(i, s)]
                    eff_end = ln if (p1 < 0 or p1 > ln) else p1
                    to = min(new_len, eff_end)
                    if to <= ln:
                        self.len[(i, s)] = to
                else:
                    self.conv[(i, s)][:] = 0
                    self.ssm[(i, s)][:] = 0
        return True

    def memory_seq_pos_max(self, seq=0):
        return max([self.len[(i, seq)] for i in range(self.g.num_layers) if self.g.is_full_layer(i)], default=-1)

    # ---- snapshots -----------------------------------------------------------
    def _layers(self, seq):
        out = []
        for i in range(self.g.num_layers):
            if self.g.is_full_layer(i):
                ln = self.len[(i, seq)]
                if ln:
                    kc, vc = self._kv(i, seq)
                    out.append(("full", kc[:ln], vc[:ln]))
                else:
                    z = np.zeros((0, self.g.kv_dim), np.float32)
                    out.append(("full", z, z))
            else:
                out.append(("linear", self.conv[(i, seq)], self.ssm[(i, seq)]))
        return out

    def state_size(self, seq=0):
        lens = [self.len[(i, seq)] for i in range(self.g.num_layers) if self.g.is_full_layer(i)]
        return snap.state_size(self.g, lens, self.snapshot_version)

    def state_save(self, seq=0) -> bytes:
        return snap.state_save(self.g, self._layers(seq), self.snapshot_version)

    def state_load(self, seq, data: bytes):
        layers = snap.state_load(self.g, data, self.max_seq)  # raises before any mutation
        for i, lay in enumerate(layers):
            if lay[0] == "full":
                n = lay[1].shape[0]
                if n:
                    self.load_kv(i, seq, lay[1], lay[2])
                else:
                    self.len[(i, seq)] = 0
            else:
                self.conv[(i, seq)][:] = lay[1]
                self.ssm[(i, seq)][:] = lay[2]
