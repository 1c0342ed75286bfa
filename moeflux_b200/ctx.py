"""``Ctx``: host-side mirror of the attention slice of ``RsCtx``
(crates/moeflux/src/riir/mod.rs: eval_token :1218, memory_clear :1950,
memory_seq_rm :1989, memory_seq_pos_max :2105, state_size :2113, state_save
:2125, state_load :2156), calling the C ABI.  Arrays are numpy float32 on the
host, or raw device pointers (ints, e.g. ``tensor.data_ptr()``) for ``*_dev``.
"""
from __future__ import annotations

import ctypes as C
import weakref
from typing import Optional, Sequence

import numpy as np

from ._lib import Config, MfcError, lib, KV_F32, KV_BF16

_F = C.POINTER(C.c_float)
_I = C.POINTER(C.c_int32)
_U16 = C.POINTER(C.c_uint16)


def _f32(a, n: Optional[int] = None, name: str = "array"):
    a = np.ascontiguousarray(a, dtype=np.float32)
    if n is not None and a.size != n:
        raise ValueError(f"{name}: expected {n} float32 values, got {a.size}")
    return a


def _fp(a):
    return a.ctypes.data_as(_F)


def _i32(a):
    a = np.ascontiguousarray(a, dtype=np.int32)
    return a, a.ctypes.data_as(_I)


def _u16(a, n: int, name: str):
    a = np.ascontiguousarray(a, dtype=np.uint16)
    if a.size != n:
        raise ValueError(f"{name}: expected {n} bf16 values, got {a.size}")
    return a


_LIVE = weakref.WeakSet()


def live_contexts():
    """The contexts of this process that are open (e.g. to verify their guard bands after a test)."""
    return [c for c in list(_LIVE) if getattr(c, "_h", None)]


class Ctx:
    """One attention backend context on one GPU."""

    def __init__(self, **overrides):
        L = lib()
        cfg = Config()
        L.mfc_default_config(C.byref(cfg))
        explicit_batch = "max_batch" in overrides
        for k, v in overrides.items():
            if not hasattr(cfg, k):
                raise TypeError(f"unknown config field {k!r}")
            setattr(cfg, k, v)
        if not explicit_batch:
            cfg.max_batch = cfg.num_layers * cfg.n_seqs
        self._lib = L
        self._h = L.mfc_open(C.byref(cfg))
        if not self._h:
            raise MfcError("mfc_open failed: " + L.mfc_last_error(None).decode())
        self.cfg = Config()
        L.mfc_get_config(self._h, C.byref(self.cfg))
        g = self.cfg
        self.q_dim = g.num_attn_heads * g.head_dim
        self.kv_dim = g.num_kv_heads * g.head_dim
        self.v_heads = g.linear_num_v_heads
        self.total_value = g.linear_num_v_heads * g.linear_value_dim
        self.conv_dim = 2 * g.linear_num_k_heads * g.linear_key_dim + self.total_value
        self.ssm_elems = g.linear_num_v_heads * g.linear_value_dim * g.linear_key_dim
        _LIVE.add(self)

    # -- lifetime -------------------------------------------------------
    def close(self):
        if getattr(self, "_h", None):
            self._lib.mfc_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def _check(self, rc, what):
        if rc != 0:
            raise MfcError(f"{what}: {self._lib.mfc_last_error(self._h).decode()}")

    def is_full_layer(self, layer: int) -> bool:
        return (layer + 1) % self.cfg.full_attn_interval == 0

    @property
    def stream(self) -> int:
        return int(self._lib.mfc_stream(self._h) or 0)

    @property
    def side_stream(self) -> int:
        """The context's second queue (GatedDeltaNet launches with the tuning "gdn_side_queue")."""
        return int(self._lib.mfc_side_stream(self._h) or 0)

    def set_stream(self, stream: int):
        """Issue all further work on the caller's stream (e.g. ``torch.cuda.Stream().cuda_stream``)."""
        self._check(self._lib.mfc_set_stream(self._h, stream or None), "mfc_set_stream")

    def synchronize(self):
        self._check(self._lib.mfc_synchronize(self._h), "mfc_synchronize")

    def set_tuning(self, key: str, value: int):
        self._check(self._lib.mfc_set_tuning(self._h, key.encode(), int(value)), f"mfc_set_tuning({key})")

    def join(self):
        """Make ``self.stream`` wait for a GatedDeltaNet launch issued on the side queue."""
        self._check(self._lib.mfc_join(self._h), "mfc_join")

    @property
    def launch_count(self) -> int:
        return int(self._lib.mfc_launch_count(self._h))

    def check_guards(self):
        """Raises when a kernel wrote into the guard bands around one of the context's device allocations."""
        self._check(self._lib.mfc_check_guards(self._h), "mfc_check_guards")

    def read_phase_trace(self, max_ctas: int = 1024) -> np.ndarray:
        """[ctas][8] uint64 nanosecond stamps of the last decode launch made with the tuning "gqa_phase_trace"."""
        out = np.zeros((max_ctas, 8), np.uint64)
        n = self._lib.mfc_read_phase_trace(self._h, out.ctypes.data, max_ctas)
        if n < 0:
            raise MfcError("mfc_read_phase_trace: " + self._lib.mfc_last_error(self._h).decode())
        return out[:n]

    # -- KV-sequence split: exchange fused into the decode kernel ---------------------
    def exchange_create(self, items_per_rank: int) -> bytes:
        """Allocates this rank's receive buffers; returns the 64-byte CUDA IPC handle the other ranks need."""
        h = (C.c_ubyte * 64)()
        self._check(self._lib.mfc_exchange_create(self._h, items_per_rank, h), "mfc_exchange_create")
        return bytes(h)

    def exchange_connect(self, handles: Sequence[bytes]):
        """``handles``: the IPC handles of all ranks, in rank order (this rank's own entry is ignored)."""
        blob = b"".join(bytes(h) for h in handles)
        buf = (C.c_ubyte * len(blob)).from_buffer_copy(blob)
        self._check(self._lib.mfc_exchange_connect(self._h, buf), "mfc_exchange_connect")

    def exchange_connect_local(self, peers: Sequence["Ctx"]):
        """Same, for contexts that live in this process (one per rank, in rank order)."""
        tab = (C.c_void_p * len(peers))(*[p._h for p in peers])
        self._check(self._lib.mfc_exchange_connect_local(self._h, tab), "mfc_exchange_connect_local")

    def full_attn_partial_exchange_dev(self, layers, seq_ids, pos, q_ptr, k_ptr, v_ptr):
        la, lp = _i32(layers)
        sa, sp = _i32(seq_ids)
        pa, pp = _i32(pos)
        rc = self._lib.mfc_full_attn_partial_exchange_dev(self._h, la.size, lp, sp, pp, q_ptr, k_ptr, v_ptr)
        self._check(rc, "mfc_full_attn_partial_exchange_dev")

    def lse_merge_gate_exchange_dev(self, gate_ptr, out_ptr):
        self._check(self._lib.mfc_lse_merge_gate_exchange_dev(self._h, gate_ptr or None, out_ptr),
                    "mfc_lse_merge_gate_exchange_dev")

    # -- weights --------------------------------------------------------
    def set_linear_weights(self, layer: int, conv_w_bf16, a_log, dt_bias_bf16, norm_w_bf16=None):
        g = self.cfg
        cw = _u16(conv_w_bf16, self.conv_dim * g.conv_kernel_size, "conv_w_bf16")
        al = _f32(a_log, g.linear_num_v_heads, "a_log")
        dt = _u16(dt_bias_bf16, g.linear_num_v_heads, "dt_bias_bf16")
        nw = None if norm_w_bf16 is None else _u16(norm_w_bf16, g.linear_value_dim, "norm_w_bf16")
        rc = self._lib.mfc_set_linear_weights(
            self._h, layer, cw.ctypes.data_as(_U16), _fp(al), dt.ctypes.data_as(_U16),
            None if nw is None else nw.ctypes.data_as(_U16))
        self._check(rc, "mfc_set_linear_weights")

    def set_full_attn_norm_weights(self, layer: int, q_norm_bf16, k_norm_bf16):
        g = self.cfg
        qn = _u16(q_norm_bf16, g.head_dim, "q_norm_bf16")
        kn = _u16(k_norm_bf16, g.head_dim, "k_norm_bf16")
        rc = self._lib.mfc_set_full_attn_norm_weights(self._h, layer, qn.ctypes.data_as(_U16), kn.ctypes.data_as(_U16))
        self._check(rc, "mfc_set_full_attn_norm_weights")

    def full_attn_step_qproj_batched(self, layers, seq_ids, pos, q_proj, k, v) -> np.ndarray:
        """q_proj: [n][heads][q | gate] as the q projection emits it; de-interleave and the
        per-head q/k RMSNorm run inside the attention kernel."""
        la, lp = _i32(layers)
        sa, sp = _i32(seq_ids)
        pa, pp = _i32(pos)
        n = la.size
        qp = _f32(q_proj, 2 * n * self.q_dim, "q_proj")
        k = _f32(k, n * self.kv_dim, "k")
        v = _f32(v, n * self.kv_dim, "v")
        out = np.empty((n, self.q_dim), np.float32)
        rc = self._lib.mfc_full_attn_step_qproj_batched(self._h, n, lp, sp, pp, _fp(qp), _fp(k), _fp(v), _fp(out))
        self._check(rc, "mfc_full_attn_step_qproj_batched")
        return out

    # -- hot path, host arrays -------------------------------------------
    def full_attn_step(self, layer: int, seq_id: int, pos: int, q, gate, k, v) -> np.ndarray:
        q = _f32(q, self.q_dim, "q")
        gate = _f32(gate, self.q_dim, "gate")
        k = _f32(k, self.kv_dim, "k")
        v = _f32(v, self.kv_dim, "v")
        out = np.empty(self.q_dim, np.float32)
        rc = self._lib.mfc_full_attn_step(self._h, layer, seq_id, pos, _fp(q), _fp(gate), _fp(k), _fp(v), _fp(out))
        self._check(rc, "mfc_full_attn_step")
        return out

    def linear_attn_step(self, layer: int, seq_id: int, qkv, z, alpha, beta) -> np.ndarray:
        qkv = _f32(qkv, self.conv_dim, "qkv")
        z = None if z is None else _f32(z, self.total_value, "z")
        alpha = _f32(alpha, self.v_heads, "alpha")
        beta = _f32(beta, self.v_heads, "beta")
        out = np.empty(self.total_value, np.float32)
        rc = self._lib.mfc_linear_attn_step(self._h, layer, seq_id, _fp(qkv), None if z is None else _fp(z),
                                            _fp(alpha), _fp(beta), _fp(out))
        self._check(rc, "mfc_linear_attn_step")
        return out

    def full_attn_step_batched(self, layers, seq_ids, pos, q, gate, k, v, out=None) -> np.ndarray:
        la, lp = _i32(layers)
        sa, sp = _i32(seq_ids)
        pa, pp = _i32(pos)
        n = la.size
        q = _f32(q, n * self.q_dim, "q")
        gate = _f32(gate, n * self.q_dim, "gate")
        k = _f32(k, n * self.kv_dim, "k")
        v = _f32(v, n * self.kv_dim, "v")
        if out is None:
            out = np.empty((n, self.q_dim), np.float32)
        rc = self._lib.mfc_full_attn_step_batched(self._h, n, lp, sp, pp, _fp(q), _fp(gate), _fp(k), _fp(v), _fp(out))
        self._check(rc, "mfc_full_attn_step_batched")
        return out

    def linear_attn_step_batched(self, layers, seq_ids, qkv, z, alpha, beta, out=None) -> np.ndarray:
        la, lp = _i32(layers)
        sa, sp = _i32(seq_ids)
        n = la.size
        qkv = _f32(qkv, n * self.conv_dim, "qkv")
        z = None if z is None else _f32(z, n * self.total_value, "z")
        alpha = _f32(alpha, n * self.v_heads, "alpha")
        beta = _f32(beta, n * self.v_heads, "beta")
        if out is None:
            out = np.empty((n, self.total_value), np.float32)
        rc = self._lib.mfc_linear_attn_step_batched(self._h, n, lp, sp, _fp(qkv), None if z is None else _fp(z),
                                                    _fp(alpha), _fp(beta), _fp(out))
        self._check(rc, "mfc_linear_attn_step_batched")
        return out

    # raw-pointer forms of the two batched host calls (pinned buffers, no numpy work per call)
    def full_attn_step_batched_ptr(self, n, layers_p, seqs_p, pos_p, q_p, gate_p, k_p, v_p, out_p):
        rc = self._lib.mfc_full_attn_step_batched(self._h, n, C.cast(layers_p, _I), C.cast(seqs_p, _I),
                                                  C.cast(pos_p, _I), C.cast(q_p, _F), C.cast(gate_p, _F),
                                                  C.cast(k_p, _F), C.cast(v_p, _F), C.cast(out_p, _F))
        self._check(rc, "mfc_full_attn_step_batched")

    def full_attn_step_batched_dev_ptr(self, n, layers_p, seqs_p, pos_p, q_ptr, gate_ptr, k_ptr, v_ptr, out_ptr):
        """``mfc_full_attn_step_batched_dev`` with the three host tables given as addresses of int32 arrays the
        caller keeps (no per-call conversions: for loops whose step is tens of microseconds)."""
        rc = self._lib.mfc_full_attn_step_batched_dev(self._h, n, C.cast(layers_p, _I), C.cast(seqs_p, _I),
                                                      C.cast(pos_p, _I), q_ptr, gate_ptr, k_ptr, v_ptr, out_ptr)
        self._check(rc, "mfc_full_attn_step_batched_dev")

    def linear_attn_step_batched_dev_ptr(self, n, layers_p, seqs_p, qkv_ptr, z_ptr, alpha_ptr, beta_ptr, out_ptr):
        """``mfc_linear_attn_step_batched_dev`` with the two host tables given as addresses of int32 arrays the
        caller keeps (no per-call conversions)."""
        rc = self._lib.mfc_linear_attn_step_batched_dev(self._h, n, C.cast(layers_p, _I), C.cast(seqs_p, _I), qkv_ptr,
                                                        z_ptr or None, alpha_ptr, beta_ptr, out_ptr)
        self._check(rc, "mfc_linear_attn_step_batched_dev")

    def linear_attn_step_batched_ptr(self, n, layers_p, seqs_p, qkv_p, z_p, alpha_p, beta_p, out_p):
        rc = self._lib.mfc_linear_attn_step_batched(self._h, n, C.cast(layers_p, _I), C.cast(seqs_p, _I),
                                                    C.cast(qkv_p, _F), C.cast(z_p, _F) if z_p else None,
                                                    C.cast(alpha_p, _F), C.cast(beta_p, _F), C.cast(out_p, _F))
        self._check(rc, "mfc_linear_attn_step_batched")

    def eval_token_attn(self, full_items, pos, q, gate, k, v, lin_items, qkv, z, alpha, beta):
        """One token step of a layer stack's attention sub-blocks: ``full_items`` and
        ``lin_items`` are lists of (layer, seq_id).  Returns (full_out [n_full, q_dim],
        lin_out [n_lin, total_value])."""
        nf, nl = len(full_items), len(lin_items)
        fl, flp = _i32([l for l, _ in full_items] or [0])
        fs, fsp = _i32([s for _, s in full_items] or [0])
        pa, pp = _i32(list(pos) or [0])
        ll, llp = _i32([l for l, _ in lin_items] or [0])
        ls, lsp = _i32([s for _, s in lin_items] or [0])
        fo = np.empty((nf, self.q_dim), np.float32)
        lo = np.empty((nl, self.total_value), np.float32)
        if nf:
            q, gate = _f32(q, nf * self.q_dim, "q"), _f32(gate, nf * self.q_dim, "gate")
            k, v = _f32(k, nf * self.kv_dim, "k"), _f32(v, nf * self.kv_dim, "v")
        if nl:
            qkv = _f32(qkv, nl * self.conv_dim, "qkv")
            z = None if z is None else _f32(z, nl * self.total_value, "z")
            alpha, beta = _f32(alpha, nl * self.v_heads, "alpha"), _f32(beta, nl * self.v_heads, "beta")
        P = lambda a: _fp(a) if a is not None else None
        rc = self._lib.mfc_eval_token_attn(
            self._h, nf, flp, fsp, pp, P(q) if nf else None, P(gate) if nf else None, P(k) if nf else None,
            P(v) if nf else None, _fp(fo) if nf else None, nl, llp, lsp, P(qkv) if nl else None,
            P(z) if nl else None, P(alpha) if nl else None, P(beta) if nl else None, _fp(lo) if nl else None)
        self._check(rc, "mfc_eval_token_attn")
        return fo, lo

    def eval_token_attn_split(self, full_items, pos, q, gate_own, k, v, lin_items, qkv, z, alpha, beta, n_own: int,
                              q_own: bool = False):
        """``eval_token_attn`` on a context of a KV split with its exchange connected: ``full_items`` is the whole
        step's item list sorted by finishing rank, ``gate_own`` holds the gate rows of the ``n_own`` items this rank
        finishes, and the returned full-attention outputs are those items' ([n_own, q_dim]).  ``q_own``: ``q`` holds
        the query rows of those ``n_own`` items only (the tuning "exchange_gather_q" must be 1 on every rank)."""
        nf, nl = len(full_items), len(lin_items)
        fl, flp = _i32([l for l, _ in full_items])
        fs, fsp = _i32([s for _, s in full_items])
        pa, pp = _i32(list(pos))
        ll, llp = _i32([l for l, _ in lin_items] or [0])
        ls, lsp = _i32([s for _, s in lin_items] or [0])
        q, gate_own = _f32(q, (n_own if q_own else nf) * self.q_dim, "q"), _f32(gate_own, n_own * self.q_dim, "gate_own")
        k, v = _f32(k, nf * self.kv_dim, "k"), _f32(v, nf * self.kv_dim, "v")
        fo = np.empty((n_own, self.q_dim), np.float32)
        lo = np.empty((nl, self.total_value), np.float32)
        if nl:
            qkv = _f32(qkv, nl * self.conv_dim, "qkv")
            z = None if z is None else _f32(z, nl * self.total_value, "z")
            alpha, beta = _f32(alpha, nl * self.v_heads, "alpha"), _f32(beta, nl * self.v_heads, "beta")
        P = lambda a: _fp(a) if a is not None else None
        rc = self._lib.mfc_eval_token_attn(
            self._h, nf, flp, fsp, pp, _fp(q), _fp(gate_own), _fp(k), _fp(v), _fp(fo), nl, llp, lsp,
            P(qkv) if nl else None, P(z) if nl else None, P(alpha) if nl else None, P(beta) if nl else None,
            _fp(lo) if nl else None)
        self._check(rc, "mfc_eval_token_attn")
        return fo, lo

    def eval_token_attn_ptr(self, nf, fl_p, fs_p, pos_p, q_p, gate_p, k_p, v_p, fo_p, nl, ll_p, ls_p, qkv_p, z_p,
                            alpha_p, beta_p, lo_p):
        """Raw-pointer form (pinned host buffers, no numpy work per call)."""
        F = lambda p: C.cast(p, _F) if p else None
        Ip = lambda p: C.cast(p, _I) if p else None
        rc = self._lib.mfc_eval_token_attn(self._h, nf, Ip(fl_p), Ip(fs_p), Ip(pos_p), F(q_p), F(gate_p), F(k_p),
                                           F(v_p), F(fo_p), nl, Ip(ll_p), Ip(ls_p), F(qkv_p), F(z_p), F(alpha_p),
                                           F(beta_p), F(lo_p))
        self._check(rc, "mfc_eval_token_attn")

    # -- hot path, device pointers (asynchronous on self.stream) ------------
    def full_attn_step_batched_dev(self, layers, seq_ids, pos, q_ptr, gate_ptr, k_ptr, v_ptr, out_ptr):
        la, lp = _i32(layers)
        sa, sp = _i32(seq_ids)
        pa, pp = _i32(pos)
        rc = self._lib.mfc_full_attn_step_batched_dev(self._h, la.size, lp, sp, pp, q_ptr, gate_ptr, k_ptr, v_ptr,
                                                      out_ptr)
        self._check(rc, "mfc_full_attn_step_batched_dev")

    def linear_attn_step_batched_dev(self, layers, seq_ids, qkv_ptr, z_ptr, alpha_ptr, beta_ptr, out_ptr):
        la, lp = _i32(layers)
        sa, sp = _i32(seq_ids)
        rc = self._lib.mfc_linear_attn_step_batched_dev(self._h, la.size, lp, sp, qkv_ptr, z_ptr or None, alpha_ptr,
                                                        beta_ptr, out_ptr)
        self._check(rc, "mfc_linear_attn_step_batched_dev")

    def full_attn_partial_batched_dev(self, layers, seq_ids, pos, q_ptr, k_ptr, v_ptr, o_ptr, m_ptr, l_ptr):
        la, lp = _i32(layers)
        sa, sp = _i32(seq_ids)
        pa, pp = _i32(pos)
        rc = self._lib.mfc_full_attn_partial_batched_dev(self._h, la.size, lp, sp, pp, q_ptr, k_ptr, v_ptr, o_ptr,
                                                         m_ptr, l_ptr)
        self._check(rc, "mfc_full_attn_partial_batched_dev")

    def full_attn_partial_packed_dev(self, layers, seq_ids, pos, q_ptr, k_ptr, v_ptr, packed_ptr):
        la, lp = _i32(layers)
        sa, sp = _i32(seq_ids)
        pa, pp = _i32(pos)
        rc = self._lib.mfc_full_attn_partial_packed_dev(self._h, la.size, lp, sp, pp, q_ptr, k_ptr, v_ptr, packed_ptr)
        self._check(rc, "mfc_full_attn_partial_packed_dev")

    def lse_merge_gate_packed_dev(self, n_parts, n, packed_ptr, gate_ptr, out_ptr):
        rc = self._lib.mfc_lse_merge_gate_packed_dev(self._h, n_parts, n, packed_ptr, gate_ptr or None, out_ptr)
        self._check(rc, "mfc_lse_merge_gate_packed_dev")

    def lse_merge_gate_dev(self, n_parts, n, o_ptr, m_ptr, l_ptr, gate_ptr, out_ptr, part_stride=0):
        rc = self._lib.mfc_lse_merge_gate_dev(self._h, n_parts, n, o_ptr, m_ptr, l_ptr, part_stride,
                                              gate_ptr or None, out_ptr)
        self._check(rc, "mfc_lse_merge_gate_dev")

    # -- prefill (device pointers, bf16 activations) ---------------------------
    def full_attn_prefill_dev(self, layer, seq_id, start_pos, n_tokens, q_ptr, gate_ptr, k_ptr, v_ptr, out_ptr):
        rc = self._lib.mfc_full_attn_prefill_dev(self._h, layer, seq_id, start_pos, n_tokens, q_ptr,
                                                 gate_ptr or None, k_ptr, v_ptr, out_ptr)
        self._check(rc, "mfc_full_attn_prefill_dev")

    def linear_attn_prefill_dev(self, layer, seq_id, n_tokens, qkv_ptr, z_ptr, alpha_ptr, beta_ptr, out_ptr):
        rc = self._lib.mfc_linear_attn_prefill_dev(self._h, layer, seq_id, n_tokens, qkv_ptr, z_ptr or None,
                                                   alpha_ptr, beta_ptr, out_ptr)
        self._check(rc, "mfc_linear_attn_prefill_dev")

    # -- bulk state import from device memory ------------------------------------
    def kv_append_rows_dev(self, layer, seq_id, pos0, n_rows, k_rows_ptr, v_rows_ptr):
        rc = self._lib.mfc_kv_append_rows_dev(self._h, layer, seq_id, pos0, n_rows, k_rows_ptr, v_rows_ptr)
        self._check(rc, "mfc_kv_append_rows_dev")

    def linear_state_set_dev(self, layer, seq_id, conv_ptr, ssm_ptr):
        rc = self._lib.mfc_linear_state_set_dev(self._h, layer, seq_id, conv_ptr, ssm_ptr)
        self._check(rc, "mfc_linear_state_set_dev")

    # -- sequence state -----------------------------------------------------
    def memory_clear(self, seq_id: int = -1):
        self._lib.mfc_memory_clear(self._h, seq_id)

    def memory_seq_rm(self, seq_id: int, p0: int, p1: int) -> bool:
        return self._lib.mfc_memory_seq_rm(self._h, seq_id, p0, p1) != 0

    def memory_seq_pos_max(self, seq_id: int = 0) -> int:
        return int(self._lib.mfc_memory_seq_pos_max(self._h, seq_id))

    def state_size(self, seq_id: int = 0) -> int:
        return int(self._lib.mfc_state_size(self._h, seq_id))

    def state_save(self, seq_id: int = 0) -> bytes:
        n = self.state_size(seq_id)
        buf = np.empty(n, np.uint8)
        wrote = self._lib.mfc_state_save(self._h, seq_id, buf.ctypes.data, n)
        if wrote < 0:
            raise MfcError("mfc_state_save: " + self._lib.mfc_last_error(self._h).decode())
        return buf[:wrote].tobytes()

    def state_save_into(self, seq_id: int, buf: np.ndarray) -> int:
        return int(self._lib.mfc_state_save(self._h, seq_id, buf.ctypes.data, buf.nbytes))

    def state_load(self, seq_id: int, data) -> None:
        arr = np.frombuffer(data, dtype=np.uint8)
        rc = self._lib.mfc_state_load(self._h, seq_id, arr.ctypes.data if arr.size else None, arr.size)
        self._check(rc, "mfc_state_load")

    # -- checkpoints (RsCtx::checkpoint_pos / restore_to) -------------------------
    def checkpoint_pos(self, pos: int, seq_id: int = 0):
        self._check(self._lib.mfc_checkpoint_pos(self._h, seq_id, pos), "mfc_checkpoint_pos")

    def restore_to(self, pos: int, seq_id: int = 0):
        self._check(self._lib.mfc_restore_to(self._h, seq_id, pos), "mfc_restore_to")

    def set_max_checkpoints(self, n: int):
        self._lib.mfc_set_max_checkpoints(self._h, n)

    def checkpoint_count(self, seq_id: int = 0) -> int:
        return int(self._lib.mfc_checkpoint_count(self._h, seq_id))

    # -- parity hooks ---------------------------------------------------------
    def apply_rotary_emb(self, pos: int, q, k):
        q = np.array(q, np.float32, copy=True).reshape(-1)
        k = np.array(k, np.float32, copy=True).reshape(-1)
        if q.size != self.q_dim or k.size != self.kv_dim:
            raise ValueError("apply_rotary_emb: wrong q/k length")
        self._check(self._lib.mfc_apply_rotary_emb(self._h, pos, _fp(q), _fp(k)), "mfc_apply_rotary_emb")
        return q, k

    def sdpa(self, kv_len: int, q, gate, k_cache, v_cache) -> np.ndarray:
        q = _f32(q, self.q_dim, "q")
        gate = _f32(gate, self.q_dim, "gate")
        kc = _f32(k_cache)
        vc = _f32(v_cache)
        if kv_len > 0 and (kc.size < kv_len * self.kv_dim or vc.size < kv_len * self.kv_dim):
            raise ValueError("sdpa: cache shorter than kv_len rows")
        out = np.empty(self.q_dim, np.float32)
        self._check(self._lib.mfc_sdpa(self._h, kv_len, _fp(q), _fp(gate), _fp(kc), _fp(vc), _fp(out)), "mfc_sdpa")
        return out

    # -- projections: 4-bit group-64 dequant matvec (cpu_matvec.rs:83, gpu_matvec.rs:84) ------
    def dequant_matvec_4bit(self, packed, scales, biases, in_dim: int, out_dim: int, x) -> np.ndarray:
        """out[v][r] = sum_c (nibble * scale + bias)(r, c) * x[v][c]; x is [in_dim] or [n_vec][in_dim]."""
        pk = np.ascontiguousarray(packed, dtype=np.uint32).reshape(-1)
        sc = np.ascontiguousarray(scales, dtype=np.uint16).reshape(-1)
        bi = np.ascontiguousarray(biases, dtype=np.uint16).reshape(-1)
        xv = np.ascontiguousarray(x, dtype=np.float32)
        single = xv.ndim == 1
        xv = xv.reshape(1, -1) if single else xv
        n_vec = xv.shape[0]
        if in_dim > 0 and in_dim % 64 == 0 and out_dim > 0:
            for name, got, exp in (("packed", pk.size, out_dim * in_dim // 8), ("scales", sc.size, out_dim * in_dim // 64),
                                   ("biases", bi.size, out_dim * in_dim // 64), ("x", xv.shape[1], in_dim)):
                if got != exp:
                    raise ValueError(f"slice length mismatch on '{name}': got {got} elements, expected {exp}")
        out = np.empty((n_vec, max(out_dim, 0)), np.float32)
        rc = self._lib.mfc_dequant_matvec_4bit(self._h, pk.ctypes.data, sc.ctypes.data, bi.ctypes.data, in_dim, out_dim,
                                               _fp(xv), n_vec, _fp(out))
        self._check(rc, "mfc_dequant_matvec_4bit")
        return out[0] if single else out

    def dequant_matvec_4bit_dev(self, packed_ptr, scales_ptr, biases_ptr, in_dim, out_dim, x_ptr, n_vec, out_ptr):
        rc = self._lib.mfc_dequant_matvec_4bit_dev(self._h, packed_ptr, scales_ptr, biases_ptr, in_dim, out_dim, x_ptr,
                                                   n_vec, out_ptr)
        self._check(rc, "mfc_dequant_matvec_4bit_dev")

    def dequant_matvec_4bit_multi_dev(self, packed_ptrs, scales_ptrs, biases_ptrs, in_dim, out_dims, x_ptr, n_vec, out_ptrs):
        """Up to 8 matrices of the same in_dim applied to the same x in one launch (device pointers)."""
        n = len(out_dims)
        if not (len(packed_ptrs) == len(scales_ptrs) == len(biases_ptrs) == len(out_ptrs) == n):
            raise ValueError("dequant_matvec_4bit_multi_dev: tables of different length")
        tab = lambda ptrs: (C.c_void_p * n)(*[int(p) for p in ptrs])
        dims = (C.c_int32 * n)(*[int(d) for d in out_dims])
        rc = self._lib.mfc_dequant_matvec_4bit_multi_dev(self._h, n, tab(packed_ptrs), tab(scales_ptrs), tab(biases_ptrs),
                                                         in_dim, dims, x_ptr, n_vec, tab(out_ptrs))
        self._check(rc, "mfc_dequant_matvec_4bit_multi_dev")

    # -- folded MLA attention (shaders.metal:1717-1987, gpu_mla.rs:146-274) -------------------------
    def mla_sdpa_folded(self, cache_len: int, softmax_scale: float, q_prime, q_pe, latent_cache, rope_k_cache) -> np.ndarray:
        """v_combine [num_heads, 512] for q_prime [num_heads, 512], q_pe [num_heads, 64] over the first cache_len rows
        of latent_cache [., 512] and rope_k_cache [., 64] (host arrays)."""
        qp = np.ascontiguousarray(q_prime, np.float32)
        H = qp.size // 512
        qp = _f32(qp, H * 512, "q_prime")
        pe = _f32(q_pe, H * 64, "q_pe")
        lat = _f32(latent_cache)
        rk = _f32(rope_k_cache)
        if cache_len > 0 and (lat.size < cache_len * 512 or rk.size < cache_len * 64):
            raise ValueError("mla_sdpa_folded: cache shorter than cache_len rows")
        out = np.empty((H, 512), np.float32)
        rc = self._lib.mfc_mla_sdpa_folded(self._h, H, cache_len, softmax_scale, _fp(qp), _fp(pe), _fp(lat), _fp(rk),
                                           _fp(out))
        self._check(rc, "mfc_mla_sdpa_folded")
        return out

    def mla_sdpa_folded_dev(self, num_heads, cache_len, softmax_scale, q_prime_ptr, q_pe_ptr, latent_ptr, rope_k_ptr,
                            out_ptr):
        rc = self._lib.mfc_mla_sdpa_folded_dev(self._h, num_heads, cache_len, softmax_scale, q_prime_ptr, q_pe_ptr,
                                               latent_ptr, rope_k_ptr, out_ptr)
        self._check(rc, "mfc_mla_sdpa_folded_dev")

    def mla_sdpa_folded_bf16_dev(self, num_heads, cache_len, softmax_scale, q_prime_ptr, q_pe_ptr, latent_bf16_ptr,
                                 rope_k_bf16_ptr, out_ptr):
        rc = self._lib.mfc_mla_sdpa_folded_bf16_dev(self._h, num_heads, cache_len, softmax_scale, q_prime_ptr, q_pe_ptr,
                                                    latent_bf16_ptr, rope_k_bf16_ptr, out_ptr)
        self._check(rc, "mfc_mla_sdpa_folded_bf16_dev")

    def linear_attn_step_stateless(self, layer: int, qkv, z, alpha, beta, conv_state, ssm_state):
        """Returns (out, new_conv_state, new_ssm_state); inputs are not modified."""
        qkv = _f32(qkv, self.conv_dim, "qkv")
        z = None if z is None else _f32(z, self.total_value, "z")
        alpha = _f32(alpha, self.v_heads, "alpha")
        beta = _f32(beta, self.v_heads, "beta")
        cs = np.array(conv_state, np.float32, copy=True).reshape(-1)
        ss = np.array(ssm_state, np.float32, copy=True).reshape(-1)
        if cs.size != 3 * self.conv_dim or ss.size != self.ssm_elems:
            raise ValueError("linear_attn_step_stateless: wrong state size")
        out = np.empty(self.total_value, np.float32)
        rc = self._lib.mfc_linear_attn_step_stateless(self._h, layer, _fp(qkv), None if z is None else _fp(z),
                                                      _fp(alpha), _fp(beta), _fp(cs), _fp(ss), _fp(out))
        self._check(rc, "mfc_linear_attn_step_stateless")
        return out, cs, ss


def sdpa_static_dev(num_attn_heads: int, num_kv_heads: int, kv_dtype: int, kv_len: int, cap_rows: int,
                    q_ptr: int, gate_ptr: int, k_cache_ptr: int, v_cache_ptr: int, out_ptr: int, stream: int = 0):
    """``mfc_sdpa_static_dev``: gated SDPA over a caller-held device cache
    ``[num_kv_heads][cap_rows][256]`` with every working byte taken from a fixed
    array inside the library, for callers that cannot allocate device memory
    (no context is needed, and none is created).  Asynchronous on ``stream``;
    calls that may overlap on the GPU race on the shared array."""
    L = lib()
    rc = L.mfc_sdpa_static_dev(num_attn_heads, num_kv_heads, kv_dtype, kv_len, cap_rows, q_ptr, gate_ptr or None,
                               k_cache_ptr, v_cache_ptr, out_ptr, stream or None)
    if rc != 0:
        raise MfcError("mfc_sdpa_static_dev: " + L.mfc_last_error(None).decode())


def sdpa_static_status(stream: int = 0):
    """``mfc_sdpa_static_status``: waits for ``stream`` and raises when a kernel of the calls since the previous
    status call gave up (its outputs are then not valid).  Allocates nothing."""
    L = lib()
    if L.mfc_sdpa_static_status(stream or None) != 0:
        raise MfcError("mfc_sdpa_static_status: " + L.mfc_last_error(None).decode())
