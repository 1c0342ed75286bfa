"""ctypes binding of ``libmoeflux_cuda.so`` (declarations of include/moeflux_cuda.h)."""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libmoeflux_cuda.so")

KV_F32 = 0
KV_BF16 = 1


class MfcError(RuntimeError):
    """An entry point of the C ABI reported failure."""


class Config(C.Structure):
    """``mfc_config``; field meaning as in ``Variant``
    (crates/moeflux/src/riir/variants.rs:132-250)."""

    _fields_ = [
        ("num_layers", C.c_int32),
        ("full_attn_interval", C.c_int32),
        ("num_attn_heads", C.c_int32),
        ("num_kv_heads", C.c_int32),
        ("head_dim", C.c_int32),
        ("rotary_dim", C.c_int32),
        ("rope_theta", C.c_float),
        ("linear_num_v_heads", C.c_int32),
        ("linear_num_k_heads", C.c_int32),
        ("linear_key_dim", C.c_int32),
        ("linear_value_dim", C.c_int32),
        ("conv_kernel_size", C.c_int32),
        ("rms_norm_eps", C.c_float),
        ("kv_dtype", C.c_int32),
        ("max_seq", C.c_int32),
        ("n_seqs", C.c_int32),
        ("device", C.c_int32),
        ("kv_rank", C.c_int32),
        ("kv_world", C.c_int32),
        ("kv_block", C.c_int32),
        ("max_batch", C.c_int32),
        ("snapshot_version", C.c_int32),
        ("max_prefill", C.c_int32),
    ]


_F = C.POINTER(C.c_float)
_I = C.POINTER(C.c_int32)
_U16 = C.POINTER(C.c_uint16)
_P = C.c_void_p

# name -> (restype, argtypes); every symbol the header declares
SIGNATURES = {
    "mfc_default_config": (None, [C.POINTER(Config)]),
    "mfc_open": (_P, [C.POINTER(Config)]),
    "mfc_free": (None, [_P]),
    "mfc_last_error": (C.c_char_p, [_P]),
    "mfc_get_config": (C.c_int, [_P, C.POINTER(Config)]),
    "mfc_stream": (_P, [_P]),
    "mfc_side_stream": (_P, [_P]),
    "mfc_set_stream": (C.c_int, [_P, _P]),
    "mfc_synchronize": (C.c_int, [_P]),
    "mfc_set_linear_weights": (C.c_int, [_P, C.c_int32, _U16, _F, _U16, _U16]),
    "mfc_set_full_attn_norm_weights": (C.c_int, [_P, C.c_int32, _U16, _U16]),
    "mfc_full_attn_step_qproj_batched": (C.c_int, [_P, C.c_int32, _I, _I, _I, _F, _F, _F, _F]),
    "mfc_full_attn_step_qproj_batched_dev": (C.c_int, [_P, C.c_int32, _I, _I, _I, _P, _P, _P, _P]),
    "mfc_full_attn_step": (C.c_int, [_P, C.c_int32, C.c_int32, C.c_int32, _F, _F, _F, _F, _F]),
    "mfc_linear_attn_step": (C.c_int, [_P, C.c_int32, C.c_int32, _F, _F, _F, _F, _F]),
    "mfc_full_attn_step_batched": (C.c_int, [_P, C.c_int32, _I, _I, _I, _F, _F, _F, _F, _F]),
    "mfc_linear_attn_step_batched": (C.c_int, [_P, C.c_int32, _I, _I, _F, _F, _F, _F, _F]),
    "mfc_eval_token_attn": (C.c_int, [_P, C.c_int32, _I, _I, _I, _F, _F, _F, _F, _F, C.c_int32, _I, _I, _F, _F, _F, _F,
                                      _F]),
    "mfc_full_attn_step_batched_dev": (C.c_int, [_P, C.c_int32, _I, _I, _I, _P, _P, _P, _P, _P]),
    "mfc_linear_attn_step_batched_dev": (C.c_int, [_P, C.c_int32, _I, _I, _P, _P, _P, _P, _P]),
    "mfc_full_attn_partial_batched_dev": (C.c_int, [_P, C.c_int32, _I, _I, _I, _P, _P, _P, _P, _P, _P]),
    "mfc_full_attn_partial_packed_dev": (C.c_int, [_P, C.c_int32, _I, _I, _I, _P, _P, _P, _P]),
    "mfc_lse_merge_gate_packed_dev": (C.c_int, [_P, C.c_int32, C.c_int32, _P, _P, _P]),
    "mfc_lse_merge_gate_dev": (C.c_int, [_P, C.c_int32, C.c_int32, _P, _P, _P, C.c_size_t, _P, _P]),
    "mfc_full_attn_prefill_dev": (C.c_int, [_P, C.c_int32, C.c_int32, C.c_int32, C.c_int32, _P, _P, _P, _P, _P]),
    "mfc_linear_attn_prefill_dev": (C.c_int, [_P, C.c_int32, C.c_int32, C.c_int32, _P, _P, _P, _P, _P]),
    "mfc_kv_append_rows_dev": (C.c_int, [_P, C.c_int32, C.c_int32, C.c_int32, C.c_int32, _P, _P]),
    "mfc_linear_state_set_dev": (C.c_int, [_P, C.c_int32, C.c_int32, _P, _P]),
    "mfc_memory_clear": (None, [_P, C.c_int32]),
    "mfc_memory_seq_rm": (C.c_int, [_P, C.c_int32, C.c_int32, C.c_int32]),
    "mfc_memory_seq_pos_max": (C.c_int, [_P, C.c_int32]),
    "mfc_state_size": (C.c_size_t, [_P, C.c_int32]),
    "mfc_state_save": (C.c_longlong, [_P, C.c_int32, _P, C.c_size_t]),
    "mfc_state_load": (C.c_int, [_P, C.c_int32, _P, C.c_size_t]),
    "mfc_apply_rotary_emb": (C.c_int, [_P, C.c_int32, _F, _F]),
    "mfc_sdpa": (C.c_int, [_P, C.c_int32, _F, _F, _F, _F, _F]),
    "mfc_linear_attn_step_stateless": (C.c_int, [_P, C.c_int32, _F, _F, _F, _F, _F, _F, _F]),
    "mfc_checkpoint_pos": (C.c_int, [_P, C.c_int32, C.c_int32]),
    "mfc_restore_to": (C.c_int, [_P, C.c_int32, C.c_int32]),
    "mfc_set_max_checkpoints": (None, [_P, C.c_int32]),
    "mfc_checkpoint_count": (C.c_int, [_P, C.c_int32]),
    "mfc_kv_local_len": (C.c_int, [C.c_int32, C.c_int32, C.c_int32, C.c_int32]),
    "mfc_kv_local_row": (C.c_int, [C.c_int32, C.c_int32, C.c_int32, C.c_int32]),
    "mfc_snapshot_validate": (C.c_longlong, [C.POINTER(Config), _P, C.c_size_t]),
    "mfc_sdpa_static_dev": (C.c_int, [C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, _P, _P, _P, _P, _P, _P]),
    "mfc_sdpa_static_status": (C.c_int, [_P]),
    "mfc_join": (C.c_int, [_P]),
    "mfc_check_guards": (C.c_int, [_P]),
    "mfc_read_phase_trace": (C.c_int, [_P, _P, C.c_int32]),
    "mfc_exchange_create": (C.c_int, [_P, C.c_int32, _P]),
    "mfc_exchange_connect": (C.c_int, [_P, _P]),
    "mfc_exchange_connect_local": (C.c_int, [_P, _P]),
    "mfc_full_attn_partial_exchange_dev": (C.c_int, [_P, C.c_int32, _I, _I, _I, _P, _P, _P]),
    "mfc_lse_merge_gate_exchange_dev": (C.c_int, [_P, _P, _P]),
    "mfc_dequant_matvec_4bit_dev": (C.c_int, [_P, _P, _P, _P, C.c_int32, C.c_int32, _P, C.c_int32, _P]),
    "mfc_dequant_matvec_4bit": (C.c_int, [_P, _P, _P, _P, C.c_int32, C.c_int32, _P, C.c_int32, _P]),
    "mfc_dequant_matvec_4bit_multi_dev": (C.c_int, [_P, C.c_int32, _P, _P, _P, C.c_int32, _P, _P, C.c_int32, _P]),
    "mfc_mla_sdpa_folded_dev": (C.c_int, [_P, C.c_int32, C.c_int32, C.c_float, _P, _P, _P, _P, _P]),
    "mfc_mla_sdpa_folded_bf16_dev": (C.c_int, [_P, C.c_int32, C.c_int32, C.c_float, _P, _P, _P, _P, _P]),
    "mfc_mla_sdpa_folded": (C.c_int, [_P, C.c_int32, C.c_int32, C.c_float, _F, _F, _F, _F, _F]),
    "mfc_set_tuning": (C.c_int, [_P, C.c_char_p, C.c_int]),
    "mfc_launch_count": (C.c_longlong, [_P]),
}

_lib = None


def lib_path() -> str:
    return _SO


def lib() -> C.CDLL:
    """Loads the shared object.  Raises if it has not been built: there is no
    fallback implementation."""
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            raise MfcError(
                f"{_SO} is missing: build it with `python -m moeflux_b200.build` "
                "(nvcc, sm_100a); this package has no CPU or PyTorch fallback")
        L = C.CDLL(_SO)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib
