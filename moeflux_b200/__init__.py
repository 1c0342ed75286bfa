"""B200-native (sm_100a) attention backend for moeflux: host-side mirror.

``Ctx`` mirrors the slice of ``moeflux::Ctx`` (``riir::RsCtx``) this backend
serves -- the attention sub-block of ``eval_token`` plus ``memory_*`` and
``state_*`` -- on top of the C ABI in ``include/moeflux_cuda.h``.  All compute
is in ``libmoeflux_cuda.so``; there is no Python or CPU fallback, and importing
the library without the built shared object raises.
"""
from ._lib import MfcError, Config, lib, lib_path, KV_F32, KV_BF16
from .ctx import Ctx, live_contexts, sdpa_static_dev, sdpa_static_status

__all__ = ["Ctx", "live_contexts", "sdpa_static_dev", "sdpa_static_status", "Config", "MfcError", "lib", "lib_path", "KV_F32", "KV_BF16"]
