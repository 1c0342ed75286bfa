"""Shared set-up of the GPU parity tests: a GPU context and its host-memory
oracle twin with identical weights."""
import numpy as np

import moeflux_b200 as M
from oracle import A17B, Geometry
from oracle.ctx import OracleCtx
from tests import inputs as I

TOL_F32 = 1e-4   # stated tolerance for the fp32 path (max|d| / max|ref|)
TOL_BF16 = 2e-2  # stated tolerance with a bf16 KV cache


def geometry_kwargs(g: Geometry):
    return dict(num_layers=g.num_layers, full_attn_interval=g.full_attn_interval,
                num_attn_heads=g.num_attn_heads, num_kv_heads=g.num_kv_heads, head_dim=g.head_dim,
                rotary_dim=g.rotary_dim, rope_theta=g.rope_theta, linear_num_v_heads=g.linear_num_v_heads,
                linear_num_k_heads=g.linear_num_k_heads)


def make_pair(g: Geometry = A17B, max_seq=1024, n_seqs=1, kv_bf16=False, seed=0, snapshot_version=1,
              linear_layers=None, **kw):
    ctx = M.Ctx(max_seq=max_seq, n_seqs=n_seqs, kv_dtype=M.KV_BF16 if kv_bf16 else M.KV_F32,
                snapshot_version=snapshot_version, **geometry_kwargs(g), **kw)
    orc = OracleCtx(g, max_seq=max_seq, n_seqs=n_seqs, kv_bf16=kv_bf16, snapshot_version=snapshot_version)
    r = I.rng(1000 + seed)
    if linear_layers is None:
        linear_layers = [i for i in range(g.num_layers) if not g.is_full_layer(i)]
    for layer in linear_layers:
        w = I.gdn_weights(r, g)
        ctx.set_linear_weights(layer, *w)
        orc.set_linear_weights(layer, *w)
    return ctx, orc
