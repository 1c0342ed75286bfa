#!/usr/bin/env python
"""Benchmark of the attention decode path on B200.

Workload ("stack"): the attention sub-blocks of one token step of the 60-layer
hybrid decode stack -- 45 GatedDeltaNet layer-steps and 15 full-attention GQA
layer-steps for each of 8 sequences at context 131072, bf16 KV cache, seeded
N(0,1) activations per (layer, sequence).  One step = 480 layer-steps =
35.4 GB of algorithmic HBM traffic.  On N GPUs the KV positions of every
sequence are split block-cyclically over the ranks; the decode kernel stores
each item's log-sum-exp partial straight into the memory of the rank that
finishes the item (peer stores over NVLink, step flags), which merges and gates
it; the GatedDeltaNet sequences are dealt round-robin; total work is fixed
("strong").  After the timed region one more step is computed and checked
against the CPU oracle ("parity" in the JSON line; non-zero exit above the
tolerance).

    python bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...     # the CPU restatement, timed on the host cores

Prints ONE JSON line (rank 0).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

N_LAYERS, INTERVAL = 60, 4
H, HKV, D = 32, 2, 256
HV, HK, DK = 64, 16, 128
CONV_DIM = 2 * HK * DK + HV * DK  # 12288
Q_DIM, KV_DIM, V_DIM = H * D, HKV * D, HV * DK
SSM_ELEMS = HV * DK * DK
FULL_LAYERS = [i for i in range(N_LAYERS) if (i + 1) % INTERVAL == 0]
LIN_LAYERS = [i for i in range(N_LAYERS) if (i + 1) % INTERVAL != 0]


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--ctx", type=int, default=131072, help="context length per sequence")
    ap.add_argument("--batch", type=int, default=8, help="sequences")
    ap.add_argument("--mla-cache", default="f32", choices=["f32", "bf16"], help="--workload mla: storage type of the latent cache")
    ap.add_argument("--trace-world", type=int, default=8, help="--workload trace: the KV split whose per-rank launch is traced")
    ap.add_argument("--workload", default="stack", choices=["stack", "ragged", "prefill", "matvec", "trace", "mla"],
                    help="stack: the decode stack (headline); ragged: 64 sequences of ragged context, one full-attention "
                         "layer-step each, sharded by sequence; prefill: 8192-token chunked prefill of one hybrid block; "
                         "matvec: the 4-bit projections around the attention sub-blocks of one hybrid block")
    ap.add_argument("--exchange", default="fused", choices=["fused", "nccl"],
                    help="KV-split exchange at N > 1: partials stored by the decode kernel into the finishing rank's "
                         "memory (fused), or one NCCL all-to-all per step (nccl)")
    ap.add_argument("--vecs", type=int, default=1, help="input vectors per projection (--workload matvec)")
    ap.add_argument("--tokens", type=int, default=8192, help="prefill tokens (--workload prefill)")
    ap.add_argument("--kv", default="bf16", choices=["bf16", "f32"], help="KV cache storage type")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--repeats", type=int, default=0, help="timed blocks of --steps steps (0: at least 7 and about a second)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--gather-q", type=int, default=0, choices=[0, 1],
                    help="N>1, fused exchange, end-to-end arm: 1 = every host sends the query rows of its own items and "
                         "the ranks gather them over NVLink (an eighth of the PCIe bytes at 8 GPUs, the same step "
                         "time); 0 = every host sends all rows")
    ap.add_argument("--no-single-step", action="store_true", help="skip the batch-1 single-step latencies (N=1, stack)")
    ap.add_argument("--other-configs", type=int, default=1,
                    help="1 (default): the stack line also carries compact lines of the ragged workload (every N) and of "
                         "the prefill workload (N=1), each run with --steps; 0: the stack workload alone")
    return ap.parse_args()


# --------------------------------------------------------------------------- byte model
def gdn_bytes_per_item():
    # state r+w, conv history r (3 rows) + w (1 row), qkv, conv weights, gates, z in, out
    return 2 * SSM_ELEMS * 4 + 4 * CONV_DIM * 4 + CONV_DIM * 4 + CONV_DIM * 4 * 2 + 4 * HV * 4 + 2 * V_DIM * 4


def gqa_bytes_per_item(rows, kv_esize=2):
    # K and V rows of both kv heads, q/gate/out, k/v in, appended row
    return 2 * rows * KV_DIM * kv_esize + 3 * Q_DIM * 4 + 2 * KV_DIM * 4 + 2 * KV_DIM * kv_esize


# --------------------------------------------------------------------------- clocks
class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.samples = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.index)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append((time.time(), line.strip()))

    def stop(self, t0, t1):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons, power = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        rows = [l for (t, l) in self.samples if t0 - 0.2 <= t <= t1 + 0.2] or [l for (_, l) in self.samples]
        for line in rows:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
                power.append(float(f[3]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


# --------------------------------------------------------------------------- CPU arm
def _host_threads():
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def cpu_sample(ctx_len, batch, seed=4, kind="port", n_full_layers=None, n_lin_layers=None):
    """Times the CPU statement of the path on a bounded sample of the stack workload and scales to one token step:
    returns (layer_steps_per_s, cores, description, kind).

    kind "port": the oracle (oracle/mf_oracle.c), OpenMP over heads.  kind "reference": the reference's own C
    functions (oracle/_ref, lifted from infer.m by oracle/ref.py), which are single-threaded, so independent
    layer-steps run side by side, one per host thread, as a batch of sequences would."""
    import oracle as O
    from oracle import A17B as G

    n_full_layers = len(FULL_LAYERS) if n_full_layers is None else n_full_layers
    n_lin_layers = len(LIN_LAYERS) if n_lin_layers is None else n_lin_layers
    O.build()
    r = np.random.Generator(np.random.Philox(seed))
    nrm = lambda *s: r.standard_normal(s, dtype=np.float32)
    conv_w = O.f32_to_bf16_bits(nrm(CONV_DIM, 4) * 0.5)
    a_log = r.uniform(0, 2.7, HV).astype(np.float32)
    dt_bias = O.f32_to_bf16_bits(nrm(HV))
    norm_w = O.f32_to_bf16_bits(1 + 0.1 * nrm(DK))
    K = O.round_bf16(nrm(ctx_len, KV_DIM))
    V = O.round_bf16(nrm(ctx_len, KV_DIM))
    n_full_items = n_full_layers * batch
    n_lin_items = n_lin_layers * batch
    if kind == "reference":
        import oracle.ref as R
        from concurrent.futures import ThreadPoolExecutor

        threads = _host_threads()
        # full attention: `threads` layer-steps at the full context side by side.  They read one copy of the cache
        # rows (a copy per thread would not fit) and append the same row, so the concurrent writes store equal values.
        n_gqa = min(threads, max(n_full_items, 1))
        q, gate, k, v = nrm(Q_DIM), nrm(Q_DIM), nrm(KV_DIM), nrm(KV_DIM)

        def gqa(i):
            R.full_attn_step(ctx_len - 1, ctx_len - 1, q, gate, k, v, K, V, H, HKV, D, G.rotary_dim)

        t_gqa = 0.0
        if n_full_items:
            with ThreadPoolExecutor(threads) as ex:
                t0 = time.perf_counter()
                list(ex.map(gqa, range(n_gqa)))
                t_gqa = (time.perf_counter() - t0) / n_gqa  # wall time per layer-step with all threads busy
        per = max(1, min(4, n_lin_items // max(threads, 1)))
        n_gdn = threads * per
        states = [(nrm(3, CONV_DIM), nrm(SSM_ELEMS) * np.float32(0.02)) for _ in range(threads)]
        gin = [(nrm(CONV_DIM), nrm(V_DIM), nrm(HV), nrm(HV)) for _ in range(threads)]

        def gdn(i):
            conv, ssm = states[i]
            for _ in range(per):
                R.linear_attn_step(*gin[i], conv_w, a_log, dt_bias, norm_w, conv, ssm, G)

        t_gdn = 0.0
        if n_lin_items:
            with ThreadPoolExecutor(threads) as ex:
                t0 = time.perf_counter()
                list(ex.map(gdn, range(threads)))
                t_gdn = (time.perf_counter() - t0) / n_gdn
        cores = threads
        how = (f"the reference's own C functions (infer.m cpu_sdpa, apply_rotary_emb, cpu_conv1d_step, "
               f"cpu_gated_delta_recurrence, cpu_rms_norm_gated; single-threaded each, {threads} independent layer-steps "
               f"side by side)")
    else:
        O.use_all_cores()
        q, gate, k, v = nrm(Q_DIM), nrm(Q_DIM), nrm(KV_DIM), nrm(KV_DIM)
        n_gqa = 2 if n_full_items else 0
        t0 = time.perf_counter()
        for _ in range(n_gqa):
            O.full_attn_step(ctx_len - 1, ctx_len - 1, q, gate, k, v, K, V, G, kv_bf16=True)
        t_gqa = (time.perf_counter() - t0) / max(n_gqa, 1)
        conv = nrm(3, CONV_DIM)
        ssm = nrm(SSM_ELEMS) * np.float32(0.02)
        n_gdn = 24 if n_lin_items else 0
        t0 = time.perf_counter()
        for _ in range(n_gdn):
            O.linear_attn_step(nrm(CONV_DIM), nrm(V_DIM), nrm(HV), nrm(HV), conv_w, a_log, dt_bias, norm_w, conv, ssm, G)
        t_gdn = (time.perf_counter() - t0) / max(n_gdn, 1)
        cores = O.num_threads()
        how = "the C restatement of the reference math (oracle/mf_oracle.c, OpenMP over heads)"
    t_step = n_full_items * t_gqa + n_lin_items * t_gdn
    desc = (f"{how}: {n_gqa} GQA layer-steps at ctx {ctx_len} ({t_gqa * 1e3:.1f} ms each at full load) and {n_gdn} "
            f"GatedDeltaNet layer-steps ({t_gdn * 1e3:.2f} ms each), scaled to {n_full_items}+{n_lin_items} per token step")
    return (n_full_items + n_lin_items) / t_step, cores, desc, kind


def reference_kind():
    """"reference" when the reference's own C functions are built (oracle/_ref) or can be built here, else "port"."""
    try:
        import oracle.ref as R

        if R.available():
            R.lib()
            return "reference"
    except Exception:
        pass
    return "port"


def run_reference(args, rank):
    if rank != 0:
        return
    kind = reference_kind()
    vals = []
    cores, desc = 1, ""
    t_begin = time.perf_counter()
    ragged = args.workload == "ragged"
    for i in range(args.warmup + args.steps):
        if ragged:
            v, cores, desc, kind = cpu_sample_ragged(args, kind, seed=4 + i)
        else:
            v, cores, desc, kind = cpu_sample(args.ctx, args.batch, seed=4 + i, kind=kind)
        if i >= args.warmup:
            vals.append(v)
        if time.perf_counter() - t_begin > 200 and len(vals) >= 1:  # keep the arm within minutes
            break
    value = len(vals) / sum(1.0 / v for v in vals)
    n_units = RAGGED_SEQS if ragged else N_LAYERS * args.batch
    line = {
        "impl": "reference", "metric": "attention decode layer-steps/sec", "value": value, "unit": "layer-steps/s",
        "n_gpus": args.gpus, "steps": len(vals), "warmup": args.warmup,
        "ms_per_step": 1e3 * n_units / value,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32 (bf16 KV values)",
        "data": "synthetic", "config": ragged_config(args, args.gpus) if ragged else workload_config(args, args.gpus),
        "cpu_baseline": {"value": value, "unit": "layer-steps/s", "cores": cores, "kind": kind, "sample": desc},
        "e2e": {"value": value, "unit": "layer-steps/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(line)


def workload_config(args, n):
    return {"workload": f"60-layer hybrid attention-only decode stack (45 GatedDeltaNet + 15 GQA), batch {args.batch}, "
                        f"ctx {args.ctx}, {args.kv} KV, fp32 state",
            "layer_steps_per_step": N_LAYERS * args.batch, "context": args.ctx, "batch": args.batch,
            "kv_dtype": args.kv, "parallelism": (f"kv-sequence split x{n}: the decode kernel stores each item's log-sum-exp "
                                                f"partial straight into the receive buffer of the rank that finishes the "
                                                f"item (peer stores over NVLink + step flags; --exchange nccl: one NCCL "
                                                f"all-to-all per step instead), merged and gated there + GatedDeltaNet "
                                                f"sequences round-robin")
            if n > 1 else "single GPU",
            "l2": "inputs (GBs of KV and state per step) exceed the 126 MB L2; no flush needed"}


def repeats_for(k_steps, est_ms_per_step):
    """Timed blocks of k_steps steps: at least 7, and enough for about a second of timed work."""
    block_s = max(k_steps * est_ms_per_step * 1e-3, 1e-6)
    return int(min(64, max(7, -(-1.0 // block_s))))


# --------------------------------------------------------------------------- GPU arm
def run_ours(args, rank, world, local_rank):
    import torch
    import torch.distributed as dist

    import moeflux_b200 as M

    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    B, CTX = args.batch, args.ctx
    W, K = args.warmup, args.steps
    do_e2e = not args.no_e2e
    fused = world > 1 and args.exchange == "fused"
    R = args.repeats or repeats_for(K, 4.9 * (CTX / 131072.0) * (B / 8.0) / world)
    We, Re = (min(W, 3), min(R, 7)) if do_e2e else (0, 0)
    total_steps = W + R * K + We + Re * K + 1  # + the step whose outputs are checked against the oracle
    L0 = CTX - total_steps  # the checked step brings every cache to exactly CTX rows
    assert L0 > 0, "context too short for this many steps"

    kv_esize = 2 if args.kv == "bf16" else 4
    ctx = M.Ctx(max_seq=CTX, n_seqs=B, kv_dtype=M.KV_BF16 if args.kv == "bf16" else M.KV_F32, device=local_rank, kv_rank=rank, kv_world=world,
                kv_block=256, max_batch=N_LAYERS * B)
    stream = torch.cuda.Stream(device=dev)  # owned by torch, so tensors allocated on it outlive the context safely
    ctx.set_stream(stream.cuda_stream)
    side = torch.cuda.ExternalStream(ctx.side_stream, device=dev)
    if world > 1:
        # the GatedDeltaNet launch runs beside the attention launch: with the KV split the attention
        # launch is short enough to leave bandwidth unused at its edges
        ctx.set_tuning("gdn_side_queue", 1)
    gen = torch.Generator(device=dev)
    kv_seed = lambda layer, s: 1234 + 1000 * layer + s
    st_seed = lambda layer, s: 500000 + 1000 * layer + s

    # ---- state: seeded fills on the device, imported through the bulk-import calls ----
    CH = 8192

    def kv_rows(layer, s, p0, n):
        """Rows [p0, p0+n) of the seeded cache of (layer, s): the same values on every rank and for the checker."""
        gen.manual_seed(kv_seed(layer, s) * 4096 + p0 // CH)
        return (torch.randn(n, KV_DIM, device=dev, generator=gen), torch.randn(n, KV_DIM, device=dev, generator=gen))

    with torch.cuda.stream(stream):
        for layer in FULL_LAYERS:
            for s in range(B):
                for p0 in range(0, L0, CH):
                    n = min(CH, L0 - p0)
                    kr, vr = kv_rows(layer, s, p0, n)
                    ctx.kv_append_rows_dev(layer, s, p0, n, kr.data_ptr(), vr.data_ptr())
                    stream.synchronize()
        my_seqs = [s for s in range(B) if s % world == rank]
        rs = np.random.Generator(np.random.Philox(77))
        lin_weights = {}
        for layer in LIN_LAYERS:
            conv_w = (rs.standard_normal((CONV_DIM, 4), dtype=np.float32) * 0.5)
            conv_w_bits = (torch.tensor(conv_w).bfloat16().view(torch.int16).numpy().astype(np.uint16))
            a_log = rs.uniform(0, 2.7, HV).astype(np.float32)
            dt_bits = torch.tensor(rs.standard_normal(HV, dtype=np.float32)).bfloat16().view(torch.int16).numpy().astype(np.uint16)
            nw_bits = torch.tensor(1 + 0.1 * rs.standard_normal(DK, dtype=np.float32)).bfloat16().view(torch.int16).numpy().astype(np.uint16)
            lin_weights[layer] = (conv_w_bits, a_log, dt_bits, nw_bits)
            ctx.set_linear_weights(layer, conv_w_bits, a_log, dt_bits, nw_bits)
            for s in my_seqs:
                gen.manual_seed(st_seed(layer, s))
                cs = torch.randn(3, CONV_DIM, device=dev, generator=gen)
                ss = torch.randn(SSM_ELEMS, device=dev, generator=gen) * 0.02
                ctx.linear_state_set_dev(layer, s, cs.data_ptr(), ss.data_ptr())
                stream.synchronize()

    # ---- items ----
    # full-attention items sorted by the rank that finishes them (the owner of the sequence), so the partial
    # blocks of one destination are contiguous
    seq_order = sorted(range(B), key=lambda s: (s % world, s))
    gqa_items = [(l, s) for s in seq_order for l in FULL_LAYERS]
    if world > 1:
        assert B % world == 0, "batch must divide over the ranks"
    gdn_items = [(l, s) for l in LIN_LAYERS for s in my_seqs]
    ng, nl = len(gqa_items), len(gdn_items)
    npr = ng // world                     # items this rank finishes
    own = slice(rank * npr, (rank + 1) * npr)
    g_layers = np.array([l for l, _ in gqa_items], np.int32)
    g_seqs = np.array([s for _, s in gqa_items], np.int32)
    l_layers = np.array([l for l, _ in gdn_items], np.int32)
    l_seqs = np.array([s for _, s in gdn_items], np.int32)

    with torch.cuda.stream(stream):
        gen.manual_seed(99)
        q = torch.randn(ng, Q_DIM, device=dev, generator=gen)
        gate = torch.randn(ng, Q_DIM, device=dev, generator=gen)
        kk = torch.randn(ng, KV_DIM, device=dev, generator=gen)
        vv = torch.randn(ng, KV_DIM, device=dev, generator=gen)
        out_g = torch.empty(ng, Q_DIM, device=dev)
        gen.manual_seed(100 + rank)
        qkv = torch.randn(max(nl, 1), CONV_DIM, device=dev, generator=gen)
        z = torch.randn(max(nl, 1), V_DIM, device=dev, generator=gen)
        alpha = torch.randn(max(nl, 1), HV, device=dev, generator=gen)
        beta = torch.randn(max(nl, 1), HV, device=dev, generator=gen)
        out_l = torch.empty(max(nl, 1), V_DIM, device=dev)
        if world > 1:
            item_floats = H * D + 2 * H           # [o | m | l] of one item
            send = torch.empty(ng * item_floats, device=dev)
            recv = torch.empty(world * npr * item_floats, device=dev)
            out_own = torch.empty(npr, Q_DIM, device=dev)
    stream.synchronize()
    if fused:
        handle = ctx.exchange_create(npr)
        handles = [None] * world
        dist.all_gather_object(handles, handle)
        ctx.exchange_connect(handles)
        dist.barrier()

    pos_now = [L0]
    ev = lambda: torch.cuda.Event(enable_timing=True)
    gqa_events = []
    gdn_events = []

    def device_step(timed):
        pos = np.full(ng, pos_now[0], np.int32)
        if timed:
            d0, d1, e0, e1 = ev(), ev(), ev(), ev()

        def gdn():
            # with the side queue on, the kernel starts when the main queue reaches this point and runs on the
            # second queue: its duration is the time from an event here to an event behind it on that queue
            if timed:
                d0.record(stream)
            if nl:
                ctx.linear_attn_step_batched_dev(l_layers, l_seqs, qkv.data_ptr(), z.data_ptr(), alpha.data_ptr(),
                                                 beta.data_ptr(), out_l.data_ptr())
            if timed:
                d1.record(side if world > 1 else stream)

        if world == 1:
            gdn()
            if timed:
                e0.record(stream)
            ctx.full_attn_step_batched_dev(g_layers, g_seqs, pos, q.data_ptr(), gate.data_ptr(), kk.data_ptr(),
                                           vv.data_ptr(), out_g.data_ptr())
            if timed:
                e1.record(stream)
        elif fused:
            gdn()  # on the side queue
            if timed:
                e0.record(stream)
            ctx.full_attn_partial_exchange_dev(g_layers, g_seqs, pos, q.data_ptr(), kk.data_ptr(), vv.data_ptr())
            if timed:
                e1.record(stream)
            ctx.lse_merge_gate_exchange_dev(gate[own].data_ptr(), out_own.data_ptr())
            ctx.join()
        else:
            gdn()  # on the side queue
            if timed:
                e0.record(stream)
            ctx.full_attn_partial_packed_dev(g_layers, g_seqs, pos, q.data_ptr(), kk.data_ptr(), vv.data_ptr(),
                                             send.data_ptr())
            if timed:
                e1.record(stream)
            # every item's partials travel to the rank that owns its sequence
            dist.all_to_all_single(recv, send)
            ctx.join()
            ctx.lse_merge_gate_packed_dev(world, npr, recv.data_ptr(), gate[own].data_ptr(), out_own.data_ptr())
        if timed:
            gqa_events.append((e0, e1))
            gdn_events.append((d0, d1))
        pos_now[0] += 1

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    sampler = ClockSampler(local_rank) if rank == 0 else None
    blocks = []
    with torch.cuda.stream(stream):
        for _ in range(W):
            device_step(False)
        if sampler:
            sampler.start()
            time.sleep(0.3)  # before the barrier: every rank enters the timed region together
        launches0 = ctx.launch_count
        t_wall0 = time.time()
        pos_first_timed = pos_now[0]
        for _ in range(R):
            barrier()
            start, stop = ev(), ev()
            start.record(stream)
            for _ in range(K):
                device_step(True)
            stop.record(stream)
            barrier()
            blocks.append(start.elapsed_time(stop))
        t_wall1 = time.time()
        launches = (ctx.launch_count - launches0) // R  # of one block of K steps
    ctx.synchronize()  # raises if a kernel reported a fault
    mean_pos = pos_first_timed + (R * K - 1) / 2.0
    gqa_ms = sum(a.elapsed_time(b) for a, b in gqa_events) / len(gqa_events)
    gdn_ms = sum(a.elapsed_time(b) for a, b in gdn_events) / len(gdn_events) if nl else 0.0
    blocks_t = torch.tensor(blocks + [gqa_ms, gdn_ms], device=dev, dtype=torch.float64)
    per_rank = None
    if world > 1:
        mine_t = torch.tensor([statistics.median(blocks) / K, gqa_ms, gdn_ms], device=dev, dtype=torch.float64)
        all_t = torch.empty(world * 3, device=dev, dtype=torch.float64)
        dist.all_gather_into_tensor(all_t, mine_t)
        per_rank = {"ms_per_step": [round(float(x), 4) for x in all_t[0::3]],
                    "gqa_ms_per_launch": [round(float(x), 4) for x in all_t[1::3]],
                    "gdn_ms_per_launch": [round(float(x), 4) for x in all_t[2::3]]}
        dist.all_reduce(blocks_t, op=dist.ReduceOp.MAX)  # every block: the slowest rank
    blocks = [float(x) for x in blocks_t[:R]]
    gqa_ms, gdn_ms = float(blocks_t[R]), float(blocks_t[R + 1])
    ms = statistics.median(blocks)
    clocks = sampler.stop(t_wall0, t_wall1) if sampler else None

    # ---- end to end: host (pinned) inputs in, host outputs back, every step, through the host-pointer call ----
    e2e = None
    if do_e2e:
        pin = lambda *shape: torch.empty(*shape, dtype=torch.float32).pin_memory()
        n_gate = ng if world == 1 else npr  # gate rows and outputs are needed only where an item is finished
        # fused exchange: every rank's host sends the query rows of the items it finishes, the rest cross the links
        gather_q = world > 1 and fused and bool(args.gather_q)
        n_q = npr if gather_q else ng
        hq, hgate, hk, hv, hout = pin(n_q, Q_DIM), pin(n_gate, Q_DIM), pin(ng, KV_DIM), pin(ng, KV_DIM), pin(n_gate, Q_DIM)
        hqkv, hz, ha, hb, hlo = pin(max(nl, 1), CONV_DIM), pin(max(nl, 1), V_DIM), pin(max(nl, 1), HV), pin(
            max(nl, 1), HV), pin(max(nl, 1), V_DIM)
        for h, d_ in ((hq, q[own] if gather_q else q), (hgate, gate if world == 1 else gate[own]), (hk, kk), (hv, vv), (hqkv, qkv), (hz, z),
                      (ha, alpha), (hb, beta)):
            h.copy_(d_.cpu())
        h2d = 4 * ((n_q + n_gate) * Q_DIM + 2 * ng * KV_DIM + nl * (CONV_DIM + V_DIM + 2 * HV))
        d2h = 4 * (n_gate * Q_DIM + nl * V_DIM)
        use_abi = world == 1 or fused

        def e2e_step():
            pos = np.full(ng, pos_now[0], np.int32)
            if use_abi:
                ctx.eval_token_attn_ptr(ng, g_layers.ctypes.data, g_seqs.ctypes.data, pos.ctypes.data, hq.data_ptr(),
                                        hgate.data_ptr(), hk.data_ptr(), hv.data_ptr(), hout.data_ptr(), nl,
                                        l_layers.ctypes.data if nl else 0, l_seqs.ctypes.data if nl else 0,
                                        hqkv.data_ptr(), hz.data_ptr(), ha.data_ptr(), hb.data_ptr(), hlo.data_ptr())
                pos_now[0] += 1
            else:
                with torch.cuda.stream(stream):
                    q.copy_(hq, non_blocking=True)
                    gate[own].copy_(hgate, non_blocking=True)
                    kk.copy_(hk, non_blocking=True)
                    vv.copy_(hv, non_blocking=True)
                    if nl:
                        qkv.copy_(hqkv, non_blocking=True)
                        z.copy_(hz, non_blocking=True)
                        alpha.copy_(ha, non_blocking=True)
                        beta.copy_(hb, non_blocking=True)
                    device_step(False)
                    hout.copy_(out_own, non_blocking=True)
                    if nl:
                        hlo.copy_(out_l, non_blocking=True)
                    stream.synchronize()

        if use_abi and world > 1:
            ctx.set_tuning("gdn_side_queue", 0)  # the call runs its two groups on its two queues itself
            ctx.set_tuning("exchange_gather_q", int(gather_q))
        for _ in range(We):
            e2e_step()
        e_blocks = []
        for _ in range(Re):
            barrier()
            t0 = time.perf_counter()
            for _ in range(K):
                e2e_step()
            barrier()
            e_blocks.append(time.perf_counter() - t0)
        if world > 1:
            t = torch.tensor(e_blocks, device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e_blocks = [float(x) for x in t]
        dt = statistics.median(e_blocks)
        e2e = {"value": N_LAYERS * B * K / dt, "unit": "layer-steps/s", "h2d_bytes_per_step": h2d,
               "d2h_bytes_per_step": d2h, "ms_per_step": 1e3 * dt / K, "steps": K, "repeats": Re,
               "min": N_LAYERS * B * K / max(e_blocks), "max": N_LAYERS * B * K / min(e_blocks),
               "api": ("mfc_eval_token_attn (host pointers; copies, kernels and exchange inside the call" +
                       ("; each host sends the query rows of its own items, gathered over NVLink)" if gather_q else ")"))
               if use_abi
               else "torch copies around the _dev calls and one NCCL all-to-all"}
        ctx.synchronize()
        if use_abi and world > 1:
            ctx.set_tuning("gdn_side_queue", 1)

    # ---- parity: one more step, its outputs against the CPU oracle on the same seeded rows ----
    parity = None
    with torch.cuda.stream(stream):
        final_pos = pos_now[0]
        device_step(False)
        stream.synchronize()
    ctx.synchronize()
    if rank == 0:
        import oracle as O
        from oracle import A17B as G

        O.build()
        O.use_all_cores()
        tol = 2e-2 if args.kv == "bf16" else 1e-4
        out_dev = out_g if world == 1 else out_own
        check = sorted({0, npr - 1}) if world > 1 else sorted({0, ng - 1})  # items this rank finished (index in out_dev)
        worst = 0.0
        rnd = O.round_bf16 if args.kv == "bf16" else (lambda a: a)
        for j in check:
            gi = j if world == 1 else rank * npr + j
            layer, s = gqa_items[gi]
            n_rows = final_pos + 1
            Kh = np.empty((n_rows, KV_DIM), np.float32)
            Vh = np.empty((n_rows, KV_DIM), np.float32)
            for p0 in range(0, L0, CH):
                n = min(CH, L0 - p0)
                kr, vr = kv_rows(layer, s, p0, n)
                Kh[p0:p0 + n] = kr.cpu().numpy()
                Vh[p0:p0 + n] = vr.cpu().numpy()
            k_in, v_in = kk[gi].cpu().numpy(), vv[gi].cpu().numpy()
            zq = np.zeros(Q_DIM, np.float32)
            for p in range(L0, final_pos):  # the rows the earlier steps appended: RoPE(k) at each position, v as is
                Kh[p] = O.apply_rotary_emb(p, zq, k_in)[1]
                Vh[p] = v_in
            Kh[:final_pos] = rnd(Kh[:final_pos])
            Vh[:final_pos] = rnd(Vh[:final_pos])
            ref = O.full_attn_step(final_pos, final_pos, q[gi].cpu().numpy(), gate[gi].cpu().numpy(), k_in, v_in, Kh, Vh, G,
                                   kv_bf16=args.kv == "bf16")
            got = out_dev[j].cpu().numpy()
            worst = max(worst, float(np.max(np.abs(got - ref)) / max(np.max(np.abs(ref)), 1e-30)))
        parity = {"max_rel_err": worst, "items": len(check), "tol": tol, "context": final_pos + 1,
                  "what": "outputs of full-attention items of the step after the timed region vs the CPU oracle on the "
                          "same seeded cache rows" + (f" (every item's partials come from all {world} ranks)" if world > 1 else "")}
        # one GatedDeltaNet item: every step since the seeded state, replayed on the CPU with the same inputs
        if nl:
            layer, s = gdn_items[0]
            gen.manual_seed(st_seed(layer, s))
            conv = torch.randn(3, CONV_DIM, device=dev, generator=gen).cpu().numpy().copy()
            ssm = (torch.randn(SSM_ELEMS, device=dev, generator=gen) * 0.02).cpu().numpy().copy()
            ins = [t[0].cpu().numpy() for t in (qkv, z, alpha, beta)]
            ref = None
            for _ in range(final_pos - L0 + 1):
                ref = O.linear_attn_step(*ins, *lin_weights[layer], conv, ssm, G)
            got = out_l[0].cpu().numpy()
            parity["gdn_max_rel_err"] = float(np.max(np.abs(got - ref)) / max(np.max(np.abs(ref)), 1e-30))
            parity["gdn_tol"] = 1e-4
            parity["gdn_steps_replayed"] = final_pos - L0 + 1
        parity["ok"] = bool(worst <= tol and parity.get("gdn_max_rel_err", 0.0) <= 1e-4)

    # ---- roofline of the dominant kernel (the GQA split-K decode launch of this rank) ----
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        peak, peak_src = float(json.load(open(peaks_path))["hbm_gbs"]), "MEASURED_PEAKS.json hbm_gbs (of measured)"
    else:
        peak, peak_src = 6650.0, "fallback 6.65 TB/s (of fallback)"
    rows_local = (mean_pos + 1) / world
    gqa_alg_bytes = ng * gqa_bytes_per_item(rows_local, kv_esize)
    achieved = gqa_alg_bytes / (gqa_ms * 1e-3) / 1e9
    step_bytes = ng * gqa_bytes_per_item(mean_pos + 1, kv_esize) + (len(LIN_LAYERS) * B) * gdn_bytes_per_item()
    # DRAM bytes (ncu dram__bytes_read.sum + dram__bytes_write.sum) over algorithmic bytes, captured on the
    # ctx-8192 case of this workload; the traffic is the streamed KV rows, so it scales with the rows of a launch.
    dram_over_algorithmic = {"bf16": 1.009, "f32": 1.007}[args.kv]
    traffic = gqa_alg_bytes * dram_over_algorithmic
    gdn_alg = nl * gdn_bytes_per_item()
    roofline = {"bound": "hbm", "kernel": f"gqa_decode_{args.kv}_kernel", "achieved": achieved, "peak": peak, "unit": "GB/s",
                "frac": achieved / peak, "traffic": traffic, "peak_source": peak_src,
                "algorithmic_bytes_per_launch": gqa_alg_bytes, "ms_per_launch": gqa_ms,
                "frac_of_8TBps": achieved / 8000.0,
                "other_kernels": {"gdn_decode_kernel": {
                    "ms_per_launch": gdn_ms, "algorithmic_bytes_per_launch": gdn_alg,
                    "achieved": (gdn_alg / (gdn_ms * 1e-3) / 1e9) if nl and gdn_ms > 0 else None,
                    "frac": (gdn_alg / (gdn_ms * 1e-3) / 1e9 / peak) if nl and gdn_ms > 0 else None,
                    "note": "runs on the second queue beside the attention launch" if world > 1 else "runs alone"}},
                "whole_step": {"algorithmic_bytes_all_gpus": step_bytes,
                               "GBps_per_gpu": step_bytes / world / (ms / K * 1e-3) / 1e9,
                               "frac_of_measured": step_bytes / world / (ms / K * 1e-3) / 1e9 / peak,
                               "frac_of_8TBps": step_bytes / world / (ms / K * 1e-3) / 1e9 / 8000.0}}

    line = None
    if rank == 0:
        value = N_LAYERS * B * K / (ms * 1e-3)
        line = {"metric": "attention decode layer-steps/sec", "value": value, "unit": "layer-steps/s", "n_gpus": world,
                "steps": K, "warmup": W, "ms_per_step": ms / K, "higher_is_better": True, "scaling": "strong",
                "vs_baseline": None, "dtype": f"{args.kv} KV, fp32 accumulate and state", "data": "synthetic",
                "config": workload_config(args, world), "repeats": R,
                "min": N_LAYERS * B * K / (max(blocks) * 1e-3), "max": N_LAYERS * B * K / (min(blocks) * 1e-3),
                "value_is": f"median of {R} timed blocks of {K} steps (CUDA events, slowest rank per block)",
                "roofline": roofline, "e2e": e2e, "parity": parity, "gpu_launches": int(launches), "clocks": clocks}
        if per_rank:
            line["per_rank"] = per_rank  # device-timed, every rank's own median: the ranks run in lock step
    if world > 1:
        dist.barrier()  # no rank unmaps its peers' buffers while another may still use them
    ctx.close()
    return line


# --------------------------------------------------------------------------- batch-1 single steps
def single_step_latencies(local_rank=0, calls=1000):
    """Configurations 0 and 1 as stated (one sequence, one layer-step per call) and the 32k target shape: microseconds
    per step by CUDA events over `calls` pipelined device-pointer calls that rotate over enough sequences to exceed
    the 126 MB L2 several times, so that every step streams its cache or state from HBM."""
    import torch

    import moeflux_b200 as M

    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    out = {}

    def timed(ctx, st, call, n_seqs, n_calls):
        with torch.cuda.stream(st):
            for i in range(n_seqs):
                call(i)
            st.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            n = n_calls - n_calls % n_seqs
            e0.record(st)
            for i in range(n):
                call(i)
            e1.record(st)
            st.synchronize()
        ctx.synchronize()
        return e0.elapsed_time(e1) / n * 1e3

    def gqa(ctx_len, bf16, n_seqs, n_calls):
        c = M.Ctx(num_layers=4, max_seq=ctx_len + n_calls // n_seqs + 8, n_seqs=n_seqs,
                  kv_dtype=M.KV_BF16 if bf16 else M.KV_F32, device=local_rank, max_batch=4)
        st = torch.cuda.Stream(device=dev)
        c.set_stream(st.cuda_stream)
        g = torch.Generator(device=dev)
        g.manual_seed(5)
        kr, vr = torch.randn(8192, KV_DIM, device=dev, generator=g), torch.randn(8192, KV_DIM, device=dev, generator=g)
        L0 = ctx_len - 1
        with torch.cuda.stream(st):
            for s in range(n_seqs):
                for p0 in range(0, L0, 8192):
                    n = min(8192, L0 - p0)
                    c.kv_append_rows_dev(3, s, p0, n, kr.data_ptr(), vr.data_ptr())
        q, gt = torch.randn(Q_DIM, device=dev, generator=g), torch.randn(Q_DIM, device=dev, generator=g)
        k, v = torch.randn(KV_DIM, device=dev, generator=g), torch.randn(KV_DIM, device=dev, generator=g)
        o = torch.empty(Q_DIM, device=dev)
        torch.cuda.synchronize(dev)
        # the host side of a call is kept to one ctypes call on tables that are passed by address
        lay_tab, seq_tab = np.full(1, 3, np.int32), np.arange(n_seqs, dtype=np.int32)
        pos = np.full(n_seqs, L0, np.int32)
        lay_p, seq_p, pos_p = lay_tab.ctypes.data, seq_tab.ctypes.data, pos.ctypes.data
        ptrs = (q.data_ptr(), gt.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr())

        def call(i):
            s = i % n_seqs
            c.full_attn_step_batched_dev_ptr(1, lay_p, seq_p + 4 * s, pos_p + 4 * s, *ptrs)
            pos[s] += 1

        us = timed(c, st, call, n_seqs, n_calls)
        c.close()
        by = gqa_bytes_per_item(ctx_len, 2 if bf16 else 4)
        return {"us_per_step": us, "algorithmic_bytes": by, "GBps": by / us / 1e3, "frac_of_8TBps": by / us / 1e3 / 8000.0,
                "sequences_rotated": n_seqs}

    out["gqa_ctx4096_f32 (configuration 0)"] = gqa(4096, False, 32, calls)
    out["gqa_ctx32768_bf16"] = gqa(32768, True, 8, calls)
    out["gqa_ctx32768_f32"] = gqa(32768, False, 8, calls)
    # GatedDeltaNet single step (configuration 1)
    n_seqs = 64
    c = M.Ctx(num_layers=4, max_seq=64, n_seqs=n_seqs, device=local_rank, max_batch=4)
    st = torch.cuda.Stream(device=dev)
    c.set_stream(st.cuda_stream)
    r = np.random.Generator(np.random.Philox(6))
    bits = lambda a: torch.tensor(np.asarray(a, np.float32)).bfloat16().view(torch.int16).numpy().astype(np.uint16)
    c.set_linear_weights(0, bits(r.standard_normal((CONV_DIM, 4)) * 0.5), r.uniform(0, 2.7, HV).astype(np.float32),
                         bits(r.standard_normal(HV)), bits(1 + 0.1 * r.standard_normal(DK)))
    qkv, z = torch.randn(CONV_DIM, device=dev), torch.randn(V_DIM, device=dev)
    a, b, o = torch.randn(HV, device=dev), torch.randn(HV, device=dev), torch.empty(V_DIM, device=dev)
    torch.cuda.synchronize(dev)
    # (a call is under 10 us: the host side must not be the slower part, so the tables are kept and passed by address)
    lay_tab, seq_tab = np.zeros(1, np.int32), np.arange(n_seqs, dtype=np.int32)
    lay_p, seq_p = lay_tab.ctypes.data, seq_tab.ctypes.data
    ptrs = (qkv.data_ptr(), z.data_ptr(), a.data_ptr(), b.data_ptr(), o.data_ptr())
    us = timed(c, st, lambda i: c.linear_attn_step_batched_dev_ptr(1, lay_p, seq_p + 4 * (i % n_seqs), *ptrs), n_seqs, 1024)
    c.close()
    by = gdn_bytes_per_item()
    out["gdn_single_step (configuration 1)"] = {"us_per_step": us, "algorithmic_bytes": by, "GBps": by / us / 1e3,
                                                "frac_of_8TBps": by / us / 1e3 / 8000.0, "sequences_rotated": n_seqs}
    out["how"] = (f"CUDA events over {calls} pipelined device-pointer calls, one (layer, sequence) item each, rotating over "
                  f"sequences whose caches or states together exceed the L2 several times")
    return out


# --------------------------------------------------------------------------- per-CTA phase trace of the decode launch
def run_trace(args):
    """Where a decode launch spends its time, from the kernel's own per-CTA time stamps (tuning "gqa_phase_trace":
    %globaltimer at kernel start, first segment's query fragments ready, its last KV tile consumed, its epilogue done,
    CTA done).  Cases: the stack's full-attention launch as one rank of an N-way KV split sees it (--trace-world N,
    emulated on this GPU by a context that holds rank 0's rows), and a lone sequence at ctx 4096 (fp32) and 32768
    (bf16, fp32).  Prints one JSON line."""
    import torch

    import moeflux_b200 as M

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    cases = []

    def summarise(name, ctx, us_per_launch, alg_bytes):
        tr = ctx.read_phase_trace().astype(np.int64)
        d = (tr[:, :5] - tr[:, 0].min()) / 1e3
        med = lambda x: float(np.median(x))
        cases.append({"case": name, "ctas": int(len(tr)), "us_per_launch_events": us_per_launch,
                      "GBps": alg_bytes / us_per_launch / 1e3 if us_per_launch else None,
                      "span_us": float(d[:, 4].max()), "start_spread_us": float(d[:, 0].max()),
                      "prologue_us": {"median": med(d[:, 1] - d[:, 0]), "max": float((d[:, 1] - d[:, 0]).max())},
                      "prologue_split_us (bf16 cache)": None if not tr[:, 5].any() else {
                          "rows_staged": med((tr[:, 5] - tr[:, 0]) / 1e3), "rotated": med((tr[:, 6] - tr[:, 5]) / 1e3),
                          "fragments_and_third_tile": med((tr[:, 1] - tr[:, 6]) / 1e3)},
                      "first_segment_stream_us": {"median": med(d[:, 2] - d[:, 1]), "max": float((d[:, 2] - d[:, 1]).max())},
                      "first_segment_epilogue_us": {"median": med(d[:, 3] - d[:, 2]), "max": float((d[:, 3] - d[:, 2]).max())},
                      "cta_total_us": {"median": med(d[:, 4] - d[:, 0]), "min": float((d[:, 4] - d[:, 0]).min()),
                                       "max": float((d[:, 4] - d[:, 0]).max())},
                      "last_stream_end_us": float(d[:, 2].max())})

    # (a) the stack's launch as one rank of a --trace-world split sees it
    world, B, CTX = args.trace_world, args.batch, args.ctx
    ctx = M.Ctx(max_seq=CTX, n_seqs=B, kv_dtype=M.KV_BF16, kv_rank=0, kv_world=world, kv_block=256, max_batch=N_LAYERS * B)
    st = torch.cuda.Stream(device=dev)
    ctx.set_stream(st.cuda_stream)
    L0 = CTX - 64
    g = torch.Generator(device=dev)
    g.manual_seed(11)
    with torch.cuda.stream(st):
        kr, vr = torch.randn(8192, KV_DIM, device=dev, generator=g), torch.randn(8192, KV_DIM, device=dev, generator=g)
        for layer in FULL_LAYERS:
            for s_ in range(B):
                for p0 in range(0, L0, 8192):
                    ctx.kv_append_rows_dev(layer, s_, p0, min(8192, L0 - p0), kr.data_ptr(), vr.data_ptr())
        st.synchronize()
    items = [(l, s_) for s_ in range(B) for l in FULL_LAYERS]
    ng = len(items)
    layers, seqs = np.array([l for l, _ in items], np.int32), np.array([s_ for _, s_ in items], np.int32)
    q, kk, vv = (torch.randn(ng, n, device=dev, generator=g) for n in (Q_DIM, KV_DIM, KV_DIM))
    gate, out = torch.randn(ng, Q_DIM, device=dev, generator=g), torch.empty(ng, Q_DIM, device=dev)
    send = torch.empty(ng * (H * D + 2 * H), device=dev)
    pos = [L0]

    def step():
        p_ = np.full(ng, pos[0], np.int32)
        if world > 1:
            ctx.full_attn_partial_packed_dev(layers, seqs, p_, q.data_ptr(), kk.data_ptr(), vv.data_ptr(), send.data_ptr())
        else:
            ctx.full_attn_step_batched_dev(layers, seqs, p_, q.data_ptr(), gate.data_ptr(), kk.data_ptr(), vv.data_ptr(),
                                           out.data_ptr())
        pos[0] += 1

    with torch.cuda.stream(st):
        for _ in range(3):
            step()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(st)
        for _ in range(20):
            step()
        e1.record(st)
        st.synchronize()
        ctx.set_tuning("gqa_phase_trace", 1)
        step()
        st.synchronize()
    summarise(f"stack launch, 120 items, one rank of a {world}-way KV split (ctx {CTX}, bf16)", ctx,
              e0.elapsed_time(e1) / 20 * 1e3, ng * gqa_bytes_per_item(pos[0] / world, 2))
    ctx.close()

    # (b) a lone sequence: the launch is a latency problem
    for ctx_len, bf16, n_seqs in ((4096, False, 32), (32768, True, 8), (32768, False, 8)):
        c = M.Ctx(num_layers=4, max_seq=ctx_len + 200, n_seqs=n_seqs, kv_dtype=M.KV_BF16 if bf16 else M.KV_F32, max_batch=4)
        st = torch.cuda.Stream(device=dev)
        c.set_stream(st.cuda_stream)
        with torch.cuda.stream(st):
            for s_ in range(n_seqs):
                for p0 in range(0, ctx_len - 1, 8192):
                    c.kv_append_rows_dev(3, s_, p0, min(8192, ctx_len - 1 - p0), kr.data_ptr(), vr.data_ptr())
            st.synchronize()
        lens = [ctx_len - 1] * n_seqs

        def call(i):
            s_ = i % n_seqs
            c.full_attn_step_batched_dev([3], [s_], [lens[s_]], q.data_ptr(), gate.data_ptr(), kk.data_ptr(),
                                         vv.data_ptr(), out.data_ptr())
            lens[s_] += 1

        with torch.cuda.stream(st):
            for i in range(n_seqs):
                call(i)
            st.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            n = 64 * n_seqs
            e0.record(st)
            for i in range(n):
                call(i)
            e1.record(st)
            st.synchronize()
            c.set_tuning("gqa_phase_trace", 1)
            call(0)
            st.synchronize()
        summarise(f"one sequence, ctx {ctx_len}, {'bf16' if bf16 else 'fp32'} KV", c, e0.elapsed_time(e1) / n * 1e3,
                  gqa_bytes_per_item(ctx_len, 2 if bf16 else 4))
        c.close()
    return {"workload": "phase trace of the decode launch (%globaltimer stamps written by the kernel)", "cases": cases}


# --------------------------------------------------------------------------- ragged batch, sharded by sequence
RAGGED_SEQS = 64
RAGGED_LO, RAGGED_HI = 1024, 32768
RAGGED_LAYER = 3  # the full-attention layer of a 4-layer block


def ragged_lengths(seed=2):
    """The 64 seeded context lengths, U[1024, 32768]."""
    r = np.random.Generator(np.random.Philox(seed))
    return [int(x) for x in r.integers(RAGGED_LO, RAGGED_HI + 1, RAGGED_SEQS)]


def ragged_shards(lens, world):
    """Sequences dealt to `world` ranks greedily, longest first, each to the rank with the fewest rows so far."""
    load = [0] * world
    shards = [[] for _ in range(world)]
    for s in sorted(range(len(lens)), key=lambda i: (-lens[i], i)):
        rk = min(range(world), key=lambda k: (load[k], k))
        shards[rk].append(s)
        load[rk] += lens[s]
    return shards, load


def ragged_config(args, n):
    lens = ragged_lengths()
    return {"workload": f"{RAGGED_SEQS} independent sequences, ragged contexts U[{RAGGED_LO},{RAGGED_HI}] (seeded: "
                        f"{sum(lens)} cached rows in all), one full-attention GQA layer-step each per step, bf16 KV, "
                        f"fp32 accumulate",
            "layer_steps_per_step": RAGGED_SEQS, "rows_total": sum(lens), "kv_dtype": "bf16",
            "parallelism": (f"sequences dealt over {n} ranks greedily, longest first; no exchange in the data path, the "
                            f"outputs are gathered (one NCCL all-gather of 32 KiB per sequence per step, running under the "
                            f"next step's kernel)") if n > 1 else "single GPU",
            "l2": "the KV rows of a step (2.2 GB in all) exceed the 126 MB L2; no flush needed"}


def cpu_sample_ragged(args, kind, seed=4):
    """CPU statement of the ragged batch on a bounded sample: four of the 64 sequences (shortest, two middle,
    longest), scaled by cached rows to the whole batch."""
    import oracle as O
    from oracle import A17B as G

    O.build()
    lens = ragged_lengths()
    order = sorted(range(RAGGED_SEQS), key=lambda i: lens[i])
    sample = [order[0], order[21], order[42], order[-1]]
    r = np.random.Generator(np.random.Philox(seed))
    nrm = lambda *s: r.standard_normal(s, dtype=np.float32)
    t_total, rows = 0.0, 0
    if kind == "reference":
        import oracle.ref as R
        from concurrent.futures import ThreadPoolExecutor

        threads = _host_threads()
        caches = {s: (O.round_bf16(nrm(lens[s] + 1, KV_DIM)), O.round_bf16(nrm(lens[s] + 1, KV_DIM))) for s in sample}
        jobs = [sample[i % len(sample)] for i in range(max(threads, len(sample)))]
        ins = {s: (nrm(Q_DIM), nrm(Q_DIM), nrm(KV_DIM), nrm(KV_DIM)) for s in sample}  # jobs of a sequence append equal rows

        def run(i):
            s = jobs[i]
            Kc, Vc = caches[s]
            R.full_attn_step(lens[s], lens[s], *ins[s], Kc, Vc, H, HKV, D, G.rotary_dim)

        with ThreadPoolExecutor(threads) as ex:
            t0 = time.perf_counter()
            list(ex.map(run, range(len(jobs))))
            t_total = time.perf_counter() - t0
        rows = sum(lens[s] + 1 for s in jobs)
        cores = threads
        how = f"the reference's own C functions (single-threaded each), {len(jobs)} layer-steps side by side on {threads} threads"
    else:
        O.use_all_cores()
        for s in sample:
            Kc, Vc = O.round_bf16(nrm(lens[s] + 1, KV_DIM)), O.round_bf16(nrm(lens[s] + 1, KV_DIM))
            ins = (nrm(Q_DIM), nrm(Q_DIM), nrm(KV_DIM), nrm(KV_DIM))
            t0 = time.perf_counter()
            O.full_attn_step(lens[s], lens[s], *ins, Kc, Vc, G, kv_bf16=True)
            t_total += time.perf_counter() - t0
            rows += lens[s] + 1
        cores = O.num_threads()
        how = "the C restatement (oracle/mf_oracle.c, OpenMP over heads), one layer-step at a time"
    t_step = t_total * (sum(lens) + RAGGED_SEQS) / rows
    desc = (f"{how}: sequences of {[lens[s] for s in sample]} rows, {rows} rows in {t_total * 1e3:.0f} ms, scaled by rows "
            f"to the {RAGGED_SEQS} sequences ({sum(lens)} rows)")
    return RAGGED_SEQS / t_step, cores, desc, kind


def run_ragged(args, rank, world, local_rank):
    """64 ragged sequences, one full-attention layer-step each per step, sharded by sequence."""
    import torch
    import torch.distributed as dist

    import moeflux_b200 as M

    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    W, K = args.warmup, args.steps
    lens = ragged_lengths()
    shards, load = ragged_shards(lens, world)
    mine = shards[rank]
    n = len(mine)
    n_max = max(len(x) for x in shards)
    R = args.repeats or repeats_for(K, 0.33 * max(load) / sum(lens))
    do_e2e = not args.no_e2e
    We, Re = (min(W, 3), min(R, 7)) if do_e2e else (0, 0)
    total_steps = W + R * K + We + Re * K + 1
    ctx = M.Ctx(num_layers=4, max_seq=RAGGED_HI + total_steps, n_seqs=max(n, 1), kv_dtype=M.KV_BF16, device=local_rank,
                max_batch=max(n, 1))
    stream = torch.cuda.Stream(device=dev)
    ctx.set_stream(stream.cuda_stream)
    gen = torch.Generator(device=dev)
    CH = 8192

    def kv_rows(s, p0, cnt):
        gen.manual_seed(7000000 + s * 64 + p0 // CH)
        return (torch.randn(cnt, KV_DIM, device=dev, generator=gen), torch.randn(cnt, KV_DIM, device=dev, generator=gen))

    with torch.cuda.stream(stream):
        for j, s in enumerate(mine):
            for p0 in range(0, lens[s], CH):
                cnt = min(CH, lens[s] - p0)
                kr, vr = kv_rows(s, p0, cnt)
                ctx.kv_append_rows_dev(RAGGED_LAYER, j, p0, cnt, kr.data_ptr(), vr.data_ptr())
                stream.synchronize()
        gen.manual_seed(4242)
        q_all = torch.randn(RAGGED_SEQS, Q_DIM, device=dev, generator=gen)
        gate_all = torch.randn(RAGGED_SEQS, Q_DIM, device=dev, generator=gen)
        k_all = torch.randn(RAGGED_SEQS, KV_DIM, device=dev, generator=gen)
        v_all = torch.randn(RAGGED_SEQS, KV_DIM, device=dev, generator=gen)
        idx = torch.tensor(mine, device=dev, dtype=torch.long)
        q, gate, kk, vv = (t[idx].contiguous() for t in (q_all, gate_all, k_all, v_all))
        # this rank's outputs, padded to the largest shard; two buffers, so that the gather of one step runs under
        # the kernel of the next (the next step does not depend on the gathered outputs)
        out_bufs = [torch.zeros(n_max, Q_DIM, device=dev) for _ in range(2)]
        gath_bufs = [torch.empty(world * n_max, Q_DIM, device=dev) for _ in range(2)] if world > 1 else None
        out_pad, gathered = out_bufs[0], (gath_bufs[0] if world > 1 else None)
    stream.synchronize()
    layers = np.full(n, RAGGED_LAYER, np.int32)
    seqs = np.arange(n, dtype=np.int32)
    step_no = [0]
    ev = lambda: torch.cuda.Event(enable_timing=True)
    k_events = []

    pending = [None, None]  # the gather that last used each buffer pair

    # a step of a rank is well under 0.1 ms at 8 GPUs: the host side of it is kept to a handful of calls (positions
    # bumped in place, pointers looked up once, the kernel's own events on every eighth timed step only)
    pos0 = np.array([lens[s] for s in mine], np.int32)
    pos = pos0.copy()
    ptrs = (q.data_ptr(), gate.data_ptr(), kk.data_ptr(), vv.data_ptr())
    out_ptrs = [o.data_ptr() for o in out_bufs]
    tab_ptrs = (layers.ctypes.data, seqs.ctypes.data, pos.ctypes.data)
    n_timed = [0]

    def device_step(timed):
        b = step_no[0] & 1
        np.add(pos0, step_no[0], out=pos)
        if pending[b] is not None:
            pending[b].wait()  # the stream waits for the gather that still reads this output buffer
            pending[b] = None
        sample = timed and (n_timed[0] & 7) == 0
        if timed:
            n_timed[0] += 1
        if sample:
            e0, e1 = ev(), ev()
            e0.record(stream)
        ctx.full_attn_step_batched_dev_ptr(n, tab_ptrs[0], tab_ptrs[1], tab_ptrs[2], *ptrs, out_ptrs[b])
        if sample:
            e1.record(stream)
            k_events.append((e0, e1))
        if world > 1:
            pending[b] = dist.all_gather_into_tensor(gath_bufs[b], out_bufs[b], async_op=True)
        step_no[0] += 1

    def barrier():
        for b in range(2):  # a block ends when its last gathers have landed
            if pending[b] is not None:
                pending[b].wait()
                pending[b] = None
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    sampler = ClockSampler(local_rank) if rank == 0 else None
    blocks = []
    with torch.cuda.stream(stream):
        for _ in range(W):
            device_step(False)
        if sampler:
            sampler.start()
            time.sleep(0.3)
        launches0 = ctx.launch_count
        t_wall0 = time.time()
        first_timed = step_no[0]
        for _ in range(R):
            barrier()
            start, stop = ev(), ev()
            start.record(stream)
            for _ in range(K):
                device_step(True)
            stop.record(stream)
            barrier()
            blocks.append(start.elapsed_time(stop))
        t_wall1 = time.time()
        launches = (ctx.launch_count - launches0) // R
    ctx.synchronize()
    k_ms = sum(a.elapsed_time(b) for a, b in k_events) / len(k_events)
    t = torch.tensor(blocks + [k_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    blocks, k_ms = [float(x) for x in t[:R]], float(t[R])
    ms = statistics.median(blocks)
    clocks = sampler.stop(t_wall0, t_wall1) if sampler else None

    e2e = None
    if do_e2e:
        pin = lambda *shape: torch.empty(*shape, dtype=torch.float32).pin_memory()
        hq, hgate, hk, hv, hout = pin(n, Q_DIM), pin(n, Q_DIM), pin(n, KV_DIM), pin(n, KV_DIM), pin(n, Q_DIM)
        for h, d_ in ((hq, q), (hgate, gate), (hk, kk), (hv, vv)):
            h.copy_(d_.cpu())

        def e2e_step():
            pos = np.array([lens[s] + step_no[0] for s in mine], np.int32)
            ctx.full_attn_step_batched_ptr(n, layers.ctypes.data, seqs.ctypes.data, pos.ctypes.data, hq.data_ptr(),
                                           hgate.data_ptr(), hk.data_ptr(), hv.data_ptr(), hout.data_ptr())
            step_no[0] += 1

        for _ in range(We):
            e2e_step()
        e_blocks = []
        for _ in range(Re):
            barrier()
            t0 = time.perf_counter()
            for _ in range(K):
                e2e_step()
            barrier()
            e_blocks.append(time.perf_counter() - t0)
        if world > 1:
            te = torch.tensor(e_blocks, device=dev, dtype=torch.float64)
            dist.all_reduce(te, op=dist.ReduceOp.MAX)
            e_blocks = [float(x) for x in te]
        dt = statistics.median(e_blocks)
        e2e = {"value": RAGGED_SEQS * K / dt, "unit": "layer-steps/s", "h2d_bytes_per_step": 4 * n * (2 * Q_DIM + 2 * KV_DIM),
               "d2h_bytes_per_step": 4 * n * Q_DIM, "ms_per_step": 1e3 * dt / K, "steps": K, "repeats": Re,
               "api": "mfc_full_attn_step_batched (host pointers; each rank's shard, results stay on the rank's host)",
               "bytes_are": "this rank's"}

    # parity: the step after the timed region, this rank's shortest and longest sequence against the oracle
    parity = None
    with torch.cuda.stream(stream):
        final = step_no[0]
        device_step(False)
        out_pad, gathered = out_bufs[final & 1], (gath_bufs[final & 1] if world > 1 else None)
        barrier()
    ctx.synchronize()
    if rank == 0 and n:
        import oracle as O
        from oracle import A17B as G

        O.build()
        O.use_all_cores()
        by_len = sorted(range(n), key=lambda j: lens[mine[j]])
        worst = 0.0
        zq = np.zeros(Q_DIM, np.float32)
        for j in sorted({by_len[0], by_len[-1]}):
            s = mine[j]
            rows = lens[s] + final
            Kh = np.empty((rows + 1, KV_DIM), np.float32)
            Vh = np.empty((rows + 1, KV_DIM), np.float32)
            for p0 in range(0, lens[s], CH):
                cnt = min(CH, lens[s] - p0)
                kr, vr = kv_rows(s, p0, cnt)
                Kh[p0:p0 + cnt] = kr.cpu().numpy()
                Vh[p0:p0 + cnt] = vr.cpu().numpy()
            k_in, v_in = kk[j].cpu().numpy(), vv[j].cpu().numpy()
            for p in range(lens[s], rows):
                Kh[p] = O.apply_rotary_emb(p, zq, k_in)[1]
                Vh[p] = v_in
            Kh[:rows] = O.round_bf16(Kh[:rows])
            Vh[:rows] = O.round_bf16(Vh[:rows])
            ref = O.full_attn_step(rows, rows, q[j].cpu().numpy(), gate[j].cpu().numpy(), k_in, v_in, Kh, Vh, G, kv_bf16=True)
            got = out_pad[j].cpu().numpy()
            worst = max(worst, float(np.max(np.abs(got - ref)) / max(np.max(np.abs(ref)), 1e-30)))
            if world > 1:  # and the gathered copy of the same row
                gg = gathered[rank * n_max + j].cpu().numpy()
                worst = max(worst, float(np.max(np.abs(gg - ref)) / max(np.max(np.abs(ref)), 1e-30)))
        parity = {"max_rel_err": worst, "items": 2, "tol": 2e-2, "ok": bool(worst <= 2e-2),
                  "what": "rank 0's shortest and longest sequence, the step after the timed region, vs the CPU oracle"}

    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        peak, peak_src = float(json.load(open(peaks_path))["hbm_gbs"]), "MEASURED_PEAKS.json hbm_gbs (of measured)"
    else:
        peak, peak_src = 6650.0, "fallback 6.65 TB/s (of fallback)"
    mean_step = first_timed + (R * K - 1) / 2.0
    # the slowest rank sets the time: its rows are what the launch time is compared with
    shard_rows = max(sum(lens[s] + mean_step + 1 for s in sh) for sh in shards)
    n_slow = max(len(sh) for sh in shards)
    alg = 2 * shard_rows * KV_DIM * 2 + n_slow * (3 * Q_DIM * 4 + 2 * KV_DIM * 4 + 2 * KV_DIM * 2)
    achieved = alg / (k_ms * 1e-3) / 1e9
    line = None
    if rank == 0:
        line = {"metric": "attention decode layer-steps/sec", "value": RAGGED_SEQS * K / (ms * 1e-3), "unit": "layer-steps/s",
                "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": ms / K, "higher_is_better": True,
                "scaling": "strong", "vs_baseline": None, "dtype": "bf16 KV, fp32 accumulate", "data": "synthetic",
                "config": ragged_config(args, world), "repeats": R,
                "min": RAGGED_SEQS * K / (max(blocks) * 1e-3), "max": RAGGED_SEQS * K / (min(blocks) * 1e-3),
                "value_is": f"median of {R} timed blocks of {K} steps (CUDA events, slowest rank per block)",
                "shard_rows": load,
                "roofline": {"bound": "hbm", "kernel": "gqa_decode_bf16_kernel", "achieved": achieved, "peak": peak,
                             "unit": "GB/s", "frac": achieved / peak, "traffic": alg * 1.009, "peak_source": peak_src,
                             "algorithmic_bytes_per_launch": alg, "ms_per_launch": k_ms,
                             "frac_of_8TBps": achieved / 8000.0, "launch_is": "the largest shard's"},
                "e2e": e2e, "parity": parity, "gpu_launches": int(launches), "clocks": clocks}
    ctx.close()
    return line


# --------------------------------------------------------------------------- prefill workload
def run_prefill(args):
    """Chunked prefill of one hybrid block (3 GatedDeltaNet layers + 1 causal GQA layer), bf16
    activations, seeded N(0,1) inputs; single GPU.  A step = the four prefill calls on an empty state."""
    import torch

    import moeflux_b200 as M

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    T, K, W = args.tokens, args.steps, args.warmup
    ctx = M.Ctx(num_layers=4, max_seq=T, n_seqs=1, kv_dtype=M.KV_BF16, max_prefill=T)
    stream = torch.cuda.Stream(device=dev)
    ctx.set_stream(stream.cuda_stream)
    rs = np.random.Generator(np.random.Philox(78))
    bits = lambda a: torch.tensor(np.asarray(a, np.float32)).bfloat16().view(torch.int16).numpy().astype(np.uint16)
    for layer in range(3):
        ctx.set_linear_weights(layer, bits(rs.standard_normal((CONV_DIM, 4), dtype=np.float32) * 0.5),
                               rs.uniform(0, 2.7, HV).astype(np.float32), bits(rs.standard_normal(HV, dtype=np.float32)),
                               bits(1 + 0.1 * rs.standard_normal(DK, dtype=np.float32)))
    gen = torch.Generator(device=dev)
    gen.manual_seed(3)
    bf = lambda *shape: torch.randn(*shape, device=dev, generator=gen).bfloat16()
    with torch.cuda.stream(stream):
        lin_in = [(bf(T, CONV_DIM), bf(T, V_DIM), bf(T, HV), bf(T, HV)) for _ in range(3)]
        lin_out = [torch.empty(T, V_DIM, device=dev, dtype=torch.bfloat16) for _ in range(3)]
        q, gate, k, v = bf(T, Q_DIM), bf(T, Q_DIM), bf(T, KV_DIM), bf(T, KV_DIM)
        out = torch.empty(T, Q_DIM, device=dev, dtype=torch.bfloat16)
    stream.synchronize()
    ev = lambda: torch.cuda.Event(enable_timing=True)
    t_lin, t_att, t_all = [], [], []
    sampler = ClockSampler(0)
    with torch.cuda.stream(stream):
        for it in range(W + K):
            ctx.memory_clear(0)
            if it == W:
                sampler.start()
                time.sleep(0.3)
                launches0 = ctx.launch_count
                t0 = time.time()
            e0, e1, e2 = ev(), ev(), ev()
            e0.record(stream)
            for layer in range(3):
                x, z, a, b = lin_in[layer]
                ctx.linear_attn_prefill_dev(layer, 0, T, x.data_ptr(), z.data_ptr(), a.data_ptr(), b.data_ptr(),
                                            lin_out[layer].data_ptr())
            e1.record(stream)
            ctx.full_attn_prefill_dev(3, 0, 0, T, q.data_ptr(), gate.data_ptr(), k.data_ptr(), v.data_ptr(),
                                      out.data_ptr())
            e2.record(stream)
            stream.synchronize()
            if it >= W:
                t_lin.append(e0.elapsed_time(e1))
                t_att.append(e1.elapsed_time(e2))
                t_all.append(e0.elapsed_time(e2))
    ctx.synchronize()
    clocks = sampler.stop(t0, time.time())
    launches = ctx.launch_count - launches0
    ms, ms_att, ms_lin = sum(t_all) / K, sum(t_att) / K, sum(t_lin) / K
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    peak = float(json.load(open(peaks_path))["bf16_tflops_sustained"]) if os.path.exists(peaks_path) else 1400.0
    att_flops = 4.0 * H * D * T * (T + 1) / 2            # QK^T and PV over the causal half
    chunk = 64
    gdn_flops_chunk = 2.0 * (2 * chunk * chunk * DK + 2 * chunk * DK * DK + chunk * chunk * DK + DK * chunk * DK)
    gdn_flops = 3 * HV * ((T + chunk - 1) // chunk) * gdn_flops_chunk
    line = {"metric": "chunked prefill tokens/sec (hybrid block: 3 GatedDeltaNet + 1 causal GQA layer)",
            "value": T / (ms * 1e-3), "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W, "ms_per_step": ms,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16 activations and KV, fp32 accumulate and state", "data": "synthetic",
            "config": {"workload": f"chunked prefill of {T} tokens, 3 GatedDeltaNet layers (chunk 64) + 1 causal GQA layer",
                       "tokens": T},
            "roofline": {"bound": "tensor", "kernel": "gqa_prefill_kernel (tcgen05)", "achieved": att_flops / (ms_att * 1e-3) / 1e12,
                         "peak": peak, "unit": "TFLOP/s", "frac": att_flops / (ms_att * 1e-3) / 1e12 / peak,
                         "traffic": None, "peak_source": "MEASURED_PEAKS.json bf16_tflops_sustained (of measured)",
                         "ms_per_launch": ms_att, "flops_per_launch": att_flops,
                         "other_kernels": {"gdn_prefill (3 layers)": {"ms": ms_lin, "flops": gdn_flops,
                                                                      "achieved": gdn_flops / (ms_lin * 1e-3) / 1e12}}},
            "e2e": None, "gpu_launches": int(launches), "clocks": clocks}
    ctx.close()
    return line


# --------------------------------------------------------------------------- projection (matvec) workload
def run_matvec(args):
    """The 4-bit group-64 projections on either side of the attention sub-blocks of one hybrid block (3
    GatedDeltaNet layers + 1 full-attention layer, hidden 4096) for one decode token (or --vecs tokens): per
    full layer q_proj 4096->16384, k_proj and v_proj 4096->512, o_proj 8192->4096; per GatedDeltaNet layer
    in_proj_qkv 4096->12288, in_proj_z 4096->8192, in_proj_a / in_proj_b 4096->64, out_proj 8192->4096.
    A step = all 24 products in 8 launches (products that share their input go together); the weights of the block (258 MB) exceed L2, so every step streams them from HBM."""
    import torch

    import moeflux_b200 as M

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    K, W, NV = max(args.steps, 200), args.warmup, args.vecs  # a step is under 0.1 ms: at least 200 of them are timed
    full = [(4096, 16384), (4096, 512), (4096, 512), (8192, 4096)]
    lin = [(4096, 12288), (4096, 8192), (4096, 64), (4096, 64), (8192, 4096)]
    shapes = lin * 3 + full
    ctx = M.Ctx(num_layers=4, max_seq=64, n_seqs=1, kv_dtype=M.KV_BF16)
    stream = torch.cuda.Stream(device=dev)
    ctx.set_stream(stream.cuda_stream)
    gen = torch.Generator(device=dev)
    gen.manual_seed(2024)
    ops = []
    with torch.cuda.stream(stream):
        for in_dim, out_dim in shapes:
            w = torch.randint(-2**31, 2**31 - 1, (out_dim, in_dim // 8), device=dev, dtype=torch.int32, generator=gen)
            sc = (torch.randn(out_dim, in_dim // 64, device=dev, generator=gen).abs() * 0.02 + 1e-3).bfloat16()
            bi = (-8.0 * sc.float() + 0.01 * torch.randn(out_dim, in_dim // 64, device=dev, generator=gen)).bfloat16()
            x = torch.randn(NV, in_dim, device=dev, generator=gen)
            out = torch.empty(NV, out_dim, device=dev)
            ops.append((w, sc, bi, in_dim, out_dim, x, out))
    stream.synchronize()
    weight_bytes = sum(o * i // 2 + 2 * 2 * o * (i // 64) for i, o in shapes)
    io_bytes = sum(4 * NV * (i + o) for i, o in shapes)

    # projections of a layer that share their input go into one launch (q/k/v_proj; in_proj_qkv/z/a/b), as the
    # reference encodes them into one command buffer; o_proj / out_proj have their own input
    groups = []
    for base, n_in, n_all in [(0, 4, 5), (5, 4, 5), (10, 4, 5), (15, 3, 4)]:
        groups.append(list(range(base, base + n_in)))
        groups.append(list(range(base + n_in, base + n_all)))

    def step():
        for idx in groups:
            sel = [ops[k] for k in idx]
            ctx.dequant_matvec_4bit_multi_dev([o[0].data_ptr() for o in sel], [o[1].data_ptr() for o in sel],
                                              [o[2].data_ptr() for o in sel], sel[0][3], [o[4] for o in sel],
                                              sel[0][5].data_ptr(), NV, [o[6].data_ptr() for o in sel])

    sampler = ClockSampler(0)
    with torch.cuda.stream(stream):
        for _ in range(W):
            step()
        stream.synchronize()
    # the 24 launches of a step are a few microseconds each: replayed as one CUDA graph, as a decode loop would
    graph = torch.cuda.CUDAGraph()
    launches0 = ctx.launch_count
    with torch.cuda.graph(graph, stream=stream):
        step()
    launches_per_step = ctx.launch_count - launches0
    with torch.cuda.stream(stream):
        graph.replay()
        stream.synchronize()
        sampler.start()
        time.sleep(0.3)
        t0 = time.time()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(K):
            graph.replay()
        e1.record(stream)
        stream.synchronize()
    ctx.synchronize()
    clocks = sampler.stop(t0, time.time())
    launches = launches_per_step * K
    ms = e0.elapsed_time(e1) / K
    # end to end: host vectors in, host results out, weights resident (they are model state)
    hx = [torch.empty(NV, i).normal_().pin_memory() for i, _ in shapes]
    ho = [torch.empty(NV, o).pin_memory() for _, o in shapes]

    def e2e_step():
        with torch.cuda.stream(stream):
            for idx in groups:  # one input per group, every product's result back to the host
                ops[idx[0]][5].copy_(hx[idx[0]], non_blocking=True)
            step()
            for k, op in enumerate(ops):
                ho[k].copy_(op[6], non_blocking=True)
            stream.synchronize()

    for _ in range(3):
        e2e_step()
    t1 = time.perf_counter()
    for _ in range(K):
        e2e_step()
    dt = (time.perf_counter() - t1) / K
    # parity: a GatedDeltaNet in-projection, a 8192-wide out-projection and the small k_proj against the CPU oracle
    import oracle as O

    O.build()
    O.use_all_cores()
    worst = 0.0
    checked = (0, 4, 16)
    x_of = {k: ops[idx[0]][5] for idx in groups for k in idx}  # the products of a launch share the first one's input
    for k in checked:
        w, sc, bi, in_dim, out_dim, _, out = ops[k]
        xk = x_of[k]
        pk = w.cpu().numpy().view(np.uint32)
        scn = sc.view(torch.int16).cpu().numpy().view(np.uint16)
        bin_ = bi.view(torch.int16).cpu().numpy().view(np.uint16)
        for v in range(NV):
            ref = O.dequant_matvec_4bit(pk, scn, bin_, in_dim, out_dim, xk[v].cpu().numpy())
            got = out[v].cpu().numpy()
            worst = max(worst, float(np.max(np.abs(got - ref)) / max(np.max(np.abs(ref)), 1e-30)))
    parity = {"max_rel_err": worst, "tol": 1e-4, "items": len(checked) * NV, "ok": bool(worst <= 1e-4),
              "what": "in_proj_qkv 4096->12288, out_proj 8192->4096 and k_proj 4096->512 of the last replay vs the CPU oracle"}
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    peak = float(json.load(open(peaks_path))["hbm_gbs"]) if os.path.exists(peaks_path) else 6650.0
    achieved = (weight_bytes + io_bytes) / (ms * 1e-3) / 1e9
    line = {"metric": "4-bit projection products/sec (attention sub-block projections of one hybrid block)",
            "value": len(shapes) * NV / (ms * 1e-3), "unit": "matvec/s", "n_gpus": 1, "steps": K, "warmup": W,
            "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "u4 weights, bf16 scales and biases, f32 vectors and accumulate", "data": "synthetic",
            "config": {"workload": f"24 group-64 4-bit projections of a hybrid block (3 GatedDeltaNet + 1 full layer, hidden "
                                   f"4096), {NV} vector(s) each; 258 MB of weights per step, larger than L2", "vecs": NV},
            "roofline": {"bound": "hbm", "kernel": "dequant_matvec_4bit_stream_kernel" if NV == 1 else f"dequant_matvec_4bit_mma_kernel<{NV}>",
                         "achieved": achieved, "peak": peak,
                         "unit": "GB/s", "frac": achieved / peak, "traffic": None,
                         "peak_source": "MEASURED_PEAKS.json hbm_gbs (of measured)",
                         "algorithmic_bytes_per_step": weight_bytes + io_bytes, "frac_of_8TBps": achieved / 8000.0},
            "e2e": {"value": len(shapes) * NV / dt, "unit": "matvec/s", "h2d_bytes_per_step": sum(4 * NV * shapes[g[0]][0] for g in groups),
                    "d2h_bytes_per_step": sum(4 * NV * o for _, o in shapes)},
            "parity": parity, "gpu_launches": int(launches), "clocks": clocks}
    ctx.close()
    return line


# --------------------------------------------------------------------------- folded MLA attention
def run_mla(args):
    """Folded MLA SDPA of one decode token (the third attention flavour): 128 heads, latent rank 512 + 64 rope dims,
    fp32 latent cache of --ctx positions (default 32768: 75 MB), seeded N(0,1) cache rows and N(0,0.3) queries.  A step
    = one call; the calls rotate over four caches (together more than twice the L2).  Single GPU."""
    import torch

    import moeflux_b200 as M
    import oracle as O

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    Hm, RANK, ROPE = 128, 512, 64
    n = args.ctx if args.ctx != 131072 else 32768
    K, W = args.steps, args.warmup
    scale = float(1.0 / np.sqrt(np.float32(192.0)))
    bf16 = args.mla_cache == "bf16"
    esize = 2 if bf16 else 4
    tol = 2e-2 if bf16 else 1e-3
    ctx = M.Ctx(num_layers=4, max_seq=64)
    st = torch.cuda.Stream(device=dev)
    ctx.set_stream(st.cuda_stream)
    g = torch.Generator(device=dev)
    g.manual_seed(31)
    n_caches = 4
    with torch.cuda.stream(st):
        lat = [torch.randn(n, RANK, device=dev, generator=g) for _ in range(n_caches)]
        rk = [torch.randn(n, ROPE, device=dev, generator=g) for _ in range(n_caches)]
        if bf16:
            lat = [x.to(torch.bfloat16).contiguous() for x in lat]
            rk = [x.to(torch.bfloat16).contiguous() for x in rk]
        qp = torch.randn(Hm, RANK, device=dev, generator=g) * 0.3
        pe = torch.randn(Hm, ROPE, device=dev, generator=g) * 0.3
        out = torch.empty(Hm, RANK, device=dev)
    st.synchronize()
    fn = ctx.mla_sdpa_folded_bf16_dev if bf16 else ctx.mla_sdpa_folded_dev
    call = lambda i: fn(Hm, n, scale, qp.data_ptr(), pe.data_ptr(), lat[i % n_caches].data_ptr(),
                        rk[i % n_caches].data_ptr(), out.data_ptr())
    R = args.repeats or 7
    sampler = ClockSampler(0)
    blocks = []
    with torch.cuda.stream(st):
        for i in range(max(W, n_caches)):
            call(i)
        st.synchronize()
        sampler.start()
        time.sleep(0.3)
        t0 = time.time()
        launches0 = ctx.launch_count
        for _ in range(R):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(st)
            for i in range(K):
                call(i)
            e1.record(st)
            st.synchronize()
            blocks.append(e0.elapsed_time(e1))
        launches = (ctx.launch_count - launches0) // R
    ctx.synchronize()
    clocks = sampler.stop(t0, time.time())
    ms = statistics.median(blocks) / K
    # end to end: the query of the token from pinned host memory, the result back; the cache is model state
    hq, hp, ho = (torch.empty(Hm, d).pin_memory() for d in (RANK, ROPE, RANK))
    hq.copy_(qp.cpu())
    hp.copy_(pe.cpu())

    def e2e_step(i):
        with torch.cuda.stream(st):
            qp.copy_(hq, non_blocking=True)
            pe.copy_(hp, non_blocking=True)
            call(i)
            ho.copy_(out, non_blocking=True)
            st.synchronize()

    for i in range(3):
        e2e_step(i)
    t1 = time.perf_counter()
    for i in range(K):
        e2e_step(i)
    dt = (time.perf_counter() - t1) / K
    # parity: the last e2e result against the oracle on the same cache
    last = (K - 1) % n_caches
    ref = O.mla_sdpa_folded(n, scale, hq.numpy(), hp.numpy(), lat[last].float().cpu().numpy(), rk[last].float().cpu().numpy())
    err = float(np.max(np.abs(ho.numpy() - ref)) / max(np.max(np.abs(ref)), 1e-30))
    # CPU arm: the oracle (the reference's C engine has no MLA twin) on the full problem, once
    O.use_all_cores()
    tc = time.perf_counter()
    O.mla_sdpa_folded(n, scale, hq.numpy(), hp.numpy(), lat[0].float().cpu().numpy(), rk[0].float().cpu().numpy())
    tc = time.perf_counter() - tc
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    peak = float(json.load(open(peaks_path))["hbm_gbs"]) if os.path.exists(peaks_path) else 6650.0
    alg = n * (RANK + ROPE) * esize + Hm * (2 * RANK + ROPE) * 4
    flops = 2.0 * Hm * n * (RANK + ROPE + RANK)
    achieved = alg / (ms * 1e-3) / 1e9
    line = {"metric": "folded MLA attention steps/sec (128 heads, one decode token)", "value": 1e3 / ms, "unit": "steps/s",
            "n_gpus": 1, "steps": K, "warmup": W, "ms_per_step": ms, "repeats": R, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16 cache, bf16 products, f32 accumulate" if bf16 else "f32 cache, two-piece bf16 products, f32 accumulate",
            "data": "synthetic",
            "config": {"workload": f"folded MLA SDPA, 128 heads, rank 512 + rope 64, {args.mla_cache} latent cache of {n} positions "
                                   f"({alg / 1e6:.0f} MB per call), four caches rotated (more than the 126 MB L2)", "context": n},
            "roofline": {"bound": "hbm", "kernel": "mla_decode_bf16_kernel" if bf16 else "mla_decode_kernel", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "traffic": None, "peak_source": "MEASURED_PEAKS.json hbm_gbs (of measured)",
                         "algorithmic_bytes_per_launch": alg, "ms_per_launch": ms, "frac_of_8TBps": achieved / 8000.0,
                         "tensor_TFLOPs_useful": flops / (ms * 1e-3) / 1e12,
                         "note": "121 (fp32 cache; x3 with the two-piece expansion) or 242 (bf16 cache) useful flop per cached byte "
                                 "on mma.sync: bound by the legacy tensor pipe before HBM; the tcgen05 form is the next step"},
            "e2e": {"value": 1.0 / dt, "unit": "steps/s", "h2d_bytes_per_step": 4 * Hm * (RANK + ROPE),
                    "d2h_bytes_per_step": 4 * Hm * RANK},
            "parity": {"max_rel_err": err, "tol": tol, "items": 1, "ok": bool(err <= tol),
                       "what": "one call's v_combine against the CPU oracle on the same cache (the reference's GPU-vs-CPU bound)"},
            "cpu_baseline": {"value": 1.0 / tc, "unit": "steps/s", "cores": O.num_threads(), "kind": "port",
                             "sample": f"one call at the full size with the C restatement (OpenMP over heads): {tc * 1e3:.0f} ms"},
            "gpu_launches": int(launches), "clocks": clocks}
    ctx.close()
    return line


def compact(line):
    """The fields of a workload's line that matter when it rides along in another line."""
    if not line:
        return None
    r = line.get("roofline") or {}
    return {"metric": line["metric"], "value": line["value"], "unit": line["unit"], "ms_per_step": line["ms_per_step"],
            "steps": line["steps"], "repeats": line.get("repeats"), "config": line["config"].get("workload"),
            "roofline": {k: r.get(k) for k in ("bound", "kernel", "achieved", "peak", "unit", "frac", "ms_per_launch")},
            "e2e": (line.get("e2e") or {}).get("value"), "parity": line.get("parity")}


_LINE_FD = None


def emit(line):
    """The one JSON line, to the process's real standard output."""
    data = (json.dumps(line) + "\n").encode()
    if _LINE_FD is None:
        sys.stdout.write(data.decode())
        sys.stdout.flush()
    else:
        os.write(_LINE_FD, data)


def main():
    # Libraries (NCCL's version banner, for one) write to file descriptor 1 behind Python's back: everything but the
    # JSON line goes to standard error, so that standard output carries that line alone.
    global _LINE_FD
    sys.stdout.flush()
    _LINE_FD = os.dup(1)
    os.dup2(2, 1)
    args = parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    import torch
    import torch.distributed as dist

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path "
                         "(use --impl reference for the CPU restatement)")
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    if world != args.gpus and rank == 0:
        print(f"warning: --gpus {args.gpus} but WORLD_SIZE={world}; using {world}", file=sys.stderr)
    if args.workload == "prefill":
        if rank == 0:
            emit(run_prefill(args))
        return
    if args.workload == "matvec":
        if rank == 0:
            line = run_matvec(args)
            emit(line)
            if not line["parity"]["ok"]:
                raise SystemExit("parity check failed: " + json.dumps(line["parity"]))
        return
    if args.workload == "trace":
        if rank == 0:
            emit(run_trace(args))
        return
    if args.workload == "mla":
        if rank == 0:
            line = run_mla(args)
            emit(line)
            if not line["parity"]["ok"]:
                raise SystemExit("parity check failed: " + json.dumps(line["parity"]))
        return
    line = run_ragged(args, rank, world, local_rank) if args.workload == "ragged" else run_ours(args, rank, world, local_rank)
    others = {}
    if args.workload == "stack" and args.other_configs:
        others["ragged (configuration 2)"] = compact(run_ragged(args, rank, world, local_rank))
        if world == 1:
            others["prefill (configuration 3)"] = compact(run_prefill(args))
            others["4-bit projections of a hybrid block"] = compact(run_matvec(args))
            others["folded MLA attention, fp32 cache"] = compact(run_mla(args))
    failed = False
    if rank == 0:
        if world == 1 and not args.no_cpu_baseline:
            kind = reference_kind()
            if args.workload == "ragged":
                v, cores, desc, kind = cpu_sample_ragged(args, kind)
            else:
                v, cores, desc, kind = cpu_sample(args.ctx, args.batch, kind=kind)
            line["cpu_baseline"] = {"value": v, "unit": "layer-steps/s", "cores": cores, "kind": kind, "sample": desc}
        if world == 1 and args.workload == "stack" and not args.no_single_step:
            line["roofline"]["single_step"] = single_step_latencies(local_rank)
        if others:
            line["other_configs"] = others
        emit(line)
        failed = (bool(line.get("parity")) and not line["parity"]["ok"]) or any(
            o and o.get("parity") and not o["parity"]["ok"] for o in others.values())
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if failed:
        raise SystemExit("parity check failed: " + json.dumps(line["parity"]))


if __name__ == "__main__":
    main()
