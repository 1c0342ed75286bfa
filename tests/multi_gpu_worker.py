"""Worker of tests/test_multi_gpu.py: one process per GPU (launched by torch.distributed.run), the KV positions of
every sequence split block-cyclically over the ranks.  Checks, against the CPU oracle on every rank, the exchange that
is fused into the decode kernel (peer stores + step flags over CUDA IPC mappings) through the device-pointer calls and
through the host-pointer step mfc_eval_token_attn, with every host sending all query rows and with the rows
gathered over the links.  Prints one line "rank R ok ..." per rank."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    import torch
    import torch.distributed as dist

    import moeflux_b200 as M
    from oracle import A17B as G
    from tests import inputs as I
    from tests.gpu_common import TOL_BF16, TOL_F32, make_pair

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    for bf16 in (False, True):
        n_seqs = world
        ctx, orc = make_pair(max_seq=640, n_seqs=n_seqs, kv_bf16=bf16, linear_layers=[0, 1], device=local, kv_rank=rank,
                             kv_world=world, kv_block=32)
        npr = 2  # layers 3 and 7 of the sequence this rank owns
        handles = [None] * world
        dist.all_gather_object(handles, ctx.exchange_create(npr))
        ctx.exchange_connect(handles)
        dist.barrier()
        items = [(layer, s) for s in range(n_seqs) for layer in (3, 7)]  # sorted by finishing rank (= sequence)
        layers, seqs = [i[0] for i in items], [i[1] for i in items]
        n = len(items)
        own = slice(rank * npr, (rank + 1) * npr)
        r = I.rng(900 + bf16)  # the same stream on every rank: all ranks see the same inputs
        tol = TOL_BF16 if bf16 else TOL_F32
        worst = 0.0
        lin_items = [(0, rank), (1, rank)]
        for pos in range(80):
            ins = [I.gqa_step_inputs(r) for _ in items]
            lin = [I.gdn_step_inputs(r) for _ in range(2 * world)][2 * rank:2 * rank + 2]
            refs = [orc.full_attn_step(layer, s, pos, *ins[j]) for j, (layer, s) in enumerate(items)]
            q, gate, k, v = (np.stack([i[c] for i in ins]) for c in range(4))
            if pos % 3 == 0:  # device-pointer calls
                dq, dg, dk, dv = (torch.tensor(a, device=dev) for a in (q, gate, k, v))
                out = torch.empty(npr, G.q_dim, device=dev)
                torch.cuda.synchronize()
                ctx.full_attn_partial_exchange_dev(layers, seqs, [pos] * n, dq.data_ptr(), dk.data_ptr(), dv.data_ptr())
                ctx.lse_merge_gate_exchange_dev(dg[own].data_ptr(), out.data_ptr())
                ctx.synchronize()
                got = out.cpu().numpy()
                for (layer, s), x in zip(lin_items, lin):
                    a, b = ctx.linear_attn_step(layer, s, *x), orc.linear_attn_step(layer, s, *x)
                    worst = max(worst, I.rel_err(a, b) * (tol / TOL_F32))
            else:             # the host-pointer step: both groups, copies and exchange inside one call
                q_own = pos % 3 == 2  # ... and the query rows gathered over the links, each host sending its own
                ctx.set_tuning("exchange_gather_q", int(q_own))
                got, lo = ctx.eval_token_attn_split(items, [pos] * n, q[own] if q_own else q, gate[own], k, v, lin_items,
                                                    np.stack([x[0] for x in lin]), np.stack([x[1] for x in lin]),
                                                    np.stack([x[2] for x in lin]), np.stack([x[3] for x in lin]), npr,
                                                    q_own=q_own)
                for j, ((layer, s), x) in enumerate(zip(lin_items, lin)):
                    worst = max(worst, I.rel_err(lo[j], orc.linear_attn_step(layer, s, *x)) * (tol / TOL_F32))
            for j in range(npr):
                worst = max(worst, I.rel_err(got[j], refs[rank * npr + j]))
        assert worst <= tol, (rank, bf16, worst)
        ctx.check_guards()
        dist.barrier()
        ctx.close()
        print(f"rank {rank} ok kv_{'bf16' if bf16 else 'f32'} worst rel err {worst:.2e}", flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
