"""The TpComm interface over REAL NVLink, one process per GPU: PeerTp (peer stores + local rank-order sum) against torch.distributed NCCL
behind the same interface - results compared, then CUDA-event timing of both for a few sizes (max over ranks).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29535 -m rexl3_b200.parallel.tpcomm_selftest
"""
from __future__ import annotations

import json
import sys

import torch
import torch.distributed as dist


def main() -> int:
    from . import runtime, tpcomm
    ctx = runtime.init(timeout_s=300)
    R, rank, dev = ctx.world, ctx.rank, ctx.device
    cap = 4 << 20
    peer = tpcomm.peer_group(rank, R, cap, dev, ctx.ctrl)
    nccl = tpcomm.NcclTp()
    g = torch.Generator(device=dev).manual_seed(100 + rank)
    x = torch.randn(1 << 16, device=dev, generator=g)
    allx = torch.empty(R, x.numel(), device=dev)
    nccl.allgather_f32(x, allx)
    want = allx[0].clone()
    for r in range(1, R):
        want += allx[r]
    a = x.clone()
    peer.allreduce_sum_f32(a)
    gath = torch.empty(R, x.numel(), device=dev)
    peer.allgather_f32(x, gath)
    torch.cuda.synchronize()
    ok = bool(torch.equal(a, want)) and bool(torch.equal(gath, allx)) and peer.async_error() is None
    rows = []
    for n in (1 << 12, 1 << 16, 1 << 20, 1 << 22):
        buf = torch.randn(n, device=dev, generator=g)
        res = {}
        for name, c in (("peer", peer), ("nccl", nccl)):
            for _ in range(5):
                c.allreduce_sum_f32(buf)
            torch.cuda.synchronize()
            dist.barrier(group=ctx.ctrl)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(20):
                c.allreduce_sum_f32(buf)
            e1.record()
            torch.cuda.synchronize()
            t = torch.tensor([e0.elapsed_time(e1) / 20 * 1e3], dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=ctx.ctrl)
            res[name] = round(float(t[0]), 1)
            buf.normal_(generator=g)
        rows.append(dict(bytes=4 * n, peer_us=res["peer"], nccl_us=res["nccl"]))
    flag = torch.tensor([1 if ok else 0], dtype=torch.int32)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=ctx.ctrl)
    if rank == 0:
        print(json.dumps(dict(bench="tpcomm_selftest", ranks=R, equal_to_rank_order_sum=bool(int(flag)), allreduce=rows)))
    torch.cuda.synchronize()
    dist.barrier(group=ctx.ctrl)
    peer.g.close()
    import os
    sys.stdout.flush()
    os._exit(0 if int(flag) else 1)          # the NCCL communicator's teardown has hung at exit on this pool: leave without it


if __name__ == "__main__":
    sys.exit(main())
