"""Process-group bring-up for one-process-per-GPU tensor parallelism (launched by torch.distributed.run or the cluster
supervisor): device selection, a CPU (gloo) control group for the lockstep messages and the IPC handle exchange, and the
symmetric arena.  NCCL is registered for CUDA tensors but no communicator is created unless a caller uses it; the hot
path moves data with the fused peer-memory kernels only.
"""
from __future__ import annotations

import datetime
import os
from dataclasses import dataclass

import torch
import torch.distributed as dist


@dataclass
class TpContext:
    rank: int
    world: int
    local_rank: int
    device: torch.device
    ctrl: object            # gloo group used for control messages


def init(timeout_s: float = 300.0) -> TpContext:
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29517")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if not dist.is_initialized():
        dist.init_process_group("cpu:gloo,cuda:nccl", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=timeout_s))
    ctrl = dist.new_group(backend="gloo", timeout=datetime.timedelta(seconds=timeout_s))
    return TpContext(rank, world, local, dev, ctrl)


def build_dense_tp(ctx: TpContext, cfg, *, num_pages: int, max_rows: int, max_slots: int, max_blocks_per_seq: int, weights=None, seed: int = 0,
                   kv_dtype: str = "bf16", collective: str = "fused"):
    """-> (shard, group).  `weights` is a full HostWeights (sliced here for this rank) or None for a random-init shard."""
    from ..models.dense_tp import DenseTPShard, shard_weights
    from .symm import IpcGroup
    layout = DenseTPShard.layout(cfg, ctx.world, max_rows)
    group = IpcGroup(layout, ctx.rank, ctx.device, group=ctx.ctrl)
    if collective == "fused":
        group.enable_nvls()       # in-switch reduction for windows above the packet size, where the fabric and the settings allow it
    w = shard_weights(weights, ctx.rank, ctx.world) if weights is not None else None
    shard = DenseTPShard(cfg, group, ctx.rank, num_pages, max_rows, max_slots, max_blocks_per_seq, weights=w, device=ctx.device, seed=seed, kv_dtype=kv_dtype,
                         collective=collective)
    shard.max_seqs = max_slots
    torch.cuda.synchronize()
    dist.barrier(group=ctx.ctrl)
    return shard, group


def shutdown(ctx: TpContext, group=None) -> None:
    torch.cuda.synchronize()
    dist.barrier(group=ctx.ctrl)
    if group is not None:
        group.close()
    dist.destroy_process_group()
