"""Timing of the fused peer-memory optimizer kernels (``csrc/fsdp_fused.cu``) against their NCCL statements.

    torchrun --nnodes=1 --nproc-per-node=<P> --master-addr 127.0.0.1 -m cosmos_rl_b200.parallel.fsdp_bench

Device time (CUDA events), max over ranks. Roofline of each kernel: the slower of the bytes it must move over
NVLink at the measured 770 GB/s per direction and its local HBM traffic at the measured copy bandwidth.
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist
import torch.nn as nn

from ..ops.kernel_cases import peaks
from ..policy.optim import FlatAdamW
from .flat import FlatParams
from .fsdp import PeerCollective
from .peer import peer_allocator

NVLINK_BPS = 770e9


def main() -> None:
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    grp = dist.new_group(list(range(world)))
    n = int(os.environ.get("FSDP_BENCH_ELEMS", str(2 << 30)))          # 2 Gi parameters: 4 GB of bf16 weights
    with torch.device("meta"):
        m = nn.Linear(n // 4096, 4096, bias=False)
    flat = FlatParams(m, torch.bfloat16, dev, shard_multiple=world, allocator=peer_allocator(dev))
    flat.data.normal_(0, 0.02)
    coll = PeerCollective(flat, grp)
    opt = FlatAdamW(flat, lr=1e-5, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.0, max_grad_norm=1.0, dp_group=grp,
                    collective=coll)
    flat.grad.normal_(0, 0.01)
    hbm, _, kind = peaks()
    shard = opt.hi - opt.lo
    sumsq = torch.zeros(1, dtype=torch.float32, device=dev)
    coef = torch.ones(1, dtype=torch.float32, device=dev)

    def timed(fn, iters=5):
        for _ in range(2):
            fn()
        dist.barrier(group=grp)
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize(dev)
        t = torch.tensor([e0.elapsed_time(e1) / iters], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=grp)
        return t.item() * 1e-3

    t_rs = timed(lambda: coll.reduce_scatter_sumsq(opt.lo, opt.hi, opt.grad_shard, sumsq))
    t_pub = timed(lambda: coll.adamw_publish(opt.master, opt.m, opt.v, opt.grad_shard, opt.lo, opt.hi, lr=1e-5,
                                             beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.0, step=3,
                                             grad_scale=coef))
    out = torch.empty(shard, dtype=torch.bfloat16, device=dev)
    t_rs_lib = timed(lambda: dist.reduce_scatter_tensor(out, flat.grad, group=grp))
    t_ag_lib = timed(lambda: dist.all_gather_into_tensor(flat.data, out, group=grp))
    # reduce-scatter: (P-1) remote shards in, P shards read in total, fp32 shard written
    rs_link = (world - 1) * shard * 2 / NVLINK_BPS
    rs_hbm = (shard * 2 + shard * 4) / hbm
    # AdamW + publish: master/m/v read+write (24 B), grad shard read (4 B), bf16 shard written locally and to P-1 peers
    pub_link = (world - 1) * shard * 2 / NVLINK_BPS
    pub_hbm = shard * (24 + 4 + 2) / hbm
    t_ar = timed(lambda: coll.all_reduce_grads())
    t_ar_lib = timed(lambda: dist.all_reduce(flat.grad, group=grp))
    ar_link = (world - 1) * shard * 2 / NVLINK_BPS           # each direction carries (P-1) shards
    if rank == 0:
        print(f"peer all-reduce (in place, one launch): {t_ar * 1e3:.2f} ms (incl. two stream barriers) | NCCL all_reduce "
              f"{t_ar_lib * 1e3:.2f} ms | roofline {ar_link * 1e3:.2f} ms -> {ar_link / t_ar:.2f} of NVLink roofline")
    if rank == 0:
        gb = shard * 2 / 1e9
        print(f"flat {flat.total / 2**30:.2f} Gi params, {world} ranks, shard {gb:.2f} GB (bf16)")
        print(f"reduce-scatter + scale + sumsq: {t_rs * 1e3:.2f} ms (incl. two stream barriers) | NCCL reduce_scatter "
              f"{t_rs_lib * 1e3:.2f} ms | roofline {max(rs_link, rs_hbm) * 1e3:.2f} ms -> "
              f"{max(rs_link, rs_hbm) / t_rs:.2f} of {kind} roofline | {(world - 1) * shard * 2 / t_rs / 1e9:.0f} GB/s in over NVLink")
        print(f"AdamW + publish to peers: {t_pub * 1e3:.2f} ms (incl. one stream barrier) | NCCL all_gather alone "
              f"{t_ag_lib * 1e3:.2f} ms | roofline {max(pub_link, pub_hbm) * 1e3:.2f} ms -> "
              f"{max(pub_link, pub_hbm) / t_pub:.2f} of {kind} roofline | {(world - 1) * shard * 2 / t_pub / 1e9:.0f} GB/s out over NVLink")
    coll.close()
    from ..utils.dist_util import safe_destroy
    safe_destroy(10.0)


if __name__ == "__main__":
    main()
