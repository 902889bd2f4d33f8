"""Timing of the fused row-parallel GEMM + all-reduce / reduce-scatter kernel against GEMM + NCCL.

    torchrun --nnodes=1 --nproc-per-node=<tp> --master-addr 127.0.0.1 -m cosmos_rl_b200.parallel.tp_fused_bench

Device time (CUDA events), max over ranks, after warm-up; inputs are rotated through a pool larger than L2.
Also prints the roofline of each shape: the slower of FLOPs at the measured GEMM peak and bytes over NVLink at
the measured 770 GB/s per direction.
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist

from ..ops import functional as F
from ..ops import native
from ..ops.kernel_cases import peaks
from .tp_fused import FusedAllGatherGemm, FusedTP

NVLINK_BPS = 770e9


def main() -> None:
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    grp = dist.new_group(list(range(world)))
    solo = [dist.new_group([r]) for r in range(world)][rank]
    N, K = 3584, 18944 // world
    ftp = FusedTP(grp, world, rank, dev, max_rows=16384, max_cols=N)
    f1 = FusedTP(solo, 1, 0, dev, max_rows=16384, max_cols=N)
    _, gemm_peak, kind = peaks()

    def timed(fn, iters):
        for _ in range(3):
            fn(0)
        dist.barrier(group=grp)
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(iters):
            fn(i)
        e1.record()
        torch.cuda.synchronize(dev)
        t = torch.tensor([e0.elapsed_time(e1) / iters], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=grp)
        return t.item() * 1e-3

    for M in (512, 8192):
        pool = max(2, int(300e6 // (N * K * 2)) + 1)
        ws = [(torch.randn(N, K, device=dev) * 0.02).to(torch.bfloat16) for _ in range(pool)]
        a = torch.randn(M, K, device=dev).to(torch.bfloat16)
        iters = 30 if M <= 2048 else 10

        def lib(i):
            y = torch.nn.functional.linear(a, ws[i % pool])
            dist.all_reduce(y, group=grp)

        def lib_rs(i):
            y = torch.nn.functional.linear(a, ws[i % pool])
            o = torch.empty(M // world, N, dtype=y.dtype, device=dev)
            dist.reduce_scatter_tensor(o, y, group=grp)

        t_fused = timed(lambda i: ftp.gemm_all_reduce(a, ws[i % pool]), iters)
        t_lib = timed(lib, iters)
        t_gemm_lib = timed(lambda i: torch.nn.functional.linear(a, ws[i % pool]), iters)
        t_gemm_own = timed(lambda i: F.gemm_nt(a, ws[i % pool]), iters)
        t_solo = timed(lambda i: f1.gemm_all_reduce(a, ws[i % pool]), iters)
        line = (f"M={M:6d} all-reduce: fused {t_fused * 1e6:8.1f} us | linear+nccl {t_lib * 1e6:8.1f} us | "
                f"cublas gemm {t_gemm_lib * 1e6:7.1f} | own gemm {t_gemm_own * 1e6:7.1f} | fused kernel, 1 rank "
                f"{t_solo * 1e6:7.1f}")
        flops = 2.0 * M * N * K
        link_ar = (world - 1) * M * N * 2 / NVLINK_BPS
        roof = max(flops / gemm_peak, link_ar)
        line += f" | roofline {roof * 1e6:.1f} us -> {roof / t_fused:.2f} of {kind} roofline"
        if M % (128 * world) == 0:
            t_rs = timed(lambda i: ftp.gemm_reduce_scatter(a, ws[i % pool]), iters)
            t_rs_lib = timed(lib_rs, iters)
            roof_rs = max(flops / gemm_peak, (world - 1) / world * M * N * 2 / NVLINK_BPS)
            line += (f" || reduce-scatter: fused {t_rs * 1e6:8.1f} us | linear+nccl {t_rs_lib * 1e6:8.1f} us | "
                     f"{roof_rs / t_rs:.2f} of roofline")
        assert native.read_status(dev) == 0
        if rank == 0:
            print(line, flush=True)
        del ws
    # ---- all-gather -> column-parallel GEMM (sequence-parallel input of gate/up: N = 2 * 18944 / tp, K = 3584)
    Kc, Nc = 3584, 2 * 18944 // world
    ag = FusedAllGatherGemm(grp, world, rank, dev, max_rows=16384, max_k=Kc)
    for M in (2048, 8192, 16384):
        pool = max(2, int(300e6 // (Nc * Kc * 2)) + 1)
        ws = [(torch.randn(Nc, Kc, device=dev) * 0.02).to(torch.bfloat16) for _ in range(pool)]
        xl = torch.randn(M // world, Kc, device=dev).to(torch.bfloat16)
        full = torch.empty(M, Kc, dtype=torch.bfloat16, device=dev)
        iters = 20 if M <= 2048 else 8

        def lib_ag(i):
            dist.all_gather_into_tensor(full, xl, group=grp)
            torch.nn.functional.linear(full, ws[i % pool])

        t_fused = timed(lambda i: ag.gemm(xl, ws[i % pool]), iters)
        t_lib = timed(lib_ag, iters)
        t_own = timed(lambda i: F.gemm_nt(full, ws[i % pool]), iters)
        flops = 2.0 * M * Nc * Kc
        roof = max(flops / gemm_peak, (world - 1) / world * M * Kc * 2 / NVLINK_BPS)
        assert native.read_status(dev) == 0
        if rank == 0:
            print(f"M={M:6d} all-gather->gemm [N={Nc}, K={Kc}]: fused {t_fused * 1e6:8.1f} us | all_gather+linear "
                  f"{t_lib * 1e6:8.1f} us | own gemm on gathered input {t_own * 1e6:8.1f} us | roofline "
                  f"{roof * 1e6:.1f} us -> {roof / t_fused:.2f} of {kind} roofline", flush=True)
        del ws
    ag.close()
    ftp.close()
    f1.close()
    from ..utils.dist_util import safe_destroy
    safe_destroy(10.0)


if __name__ == "__main__":
    main()
