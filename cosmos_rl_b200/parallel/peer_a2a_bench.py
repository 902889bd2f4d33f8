"""Timing of the peer-memory all-to-all-v (``csrc/a2av.cu``) against ``all_to_all_single`` with split sizes.

    torchrun --nnodes=1 --nproc-per-node=<ep> --master-addr 127.0.0.1 -m cosmos_rl_b200.parallel.peer_a2a_bench

Shape of the Qwen3-30B-A3B dispatch: T tokens x top-8 copies of 2048 bf16 per rank, uniformly spread over the
ranks. Device time (CUDA events), max over ranks; the peer path includes its bounded flag wait and the copy out of
the receive ring. Roofline: bytes leaving a rank / 770 GB/s.
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist

from ..ops import native
from .peer_a2a import PeerAllToAll

NVLINK_BPS = 770e9


def main() -> None:
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    grp = dist.new_group(list(range(world)))
    H = 2048
    for T in (4096, 16384):
        rows = T * 8
        per = rows // world
        counts = [per] * world
        mat = [[per] * world for _ in range(world)]
        x = torch.randn(rows, H, device=dev).to(torch.bfloat16)
        a2a = PeerAllToAll(grp, world, rank, dev, max_rows=rows, row_bytes=H * 2)
        out = torch.empty(rows, H, dtype=torch.bfloat16, device=dev)

        def timed(fn, iters=10):
            for _ in range(3):
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

        t_peer = timed(lambda: a2a.exchange(x, counts, mat))
        t_lib = timed(lambda: dist.all_to_all_single(out, x, counts, counts, group=grp))
        assert native.read_status(dev) == 0
        off_bytes = (world - 1) * per * H * 2
        if rank == 0:
            print(f"T={T}: {rows} rows x {H} bf16 per rank, {off_bytes / 1e6:.0f} MB leave each rank | peer all-to-all-v "
                  f"{t_peer * 1e6:.0f} us ({off_bytes / t_peer / 1e9:.0f} GB/s out, {off_bytes / NVLINK_BPS / t_peer:.2f} "
                  f"of the NVLink roofline) | all_to_all_single {t_lib * 1e6:.0f} us", flush=True)
        a2a.close()
    # ---- whole expert-parallel MoE layer forward (Qwen3-30B-A3B layer: 128 experts, top-8, H 2048, I 768)
    import copy
    from ..models.qwen3_moe import ARCHS, MoEFeedForward
    from .ep_fused import FusedEPForward
    a = copy.deepcopy(ARCHS["qwen3-30b-a3b"])
    a.ep_size, a.ep_rank, a.aux_loss_coeff = world, rank, 0.0
    layer = MoEFeedForward(a).to(dev).to(torch.bfloat16)
    for p_ in layer.parameters():
        torch.nn.init.normal_(p_, std=0.02)
    layer.ep_group = grp
    for T in (4096, 8192):
        xt = torch.randn(T, a.dim, device=dev).to(torch.bfloat16)
        fe = FusedEPForward(grp, world, rank, dev, a.n_experts, a.dim, max_tokens=T, top_k=a.top_k)
        pa = PeerAllToAll(grp, world, rank, dev, max_rows=2 * T * a.top_k, row_bytes=a.dim * 2)
        with torch.no_grad():
            pr, ix, _, _ = layer.route(xt)

            def timed2(fn, iters=10):
                for _ in range(3):
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

            t_fused = timed2(lambda: fe.forward(xt, pr, ix, layer.w_gate_up, layer.w_down))
            layer.peer_a2a = None
            t_lib = timed2(lambda: layer._forward_ep(xt, pr, ix))
            layer.peer_a2a = pa
            t_peer = timed2(lambda: layer._forward_ep(xt, pr, ix))
            layer.peer_a2a = None
        assert native.read_status(dev) == 0
        flops = 2.0 * T * a.top_k * a.dim * 3 * a.moe_ffn_dim
        if rank == 0:
            print(f"EP{world} MoE layer forward, T={T} tokens per rank: fused dispatch+GEMM {t_fused * 1e6:.0f} us "
                  f"({flops / t_fused / 1e12:.0f} TFLOP/s per GPU) | peer all-to-all-v + grouped GEMMs {t_peer * 1e6:.0f} us | "
                  f"all_to_all_single + grouped GEMMs {t_lib * 1e6:.0f} us", flush=True)
        fe.close()
        pa.close()
    from ..utils.dist_util import safe_destroy
    safe_destroy(10.0)


if __name__ == "__main__":
    main()
