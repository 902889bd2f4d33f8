"""One decoder block under tensor parallelism, forward + backward, three ways:

    torchrun --nnodes=1 --nproc-per-node=<tp> --master-addr 127.0.0.1 -m cosmos_rl_b200.parallel.sp_block_bench

* ``tp``: replicated activations, row-parallel outputs all-reduced by the library (the plan without sequence
  parallelism);
* ``sp-library``: sequence-parallel plan, all-gather / reduce-scatter by the library around cuBLAS GEMMs, gathered
  inputs kept for the weight gradients (``sp-library-regather``: gathered again in backward instead);
* ``sp-fused``: the same plan with the all-gather -> GEMM and GEMM -> reduce-scatter kernels over peer memory in
  forward and for the input gradients.

Qwen2.5-7B block shapes (hidden 3584, FFN 18944, 28 / 4 heads), packed sequences of 2048 tokens; device time between
CUDA events, max over ranks, after warm-up. Weights of several layers are rotated so they do not stay in L2."""
from __future__ import annotations

import argparse
import os

import torch
import torch.distributed as dist

from ..models.gpt import GPT, GPTArgs
from ..ops import native
from .flat import FlatParams
from .tp import TensorParallel


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--iters", type=int, default=5)
    a = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    grp = dist.new_group(list(range(world)))
    args = GPTArgs(vocab_size=4096, dim=3584, n_layers=a.layers, n_heads=28, n_kv_heads=4, head_dim=128, ffn_dim=18944,
                   qkv_bias=True, model_type="qwen2", tp_size=world, tp_rank=rank)
    with torch.device("meta"):
        model = GPT(args)
    flat = FlatParams(model, torch.bfloat16, dev)
    model.init_weights_on_device(0)
    T = a.tokens
    g = torch.Generator(device=dev).manual_seed(1)
    ids = torch.randint(0, 4096, (T,), device=dev, generator=g)
    cu = torch.arange(0, T + 1, 2048, dtype=torch.int32, device=dev)
    pos = model.get_position_ids(cu, T)

    def step():
        flat.zero_grad()
        h = model(ids, pos, cu, 2048)
        h.float().square().mean().backward()

    def timed(label):
        for _ in range(2):
            step()
        dist.barrier(group=grp)
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(a.iters):
            step()
        e1.record()
        torch.cuda.synchronize(dev)
        assert native.read_status(dev) == 0, label
        t = torch.tensor([e0.elapsed_time(e1) / a.iters], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=grp)
        return t.item()

    res = {}
    model.tp = TensorParallel(grp, world, rank)
    res["tp"] = timed("tp")
    model.tp.sequence_parallel = True
    res["sp-library"] = timed("sp-library")
    model.tp.keep_gathered = False
    res["sp-library-regather"] = timed("sp-library-regather")
    model.tp.keep_gathered = True
    model.tp.attach_fused(dev, T, args.dim, all_gather_k=args.dim)
    res["sp-fused"] = timed("sp-fused")
    if rank == 0:
        per = {k: v / a.layers for k, v in res.items()}
        print(f"TP{world} decoder block fwd+bwd, {T} tokens, Qwen2.5-7B shapes (ms per block, max over ranks): "
              + " | ".join(f"{k} {v:.2f}" for k, v in per.items())
              + f" | sp-fused vs tp {res['tp'] / res['sp-fused']:.2f}x, vs sp-library {res['sp-library'] / res['sp-fused']:.2f}x",
              flush=True)
    model.tp.fused.close()
    model.tp.fused_ag.close()
    from ..utils.dist_util import safe_destroy
    safe_destroy(10.0)


if __name__ == "__main__":
    main()
