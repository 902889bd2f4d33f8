"""2-GPU worker: parameter-sharded training (units gathered on a side stream, gradients reduce-scattered per unit)
against the resident-weights trainer on the same two GPUs. Launched by ``tests/test_multi_gpu.py`` under torchrun."""
import os
import sys
import tempfile

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from cosmos_rl_b200.config import Config
    from cosmos_rl_b200.ops import native
    from cosmos_rl_b200.parallel.dims import ParallelDims
    from cosmos_rl_b200.policy.trainer.sft_trainer import SFTTrainer
    out_dir = tempfile.mkdtemp()
    model = sys.argv[1] if len(sys.argv) > 1 else "tiny-qwen2-d128"

    def cfg(**b200):
        return Config.from_dict({
            "policy": {"model_name_or_path": model, "model_max_length": 1024, "model_gradient_checkpointing": True,
                       "parallelism": {"tp_size": 1, "cp_size": 1, "pp_size": 1, "dp_shard_size": world}},
            "b200": dict({"recompute": "swiglu"}, **b200),
            "train": {"seed": 0, "optm_lr": 1e-4, "optm_warmup_steps": 0, "output_dir": out_dir,
                      "optm_grad_norm_clip": 1.0, "fsdp_reduce_dtype": "float32",
                      "train_policy": {"type": "sft", "trainer_type": "sft", "mini_batch": 4},
                      "ckpt": {"enable_checkpoint": False}}})
    trainers = {}
    for name, kw in (("resident", {}), ("sharded", {"shard_params": True})):
        c = cfg(**kw)
        dims = ParallelDims.from_config_parallelism(c.policy.parallelism, world, rank, dev)
        if name == "resident":
            dims.build_groups()
            groups = dims
        else:
            dims = groups                                    # the same process groups for both trainers
        tr = SFTTrainer(c, dims, device=dev)
        tr.model_load_from_hf()
        trainers[name] = tr
    sp = trainers["sharded"].flat
    assert sp.sharded and sp.n_shard * world == sp.total
    g = torch.Generator().manual_seed(5 + rank)
    vocab = trainers["resident"].model.args.vocab_size
    batch = [{"input_ids": torch.randint(0, vocab, (n,), generator=g).tolist()} for n in (700, 512, 900, 333, 640, 128, 1000, 256)]
    times = {}
    for name, tr in trainers.items():
        losses = []
        for i in range(4):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            rep = tr.step_training(batch, total_steps=10, train_step=i + 1)
            e1.record()
            torch.cuda.synchronize()
            losses.append((rep["train/loss_avg"], rep["train/grad_norm"]))
            times.setdefault(name, []).append(e0.elapsed_time(e1))
        trainers[name].losses = losses
    assert native.read_status(dev) == 0
    if rank == 0:
        print("resident (loss, grad norm) per step:", [(round(l, 4), round(g, 4)) for l, g in trainers["resident"].losses])
        print("sharded  (loss, grad norm) per step:", [(round(l, 4), round(g, 4)) for l, g in trainers["sharded"].losses],
              flush=True)
    # the first step starts from identical weights: tight. Later steps compound bf16 rounding of two different
    # reduction orders on a model that is memorising one batch: loose.
    for i, ((la, ga), (lb, gb)) in enumerate(zip(trainers["resident"].losses, trainers["sharded"].losses)):
        tol_l, tol_g = (2e-3, 2e-2) if i == 0 else (1e-1, 2.5e-1)
        assert abs(la - lb) < tol_l * abs(la) + 1e-3, (i, la, lb)
        assert abs(ga - gb) < tol_g * abs(ga) + 1e-3, (i, ga, gb)
    full = sp.gather_full()
    res = trainers["resident"]
    worst = 0.0
    for n, q in res.model.named_parameters():
        worst = max(worst, (sp.view(n, full).float() - q.float()).abs().max().item())
    assert worst < 5e-2, worst                               # bf16 weights after four steps of lr 1e-4
    t = torch.tensor([min(times["resident"][1:]), min(times["sharded"][1:])], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        mem = {k: round(v, 3) for k, v in sp.memory_report().items()}
        print(f"parameter-sharded training on {world} GPUs ({model}): losses and gradient norms of four steps match the "
              f"resident-weights trainer, weights within {worst:.2e}; step {t[1].item():.1f} ms sharded vs "
              f"{t[0].item():.1f} ms resident; {sp.n_gathers} gathers, {sp.n_reduces} reductions; memory {mem}", flush=True)
        print("SHARD OK", flush=True)
    from cosmos_rl_b200.utils.dist_util import safe_destroy
    safe_destroy(10.0)


if __name__ == "__main__":
    main()
