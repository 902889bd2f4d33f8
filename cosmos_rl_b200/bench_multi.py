"""Multi-GPU GRPO benchmark loop: policy ranks (data parallel over peer memory) and rollout replicas
(tensor parallel) in one launch, stitched by the same mechanisms the workers use: the resharding plan, the
peer-memory weight pull, object exchange of rollouts. Generation of batch i+1 overlaps training of batch i
(one step off-policy, as the asynchronous mode of the framework does); every timed iteration contains one
generation batch, one policy update and one weight synchronisation.

Layout by GPU count N (per-GPU work is constant: 16 prompts x 8 responses x 1536 tokens per GPU):
  N=2: policy 1 GPU            | rollout 1 replica  x TP1
  N=4: policy FSDP2            | rollout 2 replicas x TP1
  N=8: policy FSDP4 (GPUs 0-3) | rollout 2 replicas x TP2 (GPUs 4-7)      <- the named configuration
"""
from __future__ import annotations

import copy
import time
from typing import Any, Dict, List, Optional

import torch
import torch.distributed as dist

from .ops import native


def layout(n: int):
    if n == 8:
        return 4, 2, 2          # policy ranks, rollout tp, rollout replicas
    if n % 2:
        raise ValueError("the disaggregated benchmark needs an even number of GPUs")
    return n // 2, 1, n // 2


def run_disaggregated(bench) -> Dict[str, Any]:
    from bench import ClockSampler
    from .bench_grpo import make_config
    from .dispatcher.algo.grpo import GRPO
    from .dispatcher.algo.reward import Reward
    from .dispatcher.data.schema import Rollout
    from .models import named_architectures
    from .models.gpt import GPT
    from .parallel.dims import ParallelDims
    from .parallel.flat import FlatParams
    from .parallel.fsdp import PeerCollective
    from .parallel.peer import PeerMapping, peer_allocator
    from .parallel.reshard import build_plan, model_parts, shard_info
    from .parallel.tp import TensorParallel
    from .policy.trainer.grpo_trainer import GRPOTrainer
    from .rollout.engine import RolloutEngine, SamplingParams
    from .rollout.weight_sync import PeerWeightSync

    a, rank, world, dev = bench.args, bench.rank, bench.world, bench.device
    P, tp, R = layout(world)
    is_policy = rank < P
    replica = (rank - P) // tp if not is_policy else -1
    tp_rank = (rank - P) % tp if not is_policy else 0

    # ---- groups (every rank creates every group, in the same order)
    gloo = dist.new_group(backend="gloo")
    policy_group = dist.new_group(list(range(P)))
    tp_groups = [dist.new_group(list(range(P + i * tp, P + (i + 1) * tp))) for i in range(R)] if tp > 1 else []
    cfg = make_config(a, P, tp, colocated=False)
    n_prompts_global = a.prompts_per_gpu * world
    prompts_per_replica = n_prompts_global // R
    seqs_per_policy_rank = n_prompts_global * a.group // P
    tokens_per_step = n_prompts_global * a.group * (a.prompt_len + a.max_response)

    trainer = engine = sync = coll = None
    if is_policy:
        dims = ParallelDims(dp_shard=P, world_size=P, global_rank=rank, device=dev)
        dims.set_group("dp_shard", policy_group)
        trainer = GRPOTrainer(cfg, dims, device=dev, allocator=peer_allocator(dev))
        trainer.model_load_from_hf()
        if P > 1:
            coll = PeerCollective(trainer.flat, policy_group)
            trainer.optimizer.collective = coll
        my = {"role": "policy", "rank": rank, "handle": trainer.flat.data._peer_buffer.export(),
              "nbytes": trainer.flat.data._peer_buffer.nbytes,
              "info": shard_info(rank, model_parts(trainer.model, trainer.flat), trainer.flat.total)}
    else:
        arch = copy.deepcopy(named_architectures()[a.model])
        arch.tp_size, arch.tp_rank = tp, tp_rank
        with torch.device("meta"):
            model = GPT(arch)
        flat = FlatParams(model, torch.bfloat16, dev, with_grad=False)
        if tp > 1:
            model.tp = TensorParallel(tp_groups[replica], tp, tp_rank)
        engine = RolloutEngine(model, max_num_seqs=prompts_per_replica * a.group,
                               max_model_len=a.prompt_len + a.max_response, page_size=128, seed=1234 + replica)
        my = {"role": "rollout", "rank": rank, "info": shard_info(rank, model_parts(model, flat), flat.total)}
        if P > 1:
            # keep the collective call sequence of the world identical on every rank
            pass
    everyone: List[dict] = [None] * world
    dist.all_gather_object(everyone, my, group=gloo)
    maps = []
    if not is_policy:
        src_infos = [e["info"] for e in everyone if e["role"] == "policy"]
        ptrs = {}
        for e in everyone:
            if e["role"] == "policy":
                m = PeerMapping(e["handle"], e["nbytes"], dev)
                maps.append(m)
                ptrs[e["rank"]] = m.ptr
        plan = build_plan(src_infos, my["info"])
        sync = PeerWeightSync(flat.data, plan, ptrs, dst_rank=rank)

    def world_barrier():
        torch.cuda.synchronize()
        dist.barrier(group=gloo)

    def weight_sync() -> float:
        """Policy weights are final (policy ranks synchronised) -> every rollout rank pulls -> all done."""
        world_barrier()
        ms = 0.0
        if not is_policy:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            sync.pull()
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1)
        world_barrier()
        return ms

    weight_sync()
    native.read_status(dev)
    sp = SamplingParams(temperature=1.0, top_p=1.0, top_k=-1, n=a.group, max_tokens=a.max_response, seed=None)
    algo = GRPO(Reward(["even_token_fraction"]))
    vocab = bench.vocab

    def generate(step: int):
        g = torch.Generator().manual_seed(1000 + step * 64 + replica)
        hp = torch.randint(0, vocab, (prompts_per_replica, a.prompt_len), generator=g, dtype=torch.int64).pin_memory()
        dp = hp.to(dev, non_blocking=True)
        outs = engine.generate([dp[j] for j in range(prompts_per_replica)], sp)
        if tp_rank != 0:
            return None
        recs = []
        hp_list = hp.tolist()
        for pi, comps in enumerate(outs):
            rewards = [algo.compute_reward(c.token_ids, None, token_ids=c.token_ids) for c in comps]
            advs = algo.compute_advantage(rewards)
            for c, rw, adv in zip(comps, rewards, advs):
                recs.append((hp_list[pi], c.token_ids, c.logprobs, rw, adv))
        return recs

    def train(batch, step: int):
        mine = batch[rank::P][:seqs_per_policy_rank]
        rollouts = [Rollout(prompt=p, completion=c, reward=rw, advantage=adv, completion_token_ids=[[t] for t in c],
                            completion_logprobs=[[l] for l in lp]) for (p, c, lp, rw, adv) in mine]
        return trainer.step_training(rollouts, step, 1 << 30)

    pending = None       # batch generated in the previous iteration
    reports: List[Dict[str, Any]] = []
    sync_ms: List[float] = []
    gen_s: List[float] = []
    train_s: List[float] = []

    def iteration(i: int):
        nonlocal pending
        t0 = time.perf_counter()
        mine = None
        if is_policy:
            if pending is not None:
                reports.append(train(pending, i))
                torch.cuda.synchronize()
                train_s.append(time.perf_counter() - t0)
        else:
            mine = generate(i)
            torch.cuda.synchronize()
            gen_s.append(time.perf_counter() - t0)
        sync_ms.append(weight_sync())
        gathered: List[Any] = [None] * world
        dist.all_gather_object(gathered, mine, group=gloo)
        pending = [r for part in gathered if part for r in part]

    for i in range(a.warmup + 1):     # +1: the first iteration only fills the pipeline (no batch to train yet)
        iteration(i)
    native.read_status(dev)
    clocks = ClockSampler(bench.local_rank)
    world_barrier()
    clocks.start()
    launches0 = native.LAUNCHES[0]
    reports.clear(); sync_ms.clear(); gen_s.clear(); train_s.clear()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(a.steps):
        iteration(a.warmup + 1 + i)
    e1.record()
    world_barrier()
    ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    launches = torch.tensor([native.LAUNCHES[0] - launches0], device=dev, dtype=torch.int64)
    dist.all_reduce(launches)
    clk = clocks.stop()
    native.read_status(dev)
    ms = float(ms.item())
    # gather per-role timings for the breakdown
    stats = {"gen_s": sum(gen_s) / max(1, len(gen_s)), "train_s": sum(train_s) / max(1, len(train_s)),
             "sync_ms": sum(sync_ms) / max(1, len(sync_ms)), "policy": is_policy}
    all_stats: List[dict] = [None] * world
    dist.all_gather_object(all_stats, stats, group=gloo)
    value = tokens_per_step * a.steps / (ms / 1e3)
    sync_bytes = sum(p.numel() for p in (trainer.model.parameters() if is_policy else [])) * 2
    out = {
        "metric": "GRPO step tokens/s (prompt+response tokens generated and trained per second)",
        "value": value, "unit": "tokens/s", "n_gpus": world, "steps": a.steps, "warmup": a.warmup,
        "ms_per_step": ms / a.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic prompts (uniform random token ids), random-init weights, "
                                 "even-token-fraction reward",
        "config": {"model": f"{a.model}-arch", "global_batch": n_prompts_global * a.group,
                   "seq_len": a.prompt_len + a.max_response, "prompts": n_prompts_global, "group": a.group,
                   "prompt_len": a.prompt_len, "max_response": a.max_response,
                   "parallelism": f"policy fsdp{P} (GPUs 0-{P - 1}) + rollout tp{tp} x {R} replicas",
                   "pipeline": "generation of batch i+1 overlaps training of batch i; weight sync every step",
                   "l2": "inputs larger than L2 (weights and KV cache streamed from HBM every step)",
                   "weight_sync": "peer-memory pull kernel over NVLink (no NCCL)"},
        "clocks": clk, "gpu_launches": int(launches.item()),
        "breakdown": {
            "rollout_s": max((s["gen_s"] for s in all_stats if not s["policy"]), default=0.0),
            "train_s": max((s["train_s"] for s in all_stats if s["policy"]), default=0.0),
            "weight_sync_ms": max((s["sync_ms"] for s in all_stats if not s["policy"]), default=0.0),
            "weight_sync_bytes_per_rollout_rank": sync.bytes if sync is not None else None,
            "loss": reports[-1]["train/loss_avg"] if reports else None,
            "grad_norm": reports[-1]["train/grad_norm"] if reports else None,
        },
    }
    if sync is not None:
        sb = torch.tensor([sync.bytes], dtype=torch.int64, device=dev)
    else:
        sb = torch.zeros(1, dtype=torch.int64, device=dev)
    dist.all_reduce(sb, op=dist.ReduceOp.MAX)
    out["breakdown"]["weight_sync_bytes_per_rollout_rank"] = int(sb.item())
    ws = out["breakdown"]["weight_sync_ms"]
    out["breakdown"]["weight_sync_GBps_per_rollout_rank"] = (sb.item() / 1e9) / (ws / 1e3) if ws > 0 else None
    if not a.no_e2e:
        # end to end: same loop, wall clock; prompts start in pinned host memory on the rollout ranks, the loss is
        # read back on the policy ranks (both happen inside iteration())
        world_barrier()
        t0 = time.perf_counter()
        for i in range(a.steps):
            iteration(10_000 + i)
        world_barrier()
        dt = torch.tensor([time.perf_counter() - t0], device=dev)
        dist.all_reduce(dt, op=dist.ReduceOp.MAX)
        out["e2e"] = {"value": tokens_per_step * a.steps / float(dt.item()), "unit": "tokens/s",
                      "h2d_bytes_per_step": n_prompts_global * a.prompt_len * 8 + tokens_per_step * 8 * 3,
                      "d2h_bytes_per_step": n_prompts_global * a.group * a.max_response * 12 + 64 * P,
                      "api": "GRPOTrainer.step_training + RolloutEngine.generate + PeerWeightSync.pull"}
    if engine is not None:
        engine.invalidate_graphs()   # CUDA graphs hold the TP communicator
    for m in maps:
        m.close()
    if coll is not None:
        coll.close()
    return out
