"""Weight-synchronisation sweep on a separated layout: policy ranks on the first half of the GPUs, rollout ranks on
the second half, one full sync of every parameter per iteration.

    torchrun --nproc-per-node 8 -m cosmos_rl_b200.rollout.weight_sync_bench --model qwen2.5-7b --rollout-tp 1 2 4

For every rollout tensor-parallel size and every mode it prints one JSON line (rank 0):

* ``peer-bf16``   one kernel per rollout rank pulls its rectangles out of the policy ranks' memory over NVLink;
* ``peer-fp8``    the same pass writes e4m3 + 128 x 128 block scales (no bf16 copy of the quantised matrices);
* ``collective-fp32`` the reference's route restated: one send / recv per rectangle in fp32 (its default
  ``transfer_dtype``), a copy into place, and for fp8 serving a second quantisation pass
  (cosmos_rl/policy/worker/rl_worker.py:419-571, cosmos_rl/rollout/worker/rollout_control.py:674-1027).

Times are CUDA events on the pulling / receiving ranks, maximum over ranks, median of ``--iters`` after warm-up.
``GBps_per_rollout_rank`` = bf16 bytes that land on one rollout rank / time; the roofline for a pull is the measured
770 GB/s peer-copy rate per direction per GPU. The policy ranks hold full copies of the bf16 weights (data-parallel
replicas with sharded optimizer state), and the plan spreads the sources over them.
"""
from __future__ import annotations

import argparse
import copy
import json
import os
import statistics

import torch
import torch.distributed as dist


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen2.5-7b")
    ap.add_argument("--rollout-tp", type=int, nargs="+", default=[1, 2, 4])
    ap.add_argument("--modes", nargs="+", default=["peer-bf16", "peer-fp8"],
                    help="add collective-fp32 for the send / recv baseline")
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=2)
    a = ap.parse_args(argv)
    from ..models import named_architectures
    from ..models.base import ModelRegistry
    from ..ops import native
    from ..parallel.flat import FlatParams
    from ..parallel.peer import PeerMapping, peer_allocator
    from ..parallel.reshard import build_plan, model_parts, shard_info
    from .weight_sync import CollectiveWeightSync, Fp8WeightStore, PeerWeightSync

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=dev)
    gloo = dist.new_group(backend="gloo")
    P = world // 2
    R = world - P
    is_policy = rank < P
    arch0 = named_architectures()[a.model]

    def build(tp: int, tp_rank: int, allocator=None):
        arch = copy.deepcopy(arch0)
        arch.tp_size, arch.tp_rank = tp, tp_rank
        with torch.device("meta"):
            model = ModelRegistry.build_model(arch.to_hf_config(), tp_size=tp, tp_rank=tp_rank)
        flat = FlatParams(model, torch.bfloat16, dev, with_grad=False, allocator=allocator)
        return model, flat

    pol_model = pol_flat = None
    if is_policy:
        pol_model, pol_flat = build(1, 0, peer_allocator(dev))
        g = torch.Generator(device=dev).manual_seed(7)           # same seed: the replicas hold the same weights
        pol_flat.data.normal_(0.0, 0.02, generator=g)
    for tp in a.rollout_tp:
        if R % tp:
            if rank == 0:
                print(json.dumps({"rollout_tp": tp, "skipped": f"{R} rollout GPUs are not a multiple of tp {tp}"}))
            continue
        ro_model = ro_flat = None
        if is_policy:
            my = {"role": "policy", "rank": rank, "handle": pol_flat.data._peer_buffer.export(),
                  "nbytes": pol_flat.data._peer_buffer.nbytes,
                  "info": shard_info(rank, model_parts(pol_model, pol_flat), pol_flat.total)}
        else:
            ro_model, ro_flat = build(tp, (rank - P) % tp)
            my = {"role": "rollout", "rank": rank, "info": shard_info(rank, model_parts(ro_model, ro_flat), ro_flat.total)}
        everyone = [None] * world
        dist.all_gather_object(everyone, my, group=gloo)
        pol = [e for e in everyone if e["role"] == "policy"]
        plans = {e["rank"]: build_plan([p["info"] for p in pol], e["info"]) for e in everyone if e["role"] == "rollout"}
        maps, ptrs = [], {}
        if not is_policy:
            for e in pol:
                m = PeerMapping(e["handle"], e["nbytes"], dev)
                maps.append(m)
                ptrs[e["rank"]] = m.ptr
        for mode in a.modes:
            sync = fp8 = coll = None
            if not is_policy and mode.startswith("peer"):
                fp8 = Fp8WeightStore(ro_flat) if mode == "peer-fp8" else None
                sync = PeerWeightSync(ro_flat.data, plans[rank], ptrs, fp8=fp8, dst_rank=rank - P)
            if mode == "collective-fp32":
                ident = {r: r for r in range(world)}
                coll = CollectiveWeightSync(None, ident, ident, transfer_dtype=torch.float32)
                send_plan = [[r, d] for r, pl in sorted(plans.items()) for d in pl if d[0] == rank] if is_policy else None
                fp8 = Fp8WeightStore(ro_flat) if (not is_policy and "peer-fp8" in a.modes) else None
            times = []
            for it in range(a.warmup + a.iters):
                torch.cuda.synchronize()
                dist.barrier(group=gloo)
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                if mode.startswith("peer"):
                    if not is_policy:
                        sync.pull()
                elif is_policy:
                    coll.send(pol_flat.data, send_plan)
                else:
                    coll.recv(ro_flat.data, plans[rank])
                    if fp8 is not None:
                        fp8.quantize_local()
                e1.record()
                torch.cuda.synchronize()
                ms = torch.tensor([e0.elapsed_time(e1) if (not is_policy or mode == "collective-fp32") else 0.0],
                                  device=dev)
                dist.all_reduce(ms, op=dist.ReduceOp.MAX)
                if it >= a.warmup:
                    times.append(float(ms))
            native.read_status(dev)
            nbytes = torch.tensor([ro_flat.total * 2 if not is_policy else 0], dtype=torch.float64, device=dev)
            dist.all_reduce(nbytes, op=dist.ReduceOp.MAX)
            if rank == 0:
                med = statistics.median(times)
                print(json.dumps({"model": a.model, "policy_gpus": P, "rollout_gpus": R, "rollout_tp": tp, "mode": mode,
                                  "ms_per_sync": round(med, 3), "GB_per_rollout_rank": round(float(nbytes) / 1e9, 3),
                                  "GBps_per_rollout_rank": round(float(nbytes) / 1e6 / med, 1),
                                  "fraction_of_770GBps": round(float(nbytes) / 1e6 / med / 770.0, 3),
                                  "rectangles_per_rank": len(next(iter(plans.values()))), "iters": a.iters}), flush=True)
            del sync, fp8, coll
        for m in maps:
            m.close()
        del ro_model, ro_flat
        torch.cuda.empty_cache()
    dist.barrier(group=gloo)
    from ..utils.dist_util import safe_destroy
    safe_destroy(20.0)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
