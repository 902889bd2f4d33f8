"""Kernel-time shares of one colocated GRPO step (rollout phase and training phase separately).

    python -m cosmos_rl_b200.tools.profiler.step_shares [--model qwen2.5-7b] [--prompts-per-gpu 16] ...

Runs one warm-up step, then one step under ``torch.profiler`` (CUPTI kernel records) and prints, per phase, the
kernels ordered by summed device time with their share. The absolute times carry profiler overhead and are not
benchmark numbers; the shares say where a step's device time goes.
"""
from __future__ import annotations

import argparse
from collections import defaultdict

import torch


def main(argv=None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen2.5-7b")
    ap.add_argument("--prompts-per-gpu", type=int, default=16)
    ap.add_argument("--group", type=int, default=8)
    ap.add_argument("--prompt-len", type=int, default=512)
    ap.add_argument("--max-response", type=int, default=1024)
    ap.add_argument("--mb-tokens", type=int, default=8192)
    ap.add_argument("--top", type=int, default=25)
    ap.add_argument("--phase", default="both", choices=["both", "rollout"])
    a = ap.parse_args(argv)
    from ...bench_grpo import make_config
    from ...colocated import ColocatedGRPO
    from ...models import named_architectures
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    job = ColocatedGRPO(make_config(a, 1, 1, colocated=True), device=dev, max_num_seqs=a.prompts_per_gpu * a.group)
    vocab = named_architectures()[a.model].vocab_size

    def prompts(seed):
        g = torch.Generator().manual_seed(seed)
        p = torch.randint(0, vocab, (a.prompts_per_gpu, a.prompt_len), generator=g).to(dev)
        return [p[i] for i in range(a.prompts_per_gpu)]

    job.step(prompts(0))
    torch.cuda.synchronize()
    from torch.profiler import ProfilerActivity, profile
    phases = {}
    for phase, fn in (("rollout", lambda: job.rollout(prompts(1))), ("train", None))[:1 if a.phase == "rollout" else 2]:
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            if phase == "rollout":
                out = fn()
            else:
                job.step_idx += 1
                job.trainer.step_training(out, job.step_idx, 1 << 30)
            torch.cuda.synchronize()
        agg = defaultdict(lambda: [0.0, 0])
        for ev in prof.events():
            if ev.device_type == torch.autograd.DeviceType.CUDA and ev.device_time_total > 0:
                agg[ev.name][0] += ev.device_time_total
                agg[ev.name][1] += 1
        phases[phase] = agg
    for phase, agg in phases.items():
        total = sum(v[0] for v in agg.values())
        print(f"== {phase}: {total / 1e3:.1f} ms of kernel time, {sum(v[1] for v in agg.values())} launches")
        for name, (t, n) in sorted(agg.items(), key=lambda kv: -kv[1][0])[:a.top]:
            print(f"{100 * t / total:5.1f}%  {t / 1e3:9.2f} ms  {n:7d}x  {t / max(n, 1):8.1f} us each  {name[:110]}")


if __name__ == "__main__":
    main()
