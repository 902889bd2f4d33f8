"""Rollout-only throughput: the generation engine on a named architecture with random-init weights and synthetic
prompts, no training (the reference's harness is tests/benchmark/rollout_benchmark.py, a torchrun loop around vLLM).

    python -m cosmos_rl_b200.rollout.rollout_bench --model qwen2.5-7b --prompts 16 --group 8 --prompt-len 512 --max-response 1024

Prints one JSON line: generated tokens/s (device time between CUDA events, after warm-up generations), decode steps
per second and the time per decode step."""
from __future__ import annotations

import argparse
import json
import time

import torch


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen2.5-7b")
    ap.add_argument("--prompts", type=int, default=16)
    ap.add_argument("--group", type=int, default=8)
    ap.add_argument("--prompt-len", type=int, default=512)
    ap.add_argument("--max-response", type=int, default=1024)
    ap.add_argument("--warmup", type=int, default=1)
    ap.add_argument("--iters", type=int, default=2)
    ap.add_argument("--temperature", type=float, default=1.0)
    a = ap.parse_args(argv)
    from ..models import hf_io
    from ..models.base import ModelRegistry
    from ..parallel.flat import FlatParams
    from .engine import RolloutEngine, SamplingParams
    cuda = torch.cuda.is_available()
    dev = torch.device("cuda", 0) if cuda else torch.device("cpu")
    cfg = hf_io.load_hf_config(a.model)
    with torch.device("meta"):
        model = ModelRegistry.build_model(cfg)
    FlatParams(model, torch.bfloat16 if cuda else torch.float32, dev, with_grad=False)
    (model.init_weights_on_device if cuda else model.init_weights)(0)
    eng = RolloutEngine(model, max_num_seqs=a.prompts * a.group, max_model_len=a.prompt_len + a.max_response)
    sp = SamplingParams(n=a.group, max_tokens=a.max_response, temperature=a.temperature)
    g = torch.Generator().manual_seed(0)
    vocab = cfg["vocab_size"]

    def prompts(i):
        return [torch.randint(0, vocab, (a.prompt_len,), generator=g).tolist() for _ in range(a.prompts)]

    for i in range(a.warmup):
        eng.generate(prompts(i), sp)
    if cuda:
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
    t0 = time.perf_counter()
    n_tok = 0
    for i in range(a.iters):
        outs = eng.generate(prompts(a.warmup + i), sp)
        n_tok += sum(len(c.token_ids) for comps in outs for c in comps)
    if cuda:
        e1.record()
        torch.cuda.synchronize()
        sec = e0.elapsed_time(e1) / 1e3
    else:
        sec = time.perf_counter() - t0
    steps = a.iters * a.max_response
    print(json.dumps({"metric": "rollout generated tokens/s", "value": n_tok / sec, "model": a.model,
                      "sequences": a.prompts * a.group, "prompt_len": a.prompt_len, "max_response": a.max_response,
                      "seconds": sec, "ms_per_decode_step": sec / steps * 1e3, "device": str(dev)}))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
