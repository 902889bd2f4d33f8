"""Multi-process CPU (gloo) tests of the parallel strategies: context parallelism, pipeline parallelism."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from cosmos_rl_b200.models.gpt import GPT, GPTArgs


def _tiny():
    return GPTArgs(vocab_size=512, dim=64, n_layers=2, n_heads=4, n_kv_heads=2, ffn_dim=128, qkv_bias=True,
                   model_type="qwen2")


def _spawn(fn, world, tmp_path, *args):
    store = str(tmp_path / "store")
    mp.spawn(fn, args=(world, store) + args, nprocs=world, join=True)


def _init(rank, world, store):
    dist.init_process_group("gloo", init_method=f"file://{store}", rank=rank, world_size=world)
    torch.manual_seed(0)


def _cp_worker(rank, world, store, mode):
    from cosmos_rl_b200.parallel.context_parallel import ContextParallel, local_cu_seqlens
    _init(rank, world, store)
    m = GPT(_tiny())
    m.init_weights(0)
    lens = [8, 20, 4]
    cu = torch.tensor([0, 8, 28, 32])
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, 512, (32,), generator=g)
    labels = torch.randint(0, 512, (32,), generator=g)
    pos = m.get_position_ids(cu, 32)
    # full model on every rank (the oracle)
    lp_full, _ = m.logprobs(m(ids, pos, cu, max(lens)), labels)
    lp_full.sum().backward()
    ref_grads = [p.grad.clone() for p in m.parameters()]
    m.zero_grad()
    cp = ContextParallel(dist.group.WORLD, world, rank, mode)
    m.attach_context_parallel(cp)
    lcu = local_cu_seqlens(cu, world)
    h = m(cp.shard(ids, cu), cp.shard(pos, cu), lcu, max(lens) // world)
    lp, _ = m.logprobs(h, cp.shard(labels, cu))
    assert torch.allclose(lp, cp.shard(lp_full.detach(), cu), atol=1e-5), (lp - cp.shard(lp_full.detach(), cu)).abs().max()
    lp.sum().backward()
    for p, r in zip(m.parameters(), ref_grads):
        gsum = p.grad.clone()
        dist.all_reduce(gsum)
        assert torch.allclose(gsum, r, atol=2e-5), (gsum - r).abs().max()
    dist.destroy_process_group()


@pytest.mark.parametrize("mode", ["kv-gather", "ulysses"])
def test_context_parallel_matches_full_model(tmp_path, mode):
    _spawn(_cp_worker, 2, tmp_path, mode)
