"""Resharding planner: for several (policy tp, rollout tp) layouts the plan, applied as plain rectangle
copies, must reproduce exactly the weights a rollout rank would have loaded from the checkpoint itself."""
import pytest
import torch

from cosmos_rl_b200.models import hf_io
from cosmos_rl_b200.models.gpt import GPT, GPTArgs
from cosmos_rl_b200.parallel.flat import FlatParams
from cosmos_rl_b200.parallel.reshard import build_plan, merge_descriptors, model_parts, plan_for_rank, shard_info


def _args(tp=1, r=0, qk_norm=False, n_kv=2):
    return GPTArgs(vocab_size=64, dim=32, n_layers=2, n_heads=4, n_kv_heads=n_kv, ffn_dim=48, qkv_bias=not qk_norm,
                   qk_norm=qk_norm, model_type="qwen3" if qk_norm else "qwen2", tp_size=tp, tp_rank=r)


def _build(tp, hf_state, cfg, qk_norm, n_kv, dp=1):
    ranks = []
    for r in range(tp):
        with torch.device("meta"):
            m = GPT(_args(tp, r, qk_norm, n_kv))
        flat = FlatParams(m, torch.float32, torch.device("cpu"), with_grad=False)
        hf_io.load_hf_state(m, lambda k: hf_state[k], hf_state, cfg, tp, r)
        ranks.append((m, flat))
    return ranks


@pytest.mark.parametrize("ptp,rtp,qk_norm,n_kv", [(1, 1, False, 2), (1, 2, False, 2), (2, 1, False, 2), (2, 4, True, 2),
                                                   (4, 2, False, 2), (1, 4, False, 1)])
def test_plan_reproduces_checkpoint_load(ptp, rtp, qk_norm, n_kv):
    torch.manual_seed(0)
    full = GPT(_args(1, 0, qk_norm, n_kv))
    full.init_weights(1)
    for p in full.parameters():  # make norms / biases non-trivial too
        if p.dim() == 1:
            p.data.normal_()
    cfg = full.args.to_hf_config()
    hf_state = hf_io.hf_state_dict(full, cfg)
    policy = _build(ptp, hf_state, cfg, qk_norm, n_kv)
    # two data-parallel copies of every policy TP rank: ranks r and ptp + r hold the same data
    src_infos, src_flats = [], {}
    for dp in range(2):
        for r, (m, flat) in enumerate(policy):
            rank = dp * ptp + r
            src_infos.append(shard_info(rank, model_parts(m, flat), flat.total))
            src_flats[rank] = flat.data
    rollout = _build(rtp, hf_state, cfg, qk_norm, n_kv)
    used_sources = set()
    for r, (m, flat) in enumerate(rollout):
        want = flat.data.clone()
        info = shard_info(r, model_parts(m, flat), flat.total)
        flat.data.zero_()
        plan = merge_descriptors(build_plan(src_infos, info))
        for src_rank, so, sld, do, dld, rows, cols in plan:
            used_sources.add(src_rank)
            src = torch.as_strided(src_flats[src_rank], (rows, cols), (sld, 1), so)
            torch.as_strided(flat.data, (rows, cols), (dld, 1), do).copy_(src)
        # padding between slots is never written; compare parameter by parameter
        for name, p in m.named_parameters():
            ref = torch.as_strided(want, p.shape, p.stride(), p.storage_offset())
            assert torch.equal(p.data, ref), name
    assert len(used_sources) > 1 or ptp * 2 == 1  # duplicates are spread over several source ranks


def test_plan_for_rank_roles_and_missing_source():
    full = GPT(_args())
    full.init_weights(0)
    flat = FlatParams(full, torch.float32, torch.device("cpu"), with_grad=False)
    info = shard_info(0, model_parts(full, flat), flat.total)
    pol, rol = {"ranks": [info]}, {"ranks": [dict(info, rank=0)]}
    recv = plan_for_rank(pol, rol, "rollout", 0)
    send = plan_for_rank(pol, rol, "policy", 0)
    assert len(recv) == len(send) and all(s[0] == 0 for s in send)
    assert sum(d[5] * d[6] for d in recv) == sum(p.numel() for p in full.parameters())
    broken = {"ranks": [dict(info, parts=info["parts"][1:])]}
    with pytest.raises(KeyError):
        plan_for_rank(broken, rol, "rollout", 0)


@pytest.mark.parametrize("family", ["qwen3_moe", "deepseek_v3"])
def test_plan_gathers_expert_parallel_shards(family):
    """Policy ranks that each own a slice of the experts (expert parallelism) -> a rollout rank that holds all of
    them: every expert is pulled from the rank that owns it, dense parameters from either."""
    import copy
    from cosmos_rl_b200.models.deepseek_v3 import ARCHS as DS, DeepseekV3
    from cosmos_rl_b200.models.qwen3_moe import ARCHS as QM, Qwen3MoE
    cls, base = (Qwen3MoE, QM["tiny-qwen3-moe"]) if family == "qwen3_moe" else (DeepseekV3, DS["tiny-deepseek-v3"])
    base = copy.deepcopy(base)
    base.vocab_size = 512
    torch.manual_seed(0)
    full = cls(base)
    full.init_weights(2)
    cfg = base.to_hf_config()
    state = hf_io.hf_state_dict(full, cfg)
    src_infos, src_flats = [], {}
    for r in range(2):
        a = copy.deepcopy(base)
        a.ep_size, a.ep_rank = 2, r
        with torch.device("meta"):
            m = cls(a)
        flat = FlatParams(m, torch.float32, torch.device("cpu"), with_grad=False)
        hf_io.load_hf_state(m, lambda k: state[k], state, cfg)
        src_infos.append(shard_info(r, model_parts(m, flat), flat.total))
        src_flats[r] = flat.data
    with torch.device("meta"):
        dst = cls(copy.deepcopy(base))
    dflat = FlatParams(dst, torch.float32, torch.device("cpu"), with_grad=False)
    plan = merge_descriptors(build_plan(src_infos, shard_info(0, model_parts(dst, dflat), dflat.total)))
    expert_sources = set()
    for src_rank, so, sld, do, dld, rows, cols in plan:
        torch.as_strided(dflat.data, (rows, cols), (dld, 1), do).copy_(
            torch.as_strided(src_flats[src_rank], (rows, cols), (sld, 1), so))
    for (n, p), (_, q) in zip(dst.named_parameters(), full.named_parameters()):
        assert torch.equal(p, q), n
    # the second half of the experts exists on rank 1 only
    E = base.n_experts
    late = next(p for p in model_parts(dst, dflat) if f"experts.{E - 1}." in p.key)
    assert any(d[0] == 1 and d[3] <= late.off < d[3] + d[4] * d[5] for d in plan)


def test_interleave_sources_mixes_sources_and_staggers_destinations():
    """A plan sorted by source becomes one that draws on all sources at every point; the destination's rank picks the
    source it starts on; nothing is dropped or duplicated."""
    from cosmos_rl_b200.parallel.reshard import interleave_sources
    plan = [[0, i * 100, 10, i * 100, 10, 10, 10] for i in range(6)] + [[1, i * 100, 10, 600 + i * 100, 10, 10, 10] for i in range(3)] \
        + [[1, 900, 10, 900, 10, 30, 10]]
    out0, out1 = interleave_sources(plan, 0), interleave_sources(plan, 1)
    assert sorted(map(tuple, out0)) == sorted(map(tuple, plan)) == sorted(map(tuple, out1))
    assert out0[0][0] == 0 and out1[0][0] == 1
    half = out0[:len(out0) // 2]
    assert {d[0] for d in half} == {0, 1}                    # both sources appear in the first half
    by = {0: 0, 1: 0}
    for d in half:
        by[d[0]] += d[5] * d[6]
    assert abs(by[0] / 600 - by[1] / 600) < 0.5              # and about the same fraction of each has been scheduled
    assert interleave_sources(plan[:6], 3) == plan[:6]       # a single source: order kept
