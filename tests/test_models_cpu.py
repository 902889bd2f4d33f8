"""Model-level checks on CPU: packed forward vs per-sequence forward, recompute modes, generation engine vs
teacher forcing, HF safetensors export / reload (dense and MoE), training checkpoint save / resume, MoE
weight-sync parts."""
import json
import os

import pytest
import torch

from cosmos_rl_b200.config import Config
from cosmos_rl_b200.dispatcher.data.schema import Rollout
from cosmos_rl_b200.models import hf_io, named_architectures
from cosmos_rl_b200.models.gpt import ARCHS, GPT
from cosmos_rl_b200.models.qwen3_moe import ARCHS as MOE_ARCHS
from cosmos_rl_b200.models.qwen3_moe import Qwen3MoE
from cosmos_rl_b200.parallel.dims import ParallelDims
from cosmos_rl_b200.parallel.flat import FlatParams
from cosmos_rl_b200.parallel.reshard import build_plan, model_parts, shard_info
from cosmos_rl_b200.policy.trainer.grpo_trainer import GRPOTrainer
from cosmos_rl_b200.rollout.engine import RolloutEngine, SamplingParams


def _tiny(kind="dense"):
    torch.manual_seed(0)
    m = GPT(ARCHS["tiny-qwen2"]) if kind == "dense" else Qwen3MoE(MOE_ARCHS["tiny-qwen3-moe"])
    m.init_weights(0)
    return m


@pytest.mark.parametrize("kind", ["dense", "moe"])
def test_packed_forward_equals_per_sequence(kind):
    m = _tiny(kind)
    a, b = torch.randint(0, 32000, (9,)), torch.randint(0, 32000, (14,))
    ids = torch.cat([a, b])
    cu = torch.tensor([0, 9, 23])
    with torch.no_grad():
        packed = m(ids, m.get_position_ids(cu, 23), cu, 14)
        ha = m(a, torch.arange(9), torch.tensor([0, 9]), 9)
        hb = m(b, torch.arange(14), torch.tensor([0, 14]), 14)
    assert torch.allclose(packed, torch.cat([ha, hb]), atol=1e-5)


def test_recompute_modes_give_identical_gradients():
    m = _tiny()
    ids, cu = torch.randint(0, 32000, (20,)), torch.tensor([0, 8, 20])
    lab = torch.randint(0, 32000, (20,))
    grads = {}
    for mode in (False, "full", "selective", "swiglu"):
        m.gradient_checkpointing = mode
        m.zero_grad()
        lp, _ = m.logprobs(m(ids, m.get_position_ids(cu, 20), cu, 12), lab)
        lp.sum().backward()
        grads[mode] = torch.cat([p.grad.flatten() for p in m.parameters()])
    assert torch.equal(grads[False], grads["full"]) and torch.equal(grads[False], grads["selective"])
    assert torch.equal(grads[False], grads["swiglu"])


@pytest.mark.parametrize("kind", ["dense", "moe"])
def test_engine_greedy_matches_teacher_forcing_and_frees_pages(kind):
    m = _tiny(kind)
    e = RolloutEngine(m, max_num_seqs=8, max_model_len=64, page_size=16)
    prompts = [torch.randint(0, 32000, (10 + 3 * i,)).tolist() for i in range(4)]
    out = e.generate(prompts, SamplingParams(n=2, max_tokens=10, temperature=0.0))
    assert len(e.free_pages) == e.num_pages - 1
    for p, comps in zip(prompts, out):
        assert comps[0].token_ids == comps[1].token_ids            # greedy samples of one prompt agree
        ids = torch.tensor(p + comps[0].token_ids)
        with torch.no_grad():
            h = m(ids, torch.arange(len(ids)), torch.tensor([0, len(ids)]), len(ids))
            lsm = torch.log_softmax(m.logits(h).float(), -1)
        for i, (tok, lp) in enumerate(zip(comps[0].token_ids, comps[0].logprobs)):
            row = lsm[len(p) - 1 + i]
            assert int(row.argmax()) == tok and abs(row[tok].item() - lp) < 1e-3


def test_engine_stop_tokens_and_more_prompts_than_slots():
    m = _tiny()
    e = RolloutEngine(m, max_num_seqs=4, max_model_len=64, page_size=16)
    prompts = [torch.randint(0, 32000, (8,)).tolist() for _ in range(6)]     # 6 prompts x 2 samples > 4 slots
    ref = e.generate(prompts, SamplingParams(n=2, max_tokens=8, temperature=0.0))
    stop = ref[0][0].token_ids[3]
    out = e.generate(prompts, SamplingParams(n=2, max_tokens=8, temperature=0.0, stop_token_ids=(stop,)))
    first = out[0][0]
    assert first.finish_reason == "stop" and first.token_ids[-1] == stop and len(first.token_ids) <= 4
    assert all(len(c.token_ids) <= 8 for r in out for c in r)
    assert len(e.free_pages) == e.num_pages - 1


@pytest.mark.parametrize("kind", ["dense", "moe"])
def test_safetensors_export_and_reload(kind, tmp_path):
    m = _tiny(kind)
    cfg = m.args.to_hf_config()
    out = str(tmp_path / "export")
    hf_io.export_safetensors(m, cfg, out)
    index = json.load(open(os.path.join(out, "model.safetensors.index.json")))
    assert "model.layers.0.self_attn.q_proj.weight" in index["weight_map"]
    if kind == "moe":
        assert "model.layers.1.mlp.experts.7.down_proj.weight" in index["weight_map"]
    else:
        assert "model.layers.0.mlp.gate_proj.weight" in index["weight_map"]
    assert hf_io.load_hf_config(out)["hidden_size"] == m.args.dim
    m2 = type(m)(m.args)
    hf_io.load_hf_weights(m2, out)
    for (n1, p1), (n2, p2) in zip(m.named_parameters(), m2.named_parameters()):
        assert torch.equal(p1, p2), n1


def test_checkpoint_save_resume_and_prune(tmp_path):
    d = {"policy": {"model_name_or_path": "tiny-qwen2", "parallelism": {"tp_size": 1}, "model_max_length": 64},
         "train": {"optm_lr": 1e-3, "seed": 0, "output_dir": str(tmp_path), "resume": True,
                   "ckpt": {"enable_checkpoint": True, "save_mode": "sync", "max_keep": 2, "export_safetensors": False},
                   "train_policy": {"type": "grpo", "mini_batch": 4}}}
    cfg = Config.from_dict(d)
    t = GRPOTrainer(cfg, ParallelDims(world_size=1))
    assert t.weight_resume() is False
    rs = [Rollout(prompt=[1, 2, 3, 4], completion=[5, 6, 7], advantage=float(i) - 1.5, reward=0.0) for i in range(4)]
    for step in (1, 2, 3):
        t.step_training(rs, step, 10, do_save=True)
    assert t.ckpt_manager.steps_on_disk() == [2, 3]                 # max_keep pruned step 1
    w = t.flat.data.clone()
    m_state = t.optimizer.m.clone()
    t2 = GRPOTrainer(cfg, ParallelDims(world_size=1))
    assert t2.weight_resume() is True
    assert t2.train_step == 3 and torch.equal(t2.flat.data, w) and torch.equal(t2.optimizer.m, m_state)
    assert t2.optimizer.step_count == t.optimizer.step_count
    # an incomplete step directory (no completion marker) is ignored by resume
    os.makedirs(os.path.join(str(tmp_path), "checkpoints", "step_9", "policy"))
    assert t2.ckpt_manager.latest_valid_step() == 3
    # both trainers continue identically
    r1 = t.step_training(rs, 4, 10)
    r2 = t2.step_training(rs, 4, 10)
    assert abs(r1["train/grad_norm"] - r2["train/grad_norm"]) < 1e-5 and torch.allclose(t.flat.data, t2.flat.data)


def test_moe_weight_sync_parts_cover_every_parameter():
    m = _tiny("moe")
    with torch.device("meta"):
        dst = Qwen3MoE(MOE_ARCHS["tiny-qwen3-moe"])
    src_flat = FlatParams(m, torch.float32, torch.device("cpu"), with_grad=False)
    dst_flat = FlatParams(dst, torch.float32, torch.device("cpu"), with_grad=False)
    plan = build_plan([shard_info(0, model_parts(m, src_flat), src_flat.total)],
                      shard_info(0, model_parts(dst, dst_flat), dst_flat.total))
    for _, so, sld, do, dld, rows, cols in plan:
        torch.as_strided(dst_flat.data, (rows, cols), (dld, 1), do).copy_(
            torch.as_strided(src_flat.data, (rows, cols), (sld, 1), so))
    for (n1, p1), (n2, p2) in zip(m.named_parameters(), dst.named_parameters()):
        assert torch.equal(p1, p2), n1


def test_named_architectures_shapes():
    archs = named_architectures()
    a = archs["qwen2.5-7b"]
    assert (a.dim, a.n_layers, a.n_heads, a.n_kv_heads, a.ffn_dim, a.vocab_size) == (3584, 28, 28, 4, 18944, 152064)
    b = archs["qwen3-30b-a3b"]
    assert (b.dim, b.n_layers, b.n_experts, b.top_k, b.moe_ffn_dim) == (2048, 48, 128, 8, 768)
    c = archs["qwen3-32b"]
    assert (c.dim, c.n_layers, c.n_heads, c.n_kv_heads, c.ffn_dim) == (5120, 64, 64, 8, 25600)
    with torch.device("meta"):
        n = sum(p.numel() for p in GPT(a).parameters())
    assert 7.5e9 < n < 7.7e9


@pytest.mark.parametrize("cfg", [
    {"model_type": "olmo2", "vocab_size": 512, "hidden_size": 64, "intermediate_size": 128, "num_hidden_layers": 2,
     "num_attention_heads": 4, "num_key_value_heads": 2},
    {"model_type": "mistral", "vocab_size": 512, "hidden_size": 64, "intermediate_size": 128, "num_hidden_layers": 2,
     "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16},
])
def test_generic_hf_wrapper_packed_forward_and_training(cfg):
    """Families without a native implementation go through the transformers wrapper (registry fallback)."""
    from cosmos_rl_b200.models.base import ModelRegistry
    from cosmos_rl_b200.parallel.flat import FlatParams
    with torch.device("meta"):
        m = ModelRegistry.build_model(dict(cfg))
    assert type(m).__name__ == "HFModel"
    flat = FlatParams(m, torch.float32, torch.device("cpu"))
    m.init_weights(0)
    m.eval()
    a, b = torch.randint(0, 512, (7,)), torch.randint(0, 512, (12,))
    ids, cu = torch.cat([a, b]), torch.tensor([0, 7, 19])
    packed = m(ids, m.get_position_ids(cu, 19), cu, 12)
    with torch.no_grad():
        ha = m(a, torch.arange(7), torch.tensor([0, 7]), 7)
        hb = m(b, torch.arange(12), torch.tensor([0, 12]), 12)
    assert torch.allclose(packed.detach(), torch.cat([ha, hb]), atol=1e-4)
    lp, ent = m.logprobs(packed, torch.randint(0, 512, (19,)))
    lp.sum().backward()
    assert flat.grad.abs().sum() > 0 and torch.isfinite(flat.grad).all()


def test_deepseek_v3_trains_exports_and_balances(tmp_path):
    """The native DeepSeek-V3 family through the SFT trainer (named tiny architecture), the HF-name export / reload
    round trip, and the load-balancing bias update."""
    from cosmos_rl_b200.config import Config
    from cosmos_rl_b200.models.deepseek_v3 import DeepseekV3
    from cosmos_rl_b200.policy.trainer.sft_trainer import SFTTrainer
    cfg = Config.from_dict({
        "policy": {"model_name_or_path": "tiny-deepseek-v3", "model_max_length": 64, "model_gradient_checkpointing": False},
        "train": {"seed": 0, "optm_lr": 2e-3, "optm_warmup_steps": 0, "output_dir": str(tmp_path),
                  "train_policy": {"type": "sft", "trainer_type": "sft", "mini_batch": 2},
                  "ckpt": {"enable_checkpoint": False}}})
    tr = SFTTrainer(cfg, ParallelDims(world_size=1, device=torch.device("cpu")), device=torch.device("cpu"))
    tr.model_load_from_hf()
    assert isinstance(tr.model, DeepseekV3)
    g = torch.Generator().manual_seed(0)
    batch = [{"input_ids": torch.randint(0, 32000, (n,), generator=g).tolist()} for n in (12, 20, 7, 16)]
    losses = [tr.step_training(batch, total_steps=10, train_step=i + 1)["train/loss_avg"] for i in range(4)]
    assert losses[-1] < losses[0] - 0.05, losses
    bias = tr.model.layers[1].mlp.gate.e_score_correction_bias
    # moved only by the load-balancing rule (4 steps of 1e-3), never by AdamW
    assert not bias.requires_grad and 0 < bias.abs().max() <= 4e-3 + 1e-9
    before = bias.clone()
    tr.model.update_router_bias(1e-2)
    load = tr.model.layers[1].mlp.last_load
    assert torch.equal(torch.sign(bias - before), torch.sign(load.mean() - load))
    # export with HF names, reload into a fresh model, same hidden states
    hf_cfg = tr.model.args.to_hf_config()
    state = hf_io.hf_state_dict(tr.model, hf_cfg)
    assert "model.layers.1.mlp.experts.3.up_proj.weight" in state and "model.layers.0.mlp.gate_proj.weight" in state
    assert "model.layers.2.mlp.shared_experts.down_proj.weight" in state
    fresh = DeepseekV3.from_hf_config(hf_cfg)
    hf_io.load_hf_state(fresh, lambda n: state[n], state, hf_cfg)
    ids, cu = torch.randint(0, 32000, (15,), generator=g), torch.tensor([0, 6, 15])
    with torch.no_grad():
        a = tr.model(ids, tr.model.get_position_ids(cu, 15), cu, 9)
        b = fresh(ids, fresh.get_position_ids(cu, 15), cu, 9)
    assert torch.allclose(a, b, atol=1e-6)


def _tiny_vlm_config():
    return {"model_type": "qwen2_5_vl",
            "text_config": dict(vocab_size=512, hidden_size=64, num_hidden_layers=2, num_attention_heads=4,
                                num_key_value_heads=2, intermediate_size=128, max_position_embeddings=256,
                                rope_parameters={"rope_type": "default", "mrope_section": [2, 3, 3], "rope_theta": 10000.0}),
            "vision_config": dict(depth=2, hidden_size=32, intermediate_size=64, num_heads=2, out_hidden_size=64,
                                  patch_size=4, spatial_merge_size=2, temporal_patch_size=2, window_size=16,
                                  fullatt_block_indexes=[1], in_channels=3),
            "image_token_id": 500, "video_token_id": 501, "vision_start_token_id": 502, "vision_end_token_id": 503}


def _vlm_sample(g, n_text):
    """One 16 x 16 image: a 4 x 4 patch grid, merged 2 x 2 -> four image tokens between the vision markers."""
    ids = [1, 2, 502, 500, 500, 500, 500, 503] + torch.randint(3, 400, (n_text,), generator=g).tolist()
    return {"input_ids": ids, "pixel_values": torch.randn(16, 3 * 2 * 4 * 4, generator=g), "image_grid_thw": torch.tensor([[1, 4, 4]])}


def test_vision_language_model_through_wrapper_packer_and_trainers(tmp_path):
    """A vision-language family (Qwen2.5-VL architecture) through the transformers wrapper: packed forward with pixel
    inputs equals the HF model per sample, the image changes the output, SFT and GRPO steps train the vision tower,
    and the HF rollout backend generates from image prompts."""
    from cosmos_rl_b200.config import Config
    from cosmos_rl_b200.data.packer import BaseDataPacker, HFVLMDataPacker, merge_mm
    from cosmos_rl_b200.policy.trainer.sft_trainer import SFTTrainer
    cfg = Config.from_dict({
        "policy": {"model_name_or_path": "tiny-vlm", "model_max_length": 64, "model_gradient_checkpointing": False},
        "custom": {"model_config": _tiny_vlm_config()},
        "rollout": {"n_generation": 2, "max_response_length": 4, "sampling_config": {"temperature": 1.0}},
        "train": {"seed": 0, "optm_lr": 2e-3, "optm_warmup_steps": 0, "output_dir": str(tmp_path),
                  "force_use_hf": True,                  # the wrapper path (the family also has a native model)
                  "train_policy": {"type": "sft", "trainer_type": "sft", "mini_batch": 2},
                  "ckpt": {"enable_checkpoint": False}}})
    assert BaseDataPacker.get_default("qwen2_5_vl") is HFVLMDataPacker
    packer = HFVLMDataPacker()
    packer.setup(cfg, None)
    cpu = torch.device("cpu")
    tr = SFTTrainer(cfg, ParallelDims(world_size=1, device=cpu), device=cpu, data_packer=packer)
    tr.model_load_from_hf()
    m = tr.model
    assert m.is_vlm and type(m.inner).__name__ == "Qwen2_5_VLForConditionalGeneration"
    g = torch.Generator().manual_seed(0)
    a, b = _vlm_sample(g, 5), _vlm_sample(g, 9)
    ids = torch.tensor(a["input_ids"] + b["input_ids"])
    cu = torch.tensor([0, len(a["input_ids"]), len(a["input_ids"]) + len(b["input_ids"])])
    m.eval()
    with torch.no_grad():
        m.mm_inputs = merge_mm([a, b])
        packed = m(ids, m.get_position_ids(cu, int(cu[-1])), cu, len(b["input_ids"]))
        for s, (lo, hi) in zip((a, b), ((0, int(cu[1])), (int(cu[1]), int(cu[2])))):
            t = torch.tensor([s["input_ids"]])
            want = m.inner.model(input_ids=t, attention_mask=torch.ones_like(t), pixel_values=s["pixel_values"],
                                 image_grid_thw=s["image_grid_thw"]).last_hidden_state[0]
            assert torch.allclose(packed[lo:hi], want, atol=1e-4)
        m.mm_inputs = merge_mm([dict(a, pixel_values=torch.randn(16, 96, generator=g) * 20), b])
        other = m(ids, m.get_position_ids(cu, int(cu[-1])), cu, len(b["input_ids"]))
        assert (other[: int(cu[1])] - packed[: int(cu[1])]).abs().max() > 1e-5                 # the image matters
        assert torch.equal(other[int(cu[1]):], packed[int(cu[1]):])                             # ... to its own sample only
    batch = [_vlm_sample(g, n) for n in (6, 10, 4, 8)]
    losses = [tr.step_training(batch, total_steps=10, train_step=i + 1)["train/loss_avg"] for i in range(4)]
    assert losses[-1] < losses[0] - 0.02, losses
    vis = [s for s in tr.flat.slots if "visual" in s.name][0]
    assert tr.optimizer.m[vis.offset: vis.offset + vis.numel].abs().sum() > 0                   # vision tower is trained
    # GRPO sample preparation carries the pixel inputs; rollouts come from the transformers generate loop
    from cosmos_rl_b200.dispatcher.data.schema import RLPayload, Rollout
    from cosmos_rl_b200.policy.trainer.grpo_trainer import GRPOTrainer
    from cosmos_rl_b200.rollout.hf_rollout import HFRollout
    gcfg = Config.from_dict({**cfg.model_dump(), "train": {**cfg.train.model_dump(), "train_policy": {
        "type": "grpo", "trainer_type": "grpo", "mini_batch": 2, "rollout_as_token_ids": True}}})
    gt = GRPOTrainer(gcfg, ParallelDims(world_size=1, device=cpu), device=cpu, data_packer=packer)
    gt.model_load_from_hf()
    ro = HFRollout(gcfg, ParallelDims(world_size=1, device=cpu), cpu)
    ro.init_engine(shared_model=gt.model)
    prompt = _vlm_sample(g, 3)
    res = ro.rollout_generation([RLPayload(prompt=prompt, prompt_idx=0)], packer)
    assert len(res[0].completion_token_ids) == 2 and all(1 <= len(t) <= 4 for t in res[0].completion_token_ids)
    ros = [Rollout(prompt=prompt, completion=t, advantage=adv, reward=adv) for t, adv in zip(res[0].completion_token_ids, (1.0, -1.0))]
    rep = gt.step_training(ros, 1, 10)
    assert rep["train/grad_norm"] > 0 and torch.isfinite(torch.tensor(rep["train/loss_avg"]))


def test_engine_repetition_penalty_matches_step_by_step_rule():
    """Greedy decoding with a repetition penalty: the engine's tokens equal a plain loop that divides positive / multiplies
    negative logits of every token already in the prompt or the output."""
    m = _tiny()
    eng = RolloutEngine(m, max_num_seqs=4, max_model_len=64, page_size=16, use_cuda_graph=False)
    prompts = [[5, 9, 9, 120, 7], [31000, 2, 2]]
    sp = SamplingParams(n=2, max_tokens=6, temperature=0.0, repetition_penalty=1.8)
    out = eng.generate(prompts, sp)
    assert eng.seen is not None and eng.rep_penalty == 1.8
    plain = eng.generate(prompts, SamplingParams(n=1, max_tokens=6, temperature=0.0))
    assert eng.rep_penalty == 1.0
    for p, comps, base in zip(prompts, out, plain):
        seq, seen = list(p), set(p)
        want = []
        for _ in range(6):
            ids = torch.tensor(seq)
            with torch.no_grad():
                h = m(ids, torch.arange(len(seq)), torch.tensor([0, len(seq)]), len(seq))
                logits = m.logits(h[-1:])[0].float()
            idx = torch.tensor(sorted(seen))
            logits[idx] = torch.where(logits[idx] > 0, logits[idx] / 1.8, logits[idx] * 1.8)
            t = int(logits.argmax())
            want.append(t)
            seq.append(t)
            seen.add(t)
        assert comps[0].token_ids == want and comps[1].token_ids == want
        assert len(base[0].token_ids) == 6


def test_weighted_pipeline_layer_split():
    """The last / first pipeline stage can be charged for lm_head / embedding in block-equivalents."""
    from cosmos_rl_b200.models.gpt import GPT, GPTArgs
    kw = dict(vocab_size=152064, dim=3584, n_layers=28, n_heads=28, n_kv_heads=4, head_dim=128, ffn_dim=18944)
    assert GPTArgs(pp_size=4, **kw).stage_bounds() == [0, 7, 14, 21, 28]
    b = GPTArgs(pp_size=4, pp_head_weight=-1, **kw).stage_bounds()           # lm_head of this shape ~ 2.3 blocks
    assert b == [0, 8, 15, 23, 28]
    small = dict(vocab_size=512, dim=64, n_heads=4, n_kv_heads=2, ffn_dim=128)
    assert GPTArgs(n_layers=7, pp_size=2, pp_head_weight=2, pp_embed_weight=1, **small).stage_bounds() == [0, 4, 7]
    assert GPTArgs(n_layers=3, pp_size=3, pp_head_weight=50, **small).stage_bounds() == [0, 1, 2, 3]   # never empty
    stages = [GPT(GPTArgs(n_layers=7, pp_size=2, pp_rank=r, pp_head_weight=2, pp_embed_weight=1, **small)) for r in (0, 1)]
    assert [len(s.layers) for s in stages] == [4, 3] and stages[1].layer_offset == 4


def _tiny_qwen25vl_config():
    from transformers import Qwen2_5_VLConfig
    return Qwen2_5_VLConfig(
        text_config=dict(hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                         intermediate_size=128, vocab_size=300, max_position_embeddings=512,
                         rope_parameters={"rope_type": "default", "rope_theta": 10000.0, "mrope_section": [2, 3, 3]}),
        vision_config=dict(depth=3, hidden_size=32, num_heads=2, intermediate_size=48, out_hidden_size=64, patch_size=14,
                           temporal_patch_size=2, spatial_merge_size=2, window_size=56, fullatt_block_indexes=[1],
                           in_channels=3),
        image_token_id=290, video_token_id=291, vision_start_token_id=292, vision_end_token_id=293)


def test_native_qwen25vl_matches_transformers_and_round_trips_weights():
    """The native Qwen2.5-VL (windowed vision tower, 2 x 2 merger, placeholder scatter, multimodal rotary positions on the
    shared GPT decoder) reproduces the transformers implementation on a packed batch of two sequences with one image each
    (different grids, so window and full-attention blocks differ); its weights export to checkpoint names and shapes and
    load back; gradients reach the vision tower. Reference family: cosmos_rl/policy/model/qwen2_5_vl/__init__.py:566."""
    from transformers import Qwen2_5_VLForConditionalGeneration
    from cosmos_rl_b200.models.base import ModelRegistry
    from cosmos_rl_b200.models.qwen2_5_vl import Qwen25VL, Qwen25VLArgs, mrope_positions
    torch.manual_seed(0)
    cfg = _tiny_qwen25vl_config()
    hf = Qwen2_5_VLForConditionalGeneration(cfg).eval().float()
    for p in hf.parameters():
        torch.nn.init.normal_(p, 0, 0.05)
    state = hf.state_dict()
    assert ModelRegistry.get("qwen2_5_vl") is Qwen25VL
    m = Qwen25VL(Qwen25VLArgs.from_hf_config(cfg.to_dict())).float()
    hf_io.load_hf_state(m, lambda k: state[k], state, cfg.to_dict())
    grids = torch.tensor([[1, 6, 4], [1, 4, 8]])
    pix = torch.randn(int((grids[:, 0] * grids[:, 1] * grids[:, 2]).sum()), 3 * 2 * 14 * 14)
    seq1 = [1, 2, 3, 4, 292] + [290] * 6 + [293, 7, 8, 9]
    seq2 = [5, 292] + [290] * 8 + [293, 11, 12]
    ids = torch.tensor(seq1 + seq2)
    cu = torch.tensor([0, len(seq1), len(seq1) + len(seq2)], dtype=torch.int32)
    m.mm_inputs = {"pixel_values": pix, "image_grid_thw": grids}
    pos = m.get_position_ids(cu, ids.numel(), ids)
    # 5 text tokens, a 3 x 2 merged grid starting at 5 (rows 5..7, columns 5..6), text resumes at 5 + max(3, 2)
    assert pos[:, :len(seq1)].tolist() == [[0, 1, 2, 3, 4, 5, 5, 5, 5, 5, 5, 8, 9, 10, 11],
                                           [0, 1, 2, 3, 4, 5, 5, 6, 6, 7, 7, 8, 9, 10, 11],
                                           [0, 1, 2, 3, 4, 5, 6, 5, 6, 5, 6, 8, 9, 10, 11]]
    assert pos[:, len(seq1)].tolist() == [0, 0, 0]                        # positions restart with every sequence
    hid = m(ids, m.get_position_ids(cu, ids.numel()), cu, 15)             # 1-D positions in: the model derives the rest
    mine = m.logits(hid)
    ref, off = [], 0
    with torch.no_grad():
        for s, g in ((seq1, grids[0:1]), (seq2, grids[1:2])):
            n = int(g[0, 0] * g[0, 1] * g[0, 2])
            t = torch.tensor([s])
            ref.append(hf(input_ids=t, pixel_values=pix[off:off + n], image_grid_thw=g,
                          mm_token_type_ids=(t == 290).long()).logits[0])
            off += n
    ref = torch.cat(ref)
    assert (mine - ref).abs().max().item() < 2e-4 * max(1.0, ref.abs().max().item()), (mine - ref).abs().max()
    mine.square().mean().backward()
    g_vis = m.visual.blocks[0].qkv.weight.grad
    assert g_vis is not None and g_vis.abs().sum() > 0 and m.visual.patch_embed.weight.grad.abs().sum() > 0
    # export: checkpoint names and shapes; load back into a fresh model
    out = hf_io.hf_state_dict(m, cfg.to_dict())
    assert set(out) == set(state), (sorted(set(state) - set(out))[:5], sorted(set(out) - set(state))[:5])
    for k, v in out.items():
        assert tuple(v.shape) == tuple(state[k].shape), k
        assert torch.allclose(v, state[k]), k
    m2 = Qwen25VL(Qwen25VLArgs.from_hf_config(cfg.to_dict())).float()
    old = {("model." + k[len("model.language_model."):] if k.startswith("model.language_model.") else
            (k[len("model."):] if k.startswith("model.visual.") else k)): v for k, v in out.items()}
    hf_io.load_hf_state(m2, lambda k: old[k], old, cfg.to_dict())         # the older, flatter checkpoint naming
    for (n, a), (_, b) in zip(m.named_parameters(), m2.named_parameters()):
        assert torch.equal(a, b), n
    # a video: 2 frames of a 2 x 2 merged grid, interval 2 tokens per second x 1 s
    vpos = mrope_positions(torch.tensor([7, 291, 291, 291, 291, 291, 291, 291, 291, 9]), torch.tensor([0, 10]), 290, 291,
                           None, torch.tensor([[2, 4, 4]]), 2, tokens_per_second=2.0, second_per_grid_ts=[1.0])
    assert vpos[0].tolist() == [0, 1, 1, 1, 1, 3, 3, 3, 3, 4] and vpos[1].tolist() == [0, 1, 1, 2, 2, 1, 1, 2, 2, 4]


@pytest.mark.parametrize("norm_type,qk_norm", [("layer_norm", False), ("rms_norm", True)])
def test_native_internvl_matches_transformers(norm_type, qk_norm):
    """Native InternVL (tile tower with class token and learned positions, layer-scaled blocks, pixel-shuffle projector,
    placeholder scatter on the shared GPT decoder) against transformers on a packed batch of two sequences with two tiles
    and one tile; checkpoint names and shapes round-trip; the weight-sync parts of a tensor-parallel pair of policy
    ranks cover an unsharded rollout model. Reference family: cosmos_rl/policy/model/internvl/__init__.py:247."""
    from transformers import InternVLConfig, InternVLForConditionalGeneration
    from cosmos_rl_b200.models.base import ModelRegistry
    from cosmos_rl_b200.models.internvl import InternVL, InternVLArgs
    torch.manual_seed(0)
    cfg = InternVLConfig(
        text_config=dict(model_type="qwen2", hidden_size=64, num_hidden_layers=2, num_attention_heads=4,
                         num_key_value_heads=2, intermediate_size=128, vocab_size=300, max_position_embeddings=512,
                         rope_theta=10000.0),
        vision_config=dict(hidden_size=32, num_hidden_layers=2, num_attention_heads=2, intermediate_size=48,
                           image_size=[56, 56], patch_size=[14, 14], norm_type=norm_type, use_qk_norm=qk_norm,
                           attention_bias=True),
        image_token_id=290, downsample_ratio=0.5)
    hf = InternVLForConditionalGeneration(cfg).eval().float()
    for p in hf.parameters():
        torch.nn.init.normal_(p, 0, 0.05)
    state = hf.state_dict()
    assert ModelRegistry.get("internvl") is InternVL
    m = InternVL(InternVLArgs.from_hf_config(cfg.to_dict())).float()
    hf_io.load_hf_state(m, lambda k: state[k], state, cfg.to_dict())
    pix = torch.randn(3, 3, 56, 56)                       # three tiles of 4 x 4 patches -> 4 tokens each
    seq1 = [1, 2, 3] + [290] * 8 + [7, 8, 9]
    seq2 = [5] + [290] * 4 + [11, 12]
    ids = torch.tensor(seq1 + seq2)
    cu = torch.tensor([0, len(seq1), len(seq1) + len(seq2)], dtype=torch.int32)
    m.mm_inputs = {"pixel_values": pix}
    mine = m.logits(m(ids, m.get_position_ids(cu, ids.numel()), cu, len(seq1)))
    with torch.no_grad():
        ref = torch.cat([hf(input_ids=torch.tensor([seq1]), pixel_values=pix[:2]).logits[0],
                         hf(input_ids=torch.tensor([seq2]), pixel_values=pix[2:]).logits[0]])
    assert (mine - ref).abs().max().item() < 1e-4, (mine - ref).abs().max()
    mine.square().mean().backward()
    assert m.visual.blocks[0].q_proj.weight.grad.abs().sum() > 0 and m.visual.patch_embed.weight.grad.abs().sum() > 0
    out = hf_io.hf_state_dict(m, cfg.to_dict())
    assert set(out) == set(state)
    for k, v in out.items():
        assert tuple(v.shape) == tuple(state[k].shape) and torch.allclose(v, state[k]), k
    # weight sync: two tensor-parallel policy ranks -> one unsharded rollout model
    flat_dst = FlatParams(m, torch.float32, torch.device("cpu"), with_grad=False)
    infos = []
    for r in range(2):
        a = InternVLArgs.from_hf_config(cfg.to_dict(), tp_size=2, tp_rank=r)
        mr = InternVL(a).float()
        hf_io.load_hf_state(mr, lambda k: state[k], state, cfg.to_dict(), 2, r)
        fr = FlatParams(mr, torch.float32, torch.device("cpu"), with_grad=False)
        infos.append((shard_info(r, model_parts(mr, fr), fr.total), fr))
    want = flat_dst.data.clone()
    flat_dst.data.zero_()
    plan = build_plan([i for i, _ in infos], shard_info(0, model_parts(m, flat_dst), flat_dst.total))
    for src, so, sld, do, dld, rows, cols in plan:
        torch.as_strided(flat_dst.data, (rows, cols), (dld, 1), do).copy_(
            torch.as_strided(infos[src][1].data, (rows, cols), (sld, 1), so))
    for name, p in m.named_parameters():
        ref_p = torch.as_strided(want, p.shape, p.stride(), p.storage_offset())
        assert torch.equal(p.data, ref_p), name


def test_native_qwen3_vl_moe_matches_transformers():
    """Native Qwen3-VL-MoE (vision tower with bilinearly resampled learned positions and deep-stack taps added behind the
    first decoder blocks, interleaved multimodal rotary positions, Qwen3-MoE decoder with stacked experts) against
    transformers on a packed batch with two images; checkpoint names and shapes round-trip; the weight-sync plan from
    two expert-parallel policy ranks covers an unsharded rollout model.
    Reference family: cosmos_rl/policy/model/qwen3_vl_moe/__init__.py:356."""
    from transformers import Qwen3VLMoeConfig, Qwen3VLMoeForConditionalGeneration
    from cosmos_rl_b200.models.base import ModelRegistry
    from cosmos_rl_b200.models.qwen3_vl_moe import Qwen3VLMoE, Qwen3VLMoEArgs
    torch.manual_seed(0)
    cfg = Qwen3VLMoeConfig(
        text_config=dict(hidden_size=64, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                         intermediate_size=128, moe_intermediate_size=32, num_experts=4, num_experts_per_tok=2,
                         vocab_size=300, max_position_embeddings=512, decoder_sparse_step=1, mlp_only_layers=[],
                         rope_parameters={"rope_type": "default", "rope_theta": 10000.0, "mrope_section": [4, 2, 2],
                                          "mrope_interleaved": True}),
        vision_config=dict(depth=3, hidden_size=32, num_heads=2, intermediate_size=48, out_hidden_size=64, patch_size=16,
                           temporal_patch_size=2, spatial_merge_size=2, num_position_embeddings=36,
                           deepstack_visual_indexes=[0, 2], in_channels=3),
        image_token_id=290, video_token_id=291, vision_start_token_id=292, vision_end_token_id=293)
    hf = Qwen3VLMoeForConditionalGeneration(cfg).eval().float()
    for p in hf.parameters():
        torch.nn.init.normal_(p, 0, 0.05)
    state = hf.state_dict()
    assert ModelRegistry.get("qwen3_vl_moe") is Qwen3VLMoE
    m = Qwen3VLMoE(Qwen3VLMoEArgs.from_hf_config(cfg.to_dict())).float()
    hf_io.load_hf_state(m, lambda k: state[k], state, cfg.to_dict())
    grids = torch.tensor([[1, 6, 4], [1, 4, 8]])
    pix = torch.randn(int((grids[:, 0] * grids[:, 1] * grids[:, 2]).sum()), 3 * 2 * 16 * 16)
    seq1 = [1, 2, 3, 4, 292] + [290] * 6 + [293, 7, 8, 9]
    seq2 = [5, 292] + [290] * 8 + [293, 11, 12]
    ids = torch.tensor(seq1 + seq2)
    cu = torch.tensor([0, len(seq1), len(seq1) + len(seq2)], dtype=torch.int32)
    m.mm_inputs = {"pixel_values": pix, "image_grid_thw": grids}
    mine = m.logits(m(ids, m.get_position_ids(cu, ids.numel()), cu, 15))
    assert all(l.ds_rows is None for l in m.layers)                    # the taps do not outlive the call
    ref, off = [], 0
    with torch.no_grad():
        for s, g in ((seq1, grids[0:1]), (seq2, grids[1:2])):
            n = int(g[0, 0] * g[0, 1] * g[0, 2])
            t = torch.tensor([s])
            ref.append(hf(input_ids=t, pixel_values=pix[off:off + n], image_grid_thw=g,
                          mm_token_type_ids=(t == 290).long()).logits[0])
            off += n
    ref = torch.cat(ref)
    assert (mine - ref).abs().max().item() < 1e-4, (mine - ref).abs().max()
    mine.square().mean().backward()
    assert m.visual.deepstack[0].fc1.weight.grad.abs().sum() > 0 and m.visual.pos_embed.weight.grad.abs().sum() > 0
    assert m.layers[0].mlp.w_gate_up.grad.abs().sum() > 0
    out = hf_io.hf_state_dict(m, cfg.to_dict())
    assert set(out) == set(state)
    for k, v in out.items():
        assert tuple(v.shape) == tuple(state[k].shape) and torch.allclose(v, state[k]), k
    # weight sync: two expert-parallel policy ranks -> one rollout model that holds every expert
    flat_dst = FlatParams(m, torch.float32, torch.device("cpu"), with_grad=False)
    infos = []
    for r in range(2):
        mr = Qwen3VLMoE(Qwen3VLMoEArgs.from_hf_config(cfg.to_dict(), ep_size=2, ep_rank=r)).float()
        hf_io.load_hf_state(mr, lambda k: state[k], state, cfg.to_dict())
        assert mr.layers[0].mlp.w_down.shape[0] == 2
        fr = FlatParams(mr, torch.float32, torch.device("cpu"), with_grad=False)
        infos.append((shard_info(r, model_parts(mr, fr), fr.total), fr))
    want = flat_dst.data.clone()
    flat_dst.data.zero_()
    plan = build_plan([i for i, _ in infos], shard_info(0, model_parts(m, flat_dst), flat_dst.total))
    for src, so, sld, do, dld, rows, cols in plan:
        torch.as_strided(flat_dst.data, (rows, cols), (dld, 1), do).copy_(
            torch.as_strided(infos[src][1].data, (rows, cols), (sld, 1), so))
    for name, p in m.named_parameters():
        assert torch.equal(p.data, torch.as_strided(want, p.shape, p.stride(), p.storage_offset())), name


def test_native_vlm_grpo_with_recompute_rollouts(tmp_path):
    """The native Qwen2.5-VL end to end on one process: the rollout side generates from image prompts by re-running the
    packed forward (pixels handed over per step, multimodal positions derived inside the model), the GRPO trainer
    trains on the completions with the pixel inputs of the prompts, and the vision tower receives gradient."""
    from cosmos_rl_b200.config import Config
    from cosmos_rl_b200.data.packer import HFVLMDataPacker
    from cosmos_rl_b200.dispatcher.data.schema import RLPayload, Rollout
    from cosmos_rl_b200.models.base import ModelRegistry
    from cosmos_rl_b200.models.qwen2_5_vl import Qwen25VL
    from cosmos_rl_b200.policy.trainer.grpo_trainer import GRPOTrainer
    from cosmos_rl_b200.rollout.base import RolloutRegistry
    cfg = Config.from_dict({
        "policy": {"model_name_or_path": "tiny-vlm", "model_max_length": 64, "model_gradient_checkpointing": False},
        "custom": {"model_config": _tiny_vlm_config()},
        "rollout": {"n_generation": 2, "max_response_length": 4, "sampling_config": {"temperature": 1.0}},
        "train": {"seed": 0, "optm_lr": 2e-3, "optm_warmup_steps": 0, "output_dir": str(tmp_path),
                  "train_policy": {"type": "grpo", "trainer_type": "grpo", "mini_batch": 2, "rollout_as_token_ids": True},
                  "ckpt": {"enable_checkpoint": False}}})
    packer = HFVLMDataPacker()
    packer.setup(cfg, None)
    cpu = torch.device("cpu")
    assert ModelRegistry.get("qwen2_5_vl") is Qwen25VL and not Qwen25VL.paged_engine
    gt = GRPOTrainer(cfg, ParallelDims(world_size=1, device=cpu), device=cpu, data_packer=packer)
    gt.model_load_from_hf()
    assert type(gt.model) is Qwen25VL
    ro = RolloutRegistry.get("recompute")(cfg, ParallelDims(world_size=1, device=cpu), cpu)
    ro.init_engine(shared_model=gt.model)
    g = torch.Generator().manual_seed(0)
    prompts = [_vlm_sample(g, 3), _vlm_sample(g, 5)]
    res = ro.rollout_generation([RLPayload(prompt=p, prompt_idx=i) for i, p in enumerate(prompts)], packer)
    assert len(res) == 2 and all(len(r.completion_token_ids) == 2 for r in res)
    assert all(1 <= len(t) <= 4 for r in res for t in r.completion_token_ids)
    ros = [Rollout(prompt=p, completion=t, advantage=adv, reward=adv)
           for p, r in zip(prompts, res) for t, adv in zip(r.completion_token_ids, (1.0, -1.0))]
    w0 = gt.model.visual.blocks[0].qkv.weight.detach().clone()
    rep = gt.step_training(ros, 1, 10)
    assert rep["train/grad_norm"] > 0 and torch.isfinite(torch.tensor(rep["train/loss_avg"]))
    assert (gt.model.visual.blocks[0].qkv.weight - w0).abs().max() > 0
