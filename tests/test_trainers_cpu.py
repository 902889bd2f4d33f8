"""CPU tests of the SFT and DPO trainers and of the GRPO loss variants against hand-written statements."""
import math

import pytest

import torch

from cosmos_rl_b200.config import Config
from cosmos_rl_b200.parallel.dims import ParallelDims
from cosmos_rl_b200.policy import loss as L


def _config(tmp_path, kind):
    return Config.from_dict({
        "policy": {"model_name_or_path": "tiny-qwen2", "model_max_length": 64, "model_gradient_checkpointing": False},
        "train": {"seed": 0, "optm_lr": 1e-3, "optm_warmup_steps": 0, "output_dir": str(tmp_path),
                  "train_policy": {"type": "sft", "trainer_type": kind, "mini_batch": 2},
                  "ckpt": {"enable_checkpoint": False}},
        "custom": {"dpo_beta": 0.2},
    })


def test_sft_trainer_reduces_loss_on_a_fixed_batch(tmp_path):
    from cosmos_rl_b200.policy.trainer.sft_trainer import SFTTrainer
    tr = SFTTrainer(_config(tmp_path, "sft"), ParallelDims(world_size=1, device=torch.device("cpu")),
                    device=torch.device("cpu"))
    tr.model_load_from_hf()
    g = torch.Generator().manual_seed(0)
    batch = [{"input_ids": torch.randint(0, 32000, (n,), generator=g).tolist()} for n in (12, 20, 7, 16)]
    batch[1]["label_ids"] = [-100] * 8 + batch[1]["input_ids"][8:]            # prompt part is not learned
    losses = [tr.step_training(batch, total_steps=10, train_step=i + 1)["train/loss_avg"] for i in range(4)]
    assert all(math.isfinite(x) for x in losses) and losses[-1] < losses[0] - 0.05, losses
    assert abs(losses[0] - math.log(32000)) < 0.5                              # random init: about ln(V)
    assert tr.step_validation(batch)["val/loss"] < losses[0]


def test_dpo_trainer_step_and_reference_is_frozen(tmp_path):
    from cosmos_rl_b200.policy.trainer.dpo_trainer import DPOTrainer
    tr = DPOTrainer(_config(tmp_path, "dpo"), ParallelDims(world_size=1, device=torch.device("cpu")),
                    device=torch.device("cpu"))
    tr.model_load_from_hf()
    g = torch.Generator().manual_seed(1)
    tok = lambda n: torch.randint(0, 32000, (n,), generator=g).tolist()
    batch = [{"prompt": tok(6), "chosen": tok(5), "rejected": tok(7)} for _ in range(4)]
    r0 = tr.step_training(batch, total_steps=10, train_step=1)
    assert abs(r0["train/loss_avg"] - math.log(2.0)) < 1e-4                    # policy == reference at step 1
    ref_state = tr.reference_state.clone()
    r1 = tr.step_training(batch, total_steps=10, train_step=2)
    r2 = tr.step_training(batch, total_steps=10, train_step=3)
    assert torch.equal(tr.reference_state, ref_state)                          # the reference never moves
    assert r2["train/loss_avg"] < r0["train/loss_avg"] and r2["train/reward_acc"] >= 0.5
    assert math.isfinite(r1["train/grad_norm"])


def test_grpo_loss_variants_by_hand():
    lp = torch.tensor([-1.0, -2.0, -0.5, -1.5], requires_grad=True)
    old = torch.tensor([-1.2, -1.5, -0.5, -3.0])
    A = torch.tensor([1.0, 1.0, -2.0, -2.0])
    seq = torch.tensor([0, 0, 1, 1])
    cfg = L.GrpoLossConfig(epsilon_low=0.2, epsilon_high=0.2, lower_bound_ratio=3.0)
    loss, m = L.grpo_loss(lp, old, A, seq, 2, cfg)
    ratio = torch.exp(lp.detach() - old)
    want = []
    for r, a in zip(ratio.tolist(), A.tolist()):
        v = -min(r * a, max(min(r, 1.2), 0.8) * a)
        if a < 0:
            v = min(v, -3.0 * a)
        want.append(v)
    assert abs(loss.item() - sum(want) / 4) < 1e-6
    assert abs(m["clip_frac"].item() - 0.25) < 1e-6                # token 0 (ratio 1.22 > 1.2); token 3 is cut by the dual clip
    loss.backward()
    assert lp.grad[0].item() == 0.0 and lp.grad[3].item() == 0.0   # clipped tokens carry no gradient
    assert abs(lp.grad[1].item() + ratio[1].item() / 4) < 1e-6
    # sequence-level reductions
    per = torch.tensor(want)
    cfg2 = L.GrpoLossConfig(loss_type="seq-mean-token-mean")
    l2, _ = L.grpo_loss(lp.detach(), old, A, seq, 2, cfg2)
    assert abs(l2.item() - ((per[0] + per[1]) / 2 + (per[2] + per[3]) / 2).item() / 2) < 1e-6
    # k3 KL term
    ref = torch.tensor([-1.1, -2.5, -0.4, -1.0])
    l3, m3 = L.grpo_loss(lp.detach(), old, A, seq, 2, L.GrpoLossConfig(kl_beta=0.5), ref_logprob=ref)
    r = ref - lp.detach()
    kl = (torch.exp(r) - r - 1).mean()
    assert abs(m3["kl"].item() - kl.item()) < 1e-6 and abs(l3.item() - (sum(want) / 4 + 0.5 * kl.item())) < 1e-6
    # GSPO: one ratio per sequence
    l4, m4 = L.grpo_loss(lp.detach(), old, A, seq, 2, L.GrpoLossConfig(variant="gspo"))
    sr = torch.exp(torch.tensor([((lp.detach() - old)[:2]).mean(), ((lp.detach() - old)[2:]).mean()]))
    w4 = [-min(sr[s].item() * a, max(min(sr[s].item(), 1.2), 0.8) * a) for s, a in zip([0, 0, 1, 1], A.tolist())]
    assert abs(l4.item() - sum(w4) / 4) < 1e-6
    # DPO loss
    d, dm = L.dpo_loss(torch.tensor([-3.0]), torch.tensor([-5.0]), torch.tensor([-4.0]), torch.tensor([-4.5]), beta=0.5)
    assert abs(d.item() + math.log(1 / (1 + math.exp(-0.5 * (2.0 - 0.5))))) < 1e-6 and dm["reward_acc"].item() == 1.0


def test_grpo_trainer_with_reference_kl_mu_iterations_and_variants(tmp_path):
    """A GRPO step with a KL reference phase, an old-log-prob phase (mu = 2) and the loss variants runs end to end:
    finite loss, weights move, the reference copy does not."""
    import pytest
    from cosmos_rl_b200.colocated import ColocatedGRPO
    for over in ({"kl_beta": 0.05, "mu_iterations": 2},
                 {"variant": "dapo", "loss_type": "seq-mean-token-mean", "epsilon_high": 0.28},
                 {"variant": "gspo", "kl_beta": 0.01, "unbiased_kl_estimate": True},
                 {"aipo_rho": 1.5, "entropy_coeff": 0.001, "positive_nll_coef": 0.1}):
        tp = {"type": "grpo", "reward_function": ["even_token_fraction"], "mini_batch": 4, "temperature": 1.0}
        tp.update(over)
        cfg = Config.from_dict({
            "mode": "colocated",
            "policy": {"model_name_or_path": "tiny-qwen2", "model_max_length": 96, "model_gradient_checkpointing": False},
            "rollout": {"n_generation": 4, "batch_size": 2, "max_response_length": 16, "seed": 3},
            "train": {"seed": 0, "optm_lr": 1e-3, "optm_warmup_steps": 0, "output_dir": str(tmp_path),
                      "train_policy": tp, "ckpt": {"enable_checkpoint": False}}})
        job = ColocatedGRPO(cfg, device=torch.device("cpu"), max_num_seqs=8)
        g = torch.Generator().manual_seed(0)
        prompts = [torch.randint(0, 32000, (10,), generator=g) for _ in range(2)]
        w0 = job.trainer.flat.data.clone()
        ref0 = None if job.trainer.reference_state is None else job.trainer.reference_state.clone()
        rep = job.step(prompts)
        assert math.isfinite(rep["train/loss_avg"]) and math.isfinite(rep["train/grad_norm"]), (over, rep)
        assert not torch.equal(job.trainer.flat.data, w0), over
        if ref0 is not None:
            assert torch.equal(job.trainer.reference_state, ref0)
            assert rep["train/kl"] >= 0.0


def test_lora_on_native_model_through_the_trainer(tmp_path):
    """[policy.lora] on the native GPT: adapters on the fused projections, base weights frozen, merge / unmerge around
    weight hand-over, PEFT-layout export with the fused adapters split back."""
    import os
    import torch
    from safetensors.torch import load_file
    from cosmos_rl_b200.policy import lora
    from cosmos_rl_b200.policy.trainer.sft_trainer import SFTTrainer
    c = _config(tmp_path, "sft")
    c = Config.from_dict({**c.model_dump(), "policy": {**c.policy.model_dump(),
                          "lora": {"r": 4, "lora_alpha": 8, "target_modules": ["q_proj", "v_proj", "down_proj"]}}})
    tr = SFTTrainer(c, ParallelDims(world_size=1, device=torch.device("cpu")), device=torch.device("cpu"))
    tr.model_load_from_hf()
    assert tr.lora_targets == ["layers.0.self_attn.qkv_proj", "layers.0.mlp.down_proj",
                               "layers.1.self_attn.qkv_proj", "layers.1.mlp.down_proj"]
    trainable = [n for n, p in tr.model.named_parameters() if p.requires_grad]
    assert trainable and all(".lora_" in n for n in trainable)
    g = torch.Generator().manual_seed(0)
    ids, cu = torch.randint(0, 32000, (20,), generator=g), torch.tensor([0, 8, 20])
    fwd = lambda: tr.model(ids, tr.model.get_position_ids(cu, 20), cu, 12).detach()
    with lora.adapters_disabled(tr.model):
        base_out = fwd()
    assert torch.equal(fwd(), base_out)                                  # B = 0: the adapted model is the base model
    base_w = {n: p.detach().clone() for n, p in tr.model.named_parameters() if ".lora_" not in n}
    batch = [{"input_ids": torch.randint(0, 32000, (n,), generator=g).tolist()} for n in (12, 20, 7, 16)]
    losses = [tr.step_training(batch, total_steps=10, train_step=i + 1)["train/loss_avg"] for i in range(5)]
    assert losses[-1] < losses[0]
    for n, p in tr.model.named_parameters():
        if ".lora_" not in n:
            assert torch.equal(p, base_w[n]), n                          # the base never moves
    qkv = tr.model.layers[0].self_attn.qkv_proj
    a = tr.model.args
    k_rows = slice(a.n_heads * a.head_dim, (a.n_heads + a.n_kv_heads) * a.head_dim)
    assert qkv.lora_B.abs().sum() > 0 and (qkv.weight._lora.delta()[k_rows] == 0).all()   # k_proj was not targeted
    out = fwd()
    assert not torch.allclose(out, base_out, atol=1e-4)
    tr.before_weight_sync()                                              # merged: dense weights carry the adapters
    assert not torch.equal(qkv.weight, base_w["layers.0.self_attn.qkv_proj.weight"])
    assert torch.allclose(fwd(), out, atol=1e-4)
    tr.after_weight_sync()
    assert torch.allclose(qkv.weight, base_w["layers.0.self_attn.qkv_proj.weight"], atol=1e-6)
    tr.export_safetensors(str(tmp_path / "adapter"))
    sd = load_file(os.path.join(str(tmp_path / "adapter"), "adapter_model.safetensors"))
    q = "base_model.model.model.layers.0.self_attn.q_proj.lora_B.weight"
    assert q in sd and sd[q].shape == (a.n_heads * a.head_dim, 4)
    assert "base_model.model.model.layers.0.self_attn.v_proj.lora_A.weight" in sd
    assert not any("k_proj" in k or "gate_proj" in k for k in sd) and any("down_proj" in k for k in sd)


def test_fp8_training_linear_and_trainer_flag(tmp_path):
    """train.fp8: forward, input gradient and weight gradient of the projections go through block-scaled fp8 GEMMs
    (checked here against the exact products; the GPU kernels are checked against the same reference)."""
    import torch
    from cosmos_rl_b200.ops import functional as F
    from cosmos_rl_b200.policy.trainer.sft_trainer import SFTTrainer
    torch.manual_seed(0)
    x = torch.randn(48, 256, requires_grad=True)
    w = (torch.randn(128, 256) * 0.05).requires_grad_(True)
    w._fp8_train = True
    go = torch.randn(48, 128)
    y = F.linear_maybe_fp8(x, w)
    y.backward(go)
    xr, wr = x.detach().clone().requires_grad_(True), w.detach().clone().requires_grad_(True)
    yr = xr @ wr.t()
    yr.backward(go)
    rel = lambda a, b: ((a.float() - b).norm() / b.norm()).item()
    assert rel(y.detach(), yr.detach()) < 0.05 and rel(x.grad, xr.grad) < 0.05 and rel(w.grad, wr.grad) < 0.05
    assert rel(y.detach(), yr.detach()) > 1e-4                    # it really went through the 8-bit path
    # ragged token count: the weight gradient falls back to the exact product, the rest stays fp8
    x2 = torch.randn(13, 256, requires_grad=True)
    F.linear_maybe_fp8(x2, w).sum().backward()
    assert x2.grad is not None
    c = _config(tmp_path, "sft")
    c.train.fp8.enable_fp8 = True
    tr = SFTTrainer(c, ParallelDims(world_size=1, device=torch.device("cpu")), device=torch.device("cpu"))
    tr.model_load_from_hf()
    assert tr.n_fp8_weights == 8 and not getattr(tr.model.lm_head_weight, "_fp8_train", False)
    g = torch.Generator().manual_seed(0)
    batch = [{"input_ids": torch.randint(0, 32000, (n,), generator=g).tolist()} for n in (12, 20, 7, 16)]
    losses = [tr.step_training(batch, total_steps=10, train_step=i + 1)["train/loss_avg"] for i in range(4)]
    assert losses[-1] < losses[0] - 0.05, losses


def test_custom_grpo_trainer_hooks(tmp_path):
    """The example custom trainer: registered type, overridden loss and learning-rate hooks are what the step uses."""
    import torch
    from cosmos_rl_b200.dispatcher.data.schema import Rollout
    from cosmos_rl_b200.policy.trainer.base import TrainerRegistry
    from cosmos_rl_b200.tools.custom_example import CustomGRPOTrainer
    assert TrainerRegistry.get_trainer_cls("custom_grpo") is CustomGRPOTrainer
    c = Config.from_dict({
        "policy": {"model_name_or_path": "tiny-qwen2", "model_max_length": 64, "model_gradient_checkpointing": False},
        "custom": {"custom_grpo": {"entropy_bonus": 0.01, "length_penalty": 0.1, "lr_drop_every": 2}},
        "train": {"seed": 0, "optm_lr": 1e-3, "optm_warmup_steps": 0, "output_dir": str(tmp_path),
                  "train_policy": {"type": "grpo", "trainer_type": "custom_grpo", "mini_batch": 2},
                  "ckpt": {"enable_checkpoint": False}}})
    tr = CustomGRPOTrainer(c, ParallelDims(world_size=1, device=torch.device("cpu")), device=torch.device("cpu"))
    tr.model_load_from_hf()
    g = torch.Generator().manual_seed(0)
    ros = [Rollout(prompt=torch.randint(0, 32000, (5,), generator=g).tolist(),
                   completion=torch.randint(0, 32000, (n,), generator=g).tolist(), advantage=a, reward=a)
           for n, a in ((6, 1.0), (9, -1.0), (4, 0.5), (7, -0.5))]
    rep = tr.step_training(ros, 1, 10)
    assert "train/entropy_bonus" in rep and "train/length_penalty" in rep and rep["train/grad_norm"] > 0
    assert tr.lr_scale(0) == 1.0 and tr.lr_scale(2) == 0.5 and tr.lr_scale(5) == 0.25


def test_freeze_and_trainable_patterns(tmp_path):
    """policy.freeze_pattern / trainable_pattern: frozen parameters receive no update at all (no decay either) and
    the gradient norm only counts what is trained."""
    import torch
    from cosmos_rl_b200.policy.trainer.sft_trainer import SFTTrainer
    c = _config(tmp_path, "sft")
    c.policy.freeze_pattern = [r"embed_tokens", r"layers\.0\."]
    c.train.optm_weight_decay = 0.1
    tr = SFTTrainer(c, ParallelDims(world_size=1, device=torch.device("cpu")), device=torch.device("cpu"))
    tr.model_load_from_hf()
    before = {n: p.detach().clone() for n, p in tr.model.named_parameters()}
    g = torch.Generator().manual_seed(0)
    batch = [{"input_ids": torch.randint(0, 32000, (n,), generator=g).tolist()} for n in (12, 20, 7, 16)]
    for i in range(2):
        tr.step_training(batch, total_steps=10, train_step=i + 1)
    moved = {n for n, p in tr.model.named_parameters() if not torch.equal(p, before[n])}
    assert moved and all(not n.startswith("layers.0.") and "embed_tokens" not in n for n in moved)
    assert any(n.startswith("layers.1.") for n in moved) and "norm" in moved
    segs = tr.optimizer.segments
    assert segs and sum(b - a for a, b in segs) == sum(p.numel() for p in tr.model.parameters() if p.requires_grad)


def test_on_policy_distillation_advantages(tmp_path):
    """Teacher log-probs per scored token become advantages: -coef * (student - teacher), discounted over the rest
    of the sequence; samples without a teacher result only keep their own advantage."""
    import torch
    from cosmos_rl_b200.dispatcher.data.schema import Rollout
    from cosmos_rl_b200.policy.trainer.grpo_trainer import GRPOTrainer
    c = Config.from_dict({
        "policy": {"model_name_or_path": "tiny-qwen2", "model_max_length": 64, "model_gradient_checkpointing": False},
        "distillation": {"enable": True, "model_name_or_path": "tiny-qwen2", "kl_penalty_coef": 2.0, "kl_discount_factor": 0.5},
        "train": {"seed": 0, "optm_lr": 1e-3, "optm_warmup_steps": 0, "output_dir": str(tmp_path),
                  "train_policy": {"type": "grpo", "trainer_type": "grpo", "mini_batch": 4},
                  "ckpt": {"enable_checkpoint": False}}})
    tr = GRPOTrainer(c, ParallelDims(world_size=1, device=torch.device("cpu")), device=torch.device("cpu"))
    tr.model_load_from_hf()
    g = torch.Generator().manual_seed(0)
    comp = [torch.randint(0, 32000, (n,), generator=g).tolist() for n in (3, 2)]
    ros = [Rollout(prompt=[5, 6, 7], completion=comp[0], advantage=0.5, reward=1.0,
                   teacher_logprobs=[[-1.0], [-2.0], [-3.0]]),
           Rollout(prompt=[8, 9], completion=comp[1], advantage=-0.5, reward=0.0)]             # no teacher result
    b = tr._pack(tr._prepare(ros))
    t = b["teacher_lp"]
    assert t[:3].tolist() == [-1.0, -2.0, -3.0] and torch.isnan(t[3:]).all()
    lp = torch.tensor([-1.5, -1.0, -3.0, -0.7, -0.9])
    adv, kl = tr.teacher_kl_advantages(lp, b)
    d = [-2.0 * (-1.5 + 1.0), -2.0 * (-1.0 + 2.0), 0.0]                   # -coef * (student - teacher) = [1, -2, 0]
    want = [d[0] + 0.5 * (d[1] + 0.5 * d[2]), d[1] + 0.5 * d[2], d[2]]
    assert torch.allclose(adv[:3], torch.tensor(want) + 0.5) and torch.allclose(adv[3:], torch.tensor([-0.5, -0.5]))
    assert abs(kl.item() - ((-0.5) + 1.0 + 0.0) / 3) < 1e-6
    rep = tr.step_training(ros, 1, 10)
    assert "train/teacher_kl_reversed" in rep and rep["train/grad_norm"] > 0


@pytest.mark.parametrize("beta", [0.0, 0.5, 1.0])
def test_topk_jsd_distillation_advantages(tmp_path, beta):
    """``distillation.top_k``: the teacher engine returns its k best tokens per completion token; the trainer scores
    the student on the same ids and subtracts the generalised JSD (forward KL at beta 0, reverse KL at beta 1) from
    the advantages. Checked against torch.nn.functional.kl_div on the same top-k slices."""
    import torch
    import torch.nn.functional as tF
    from cosmos_rl_b200.dispatcher.data.schema import Rollout
    from cosmos_rl_b200.policy.trainer.grpo_trainer import GRPOTrainer
    from cosmos_rl_b200.reference.teacher_worker import TeacherEngine
    k = 4
    c = Config.from_dict({
        "policy": {"model_name_or_path": "tiny-qwen2", "model_max_length": 64, "model_gradient_checkpointing": False},
        "distillation": {"enable": True, "model_name_or_path": "tiny-qwen2", "kl_penalty_coef": 1.5, "top_k": k,
                         "jsd_beta": beta, "seed": 7},
        "train": {"seed": 0, "optm_lr": 1e-3, "optm_warmup_steps": 0, "output_dir": str(tmp_path),
                  "train_policy": {"type": "grpo", "trainer_type": "grpo", "mini_batch": 4},
                  "ckpt": {"enable_checkpoint": False}}})
    dims = ParallelDims(world_size=1, device=torch.device("cpu"))
    tr = GRPOTrainer(c, dims, device=torch.device("cpu"))
    tr.model_load_from_hf()
    teacher = TeacherEngine(c, torch.device("cpu"), dims)
    g = torch.Generator().manual_seed(0)
    prompts = [[5, 6, 7], [8, 9]]
    comp = [torch.randint(0, 32000, (n,), generator=g).tolist() for n in (3, 2)]
    res = teacher.score([p + c_ for p, c_ in zip(prompts, comp)], [len(p) for p in prompts])
    assert len(res[0]["topk_ids"]) == 3 and len(res[0]["topk_ids"][0]) == k
    ros = [Rollout(prompt=prompts[0], completion=comp[0], advantage=0.5, reward=1.0,
                   teacher_logprobs=[[v] for v in res[0]["logprobs"]], teacher_topk_ids=res[0]["topk_ids"],
                   teacher_topk_logprobs=res[0]["topk_logprobs"]),
           Rollout(prompt=prompts[1], completion=comp[1], advantage=-0.5, reward=0.0)]        # no teacher result
    b = tr._pack(tr._prepare(ros))
    assert b["teacher_topk_ids"].shape == (5, k) and (b["teacher_topk_ids"][3:] == -1).all()
    with torch.no_grad():
        hidden = tr.model(b["input_ids"], b["position_ids"], b["cu_seqlens"], b["max_seqlen"])
        tr.compute_logprobs(hidden, b)
        full = torch.log_softmax(tr.model.logits(hidden[b["sel"]]).float(), -1)
    s = full.gather(1, b["teacher_topk_ids"].clamp_min(0))
    assert torch.allclose(b["student_topk_lp"], s, atol=1e-5)
    t = b["teacher_topk_lp"]
    if beta == 0.0:
        want = tF.kl_div(s, t, reduction="none", log_target=True)
    elif beta == 1.0:
        want = tF.kl_div(t, s, reduction="none", log_target=True)
    else:
        m = torch.logsumexp(torch.stack([s + math.log(1 - beta), t + math.log(beta)]), 0)
        want = beta * tF.kl_div(m, t, reduction="none", log_target=True) + \
            (1 - beta) * tF.kl_div(m, s, reduction="none", log_target=True)
    want = want.sum(-1)
    adv, div = tr.teacher_topk_jsd_advantages(b)
    assert torch.allclose(adv[:3], 0.5 - 1.5 * want[:3], atol=1e-5) and torch.allclose(adv[3:], torch.tensor([-0.5, -0.5]))
    assert abs(div.item() - want[:3].mean().item()) < 1e-5     # truncated to k tokens the sum may be negative
    rep = tr.step_training(ros, 1, 10)
    assert f"train/teacher_jsd_top{k}" in rep and rep["train/grad_norm"] > 0


def test_ema_tracks_weights_on_the_optimizer_shard_and_is_exported(tmp_path):
    """``train.ema_enable``: after every optimizer step the average moves towards the fp32 master weights with the
    warm-up decay; exports read the averaged weights and leave the trained ones in place; checkpoints carry it."""
    import torch
    from cosmos_rl_b200.policy.trainer.sft_trainer import SFTTrainer
    c = _config(tmp_path, "sft")
    c.train.ema_enable, c.train.ema_decay, c.train.ema_update_step_interval = True, 0.9, 1
    c.train.ckpt.enable_checkpoint = True
    dims = ParallelDims(world_size=1, device=torch.device("cpu"))
    tr = SFTTrainer(c, dims, device=torch.device("cpu"))
    tr.model_load_from_hf()
    assert tr.ema is not None and torch.equal(tr.ema.shard, tr.optimizer.master)
    g = torch.Generator().manual_seed(0)
    batch = [{"input_ids": torch.randint(0, 32000, (12,), generator=g).tolist()} for _ in range(4)]
    want = tr.optimizer.master.clone()
    for step in range(3):
        tr.step_training(batch, 10, step + 1)
        d = min((1 + step) / (10 + step), 0.9)
        want = d * want + (1 - d) * tr.optimizer.master
    assert torch.allclose(tr.ema.shard, want, atol=1e-6)
    assert not torch.allclose(tr.ema.shard, tr.optimizer.master)
    live = tr.flat.data.clone()
    with tr.ema.swapped_in():
        assert torch.allclose(tr.flat.data.float(), tr.ema.shard, atol=1e-6)
    assert torch.equal(tr.flat.data, live)
    tr.save_checkpoint(3, 10)
    tr.ckpt_manager.finalize()
    c.train.resume = True
    tr2 = SFTTrainer(c, dims, device=torch.device("cpu"))
    assert tr2.weight_resume() and torch.equal(tr2.ema.shard, tr.ema.shard) and tr2.ema.updates == 3
    assert any(n == "ema.shard" for n, _ in tr2.state_tensors())


def test_8bit_optimizer_moments_track_the_fp32_optimizer(tmp_path):
    """``optm_name = "AdamW8bit"``: moments in int8 / uint8 blocks of 256 with fp32 scales. After several steps on the
    same gradients the weights stay close to the fp32 optimizer's, the state is a quarter of the size, frozen
    stretches and unaligned segment edges are handled, and the state survives a save / load round trip."""
    import torch
    from cosmos_rl_b200.models.gpt import GPT, GPTArgs
    from cosmos_rl_b200.parallel.flat import FlatParams
    from cosmos_rl_b200.policy.optim import FlatAdamW

    def make(bits, freeze):
        m = GPT(GPTArgs(vocab_size=512, dim=64, n_layers=2, n_heads=4, n_kv_heads=2, ffn_dim=160))
        if freeze:
            for n, p in m.named_parameters():
                if n.startswith("layers.0."):
                    p.requires_grad_(False)
        flat = FlatParams(m, torch.float32, torch.device("cpu"))
        m.init_weights(0)
        return flat, FlatAdamW(flat, lr=1e-2, weight_decay=0.1, max_grad_norm=1e9, state_bits=bits)

    for freeze in (False, True):
        (f32, o32), (f8, o8) = make(32, freeze), make(8, freeze)
        w0 = f32.data.clone()
        for step in range(6):
            g = torch.Generator().manual_seed(step)
            grad = torch.randn(f32.total, generator=g) * torch.logspace(-4, 0, f32.total)     # wide dynamic range
            f32.grad.copy_(grad)
            f8.grad.copy_(grad)
            o32.step()
            o8.step()
        moved = (f32.data - w0).abs()
        err = (f8.data - f32.data).abs()
        assert moved.max() > 0.03 and err.max() < 0.3 * moved.max() and err.mean() < 0.05 * moved.mean()
        if freeze:
            assert torch.equal(f8.data[moved == 0], w0[moved == 0]) and (moved == 0).sum() > 1000
    bytes8 = sum(t.numel() * t.element_size() for _, t in o8.m8.tensors("m") + o8.v8.tensors("v"))
    assert bytes8 < 0.27 * (o32.m.numel() + o32.v.numel()) * 4
    sd = o8.state_dict()
    _, o8b = make(8, True)
    o8b.load_state_dict(sd)
    assert torch.equal(o8b.m8.q, o8.m8.q) and torch.equal(o8b.v8.scale, o8.v8.scale) and o8b.step_count == 6
    assert [n for n, _ in o8.state_tensors()] == ["optim.master", "optim.m.q", "optim.m.scale", "optim.v.q", "optim.v.scale"]


def test_sft_trainer_with_8bit_adam(tmp_path):
    import torch
    from cosmos_rl_b200.policy.trainer.sft_trainer import SFTTrainer
    c = _config(tmp_path, "sft")
    c.train.optm_name = "AdamW8bit"
    tr = SFTTrainer(c, ParallelDims(world_size=1, device=torch.device("cpu")), device=torch.device("cpu"))
    tr.model_load_from_hf()
    assert tr.optimizer.state_bits == 8 and tr.optimizer.m is None
    g = torch.Generator().manual_seed(0)
    batch = [{"input_ids": torch.randint(0, 32000, (12,), generator=g).tolist()} for _ in range(4)]
    losses = [tr.step_training(batch, 10, i + 1)["train/loss_avg"] for i in range(5)]
    assert losses[-1] < losses[0] - 0.5


def test_force_use_hf_and_lora_init_modes(tmp_path):
    """``train.force_use_hf`` trains the generic transformers wrapper although a native model exists for the type;
    ``policy.lora.init_lora_weights`` picks the adapter initialisation."""
    import torch
    from cosmos_rl_b200.models.hf_model import HFModel
    from cosmos_rl_b200.policy.trainer.sft_trainer import SFTTrainer
    dims = ParallelDims(world_size=1, device=torch.device("cpu"))
    c = _config(tmp_path, "sft")
    c.train.force_use_hf = True
    tr = SFTTrainer(c, dims, device=torch.device("cpu"))
    tr.model_load_from_hf()
    assert isinstance(tr.model, HFModel)
    g = torch.Generator().manual_seed(0)
    batch = [{"input_ids": torch.randint(0, 32000, (12,), generator=g).tolist()} for _ in range(4)]
    assert tr.step_training(batch, 10, 1)["train/grad_norm"] > 0
    for init, b_zero in ((True, True), ("gaussian", True), (False, False)):
        c = _config(tmp_path, "sft")
        c.policy.lora = type(c.policy).model_fields["lora"].annotation.__args__[0](r=4, lora_alpha=8, init_lora_weights=init, target_modules=["q_proj", "v_proj"])
        tr = SFTTrainer(c, dims, device=torch.device("cpu"))
        tr.model_load_from_hf()
        bs = [p for n, p in tr.model.named_parameters() if n.endswith("lora_B")]
        assert bs and all((p.abs().sum() == 0) == b_zero for p in bs)


def test_reference_weights_survive_checkpoint_resume_and_optimizer_reset(tmp_path):
    """The KL anchor is run state: a resume restores the weights the run started from (not the resumed policy), a
    new replica receives it with the rest of the state, and a reference reset with 8-bit moments clears them."""
    from cosmos_rl_b200.colocated import ColocatedGRPO

    def cfg(resume, optm="AdamW"):
        return Config.from_dict({
            "mode": "colocated",
            "policy": {"model_name_or_path": "tiny-qwen2", "model_max_length": 96, "model_gradient_checkpointing": False},
            "rollout": {"n_generation": 4, "batch_size": 2, "max_response_length": 16, "seed": 3},
            "train": {"seed": 0, "optm_lr": 1e-2, "optm_warmup_steps": 0, "output_dir": str(tmp_path), "resume": resume,
                      "optm_name": optm,
                      "train_policy": {"type": "grpo", "reward_function": ["even_token_fraction"], "mini_batch": 4,
                                       "kl_beta": 0.05, "reset_optimizer_with_reference": True},
                      "ckpt": {"enable_checkpoint": True, "save_mode": "sync"}}})

    job = ColocatedGRPO(cfg(False), device=torch.device("cpu"), max_num_seqs=8)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 32000, (10,), generator=g) for _ in range(2)]
    w_init = job.trainer.flat.data.clone()
    job.step(prompts)
    job.step(prompts)
    tr = job.trainer
    assert torch.equal(tr.reference_state, w_init) and not torch.equal(tr.flat.data, w_init)
    tr.save_checkpoint(2, 10)
    # a state hand-over to a new replica carries the anchor
    names = dict(tr.state_tensors())
    assert torch.equal(names["reference"].cpu(), w_init)

    job2 = ColocatedGRPO(cfg(True), device=torch.device("cpu"), max_num_seqs=8)
    tr2 = job2.trainer
    assert tr2.train_step == 2 and torch.equal(tr2.flat.data, tr.flat.data)
    assert torch.equal(tr2.reference_state, w_init)                  # anchored to the original model, not the resumed one
    # reference log-probs of the resumed run equal those of the uninterrupted one
    samples = tr._prepare(job.rollout(prompts))
    b = tr._pack(samples[:4])
    lp1 = tr._reference_logprobs([b])[0]
    lp2 = tr2._reference_logprobs([tr2._pack(tr2._prepare(job.rollout(prompts))[:4])])[0]
    assert lp1.shape == lp2.shape
    b2 = tr2._pack(samples[:4])
    assert torch.allclose(tr2._reference_logprobs([b2])[0], lp1, atol=1e-6)

    # reference reset clears the moments in every representation
    job8 = ColocatedGRPO(cfg(False, "AdamW8bit"), device=torch.device("cpu"), max_num_seqs=8)
    job8.step(prompts)
    opt = job8.trainer.optimizer
    assert opt.m is None and opt.m8.q.abs().sum() > 0
    job8.trainer.reference_reset()
    assert opt.m8.q.abs().sum() == 0 and opt.v8.scale.abs().sum() == 0
    assert torch.equal(job8.trainer.reference_state, job8.trainer.flat.data.cpu())


def test_grpo_loss_masking_kl_and_divisor_follow_the_reference_rules():
    """Off-policy sequence masking drops the surrogate of a masked sequence but keeps its KL penalty and its tokens in
    the denominator; the unbiased KL estimate differentiates through the importance weight and clamps the product;
    a non-positive ``unbiased_loss_max_tokens`` means "divide by the sequence length"."""
    lp = torch.tensor([-1.0, -2.0, -0.5, -1.5], requires_grad=True)
    old = torch.tensor([-1.0, -2.0, -3.0, -4.0])         # sequence 1 drifted: mean(old - lp) = -2.5 ... use rollout lp
    roll = torch.tensor([-1.0, -2.0, 1.5, 0.5])          # behaviour - current = +2.0 on sequence 1
    ref = torch.tensor([-1.2, -1.8, -0.7, -1.0])
    A = torch.tensor([1.0, 1.0, -1.0, -1.0])
    seq = torch.tensor([0, 0, 1, 1])
    cfg = L.GrpoLossConfig(kl_beta=0.5, off_policy_masking_delta=1.0)
    loss, m = L.grpo_loss(lp, old, A, seq, 2, cfg, ref_logprob=ref, rollout_logprob=roll)
    r = ref - lp.detach()
    kl = torch.exp(r) - r - 1.0
    ratio = torch.exp((lp.detach() - old).clamp(-20, 20))
    pg = -torch.minimum(ratio * A, ratio.clamp(0.8, 1.2) * A)
    pg[2:] = 0.0                                          # sequence 1 is masked: surrogate gone ...
    want = (pg + 0.5 * kl).sum() / 4                      # ... its KL and its two tokens stay
    assert abs(loss.item() - want.item()) < 1e-5, (loss.item(), want.item())
    assert abs(m["kl"].item() - kl.mean().item()) < 1e-6
    # unbiased KL: d/dlp of w * k3 with w = exp(lp - old) differentiable
    cfg_u = L.GrpoLossConfig(kl_beta=1.0, unbiased_kl_estimate=True, epsilon_low=1e9, epsilon_high=1e9)
    lp2 = torch.tensor([-1.0, -2.0], requires_grad=True)
    old2 = torch.tensor([-1.1, -1.9])
    ref2 = torch.tensor([-1.3, -1.6])
    loss2, _ = L.grpo_loss(lp2, old2, torch.zeros(2), torch.tensor([0, 0]), 1, cfg_u, ref_logprob=ref2)
    loss2.backward()
    w = torch.exp(lp2.detach() - old2)
    r2 = ref2 - lp2.detach()
    g = (w * (torch.exp(r2) - r2 - 1.0) + w * (-(torch.exp(r2) - 1.0))) / 2
    assert torch.allclose(lp2.grad, g, atol=1e-6)
    # Dr.GRPO divisor: 0 falls back to the sequence length
    c0 = L.GrpoLossConfig(loss_type="seq-mean-token-mean", unbiased_loss_max_tokens=0)
    c1 = L.GrpoLossConfig(loss_type="seq-mean-token-mean")
    l0, _ = L.grpo_loss(lp.detach(), old, A, seq, 2, c0)
    l1, _ = L.grpo_loss(lp.detach(), old, A, seq, 2, c1)
    assert math.isfinite(l0.item()) and abs(l0.item() - l1.item()) < 1e-7


def test_dpo_on_vision_language_preference_pairs(tmp_path):
    """Multimodal preference data (an image prompt with a chosen and a rejected answer): the data packer returns the
    prompt's pixel inputs with the tokens, both completions of a pair are scored against the same image, the loss
    starts at ln 2 and falls, and the gradient reaches the vision tower."""
    from cosmos_rl_b200.data.packer import HFVLMDataPacker
    from cosmos_rl_b200.policy.trainer.dpo_trainer import DPOTrainer
    cfg = _config(tmp_path, "dpo")
    cfg.policy.model_name_or_path = "tiny-internvl"
    packer = HFVLMDataPacker()
    packer.setup(cfg, None)
    cpu = torch.device("cpu")
    tr = DPOTrainer(cfg, ParallelDims(world_size=1, device=cpu), device=cpu, data_packer=packer)
    tr.model_load_from_hf()
    assert type(tr.model).__name__ == "InternVL"
    g = torch.Generator().manual_seed(3)
    tok = lambda n: torch.randint(0, 31000, (n,), generator=g).tolist()               # noqa: E731
    batch = []
    for _ in range(4):
        prompt = {"input_ids": tok(3) + [31990] * 4 + tok(3), "pixel_values": torch.randn(1, 3, 56, 56, generator=g)}
        batch.append({"prompt": prompt, "chosen": tok(5), "rejected": tok(6)})
    r0 = tr.step_training(batch, total_steps=10, train_step=1)
    assert abs(r0["train/loss_avg"] - math.log(2.0)) < 1e-4
    vis = [s for s in tr.flat.slots if s.name.startswith("visual.patch_embed.weight")][0]
    assert tr.optimizer.m[vis.offset: vis.offset + vis.numel].abs().sum() > 0        # the tower is trained
    for i in range(2, 6):
        r = tr.step_training(batch, total_steps=10, train_step=i)
    assert r["train/loss_avg"] < r0["train/loss_avg"] - 0.01 and r["train/reward_acc"] >= 0.75
    # another image changes the preference margin of the same token sequences
    enc = [tr._encode(s) for s in batch[:1]]
    with torch.no_grad():
        a = tr._seq_logprobs(enc)
        other = dict(batch[0], prompt=dict(batch[0]["prompt"], pixel_values=torch.randn(1, 3, 56, 56, generator=g) * 3))
        b = tr._seq_logprobs([tr._encode(other)])
    assert (a - b).abs().max() > 1e-5
