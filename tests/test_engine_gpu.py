"""GPU tests of the rollout engine: CUDA-graph decode against teacher forcing, shared-prefix decode option."""
import pytest
import torch

from cosmos_rl_b200.models.gpt import GPT, GPTArgs
from cosmos_rl_b200.ops import native
from cosmos_rl_b200.parallel.flat import FlatParams
from cosmos_rl_b200.rollout.engine import RolloutEngine, SamplingParams

pytestmark = pytest.mark.gpu


def _model():
    a = GPTArgs(vocab_size=4096, dim=512, n_layers=2, n_heads=4, n_kv_heads=2, head_dim=128, ffn_dim=1024,
                qkv_bias=True, model_type="qwen2")
    with torch.device("meta"):
        m = GPT(a)
    FlatParams(m, torch.bfloat16, torch.device("cuda"), with_grad=False)
    m.init_weights_on_device(3)
    return m


@pytest.mark.parametrize("shared_prefix", [False, True])
def test_engine_logprobs_match_teacher_forcing(shared_prefix):
    m = _model()
    eng = RolloutEngine(m, max_num_seqs=16, max_model_len=1024, page_size=128, shared_prefix_decode=shared_prefix)
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, 4096, (n,), generator=g).tolist() for n in (300, 130, 517, 64)]
    out = eng.generate(prompts, SamplingParams(n=4, max_tokens=40, temperature=1.0, seed=11))
    assert native.read_status(torch.device("cuda")) == 0
    assert len(eng.free_pages) == eng.num_pages - 1
    n_tok = 0
    for p, comps in zip(prompts, out):
        assert len({tuple(c.token_ids) for c in comps}) > 1            # sampled, not identical
        for c in comps:
            ids = torch.tensor(p + c.token_ids, device="cuda")
            cu = torch.tensor([0, ids.numel()], dtype=torch.int32, device="cuda")
            with torch.no_grad():
                h = m(ids, torch.arange(ids.numel(), device="cuda"), cu, int(ids.numel()))
                lsm = torch.log_softmax(m.logits(h).float(), -1)
            for i, (tok, lp) in enumerate(zip(c.token_ids, c.logprobs)):
                assert abs(lsm[len(p) - 1 + i, tok].item() - lp) < 0.08, (i, lsm[len(p) - 1 + i, tok].item(), lp)
                n_tok += 1
    assert n_tok == 4 * 4 * 40


@pytest.mark.parametrize("arch", ["tiny-qwen3-moe", "tiny-qwen2-d128"])
def test_colocated_grpo_step_on_gpu(arch, tmp_path):
    """One full GRPO step (generate, score, train, publish) of a tiny dense and a tiny MoE model on the GPU."""
    import math
    from cosmos_rl_b200.colocated import ColocatedGRPO
    from cosmos_rl_b200.config import Config
    cfg = Config.from_dict({
        "mode": "colocated",
        "policy": {"model_name_or_path": arch, "model_max_length": 192, "parallelism": {"tp_size": 1}},
        "rollout": {"n_generation": 4, "batch_size": 4, "max_response_length": 32, "parallelism": {"tp_size": 1}},
        "train": {"seed": 0, "optm_lr": 1e-4, "output_dir": str(tmp_path),
                  "train_policy": {"type": "grpo", "reward_function": ["even_token_fraction"], "mini_batch": 8,
                                   "kl_beta": 0.01}}})
    job = ColocatedGRPO(cfg, device=torch.device("cuda", 0), max_num_seqs=16)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 32000, (48,), generator=g) for _ in range(4)]
    w0 = job.trainer.flat.data.clone()
    for _ in range(2):
        rep = job.step(prompts)
    torch.cuda.synchronize()
    assert native.read_status(torch.device("cuda", 0)) == 0
    assert math.isfinite(rep["train/loss_avg"]) and math.isfinite(rep["train/grad_norm"]) and rep["train/grad_norm"] > 0
    assert not torch.equal(job.trainer.flat.data, w0)
    assert 0.0 <= rep["rollout/reward_mean"] <= 1.0
