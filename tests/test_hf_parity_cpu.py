"""Native models against the transformers implementations of the same architectures: a tiny random HF model is
saved as safetensors, loaded through the framework's weight mapper, and the logits of a packed batch are compared
with the HF model run per sequence. This covers the parameter mapping (fused qkv / gate_up, stacked experts), RoPE
conventions, norms, routing and the packed-sequence attention."""
import pytest
import torch

from cosmos_rl_b200.models import hf_io
from cosmos_rl_b200.models.base import ModelRegistry

transformers = pytest.importorskip("transformers")


def _native_from(path):
    cfg = hf_io.load_hf_config(path)
    model = ModelRegistry.build_model(cfg)
    hf_io.load_hf_weights(model, path)
    return model.eval()


def _compare(hf, native, vocab, atol):
    g = torch.Generator().manual_seed(3)
    seqs = [torch.randint(0, vocab, (n,), generator=g) for n in (11, 5, 17)]
    ids = torch.cat(seqs)
    cu = torch.tensor([0, 11, 16, 33])
    with torch.no_grad():
        h = native(ids, native.get_position_ids(cu, 33), cu, 17)
        logits = (h @ native.lm_head_weight.t()).float()
        want = torch.cat([hf(s[None]).logits[0] for s in seqs]).float()
    err = (logits - want).abs().max().item()
    assert err < atol, err
    assert (logits.argmax(-1) == want.argmax(-1)).float().mean() > 0.98


CASES = {
    "qwen2": lambda t: t.Qwen2ForCausalLM(t.Qwen2Config(
        vocab_size=512, hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
        intermediate_size=128, max_position_embeddings=128, rope_theta=50000.0, tie_word_embeddings=False)),
    "qwen2-tied": lambda t: t.Qwen2ForCausalLM(t.Qwen2Config(
        vocab_size=512, hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=4,
        intermediate_size=128, max_position_embeddings=128, tie_word_embeddings=True)),
    "llama": lambda t: t.LlamaForCausalLM(t.LlamaConfig(
        vocab_size=512, hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
        intermediate_size=96, max_position_embeddings=128, rope_theta=500000.0)),
    "qwen3": lambda t: t.Qwen3ForCausalLM(t.Qwen3Config(
        vocab_size=512, hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=32,
        intermediate_size=128, max_position_embeddings=128, tie_word_embeddings=False)),
    "qwen3_moe": lambda t: t.Qwen3MoeForCausalLM(t.Qwen3MoeConfig(
        vocab_size=512, hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
        intermediate_size=128, moe_intermediate_size=32, num_experts=4, num_experts_per_tok=2,
        max_position_embeddings=128, norm_topk_prob=True)),
    "deepseek_v3": lambda t: t.DeepseekV3ForCausalLM(t.DeepseekV3Config(
        vocab_size=512, hidden_size=64, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=4,
        intermediate_size=128, moe_intermediate_size=32, n_routed_experts=8, n_shared_experts=1, num_experts_per_tok=3,
        n_group=4, topk_group=2, first_k_dense_replace=1, q_lora_rank=24, kv_lora_rank=16, qk_nope_head_dim=16,
        qk_rope_head_dim=8, v_head_dim=16, max_position_embeddings=128)),
    "deepseek_v3-yarn-noqlora": lambda t: t.DeepseekV3ForCausalLM(t.DeepseekV3Config(
        vocab_size=512, hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=4,
        intermediate_size=128, moe_intermediate_size=32, n_routed_experts=4, n_shared_experts=2, num_experts_per_tok=2,
        n_group=1, topk_group=1, first_k_dense_replace=1, q_lora_rank=None, kv_lora_rank=16, qk_nope_head_dim=16,
        qk_rope_head_dim=8, v_head_dim=24, max_position_embeddings=128, norm_topk_prob=False, rope_interleave=False,
        rope_parameters={"rope_type": "yarn", "rope_theta": 10000.0, "factor": 8.0, "beta_fast": 32.0, "beta_slow": 1.0,
                         "mscale": 1.0, "mscale_all_dim": 0.7, "original_max_position_embeddings": 16})),
}


@pytest.mark.parametrize("family", sorted(CASES))
def test_native_model_matches_transformers(family, tmp_path):
    torch.manual_seed(0)
    hf = CASES[family](transformers).eval()
    with torch.no_grad():                      # HF initialises norms to one and biases to zero: make them matter
        for n, p in hf.named_parameters():
            if "norm" in n or n.endswith(".bias") or n.endswith("e_score_correction_bias"):
                p.add_(0.1 * torch.randn_like(p))
    hf.save_pretrained(str(tmp_path))
    native = _native_from(str(tmp_path))
    _compare(hf, native, 512, 2e-4)
