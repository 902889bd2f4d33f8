"""SD3-style multimodal diffusion transformer: the packed two-stream implementation against a per-sample restatement
written with plain torch ops on the exported checkpoint, its invariances, and training through the diffusion trainer."""
import math

import torch

from cosmos_rl_b200.config import Config
from cosmos_rl_b200.models import hf_io
from cosmos_rl_b200.models.base import ModelRegistry
from cosmos_rl_b200.models.mmdit import ARCHS, MMDiT, sincos_2d, timestep_sinusoid
from cosmos_rl_b200.parallel.dims import ParallelDims


def _plain_forward(sd, a, z, t, text, lens):
    """One sample at a time, no packing: the published block equations on the checkpoint tensors."""
    lin = lambda x, n: torch.nn.functional.linear(x, sd[n + ".weight"], sd[n + ".bias"])        # noqa: E731
    ln = lambda x: torch.nn.functional.layer_norm(x, (x.shape[-1],), eps=1e-6)                   # noqa: E731
    silu, D, h, d, p = torch.nn.functional.silu, a.dim, a.num_attention_heads, a.attention_head_dim, a.patch_size
    outs = []
    for b in range(z.shape[0]):
        C, H, W = z[b].shape
        gh, gw = H // p, W // p
        conv = torch.nn.functional.conv2d(z[b:b + 1], sd["pos_embed.proj.weight"], sd["pos_embed.proj.bias"], stride=p)
        x = conv.flatten(2).transpose(1, 2)[0]                                             # [n, D]
        m = a.pos_embed_max_size
        table = sincos_2d(D, m, a.sample_size // p, z.device).view(m, m, D)
        top, left = (m - gh) // 2, (m - gw) // 2
        x = x + table[top:top + gh, left:left + gw].reshape(-1, D)
        temb = lin(silu(lin(timestep_sinusoid(t[b:b + 1] * 1000.0), "time_text_embed.timestep_embedder.linear_1")),
                   "time_text_embed.timestep_embedder.linear_2")
        pooled = text[b, 0, :a.pooled_projection_dim][None]
        pemb = lin(silu(lin(pooled, "time_text_embed.text_embedder.linear_1")), "time_text_embed.text_embedder.linear_2")
        emb = silu(temb + pemb)[0]
        c = lin(text[b, 1:1 + lens[b]], "context_embedder")
        for i in range(a.num_layers):
            pre = f"transformer_blocks.{i}."
            last = i == a.num_layers - 1
            sh_a, sc_a, g_a, sh_m, sc_m, g_m = lin(emb, pre + "norm1.linear").chunk(6)
            xn = ln(x) * (1 + sc_a) + sh_a
            if last:
                csc, csh = lin(emb, pre + "norm1_context.linear").chunk(2)
                cn = ln(c) * (1 + csc) + csh
            else:
                csh_a, csc_a, cg_a, csh_m, csc_m, cg_m = lin(emb, pre + "norm1_context.linear").chunk(6)
                cn = ln(c) * (1 + csc_a) + csh_a
            heads = lambda y: y.view(-1, h, d).transpose(0, 1)                                # noqa: E731
            q = torch.cat([heads(lin(xn, pre + "attn.to_q")), heads(lin(cn, pre + "attn.add_q_proj"))], dim=1)
            k = torch.cat([heads(lin(xn, pre + "attn.to_k")), heads(lin(cn, pre + "attn.add_k_proj"))], dim=1)
            v = torch.cat([heads(lin(xn, pre + "attn.to_v")), heads(lin(cn, pre + "attn.add_v_proj"))], dim=1)
            o = torch.softmax(q @ k.transpose(1, 2) / math.sqrt(d), dim=-1) @ v
            o = o.transpose(0, 1).reshape(-1, D)
            n = x.shape[0]
            x = x + g_a * lin(o[:n], pre + "attn.to_out.0")
            y = ln(x) * (1 + sc_m) + sh_m
            x = x + g_m * lin(torch.nn.functional.gelu(lin(y, pre + "ff.net.0.proj"), approximate="tanh"), pre + "ff.net.2")
            if not last:
                c = c + cg_a * lin(o[n:], pre + "attn.to_add_out")
                y = ln(c) * (1 + csc_m) + csh_m
                c = c + cg_m * lin(torch.nn.functional.gelu(lin(y, pre + "ff_context.net.0.proj"), approximate="tanh"),
                                   pre + "ff_context.net.2")
        sc, sh = lin(emb, "norm_out.linear").chunk(2)
        out = lin(ln(x) * (1 + sc) + sh, "proj_out")                                          # [n, p*p*C]
        oc = a.out_channels
        outs.append(out.view(gh, gw, p, p, oc).permute(4, 0, 2, 1, 3).reshape(oc, H, W))
    return torch.stack(outs)


def test_mmdit_matches_the_per_sample_equations_and_uses_published_names():
    torch.manual_seed(0)
    a = ARCHS["tiny-mmdit"]
    assert ModelRegistry.get("mmdit") is MMDiT
    m = MMDiT(a).float()
    m.init_weights(0)
    with torch.no_grad():
        for n, p in m.named_parameters():                      # zero-initialised layers off zero, biases off zero
            p.add_(0.05 * torch.randn_like(p))
    z0 = torch.randn(2, 4, 8, 8)
    sd = hf_io.hf_state_dict(m, a.to_hf_config())
    assert sd["pos_embed.proj.weight"].shape == (128, 4, 2, 2)
    for k in ("transformer_blocks.0.attn.add_q_proj.weight", "transformer_blocks.0.attn.to_out.0.bias",
              "transformer_blocks.1.ff_context.net.0.proj.weight", "transformer_blocks.2.norm1_context.linear.weight",
              "time_text_embed.text_embedder.linear_2.bias", "context_embedder.weight", "norm_out.linear.weight"):
        assert k in sd, k
    assert "transformer_blocks.2.attn.to_add_out.weight" not in sd and "transformer_blocks.2.ff_context.net.2.weight" not in sd
    assert sd["transformer_blocks.2.norm1_context.linear.weight"].shape[0] == 2 * 128        # the last block only reads text
    t = torch.tensor([0.3, 0.9])
    text = torch.randn(2, 1 + 5, 64)
    mask = torch.tensor([[1, 1, 1, 1, 1, 1], [1, 1, 1, 0, 0, 0]], dtype=torch.bool)
    with torch.no_grad():
        mine = m(z0, t, text, mask)
        ref = _plain_forward(sd, a, z0, t, text, [5, 2])
    assert mine.shape == z0.shape and (mine - ref).abs().max().item() < 2e-4, (mine - ref).abs().max()
    with torch.no_grad():
        text2 = text.clone()
        text2[1, 3:] = 7.0                                      # padding rows do not matter
        assert torch.allclose(m(z0, t, text2, mask), mine, atol=1e-6)
        assert torch.allclose(m(z0.unsqueeze(2), t, text, mask).squeeze(2), mine, atol=1e-6)   # single-frame video layout
    m2 = MMDiT(a).float()
    hf_io.load_hf_state(m2, lambda k: sd[k], sd, a.to_hf_config())
    with torch.no_grad():
        assert torch.allclose(m2(z0, t, text, mask), mine, atol=1e-6)
    fresh = MMDiT(a).float()
    fresh.init_weights(0)
    with torch.no_grad():
        assert fresh(z0, t, text, mask).abs().max() == 0        # adaLN-zero start: zero velocity


def test_mmdit_trains_through_the_flow_matching_trainer(tmp_path):
    from cosmos_rl_b200.policy.trainer.diffusion_trainer import DiffusionSFTTrainer
    c = Config.from_dict({
        "custom": {"diffusion": {"latent_shape": [4, 8, 8]}},
        "policy": {"model_name_or_path": "tiny-mmdit", "model_gradient_checkpointing": True},
        "train": {"seed": 0, "optm_lr": 2e-3, "optm_warmup_steps": 0, "output_dir": str(tmp_path), "optm_weight_decay": 0.0,
                  "train_batch_per_replica": 8,
                  "train_policy": {"type": "sft", "trainer_type": "diffusion_sft", "mini_batch": 8},
                  "ckpt": {"enable_checkpoint": False}}})
    tr = DiffusionSFTTrainer(c, ParallelDims(world_size=1, device=torch.device("cpu")), device=torch.device("cpu"))
    tr.model_load_from_hf()
    assert type(tr.model).__name__ == "MMDiT"
    g = torch.Generator().manual_seed(0)
    base = torch.randn(4, 8, 8, generator=g)
    batch = [{"latents": (base + 0.05 * torch.randn(4, 8, 8, generator=g)).tolist(),
              "text_embeds": torch.randn(4, 64, generator=g).tolist()} for _ in range(8)]
    torch.manual_seed(0)
    losses = [tr.step_training(batch, total_steps=100, train_step=i + 1)["train/loss_avg"] for i in range(100)]
    assert sum(losses[-10:]) < 0.6 * sum(losses[:10]), (losses[:10], losses[-10:])      # measured: 0.27
