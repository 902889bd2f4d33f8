"""OpenVLA and the SD3-style transformer on the GPU in bf16 against the same weights in fp32 on the CPU."""
import copy

import pytest
import torch

from cosmos_rl_b200.ops import native


@pytest.mark.gpu
def test_openvla_bf16_on_gpu_matches_fp32_reference():
    """Decoder with head_dim 128 on the tcgen05 attention and GEMM kernels, featurizers with the head sizes 64 and 72 of
    the published towers (library attention for those sizes): logits of a packed batch of two prompts with one image
    each, and the gradient that reaches the first featurizer."""
    from cosmos_rl_b200.models.openvla import OpenVLA, OpenVLAArgs, ViTArgs, build_prompt
    torch.manual_seed(0)
    a = OpenVLAArgs(vocab_size=2048 + 64, dim=512, n_layers=2, n_heads=4, n_kv_heads=4, ffn_dim=1024, rope_theta=1e4,
                    qkv_bias=False, model_type="openvla", image_token_id=2048)
    a.towers = [ViTArgs(embed_dim=128, depth=3, num_heads=2, mlp_dim=256, image_size=56, patch_size=14, class_token=True,
                        reg_tokens=4, layer_scale=True),
                ViTArgs(embed_dim=144, depth=3, num_heads=2, mlp_dim=288, image_size=56, patch_size=14, class_token=False)]
    ref = OpenVLA(a).float()
    with torch.no_grad():
        for n, p in ref.named_parameters():
            if p.dim() > 1:
                p.normal_(0, 0.05)
            else:
                p.fill_(1.0 if ("norm" in n and not n.endswith("bias")) else (0.1 if n.endswith(("ls1", "ls2")) else 0.0))
    g = torch.Generator().manual_seed(1)
    seq1 = build_prompt([1] + torch.randint(3, 1900, (30,), generator=g).tolist(), ref.n_patches, a.image_token_id)
    seq2 = build_prompt([1] + torch.randint(3, 1900, (12,), generator=g).tolist(), ref.n_patches, a.image_token_id)
    ids = torch.tensor(seq1 + seq2)
    cu = torch.tensor([0, len(seq1), len(seq1) + len(seq2)], dtype=torch.int32)
    mm = {"pixel_values": torch.randn(2, 6, 56, 56, generator=g)}
    ref.mm_inputs = mm
    want = ref.logits(ref(ids, ref.get_position_ids(cu, ids.numel()), cu, len(seq1)))
    want.square().mean().backward()
    gpu = copy.deepcopy(ref).to("cuda", torch.bfloat16)
    gpu.zero_grad()
    gpu.mm_inputs = {"pixel_values": mm["pixel_values"].cuda()}
    cu_g = cu.cuda()
    got = gpu.logits(gpu(ids.cuda(), gpu.get_position_ids(cu_g, ids.numel()), cu_g, len(seq1)))
    got.square().mean().backward()
    torch.cuda.synchronize()
    assert native.read_status(torch.device("cuda")) == 0
    err = (got.float().cpu() - want).abs().max()
    assert want.abs().max() > 0.5 and err < 0.06 * want.abs().max() + 0.03, (float(err), float(want.abs().max()))
    # the gradients that reach the towers through three projector layers are tiny: cosine in float64, no epsilon
    for probe in (lambda m: m.projector.fc1.weight, lambda m: m.visual.featurizer.blocks[0].qkv.weight):
        g_ref, g_gpu = probe(ref).grad.double().flatten(), probe(gpu).grad.double().cpu().flatten()
        assert g_ref.norm() > 0 and g_gpu.norm() > 0
        cos = float(g_ref @ g_gpu / (g_ref.norm() * g_gpu.norm()))
        assert cos > 0.95, cos


@pytest.mark.gpu
@pytest.mark.parametrize("head_dim", [64, 128])
def test_mmdit_bf16_on_gpu_matches_fp32_reference(head_dim):
    """Joint attention over [image tokens; text tokens] of samples with different text lengths: head_dim 128 runs the
    tcgen05 non-causal kernel, 64 (the published size) the library kernel."""
    from cosmos_rl_b200.models.mmdit import MMDiT, MMDiTArgs
    torch.manual_seed(0)
    a = MMDiTArgs(sample_size=16, patch_size=2, in_channels=4, out_channels=4, num_layers=3, attention_head_dim=head_dim,
                  num_attention_heads=256 // head_dim, joint_attention_dim=96, caption_projection_dim=256,
                  pooled_projection_dim=64, pos_embed_max_size=24)
    ref = MMDiT(a).float()
    with torch.no_grad():
        for n, p in ref.named_parameters():
            p.normal_(0, 0.05) if p.dim() > 1 else p.zero_()
    g = torch.Generator().manual_seed(2)
    z = torch.randn(3, 4, 16, 16, generator=g)
    t = torch.tensor([0.2, 0.6, 0.95])
    text = torch.randn(3, 1 + 9, 96, generator=g)
    mask = torch.ones(3, 10, dtype=torch.bool)
    mask[1, 4:] = False
    mask[2, 7:] = False
    want = ref(z, t, text, mask)
    want.square().mean().backward()
    gpu = copy.deepcopy(ref).to("cuda", torch.bfloat16)
    gpu.zero_grad()
    got = gpu(z.cuda().bfloat16(), t.cuda(), text.cuda().bfloat16(), mask.cuda())
    got.square().mean().backward()
    torch.cuda.synchronize()
    assert native.read_status(torch.device("cuda")) == 0
    err = (got.float().cpu() - want).abs().max()
    assert err < 0.06 * want.abs().max() + 0.03, (float(err), float(want.abs().max()))
    g_ref = ref.transformer_blocks[0].attn.add_q_proj.weight.grad
    g_gpu = gpu.transformer_blocks[0].attn.add_q_proj.weight.grad.float().cpu()
    cos = torch.nn.functional.cosine_similarity(g_ref.flatten(), g_gpu.flatten(), dim=0)
    assert cos > 0.95, float(cos)
