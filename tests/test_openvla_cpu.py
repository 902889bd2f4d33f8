"""Native OpenVLA: featurizers against transformers' DINOv2-with-registers and SigLIP towers, the whole model against a
Llama of transformers fed with the spliced embeddings, checkpoint names, action bins against numpy, OFT heads."""
import numpy as np
import torch

from cosmos_rl_b200.models import hf_io
from cosmos_rl_b200.models.base import ModelRegistry
from cosmos_rl_b200.models.openvla import ARCHS, ActionBins, L1ActionHead, OpenVLA, OpenVLAArgs, build_prompt


def _dinov2_reference(state, prefix, v):
    from transformers import Dinov2WithRegistersConfig, Dinov2WithRegistersModel
    cfg = Dinov2WithRegistersConfig(hidden_size=v.embed_dim, num_hidden_layers=v.depth - 1, num_attention_heads=v.num_heads,
                                    mlp_ratio=v.mlp_dim // v.embed_dim, image_size=v.image_size, patch_size=v.patch_size,
                                    num_register_tokens=v.reg_tokens, layerscale_value=1.0, layer_norm_eps=v.eps,
                                    hidden_act="gelu")
    hf = Dinov2WithRegistersModel(cfg).eval().float()
    g = lambda k: state[prefix + k]                                                      # noqa: E731
    sd = {"embeddings.cls_token": g("cls_token"), "embeddings.register_tokens": g("reg_token"),
          "embeddings.mask_token": torch.zeros(1, v.embed_dim),
          "embeddings.position_embeddings": torch.cat([torch.zeros(1, 1, v.embed_dim), g("pos_embed")], dim=1),
          "embeddings.patch_embeddings.projection.weight": g("patch_embed.proj.weight"),
          "embeddings.patch_embeddings.projection.bias": g("patch_embed.proj.bias"),
          "layernorm.weight": torch.ones(v.embed_dim), "layernorm.bias": torch.zeros(v.embed_dim)}
    for i in range(v.depth - 1):
        b, h = f"blocks.{i}.", f"encoder.layer.{i}."
        qw, kw, vw = g(b + "attn.qkv.weight").chunk(3)
        qb, kb, vb = g(b + "attn.qkv.bias").chunk(3)
        sd.update({h + "attention.attention.query.weight": qw, h + "attention.attention.query.bias": qb,
                   h + "attention.attention.key.weight": kw, h + "attention.attention.key.bias": kb,
                   h + "attention.attention.value.weight": vw, h + "attention.attention.value.bias": vb,
                   h + "attention.output.dense.weight": g(b + "attn.proj.weight"),
                   h + "attention.output.dense.bias": g(b + "attn.proj.bias"),
                   h + "layer_scale1.lambda1": g(b + "ls1.scale_factor"), h + "layer_scale2.lambda1": g(b + "ls2.scale_factor")})
        for n in ("norm1", "norm2", "mlp.fc1", "mlp.fc2"):
            sd[h + n + ".weight"], sd[h + n + ".bias"] = g(b + n + ".weight"), g(b + n + ".bias")
    missing = hf.load_state_dict(sd, strict=True)
    return lambda px: hf(pixel_values=px, output_hidden_states=True).hidden_states[-1][:, 1 + v.reg_tokens:]


def _siglip_reference(state, prefix, v):
    from transformers import SiglipVisionConfig, SiglipVisionModel
    cfg = SiglipVisionConfig(hidden_size=v.embed_dim, num_hidden_layers=v.depth - 1, num_attention_heads=v.num_heads,
                             intermediate_size=v.mlp_dim, image_size=v.image_size, patch_size=v.patch_size,
                             layer_norm_eps=v.eps, hidden_act="gelu")
    hf = SiglipVisionModel(cfg).eval().float()
    g = lambda k: state[prefix + k]                                                      # noqa: E731
    sd = dict(hf.state_dict())                                                           # keeps the unused pooling head
    sd.update({"vision_model.embeddings.patch_embedding.weight": g("patch_embed.proj.weight"),
               "vision_model.embeddings.patch_embedding.bias": g("patch_embed.proj.bias"),
               "vision_model.embeddings.position_embedding.weight": g("pos_embed")[0]})
    for i in range(v.depth - 1):
        b, h = f"blocks.{i}.", f"vision_model.encoder.layers.{i}."
        for j, n in enumerate(("q_proj", "k_proj", "v_proj")):
            sd[h + f"self_attn.{n}.weight"] = g(b + "attn.qkv.weight").chunk(3)[j]
            sd[h + f"self_attn.{n}.bias"] = g(b + "attn.qkv.bias").chunk(3)[j]
        for mine, theirs in (("attn.proj", "self_attn.out_proj"), ("norm1", "layer_norm1"), ("norm2", "layer_norm2"),
                             ("mlp.fc1", "mlp.fc1"), ("mlp.fc2", "mlp.fc2")):
            sd[h + theirs + ".weight"], sd[h + theirs + ".bias"] = g(b + mine + ".weight"), g(b + mine + ".bias")
    hf.load_state_dict(sd, strict=True)
    return lambda px: hf(pixel_values=px, output_hidden_states=True).hidden_states[-1]


def test_native_openvla_matches_a_composition_of_transformers_modules():
    """The published model is remote code, so the oracle is assembled from library parts fed with this model's exported
    checkpoint: DINOv2-with-registers and SigLIP towers (patch tokens before the final norm), the three-layer fused
    projector written out, and a Llama that receives the spliced embeddings. Checks the export names on the way."""
    from transformers import LlamaConfig, LlamaForCausalLM
    torch.manual_seed(0)
    args = ARCHS["tiny-openvla"]
    cfg = args.to_hf_config()
    assert ModelRegistry.get("openvla") is OpenVLA
    m = OpenVLA(OpenVLAArgs.from_hf_config(cfg)).float()
    m.init_weights(0)
    with torch.no_grad():
        for n, p in m.named_parameters():
            if n.startswith(("visual.", "projector.")) and p.dim() == 1 and not n.endswith(("ls1", "ls2")):
                p.add_(0.05 * torch.randn_like(p))                       # biases and norm weights off their defaults
            if n.endswith((".pos_embed", ".cls_token", ".reg_token")):
                p.copy_(0.1 * torch.randn_like(p))
    state = hf_io.hf_state_dict(m, cfg)
    names = set(state)
    assert "language_model.model.layers.1.self_attn.q_proj.weight" in names and "language_model.lm_head.weight" in names
    assert state["vision_backbone.featurizer.patch_embed.proj.weight"].shape == (64, 3, 14, 14)
    assert state["vision_backbone.featurizer.pos_embed"].shape == (1, 16, 64)
    assert state["vision_backbone.featurizer.reg_token"].shape == (1, 4, 64)
    assert "vision_backbone.featurizer.blocks.1.ls2.scale_factor" in names
    assert "vision_backbone.fused_featurizer.blocks.0.attn.qkv.bias" in names and "projector.fc3.weight" in names
    # ---- the oracle
    dino = _dinov2_reference(state, "vision_backbone.featurizer.", args.towers[0])
    sig = _siglip_reference(state, "vision_backbone.fused_featurizer.", args.towers[1])
    t = cfg["text_config"]
    lcfg = LlamaConfig(vocab_size=t["vocab_size"], hidden_size=t["hidden_size"], num_hidden_layers=t["num_hidden_layers"],
                       num_attention_heads=t["num_attention_heads"], num_key_value_heads=t["num_key_value_heads"],
                       intermediate_size=t["intermediate_size"], rope_theta=t["rope_theta"],
                       rms_norm_eps=t.get("rms_norm_eps", 1e-6), max_position_embeddings=512, tie_word_embeddings=False,
                       attention_bias=False)
    llama = LlamaForCausalLM(lcfg).eval().float()
    llama.load_state_dict({k[len("language_model."):]: v for k, v in state.items() if k.startswith("language_model.")})
    gelu = torch.nn.functional.gelu
    lin = lambda x, n: torch.nn.functional.linear(x, state[f"projector.{n}.weight"], state[f"projector.{n}.bias"])  # noqa: E731

    def reference(text_ids, px):
        with torch.no_grad():
            patches = torch.cat([dino(px[:, :3]), sig(px[:, 3:])], dim=2)
            proj = lin(gelu(lin(gelu(lin(patches, "fc1")), "fc2")), "fc3")
            emb = llama.get_input_embeddings()(torch.tensor([text_ids]))
            spliced = torch.cat([emb[:, :1], proj, emb[:, 1:]], dim=1)
            return llama(inputs_embeds=spliced).logits[0]

    pix = torch.randn(2, 6, 56, 56)
    text1, text2 = [1, 10, 11, 12, 13], [1, 20, 21]
    seq1 = build_prompt(text1, m.n_patches, args.image_token_id)
    seq2 = build_prompt(text2, m.n_patches, args.image_token_id)
    assert seq1[:2] == [1, 32000] and len(seq1) == 5 + 16
    ids = torch.tensor(seq1 + seq2)
    cu = torch.tensor([0, len(seq1), len(seq1) + len(seq2)], dtype=torch.int32)
    m.mm_inputs = {"pixel_values": pix}
    mine = m.logits(m(ids, m.get_position_ids(cu, ids.numel()), cu, len(seq1)))
    ref = torch.cat([reference(text1, pix[:1]), reference(text2, pix[1:])])
    assert (mine - ref).abs().max().item() < 2e-4, (mine - ref).abs().max()
    mine.square().mean().backward()
    assert m.visual.featurizer.blocks[0].qkv.weight.grad.abs().sum() > 0
    assert m.visual.fused_featurizer.patch_embed.weight.grad.abs().sum() > 0 and m.projector.fc1.weight.grad.abs().sum() > 0
    # ---- a second model loads the exported checkpoint and computes the same logits
    m2 = OpenVLA(OpenVLAArgs.from_hf_config(cfg)).float()
    hf_io.load_hf_state(m2, lambda k: state[k], state, cfg)
    m2.mm_inputs = {"pixel_values": pix}
    with torch.no_grad():
        again = m2.logits(m2(ids, m2.get_position_ids(cu, ids.numel()), cu, len(seq1)))
    assert torch.allclose(again, mine.detach(), atol=1e-6)


def test_action_bins_follow_the_published_tokenizer_rules():
    """Encoding is ``vocab - numpy.digitize(clip(normalised action), linspace(-1, 1, 256))``; decoding takes bin centres,
    clips the index to the 255 centres and un-normalises only the masked dimensions with q01 / q99."""
    stats = {"demo": {"action": {"q01": [-1.0, -0.5, 0.0], "q99": [1.0, 0.5, 2.0], "mask": [True, True, False]}}}
    bins = ActionBins(32000, 256, stats)
    assert bins.action_dim() == 3
    g = torch.Generator().manual_seed(0)
    a = torch.rand(50, 3, generator=g) * 2 - 1
    a[:, 1] *= 0.5
    tok = bins.encode(a)
    edges = np.linspace(-1, 1, 256)
    norm = a.numpy().copy()
    norm[:, 1] = 2 * (norm[:, 1] + 0.5) / 1.0 - 1
    want = 32000 - np.digitize(np.clip(norm, -1, 1), edges)
    assert np.array_equal(tok.numpy(), want) and tok.min() >= 32000 - 256 and tok.max() <= 31999
    back = bins.decode(tok)
    centers = (edges[:-1] + edges[1:]) / 2
    idx = np.clip(32000 - tok.numpy() - 1, 0, 254)
    ref = centers[idx]
    ref[:, 0] = 0.5 * (ref[:, 0] + 1) * 2 - 1
    ref[:, 1] = 0.5 * (ref[:, 1] + 1) * 1.0 - 0.5
    assert np.allclose(back.numpy(), ref, atol=1e-6)
    assert (back[:, :2] - a[:, :2]).abs().max() < 2.0 / 255                       # within one bin of the input
    plain = ActionBins(32000, 256)
    assert float(plain.decode(torch.tensor([32000 - 256]))) == float(plain.decode(torch.tensor([32000 - 255])))  # top clipped
    m = OpenVLA(ARCHS["tiny-openvla"])
    assert m.bins.vocab == 32000 and m.decode_actions(torch.tensor([[31999, 31872, 31744]])).shape == (1, 3)


def test_oft_state_projector_and_l1_head():
    """The state becomes one more prompt embedding behind the patches; the regression head turns the hidden states at the
    action positions into a chunk of continuous actions and fits a target under the L1 loss."""
    import copy
    torch.manual_seed(0)
    a = copy.deepcopy(ARCHS["tiny-openvla"])
    a.proprio_dim, a.action_head, a.action_chunk = 5, True, 2
    m = OpenVLA(OpenVLAArgs.from_hf_config(a.to_hf_config())).float()
    m.init_weights(0)
    assert isinstance(m.action_head, L1ActionHead) and m.proprio_projector is not None
    n_act = a.action_chunk * a.action_dim
    text = [1, 10, 11] + [31000] * n_act                                   # action positions at the end
    seq = build_prompt(text, m.n_patches, a.image_token_id, extra=1)
    ids = torch.tensor(seq)
    cu = torch.tensor([0, len(seq)], dtype=torch.int32)
    m.mm_inputs = {"pixel_values": torch.randn(1, 6, 56, 56), "proprio": torch.randn(1, 5)}
    target = torch.tensor([[[0.5, -0.5, 0.2], [-0.3, 0.1, 0.9]]])
    opt = torch.optim.Adam(m.parameters(), lr=1e-3)
    losses = []
    for _ in range(120):
        h = m(ids, m.get_position_ids(cu, ids.numel()), cu, len(seq))
        loss = m.action_head.l1_loss(h[-n_act:][None], target)
        opt.zero_grad()
        loss.backward()
        opt.step()
        losses.append(float(loss))
    assert m.proprio_projector.fc1.weight.grad.abs().sum() > 0
    assert losses[-1] < 0.5 * losses[0], (losses[0], losses[-1])
    assert m.action_head(h[-n_act:][None]).shape == (1, 2, 3)


def test_openvla_sft_through_the_trainer_and_data_packer(tmp_path):
    """Robot records -> ``OpenVLADataPacker`` (prompt with patch placeholders, actions as tokens, labels on the action
    tokens only) -> the SFT trainer on the native model: the action-token loss falls, the featurizers are trained, and the
    greedy next-token prediction at the action positions decodes to the demonstrated actions."""
    from cosmos_rl_b200.config import Config
    from cosmos_rl_b200.data.packer import BaseDataPacker, OpenVLADataPacker
    from cosmos_rl_b200.parallel.dims import ParallelDims
    from cosmos_rl_b200.policy.trainer.sft_trainer import SFTTrainer
    cfg = Config.from_dict({
        "policy": {"model_name_or_path": "tiny-openvla", "model_max_length": 64, "model_gradient_checkpointing": False},
        "train": {"seed": 0, "optm_lr": 2e-3, "optm_warmup_steps": 0, "output_dir": str(tmp_path),
                  "train_policy": {"type": "sft", "trainer_type": "sft", "mini_batch": 4},
                  "ckpt": {"enable_checkpoint": False}}})
    assert BaseDataPacker.get_default("openvla") is OpenVLADataPacker
    packer = OpenVLADataPacker()
    packer.setup(cfg, None)
    cpu = torch.device("cpu")
    tr = SFTTrainer(cfg, ParallelDims(world_size=1, device=cpu), device=cpu, data_packer=packer)
    tr.model_load_from_hf()
    assert type(tr.model).__name__ == "OpenVLA"
    g = torch.Generator().manual_seed(0)
    imgs = [torch.randn(6, 56, 56, generator=g) for _ in range(4)]
    demo = [[0.8, 0.3, 0.9], [-0.6, -0.2, 0.5], [0.1, 0.45, 0.1], [-0.9, 0.0, -0.7]]   # third dimension is not normalised
    batch = [{"instruction_ids": [1, 100 + i, 200, 201], "image": imgs[i], "actions": [demo[i]]} for i in range(4)]
    one = packer.sft_process_sample(batch[0])
    assert len(one["input_ids"]) == 4 + 16 + 3 and one["label_ids"][:-3] == [-100] * 20 and one["label_ids"][-3:] == one["input_ids"][-3:]
    assert all(32000 - 256 <= t <= 31999 for t in one["input_ids"][-3:])
    losses = [tr.step_training(batch, total_steps=60, train_step=i + 1)["train/loss_avg"] for i in range(60)]
    assert losses[-1] < 0.2 * losses[0], (losses[0], losses[-1])
    vis = [s for s in tr.flat.slots if s.name.startswith("visual.featurizer.blocks.0.qkv")][0]
    assert tr.optimizer.m[vis.offset: vis.offset + vis.numel].abs().sum() > 0
    # greedy prediction of the first action token, then decoding
    m = tr.model.eval()
    hits = 0
    for i, b in enumerate(batch):
        s = packer.sft_process_sample(b)
        ids = torch.tensor(s["input_ids"])
        cu = torch.tensor([0, ids.numel()], dtype=torch.int32)
        m.mm_inputs = s["mm"]
        with torch.no_grad():
            logits = m.logits(m(ids, m.get_position_ids(cu, ids.numel()), cu, ids.numel()))
        pred = logits[-4:-1].argmax(-1)                                       # positions that predict the 3 action tokens
        act = m.decode_actions(pred[None], "demo")[0]
        hits += int((act - torch.tensor(demo[i])).abs().max() < 0.05)
    assert hits >= 3, hits


def test_robot_episodes_to_records_and_sft_worker(tmp_path):
    """Demonstration episodes in a tar shard -> per-step records (published prompt wording, letter-boxed camera frame
    normalised once per featurizer, action chunk, state) -> data packer -> the standalone SFT worker on the native
    model; the action statistics give the q01 / q99 the bins un-normalise with."""
    from cosmos_rl_b200.config import Config
    from cosmos_rl_b200.parallel.dims import ParallelDims
    from cosmos_rl_b200.policy.worker.sft_worker import SFTPolicyWorker
    from cosmos_rl_b200.tools.dataset import robot_records as R
    from cosmos_rl_b200.tools.dataset.tar_shards import write_shard
    g = torch.Generator().manual_seed(0)
    episodes = []
    for e in range(3):
        T = 6
        acts = torch.rand(T, 3, generator=g) * 2 - 1
        acts[:, 2] = (acts[:, 2] > 0).float()                               # gripper open / closed
        episodes.append({"instruction": f"Pick up the block number {e}", "actions": acts,
                         "images": torch.randint(0, 256, (T, 40, 72, 3), generator=g, dtype=torch.uint8)})
    write_shard(str(tmp_path / "demo-000.tar"), [{"__key__": f"{i:04d}", "episode.pt": R.episode_bytes(ep)}
                                                 for i, ep in enumerate(episodes)])
    loaded = R.load_episodes(str(tmp_path / "demo-{000..000}.tar"))
    assert len(loaded) == 3 and torch.equal(loaded[1]["actions"], episodes[1]["actions"])
    stats = R.action_statistics(loaded)
    assert stats["action"]["mask"] == [True, True, False] and stats["num_transitions"] == 18
    assert all(lo < hi for lo, hi in zip(stats["action"]["q01"], stats["action"]["q99"]))
    px = R.featurizer_pixels(loaded[0]["images"][0], 56, 2)
    assert px.shape == (6, 56, 56)
    band = px[3:, :12]                                                       # letter-box rows above the 72 x 40 frame
    assert torch.allclose(band, torch.full_like(band, -1.0))                # black after the 0.5 / 0.5 normalisation
    cfg = Config.from_dict({
        "policy": {"model_name_or_path": "tiny-openvla", "model_max_length": 64, "model_gradient_checkpointing": False},
        "train": {"seed": 0, "optm_lr": 1e-3, "optm_warmup_steps": 0, "output_dir": str(tmp_path / "out"), "epoch": 1,
                  "train_batch_per_replica": 6, "max_num_steps": 3,
                  "train_policy": {"type": "sft", "trainer_type": "sft", "mini_batch": 3},
                  "ckpt": {"enable_checkpoint": False}}})
    ds = R.RobotStepDataset(episodes=loaded, unnorm_key="demo")
    ds.setup(cfg, None)
    assert len(ds) == 18 and ds.image_size == 56 and ds.n_feat == 2
    rec = ds[7]
    assert rec["instruction_ids"][0] == 1 and rec["image"].shape == (6, 56, 56) and len(rec["actions"]) == 1
    cpu = torch.device("cpu")
    w = SFTPolicyWorker(cfg, ParallelDims(world_size=1, device=cpu), dataset=ds, standalone=True, device=cpu)
    assert type(w.trainer.data_packer).__name__ == "OpenVLADataPacker" and type(w.trainer.model).__name__ == "OpenVLA"
    w.main_loop()
    assert [h["step"] for h in w.history] == [1, 2, 3] and all(h["train/loss_avg"] > 0 for h in w.history)


class _Seeds:
    def __init__(self, n):
        self.n = n

    def __len__(self):
        return self.n

    def __getitem__(self, i):
        return {"seed": i}

    def get_reference_answer(self, i):
        return ""


def push_right_reward(completion, reference=None, **kw) -> float:
    a = completion["actions"]
    return float(sum(a)) / max(1, len(a))                       # share of "push right" actions of the episode


def test_openvla_closed_loop_grpo_on_rendered_cartpole(tmp_path):
    """The image-conditioned policy as an RL job: the cart-pole state is drawn by the software rasteriser, the policy
    samples its action token from the softmax over the action bins, the environment steps; the trainer scores the same
    tokens under the same restricted distribution (ratio 1 before any update: nothing is clipped at the first step),
    every step of an episode inherits the episode's advantage, traces are released after the step. The reward reads
    the executed actions, and the share of rewarded actions in greedy evaluation episodes rises."""
    from cosmos_rl_b200.colocated.worker import ColocatedRLControlWorker
    from cosmos_rl_b200.config import Config
    from cosmos_rl_b200.dispatcher.data.schema import RLPayload
    from cosmos_rl_b200.rollout.diffusion_rollout import LatentStore
    from cosmos_rl_b200.simulators.render import render_state
    a, b = render_state("cartpole", [0.5, 0, 0.15, 0], 56), render_state("cartpole", [0.5, 0, -0.15, 0], 56)
    assert a.shape == (56, 56, 3) and a.dtype == torch.uint8 and int((a != b).any(-1).sum()) > 50   # the pole leans the other way
    c = Config.from_dict({
        "mode": "colocated", "custom": {"vla": {"env_name": "cartpole", "max_steps": 12, "num_envs": 16}},
        "policy": {"model_name_or_path": "tiny-openvla", "model_max_length": 64, "model_gradient_checkpointing": False},
        "rollout": {"backend": "openvla", "batch_size": 4, "n_generation": 4, "seed": 0,
                    "sampling_config": {"temperature": 1.0, "top_p": 1.0, "top_k": -1}},
        "validation": {"n_generation": 1},
        "train": {"seed": 0, "optm_lr": 3e-4, "optm_warmup_steps": 0, "output_dir": str(tmp_path),
                  "train_batch_per_replica": 16, "epoch": 1,
                  "train_policy": {"type": "grpo", "trainer_type": "openvla_grpo", "mini_batch": 64,
                                   "rollout_as_token_ids": True},
                  "ckpt": {"enable_checkpoint": False}}})
    torch.manual_seed(0)
    w = ColocatedRLControlWorker(c, _Seeds(40), reward_fns=[push_right_reward], device=torch.device("cpu"))
    assert type(w.rollout).__name__ == "OpenVLARollout" and type(w.trainer).__name__ == "OpenVLAGRPOTrainer"
    assert type(w.packer).__name__ == "OpenVLADataPacker" and w.trainer.model.action_only_logprobs
    lo, hi = w.trainer.model.action_token_range
    assert (lo, hi) == (32000 - 256, 32000)

    def evaluate():
        pl = [RLPayload(prompt={"seed": 900 + i}, prompt_idx=i) for i in range(8)]
        res = w.rollout.rollout_generation(pl, None, is_validation=True)
        return sum(push_right_reward(r.completions[0]) for r in res) / len(res)

    before = evaluate()
    LatentStore._items.clear()
    reports = w.run(max_iterations=400)
    assert len(reports) == 10 and all(r["train/transitions"] >= 16 for r in reports)
    assert reports[0]["train/clip_frac"] == 0 and abs(reports[0]["train/ratio_mean"] - 1.0) < 1e-4
    assert not LatentStore._items
    after = evaluate()
    assert after > before + 0.1 or after > 0.9, (before, after)
