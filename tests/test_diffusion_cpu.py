"""Diffusion transformer, flow-matching SFT, and the two diffusion RL algorithms (DiffusionNFT, FlowGRPO) through the
colocated worker on CPU with a tiny DiT."""
import math

import pytest
import torch

from cosmos_rl_b200.config import Config
from cosmos_rl_b200.models.dit import ARCHS, DiT
from cosmos_rl_b200.parallel.dims import ParallelDims
from cosmos_rl_b200.policy import diffusion as D
from cosmos_rl_b200.rollout.diffusion_rollout import LatentStore


def _dit(seed=0, randomize_zero_init=True):
    torch.manual_seed(seed)
    m = DiT(ARCHS["tiny-dit"])
    m.init_weights(seed)
    if randomize_zero_init:                      # adaLN-zero starts as the zero map: make the blocks matter
        with torch.no_grad():
            for n, p in m.named_parameters():
                if "modulation" in n or n.startswith("patch_out"):
                    p.normal_(0, 0.05)
    return m.eval()


def test_dit_shapes_zero_init_and_text_padding():
    m0 = _dit(randomize_zero_init=False)
    z = torch.randn(2, 4, 3, 8, 8)
    text = torch.randn(2, 5, 64)
    assert m0(z, torch.tensor([0.3, 0.9]), text).abs().max() == 0          # adaLN-zero
    m = _dit()
    v = m(z, torch.tensor([0.3, 0.9]), text)
    assert v.shape == z.shape and v.abs().max() > 0
    img = m(z[:, :, 0], torch.tensor([0.3, 0.9]), text)
    assert img.shape == (2, 4, 8, 8)
    # padded text positions are invisible; samples do not see each other
    pad = torch.cat([text, torch.randn(2, 3, 64)], 1)
    mask = torch.tensor([[1] * 5 + [0] * 3] * 2, dtype=torch.bool)
    assert torch.allclose(m(z, torch.tensor([0.3, 0.9]), pad, mask), v, atol=1e-5)
    assert torch.allclose(m(z[:1], torch.tensor([0.3]), text[:1]), v[:1], atol=1e-5)
    tok, grid = m.patchify(z)
    assert grid == (3, 4, 4) and torch.equal(m.unpatchify(tok, grid), z)


def test_flow_math():
    t = D.sample_timesteps(4096, "logit_normal", shift=3.0)
    assert 0 < t.min() and t.max() < 1 and t.mean() > 0.6                       # shift moves mass to the noisy end
    x0, eps = torch.randn(3, 4, 8, 8), torch.randn(3, 4, 8, 8)
    # a model that knows the true velocity transports noise exactly onto the data, with any step count
    oracle = lambda x, tt, text, mask: eps - x0
    assert torch.allclose(D.euler_sample(oracle, eps, None, steps=3), x0, atol=1e-5)
    # SDE transition: the recorded log-prob is the Gaussian density of the step actually taken
    out = D.sde_sample(oracle, eps, None, steps=4, noise_level=0.5)
    ts = out["timesteps"].tolist()
    assert out["states"].shape == (3, 3, 4, 8, 8) and out["logprobs"].shape == (3, 3)
    mean = D.sde_mean(out["states"][:, 1], eps - x0, ts[1], ts[2], 0.5)
    _, std = D.sde_coeffs(ts[1], ts[2], 0.5)
    assert torch.allclose(D.sde_logprob(out["next_states"][:, 1], mean, std), out["logprobs"][:, 1], atol=1e-5)
    # NFT: with v == v_old the two branches coincide, the gradient pushes good samples' x0-prediction to x0
    v = torch.zeros_like(x0, requires_grad=True)
    tt = torch.tensor([0.5, 0.5, 0.5])
    xt = D.add_noise(x0, tt, eps)
    loss, m = D.nft_loss(v, torch.zeros_like(x0), torch.zeros_like(x0), xt, x0, tt, torch.tensor([5.0, -5.0, 0.0]),
                         beta=1.0, adv_clip=5.0, kl_beta=0.1)
    loss.backward()
    err = xt - x0                                                               # x0-prediction error at v = 0
    cos = lambda a, b: torch.nn.functional.cosine_similarity(a.flatten(), b.flatten(), dim=0)
    assert cos(-v.grad[0], err[0]) > 0.99 and cos(-v.grad[1], -err[1]) > 0.99   # good: towards x0; bad: away
    assert v.grad[2].abs().max() < 1e-6 and m["kl_loss"] == 0                   # r = 1/2: branches cancel


def _config(tmp_path, trainer_type, **diff):
    d = {"latent_shape": [4, 8, 8], "sample_steps": 4, "train_timesteps": 2, "nft_beta": 1.0, "old_decay": "copy"}
    d.update(diff)
    return Config.from_dict({
        "mode": "colocated", "custom": {"diffusion": d},
        "policy": {"model_name_or_path": "tiny-dit", "model_gradient_checkpointing": False},
        "rollout": {"backend": "diffusion", "batch_size": 4, "n_generation": 4, "seed": 0},
        "train": {"seed": 0, "optm_lr": 2e-3, "optm_warmup_steps": 0, "output_dir": str(tmp_path),
                  "train_batch_per_replica": 16, "epoch": 1, "optm_weight_decay": 0.0,
                  "train_policy": {"type": "grpo", "trainer_type": trainer_type, "mini_batch": 8, "kl_beta": 1e-3,
                                   "advantage_high": 2.0, "advantage_low": -2.0},
                  "ckpt": {"enable_checkpoint": False}}})


def test_flow_matching_sft_learns_a_fixed_batch(tmp_path):
    from cosmos_rl_b200.policy.trainer.diffusion_trainer import DiffusionSFTTrainer
    c = _config(tmp_path, "diffusion_sft")
    c.train.train_policy.type = "sft"
    tr = DiffusionSFTTrainer(c, ParallelDims(world_size=1, device=torch.device("cpu")), device=torch.device("cpu"))
    tr.model_load_from_hf()
    g = torch.Generator().manual_seed(0)
    base = torch.randn(4, 8, 8, generator=g)
    batch = [{"latents": (base + 0.05 * torch.randn(4, 8, 8, generator=g)).tolist(),
              "text_embeds": torch.randn(3, 64, generator=g).tolist()} for _ in range(8)]
    torch.manual_seed(0)
    losses = [tr.step_training(batch, total_steps=40, train_step=i + 1)["train/loss_avg"] for i in range(40)]
    assert sum(losses[-5:]) / 5 < 0.8 * sum(losses[:5]) / 5, (losses[:5], losses[-5:])


class _Prompts:
    def __init__(self, n):
        g = torch.Generator().manual_seed(5)
        self.rows = [{"text_embeds": torch.randn(3, 64, generator=g).tolist(), "seed": i} for i in range(n)]

    def __len__(self):
        return len(self.rows)

    def __getitem__(self, i):
        return self.rows[i]

    def get_reference_answer(self, i):
        return ""


def brightness_reward(completion, reference=None, **kw) -> float:
    return float(LatentStore.get(completion)["x0"].float().mean())


@pytest.mark.parametrize("trainer_type,extra", [("diffusion_nft", {}), ("flow_grpo", {"sampler": "sde", "noise_level": 0.7})])
def test_diffusion_rl_raises_the_reward(tmp_path, trainer_type, extra):
    from cosmos_rl_b200.colocated.worker import ColocatedRLControlWorker
    torch.manual_seed(0)
    c = _config(tmp_path, trainer_type, **extra)
    w = ColocatedRLControlWorker(c, _Prompts(96), reward_fns=[brightness_reward], device=torch.device("cpu"))
    reports = w.run(max_iterations=400)
    assert len(reports) == 24 and all(math.isfinite(r["train/loss_avg"]) for r in reports)
    assert not LatentStore._items                                    # every latent was released after its step
    # the trained model generates brighter latents than the initial one from the same noise
    g = torch.Generator().manual_seed(1)
    noise, text = torch.randn(16, 4, 8, 8, generator=g), torch.randn(16, 3, 64, generator=g)
    after = D.euler_sample(w.trainer.model.eval(), noise, text, steps=4).mean().item()
    fresh = DiT(ARCHS["tiny-dit"])
    fresh.init_weights(0)
    before = D.euler_sample(fresh.eval(), noise, text, steps=4).mean().item()
    assert after > before + 0.02, (before, after)


def test_generation_mini_batches_give_the_same_latents(tmp_path):
    """``rollout.n_generation_mini_batch``: the ODE sampler run on slices of a group returns the latents of one pass."""
    from cosmos_rl_b200.parallel.dims import ParallelDims
    from cosmos_rl_b200.rollout.diffusion_rollout import DiffusionRollout

    def run(mb):
        c = _config(tmp_path, "diffusion_nft", sampler="ode")
        c.rollout.n_generation_mini_batch = mb
        r = DiffusionRollout(c, ParallelDims(world_size=1, device=torch.device("cpu")), torch.device("cpu"))
        r.init_engine()
        g = torch.Generator().manual_seed(1)
        samples = [(torch.randn(5, r.model.args.text_dim, generator=g), 7), (torch.randn(3, r.model.args.text_dim, generator=g), 8)]
        out, n = r._generate(r._collate_batch(samples, False), False)
        return out["x0"], n

    full, n = run(None)
    part, _ = run(3)
    assert n == 4 and full.shape[0] == 8 and torch.allclose(full, part, atol=1e-5)


def test_ode_solvers_converge_at_their_order_on_a_gaussian_flow():
    """For data ~ N(mu, s^2) the optimal velocity field is known in closed form and its flow carries noise z to
    mu + s z. Every solver reaches that end point; halving the step divides the error by about 2^order (Euler 1; midpoint,
    Heun, two-step Adams-Bashforth and the exponential data-prediction integrator 2; Kutta 3); the one-call second-order
    solvers beat Euler at equal network calls. Also the parametrisation helpers."""
    import math
    from cosmos_rl_b200.policy.diffusion import timestep_grid
    from cosmos_rl_b200.policy.diffusion_solvers import (EDMScaling, LogNormalSigma, RectifiedFlowScaling, calls_per_step,
                                                         integrate, is_solver_supported, karras_sigmas, sample)
    mu, s = 0.7, 0.4

    def f(x, t):
        var = (1 - t) ** 2 * s * s + t * t
        return (x - (1 - t) * mu) * (t - (1 - t) * s * s) / var - mu

    z = torch.linspace(-2.0, 2.0, 9, dtype=torch.float64)
    want = mu + s * z

    def err(solver, steps):
        ts = timestep_grid(steps).double()
        return float((integrate(f, z.clone(), ts, solver) - want).abs().max())
    orders = {"euler": 1, "midpoint": 2, "heun": 2, "ab2": 2, "exp2": 2, "kutta3": 3}
    for name, order in orders.items():
        assert is_solver_supported(name)
        e1, e2 = err(name, 40), err(name, 80)
        assert e2 < 2e-2 and e1 / e2 > 2 ** order * 0.6, (name, e1, e2)
    assert not is_solver_supported("rk9")
    assert err("ab2", 40) < err("euler", 40) / 5 and err("exp2", 40) < err("euler", 40) / 5     # same number of calls
    assert err("heun", 20) < err("euler", 40)                                                    # same number of calls
    assert calls_per_step("kutta3") == 3 and calls_per_step("exp2") == 1
    assert err("exp2", 8) < 0.05                                           # usable at very few steps
    # through the public entry point with a "network" of the same field, guidance mixing two fields
    net = lambda x, t, text, mask: f(x.double(), t.double()[:, None]).to(x.dtype) if text == "c" else torch.zeros_like(x)
    out = sample(net, z.float()[:, None], "c", steps=30, solver="heun", guidance=1.0)
    assert torch.allclose(out[:, 0].double(), want, atol=2e-3)
    half = sample(net, z.float()[:, None], "c", steps=30, solver="euler", guidance=0.5, null_text="u")
    assert torch.allclose(half, z.float()[:, None] + 0.5 * (sample(net, z.float()[:, None], "c", steps=30, solver="euler") - z.float()[:, None]), atol=0.2)
    # parametrisations
    sig = torch.tensor([0.01, 0.5, 10.0])
    c_skip, c_out, c_in, c_noise = EDMScaling(0.5)(sig)
    assert torch.allclose(c_skip[1], torch.tensor(0.5)) and c_skip[0] > 0.99 and c_skip[2] < 0.01
    assert torch.allclose(c_in * (sig ** 2 + 0.25).sqrt(), torch.ones(3)) and torch.allclose(c_noise, sig.log() / 4)
    rf = RectifiedFlowScaling()
    assert torch.allclose(rf.t_to_sigma(rf.sigma_to_t(sig)), sig, rtol=1e-5)
    x0, eps = torch.randn(5), torch.randn(5)
    for sg in (0.3, 2.0):
        t = rf.sigma_to_t(torch.tensor(sg))
        xt = (1 - t) * x0 + t * eps
        cs, co, ci, cn = rf(torch.tensor(sg))
        assert torch.allclose(ci * (x0 + sg * eps), xt, atol=1e-6)        # the scaled EDM input is the flow's x_t
        assert torch.allclose(cs * xt + co * (eps - x0), x0, atol=1e-6)   # denoiser from the true velocity
    sm = LogNormalSigma().sample(4000, generator=torch.Generator().manual_seed(0))
    assert abs(float(sm.log().mean()) + 1.2) < 0.1 and sm.min() >= 0.002 and sm.max() <= 80.0
    ks = karras_sigmas(10)
    assert ks.shape == (11,) and abs(float(ks[0]) - 80.0) < 1e-3 and ks[-1] == 0 and bool((ks[:-1].diff() < 0).all())


def test_causal_video_vae_shapes_causality_and_training():
    """The tokenizer in front of the DiT: 1 + 4 k frames -> 1 + k latent frames at 1/8 resolution and back; a single
    frame is a valid clip; latents of a prefix equal the prefix of the latents (nothing flows from the future, neither
    in the encoder nor in the decoder); a few optimisation steps reduce the reconstruction loss; latent statistics
    normalise what the DiT sees."""
    from cosmos_rl_b200.models.video_vae import VideoVAE, VideoVAEArgs
    torch.manual_seed(0)
    vae = VideoVAE(VideoVAEArgs(base_dim=8, dim_mult=(1, 2, 2, 2), num_res_blocks=1, z_dim=4))
    assert vae.args.spatial_factor == 8 and vae.args.temporal_factor == 4 and vae.latent_frames(9) == 3
    x = torch.rand(2, 3, 9, 32, 32) * 2 - 1
    mean, logvar = vae.encode(x)
    assert mean.shape == (2, 4, 3, 4, 4) == logvar.shape
    assert vae.decode(vae.tokenize(x)).shape == x.shape
    assert vae.encode(x[:, :, :1])[0].shape == (2, 4, 1, 4, 4) and vae.decode(mean[:, :, :1], False).shape == (2, 3, 1, 32, 32)
    with pytest.raises(ValueError):
        vae.encode(x[:, :, :8])
    with torch.no_grad():
        # encoder: frames 5.. do not reach latent frames 0 and 1 (which cover pixel frames 0..4)
        y = x.clone()
        y[:, :, 5:] = torch.rand(2, 3, 4, 32, 32)
        m2 = vae.encode(y)[0]
        assert torch.allclose(m2[:, :, :2], mean[:, :, :2], atol=1e-5) and not torch.allclose(m2[:, :, 2], mean[:, :, 2], atol=1e-3)
        assert torch.allclose(vae.encode(x[:, :, :5])[0], mean[:, :, :2], atol=1e-5)       # prefix of a clip
        # decoder: the last latent frame does not reach pixel frames 0..4
        z2 = mean.clone()
        z2[:, :, 2] += 1.0
        a, b = vae.decode(mean, False), vae.decode(z2, False)
        assert torch.allclose(a[:, :, :5], b[:, :, :5], atol=1e-5) and not torch.allclose(a[:, :, 5:], b[:, :, 5:], atol=1e-3)
    opt = torch.optim.Adam(vae.parameters(), lr=2e-3)
    clip = torch.sin(torch.linspace(0, 6, 32))[None, None, None, None, :].expand(1, 3, 5, 32, 32).contiguous()
    first = None
    for _ in range(30):
        out = vae.loss(clip)
        opt.zero_grad()
        out["loss"].backward()
        opt.step()
        first = first if first is not None else float(out["rec"])
    assert float(out["rec"]) < 0.7 * first, (first, float(out["rec"]))
    vae.fit_latent_stats([clip, x[:1, :, :5]])
    z = vae.tokenize(torch.cat([clip, x[:1, :, :5]]))
    assert z.transpose(0, 1).reshape(4, -1).mean(1).abs().max() < 0.2


@pytest.mark.timeout(300)
def test_flow_grpo_job_with_separate_rollout_and_policy_processes(tmp_path):
    """FlowGRPO as a disaggregated job through the launcher: the rollout process samples latents with the SDE sampler and
    writes latent + trace to the trajectory store on a shared folder (``[custom] replay_buffer_dir``), only the id
    travels through the controller, the policy process loads the traces, trains, releases them, and the new weights of
    the diffusion transformer reach the rollout process over the pair's communicator. Plus the store's own contract."""
    import os
    import subprocess
    import sys
    from cosmos_rl_b200.config import dump_toml
    from cosmos_rl_b200.utils.replay_buffer import ReplayBuffer
    rb = ReplayBuffer(str(tmp_path / "rb"))
    k = rb.save({"x": torch.arange(4)})
    assert k in rb and torch.equal(rb.load(k)["x"], torch.arange(4)) and len(rb) == 1
    with pytest.raises(KeyError):
        rb.load("0" * 32)
    with pytest.raises(ValueError):
        rb.load("../etc")
    assert rb.cleanup(max_age_s=3600) == 0 and rb.delete([k, "missing"]) == 1 and len(rb) == 0
    here = os.path.dirname(os.path.abspath(__file__))
    root = os.path.dirname(here)
    raw = {"mode": "disaggregated",
           "custom": {"replay_buffer_dir": str(tmp_path / "replay"),
                      "diffusion": {"latent_shape": [4, 8, 8], "sample_steps": 4, "sampler": "sde", "noise_level": 0.7}},
           "policy": {"model_name_or_path": "tiny-dit", "model_gradient_checkpointing": False,
                      "parallelism": {"tp_size": 1, "dp_shard_size": 1}},
           "rollout": {"backend": "diffusion", "batch_size": 4, "n_generation": 4, "seed": 0,
                       "parallelism": {"tp_size": 1}},
           "train": {"seed": 0, "epoch": 1, "optm_lr": 2e-3, "optm_warmup_steps": 0, "optm_weight_decay": 0.0,
                     "output_dir": str(tmp_path / "out"), "train_batch_per_replica": 16,
                     "train_policy": {"type": "grpo", "trainer_type": "flow_grpo", "mini_batch": 8,
                                      "dataloader_shuffle": False},   # default staleness bound (4): nothing is dropped in 4 steps
                     "ckpt": {"enable_checkpoint": False}},
           "logging": {"logger": ["console"]}}
    cfg = tmp_path / "job.toml"
    cfg.write_text(dump_toml(raw))
    env = dict(os.environ, COSMOS_LOG_LEVEL="INFO", PYTHONPATH=root, OMP_NUM_THREADS="2", N_PROMPTS="16")
    cmd = [sys.executable, "-m", "cosmos_rl_b200.launcher.launch_all", "--config", str(cfg), "--policy", "1",
           "--rollout", "1", "--cpu", "--rdzv-port", "29851", "--log-dir", str(tmp_path / "logs"),
           os.path.join(here, "diffusion_job_script.py")]
    p = subprocess.Popen(cmd, env=env, cwd=root, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                         start_new_session=True)
    try:
        out, _ = p.communicate(timeout=260)
    except subprocess.TimeoutExpired:
        import signal
        os.killpg(p.pid, signal.SIGKILL)                  # the group this test started, by its exact id
        out, _ = p.communicate()
    latest = tmp_path / "logs" / "logs_latest"
    logs = {f: open(latest / f).read() for f in sorted(os.listdir(latest))} if latest.exists() else {}
    detail = "\n".join(f"==== {k}\n{v[-2500:]}" for k, v in logs.items())
    assert p.returncode == 0, out[-2000:] + detail
    assert "training finished at step 4" in logs["controller.log"], detail
    assert "weight version" in logs["rollout_0.log"] and "transport=collective" in logs["rollout_0.log"], detail
    assert os.listdir(tmp_path / "replay") == []                          # every trace was fetched and released
