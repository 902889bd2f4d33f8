"""End-to-end GRPO on CPU/gloo through the real launcher: controller + 1 policy rank + 1 rollout rank as
separate processes, tiny Qwen2-architecture model, 16 prompts of 64 tokens, group 4, 64 response tokens,
even-token reward. Two training steps with a weight synchronisation in between; every process must exit 0."""
import json
import os
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


def _run_job(cmd, env, timeout):
    """Run a launcher command in its own process group; on a timeout the whole group (launcher, controller, replicas)
    is killed, so a hung job never leaves processes behind."""
    import signal
    p = subprocess.Popen(cmd, env=env, cwd=ROOT, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True,
                         start_new_session=True)
    try:
        out, err = p.communicate(timeout=timeout)
    except subprocess.TimeoutExpired:
        os.killpg(p.pid, signal.SIGKILL)          # the group this test started, by its exact id
        out, err = p.communicate()
        return subprocess.CompletedProcess(cmd, -9, out, err + "\n[test] job timed out and was killed")
    return subprocess.CompletedProcess(cmd, p.returncode, out, err)


@pytest.mark.timeout(420)
def test_tiny_grpo_job_runs_to_completion(tmp_path):
    log_dir = tmp_path / "logs"
    env = dict(os.environ, COSMOS_LOG_LEVEL="INFO", COSMOS_HEARTBEAT_SEND_INTERVAL="2", PYTHONPATH=ROOT,
               OMP_NUM_THREADS="2")
    cmd = [sys.executable, "-m", "cosmos_rl_b200.launcher.launch_all", "--config",
           os.path.join(HERE, "configs", "tiny_grpo_cpu.toml"), "--policy", "1", "--rollout", "1", "--cpu",
           "--log-dir", str(log_dir), os.path.join(HERE, "e2e_script.py")]
    r = _run_job(cmd, env, 400)
    logs = {}
    latest = log_dir / "logs_latest"
    for f in sorted(os.listdir(latest)):
        logs[f] = open(latest / f).read()
    detail = "\n".join(f"==== {k}\n{v[-3000:]}" for k, v in logs.items())
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:] + detail
    ctrl = logs["controller.log"]
    assert "step 1/2" in ctrl and "step 2/2" in ctrl, detail
    assert "training finished at step 2" in ctrl, detail


@pytest.mark.timeout(300)
def test_tiny_grpo_job_colocated_single_process(tmp_path):
    """The same job with ``mode = "colocated"``: the launcher starts ONE process that holds the controller logic,
    the trainer and the generation engine (sharing one set of weights)."""
    from cosmos_rl_b200.config import dump_toml, load_toml
    raw = load_toml(os.path.join(HERE, "configs", "tiny_grpo_cpu.toml"))
    raw["mode"] = "colocated"
    raw["train"]["output_dir"] = str(tmp_path / "out")
    cfg = tmp_path / "job.toml"
    cfg.write_text(dump_toml(raw))
    log_dir = tmp_path / "logs"
    env = dict(os.environ, COSMOS_LOG_LEVEL="INFO", PYTHONPATH=ROOT, OMP_NUM_THREADS="2")
    cmd = [sys.executable, "-m", "cosmos_rl_b200.launcher.launch_all", "--config", str(cfg), "--cpu",
           "--log-dir", str(log_dir), os.path.join(HERE, "e2e_script.py")]
    r = _run_job(cmd, env, 280)
    files = sorted(os.listdir(log_dir / "logs_latest"))
    log = open(log_dir / "logs_latest" / "colocated_0.log").read()
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:] + log[-3000:]
    assert files == ["colocated_0.log"]                                  # no controller / rollout processes
    assert "[Colocated] finished after 2 training steps" in log, log[-3000:]


@pytest.mark.timeout(420)
def test_tiny_grpo_job_with_distillation_teacher(tmp_path):
    """On-policy distillation end to end: controller + policy + rollout + teacher replica; the rollout side asks the
    teacher to score every completion, the policy fetches the scores and reports the teacher KL."""
    from cosmos_rl_b200.config import dump_toml, load_toml
    raw = load_toml(os.path.join(HERE, "configs", "tiny_grpo_cpu.toml"))
    raw["train"]["output_dir"] = str(tmp_path / "out")
    raw["distillation"] = {"enable": True, "model_name_or_path": "tiny-qwen2", "kl_penalty_coef": 1.0,
                           "parallelism": {"tp_size": 1, "dp_shard_size": 1, "n_init_replicas": 1}}
    cfg = tmp_path / "job.toml"
    cfg.write_text(dump_toml(raw))
    log_dir = tmp_path / "logs"
    env = dict(os.environ, COSMOS_LOG_LEVEL="INFO", COSMOS_HEARTBEAT_SEND_INTERVAL="2", PYTHONPATH=ROOT,
               OMP_NUM_THREADS="2")
    cmd = [sys.executable, "-m", "cosmos_rl_b200.launcher.launch_all", "--config", str(cfg), "--policy", "1",
           "--rollout", "1", "--reference", "1", "--cpu", "--log-dir", str(log_dir), os.path.join(HERE, "e2e_script.py")]
    r = _run_job(cmd, env, 400)
    latest = log_dir / "logs_latest"
    logs = {f: open(latest / f).read() for f in sorted(os.listdir(latest))}
    detail = "\n".join(f"==== {k}\n{v[-2500:]}" for k, v in logs.items())
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:] + detail
    assert "reference_0.log" in logs, list(logs)
    ctrl = logs["controller.log"]
    assert "training finished at step 2" in ctrl and "train/teacher_kl_reversed" in ctrl, detail


@pytest.mark.timeout(420)
def test_tiny_grpo_job_with_lora(tmp_path):
    """[policy.lora] through the whole disaggregated flow: only adapters train, the policy folds them into the dense
    weights while a rollout replica pulls them, and the job completes."""
    from cosmos_rl_b200.config import dump_toml, load_toml
    raw = load_toml(os.path.join(HERE, "configs", "tiny_grpo_cpu.toml"))
    raw["train"]["output_dir"] = str(tmp_path / "out")
    raw["policy"]["lora"] = {"r": 4, "lora_alpha": 8, "target_modules": ["q_proj", "v_proj", "down_proj"]}
    cfg = tmp_path / "job.toml"
    cfg.write_text(dump_toml(raw))
    log_dir = tmp_path / "logs"
    env = dict(os.environ, COSMOS_LOG_LEVEL="INFO", COSMOS_HEARTBEAT_SEND_INTERVAL="2", PYTHONPATH=ROOT,
               OMP_NUM_THREADS="2", COSMOS_WEIGHT_SYNC_CHECK="1")
    cmd = [sys.executable, "-m", "cosmos_rl_b200.launcher.launch_all", "--config", str(cfg), "--policy", "1",
           "--rollout", "1", "--cpu", "--log-dir", str(log_dir), os.path.join(HERE, "e2e_script.py")]
    r = _run_job(cmd, env, 400)
    latest = log_dir / "logs_latest"
    logs = {f: open(latest / f).read() for f in sorted(os.listdir(latest))}
    detail = "\n".join(f"==== {k}\n{v[-2500:]}" for k, v in logs.items())
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:] + detail
    assert "training finished at step 2" in logs["controller.log"], detail
    assert "[WeightSyncCheck] coverage ok" in logs["rollout_0.log"], detail      # the first sync was verified too


@pytest.mark.timeout(420)
def test_tiny_grpo_job_with_async_rollout_scheduler(tmp_path):
    """``rollout.mode = "async"``: generation runs on the scheduler's thread, the control loop feeds it and reports;
    weight updates are fenced by the scheduler's pause."""
    from cosmos_rl_b200.config import dump_toml, load_toml
    raw = load_toml(os.path.join(HERE, "configs", "tiny_grpo_cpu.toml"))
    raw["rollout"]["mode"] = "async"
    raw["rollout"]["async_config"] = {"max_concurrent_requests": 8}
    raw["train"]["output_dir"] = str(tmp_path / "out")
    cfg = tmp_path / "job.toml"
    cfg.write_text(dump_toml(raw))
    log_dir = tmp_path / "logs"
    env = dict(os.environ, COSMOS_LOG_LEVEL="INFO", COSMOS_HEARTBEAT_SEND_INTERVAL="2", PYTHONPATH=ROOT,
               OMP_NUM_THREADS="2")
    cmd = [sys.executable, "-m", "cosmos_rl_b200.launcher.launch_all", "--config", str(cfg), "--policy", "1",
           "--rollout", "1", "--cpu", "--log-dir", str(log_dir), os.path.join(HERE, "e2e_script.py")]
    r = _run_job(cmd, env, 400)
    latest = log_dir / "logs_latest"
    logs = {f: open(latest / f).read() for f in sorted(os.listdir(latest))}
    detail = "\n".join(f"==== {k}\n{v[-3000:]}" for k, v in logs.items())
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:] + detail
    assert "training finished at step 2" in logs["controller.log"], detail
    assert "async scheduler" in logs["rollout_0.log"], detail


@pytest.mark.timeout(420)
def test_tiny_grpo_job_with_pair_payload_transport(tmp_path):
    """``[custom] payload_transfer = "nccl"``: token ids and log-probs of finished rollouts stay on the rollout worker
    and reach the policy over a two-rank communicator (gloo here) after a request / answer handshake through the
    controller's broker; the job trains to completion from the fetched data."""
    from cosmos_rl_b200.config import dump_toml, load_toml
    raw = load_toml(os.path.join(HERE, "configs", "tiny_grpo_cpu.toml"))
    raw["custom"] = {"payload_transfer": "nccl"}
    raw["train"]["output_dir"] = str(tmp_path / "out")
    cfg = tmp_path / "job.toml"
    cfg.write_text(dump_toml(raw))
    log_dir = tmp_path / "logs"
    env = dict(os.environ, COSMOS_LOG_LEVEL="INFO", COSMOS_HEARTBEAT_SEND_INTERVAL="2", PYTHONPATH=ROOT,
               OMP_NUM_THREADS="2")
    cmd = [sys.executable, "-m", "cosmos_rl_b200.launcher.launch_all", "--config", str(cfg), "--policy", "1",
           "--rollout", "1", "--cpu", "--log-dir", str(log_dir), os.path.join(HERE, "e2e_script.py")]
    r = _run_job(cmd, env, 400)
    latest = log_dir / "logs_latest"
    logs = {f: open(latest / f).read() for f in sorted(os.listdir(latest))}
    detail = "\n".join(f"==== {k}\n{v[-2500:]}" for k, v in logs.items())
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:] + detail
    assert "training finished at step 2" in logs["controller.log"], detail
    assert "'nccl' payload transport" in logs["rollout_0.log"], detail
    assert "through the payload transport" in logs["policy_0.log"], detail
    assert "could not be fetched" not in logs["policy_0.log"], detail


@pytest.mark.timeout(300)
def test_sft_job_with_two_policy_replicas(tmp_path):
    """Multi-replica SFT through the launcher (cosmos_rl/policy/worker/multi_replica_sft_worker.py:44-565): the
    controller sends the membership once both replicas have registered, each replica takes its slice of every global
    batch (half the steps of a single replica), and the gradients are averaged over the inter-replica communicator, so
    both report the same gradient norm on different losses."""
    import re
    from cosmos_rl_b200.config import dump_toml
    raw = {"mode": "disaggregated",
           "train": {"epoch": 1, "output_dir": str(tmp_path / "out"), "train_batch_per_replica": 4, "optm_lr": 1e-3,
                     "optm_warmup_steps": 0, "seed": 0, "train_policy": {"type": "sft", "mini_batch": 2,
                                                                         "dataloader_shuffle": False},
                     "ckpt": {"enable_checkpoint": False}},
           "policy": {"model_name_or_path": "tiny-qwen2", "model_max_length": 128, "model_gradient_checkpointing": False,
                      "parallelism": {"tp_size": 1, "dp_shard_size": 1, "n_init_replicas": 2}},
           "logging": {"logger": ["console"]}}
    cfg = tmp_path / "job.toml"
    cfg.write_text(dump_toml(raw))
    log_dir = tmp_path / "logs"
    env = dict(os.environ, COSMOS_LOG_LEVEL="INFO", COSMOS_HEARTBEAT_SEND_INTERVAL="2", PYTHONPATH=ROOT,
               OMP_NUM_THREADS="2", E2E_N_PROMPTS="32")
    cmd = [sys.executable, "-m", "cosmos_rl_b200.launcher.launch_all", "--config", str(cfg), "--policy", "2", "--cpu",
           "--rdzv-port", "29761", "--log-dir", str(log_dir), os.path.join(HERE, "e2e_script.py")]
    r = _run_job(cmd, env, 280)
    latest = log_dir / "logs_latest"
    logs = {f: open(latest / f).read() for f in sorted(os.listdir(latest))}
    detail = "\n".join(f"==== {k}\n{v[-2500:]}" for k, v in logs.items())
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:] + detail
    steps = {}
    for name in ("policy_0.log", "policy_1.log"):
        assert re.search(r"replica [01] of 2: data-parallel slice [01] of 2", logs[name]), detail
        steps[name] = re.findall(r"\[SFT\] step (\d+)/(\d+) loss=([\d.]+) grad_norm=([\d.]+)", logs[name])
        assert [s[0] for s in steps[name]] == ["1", "2", "3", "4"] and steps[name][0][1] == "4", detail
    a, b = steps["policy_0.log"], steps["policy_1.log"]
    assert [s[3] for s in a] == [s[3] for s in b], detail                 # one averaged gradient
    assert [s[2] for s in a] != [s[2] for s in b], detail                 # from different halves of the batch


@pytest.mark.timeout(300)
def test_launcher_layout_benchmark_reads_the_controllers_step_reports():
    """``bench.py --layout launcher``: the job runs through ``launcher.launch_all`` and the figure comes from the
    stamps of the controller's step reports (here the colocated worker on CPU with a tiny model)."""
    import argparse
    from cosmos_rl_b200 import bench_launcher as BL
    rows = [{"step": s, "time": 100.0 + 2.0 * s} for s in range(1, 5)]
    t = BL.throughput(rows, warmup=1, steps=3, tokens_per_step=1000)
    assert abs(t["value"] - 500.0) < 1e-9 and abs(t["ms_per_step"] - 2000.0) < 1e-6
    with pytest.raises(ValueError):
        BL.throughput(rows, warmup=2, steps=3, tokens_per_step=1000)
    assert BL.job_layout(1)[0] == "colocated" and BL.job_layout(8) == ("disaggregated", 4, 2, 2)
    a = argparse.Namespace(gpus=1, steps=2, warmup=1, model="tiny-qwen2", prompts_per_gpu=2, group=2, prompt_len=16,
                           max_response=8, mb_tokens=256, rdzv_port=29781)
    out = BL.run(a, cpu=True, timeout_s=240)
    assert out["breakdown"]["steps_reported"] == 3 and out["value"] > 0
    assert out["breakdown"]["tokens_trained_per_step"] == 2 * 2 * 24 and out["config"]["layout"] == "launcher"


@pytest.mark.timeout(420)
def test_job_over_three_nodes_with_a_policy_replica_that_spans_two(tmp_path):
    """Three launchers stand in three nodes of two ranks each (``--num-workers 3 --gpus-per-node 2``): every one
    derives the same plan from the job-wide replica counts. The policy replica (dp_shard 4) spans nodes 0 and 1 (two
    ``torchrun`` groups that meet at node 0's rendezvous port), the rollout replica lands on node 2; nodes 1 and 2
    find the controller of node 0 through ``--node-ip-list`` and ``--port``. Each node claims its own machine
    identity, so the weights take the communicator route."""
    import socket
    import time as _time
    from cosmos_rl_b200.config import dump_toml, load_toml
    from cosmos_rl_b200.launcher import launch_all as L
    from cosmos_rl_b200.config import Config
    raw = load_toml(os.path.join(HERE, "configs", "tiny_grpo_cpu.toml"))
    raw["policy"]["parallelism"]["dp_shard_size"] = 4
    raw["train"]["output_dir"] = str(tmp_path / "out")
    cfg = tmp_path / "job.toml"
    cfg.write_text(dump_toml(raw))
    plan = L.plan_nodes(1, 1, 0, Config.from_dict(raw), 2)
    assert [[(e["role"], e["nnodes"], e["node_rank"], e["rdzv_node"]) for e in row] for row in plan] == \
        [[("policy", 2, 0, 0)], [("policy", 2, 1, 0)], [("rollout", 1, 0, 2)]]
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    procs = []
    import signal
    try:
        for idx in range(3):
            env = dict(os.environ, COSMOS_LOG_LEVEL="INFO", COSMOS_HEARTBEAT_SEND_INTERVAL="2", PYTHONPATH=ROOT,
                       OMP_NUM_THREADS="1", COSMOS_HOST_ID=f"node{idx}")
            cmd = [sys.executable, "-m", "cosmos_rl_b200.launcher.launch_all", "--config", str(cfg), "--policy", "1",
                   "--rollout", "1", "--cpu", "--num-workers", "3", "--worker-idx", str(idx), "--gpus-per-node", "2",
                   "--node-ip-list", "127.0.0.1;127.0.0.1;127.0.0.1", "--port", str(port), "--rdzv-port", "29801",
                   "--log-dir", str(tmp_path / f"logs{idx}"), os.path.join(HERE, "e2e_script.py")]
            procs.append(subprocess.Popen(cmd, env=env, cwd=ROOT, stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                                          text=True, start_new_session=True))
        deadline = _time.time() + 380
        while _time.time() < deadline and any(p.poll() is None for p in procs):
            _time.sleep(0.5)
    finally:
        for p in procs:
            if p.poll() is None:
                os.killpg(p.pid, signal.SIGKILL)          # the groups this test started, by their exact ids
    outs = [p.communicate()[0] for p in procs]
    logs = {}
    for idx in range(3):
        d = tmp_path / f"logs{idx}" / "logs_latest"
        for f in (sorted(os.listdir(d)) if d.exists() else []):
            logs[f"node{idx}/{f}"] = open(d / f).read()
    detail = "\n".join(f"==== {k}\n{v[-2500:]}" for k, v in logs.items()) + "\n".join(o[-1500:] for o in outs)
    assert [p.returncode for p in procs] == [0, 0, 0], detail
    assert sorted(logs) == ["node0/controller.log", "node0/policy_0.log", "node1/policy_0.log", "node2/rollout_0.log"]
    assert "training finished at step 2" in logs["node0/controller.log"], detail
    assert "transport=collective" in logs["node2/rollout_0.log"], detail
