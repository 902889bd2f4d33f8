"""GRPO jobs on GPUs through the real process stack: launcher -> controller process -> policy and rollout replica
processes (torchrun groups) -> trainer / generation engine, with the weights handed over by the peer-memory pull
(CUDA IPC handles exchanged through the controller). The reference tests the same flow with dummy models
(tests/test_process_flow.py:119-653, tests/test_policy_to_rollout.py:36-110). With one GPU visible the replicas share
it (``--share-gpus``); with two or more each replica gets its own."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


def _run_job(cmd, env, timeout):
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


def _launch(tmp_path, mode, extra_env=None, n_prompts="12"):
    from cosmos_rl_b200.config import dump_toml, load_toml
    raw = load_toml(os.path.join(HERE, "configs", "tiny_grpo_gpu.toml"))
    raw["mode"] = mode
    raw["train"]["output_dir"] = str(tmp_path / "out")
    cfg = tmp_path / "job.toml"
    cfg.write_text(dump_toml(raw))
    log_dir = tmp_path / "logs"
    env = dict(os.environ, COSMOS_LOG_LEVEL="INFO", COSMOS_HEARTBEAT_SEND_INTERVAL="2", PYTHONPATH=ROOT,
               COSMOS_WEIGHT_SYNC_CHECK="1", E2E_N_PROMPTS=n_prompts, NCCL_NVLS_ENABLE="0")
    env.update(extra_env or {})
    cmd = [sys.executable, "-m", "cosmos_rl_b200.launcher.launch_all", "--config", str(cfg), "--policy", "1",
           "--rollout", "1", "--share-gpus", "--log-dir", str(log_dir), os.path.join(HERE, "e2e_script.py")]
    r = _run_job(cmd, env, 400)
    latest = log_dir / "logs_latest"
    logs = {f: open(latest / f).read() for f in sorted(os.listdir(latest))} if latest.exists() else {}
    detail = "\n".join(f"==== {k}\n{v[-3000:]}" for k, v in logs.items())
    return r, logs, detail


@pytest.mark.timeout(460)
def test_disaggregated_job_through_launcher_on_gpu(tmp_path):
    """12 prompts x 4 samples / 16 per step = 3 training steps, a peer-memory weight pull before every generation
    round; the first pull is verified against a zeroed buffer (COSMOS_WEIGHT_SYNC_CHECK)."""
    r, logs, detail = _launch(tmp_path, "disaggregated")
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:] + detail
    ctrl = logs["controller.log"]
    assert "step 3/3" in ctrl and "training finished at step 3" in ctrl, detail
    ro = logs["rollout_0.log"]
    assert "[WeightSyncCheck] coverage ok" in ro, detail
    assert "transport=peer" in ro, detail                      # IPC pull, not the collective fallback
    assert "weight version 2 committed" in ro and "device cuda" in ro, detail


@pytest.mark.timeout(460)
def test_colocated_separated_job_on_gpu(tmp_path):
    """``colocated_separated``: the launcher pairs the policy and the rollout replica on the SAME GPU as two processes;
    the rollout process pulls the weights out of the policy process's memory on that GPU."""
    r, logs, detail = _launch(tmp_path, "colocated_separated")
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:] + detail
    assert "training finished at step 3" in logs["controller.log"], detail
    assert "transport=peer" in logs["rollout_0.log"], detail
