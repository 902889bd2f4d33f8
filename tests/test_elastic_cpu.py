"""Elasticity at process level on CPU/gloo: a job with 2 policy and 2 rollout replicas (policy-to-policy state
broadcast, inter-replica gradient all-reduce, rollout-to-rollout weight commit), in which one policy replica is
killed on the host between steps. The controller must notice the missing heartbeat, drop the replica, rebuild the
mesh of the survivor and finish the job. The failure is made on the host (SIGKILL of processes this test started,
found by the tag the launcher gave them); nothing on a device is faulted. The reference tests the same scenario
with fake replicas around its ``HighAvailabilitylNccl`` (tests/test_high_availability_nccl.py:1-447)."""
import os
import signal
import subprocess
import sys
import time

import psutil
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


def _tagged(root_pid: int, tag: str):
    out = []
    try:
        for p in psutil.Process(root_pid).children(recursive=True):
            try:
                if p.environ().get("COSMOS_REPLICA_TAG") == tag:
                    out.append(p)
            except (psutil.NoSuchProcess, psutil.AccessDenied):
                pass
    except psutil.NoSuchProcess:
        pass
    return out


@pytest.mark.timeout(600)
def test_policy_replica_killed_between_steps_job_continues(tmp_path):
    from cosmos_rl_b200.config import dump_toml, load_toml
    raw = load_toml(os.path.join(HERE, "configs", "tiny_grpo_cpu.toml"))
    raw["train"]["output_dir"] = str(tmp_path / "out")
    raw["train"]["train_policy"]["allowed_outdated_steps"] = 0      # one generation round per weight version
    cfg = tmp_path / "job.toml"
    cfg.write_text(dump_toml(raw))
    log_dir = tmp_path / "logs"
    env = dict(os.environ, COSMOS_LOG_LEVEL="INFO", COSMOS_HEARTBEAT_SEND_INTERVAL="1", COSMOS_HEARTBEAT_TIMEOUT="8",
               COSMOS_ROLLOUT_SCAN_INTERVAL="1", COSMOS_NCCL_TIMEOUT_MS="15000", PYTHONPATH=ROOT, OMP_NUM_THREADS="2",
               E2E_N_PROMPTS="48")                                    # 48 x 4 samples: one step of 2 x 32, then steps of 32
    cmd = [sys.executable, "-m", "cosmos_rl_b200.launcher.launch_all", "--config", str(cfg), "--policy", "2",
           "--rollout", "2", "--cpu", "--tolerate-replica-failures", "--log-dir", str(log_dir),
           os.path.join(HERE, "e2e_script.py")]
    job = subprocess.Popen(cmd, env=env, cwd=ROOT, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                           start_new_session=True)
    latest = log_dir / "logs_latest"
    killed = False
    try:
        deadline = time.time() + 300
        while time.time() < deadline and job.poll() is None:
            # a quiet moment: step 1 is trained and both rollout replicas have committed its weights
            quiet = all((latest / f).exists() and "weight version 1 committed" in (latest / f).read_text()
                        for f in ("rollout_0.log", "rollout_1.log"))
            if quiet:
                # the victim is the policy replica that is not the weight source (the source is the replica that
                # loaded the initial weights; the other one received them by a policy-to-policy broadcast)
                first = [t for t in ("policy_0", "policy_1") if "random-init weights" in (latest / f"{t}.log").read_text()]
                victim = "policy_1" if first == ["policy_0"] or not first else "policy_0"
                victims = _tagged(job.pid, victim)
                assert victims, f"{victim} processes not found"
                for p in victims:                                      # exact pids of processes this job started
                    try:
                        p.send_signal(signal.SIGKILL)
                    except psutil.NoSuchProcess:
                        pass
                killed = True
                break
            time.sleep(0.2)
        assert killed, "the job never reached step 1"
        out, _ = job.communicate(timeout=420)
    except BaseException:
        if job.poll() is None:
            os.killpg(job.pid, signal.SIGKILL)
        raise
    logs = {f: open(latest / f).read() for f in sorted(os.listdir(latest))}
    detail = "\n".join(f"==== {k}\n{v[-3500:]}" for k, v in logs.items())
    ctrl = logs["controller.log"]
    assert job.returncode == 0, out[-3000:] + detail
    assert "training finished" in ctrl, detail
    assert "missed its heartbeat; removing it" in ctrl, detail           # the dead replica was dropped ...
    assert ctrl.count("[Controller] step ") >= 3, detail                # ... and training went on after the kill


@pytest.mark.timeout(600)
def test_rollout_replica_joins_a_running_job(tmp_path):
    """Scale-up while the job runs: a second launcher attaches one more rollout replica to the controller of a job
    that already trains (``--url ... --no-controller --policy 0 --rollout 1``). The controller registers it, rebuilds
    the rollout mesh, the newcomer receives the current weights and takes prompts; the job finishes with both
    launchers exiting 0."""
    import socket
    from cosmos_rl_b200.config import dump_toml, load_toml
    raw = load_toml(os.path.join(HERE, "configs", "tiny_grpo_cpu.toml"))
    raw["train"]["output_dir"] = str(tmp_path / "out")
    raw["train"]["train_policy"]["allowed_outdated_steps"] = 0
    cfg = tmp_path / "job.toml"
    cfg.write_text(dump_toml(raw))
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    env = dict(os.environ, COSMOS_LOG_LEVEL="INFO", COSMOS_HEARTBEAT_SEND_INTERVAL="1", COSMOS_ROLLOUT_SCAN_INTERVAL="1",
               COSMOS_NCCL_TIMEOUT_MS="30000", PYTHONPATH=ROOT, OMP_NUM_THREADS="2", E2E_N_PROMPTS="96")   # 12 steps of 32: long enough for the newcomer to come up on a fast machine
    base = [sys.executable, "-m", "cosmos_rl_b200.launcher.launch_all", "--config", str(cfg), "--cpu"]
    first = subprocess.Popen(base + ["--policy", "1", "--rollout", "1", "--port", str(port), "--rdzv-port", "29821",
                                     "--log-dir", str(tmp_path / "logs_a"), os.path.join(HERE, "e2e_script.py")],
                             env=env, cwd=ROOT, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                             start_new_session=True)
    second = None
    la, lb = tmp_path / "logs_a" / "logs_latest", tmp_path / "logs_b" / "logs_latest"
    try:
        deadline = time.time() + 300
        while time.time() < deadline and first.poll() is None:
            f = la / "controller.log"
            if f.exists() and "[Controller] step 1/" in f.read_text():
                break
            time.sleep(0.2)
        assert first.poll() is None, "the job ended before a replica could join"
        second = subprocess.Popen(base + ["--policy", "0", "--rollout", "1", "--url", f"127.0.0.1:{port}",
                                          "--no-controller", "--rdzv-port", "29831", "--log-dir", str(tmp_path / "logs_b"),
                                          os.path.join(HERE, "e2e_script.py")],
                                  env=env, cwd=ROOT, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                                  start_new_session=True)
        out_a, _ = first.communicate(timeout=420)
        out_b, _ = second.communicate(timeout=120)
    except BaseException:
        for p in (first, second):
            if p is not None and p.poll() is None:
                os.killpg(p.pid, signal.SIGKILL)
        raise
    logs = {f"a/{f}": open(la / f).read() for f in sorted(os.listdir(la))}
    logs.update({f"b/{f}": open(lb / f).read() for f in (sorted(os.listdir(lb)) if lb.exists() else [])})
    detail = "\n".join(f"==== {k}\n{v[-3000:]}" for k, v in logs.items())
    assert first.returncode == 0 and second.returncode == 0, out_a[-2000:] + out_b[-2000:] + detail
    assert "training finished" in logs["a/controller.log"], detail
    newcomer = logs["b/rollout_0.log"]
    assert "[Rollout] weight version" in newcomer and "committed" in newcomer, detail   # it received current weights
