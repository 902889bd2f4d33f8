"""Runs a batched environment either inside the worker process or in a spawned child process and forwards method
calls to it (cosmos_rl/simulators/env_manager.py:165-420). The child keeps simulator state out of the worker's
address space and off its CUDA context; ``stop_simulator`` saves the environment state so that a later
``start_simulator`` continues where it stopped (simulators are parked while the policy trains)."""
from __future__ import annotations

import multiprocessing as mp
import traceback
from typing import Any, Optional

_OWN = ("cfg", "rank", "num_envs", "process", "command_queue", "result_queue", "state_buffer", "env_cls", "env",
        "use_subprocess", "context", "timeout_s")


def _simulator_worker(cfg, rank, num_envs, env_cls, commands, results, state_buffer):
    try:
        env = env_cls(cfg, num_envs)
        if state_buffer:
            env.load_state(state_buffer)
        results.put({"status": "ready"})
    except Exception as e:  # noqa: BLE001
        results.put({"status": "error", "error": f"{e}\n{traceback.format_exc()}"})
        return
    while True:
        msg = commands.get()
        if msg["method"] == "shutdown":
            break
        try:
            data = getattr(env, msg["method"])(*msg["args"], **msg["kwargs"])
            results.put({"status": "success", "data": data})
        except Exception as e:  # noqa: BLE001
            results.put({"status": "error", "error": f"{e}\n{traceback.format_exc()}"})
    if hasattr(env, "close"):
        env.close()


class EnvManager:
    def __init__(self, cfg: Any, rank: int, env_cls, use_subprocess: bool = True, timeout_s: float = 60.0):
        self.cfg, self.rank, self.env_cls = cfg, rank, env_cls
        self.num_envs = cfg["num_envs"] if isinstance(cfg, dict) else cfg.num_envs
        self.use_subprocess = use_subprocess
        self.timeout_s = timeout_s
        self.process: Optional[mp.Process] = None
        self.command_queue = None
        self.result_queue = None
        self.state_buffer: Optional[bytes] = None
        self.env = None
        self.context = None

    def start_simulator(self) -> None:
        if self.env is not None or (self.process is not None and self.process.is_alive()):
            return
        if not self.use_subprocess:
            self.env = self.env_cls(self.cfg, self.num_envs)
            if self.state_buffer:
                self.env.load_state(self.state_buffer)
            return
        self.context = mp.get_context("spawn")      # never fork a process that may hold a CUDA context
        self.command_queue, self.result_queue = self.context.Queue(), self.context.Queue()
        self.process = self.context.Process(
            target=_simulator_worker, daemon=True,
            args=(self.cfg, self.rank, self.num_envs, self.env_cls, self.command_queue, self.result_queue,
                  self.state_buffer))
        self.process.start()
        ready = self.result_queue.get(timeout=self.timeout_s)
        if ready["status"] != "ready":
            self.process.join(timeout=5)
            self.process = None
            raise RuntimeError(f"simulator failed to start: {ready.get('error')}")

    def stop_simulator(self) -> None:
        if self.env is not None:
            if hasattr(self.env, "get_state"):
                self.state_buffer = self.env.get_state()
            if hasattr(self.env, "close"):
                self.env.close()
            self.env = None
            return
        if self.process is None or not self.process.is_alive():
            self.process = None
            return
        try:
            self.state_buffer = self._call("get_state")
        except Exception:  # noqa: BLE001  (an environment without state hand-over restarts fresh)
            pass
        self.command_queue.put({"method": "shutdown", "args": [], "kwargs": {}})
        self.process.join(timeout=5)
        if self.process.is_alive():
            self.process.terminate()       # the exact child this manager started
            self.process.join()
        self.process = self.command_queue = self.result_queue = None

    def _call(self, name: str, *args, **kwargs):
        if self.process is None or not self.process.is_alive():
            raise RuntimeError("simulator not running")
        self.command_queue.put({"method": name, "args": args, "kwargs": kwargs})
        res = self.result_queue.get(timeout=self.timeout_s)
        if res["status"] == "error":
            raise RuntimeError(res["error"])
        return res["data"]

    def __getattr__(self, name: str):
        if name.startswith("_") or name in _OWN:
            raise AttributeError(name)
        env = self.__dict__.get("env")
        if env is not None:
            return getattr(env, name)
        return lambda *a, **kw: self._call(name, *a, **kw)
