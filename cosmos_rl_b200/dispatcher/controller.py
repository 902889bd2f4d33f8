"""The single controller ("dispatcher") of a job.

It owns the configuration, the stream broker, the prompt source and both status managers. Everything a
worker needs goes through it: registration, heartbeats, prompts (tagged with the weight version they are
meant for, throttled so that generation cannot run arbitrarily far ahead of training), rollout results,
training acks, handshake key/values (NCCL unique ids, CUDA-IPC handles of peer-mapped weight buffers) and
the weight-sync shard plans (cosmos_rl/dispatcher/controller.py:71-863).
"""
from __future__ import annotations

import base64
import os
import signal
import threading
import time
from typing import Any, Callable, Dict, List, Optional, Tuple

from ..comm.broker import InProcessBroker, StreamBroker
from ..config import Config
from ..utils import constant
from ..utils.logging import logger
from ..utils.report import build_report_hooks
from . import command as cmd
from .data import ControllerDataFetcher, CosmosDataset
from ..utils.payload_transport import PayloadTransportRegistry
from .data.schema import RLPayload, Rollout, payload_to_rollouts
from .protocol import RegisterRequest, Role
from .replica import Atom
from .status import PolicyStatusManager, RolloutStatusManager


class Controller:
    def __init__(self, config: Config, dataset=None, val_dataset=None, broker: Optional[StreamBroker] = None,
                 sampler=None, custom_logger_fns: Optional[List[Callable]] = None):
        self.config = config
        self.broker = broker or InProcessBroker()
        from ..utils.payload_transport import PayloadTransportRegistry, get_payload_transfer_mode
        if get_payload_transfer_mode(config) != "broker":
            # the controller only ever releases parked payloads of rollouts it discards
            PayloadTransportRegistry.get(get_payload_transfer_mode(config)).setup(config, self.broker, None,
                                                                                 owner="controller")
        self.is_rl = config.train.train_policy.type == "grpo"
        ds = CosmosDataset.wrap(dataset, config)
        vds = CosmosDataset.wrap(val_dataset, config)
        self.data_fetcher = ControllerDataFetcher(config, ds, vds, sampler=sampler, is_rl=self.is_rl)
        self.rollout_status_manager = RolloutStatusManager(config, self.broker)
        self.policy_status_manager = PolicyStatusManager(
            config, self.broker, self.data_fetcher, self.rollout_status_manager,
            report_hooks=list(custom_logger_fns or []) + build_report_hooks(config))
        self.rollout_status_manager.policy_manager = self.policy_status_manager
        self.reference_replicas: Dict[str, Any] = {}
        self.policy_status_manager.recompute_total_steps()
        self.lock = threading.RLock()
        self.prompts_handed_out = 0
        self.start_time = time.time()
        self.stat_completion_tokens = 0
        self.stat_samples = 0
        self.stat_invalid = 0
        self._retry_warned = False
        self.shard_infos: Dict[str, Any] = {}
        self.nccl_errors: Dict[str, Tuple[float, str]] = {}
        self.trace_paths: Dict[str, Dict[int, str]] = {}
        self.validation_reports: Dict[int, List[RLPayload]] = {}
        self._monitor: Optional[threading.Thread] = None
        self._stop_monitor = threading.Event()
        self.finalized = threading.Event()
        self.self_terminate = False
        self.failed: Optional[str] = None       # why the job was ended without finishing (exit status 3)
        self._starved_since: Optional[float] = None
        self.rollouts_have_checked_out = False

    # ------------------------------------------------------------------ meta
    def meta(self) -> Dict[str, Any]:
        return {"config": self.config.to_dict(), "total_steps": self.policy_status_manager.total_steps,
                "current_step": self.policy_status_manager.current_step}

    def status(self) -> Dict[str, Any]:
        pm, rm = self.policy_status_manager, self.rollout_status_manager
        return {
            "policy_replicas": [r.summary() for r in pm.replicas.values()],
            "rollout_replicas": [r.summary() for r in rm.replicas.values()],
            "current_step": pm.current_step, "total_steps": pm.total_steps,
            "rollout_buffer": len(pm.rollout_buffer), "samples_on_the_fly": pm.samples_on_the_fly,
            "filtered_outdated": pm.filtered_outdated, "elapsed": time.time() - self.start_time,
            "completion_tokens": self.stat_completion_tokens, "samples": self.stat_samples,
            "history": pm.history[-20:],
        }

    # ------------------------------------------------------------------ registration / liveness
    def register(self, req: RegisterRequest) -> None:
        atom = Atom.from_request(req)
        if req.role == Role.POLICY:
            self.policy_status_manager.register(atom, req.replica_name)
        elif req.role == Role.ROLLOUT:
            self.rollout_status_manager.register(atom, req.replica_name)
        elif req.role == Role.REFERENCE:
            self.reference_replicas.setdefault(req.replica_name, []).append(atom)
        else:
            raise ValueError(f"unknown role {req.role}")

    def unregister(self, replica_name: str) -> None:
        if replica_name in self.policy_status_manager:
            self.policy_status_manager.unregister(replica_name)
        elif replica_name in self.rollout_status_manager:
            self.rollout_status_manager.unregister(replica_name)
            self.rollouts_have_checked_out = True
        else:
            self.reference_replicas.pop(replica_name, None)
        self.rollout_status_manager.maybe_broadcast_stop(self.policy_status_manager)
        self._stop_references_if_done()
        self._maybe_finalize()

    def _stop_references_if_done(self) -> None:
        """Teacher replicas serve until the job ends: once the stop broadcast went out to the rollout side (or no
        policy and no rollout replica is left) they get a ``StopCommand`` too."""
        done = self.rollout_status_manager.stop_broadcast_sent or (
            self.policy_status_manager.had_replicas and not self.policy_status_manager.replicas
            and not self.rollout_status_manager.replicas)
        if done and not getattr(self, "_references_stopped", False):
            self._references_stopped = True
            from ..comm.broker import command_stream
            for name in list(self.reference_replicas):
                self.broker.publish(command_stream(name), cmd.StopCommand(name).pack())

    def heartbeat(self, replica_name: str) -> bool:
        return (self.policy_status_manager.heartbeat(replica_name)
                or self.rollout_status_manager.heartbeat(replica_name)
                or replica_name in self.reference_replicas)

    def _maybe_finalize(self) -> None:
        no_replicas = (not self.policy_status_manager.replicas and not self.rollout_status_manager.replicas
                       and not self.reference_replicas)
        if no_replicas and self.policy_status_manager.had_replicas:
            self.finalized.set()
            if self.self_terminate:
                if self.failed:
                    logger.error("[Controller] job ended without finishing: %s", self.failed)
                    os._exit(3)                 # not the coordinated SIGTERM exit: the launcher reports a failure
                os.kill(os.getpid(), signal.SIGTERM)

    def monitor_once(self, now: Optional[float] = None) -> List[str]:
        """Reap replicas whose heartbeat is older than COSMOS_HEARTBEAT_TIMEOUT; returns the reaped names."""
        reaped = []
        for mgr in (self.policy_status_manager, self.rollout_status_manager):
            for name in mgr.silent_replicas(constant.COSMOS_HEARTBEAT_TIMEOUT, now):
                logger.warning("[Controller] replica %s missed its heartbeat; removing it", name)
                self.unregister(name)
                reaped.append(name)
        self._settle_nccl_errors(now)
        self._check_rollout_starvation(now)
        return reaped

    def _check_rollout_starvation(self, now: Optional[float] = None) -> bool:
        """An RL job that has lost EVERY rollout replica cannot make another step once the buffered rollouts are used
        up: the policies would wait for data forever (on several nodes nobody else notices a node that went away).
        After ``COSMOS_NO_ROLLOUT_GRACE_S`` in that state with no new rollout replica registering, the job is ended in
        order: the policies get ``TrainingComplete`` (final checkpoint when checkpoints are on) and the controller
        leaves with a failure status. Returns True when it just did that."""
        pm, rm = self.policy_status_manager, self.rollout_status_manager
        if self.config.train.train_policy.type == "sft" or self.failed:
            return False
        from .replica import ReplicaStatus
        reps = pm.mesh_replicas()
        stuck = (rm.had_replicas and not rm.replicas and bool(reps) and not pm.complete_sent
                 and not (pm.total_steps and pm.current_step >= pm.total_steps)
                 and not any(r.status == ReplicaStatus.RUNNING for r in reps)
                 and len(pm.rollout_buffer) < pm.batch_per_replica * len(reps))
        if not stuck:
            self._starved_since = None
            return False
        now = time.time() if now is None else now
        if self._starved_since is None:
            self._starved_since = now
            return False
        if now - self._starved_since < constant.COSMOS_NO_ROLLOUT_GRACE_S:
            return False
        self.failed = (f"no rollout replica for {now - self._starved_since:.0f} s at step {pm.current_step} of "
                       f"{pm.total_steps}")
        logger.error("[Controller] %s: ending the job", self.failed)
        with pm.lock:
            pm._send_training_complete()
        return True

    def start_monitor(self, interval: Optional[float] = None) -> None:
        interval = interval if interval is not None else constant.COSMOS_ROLLOUT_SCAN_INTERVAL

        def loop():
            while not self._stop_monitor.wait(interval):
                try:
                    self.monitor_once()
                except Exception as e:  # the monitor must survive any single failure
                    logger.error("monitor error: %s", e)

        self._monitor = threading.Thread(target=loop, name="monitor_replica_status", daemon=True)
        self._monitor.start()

    def stop_monitor(self) -> None:
        self._stop_monitor.set()

    # ------------------------------------------------------------------ NCCL error consensus
    def set_replica_ncclerror(self, replica_name: str, error: str, now: Optional[float] = None) -> None:
        """A replica reports a failed / timed-out inter-replica collective. After a grace period every live
        policy replica that did NOT report is presumed hung and removed, and the mesh is rebuilt
        (cosmos_rl/dispatcher/controller.py:804-863)."""
        with self.lock:
            self.nccl_errors[replica_name] = (now if now is not None else time.time(), error)

    def _settle_nccl_errors(self, now: Optional[float] = None) -> List[str]:
        with self.lock:
            if not self.nccl_errors:
                return []
            now = now if now is not None else time.time()
            first = min(t for t, _ in self.nccl_errors.values())
            if now - first < constant.COSMOS_NCCL_ERROR_CLEAN_REPLICA_DELAY:
                return []
            reporters = set(self.nccl_errors)
            self.nccl_errors = {}
        pm = self.policy_status_manager
        hung = [r.name for r in pm.mesh_replicas() if r.name not in reporters]
        for name in hung:
            logger.warning("[Controller] replica %s never reported the collective failure; presumed hung", name)
            pm.unregister(name)
        if not hung and reporters:
            # everybody reported: rebuild the same membership with fresh communicators
            pm.mesh_built_for = ()
            pm._build_mesh([r for r in pm.live() if r.in_mesh])
        return hung

    # ------------------------------------------------------------------ prompts
    def prompts_per_step(self) -> int:
        pm = self.policy_status_manager
        return max(1, pm.global_batch // max(1, self.config.rollout.n_generation))

    def get_batched_prompt(self, n: int, validation_step: Optional[int] = None
                           ) -> Tuple[List[Tuple[int, RLPayload]], bool]:
        with self.lock:
            if validation_step is not None:
                return self.data_fetcher.get_validation_prompts(n, validation_step)
            pm = self.policy_status_manager
            if pm.total_steps and pm.training_finished():
                return [], True
            tp = self.config.train.train_policy
            n_gen = max(1, self.config.rollout.n_generation)
            gb = max(1, pm.global_batch)
            # soft throttle: at most (allowed_outdated_steps + 1) global batches generated ahead of training;
            # hard ceiling max_inflight_steps when configured
            ahead = (tp.allowed_outdated_steps + 1) if not tp.on_policy else 1
            limit = ahead * gb
            if tp.max_inflight_steps is not None:
                limit = min(limit, tp.max_inflight_steps * gb)
            room = limit - pm.samples_on_the_fly
            if room < n_gen:
                return [], False
            n = min(n, room // n_gen)
            # never hand out more prompts than the remaining steps can consume
            pps_now = max(1, gb // n_gen)

            def still_needed() -> int:
                # prompts the steps that have not started yet still need, beyond those already handed out and waiting
                # (generated or being generated). Counted from the steps left, not from the start of the job, so a
                # change of the batch size (a policy replica joined or was reaped) keeps the budget right; groups
                # dropped by dynamic sampling leave the "waiting" count and are thereby replaced by fresh prompts
                waiting_ = max(0, pm.samples_on_the_fly - pm.dispatched_in_step) // n_gen
                return (pm.total_steps - pm.current_step) * pps_now - waiting_

            if pm.total_steps:
                budget = still_needed()
                if budget <= 0:
                    return [], True
                n = min(n, budget)
            batch, is_end = self.data_fetcher.get_batched_prompt(n)
            pps = self.prompts_per_step()
            for _, payload in batch:
                # the step that will consume this prompt is current_step + 1 + (prompts handed out and not yet in
                # training) // prompts_per_step; it needs the weights of the step before. Counting from the samples
                # in flight keeps the tags right when the number of policy replicas (and so the batch) changes
                waiting = max(0, pm.samples_on_the_fly - pm.dispatched_in_step) // n_gen
                payload.weight_version = pm.current_step + waiting // pps
                self.prompts_handed_out += 1
                pm.samples_on_the_fly += n_gen
            if pm.total_steps and still_needed() <= 0:
                # nothing more to hand out for now; a group dropped later reopens the budget, so the stream of a
                # job with dynamic sampling only ends with the training itself
                is_end = tp.variant != "dapo"
            retry = tp.max_retry_for_on_policy
            if retry > 0 and self.stat_invalid > retry * max(1, pm.total_steps) * pps and not self._retry_warned:
                self._retry_warned = True
                logger.warning("[Controller] %d prompt groups were dropped for lack of reward signal, more than "
                               "max_retry_for_on_policy (%d) per step on average: check the reward function",
                               self.stat_invalid, retry)
            return batch, is_end

    # ------------------------------------------------------------------ rollouts
    def put_rollouts(self, src_replica_name: str, payloads: List[RLPayload], is_end: bool,
                     metrics: Optional[Dict[str, Any]] = None) -> None:
        rollouts: List[Rollout] = []
        discarded = 0
        n_gen = max(1, self.config.rollout.n_generation)
        for p in payloads:
            if p.valid is False or not p.completions:
                # DAPO-style dynamic sampling: the whole group is dropped
                discarded += n_gen
                self.stat_invalid += 1
                if p.payload_refs:
                    PayloadTransportRegistry.handle_discarded(p.payload_refs)
                continue
            rs = payload_to_rollouts(p)
            discarded += max(0, n_gen - len(rs))
            rollouts.extend(rs)
            self.rollout_status_manager.note_adopted_version(src_replica_name, p.weight_version)
            if p.completion_token_ids:
                self.stat_completion_tokens += sum(len(c) for c in p.completion_token_ids)
            elif p.payload_refs and p.extra_info:
                self.stat_completion_tokens += sum(p.extra_info.get("completion_lengths", []))
        self.stat_samples += len(rollouts)
        if is_end:
            self.rollout_status_manager.mark_ended(src_replica_name)
        self.policy_status_manager.put_rollouts(rollouts, n_discarded=discarded)
        if is_end:
            self.policy_status_manager.try_trigger_data_fetch_and_training(rollouts_ended=True)
        if self.stat_samples and self.stat_samples % (16 * n_gen) < len(rollouts):
            logger.info("[Controller] Stat: samples=%d completion_tokens=%d pending=%d in_flight=%d filtered=%d "
                        "invalid_groups=%d elapsed=%.1fs", self.stat_samples, self.stat_completion_tokens,
                        len(self.policy_status_manager.rollout_buffer), self.policy_status_manager.samples_on_the_fly,
                        self.policy_status_manager.filtered_outdated, self.stat_invalid,
                        time.time() - self.start_time)

    def put_validation_report(self, src: str, validation_step: int, payloads: List[RLPayload], is_end: bool) -> None:
        self.validation_reports.setdefault(validation_step, []).extend(payloads)
        if is_end:
            rewards = [r for p in self.validation_reports[validation_step] for r in (p.rewards or [])]
            if rewards:
                avg = sum(rewards) / len(rewards)
                logger.info("[Controller] validation step %d: reward_mean=%.4f over %d samples", validation_step,
                            avg, len(rewards))
                self.policy_status_manager.history.append({"step": validation_step, "val/reward_mean": avg})

    def train_ack(self, replica_name: str, step: int, total_steps: int, profile_finished: bool,
                  report_data: Dict[str, Any]) -> None:
        self.policy_status_manager.train_ack(replica_name, step, total_steps, profile_finished, report_data)

    # ------------------------------------------------------------------ handshake KV (NCCL ids, IPC handles)
    def kv_put(self, key: str, value_b64: str) -> None:
        self.broker.kv_set("hs:" + key, value_b64.encode())

    def kv_get(self, key: str, timeout_s: float = 0.0) -> Optional[str]:
        if timeout_s > 0 and hasattr(self.broker, "kv_wait"):
            v = self.broker.kv_wait("hs:" + key, timeout_s)
        else:
            v = self.broker.kv_get("hs:" + key)
        return v.decode() if v is not None else None

    def kv_clear(self, key: str) -> None:
        self.broker.kv_del("hs:" + key)

    def kv_all(self) -> Dict[str, str]:
        if isinstance(self.broker, InProcessBroker):
            return {k[3:]: v[0].decode() for k, v in self.broker._kv.items() if k.startswith("hs:")}
        return {}

    # ------------------------------------------------------------------ profiling
    def set_profile(self, request: Dict[str, Any]) -> bool:
        name = request.pop("replica_name")
        return self.policy_status_manager.set_profile(name, request)

    def set_trace_path(self, replica_name: str, trace_path: str, global_rank: int) -> None:
        self.trace_paths.setdefault(replica_name, {})[global_rank] = trace_path

    # ------------------------------------------------------------------ weight-sync shard plans
    def set_shard_infos(self, role: str, infos: Dict[str, Any]) -> None:
        self.shard_infos[role] = infos

    def get_shard_infos(self, role: str) -> Optional[Dict[str, Any]]:
        return self.shard_infos.get(role)

    # ------------------------------------------------------------------ resume
    def set_resume_info(self, extra_info: Dict[str, Any]) -> None:
        """Position the prompt source after a checkpoint resume (validated against the dataset size)."""
        pm = self.policy_status_manager
        remain = extra_info.get("remain_samples_num")
        step = int(extra_info.get("step", 0))
        if remain is not None and 0 <= remain <= self.data_fetcher.total_samples:
            self.data_fetcher.restore(int(remain))
        pm.current_step = step
        pm.start_step = step
        self.data_fetcher.ckpt_extra_info = extra_info
