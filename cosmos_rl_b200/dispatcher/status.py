"""Replica lifecycle and step scheduling on the controller.

``PolicyStatusManager`` owns the rollout buffer and decides when a training step starts (every policy
replica idle and enough rollouts buffered), aggregates ``train_ack`` reports, decides weight syncs and
checkpoints, and drives the end-of-training protocol. ``RolloutStatusManager`` tracks rollout replicas,
their adopted weight versions and the end / STOP protocol. The decisions themselves are pure functions so
they can be tested without any process (cosmos_rl/dispatcher/status.py:62-192, 256-2512).
"""
from __future__ import annotations

import math
import threading
import time
from collections import deque
from typing import Any, Callable, Deque, Dict, List, Optional

import numpy as np

from ..comm.broker import StreamBroker, command_stream, rollout_stream
from ..utils import constant
from ..utils.logging import logger
from . import command as cmd
from .data.schema import Rollout
from .protocol import Role
from .replica import Atom, Replica, ReplicaStatus


# ---------------------------------------------------------------------------------------------------
# pure decisions
# ---------------------------------------------------------------------------------------------------
def need_weight_sync(*, step: int, total_steps: int, sync_weight_interval: int, validation_enabled: bool,
                     validation_freq: Optional[int]) -> bool:
    """Sync after ``step``? Every ``sync_weight_interval`` steps; with validation also on validation steps and
    on the last step (the rollout validates with those weights). Without validation the last step is never
    synced: nothing would consume those weights and the transfer would race the rollouts' shutdown."""
    need = step % max(sync_weight_interval, 1) == 0
    if validation_enabled:
        if validation_freq:
            need = need or step % validation_freq == 0
        return need or step == total_steps
    return need and step != total_steps


def should_broadcast_stop(*, n_policy: int, had_policy_replicas: bool, stop_broadcast_sent: bool,
                          validation_enabled: bool, training_finished: bool, all_rollouts_ended: bool) -> bool:
    """One-shot STOP to the rollouts: all policies gone (and there were some), the job really is over
    (finished, or every rollout reported end-of-data), no validation-driven shutdown in charge."""
    return (n_policy == 0 and had_policy_replicas and not stop_broadcast_sent and not validation_enabled
            and (training_finished or all_rollouts_ended))


def should_coalesce_skip(*, coalesce_enabled: bool, forced: bool, last_staged_step: int,
                         max_adopted_version: int) -> bool:
    """Skip this sync because an earlier one is still in flight (issued but not yet adopted by any rollout)?"""
    if not coalesce_enabled or forced:
        return False
    return last_staged_step > max_adopted_version


def rollout_is_outdated(*, consume_step: int, weight_version: int, allowed_outdated_steps: int) -> bool:
    """A rollout generated with weights ``weight_version`` and consumed by training step ``consume_step``
    (which starts from weights ``consume_step - 1``) is too stale when the gap exceeds the allowance."""
    return (consume_step - 1) - weight_version > allowed_outdated_steps


def compute_total_steps(*, n_samples: int, n_generation: int, epochs: int, global_batch: int,
                        max_num_steps: Optional[int]) -> int:
    if global_batch <= 0:
        return 0
    steps = (n_samples * epochs * max(n_generation, 1)) // global_batch
    if max_num_steps is not None and max_num_steps > 0:
        steps = min(steps, max_num_steps)
    return steps


def should_save_checkpoint(*, step: int, total_steps: int, enable: bool, save_freq: int,
                           force: bool = False) -> bool:
    if not enable:
        return False
    return force or step == total_steps or (save_freq > 0 and step % save_freq == 0)


# ---------------------------------------------------------------------------------------------------
class _ManagerBase:
    role = ""

    def __init__(self, config, broker: StreamBroker):
        self.config = config
        self.broker = broker
        self.replicas: Dict[str, Replica] = {}
        self.lock = threading.RLock()

    def publish(self, replica_name: str, command: cmd.Command) -> None:
        logger.debug("[Controller] -> %s: %r", replica_name, command)
        self.broker.publish(command_stream(replica_name), command.pack())

    def live(self) -> List[Replica]:
        return [r for r in self.replicas.values() if r.all_atoms_arrived]

    def __len__(self):
        return len(self.live())

    def __contains__(self, name):
        return name in self.replicas

    def heartbeat(self, name: str) -> bool:
        r = self.replicas.get(name)
        if r is None:
            return False
        r.heartbeat()
        return True

    def silent_replicas(self, timeout: float, now: Optional[float] = None) -> List[str]:
        return [r.name for r in self.replicas.values() if r.silent_for(now) > timeout]


# ---------------------------------------------------------------------------------------------------
class PolicyStatusManager(_ManagerBase):
    role = Role.POLICY

    def __init__(self, config, broker, data_fetcher=None, rollout_manager: "RolloutStatusManager" = None,
                 report_hooks: Optional[List[Callable]] = None):
        super().__init__(config, broker)
        self.data_fetcher = data_fetcher
        self.rollout_manager = rollout_manager
        self.report_hooks = report_hooks or []
        self.rollout_buffer: Deque[Rollout] = deque()
        self.current_step = 0
        self.total_steps = 0
        self.start_step = 0
        self.had_replicas = False
        self.mesh_built_for: tuple = ()
        self.samples_on_the_fly = 0          # rollouts handed out as prompts and not yet trained
        self.dispatched_in_step = 0
        self.last_staged_sync_step = -1
        self.filtered_outdated = 0
        self.train_reports: Dict[str, Dict[str, Any]] = {}
        self.step_rollout_stats: Dict[str, float] = {}
        self.history: List[Dict[str, Any]] = []
        self.force_save_next = False
        self.complete_sent = False
        self.step_started_at = 0.0

    # ------------------------------------------------------------------ sizes
    @property
    def n_init_replicas(self) -> int:
        return max(1, self.config.policy.parallelism.n_init_replicas)

    @property
    def batch_per_replica(self) -> int:
        return self.config.train.train_batch_per_replica

    def mesh_replicas(self) -> List[Replica]:
        return sorted([r for r in self.live() if r.in_mesh], key=lambda r: r.mesh_rank)

    @property
    def global_batch(self) -> int:
        n = len(self.mesh_replicas()) or self.n_init_replicas
        return self.batch_per_replica * n

    def n_generation(self) -> int:
        return max(1, self.config.rollout.n_generation)

    def recompute_total_steps(self) -> None:
        if self.data_fetcher is None:
            return
        tp = self.config.train.train_policy
        if tp.type != "grpo":
            return
        total = compute_total_steps(
            n_samples=self.data_fetcher.n, n_generation=self.n_generation(), epochs=self.data_fetcher.epochs,
            global_batch=self.global_batch, max_num_steps=self.config.train.max_num_steps)
        consumed = getattr(self, "samples_dispatched_total", 0)
        if consumed and self.global_batch > 0:
            # a membership change in the middle of the run: the steps already taken used a different batch, so the
            # remaining samples decide how many steps of the new size are left
            all_samples = self.data_fetcher.n * self.data_fetcher.epochs * max(self.n_generation(), 1)
            total = self.current_step + max(0, all_samples - consumed) // self.global_batch
            mx = self.config.train.max_num_steps
            if mx is not None and mx > 0:
                total = min(total, mx)
        self.total_steps = total

    def training_finished(self) -> bool:
        return self.total_steps > 0 and self.current_step >= self.total_steps and self.all_reduced()

    # ------------------------------------------------------------------ registration
    def register(self, atom: Atom, replica_name: str) -> Replica:
        with self.lock:
            rep = self.replicas.get(replica_name)
            if rep is None:
                rep = Replica(replica_name, Role.POLICY)
                self.replicas[replica_name] = rep
            rep.add_atom(atom)
            rep.heartbeat()
            if rep.all_atoms_arrived:
                self.had_replicas = True
                self._post_register(rep)
            return rep

    def _post_register(self, rep: Replica) -> None:
        loaded = [r for r in self.live() if r.weights_loaded]
        if not loaded:
            # first policy replica: it loads the weights (checkpoint or HF) itself
            self.publish(rep.name, cmd.WeightResumeCommand(rep.name))
            rep.weights_loaded = True
            rep.status = ReplicaStatus.READY
            if self.rollout_manager is not None:
                self.rollout_manager.on_policy_weights_available(self)
        live = self.live()
        if len(live) < self.n_init_replicas:
            return
        in_mesh_before = [r for r in live if r.in_mesh]
        self._build_mesh(live)
        if not in_mesh_before:
            # initial mesh: broadcast the state of the loaded replica to all others
            src = next(r for r in live if r.weights_loaded)
            others = [r for r in live if r is not src]
            if others:
                c = cmd.PolicyToPolicyBroadcastCommand(src.name, [r.name for r in live], self.total_steps)
                for r in live:
                    self.publish(r.name, c)
                for r in others:
                    r.weights_loaded = True
                    r.status = ReplicaStatus.READY
        elif not rep.weights_loaded:
            # elastic scale-up: unicast the full state to the newcomer
            src = next(r for r in in_mesh_before if r.weights_loaded)
            c = cmd.PolicyToPolicyUnicastCommand(src.name, rep.name, self.total_steps)
            self.publish(src.name, c)
            self.publish(rep.name, c)
            rep.weights_loaded = True
            rep.status = ReplicaStatus.READY
        self.recompute_total_steps()
        self.try_trigger_data_fetch_and_training()

    def _build_mesh(self, members: List[Replica]) -> None:
        members = sorted(members, key=lambda r: r.start_time)
        mapping = {r.name: i for i, r in enumerate(members)}
        key = tuple(sorted(mapping.items()))
        if key == self.mesh_built_for:
            return
        self.mesh_built_for = key
        for r in members:
            r.in_mesh = True
            r.mesh_rank = mapping[r.name]
        c = cmd.BuildMeshCommand(mapping)
        for r in members:
            self.publish(r.name, c)

    def unregister(self, replica_name: str) -> None:
        with self.lock:
            rep = self.replicas.pop(replica_name, None)
            if rep is None:
                return
            survivors = [r for r in self.live() if r.in_mesh]
            if rep.in_mesh and survivors and not self.training_finished():
                self._build_mesh(survivors)
                self.recompute_total_steps()
                self.train_reports.pop(replica_name, None)
                self._maybe_finish_step()
                # the lost replica may have been the source of a weight hand-over that no rollout replica has
                # adopted yet: the survivors hold the same weights, so stage it again from one of them
                rm = self.rollout_manager
                if rm is not None and self.last_staged_sync_step > rm.max_adopted_version() and rm.live():
                    logger.info("[Controller] re-staging the weight sync of step %d from a surviving policy replica",
                                self.last_staged_sync_step)
                    self.trigger_weight_sync(self.last_staged_sync_step)

    # ------------------------------------------------------------------ rollouts in
    def filter_outdated(self, rollouts: List[Rollout]) -> List[Rollout]:
        tp = self.config.train.train_policy
        allowed = tp.allowed_outdated_steps
        gb = max(self.global_batch, 1)
        kept = []
        dropped_refs: List[str] = []
        pending = len(self.rollout_buffer)
        for i, r in enumerate(rollouts):
            consume_step = self.current_step + 1 + (pending + len(kept)) // gb
            if rollout_is_outdated(consume_step=consume_step, weight_version=r.weight_version,
                                   allowed_outdated_steps=allowed):
                self.filtered_outdated += 1
                if r.payload_ref:
                    dropped_refs.append(r.payload_ref)
                continue
            kept.append(r)
        if dropped_refs:
            # producers free the parked tensors of rollouts that will never be trained
            from ..utils.payload_transport import PayloadTransportRegistry
            try:
                PayloadTransportRegistry.handle_discarded(dropped_refs)
            except Exception as e:
                logger.warning("[Controller] releasing %d discarded payloads failed: %s", len(dropped_refs), e)
        return kept

    def put_rollouts(self, rollouts: List[Rollout], n_discarded: int = 0) -> None:
        with self.lock:
            kept = self.filter_outdated(rollouts)
            dropped = len(rollouts) - len(kept) + n_discarded
            if dropped:
                # samples that will never be trained no longer count as in flight
                self.samples_on_the_fly = max(0, self.samples_on_the_fly - dropped)
            self.rollout_buffer.extend(kept)
            self.try_trigger_data_fetch_and_training()

    # ------------------------------------------------------------------ step scheduling
    def all_ready(self) -> bool:
        reps = self.mesh_replicas()
        return bool(reps) and all(r.status in (ReplicaStatus.READY, ReplicaStatus.REDUCED) and r.weights_loaded
                                  for r in reps)

    def all_reduced(self) -> bool:
        reps = self.mesh_replicas()
        return all(r.status != ReplicaStatus.RUNNING for r in reps)

    def try_trigger_data_fetch_and_training(self, rollouts_ended: bool = False) -> bool:
        with self.lock:
            reps = self.mesh_replicas()
            # the job starts when all of its initial replicas arrived; once it runs, a smaller membership (a replica
            # was reaped) keeps training with the survivors
            if not reps or not self.all_ready():
                return False
            if len(self.live()) < self.n_init_replicas and not getattr(self, "_started", False):
                return False
            if self.total_steps and self.current_step >= self.total_steps:
                return False
            need = self.batch_per_replica * len(reps)
            if len(self.rollout_buffer) < need:
                if rollouts_ended or (self.rollout_manager is not None and self.rollout_manager.all_ended()):
                    self._send_training_complete()
                return False
            self.current_step += 1
            self._started = True
            self.step_started_at = time.time()
            batch = [self.rollout_buffer.popleft() for _ in range(need)]
            self._record_rollout_stats(batch)
            self.dispatched_in_step = need
            self.samples_dispatched_total = getattr(self, "samples_dispatched_total", 0) + need
            for i, r in enumerate(batch):
                rep = reps[i % len(reps)]
                self.broker.publish(rollout_stream(rep.name), r.model_dump_json().encode())
            ck = self.config.train.ckpt
            do_save = should_save_checkpoint(step=self.current_step, total_steps=self.total_steps,
                                             enable=ck.enable_checkpoint, save_freq=ck.save_freq,
                                             force=self.force_save_next)
            self.force_save_next = False
            remain = self.data_fetcher.remain_samples_num if self.data_fetcher is not None else 0
            self.train_reports = {}
            for rep in reps:
                prof = rep.pending_profile or {}
                c = cmd.DataFetchCommand(rep.name, self.batch_per_replica, self.current_step, self.total_steps,
                                         remain_samples_num=remain, do_save=do_save,
                                         do_profile=bool(prof), **{k: v for k, v in prof.items()})
                rep.status = ReplicaStatus.RUNNING
                self.publish(rep.name, c)
            return True

    def _send_training_complete(self) -> None:
        if self.complete_sent:
            return
        self.complete_sent = True
        ck = self.config.train.ckpt
        for rep in self.mesh_replicas():
            self.publish(rep.name, cmd.TrainingCompleteCommand(
                rep.name, self.current_step + 1, self.total_steps, final_step=self.current_step,
                do_save=ck.enable_checkpoint))
        # the job will run no further step: make "finished" observable
        self.total_steps = self.current_step

    def _record_rollout_stats(self, batch: List[Rollout]) -> None:
        rewards = np.array([r.reward for r in batch], dtype=np.float64)
        adv = np.array([r.advantage for r in batch], dtype=np.float64)
        lens = np.array([len(r.completion_token_ids) if r.completion_token_ids else
                         (len(r.completion) if isinstance(r.completion, (str, list)) else 0) for r in batch])
        stale = np.array([max(0, self.current_step - 1 - r.weight_version) for r in batch])
        self.step_rollout_stats = {
            "train/reward_mean": float(rewards.mean()), "train/reward_std": float(rewards.std()),
            "train/reward_max": float(rewards.max()), "train/reward_min": float(rewards.min()),
            "rollout/completion_length_mean": float(lens.mean()), "rollout/completion_length_max": float(lens.max()),
            "rollout/advantage_mean": float(adv.mean()), "rollout/advantage_abs_mean": float(np.abs(adv).mean()),
            "rollout/weight_staleness_p50": float(np.percentile(stale, 50)),
            "rollout/weight_staleness_p99": float(np.percentile(stale, 99)),
            "rollout/weight_staleness_max": float(stale.max()),
        }

    # ------------------------------------------------------------------ train ack
    def train_ack(self, replica_name: str, step: int, total_steps: int, profile_finished: bool,
                  report_data: Dict[str, Any]) -> None:
        with self.lock:
            rep = self.replicas.get(replica_name)
            if rep is None:
                return
            rep.status = ReplicaStatus.REDUCED
            rep.acked_step = step
            rep.weight_step = step
            if profile_finished:
                rep.pending_profile = None
            self.train_reports[replica_name] = report_data or {}
            self._maybe_finish_step()

    def _maybe_finish_step(self) -> None:
        reps = self.mesh_replicas()
        if not reps or any(r.status == ReplicaStatus.RUNNING for r in reps):
            return
        if not all(r.name in self.train_reports for r in reps):
            return
        step = self.current_step
        self.samples_on_the_fly = max(0, self.samples_on_the_fly - self.dispatched_in_step)
        self.dispatched_in_step = 0
        report = self._aggregate_reports(list(self.train_reports.values()))
        report.update(self.step_rollout_stats)
        report["train/step_wall_time"] = time.time() - self.step_started_at
        self.history.append({"step": step, **report})
        if step % max(1, self.config.logging.log_interval) == 0:
            logger.info("[Controller] step %d/%d: %s", step, self.total_steps,
                        ", ".join(f"{k}={v:.4g}" for k, v in sorted(report.items()) if isinstance(v, (int, float))))
        for hook in self.report_hooks:
            try:
                hook(report, step)
            except Exception as e:  # a logging hook must never take the job down
                logger.warning("report hook failed: %s", e)
        self.train_reports = {}
        val = self.config.validation
        forced = bool(val.enable and val.freq and step % val.freq == 0)
        if need_weight_sync(step=step, total_steps=self.total_steps,
                            sync_weight_interval=self.config.train.sync_weight_interval,
                            validation_enabled=val.enable, validation_freq=val.freq):
            adopted = self.rollout_manager.max_adopted_version() if self.rollout_manager else step
            if not should_coalesce_skip(coalesce_enabled=self.config.train.coalesce_weight_sync, forced=forced,
                                        last_staged_step=self.last_staged_sync_step, max_adopted_version=adopted):
                self.trigger_weight_sync(step)
        if self.total_steps and step >= self.total_steps:
            logger.info("[Controller] training finished at step %d", step)
            return
        self.try_trigger_data_fetch_and_training()

    @staticmethod
    def _aggregate_reports(reports: List[Dict[str, Any]]) -> Dict[str, Any]:
        out: Dict[str, Any] = {}
        keys = set().union(*[r.keys() for r in reports]) if reports else set()
        for k in keys:
            vals = [r[k] for r in reports if isinstance(r.get(k), (int, float))]
            if not vals:
                continue
            out[k] = max(vals) if k.endswith("_max") or k.endswith("iteration_time") else sum(vals) / len(vals)
        return out

    def trigger_weight_sync(self, step: int) -> None:
        if self.rollout_manager is None:
            return
        srcs = self.mesh_replicas()
        if not srcs:
            return
        self.last_staged_sync_step = step
        self.rollout_manager.sync_from_policy(srcs[0], step, self.total_steps, trainable_only=True)

    def set_profile(self, replica_name: str, request: Dict[str, Any]) -> bool:
        rep = self.replicas.get(replica_name)
        if rep is None:
            return False
        rep.pending_profile = request
        return True


# ---------------------------------------------------------------------------------------------------
class RolloutStatusManager(_ManagerBase):
    role = Role.ROLLOUT

    def __init__(self, config, broker):
        super().__init__(config, broker)
        self.policy_manager: Optional[PolicyStatusManager] = None
        self.had_replicas = False
        self.left_after_end = 0
        self.ended: set = set()
        self.stop_broadcast_sent = False
        self.adopted_versions: Dict[str, int] = {}
        self.mesh_built_for: tuple = ()
        self.total_completion_tokens = 0
        self.total_samples = 0

    @property
    def n_init_replicas(self) -> int:
        return max(1, self.config.rollout.parallelism.n_init_replicas)

    def register(self, atom: Atom, replica_name: str) -> Replica:
        with self.lock:
            rep = self.replicas.get(replica_name)
            if rep is None:
                rep = Replica(replica_name, Role.ROLLOUT)
                self.replicas[replica_name] = rep
            rep.add_atom(atom)
            rep.heartbeat()
            if rep.all_atoms_arrived:
                self.had_replicas = True
                self._post_register(rep)
            return rep

    def _policy_source(self) -> Optional[Replica]:
        if self.policy_manager is None:
            return None
        return next((r for r in self.policy_manager.live() if r.weights_loaded), None)

    def _post_register(self, rep: Replica) -> None:
        live = self.live()
        if len(live) >= self.n_init_replicas:
            self._build_mesh(live)
        src = self._policy_source()
        if src is None:
            return  # weights arrive once a policy replica has loaded them
        step = self.policy_manager.current_step if self.policy_manager else 0
        total = self.policy_manager.total_steps if self.policy_manager else 0
        loaded = [r for r in live if r.weights_loaded]
        if not loaded or self.config.b200.peer_weight_sync:
            self._p2r(src, rep, step, total, trainable_only=False)
        if len(live) >= self.n_init_replicas:
            self._r2r(step, total, trainable_only=False)

    def on_policy_weights_available(self, policy_manager: PolicyStatusManager) -> None:
        """Called when the first policy replica has its weights: serve the rollouts that were waiting."""
        self.policy_manager = policy_manager
        with self.lock:
            live = self.live()
            src = self._policy_source()
            if not live or src is None:
                return
            targets = live if self.config.b200.peer_weight_sync else live[:1]
            for r in targets:
                if not r.weights_loaded:
                    self._p2r(src, r, policy_manager.current_step, policy_manager.total_steps, trainable_only=False)
            if len(live) >= self.n_init_replicas:
                self._r2r(policy_manager.current_step, policy_manager.total_steps, trainable_only=False)

    def _build_mesh(self, members: List[Replica]) -> None:
        members = sorted(members, key=lambda r: r.start_time)
        mapping = {r.name: i for i, r in enumerate(members)}
        key = tuple(sorted(mapping.items()))
        if key == self.mesh_built_for:
            return
        self.mesh_built_for = key
        for r in members:
            r.in_mesh, r.mesh_rank = True, mapping[r.name]
        c = cmd.BuildMeshCommand(mapping)
        for r in members:
            self.publish(r.name, c)

    def _p2r(self, src: Replica, dst: Replica, step: int, total: int, trainable_only: bool) -> None:
        first = not getattr(dst, "sync_checked", False)
        dst.sync_checked = True
        c = cmd.PolicyToRolloutUnicastCommand(src.name, dst.name, src.n_gpus, dst.n_gpus, weight_step=step,
                                              total_steps=total, trainable_only=trainable_only,
                                              do_weight_sync_check=bool(first and constant.COSMOS_WEIGHT_SYNC_CHECK))
        self.publish(src.name, c)
        self.publish(dst.name, c)
        dst.weights_loaded = True
        dst.status = ReplicaStatus.READY

    def _r2r(self, step: int, total: int, trainable_only: bool) -> None:
        members = [r for r in self.live() if r.in_mesh and r.name not in self.ended]
        src = next((r for r in members if r.weights_loaded), None)
        if src is None:
            return
        c = cmd.RolloutToRolloutBroadcastCommand(src.name, [r.name for r in members], weight_step=step,
                                                 total_steps=total, trainable_only=trainable_only)
        for r in members:
            self.publish(r.name, c)
            r.weights_loaded = True
            r.status = ReplicaStatus.READY

    def sync_from_policy(self, src: Replica, step: int, total: int, trainable_only: bool) -> None:
        """One weight-sync round after training step ``step``. With peer-memory sync every rollout replica
        pulls from the policy in parallel (NVSwitch gives each pair full bandwidth) and the broadcast command
        only commits the new version; otherwise replica 0 receives and fans out."""
        with self.lock:
            members = [r for r in self.live() if r.name not in self.ended]
            if not members:
                return
            targets = members if self.config.b200.peer_weight_sync else members[:1]
            for r in targets:
                self._p2r(src, r, step, total, trainable_only)
            self._r2r(step, total, trainable_only)

    def unregister(self, name: str) -> None:
        with self.lock:
            rep = self.replicas.pop(name, None)
            if name in self.ended:
                self.left_after_end += 1        # it had reported the end of its prompt stream: a regular exit
            self.ended.discard(name)
            if rep is not None and rep.in_mesh:
                survivors = [r for r in self.live() if r.in_mesh]
                if survivors:
                    self._build_mesh(survivors)

    # ------------------------------------------------------------------ end / stop protocol
    def mark_ended(self, name: str) -> None:
        with self.lock:
            self.ended.add(name)

    def all_ended(self) -> bool:
        """Every rollout replica has reported the end of its prompt stream. Replicas that reported it and then left
        count too: with nobody left to generate, a policy whose buffer runs short of a step (rollouts dropped as
        outdated, say) must be told that training is over instead of waiting for data that will never come."""
        live = self.live()
        if live:
            return all(r.name in self.ended for r in live)
        return self.left_after_end > 0

    def note_adopted_version(self, name: str, version: int) -> None:
        self.adopted_versions[name] = max(version, self.adopted_versions.get(name, -1))

    def max_adopted_version(self) -> int:
        return max(self.adopted_versions.values(), default=-1)

    def maybe_broadcast_stop(self, policy_manager: PolicyStatusManager) -> bool:
        with self.lock:
            if should_broadcast_stop(n_policy=len(policy_manager.replicas), had_policy_replicas=policy_manager.had_replicas,
                                     stop_broadcast_sent=self.stop_broadcast_sent,
                                     validation_enabled=self.config.validation.enable,
                                     training_finished=policy_manager.training_finished(),
                                     all_rollouts_ended=self.all_ended()):
                self.stop_broadcast_sent = True
                for r in list(self.replicas.values()):
                    self.publish(r.name, cmd.StopCommand(r.name))
                return True
            return False
