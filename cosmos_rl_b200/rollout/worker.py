"""Rollout control worker: the producer side of the asynchronous loop
(cosmos_rl/rollout/worker/rollout_control.py:129-2936).

Main loop: consume commands (weight sync, mesh, stop) -> fetch prompts from the controller (rank 0, then
broadcast / scatter) -> hold back while the head prompt asks for weights newer than
``current_weight_version + allowed_outdated_steps`` -> generate -> hand completions to the reward pool ->
report finished payloads. The end of the prompt stream (``is_end``) and the STOP command both lead to an
orderly exit.
"""
from __future__ import annotations

import queue
import threading
import time
from typing import Any, Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from ..comm.base import CommMixin
from ..data.packer import BaseDataPacker
from ..dispatcher import command as cmd
from ..dispatcher.data import CosmosDataset, WorkerDataFetcher
from ..dispatcher.data.schema import RLPayload
from ..dispatcher.protocol import Role
from ..parallel.dims import ParallelDims
from ..parallel.reshard import build_plan, model_parts, shard_info
from ..reward.dispatcher import RewardDispatcher, make_reward_calculator
from ..utils import constant
from ..utils.logging import logger
from .base import RolloutRegistry
from . import (b200_rollout, diffusion_rollout, hf_rollout, openvla_rollout, vla_flow_rollout,  # noqa: F401
               vla_rollout)                               # (registers the built-in backends)


class DisaggregatedRolloutControlWorker(CommMixin):
    role = Role.ROLLOUT

    def __init__(self, config, parallel_dims: ParallelDims, dataset=None, val_dataset=None, data_packer=None,
                 val_data_packer=None, reward_fns=None, filter_reward_fns=None, val_reward_fns=None, api=None,
                 device=None, tokenizer=None, **kw):
        self.config = config
        self.parallel_dims = parallel_dims
        self.device = device or parallel_dims.device
        self.init_comm(api)
        ds = CosmosDataset.wrap(dataset, config)
        vds = CosmosDataset.wrap(val_dataset, config)
        self.data_fetcher = WorkerDataFetcher(config, ds, vds)
        self.tokenizer = tokenizer
        backend = config.rollout.backend
        if backend == "b200":
            # families without a native model are served by the generic transformers wrapper and its backend
            from ..models import hf_io
            from ..models.base import ModelRegistry
            mtype = hf_io.load_hf_config(config.policy.model_name_or_path, config.custom.get("model_config")).get("model_type")
            cls = ModelRegistry.get(mtype)
            if cls.__name__ == "HFModel":
                backend = "hf"
            elif not getattr(cls, "paged_engine", True):
                backend = "recompute"      # native family without a paged-attention path in the engine
        self.rollout = RolloutRegistry.get(backend)(config, parallel_dims, self.device, tokenizer=tokenizer)
        self.rollout.init_engine(load_format="dummy", seed=(config.rollout.seed or 0) + hash(self.replica_name) % 9973)
        mt = getattr(self.rollout.model.args, "model_type", "hfmodel")
        self.data_packer = data_packer or BaseDataPacker.get_default(mt)()
        self.data_packer.setup(config, tokenizer)
        self.reward_dispatcher = RewardDispatcher(make_reward_calculator(config, reward_fns, filter_reward_fns))
        self.val_reward_dispatcher = RewardDispatcher(
            make_reward_calculator(config, val_reward_fns or reward_fns, validation=True))
        self.current_weight_version = -1
        self.weights_ready = False
        self.prompt_queue: List[Tuple[int, RLPayload]] = []
        self.prompt_end = False
        self.stopped = False
        self.scheduler = None          # RolloutTaskScheduler when rollout.mode == "async"
        self.total_steps: Optional[int] = None
        self.batch_size = config.rollout.batch_size
        self.handlers = cmd.RolloutCommandRegistry()
        for c, h in ((cmd.BuildMeshCommand, self.execute_build_mesh),
                     (cmd.PolicyToRolloutUnicastCommand, self.policy_to_rollout_unicast),
                     (cmd.RolloutToRolloutBroadcastCommand, self.rollout_to_rollout_broadcast),
                     (cmd.StopCommand, self.execute_stop)):
            self.handlers.register(c, h)
        self.mesh: Dict[str, int] = {}
        self.p2r_comms: Dict[str, Any] = {}
        self.peer_sync = None
        self.recv_plan = None
        self.r2r_comm = None
        self.stats = {"generated_tokens": 0, "batches": 0, "sync_ms": []}
        self.post_shard_infos()

    # ------------------------------------------------------------------ shard infos
    def post_shard_infos(self) -> None:
        if self.rollout.flat is None:
            return
        info = shard_info(self.global_rank, model_parts(self.rollout.model, self.rollout.flat), self.rollout.flat.total)
        infos = [None] * self.world_size
        if self.world_size > 1:
            dist.all_gather_object(infos, info)
        else:
            infos = [info]
        self.my_shard_info = info
        if self.global_rank == 0:
            self.api.post_shard_infos("rollout", {"ranks": infos, "replica": self.replica_name})

    # ------------------------------------------------------------------ command handlers
    def execute_build_mesh(self, c: cmd.BuildMeshCommand) -> bool:
        self.mesh = dict(c.replica_name_to_rank)
        return False

    def execute_stop(self, c: cmd.StopCommand) -> bool:
        self.stopped = True
        return True

    def _policy_infos(self):
        return self.api.get_shard_infos("policy")

    def policy_to_rollout_unicast(self, c: cmd.PolicyToRolloutUnicastCommand) -> bool:
        if c.dst_replica_name != self.replica_name:
            return False
        t0 = time.perf_counter()
        key = f"p2r:{c.uuid_value}"
        peer = self._pair_transport(c) == "peer"
        check = None
        if getattr(c, "do_weight_sync_check", False) and getattr(self.rollout, "flat", None) is not None \
                and not c.trainable_only:
            from ..utils.debug import WeightSyncCheck
            check = WeightSyncCheck(self.rollout.flat.data, slots=self.rollout.flat.slots)
        try:
            if peer:
                self._peer_pull(c, key)
            else:
                self._collective_recv(c)
        except (RuntimeError, TimeoutError) as e:
            # the sending policy replica went away mid-transfer: drop the communicator that spans it and keep the
            # current weights; the controller stages the hand-over again from a surviving replica
            logger.warning("[Rollout] weight hand-over of step %s from %s failed (%s); keeping weight version %d",
                           c.weight_step, c.src_replica_name, str(e).splitlines()[0][:200], self.current_weight_version)
            pair = f"p2r-{c.src_replica_name}-{c.dst_replica_name}"
            comm = self.p2r_comms.pop(pair, None)
            if comm is not None:
                try:
                    comm.abort()
                except Exception:
                    pass
            self.recv_plan = None
            return False
        if check is not None:
            if self.device.type == "cuda":
                torch.cuda.synchronize()
            self.stats["sync_check"] = check.finish()
        self.weights_ready = True
        self._pending_version = c.weight_step if c.weight_step is not None else 0
        self.total_steps = c.total_steps
        self.stats["sync_ms"].append((time.perf_counter() - t0) * 1e3)
        logger.info("[Rollout] weights of step %s received: transport=%s, %.1f ms, device %s", c.weight_step,
                    "peer" if peer else "collective", self.stats["sync_ms"][-1], self.device)
        return False

    def _pair_transport(self, c) -> str:
        """Choose how the weights of this (policy replica, rollout replica) pair travel: "peer" (this replica reads the
        policy's buffers through CUDA IPC mappings) needs every policy rank's buffer exported and on this machine,
        for every rank of this replica; otherwise "collective" (send / recv over the pair's communicator, which also
        crosses machines). Decided once per pair and announced to the policy under ``p2r-mode:<src>:<dst>``."""
        pair = f"p2r-mode:{c.src_replica_name}:{c.dst_replica_name}"
        cache = self.__dict__.setdefault("_pair_modes", {})
        if pair in cache:
            return cache[pair]
        from ..utils.dist_util import host_id
        pol, deadline = self._policy_infos(), time.time() + 600
        while pol is None:                              # the policy posts them when it takes up the same command
            if time.time() > deadline:
                raise TimeoutError("the policy replica never posted its shard infos")
            time.sleep(0.02)
            pol = self._policy_infos()
        exported = all("ipc_handle" in i for i in pol["ranks"])
        if not exported:
            cache[pair] = "collective"                  # the policy serves no buffers: it does not wait for a choice
            return cache[pair]
        mine = bool(self.config.b200.peer_weight_sync and self.device.type == "cuda"
                    and all(i.get("host") == host_id() for i in pol["ranks"]))
        if self.world_size > 1:
            votes = [None] * self.world_size
            dist.all_gather_object(votes, mine)
            mine = all(votes)
        cache[pair] = "peer" if mine else "collective"
        if self.global_rank == 0:
            self.broker.kv_set(pair, cache[pair].encode(), ttl_s=7 * 24 * 3600)
        return cache[pair]

    def _peer_pull(self, c, key: str) -> None:
        from ..parallel.peer import PeerMapping
        from .weight_sync import PeerWeightSync
        deadline = time.time() + 600
        while not self.broker.kv_get(key + ":ready"):
            if time.time() > deadline:
                raise TimeoutError(f"policy never announced weights for {key}")
            time.sleep(0.005)
        if self.peer_sync is None:
            infos = self.api.get_shard_insts("rollout", self.global_rank)  # plan rows
            pol = self._policy_infos()
            ptrs, self._peer_maps = {}, []
            for info in pol["ranks"]:
                m = PeerMapping(info["ipc_handle"], info["nbytes"], self.device)
                self._peer_maps.append(m)
                ptrs[info["rank"]] = m.ptr
            self.peer_sync = PeerWeightSync(self.rollout.flat.data, infos, ptrs, fp8=getattr(self.rollout, "fp8", None),
                                          dst_rank=self.global_rank)
        self.peer_sync.pull()
        torch.cuda.synchronize()
        from ..ops import native
        native.read_status(self.device)
        self.broker.kv_set(f"{key}:done:{self.global_rank}", b"1", ttl_s=3600)

    def _collective_recv(self, c) -> None:
        from ..parallel.dyncomm import create_comm
        from ..utils.misc import str2dtype
        pair = f"p2r-{c.src_replica_name}-{c.dst_replica_name}"
        comm = self.p2r_comms.get(pair)
        P = c.src_replica_size
        if comm is None or comm.aborted:
            comm = create_comm(self.api, f"{pair}-{c.uuid_value}" if comm is not None else pair,
                               P + self.global_rank, P + c.dst_replica_size, self.device, is_initiator=False)
            self.p2r_comms[pair] = comm
        if self.recv_plan is None:
            self.recv_plan = self.api.get_shard_insts("rollout", self.global_rank)
        flat = self.rollout.flat.data
        tdt = str2dtype(self.config.train.transfer_dtype) if self.device.type == "cuda" else flat.dtype
        from ..parallel.dyncomm import watchdog
        with watchdog(wait_stream=True):                 # the receives are enqueues; bound the device side too
            for d in self.recv_plan:
                buf = torch.empty(d[5], d[6], dtype=tdt, device=self.device)
                comm.recv(buf, d[0])
                torch.as_strided(flat, (d[5], d[6]), (d[4], 1), flat.storage_offset() + d[3]).copy_(buf)
        if getattr(self.rollout, "fp8", None) is not None:
            self.rollout.fp8.quantize_local()      # no in-flight quantisation on this route: second pass

    def rollout_to_rollout_broadcast(self, c: cmd.RolloutToRolloutBroadcastCommand) -> bool:
        """Commit a weight version. With peer sync every replica has already pulled its own copy, so this
        carries no data; otherwise the source replica broadcasts its parameters to the others."""
        if self.replica_name not in c.dst_replica_names:
            return False
        peer = bool(self.config.b200.peer_weight_sync and self.device.type == "cuda")
        if not peer and len(c.dst_replica_names) > 1:
            self._r2r_data(c)
        if c.weight_step is not None:
            self.current_weight_version = c.weight_step
        else:
            self.current_weight_version = getattr(self, "_pending_version", 0)
        self.weights_ready = True
        logger.info("[Rollout] weight version %d committed", self.current_weight_version)
        engine = getattr(self.rollout, "engine", None)      # backends without a token engine (diffusion, action flows)
        if engine is not None:
            engine.weight_version = self.current_weight_version
        if c.total_steps is not None:
            self.total_steps = c.total_steps
        return bool(c.replica_should_stop())

    def _r2r_data(self, c) -> None:
        from ..parallel.dyncomm import create_comm
        names = sorted(c.dst_replica_names, key=lambda n: self.mesh.get(n, 0))
        rank = names.index(self.replica_name)
        key = f"r2r-{'-'.join(n[:8] for n in names)}-r{self.global_rank}"
        if self.r2r_comm is None or self.r2r_comm.aborted or self.r2r_comm.size != len(names):
            self.r2r_comm = create_comm(self.api, key + f"-{c.uuid_value}", rank, len(names), self.device,
                                        is_initiator=rank == 0)
        src = names.index(c.src_replica_name)
        from ..parallel.dyncomm import watchdog
        with watchdog(wait_stream=True):
            self.r2r_comm.broadcast(self.rollout.flat.data, src)

    # ------------------------------------------------------------------ prompts
    def request_new_prompts(self, n: int, validation_step: Optional[int] = None) -> None:
        batch, is_end = [], False
        if self.global_rank == 0:
            batch, is_end = self.api.get_next_prompt(n, validation_step=validation_step)
            for _, p in batch:
                self.data_fetcher.fill(p, validation=validation_step is not None)
        if self.world_size > 1:
            box = [([(i, p.model_dump()) for i, p in batch], is_end)]
            dist.broadcast_object_list(box, src=0)
            raw, is_end = box[0]
            batch = [(i, RLPayload.model_validate(p)) for i, p in raw]
        self.prompt_queue.extend(batch)
        if is_end:
            self.prompt_end = True

    def consume_commands(self, block: float = 0.0) -> bool:
        """Run every queued command; True when one of them asks the loop to stop."""
        stop = False
        while True:
            c = self.next_command(timeout=block)
            block = 0.0
            if c is None:
                return stop
            h = self.handlers.get_command_handler(c)
            if h is not None:
                if self.scheduler is not None:          # async mode: no engine call while weights or the mesh change
                    with self.scheduler.paused():
                        stop = bool(h(c)) or stop
                else:
                    stop = bool(h(c)) or stop

    def report_rollouts(self, block: bool = False, is_end: bool = False) -> None:
        done = self.reward_dispatcher.dequeue(block=block and not self.reward_dispatcher.is_empty())
        if self.global_rank != 0:
            return
        if done and self._payload_transport() is not None:
            from ..utils.payload_transport import park_payload
            for p in done:
                park_payload(self._payload_tx, p, self.device if self.device.type == "cuda" else None)
        if done or is_end:
            self.api.post_rollout_completion(self.replica_name, done, is_end=is_end,
                                             metrics={"generated_tokens": self.stats["generated_tokens"]})

    def _payload_transport(self):
        """The transport per-token data of finished rollouts is parked with (``[custom] payload_transfer``); None for
        the inline default."""
        if not hasattr(self, "_payload_tx"):
            from ..utils.payload_transport import PayloadTransportRegistry, get_payload_transfer_mode
            mode = get_payload_transfer_mode(self.config)
            self._payload_tx = None
            if mode != "broker":
                tx = type(PayloadTransportRegistry.get(mode))()          # an instance of this worker's own
                tx.setup(self.config, self.broker, self.device, owner=f"{self.replica_name[:12]}-r{self.global_rank}")
                self._payload_tx = tx
                logger.info("[Rollout] per-token data of rollouts travels by the %r payload transport", mode)
        return self._payload_tx

    # ------------------------------------------------------------------ generation
    def one_step_generation(self) -> None:
        n = min(self.batch_size, len(self.prompt_queue))
        batch = self.prompt_queue[:n]
        del self.prompt_queue[:n]
        payloads = [p for _, p in batch]
        results = self.rollout.rollout_generation(payloads, self.data_packer, self.data_fetcher)
        self._finish_generation(payloads, results, self.current_weight_version)

    def _finish_generation(self, payloads, results, weight_version: int) -> None:
        """Results into payloads, teacher requests, reward queue."""
        reporter = self.parallel_dims.tp_coord == 0 and self.parallel_dims.pp_coord == self.parallel_dims.pp - 1
        for p, r in zip(payloads, results):
            p.completions = r.completions
            p.completed_conversations = r.completed_conversations      # multi-turn paths (None otherwise)
            if r.extra_info is not None:
                p.extra_info = r.extra_info
            if r.completion_token_ids is not None:
                p.completion_token_ids = [[[t] for t in toks] for toks in r.completion_token_ids]
                if self.config.train.train_policy.collect_rollout_logprobs or \
                        self.config.train.train_policy.use_rollout_logprobs_for_loss:
                    p.completion_logprobs = [[[l] for l in lps] for lps in r.completion_logprobs]
                self.stats["generated_tokens"] += sum(len(t) for t in r.completion_token_ids)
            p.cumulative_logprob = r.cumulative_logprob
            p.weight_version = weight_version
            if self.config.distillation.enable and r.completion_token_ids is not None and reporter:
                # on-policy distillation: the teacher scores every sampled completion; the policy fetches the result
                # by uuid when it trains on the rollout (cosmos_rl/rollout/worker/rollout_control.py teacher requests)
                from ..reference.teacher_worker import submit_teacher_request
                prompt_ids = list(self.data_packer.get_rollout_input(p.prompt))
                p.teacher_result_uuids = [submit_teacher_request(self.broker, prompt_ids + list(toks), len(prompt_ids))
                                          for toks in r.completion_token_ids]
        self.stats["batches"] += 1
        if reporter:
            self.reward_dispatcher.enqueue_rewards_cal(payloads)

    # ------------------------------------------------------------------ asynchronous generation
    def _start_scheduler(self) -> None:
        from .task_scheduler import RolloutTaskScheduler

        def generate(payloads, is_validation):
            version = self.current_weight_version        # fixed for the batch: updates wait in scheduler.paused()
            results = self.rollout.rollout_generation(list(payloads), self.data_packer, self.data_fetcher)
            return [(r, version) for r in results]

        self.scheduler = RolloutTaskScheduler(generate, self.config.rollout.async_config.max_concurrent_requests)
        self.scheduler.start()

    def _async_step(self, allowed: int) -> bool:
        """Feed the scheduler, collect what finished. Returns False when there was nothing to do."""
        from .task_scheduler import RolloutTask
        sch = self.scheduler
        fed = 0
        while self.prompt_queue and sch.pending() < 2 * sch.max_batch:
            idx, payload = self.prompt_queue[0]
            if payload.weight_version > self.current_weight_version + allowed:
                break                                     # weight-version gate, as in the synchronous loop
            self.prompt_queue.pop(0)
            sch.put_rollout(RolloutTask(idx, payload))
            fed += 1
        done = sch.get_all()
        ok = [c for c in done if c.error is None]
        for c in done:
            if c.error is not None:
                logger.error("[Rollout] payload %s dropped after a generation error: %s", c.idx, c.error)
        by_version = {}
        for c in ok:
            by_version.setdefault(c.result[1], []).append(c)
        for version, cs in by_version.items():
            self._finish_generation([c.payload for c in cs], [c.result[0] for c in cs], version)
        return bool(fed or done)

    def main_loop(self) -> None:
        self.start_command_thread()
        allowed = getattr(self.config.train.train_policy, "allowed_outdated_steps", 0)
        if self.config.rollout.mode == "async":
            if self.world_size > 1:
                logger.warning("[Rollout] rollout.mode = 'async' needs single-GPU rollout replicas (the ranks of a "
                               "replica generate in lockstep): running synchronously")
            else:
                self._start_scheduler()
        while self.scheduler is not None and not self.shutdown_signal.is_set():
            if self.consume_commands(block=0.05 if not self.weights_ready else 0.0) or self.stopped:
                break
            if not self.weights_ready:
                continue
            if not self.prompt_queue and not self.prompt_end:
                self.request_new_prompts(self.batch_size)
            busy = self._async_step(allowed)
            self.report_rollouts()
            if not self.prompt_queue and self.prompt_end and self.scheduler.is_idle() \
                    and self.scheduler.done.empty() and self.reward_dispatcher.is_empty():
                break
            if not busy:
                time.sleep(constant.COSMOS_WEIGHT_GATE_SLEEP)
        if self.scheduler is not None:
            self.scheduler.stop(wait_for_queue=not self.stopped)
            self._async_step(allowed)
            st = self.scheduler.stats
            logger.info("[Rollout] async scheduler: %d payloads in %d engine calls, %.1f s generating, %d errors",
                        st["tasks"], st["batches"], st["busy_s"], st["errors"])
            self.report_rollouts(block=True, is_end=True)
            self._serve_parked_payloads()
            self.handle_shutdown()
            return
        while not self.shutdown_signal.is_set():
            if self.consume_commands(block=0.05 if not self.weights_ready else 0.0) or self.stopped:
                break
            if not self.weights_ready:
                continue
            if not self.prompt_queue and not self.prompt_end:
                self.request_new_prompts(self.batch_size)
            if not self.prompt_queue:
                self.report_rollouts()
                if self.prompt_end and self.reward_dispatcher.is_empty():
                    break
                time.sleep(constant.COSMOS_WEIGHT_GATE_SLEEP)
                continue
            # weight-version gate: never run further ahead of training than the allowed staleness
            head_version = self.prompt_queue[0][1].weight_version
            if head_version > self.current_weight_version + allowed:
                self.report_rollouts()
                time.sleep(constant.COSMOS_WEIGHT_GATE_SLEEP)
                continue
            self.one_step_generation()
            self.report_rollouts()
        # drain: finish rewards, report the end of this replica's stream
        self.report_rollouts(block=True, is_end=True)
        self._serve_parked_payloads()
        self.handle_shutdown()

    work = main_loop

    def _serve_parked_payloads(self) -> None:
        """With a pull-based payload transport the per-token data of reported rollouts still sits on this worker:
        keep answering fetches (and commands) until every parked buffer was fetched or released, the controller stops
        the replica, or ``[custom] payload_drain_timeout`` seconds have passed."""
        tx = getattr(self, "_payload_tx", None)
        reg = getattr(tx, "registry", None)
        if reg is None or self.stopped:
            return
        limit = float((self.config.custom or {}).get("payload_drain_timeout", 600.0))
        t0 = time.time()
        while len(reg) and time.time() - t0 < limit and not self.shutdown_signal.is_set():
            if self.consume_commands(block=0.05) or self.stopped:
                break
        if len(reg):
            logger.warning("[Rollout] leaving with %d parked payloads that nobody fetched", len(reg))

    def handle_shutdown(self) -> None:
        if getattr(self, "_shut", False):
            return
        self._shut = True
        self.shutdown_signal.set()
        self.reward_dispatcher.shutdown()
        self.val_reward_dispatcher.shutdown()
        for c in self.p2r_comms.values():
            c.abort()
        if self.r2r_comm is not None:
            self.r2r_comm.abort()
        for m in getattr(self, "_peer_maps", []):
            m.close()
        if getattr(self, "_payload_tx", None) is not None:
            self._payload_tx.shutdown()
        self.unregister_from_controller()
