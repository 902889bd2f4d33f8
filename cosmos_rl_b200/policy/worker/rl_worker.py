"""RL policy worker: the consumer side of the asynchronous loop
(cosmos_rl/policy/worker/rl_worker.py:80-1067).

Rank 0 runs two fetch threads (commands, rollouts); the main loop takes the next command, shares it with the
other ranks of the replica and executes its handler: load weights, (re)build the inter-replica mesh, ship the
full training state to other policy replicas, synchronise weights to a rollout replica, train a step on
``items_count`` rollouts, or finish.
"""
from __future__ import annotations

import queue
import signal
import threading
import time
from typing import Any, Dict, List, Optional

import torch
import torch.distributed as dist

from ...comm.base import CommMixin
from ...comm.broker import rollout_stream
from ...dispatcher import command as cmd
from ...dispatcher.data import CosmosDataset, WorkerDataFetcher
from ...dispatcher.data.schema import Rollout
from ...dispatcher.protocol import Role
from ...parallel.dims import ParallelDims
from ...parallel.inter_replica import InterReplicaComm
from ...parallel.reshard import model_parts, shard_info
from ...utils.logging import logger
from ..trainer.base import TrainerRegistry


def agree_force_save(event: threading.Event, world_size: int) -> bool:
    """MAX-reduce the "a checkpoint was requested by a signal" flag over the ranks of the replica and clear it where it
    was set. Every rank must call this on every step (whether it runs is decided by configuration, never by the
    signal itself): ranks see a forwarded signal at different moments, and a rank that reduced alone would pair its
    flag with the first collective of the others' training step (cosmos_rl/policy/worker/rl_worker.py:598-608
    gathers the flag on every step for the same reason)."""
    flag = torch.tensor([1 if event.is_set() else 0])
    if world_size > 1:
        dist.all_reduce(flag, op=dist.ReduceOp.MAX)
    if int(flag) > 0:
        event.clear()
        return True
    return False


class RLPolicyWorker(CommMixin):
    role = Role.POLICY

    def __init__(self, config, parallel_dims: ParallelDims, dataset=None, val_dataset=None, data_packer=None,
                 val_data_packer=None, hook_fns=None, api=None, device=None, **kw):
        self.config = config
        self.parallel_dims = parallel_dims
        self.device = device or parallel_dims.device
        self.init_comm(api)
        ds = CosmosDataset.wrap(dataset, config)
        self.data_fetcher = WorkerDataFetcher(config, ds)
        tp = config.train.train_policy
        self.inter_replica = InterReplicaComm(self.api, self.replica_name, self.global_rank, self.device)
        trainer_kw = dict(device=self.device, data_packer=data_packer, val_data_packer=val_data_packer,
                          hook_fns=hook_fns, inter_replica=self.inter_replica)
        if self.device.type == "cuda" and config.b200.peer_weight_sync:
            from ...parallel.peer import peer_allocator
            trainer_kw["allocator"] = peer_allocator(self.device)
        trainer_kw.update(kw)
        self.trainer = TrainerRegistry.get_trainer_cls(tp.trainer_type)(config, parallel_dims, **trainer_kw)
        from ...utils.dist_util import group_on_one_host
        if (parallel_dims.dp_shard > 1 and self.device.type == "cuda" and config.b200.peer_weight_sync
                and not getattr(self.trainer, "shard_params", False)
                and group_on_one_host(parallel_dims.group("dp_shard"))):
            # peer loads / stores need every rank of the group on this machine; a group that spans machines keeps
            # the NCCL reduce-scatter / all-gather of the optimizer
            from ...parallel.fsdp import PeerCollective
            self.trainer.optimizer.collective = PeerCollective(self.trainer.flat, parallel_dims.group("dp_shard"))
        self.data_queue: "queue.Queue[Rollout]" = queue.Queue()
        self._last_rollout_id = 0
        self.handlers = cmd.PolicyCommandRegistry()
        for c, h in ((cmd.WeightResumeCommand, self.execute_weight_resume),
                     (cmd.BuildMeshCommand, self.execute_build_mesh),
                     (cmd.PolicyToPolicyBroadcastCommand, self.execute_policy_to_policy_broadcast),
                     (cmd.PolicyToPolicyUnicastCommand, self.execute_policy_to_policy_unicast),
                     (cmd.PolicyToRolloutUnicastCommand, self.execute_policy_to_rollout_unicast),
                     (cmd.DataFetchCommand, self.execute_data_fetch),
                     (cmd.TrainingCompleteCommand, self.execute_training_complete)):
            self.handlers.register(c, h)
        self.p2r_comms: Dict[str, Any] = {}
        self.p2r_send_plan = None
        self.shard_infos_posted = False
        self.force_save = threading.Event()
        # a forced checkpoint can only come from a handled signal or the exit hook; both are configuration, so every
        # rank agrees on whether the per-step flag reduction exists
        self.force_save_possible = bool(config.train.save_ckpt_at_exit or config.train.signal_to_handle)
        self.profiler = None
        if config.profiler.enable_profiler:
            from ...utils.profiler import CosmosProfiler
            self.profiler = CosmosProfiler(config, self.replica_name, self.global_rank, self.api)
        self._install_signal_handlers()

    # ------------------------------------------------------------------ signals
    def _install_signal_handlers(self) -> None:
        if threading.current_thread() is not threading.main_thread():
            return
        for name in self.config.train.signal_to_handle:
            sig = getattr(signal, name, None)
            if sig is None:
                continue
            try:
                signal.signal(sig, lambda *_: self.force_save.set())
            except (ValueError, OSError):
                pass

    def _payload_prefetcher(self):
        if not hasattr(self, "_payload_pf"):
            from ...utils.payload_transport import (PayloadPrefetcher, PayloadTransportRegistry,
                                                    get_payload_transfer_mode)
            mode = get_payload_transfer_mode(self.config)
            self._payload_pf = None
            if mode != "broker":
                tx = type(PayloadTransportRegistry.get(mode))()
                tx.setup(self.config, self.broker, self.device, owner=f"{self.replica_name[:12]}-p{self.global_rank}")
                self._payload_pf = PayloadPrefetcher(tx)
        return self._payload_pf

    # ------------------------------------------------------------------ shard infos for weight sync
    def _sync_buffer(self) -> torch.Tensor:
        fn = getattr(self.trainer, "sync_buffer", None)
        return fn() if fn is not None else self.trainer.flat.data

    def post_shard_infos(self) -> None:
        if self.shard_infos_posted:
            return
        info = shard_info(self.global_rank, model_parts(self.trainer.model, self.trainer.flat), self.trainer.flat.total)
        buf = getattr(self._sync_buffer(), "_peer_buffer", None)
        if buf is not None:
            info["ipc_handle"] = buf.export()
            info["nbytes"] = buf.nbytes
            from ...utils.dist_util import host_id
            info["host"] = host_id()
        infos = [None] * self.world_size
        if self.world_size > 1:
            dist.all_gather_object(infos, info)
        else:
            infos = [info]
        if self.global_rank == 0:
            trainable = [n for n, p in self.trainer.model.named_parameters() if p.requires_grad]
            self.api.post_shard_infos("policy", {"ranks": infos, "trainable_params": trainable,
                                                 "replica": self.replica_name})
        self.shard_infos_posted = True

    # ------------------------------------------------------------------ handlers
    def execute_weight_resume(self, c: cmd.WeightResumeCommand) -> bool:
        resumed = self.trainer.weight_resume()
        if resumed and self.global_rank == 0:
            self.api.post_resume_info(getattr(self.trainer, "resume_extra_info", {}))
        self.post_shard_infos()
        return False

    def execute_build_mesh(self, c: cmd.BuildMeshCommand) -> bool:
        self.inter_replica.rebuild(c.replica_name_to_rank, c.uuid_value)
        return False

    # A membership change must reach the inter-replica communicator even while the main loop sits inside a training
    # step (a peer replica died: the step's gradient all-reduce fails and waits for the new mesh). Rank 0's command
    # thread therefore also publishes every BuildMesh command under a key of the controller's KV store, and a
    # watcher thread on every rank applies it (the reference hands the command to its HA_NCCL thread the same way,
    # cosmos_rl/policy/worker/rl_worker.py:717-758, cosmos_rl/utils/distributed.py:600-620).
    def on_command_received(self, c, raw: bytes) -> None:
        if isinstance(c, cmd.BuildMeshCommand):
            try:
                self.broker.kv_set(f"mesh:{self.replica_name}", raw, ttl_s=24 * 3600)
            except Exception as e:
                logger.warning("[Policy] could not publish the mesh command: %s", e)

    def start_mesh_watcher(self) -> None:
        key = f"mesh:{self.replica_name}"

        def loop():
            seen = None
            while not self.shutdown_signal.is_set():
                try:
                    raw = self.broker.kv_get(key)
                except Exception:
                    raw = None
                if raw and raw != seen:
                    seen = raw
                    try:
                        c = cmd.Command.depack(raw)
                        self.inter_replica.rebuild(c.replica_name_to_rank, c.uuid_value)
                    except Exception as e:
                        logger.warning("[Policy] mesh rebuild from the watcher failed: %s", e)
                time.sleep(0.3)

        t = threading.Thread(target=loop, name="mesh_watcher", daemon=True)
        t.start()
        self._threads.append(t)

    def execute_policy_to_policy_broadcast(self, c: cmd.PolicyToPolicyBroadcastCommand) -> bool:
        src = self.inter_replica.mapping.get(c.src_replica_name, 0)
        tensors = self.trainer.state_tensors()
        self.inter_replica.broadcast_state(tensors, src)
        if self.replica_name != c.src_replica_name:
            self.trainer.after_state_received(dict(tensors)["meta"])
        self.post_shard_infos()
        return False

    def execute_policy_to_policy_unicast(self, c: cmd.PolicyToPolicyUnicastCommand) -> bool:
        tensors = self.trainer.state_tensors()
        if self.replica_name == c.src_replica_name:
            self.inter_replica.send_state(tensors, self.inter_replica.mapping[c.dst_replica_name])
        else:
            self.inter_replica.recv_state(tensors, self.inter_replica.mapping[c.src_replica_name])
            self.trainer.after_state_received(dict(tensors)["meta"])
            self.post_shard_infos()
        return False

    def execute_policy_to_rollout_unicast(self, c: cmd.PolicyToRolloutUnicastCommand) -> bool:
        """Make this replica's weights available to one rollout replica.

        Peer mode (GPUs of one node): the weights already sit in IPC-exported memory; the policy only has to
        guarantee they are final (device synchronise), announce it, and wait for the puller's completion mark
        so that the next optimizer step cannot overwrite them mid-pull. Collective mode: send the rectangles
        of the plan over a dynamic communicator that spans both replicas (policy ranks first)."""
        if self.replica_name != c.src_replica_name:
            return False
        self.post_shard_infos()
        self.trainer.before_weight_sync()
        try:
            return self._serve_weights(c)
        finally:
            self.trainer.after_weight_sync()

    def _serve_weights(self, c: cmd.PolicyToRolloutUnicastCommand) -> bool:
        if self.device.type == "cuda":
            torch.cuda.synchronize()
        key = f"p2r:{c.uuid_value}"
        if self._peer_mode() and self._pair_transport(c) == "peer":
            if self.world_size > 1:
                dist.barrier()
            if self.global_rank == 0:
                self.broker.kv_set(key + ":ready", b"1", ttl_s=3600)
                deadline = time.time() + 600
                done = 0
                while done < c.dst_replica_size and time.time() < deadline:
                    done = sum(1 for r in range(c.dst_replica_size) if self.broker.kv_get(f"{key}:done:{r}"))
                    if done < c.dst_replica_size:
                        time.sleep(0.01)
                if done < c.dst_replica_size:
                    logger.warning("[Policy] weight sync %s: only %d/%d rollout ranks confirmed", key, done,
                                   c.dst_replica_size)
            if self.world_size > 1:
                dist.barrier()
            return False
        from ...parallel.dyncomm import create_comm
        from ...rollout.weight_sync import CollectiveWeightSync
        pair = f"p2r-{c.src_replica_name}-{c.dst_replica_name}"
        comm = self.p2r_comms.get(pair)
        if comm is None or comm.aborted:
            comm = create_comm(self.api, f"{pair}-{c.uuid_value}" if comm is not None else pair, self.global_rank,
                               c.src_replica_size + c.dst_replica_size, self.device,
                               is_initiator=self.global_rank == 0)
            self.p2r_comms[pair] = comm
        if self.p2r_send_plan is None:
            self.p2r_send_plan = self.api.get_shard_insts("policy", self.global_rank)
        flat = self._sync_buffer()
        from ...utils.misc import str2dtype
        tdt = str2dtype(self.config.train.transfer_dtype) if self.device.type == "cuda" else None
        P = c.src_replica_size
        from ...parallel.dyncomm import watchdog
        with watchdog(wait_stream=True):                 # the sends are enqueues; bound the device side too
            for dst_rank, d in self.p2r_send_plan:
                t = torch.as_strided(flat, (d[5], d[6]), (d[2], 1), flat.storage_offset() + d[1]).contiguous()
                comm.send(t.to(tdt) if tdt is not None else t, P + dst_rank)
        return False

    def _pair_transport(self, c) -> str:
        """"peer" or "collective" for this (policy replica, rollout replica) pair. The rollout replica knows where the
        policy's buffers live (the posted shard infos carry the machine's identity) and announces its choice under
        ``p2r-mode:<src>:<dst>``; rank 0 reads it once per pair and tells the other ranks."""
        pair = f"p2r-mode:{c.src_replica_name}:{c.dst_replica_name}"
        cache = self.__dict__.setdefault("_pair_modes", {})
        if pair not in cache:
            box = [None]
            if self.global_rank == 0:
                deadline = time.time() + 600
                while box[0] is None and time.time() < deadline:
                    v = self.broker.kv_get(pair)
                    if v:
                        box[0] = v.decode() if isinstance(v, (bytes, bytearray)) else str(v)
                    else:
                        time.sleep(0.01)
                if box[0] is None:
                    raise TimeoutError(f"rollout replica {c.dst_replica_name} never announced its weight transport")
            if self.world_size > 1:
                dist.broadcast_object_list(box, src=0)
            cache[pair] = box[0]
            logger.info("[Policy] weights for %s travel by the %s transport", c.dst_replica_name, box[0])
        return cache[pair]

    def _peer_mode(self) -> bool:
        return bool(self.config.b200.peer_weight_sync and self.device.type == "cuda"
                    and getattr(self._sync_buffer(), "_peer_buffer", None) is not None)

    # ------------------------------------------------------------------ data path
    def start_rollout_thread(self) -> None:
        if self.global_rank != 0:
            return

        def loop():
            stream = rollout_stream(self.replica_name)
            while not self.shutdown_signal.is_set():
                try:
                    msgs = self.broker.read(stream, self._last_rollout_id, count=64, block_ms=500)
                except Exception as e:
                    logger.warning("[Policy] rollout read failed: %s", e)
                    time.sleep(0.5)
                    continue
                for mid, data in msgs:
                    self._last_rollout_id = mid
                    r = Rollout.model_validate_json(data)
                    if r.payload_ref and self._payload_prefetcher() is not None:
                        self._payload_pf.prefetch([r.payload_ref])      # resolved in the background before the step
                    self.data_queue.put(r)

        t = threading.Thread(target=loop, name="fetch_rollouts", daemon=True)
        t.start()
        self._threads.append(t)

    def dispatch_rollouts(self, items_count: int) -> List[Rollout]:
        """Rank 0 pops ``items_count`` rollouts and deals them round-robin to the data-parallel ranks."""
        dp = self.parallel_dims.dp_shard * self.parallel_dims.dp_replicate
        per_rank: List[List[Rollout]] = [[] for _ in range(self.world_size)]
        if self.global_rank == 0:
            got: List[Rollout] = []
            deadline = time.time() + 600
            while len(got) < items_count and time.time() < deadline:
                try:
                    got.append(self.data_queue.get(timeout=1.0))
                except queue.Empty:
                    continue
            n_ref = sum(1 for r in got if r.payload_ref)
            if n_ref:
                logger.info("[Policy] fetching the per-token data of %d rollouts through the payload transport", n_ref)
            for r in got:
                if r.payload_ref:
                    from ...utils.payload_transport import restore_rollout
                    if self._payload_prefetcher() is None or not restore_rollout(self._payload_pf, r):
                        logger.warning("[Policy] payload %s could not be fetched: the rollout trains from its text",
                                       r.payload_ref[:48])
                if r.prompt is None:
                    self.data_fetcher.fill(r)
                if self.config.distillation.enable and r.teacher_result_uuid and r.teacher_logprobs is None:
                    from ...reference.teacher_worker import fetch_teacher_result
                    res = fetch_teacher_result(self.broker, r.teacher_result_uuid, timeout_s=120.0)
                    if res is not None:
                        r.teacher_logprobs = [[v] for v in res["logprobs"]]
                        if res.get("topk_ids"):
                            r.teacher_topk_ids, r.teacher_topk_logprobs = res["topk_ids"], res["topk_logprobs"]
                    else:
                        logger.warning("[Policy] no teacher result for %s: the rollout trains without it",
                                       r.teacher_result_uuid)
            for rank in range(self.world_size):
                coords = self.parallel_dims.coords_of(rank)
                dp_idx = coords["dp_replicate"] * self.parallel_dims.dp_shard + coords["dp_shard"]
                per_rank[rank] = got[dp_idx::dp]
        if self.world_size > 1:
            out = [None]
            dist.scatter_object_list(out, per_rank if self.global_rank == 0 else None, src=0)
            return out[0]
        return per_rank[0]

    def execute_data_fetch(self, c: cmd.DataFetchCommand) -> bool:
        if c.replica_name != self.replica_name:
            return False
        rollouts = self.dispatch_rollouts(c.items_count)
        do_save = bool(c.do_save)
        if self.force_save_possible and agree_force_save(self.force_save, self.world_size):
            do_save = True
        if self.profiler is not None and c.do_profile:
            self.profiler.start_dynamic(c)
        is_master = self.inter_replica.rank == 0
        report = self.trainer.step_training(rollouts, c.global_step, c.total_steps, c.remain_samples_num,
                                            do_save=do_save and is_master)
        profile_finished = False
        if self.profiler is not None:
            profile_finished = self.profiler.step()
        if self.global_rank == 0:
            self.api.post_train_ack(self.replica_name, c.global_step, c.total_steps, profile_finished, report)
        return c.replica_should_stop()

    def execute_training_complete(self, c: cmd.TrainingCompleteCommand) -> bool:
        if c.do_save and self.inter_replica.rank == 0:
            self.trainer.save_checkpoint(c.final_step, c.checkpoint_total_steps, c.remain_samples_num, is_final=True)
        return True

    # ------------------------------------------------------------------ main loop
    def main_loop(self) -> None:
        self.start_command_thread()
        self.start_rollout_thread()
        self.start_mesh_watcher()
        stop = False
        while not stop and not self.shutdown_signal.is_set():
            c = self.next_command(timeout=0.2)
            if c is None:
                continue
            handler = self.handlers.get_command_handler(c)
            if handler is None:
                logger.warning("[Policy] no handler for %r", c)
                continue
            logger.debug("[Policy] executing %r", c)
            stop = bool(handler(c))
        self.handle_shutdown()

    execute = main_loop

    def handle_shutdown(self) -> None:
        """Order matters: stop producing work, finish checkpoints, abort dynamic communicators, unregister."""
        if getattr(self, "_shut", False):
            return
        self._shut = True
        self.shutdown_signal.set()
        try:
            self.trainer.ckpt_manager.finalize()
        except Exception as e:
            logger.warning("checkpoint finalize failed: %s", e)
        self.inter_replica.shutdown()
        for c in self.p2r_comms.values():
            c.abort()
        self.unregister_from_controller()
