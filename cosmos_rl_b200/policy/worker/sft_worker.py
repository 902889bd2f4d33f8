"""SFT / DPO policy worker: owns its dataloader (data-parallel sampler, epochs, resume position), runs
``trainer.step_training`` per global batch, validates every ``validation.freq`` steps and checkpoints
(cosmos_rl/policy/worker/sft_worker.py:308-1097). With several policy replicas the gradients are averaged over
the elastic inter-replica communicator, as in cosmos_rl/policy/worker/multi_replica_sft_worker.py:44-565."""
from __future__ import annotations

import contextlib
import random
from typing import Any, List, Optional

import torch
import torch.distributed as dist

from ...comm.base import CommMixin
from ...dispatcher import command as cmd
from ...dispatcher.data import CosmosDataset
from ...dispatcher.protocol import Role
from ...parallel.inter_replica import InterReplicaComm
from ...utils.logging import logger
from ..trainer.base import TrainerRegistry


class SFTPolicyWorker(CommMixin):
    role = Role.POLICY

    def __init__(self, config, parallel_dims, dataset=None, val_dataset=None, data_packer=None, val_data_packer=None,
                 hook_fns=None, api=None, device=None, tokenizer=None, standalone: bool = False, **kw):
        self.config, self.parallel_dims = config, parallel_dims
        self.device = device or parallel_dims.device
        self.standalone = standalone or api is None and False
        if not standalone:
            self.init_comm(api)
            self.inter_replica = InterReplicaComm(self.api, self.replica_name, self.global_rank, self.device)
        else:
            self.global_rank = dist.get_rank() if dist.is_initialized() else 0
            self.world_size = dist.get_world_size() if dist.is_initialized() else 1
            self.inter_replica = None
        self.dataset = CosmosDataset.wrap(dataset, config, tokenizer)
        self.val_dataset = CosmosDataset.wrap(val_dataset, config, tokenizer)
        tp = config.train.train_policy
        self.trainer = TrainerRegistry.get_trainer_cls(tp.trainer_type)(
            config, parallel_dims, device=self.device, data_packer=data_packer, val_data_packer=val_data_packer,
            hook_fns=hook_fns, tokenizer=tokenizer, inter_replica=self.inter_replica, **kw)
        resumed = self.trainer.weight_resume()
        self.start_step = self.trainer.train_step if resumed else 0
        self.dp = parallel_dims.dp_shard * parallel_dims.dp_replicate
        c = parallel_dims.coords
        self.dp_rank = c["dp_replicate"] * parallel_dims.dp_shard + c["dp_shard"]
        self.batch_per_rank = max(1, config.train.train_batch_per_replica // self.dp)
        # several replicas: each one is a further data-parallel slice. The controller sends the membership as a
        # BuildMesh command once the configured number of replicas has registered; the replicas then divide every
        # global batch between them and average their gradients over the inter-replica communicator
        self.stop_requested = False
        if not standalone:
            self.start_command_thread()
            want = max(1, config.policy.parallelism.n_init_replicas)
            if want > 1:
                self._await_mesh(want)
            self.dp, self.dp_rank = self.dp * self.inter_replica.world, self.inter_replica.rank * self.dp + self.dp_rank
            if self.inter_replica.world > 1:
                logger.info("[SFT] replica %d of %d: data-parallel slice %d of %d", self.inter_replica.rank,
                            self.inter_replica.world, self.dp_rank, self.dp)
        n = len(self.dataset) if self.dataset is not None else 0
        per_step = self.batch_per_rank * self.dp
        self.steps_per_epoch = n // per_step if tp.dataloader_drop_last else -(-n // per_step)
        self.total_steps = self.steps_per_epoch * config.train.epoch
        if config.train.max_num_steps:
            self.total_steps = min(self.total_steps, config.train.max_num_steps)
        self.history: List[dict] = []
        self.sample_cache = None
        if tp.enable_dataset_cache and self.dataset is not None:
            # processed samples (tokenised conversations, image-processor outputs) are kept on disk per sample index;
            # the folder name carries the data set, the model and the length limit, which decide the processed form
            import hashlib
            import os
            from ...utils.cache import DiskCache
            key = hashlib.sha1(repr((getattr(tp.dataset, "name", ""), getattr(tp.dataset, "subset", ""),
                                     config.policy.model_name_or_path, config.policy.model_max_length,
                                     getattr(tp, "conversation_column_name", ""))).encode()).hexdigest()[:16]
            root = os.environ.get("COSMOS_CACHE", os.path.join(os.path.expanduser("~"), ".cache", "cosmos"))
            self.sample_cache = DiskCache(os.path.join(root, "datasets_cache", f"{getattr(tp.dataset, 'name', 'dataset') or 'dataset'}-{key}"))
            logger.info("[SFT] processed samples are cached under %s", self.sample_cache.path)
        self.balancer = None
        if tp.enable_dp_load_balancing and self.dataset is not None:
            # token-budgeted batches from a per-rank pool instead of a fixed sample count per rank; the cost of a
            # batch is the sum of its lengths because the trainers concatenate sequences instead of padding them
            from ...data.load_balanced import LoadBalancedBatcher
            self.balancer = LoadBalancedBatcher(
                self.dataset, pool_size=tp.load_balanced_pool_size,
                max_tokens_for_batch=tp.load_balanced_max_tokens_for_batch or config.policy.model_max_length,
                batching_strategy=tp.load_balanced_batching_strategy, max_tokens_len=config.policy.model_max_length,
                packed=True, seed=tp.dataloader_seed, shuffle=tp.dataloader_shuffle, dp_rank=self.dp_rank,
                dp_world_size=self.dp, accumulate_steps=tp.load_balanced_batches_per_optimizer_step,
                process_fn=self.trainer.data_packer.sft_process_sample)
            if self.start_step:
                self.balancer.skip_steps(self.start_step)

    def _consume_commands(self, block: float = 0.0) -> None:
        """Membership changes and stop requests from the controller (every rank of the replica sees the same)."""
        while True:
            c = self.next_command(timeout=block)
            block = 0.0
            if c is None:
                return
            if isinstance(c, cmd.BuildMeshCommand):
                self.inter_replica.rebuild(c.replica_name_to_rank, c.uuid_value)
            elif isinstance(c, cmd.StopCommand):
                self.stop_requested = True

    def _await_mesh(self, n_replicas: int, timeout_s: float = 300.0) -> None:
        import time
        end = time.time() + timeout_s
        while self.inter_replica.world < n_replicas and time.time() < end:
            self._consume_commands(block=0.2)
        if self.inter_replica.world < n_replicas:
            logger.warning("[SFT] only %d of %d replicas joined within %.0f s: training with those",
                           self.inter_replica.world, n_replicas, timeout_s)

    def _epoch_order(self, epoch: int) -> List[int]:
        tp = self.config.train.train_policy
        order = list(range(len(self.dataset)))
        if tp.dataloader_shuffle:
            random.Random(tp.dataloader_seed + epoch).shuffle(order)
        return order

    def _batch(self, step: int) -> List[Any]:
        """Samples of this data-parallel rank for global step ``step`` (0-based)."""
        if self.balancer is not None:
            return [s for b in self.balancer.next_step() for s in b]
        epoch, k = divmod(step, max(1, self.steps_per_epoch))
        order = self._epoch_order(epoch)
        per_step = self.batch_per_rank * self.dp
        idxs = order[k * per_step:(k + 1) * per_step][self.dp_rank::self.dp]
        return [self._sample(i) for i in idxs]

    def _sample(self, i: int) -> Any:
        """Sample ``i``, processed once and read back from the disk cache afterwards when the cache is on."""
        if self.sample_cache is None:
            return self.dataset[i]
        got = self.sample_cache.get(i)
        if got is None:
            got = self.trainer.data_packer.sft_process_sample(self.dataset[i])
            self.sample_cache.set(i, got)
        flat = dict(got)
        flat.update(flat.pop("mm", None) or {})        # processed vision inputs go back where the packer looks for them
        return flat

    def validate(self, step: int) -> Optional[float]:
        if self.val_dataset is None:
            return None
        bs = self.config.validation.batch_size or self.batch_per_rank
        total, n = 0.0, 0
        ema = getattr(self.trainer, "ema", None)
        with (ema.swapped_in() if ema is not None else contextlib.nullcontext()):   # the averaged weights are scored
            for i in range(self.dp_rank * bs, len(self.val_dataset), bs * self.dp):
                batch = [self.val_dataset[j] for j in range(i, min(i + bs, len(self.val_dataset)))]
                total += self.trainer.step_validation(batch).get("val/loss", 0.0)
                n += 1
        score = -total / max(n, 1)
        self.trainer.ckpt_manager.report_validation_score(step, score)
        logger.info("[SFT] validation at step %d: loss=%.4f", step, -score)
        return -score

    def main_loop(self) -> None:
        ck, val = self.config.train.ckpt, self.config.validation
        if val.enable and val.val_before_train:
            self.validate(self.start_step)
        save_freq = max(1, ck.save_freq)
        if ck.save_freq_in_epoch > 0:           # takes priority over the step cadence (sft_worker.py:739-746)
            save_freq = max(1, ck.save_freq_in_epoch * max(1, self.steps_per_epoch))
        for step in range(self.start_step, self.total_steps):
            if not self.standalone:
                self._consume_commands()
                if self.stop_requested:
                    break
            do_save = ck.enable_checkpoint and ((step + 1) % save_freq == 0 or step + 1 == self.total_steps)
            report = self.trainer.step_training(self._batch(step), self.total_steps, step + 1, do_save=do_save)
            self.history.append({"step": step + 1, **report})
            if (step + 1) % max(1, self.config.logging.log_interval) == 0 and self.global_rank == 0:
                logger.info("[SFT] step %d/%d loss=%.4f grad_norm=%.3f", step + 1, self.total_steps,
                            report["train/loss_avg"], report["train/grad_norm"])
            if val.enable and val.freq and (step + 1) % val.freq == 0:
                self.validate(step + 1)
            if not self.standalone and self.global_rank == 0:
                try:
                    self.api.post_train_ack(self.replica_name, step + 1, self.total_steps, False, report)
                except Exception as e:
                    logger.warning("train_ack failed: %s", e)
        self.handle_shutdown()

    execute = main_loop

    def handle_shutdown(self) -> None:
        if getattr(self, "_shut", False):
            return
        self._shut = True
        self.trainer.ckpt_manager.finalize()
        if not self.standalone:
            self.shutdown_signal.set()
            if self.inter_replica is not None:
                self.inter_replica.shutdown()
            self.unregister_from_controller()
