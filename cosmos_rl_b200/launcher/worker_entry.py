"""User-facing entry point of every process of a job
(cosmos_rl/launcher/worker_entry.py:10-105).

A user script calls ``main(dataset=..., reward_fns=[...], data_packer=...)``; the launcher starts that same
script once per role with ``COSMOS_ROLE`` set to ``Controller``, ``Policy``, ``Rollout`` or ``Reference``
and this function dispatches accordingly.
"""
from __future__ import annotations

import argparse
import os
import sys
from typing import Any, Callable, Dict, List, Optional

from ..utils.logging import logger


def _worker_setup(role: str):
    import torch
    from ..config import Config
    from ..dispatcher.api.client import APIClient
    from ..parallel.dims import ParallelDims
    from ..utils.dist_util import init_distributed
    api = APIClient(role)
    meta = api.get_controller_metadata()
    config = Config.from_dict(meta["config"])
    init_distributed()
    import torch.distributed as dist
    world = dist.get_world_size() if dist.is_initialized() else 1
    rank = dist.get_rank() if dist.is_initialized() else 0
    if torch.cuda.is_available():
        device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")) % torch.cuda.device_count())
    else:
        device = torch.device("cpu")
    par = {"POLICY": config.policy.parallelism, "ROLLOUT": config.rollout.parallelism,
           "REFERENCE": config.distillation.parallelism}[role.upper()]
    dims = ParallelDims.from_config_parallelism(par, world, rank, device)
    dims.build_groups()
    return config, dims, device, api


def _leave(ok: bool) -> None:
    """End a worker PROCESS that finished its work and shut down in order (checkpoints finalised, communicators
    aborted, process group destroyed) without running interpreter teardown: communication libraries keep helper
    threads whose destruction order at exit is not defined, and a process that did all its work must not end in an
    abort raised there. Only in processes the launcher started (``COSMOS_ROLE`` set); ``COSMOS_HARD_EXIT=0`` keeps the
    ordinary exit."""
    if not ok or not os.environ.get("COSMOS_ROLE") or os.environ.get("COSMOS_HARD_EXIT", "1") == "0":
        return
    import logging
    logging.shutdown()
    sys.stdout.flush()
    sys.stderr.flush()
    os._exit(0)


def _tokenizer(config):
    path = config.policy.model_name_or_path
    from ..utils.extension import load_tokenizer
    tok, handled = load_tokenizer(path)
    if handled:
        return tok
    if os.path.isdir(path):
        try:
            from transformers import AutoTokenizer
            return AutoTokenizer.from_pretrained(path)
        except Exception as e:
            logger.warning("no tokenizer loaded from %s: %s", path, e)
    return None


def policy_entry(dataset=None, val_dataset=None, data_packer=None, val_data_packer=None, hook_fns=None, **kw):
    config, dims, device, api = _worker_setup("POLICY")
    from ..policy.trainer import (diffusion_trainer, dpo_trainer, grpo_trainer, sft_trainer,  # noqa: F401 (registry)
                                  vla_flow_trainer, vla_trainer)
    tp = config.train.train_policy
    if tp.type == "sft":
        from ..policy.worker.sft_worker import SFTPolicyWorker
        worker = SFTPolicyWorker(config, dims, dataset=dataset, val_dataset=val_dataset, data_packer=data_packer,
                                 val_data_packer=val_data_packer, hook_fns=hook_fns, api=api, device=device,
                                 tokenizer=_tokenizer(config))
    else:
        from ..policy.worker.rl_worker import RLPolicyWorker
        worker = RLPolicyWorker(config, dims, dataset=dataset, val_dataset=val_dataset, data_packer=data_packer,
                                val_data_packer=val_data_packer, hook_fns=hook_fns, api=api, device=device,
                                tokenizer=_tokenizer(config))
    ok = False
    try:
        worker.execute()
        ok = True
    finally:
        worker.handle_shutdown()
        from ..parallel.dyncomm import abort_all
        from ..utils.dist_util import safe_destroy
        abort_all()
        safe_destroy()
    _leave(ok)


def rollout_entry(dataset=None, val_dataset=None, data_packer=None, val_data_packer=None, reward_fns=None,
                  filter_reward_fns=None, val_reward_fns=None, **kw):
    config, dims, device, api = _worker_setup("ROLLOUT")
    from ..rollout.worker import DisaggregatedRolloutControlWorker
    worker = DisaggregatedRolloutControlWorker(
        config, dims, dataset=dataset, val_dataset=val_dataset, data_packer=data_packer,
        val_data_packer=val_data_packer, reward_fns=reward_fns, filter_reward_fns=filter_reward_fns,
        val_reward_fns=val_reward_fns, api=api, device=device, tokenizer=_tokenizer(config))
    ok = False
    try:
        worker.work()
        ok = True
    finally:
        worker.handle_shutdown()
        from ..parallel.dyncomm import abort_all
        from ..utils.dist_util import safe_destroy
        abort_all()
        safe_destroy()
    _leave(ok)


def reference_entry(**kw):
    config, dims, device, api = _worker_setup("REFERENCE")
    from ..reference.teacher_worker import TeacherWorker
    worker = TeacherWorker(config, dims, api=api, device=device)
    ok = False
    try:
        worker.execute()
        ok = True
    finally:
        worker.handle_shutdown()
    _leave(ok)


def colocated_entry(dataset=None, val_dataset=None, data_packer=None, reward_fns=None, custom_logger_fns=None, **kw):
    """Single-process job: controller logic, trainer and rollout backend in this process."""
    import torch
    from ..colocated.worker import ColocatedRLControlWorker
    from ..config import Config, load_toml
    config = Config.from_dict(load_toml(os.environ["COSMOS_CONFIG"]))
    device = torch.device("cuda", 0) if torch.cuda.is_available() else torch.device("cpu")
    worker = ColocatedRLControlWorker(config, dataset, val_dataset=val_dataset, reward_fns=reward_fns,
                                      data_packer=data_packer, device=device, custom_logger_fns=custom_logger_fns,
                                      tokenizer=_tokenizer(config))
    reports = worker.run()
    logger.info("[Colocated] finished after %d training steps", len(reports))
    return reports


def controller_entry(dataset=None, val_dataset=None, custom_logger_fns=None, sampler=None, args=None, **kw):
    from ..dispatcher.run_web_panel import main as controller_main
    controller_main(args, dataset=dataset, val_dataset=val_dataset, custom_logger_fns=custom_logger_fns,
                    sampler=sampler)


def main(dataset=None, val_dataset=None, data_packer=None, val_data_packer=None, reward_fns=None,
         filter_reward_fns=None, val_reward_fns=None, custom_logger_fns=None, hook_fns=None, sampler=None,
         batch_sampler=None, args=None, **kw):
    role = os.environ.get("COSMOS_ROLE", "Controller").lower()
    try:
        # SIGUSR2 writes every thread's Python stack to stderr (the replica's log): where is a stuck job waiting?
        import faulthandler
        import signal
        faulthandler.register(signal.SIGUSR2, all_threads=True, chain=False)
    except Exception:
        pass
    if dataset is None:
        # no dataset from the entry script: the rows of train_policy.dataset.name, read by the configured columns
        from ..tools.dataset.common import config_dataset
        dataset = lambda config: config_dataset(config)                                    # noqa: E731
        if val_dataset is None:
            val_dataset = lambda config: config_dataset(config, validation=True)          # noqa: E731
    if role == "controller":
        return controller_entry(dataset=dataset, val_dataset=val_dataset, custom_logger_fns=custom_logger_fns,
                                sampler=sampler, args=args)
    if role == "policy":
        return policy_entry(dataset=dataset, val_dataset=val_dataset, data_packer=data_packer,
                            val_data_packer=val_data_packer, hook_fns=hook_fns)
    if role == "rollout":
        return rollout_entry(dataset=dataset, val_dataset=val_dataset, data_packer=data_packer,
                             val_data_packer=val_data_packer, reward_fns=reward_fns,
                             filter_reward_fns=filter_reward_fns, val_reward_fns=val_reward_fns)
    if role == "reference":
        return reference_entry()
    if role == "colocated":
        return colocated_entry(dataset=dataset, val_dataset=val_dataset, data_packer=data_packer,
                               reward_fns=reward_fns, custom_logger_fns=custom_logger_fns)
    raise ValueError(f"unknown COSMOS_ROLE {role!r}")


if __name__ == "__main__":
    main()
