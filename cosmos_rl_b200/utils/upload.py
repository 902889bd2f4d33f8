"""Copies of checkpoints and exports in object storage or a model hub.

The reference uploads every file it writes when ``train.ckpt.upload_s3`` is ``"all"`` (or only the last save when
``"final"``) and pushes the exported safetensors folder to a hub repository when ``upload_hf`` is set
(cosmos_rl/utils/checkpoint.py:60-70, 479-491; cosmos_rl/utils/s3_utils.py; llm_trainer.py:700-790). Both clients
are optional packages and need a network: when one is missing or a transfer fails the job logs it and goes on, a
failed upload never fails a training step.
"""
from __future__ import annotations

import os
from typing import List, Optional

from .logging import logger


def wants_s3(ckpt_cfg, is_final: bool) -> bool:
    mode = ckpt_cfg.upload_s3
    if not mode or not ckpt_cfg.s3_bucket:
        return False
    return mode in (True, "all") or (mode == "final" and is_final)


def upload_folder_to_s3(local_dir: str, bucket: str, prefix: str, client=None) -> List[str]:
    """Every file under ``local_dir`` to ``s3://bucket/prefix/<relative path>``; returns the keys written."""
    if client is None:
        try:
            import boto3
        except ImportError:
            logger.warning("upload_s3 is set but boto3 is not installed: nothing uploaded from %s", local_dir)
            return []
        client = boto3.client("s3")
    keys: List[str] = []
    for root, _, files in os.walk(local_dir):
        for f in sorted(files):
            if f.endswith(".tmp"):
                continue
            path = os.path.join(root, f)
            key = "/".join([prefix.strip("/"), os.path.relpath(path, local_dir).replace(os.sep, "/")]).lstrip("/")
            try:
                client.upload_file(path, bucket, key)
                keys.append(key)
            except Exception as e:          # noqa: BLE001 (any client error: log and carry on)
                logger.warning("upload of %s to s3://%s/%s failed: %s", path, bucket, key, e)
    return keys


def upload_folder_to_hub(local_dir: str, repo_name: str, api=None) -> Optional[str]:
    if api is None:
        try:
            from huggingface_hub import HfApi
        except ImportError:
            logger.warning("upload_hf is set but huggingface_hub is not installed: %s stays local", local_dir)
            return None
        api = HfApi()
    try:
        api.create_repo(repo_name, exist_ok=True)
        api.upload_folder(folder_path=local_dir, repo_id=repo_name)
        return repo_name
    except Exception as e:                  # noqa: BLE001
        logger.warning("upload of %s to hub repository %s failed: %s", local_dir, repo_name, e)
        return None
