"""Reference / teacher replica for on-policy distillation: a forward-only model that scores token sequences
sent by the rollout side and stores the per-token (top-k) log-probs under a uuid for the policy to fetch
(cosmos_rl/reference/worker/teacher_worker.py:57-367, reference/engine/torch_engine.py:119-730,
teacher streams cosmos_rl/utils/redis_stream.py:287-478).

Requests travel on the ``teacher-request`` stream read through a consumer group (each request is served by
exactly one teacher replica); results are written to the key/value store as ``teacher:<uuid>``.
"""
from __future__ import annotations

import time
import uuid
from typing import Any, Dict, List, Optional

import msgpack
import torch

from ..comm.base import CommMixin
from ..comm.broker import TEACHER_REQUEST_STREAM
from ..dispatcher.protocol import Role
from ..models import hf_io
from ..models.base import ModelRegistry
from ..parallel.flat import FlatParams
from ..utils.logging import logger
from ..utils.sequence_packing import pack_sequences


def teacher_key(uid: str) -> str:
    return f"teacher:{uid}"


def submit_teacher_request(broker, token_ids: List[int], n_prompt: int, uid: Optional[str] = None) -> str:
    """Rollout side: ask for the teacher's log-probs of ``token_ids[n_prompt:]``. Returns the result uuid."""
    uid = uid or str(uuid.uuid4())
    broker.publish(TEACHER_REQUEST_STREAM, msgpack.packb({"uuid": uid, "ids": list(token_ids), "n_prompt": n_prompt}))
    return uid


def fetch_teacher_result(broker, uid: str, timeout_s: float = 60.0) -> Optional[Dict[str, Any]]:
    """Policy side: wait (bounded) for the result stored under ``uid``."""
    deadline = time.time() + timeout_s
    while time.time() < deadline:
        raw = broker.kv_get(teacher_key(uid))
        if raw is not None:
            return msgpack.unpackb(raw, raw=False)
        time.sleep(0.01)
    return None


class TeacherEngine:
    """Forward-only scorer on the distillation model."""

    def __init__(self, config, device: torch.device, parallel_dims=None):
        d = config.distillation
        name = d.model_name_or_path or config.policy.model_name_or_path
        hf_config = hf_io.load_hf_config(name, config.custom.get("teacher_model_config"))
        with torch.device("meta"):
            self.model = ModelRegistry.build_model(hf_config)
        dtype = torch.bfloat16 if device.type == "cuda" else torch.float32
        self.flat = FlatParams(self.model, dtype, device, with_grad=False)
        import os
        if os.path.isdir(name) and hf_io.has_safetensors(name):
            hf_io.load_hf_weights(self.model, name, parallel_dims)
        else:
            seed = d.seed if d.seed is not None else 1
            (self.model.init_weights_on_device if device.type == "cuda" else self.model.init_weights)(seed)
        self.device = device
        self.top_k = max(0, d.top_k)

    @torch.no_grad()
    def score(self, seqs: List[List[int]], n_prompts: List[int]) -> List[Dict[str, Any]]:
        masks = [[1 if (i + 1 >= n and i + 1 < len(s)) else 0 for i in range(len(s))] for s, n in zip(seqs, n_prompts)]
        b = pack_sequences(seqs, masks, device=self.device)
        sel = (b["label_ids"] >= 0).nonzero(as_tuple=True)[0]
        hidden = self.model(b["input_ids"], b["position_ids"], b["cu_seqlens"], b["max_seqlen"])
        lp, _ = self.model.logprobs(hidden[sel], b["label_ids"][sel], 1.0)
        seq_of = b["seq_ids"][sel].tolist()
        lp_l = lp.float().tolist()
        out: List[Dict[str, Any]] = [{"logprobs": [], "topk_ids": None, "topk_logprobs": None} for _ in seqs]
        for s, v in zip(seq_of, lp_l):
            out[s]["logprobs"].append(v)
        if self.top_k > 0:
            lsm = torch.log_softmax(self.model.logits(hidden[sel]).float(), -1)
            tv, ti = torch.topk(lsm, self.top_k, dim=-1)
            tv, ti = tv.tolist(), ti.tolist()
            for o in out:
                o["topk_ids"], o["topk_logprobs"] = [], []
            for s, ids, vals in zip(seq_of, ti, tv):
                out[s]["topk_ids"].append(ids)
                out[s]["topk_logprobs"].append(vals)
        return out


class TeacherWorker(CommMixin):
    role = Role.REFERENCE

    def __init__(self, config, parallel_dims, api=None, device=None, **kw):
        self.config, self.parallel_dims = config, parallel_dims
        self.device = device or parallel_dims.device
        self.init_comm(api)
        self.engine = TeacherEngine(config, self.device, parallel_dims)
        self.batch = max(1, config.distillation.batch_size_per_replica)
        self.group = "teachers"
        self.served = 0

    def serve_once(self, block_ms: int = 200) -> int:
        broker = self.broker
        msgs = broker.read_group(TEACHER_REQUEST_STREAM, self.group, self.batch, block_ms)
        if not msgs:
            return 0
        reqs = [msgpack.unpackb(d, raw=False) for _, d in msgs]
        res = self.engine.score([r["ids"] for r in reqs], [r["n_prompt"] for r in reqs])
        for r, o in zip(reqs, res):
            broker.kv_set(teacher_key(r["uuid"]), msgpack.packb(o), ttl_s=3600)
        self.served += len(reqs)
        return len(reqs)

    def execute(self) -> None:
        """Serve until the controller sends ``StopCommand`` (job over) or stays unreachable."""
        from ..dispatcher import command as cmd
        self.start_command_thread()
        failures = 0
        while not self.shutdown_signal.is_set():
            c = self.next_command()
            if isinstance(c, cmd.StopCommand):
                logger.info("[Teacher] stop received after %d scored requests", self.served)
                break
            try:
                self.serve_once()
                failures = 0
            except Exception as e:
                failures += 1
                logger.error("[Teacher] request failed: %s", e)
                if failures >= 3:
                    logger.error("[Teacher] the controller stays unreachable: leaving")
                    break
                time.sleep(0.5)          # do not spin on a persistent error

    def handle_shutdown(self) -> None:
        self.shutdown_signal.set()
        self.unregister_from_controller()
