"""Worker-side client of the controller API: one method per route, retry with exponential backoff over a
list of candidate controller addresses (cosmos_rl/dispatcher/api/client.py:68-606,
cosmos_rl/utils/network_util.py:55-143). ``LocalAPIClient`` offers the same methods on a Controller object
living in the same process (colocated mode, tests)."""
from __future__ import annotations

import base64
import os
import time
from typing import Any, Dict, List, Optional, Tuple

import msgpack

from ...utils import api_suffix as S
from ...utils import constant
from ...utils.logging import logger
from ..data.schema import RLPayload


class ControllerUnreachable(RuntimeError):
    pass


def make_request_with_retry(fn, urls: List[str], max_retries: Optional[int] = None,
                            initial_delay: Optional[float] = None, max_delay: Optional[float] = None):
    """Call ``fn(url)`` over the candidate urls until one answers; back off exponentially between rounds."""
    max_retries = constant.COSMOS_HTTP_RETRY_MAX if max_retries is None else max_retries
    delay = constant.COSMOS_HTTP_RETRY_INITIAL_DELAY if initial_delay is None else initial_delay
    max_delay = constant.COSMOS_HTTP_RETRY_MAX_DELAY if max_delay is None else max_delay
    last: Optional[Exception] = None
    for attempt in range(max_retries + 1):
        for url in urls:
            try:
                return fn(url)
            except Exception as e:  # connection refused, timeout, 5xx
                last = e
        if attempt < max_retries:
            time.sleep(delay)
            delay = min(delay * 2, max_delay)
    raise ControllerUnreachable(f"no controller address answered after {max_retries} retries: {last}")


class APIClient:
    def __init__(self, role: str, remote_hosts: Optional[List[str]] = None, max_retries: Optional[int] = None):
        import requests
        self.role = role.upper()
        hosts = remote_hosts or os.environ.get("COSMOS_CONTROLLER_HOST", "127.0.0.1:8000").split(";")
        self.base_urls = [h if h.startswith("http") else f"http://{h}" for h in hosts if h]
        self.session = requests.Session()
        self.max_retries = max_retries

    # ------------------------------------------------------------------ raw
    def get(self, suffix: str, params: Optional[Dict[str, Any]] = None, timeout: float = 30.0) -> Dict[str, Any]:
        def call(url):
            r = self.session.get(url + suffix, params={k: v for k, v in (params or {}).items() if v is not None},
                                 timeout=timeout)
            if r.status_code >= 500:
                raise RuntimeError(f"{r.status_code} {r.text[:200]}")
            return r.json()
        return make_request_with_retry(call, self.base_urls, self.max_retries)

    def post(self, suffix: str, body: Any = None, raw: Optional[bytes] = None, timeout: float = 60.0) -> Dict[str, Any]:
        def call(url):
            if raw is not None:
                r = self.session.post(url + suffix, data=raw, timeout=timeout,
                                      headers={"Content-Type": "application/msgpack"})
            else:
                r = self.session.post(url + suffix, json=body, timeout=timeout)
            if r.status_code >= 500:
                raise RuntimeError(f"{r.status_code} {r.text[:200]}")
            return r.json()
        return make_request_with_retry(call, self.base_urls, self.max_retries)

    # ------------------------------------------------------------------ routes
    def get_controller_metadata(self) -> Dict[str, Any]:
        return self.get(S.COSMOS_API_META_SUFFIX)

    def register(self, replica_name: str, role: str, mesh_names, ranks, group_size, global_rank: int,
                 host_ip: str = "127.0.0.1", host_name: str = "localhost"):
        return self.post(S.COSMOS_API_REGISTER_SUFFIX, dict(
            replica_name=replica_name, role=role, mesh_names=list(mesh_names), ranks=list(ranks),
            group_size=list(group_size), global_rank=global_rank, host_ip=host_ip, host_name=host_name))

    def unregister(self, replica_name: str):
        return self.post(S.COSMOS_API_UNREGISTER_SUFFIX, {"replica_name": replica_name})

    def heartbeat(self, replica_name: str):
        return self.post(S.COSMOS_API_HEARTBEAT_SUFFIX, {"replica_name": replica_name}, timeout=10.0)

    def post_nccl_comm_initiator(self, unique_pair_name: str, handle_base64: str):
        return self.post(S.COSMOS_API_NCCL_COMM_INITIATOR_SUFFIX,
                         {"unique_pair_name": unique_pair_name, "handle_base64": handle_base64})

    def post_nccl_comm_acceptor(self, unique_pair_name: str, timeout_s: float = 600.0) -> str:
        deadline = time.time() + timeout_s
        while True:
            r = self.post(S.COSMOS_API_NCCL_COMM_ACCEPTOR_SUFFIX, {"unique_pair_name": unique_pair_name})
            if "handle_base64" in r:
                return r["handle_base64"]
            if time.time() > deadline:
                raise TimeoutError(f"handshake key {unique_pair_name!r} never appeared")
            time.sleep(0.1)

    def post_nccl_comm_error(self, replica_name: str, error: str):
        return self.post(S.COSMOS_API_NCCL_COMM_ERROR_SUFFIX, {"replica_name": replica_name, "error": error})

    def post_nccl_comm_store_clear(self, unique_pair_name: str):
        return self.post(S.COSMOS_API_NCCL_COMM_STORE_CLEAR_SUFFIX, {"unique_pair_name": unique_pair_name})

    def get_next_prompt(self, n: int, validation_step: Optional[int] = None, rank_in_mesh: Optional[int] = None
                        ) -> Tuple[List[Tuple[int, RLPayload]], bool]:
        r = self.get(S.COSMOS_API_NEXT_PROMPT_SUFFIX,
                     {"n": n, "validation_step": validation_step, "rank_in_mesh": rank_in_mesh})
        return [(i, RLPayload.model_validate(p)) for i, p in r.get("prompt_id_and_payload_list", [])], r["is_end"]

    def post_rollout_completion(self, src_replica_name: str, payloads: List[RLPayload], is_end: bool = False,
                                metrics: Optional[Dict[str, Any]] = None, src_global_rank: Optional[int] = None):
        return self.post(S.COSMOS_API_ROLLOUT_SUFFIX, dict(
            src_replica_name=src_replica_name, src_global_rank=src_global_rank,
            payloads=[p.model_dump() for p in payloads], metrics=metrics or {}, is_end=is_end))

    def post_validation_report(self, src_replica_name: str, validation_step: int, payloads, is_end: bool = False):
        return self.post(S.COSMOS_API_VALIDATION_REPORT_SUFFIX, dict(
            src_replica_name=src_replica_name, validation_step=validation_step,
            payloads=[p.model_dump() for p in payloads], is_end=is_end))

    def post_train_ack(self, replica_name: str, weight_step: int, total_steps: int, profile_finished: bool,
                       report_data: Dict[str, Any]):
        return self.post(S.COSMOS_API_POLICY_TRAIN_ACK_SUFFIX, dict(
            replica_name=replica_name, weight_step=weight_step, total_steps=total_steps,
            profile_finished=profile_finished, report_data=report_data))

    def post_shard_infos(self, role: str, infos: Dict[str, Any]):
        suffix = S.COSMOS_API_POLICY_SHARD_INFOS_SUFFIX if role == "policy" else S.COSMOS_API_ROLLOUT_SHARD_INFOS_SUFFIX
        return self.post(suffix, raw=msgpack.packb(infos, use_bin_type=True))

    def get_shard_insts(self, role: str, rank: int):
        suffix = (S.COSMOS_API_POLICY_SHARD_SEND_INSTS_SUFFIX if role == "policy"
                  else S.COSMOS_API_ROLLOUT_SHARD_RECV_INSTS_SUFFIX)
        r = self.post(suffix, {"rank": rank})
        return msgpack.unpackb(base64.b64decode(r["insts_b64"]), raw=False, strict_map_key=False)

    def get_shard_infos(self, role: str):
        r = self.get(S.COSMOS_API_SHARD_INFOS_SUFFIX, {"role": role})
        raw = r.get("infos_b64")
        return msgpack.unpackb(base64.b64decode(raw), raw=False, strict_map_key=False) if raw else None

    def post_resume_info(self, extra_info: Dict[str, Any]):
        return self.post(S.COSMOS_API_RESUME_INFO_SUFFIX, {"ckpt_extra_info": extra_info})

    def set_trace_path(self, replica_name: str, trace_path: str, global_rank: int):
        return self.post(S.COSMOS_API_SET_TRACE_PATH_SUFFIX,
                         dict(replica_name=replica_name, trace_path=trace_path, global_rank=global_rank))

    def set_profile(self, replica_name: str, **kw):
        return self.post(S.COSMOS_API_SET_PROFILE_SUFFIX, dict(replica_name=replica_name, **kw))

    def post_ipc_info(self, mesh_key: str, ipc_addr: str):
        return self.post(S.COSMOS_API_IPC_INFO_SUFFIX, {"mesh_key": mesh_key, "ipc_addr": ipc_addr})

    def query_ipc_info(self, mesh_key: str) -> Optional[str]:
        return self.post(S.COSMOS_API_QUERY_IPC_INFO_SUFFIX, {"mesh_key": mesh_key}).get("ipc_addr")

    def status(self):
        return self.get(S.COSMOS_API_STATUS_SUFFIX)

    def broker(self):
        from ...comm.broker import HttpBrokerClient
        return HttpBrokerClient(self)


class LocalAPIClient:
    """Same surface as :class:`APIClient`, served by a Controller in this process (no HTTP, no pickling)."""

    def __init__(self, controller, role: str = "POLICY"):
        self.c = controller
        self.role = role.upper()

    def get_controller_metadata(self):
        return self.c.meta()

    def register(self, replica_name, role, mesh_names, ranks, group_size, global_rank, host_ip="127.0.0.1",
                 host_name="localhost"):
        from ..protocol import RegisterRequest
        self.c.register(RegisterRequest(replica_name=replica_name, role=role, mesh_names=list(mesh_names),
                                        ranks=list(ranks), group_size=list(group_size), global_rank=global_rank,
                                        host_ip=host_ip, host_name=host_name))

    def unregister(self, replica_name):
        self.c.unregister(replica_name)

    def heartbeat(self, replica_name):
        self.c.heartbeat(replica_name)

    def post_nccl_comm_initiator(self, name, handle):
        self.c.kv_put(name, handle)

    def post_nccl_comm_acceptor(self, name, timeout_s: float = 600.0):
        v = self.c.kv_get(name, timeout_s)
        if v is None:
            raise TimeoutError(f"handshake key {name!r} never appeared")
        return v

    def post_nccl_comm_error(self, replica_name, error):
        self.c.set_replica_ncclerror(replica_name, error)

    def post_nccl_comm_store_clear(self, name):
        self.c.kv_clear(name)

    def get_next_prompt(self, n, validation_step=None, rank_in_mesh=None):
        batch, is_end = self.c.get_batched_prompt(n, validation_step)
        return [(i, p.model_copy(deep=True)) for i, p in batch], is_end

    def post_rollout_completion(self, src_replica_name, payloads, is_end=False, metrics=None, src_global_rank=None):
        self.c.put_rollouts(src_replica_name, payloads, is_end, metrics)

    def post_validation_report(self, src, validation_step, payloads, is_end=False):
        self.c.put_validation_report(src, validation_step, payloads, is_end)

    def post_train_ack(self, replica_name, weight_step, total_steps, profile_finished, report_data):
        self.c.train_ack(replica_name, weight_step, total_steps, profile_finished, report_data)

    def post_shard_infos(self, role, infos):
        self.c.set_shard_infos(role, infos)

    def get_shard_insts(self, role, rank):
        from ...parallel.reshard import plan_for_rank
        return plan_for_rank(self.c.get_shard_infos("policy"), self.c.get_shard_infos("rollout"), role, rank)

    def get_shard_infos(self, role):
        return self.c.get_shard_infos(role)

    def post_resume_info(self, extra_info):
        self.c.set_resume_info(extra_info)

    def set_trace_path(self, replica_name, trace_path, global_rank):
        self.c.set_trace_path(replica_name, trace_path, global_rank)

    def set_profile(self, replica_name, **kw):
        return self.c.set_profile(dict(replica_name=replica_name, **kw))

    def post_ipc_info(self, mesh_key, ipc_addr):
        self.c.kv_put("ipc:" + mesh_key, ipc_addr)

    def query_ipc_info(self, mesh_key):
        return self.c.kv_get("ipc:" + mesh_key, 10.0)

    def status(self):
        return self.c.status()

    def broker(self):
        return self.c.broker
