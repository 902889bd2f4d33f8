"""HTTP request/response models of the controller API and the mesh-axis naming shared by all replicas
(cosmos_rl/dispatcher/protocol.py:21-180)."""
from __future__ import annotations

from typing import Any, Dict, List, Optional

from pydantic import BaseModel, model_validator

from .data.schema import RLPayload

MESH_NAMES = ["pp", "dp_shard", "cp", "tp"]


class Role:
    POLICY = "POLICY"
    ROLLOUT = "ROLLOUT"
    REFERENCE = "REFERENCE"
    ALL = [POLICY, ROLLOUT, REFERENCE]


class ErrorResponse(BaseModel):
    object: str = "error"
    message: str
    code: int


class RegisterRequest(BaseModel):
    replica_name: str
    role: str
    mesh_names: List[str]
    global_rank: int
    host_ip: str = "127.0.0.1"
    host_name: str = "localhost"
    ranks: List[int]
    group_size: List[int]

    @model_validator(mode="after")
    def _normalise(self):
        if not (len(self.mesh_names) == len(self.ranks) == len(self.group_size)):
            raise ValueError("mesh_names, ranks and group_size must have the same length")
        if not set(self.mesh_names) <= set(MESH_NAMES):
            raise ValueError(f"mesh_names must be a subset of {MESH_NAMES}")
        if self.role not in Role.ALL:
            raise ValueError("role must be one of POLICY, ROLLOUT, REFERENCE")
        if not self.replica_name:
            raise ValueError("replica_name must be non-empty")
        given = {m: (r, g) for m, r, g in zip(self.mesh_names, self.ranks, self.group_size)}
        self.ranks = [given.get(m, (0, 1))[0] for m in MESH_NAMES]
        self.group_size = [given.get(m, (0, 1))[1] for m in MESH_NAMES]
        self.mesh_names = list(MESH_NAMES)
        return self


class UnregisterRequest(BaseModel):
    replica_name: str


class HeartbeatRequest(BaseModel):
    replica_name: str


class SetProfileRequest(HeartbeatRequest):
    active_steps: int = 1
    rank_filter: List[int] = [0]
    record_shape: bool = False
    profile_memory: bool = False
    with_stack: bool = False
    with_modules: bool = False


class SetTracePathRequest(HeartbeatRequest):
    trace_path: str
    global_rank: int


class HandshakeInitiatorRequest(BaseModel):
    unique_pair_name: str
    handle_base64: str


class HandshakeAcceptorRequest(BaseModel):
    unique_pair_name: str


class NcclStoreClearRequest(BaseModel):
    unique_pair_name: str


class NcclErrRequest(BaseModel):
    replica_name: str
    error: str


class IpcInfoRequest(BaseModel):
    mesh_key: str
    ipc_addr: str


class QueryIpcInfoRequest(BaseModel):
    mesh_key: str


class TrainAckRequest(BaseModel):
    replica_name: str
    weight_step: int
    total_steps: int
    profile_finished: bool = False
    report_data: Dict[str, Any] = {}


class RolloutRequest(BaseModel):
    src_replica_name: str
    src_global_rank: Optional[int] = None
    stays_command_participant: bool = False
    payloads: List[RLPayload]
    metrics: Dict[str, Any] = {}
    is_end: bool = False


class ValidationReportRequest(BaseModel):
    src_replica_name: str
    validation_step: int
    payloads: List[RLPayload]
    is_end: bool = False


class SetShardInfosRequest(BaseModel):
    shard_infos: List[Dict[str, Any]]
    param_groups: List[List[str]] = []
    sorted_params: List[List[str]] = []


class GetShardSendRecvInstsRequest(BaseModel):
    rank: int


class ResumeInfoRequest(BaseModel):
    ckpt_extra_info: Dict[str, Any]
