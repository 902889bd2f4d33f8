"""HTTP front-end of the controller (FastAPI + uvicorn), routes of cosmos_rl/dispatcher/run_web_panel.py:377-766.

``python -m cosmos_rl_b200.dispatcher.run_web_panel --config job.toml --port 8000`` starts a controller.
The listening socket may be inherited from the launcher through ``COSMOS_CONTROLLER_LISTEN_FD`` so the port
it reserved cannot be lost between reservation and bind.
"""
from __future__ import annotations

import argparse
import asyncio
import base64
import os
import socket
import sys
from typing import Any, Dict, Optional

import msgpack
from fastapi import FastAPI, Request
from fastapi.responses import HTMLResponse, JSONResponse

from ..config import Config, load_toml
from ..utils import api_suffix as S
from ..utils.logging import logger
from . import protocol as P
from .controller import Controller


def _err(message: str, code: int = 400):
    return JSONResponse(P.ErrorResponse(message=message, code=code).model_dump(), status_code=code)


def create_app(controller: Controller) -> FastAPI:
    app = FastAPI(title="cosmos-rl controller")
    app.state.controller = controller
    c = controller

    @app.get(S.COSMOS_API_PANEL_SUFFIX, response_class=HTMLResponse)
    async def panel():
        st = c.status()
        rows = "".join(f"<tr><td>{r['role']}</td><td>{r['name']}</td><td>{r['status']}</td><td>{r['n_atoms']}/"
                       f"{r['expected_atoms']}</td><td>{r['weight_step']}</td></tr>"
                       for r in st["policy_replicas"] + st["rollout_replicas"])
        return (f"<html><body><h3>step {st['current_step']}/{st['total_steps']} &middot; buffer "
                f"{st['rollout_buffer']} &middot; in flight {st['samples_on_the_fly']}</h3><table border=1>"
                f"<tr><th>role</th><th>replica</th><th>status</th><th>atoms</th><th>weight step</th></tr>{rows}"
                f"</table></body></html>")

    @app.get(S.COSMOS_API_STATUS_SUFFIX)
    async def status():
        return c.status()

    @app.get(S.COSMOS_API_META_SUFFIX)
    async def meta():
        return c.meta()

    @app.post(S.COSMOS_API_REGISTER_SUFFIX)
    async def register(req: P.RegisterRequest):
        try:
            c.register(req)
        except Exception as e:
            return _err(str(e))
        return {"message": "Registered"}

    @app.post(S.COSMOS_API_UNREGISTER_SUFFIX)
    async def unregister(req: P.UnregisterRequest):
        c.unregister(req.replica_name)
        return {"message": "Unregistered"}

    @app.post(S.COSMOS_API_HEARTBEAT_SUFFIX)
    async def heartbeat(req: P.HeartbeatRequest):
        c.heartbeat(req.replica_name)
        return {"message": "Heartbeat received"}

    @app.post(S.COSMOS_API_SET_PROFILE_SUFFIX)
    async def set_profile(req: P.SetProfileRequest):
        ok = c.set_profile(req.model_dump())
        return {"message": "profile set" if ok else "replica not found"}

    @app.post(S.COSMOS_API_SET_TRACE_PATH_SUFFIX)
    async def set_trace_path(req: P.SetTracePathRequest):
        c.set_trace_path(req.replica_name, req.trace_path, req.global_rank)
        return {"message": "ok"}

    # ---- handshake key/value store (NCCL unique ids, peer-memory IPC handles)
    @app.post(S.COSMOS_API_NCCL_COMM_INITIATOR_SUFFIX)
    async def comm_initiator(req: P.HandshakeInitiatorRequest):
        c.kv_put(req.unique_pair_name, req.handle_base64)
        return {"message": "ok"}

    @app.post(S.COSMOS_API_NCCL_COMM_ACCEPTOR_SUFFIX)
    async def comm_acceptor(req: P.HandshakeAcceptorRequest):
        v = await asyncio.to_thread(c.kv_get, req.unique_pair_name, 10.0)
        if v is None:
            return _err("Unique pair name not found", 404)
        return {"handle_base64": v}

    @app.get(S.COSMOS_API_NCCL_COMM_GET_ALL_SUFFIX)
    async def comm_all():
        return {"comm_info": c.kv_all()}

    @app.post(S.COSMOS_API_NCCL_COMM_ERROR_SUFFIX)
    async def comm_error(req: P.NcclErrRequest):
        c.set_replica_ncclerror(req.replica_name, req.error)
        return {"message": "ok"}

    @app.post(S.COSMOS_API_NCCL_COMM_STORE_CLEAR_SUFFIX)
    async def comm_clear(req: P.NcclStoreClearRequest):
        c.kv_clear(req.unique_pair_name)
        return {"message": "ok"}

    @app.post(S.COSMOS_API_IPC_INFO_SUFFIX)
    async def ipc_info(req: P.IpcInfoRequest):
        c.kv_put("ipc:" + req.mesh_key, req.ipc_addr)
        return {"message": "ok"}

    @app.post(S.COSMOS_API_QUERY_IPC_INFO_SUFFIX)
    async def query_ipc_info(req: P.QueryIpcInfoRequest):
        v = await asyncio.to_thread(c.kv_get, "ipc:" + req.mesh_key, 10.0)
        if v is None:
            return _err("mesh key not found", 404)
        return {"ipc_addr": v}

    # ---- data plane
    @app.get(S.COSMOS_API_NEXT_PROMPT_SUFFIX)
    async def next_prompt(n: int, validation_step: Optional[int] = None, rank_in_mesh: Optional[int] = None):
        batch, is_end = c.get_batched_prompt(n, validation_step)
        return {"prompt_id_and_payload_list": [(i, p.model_dump()) for i, p in batch], "is_end": is_end}

    @app.post(S.COSMOS_API_ROLLOUT_SUFFIX)
    async def rollout(req: P.RolloutRequest):
        await asyncio.to_thread(c.put_rollouts, req.src_replica_name, req.payloads, req.is_end, req.metrics)
        return {"message": "Rollout put"}

    @app.post(S.COSMOS_API_VALIDATION_REPORT_SUFFIX)
    async def validation_report(req: P.ValidationReportRequest):
        c.put_validation_report(req.src_replica_name, req.validation_step, req.payloads, req.is_end)
        return {"message": "ok"}

    @app.post(S.COSMOS_API_POLICY_TRAIN_ACK_SUFFIX)
    async def train_ack(req: P.TrainAckRequest):
        await asyncio.to_thread(c.train_ack, req.replica_name, req.weight_step, req.total_steps,
                                req.profile_finished, req.report_data)
        return {"message": "ok"}

    @app.post(S.COSMOS_API_POLICY_SHARD_INFOS_SUFFIX)
    async def policy_shard_infos(request: Request):
        c.set_shard_infos("policy", msgpack.unpackb(await request.body(), raw=False, strict_map_key=False))
        return {"message": "ok"}

    @app.post(S.COSMOS_API_ROLLOUT_SHARD_INFOS_SUFFIX)
    async def rollout_shard_infos(request: Request):
        c.set_shard_infos("rollout", msgpack.unpackb(await request.body(), raw=False, strict_map_key=False))
        return {"message": "ok"}

    @app.post(S.COSMOS_API_POLICY_SHARD_SEND_INSTS_SUFFIX)
    async def policy_send_insts(req: P.GetShardSendRecvInstsRequest):
        from ..parallel.reshard import plan_for_rank
        plan = await asyncio.to_thread(plan_for_rank, c.get_shard_infos("policy"), c.get_shard_infos("rollout"),
                                       "policy", req.rank)
        return JSONResponse({"insts_b64": base64.b64encode(msgpack.packb(plan)).decode()})

    @app.post(S.COSMOS_API_ROLLOUT_SHARD_RECV_INSTS_SUFFIX)
    async def rollout_recv_insts(req: P.GetShardSendRecvInstsRequest):
        from ..parallel.reshard import plan_for_rank
        plan = await asyncio.to_thread(plan_for_rank, c.get_shard_infos("policy"), c.get_shard_infos("rollout"),
                                       "rollout", req.rank)
        return JSONResponse({"insts_b64": base64.b64encode(msgpack.packb(plan)).decode()})

    @app.get(S.COSMOS_API_SHARD_INFOS_SUFFIX)
    async def shard_infos(role: str):
        infos = c.get_shard_infos(role)
        if infos is None:
            return {"infos_b64": None}
        return {"infos_b64": base64.b64encode(msgpack.packb(infos, use_bin_type=True)).decode()}

    @app.get(S.COSMOS_API_GET_TRAINABLE_PARAMS_SUFFIX)
    async def trainable_params():
        infos = c.get_shard_infos("policy") or {}
        return {"trainable_params": infos.get("trainable_params", [])}

    @app.post(S.COSMOS_API_RESUME_INFO_SUFFIX)
    async def resume_info(req: P.ResumeInfoRequest):
        c.set_resume_info(req.ckpt_extra_info)
        return {"message": "ok"}

    # ---- stream broker (replaces the external Redis server)
    @app.get(S.COSMOS_API_STREAM_READ_SUFFIX)
    async def stream_read(stream: str, last_id: int = 0, count: int = 1, block_ms: int = 0, group: str = ""):
        if group:       # consumer-group read: every message goes to exactly one reader of the group (teacher requests)
            msgs = await asyncio.to_thread(c.broker.read_group, stream, group, count, min(block_ms, 5000))
        else:
            msgs = await asyncio.to_thread(c.broker.read, stream, last_id, count, min(block_ms, 5000))
        return {"messages": [{"id": i, "data": base64.b64encode(d).decode()} for i, d in msgs]}

    @app.post(S.COSMOS_API_STREAM_PUBLISH_SUFFIX)
    async def stream_publish(body: Dict[str, Any]):
        mid = c.broker.publish(body["stream"], base64.b64decode(body["data"]))
        return {"id": mid}

    @app.api_route(S.COSMOS_API_KV_SUFFIX, methods=["GET", "POST"])
    async def kv(request: Request):
        if request.method == "GET":
            v = c.broker.kv_get(request.query_params["key"])
            return {"value": base64.b64encode(v).decode() if v is not None else None}
        body = await request.json()
        if body.get("delete"):
            c.broker.kv_del(body["key"])
        else:
            c.broker.kv_set(body["key"], base64.b64decode(body["value"]), body.get("ttl_s"))
        return {"message": "ok"}

    return app


def serve(controller: Controller, host: str = "0.0.0.0", port: int = 8000, listen_fd: Optional[int] = None,
          log_level: str = "warning"):
    """Blocking: run uvicorn until the process is told to stop."""
    import uvicorn
    app = create_app(controller)
    controller.start_monitor()
    cfg = uvicorn.Config(app, host=host, port=port, log_level=log_level, access_log=False)
    server = uvicorn.Server(cfg)
    if listen_fd is not None:
        sock = socket.socket(fileno=listen_fd)
        server.run(sockets=[sock])
    else:
        server.run()


def main(argv=None, dataset=None, val_dataset=None, custom_logger_fns=None, sampler=None):
    ap = argparse.ArgumentParser(description="cosmos-rl controller")
    ap.add_argument("--config", required=True)
    ap.add_argument("--port", type=int, default=8000)
    ap.add_argument("--host", default="0.0.0.0")
    ap.add_argument("--self-terminate", action="store_true",
                    help="exit (SIGTERM to self) once every replica has unregistered")
    args, _ = ap.parse_known_args(argv)
    config = Config.from_dict(load_toml(args.config))
    controller = Controller(config, dataset=dataset, val_dataset=val_dataset, custom_logger_fns=custom_logger_fns,
                            sampler=sampler)
    controller.self_terminate = args.self_terminate or os.environ.get("COSMOS_CONTROLLER_SELF_TERMINATE") == "1"
    fd = os.environ.get("COSMOS_CONTROLLER_LISTEN_FD")
    logger.info("[Controller] listening on %s:%d", args.host, args.port)
    serve(controller, args.host, args.port, int(fd) if fd else None)


if __name__ == "__main__":
    main()
