"""What every worker shares: identity, controller client, registration, heartbeat, command plumbing
(cosmos_rl/comm/base.py:59-560)."""
from __future__ import annotations

import os
import queue
import socket
import threading
import time
import uuid
from typing import Any, Callable, Dict, List, Optional

import torch.distributed as dist

from ..dispatcher import command as cmd
from ..dispatcher.api.client import APIClient
from ..utils import constant
from ..utils.logging import logger
from .broker import command_stream, rollout_stream


class CommMixin:
    role: str = ""

    def init_comm(self, api=None) -> None:
        self.global_rank = dist.get_rank() if dist.is_initialized() else 0
        self.world_size = dist.get_world_size() if dist.is_initialized() else 1
        # one name for the whole replica: rank 0 draws it, everybody learns it
        names = [os.environ.get("COSMOS_REPLICA_NAME") or str(uuid.uuid4())]
        if self.world_size > 1:
            dist.broadcast_object_list(names, src=0)
        self.replica_name = names[0]
        self.api = api or APIClient(self.role)
        self.broker = self.api.broker()
        self.shutdown_signal = threading.Event()
        self._cmd_queue: "queue.Queue[cmd.Command]" = queue.Queue()
        self._last_cmd_id = 0
        self._threads: List[threading.Thread] = []
        self.register_to_controller()

    # ------------------------------------------------------------------ registration / heartbeat
    def register_to_controller(self) -> None:
        names, ranks, sizes = self.parallel_dims.mesh_register_fields()
        try:
            host_ip = socket.gethostbyname(socket.gethostname())
        except Exception:
            host_ip = "127.0.0.1"
        self.api.register(self.replica_name, self.role, names, ranks, sizes, self.global_rank, host_ip,
                          socket.gethostname())
        if self.world_size > 1:
            dist.barrier()
        if self.global_rank == 0:
            if constant.COSMOS_HEARTBEAT_PROCESS and hasattr(self.api, "base_urls"):
                # a separate process keeps reporting while this one sits in a long native call that holds the
                # interpreter; it is killed by the kernel when this process dies, so a dead worker falls silent
                from .heartbeat_process import start_heartbeat_process
                self._heartbeat_proc = start_heartbeat_process(self.api.base_urls, self.replica_name,
                                                               constant.COSMOS_HEARTBEAT_SEND_INTERVAL)
                return
            t = threading.Thread(target=self._heartbeat_loop, name="heartbeat", daemon=True)
            t.start()
            self._threads.append(t)

    def _heartbeat_loop(self) -> None:
        while not self.shutdown_signal.wait(constant.COSMOS_HEARTBEAT_SEND_INTERVAL):
            try:
                self.api.heartbeat(self.replica_name)
            except Exception as e:
                logger.warning("[%s] heartbeat failed: %s", self.role, e)

    def unregister_from_controller(self) -> None:
        if self.global_rank == 0:
            try:
                self.api.unregister(self.replica_name)
            except Exception as e:
                logger.warning("[%s] unregister failed: %s", self.role, e)

    # ------------------------------------------------------------------ commands
    def start_command_thread(self) -> None:
        if self.global_rank != 0:
            return

        def loop():
            stream = command_stream(self.replica_name)
            while not self.shutdown_signal.is_set():
                try:
                    msgs = self.broker.read(stream, self._last_cmd_id, count=5, block_ms=500)
                except Exception as e:
                    logger.warning("[%s] command read failed: %s", self.role, e)
                    time.sleep(0.5)
                    continue
                for mid, data in msgs:
                    self._last_cmd_id = mid
                    try:
                        c = cmd.Command.depack(data)
                        self.on_command_received(c, data)
                        self._cmd_queue.put(c)
                    except Exception as e:
                        logger.error("[%s] undecodable command: %s", self.role, e)

        t = threading.Thread(target=loop, name="fetch_command", daemon=True)
        t.start()
        self._threads.append(t)

    def on_command_received(self, c: "cmd.Command", raw: bytes) -> None:
        """Called on the command thread (rank 0) for every command, before it is queued for the main loop. Workers
        override it for commands that must take effect while the main loop is busy (membership changes)."""

    def next_command(self, timeout: float = 0.0) -> Optional[cmd.Command]:
        """Rank 0 pops a command; every rank of the replica returns the same one."""
        c = None
        if self.global_rank == 0:
            try:
                c = self._cmd_queue.get(timeout=timeout) if timeout > 0 else self._cmd_queue.get_nowait()
            except queue.Empty:
                c = None
        if self.world_size > 1:
            box = [c.to_dict() if c is not None else None]
            dist.broadcast_object_list(box, src=0)
            c = cmd.Command.from_dict(box[0]) if box[0] is not None else None
        return c
