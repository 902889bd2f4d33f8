"""Preflight for the payload transport and the dynamic communicators, run on a node before a job is sent to it.

    python -m cosmos_rl_b200.tools.profiler.check_nccl [-v] [--broker HOST:PORT]

Checks, each reported as ok / WARN / FAIL: torch and the device; the native library and its status word; that the
transport named ``nccl`` is registered; that a rendezvous store can be opened on a local port; a real loop-back
transfer through two ``PairTransport`` ends in this process (request / answer handshake over an in-process broker, a
two-rank communicator on gloo, one tensor out and back, cleanup); the controller's broker when an address is given.
On a GPU node the NCCL library version and the tuning variables of the environment are printed for the record. Exit
code 0 when no check failed. The reference ships a preflight of the same purpose
(cosmos_rl/tools/profiler/check_nccl.py); a two-rank NCCL transfer needs two GPUs and is covered by the multi-GPU tests.
"""
from __future__ import annotations

import argparse
import os
import sys
import time
from typing import Callable, List, Tuple


def run_checks(verbose: bool = False, broker_addr: str = "") -> List[Tuple[str, str, str]]:
    out: List[Tuple[str, str, str]] = []

    def check(name: str, fn: Callable[[], str], critical: bool = True) -> None:
        try:
            out.append((name, "ok", fn() or ""))
        except Exception as e:  # noqa: BLE001  (a preflight reports, it does not raise)
            out.append((name, "FAIL" if critical else "WARN", f"{type(e).__name__}: {e}"))

    def torch_and_device() -> str:
        import torch
        if not torch.cuda.is_available():
            return f"torch {torch.__version__}, no CUDA device (communicators fall back to gloo)"
        p = torch.cuda.get_device_properties(0)
        return f"torch {torch.__version__}, {torch.cuda.device_count()} x {p.name} (sm_{p.major}{p.minor}, {p.total_memory >> 30} GiB)"

    def native_library() -> str:
        import torch
        from ...ops import native
        if not torch.cuda.is_available():
            return "skipped without a device"
        lib = native.lib()
        dev = torch.device("cuda", 0)
        native.status_word(dev)
        return f"{getattr(lib, '_name', 'libb200rl')} loaded, status word {native.read_status(dev)}"

    def nccl_version() -> str:
        import torch
        if not torch.cuda.is_available():
            return "skipped without a device"
        v = torch.cuda.nccl.version()
        env = {k: v2 for k, v2 in os.environ.items() if k.startswith("NCCL_") or k.startswith("COSMOS_NCCL")}
        return f"NCCL {'.'.join(map(str, v))}; environment: {env or 'no NCCL_* variables set'}"

    def transport_registered() -> str:
        from ...utils.payload_transport import PayloadTransportRegistry
        t = PayloadTransportRegistry.get("nccl")
        return f"{type(t).__name__}, references start with {t.completion_prefix!r}"

    def rendezvous_store() -> str:
        from datetime import timedelta
        import torch.distributed as dist
        from ...utils.misc import free_port, local_ips
        port = free_port("0.0.0.0")
        master = dist.TCPStore("0.0.0.0", port, 1, is_master=True, timeout=timedelta(seconds=5), wait_for_workers=False)
        client = dist.TCPStore("127.0.0.1", port, 1, is_master=False, timeout=timedelta(seconds=5))
        client.set("k", "v")
        assert master.get("k") == b"v"
        return f"TCPStore on port {port}; addresses a peer would try: {local_ips()}"

    def loopback_transfer() -> str:
        import torch
        from ...comm.broker import InProcessBroker
        from ...utils.payload_transport.pair import PairTransport
        broker = InProcessBroker()
        prod, cons = PairTransport(), PairTransport()
        cpu = torch.device("cpu")                      # one process cannot hold both ranks of an NCCL communicator
        prod.setup(broker=broker, device=cpu, owner="preflight-producer", recv_timeout_s=5.0)
        cons.setup(broker=broker, device=cpu, owner="preflight-consumer", recv_timeout_s=5.0)
        try:
            x = torch.arange(1 << 16, dtype=torch.float32)
            t0 = time.perf_counter()
            got = cons.sync_fetch(prod.publish(x))
            dt = time.perf_counter() - t0
            if got is None or not torch.equal(got, x):
                raise RuntimeError("the tensor did not come back intact")
            return f"{x.numel() * 4 >> 10} KiB through handshake + two-rank communicator in {dt * 1e3:.0f} ms"
        finally:
            prod.shutdown()
            cons.shutdown()

    def controller_broker() -> str:
        import urllib.request
        host, _, port = broker_addr.partition(":")
        with urllib.request.urlopen(f"http://{host}:{port or 8000}/api/status", timeout=3) as r:
            return f"controller answered {r.status}"

    check("torch / device", torch_and_device)
    check("native library", native_library)
    check("NCCL", nccl_version, critical=False)
    check("transport registered", transport_registered)
    check("rendezvous store", rendezvous_store)
    check("loop-back transfer", loopback_transfer)
    if broker_addr:
        check("controller broker", controller_broker, critical=False)
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("-v", "--verbose", action="store_true")
    ap.add_argument("--broker", default=os.environ.get("COSMOS_CONTROLLER_HOST", ""),
                    help="HOST:PORT of a running controller (optional)")
    a = ap.parse_args(argv)
    results = run_checks(a.verbose, a.broker)
    for name, status, detail in results:
        print(f"[{status:>4}] {name}: {detail}")
    failed = [n for n, s, _ in results if s == "FAIL"]
    print("preflight " + ("FAILED: " + ", ".join(failed) if failed else "passed"))
    return 1 if failed else 0


if __name__ == "__main__":
    sys.exit(main())
