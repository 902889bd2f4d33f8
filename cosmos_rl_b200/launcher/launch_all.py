"""``cosmos-rl`` launcher: read the job file, size and place the replicas, reserve the controller port, start
the controller and one ``torchrun`` group per replica, forward pre-emption signals to the policy processes
and supervise everything (cosmos_rl/launcher/launch_all.py:104-1017, launcher/utility.py:454-850).

    cosmos-rl --config job.toml [--policy N] [--rollout M] [--port P] [--log-dir DIR] [user_script.py ...]
"""
from __future__ import annotations

import argparse
import os
import signal
import socket
import subprocess
import sys
import tempfile
import time
from typing import Dict, List, Optional, Tuple

from ..config import Config, dump_toml, load_toml
from ..utils.logging import logger


def parse_args(argv=None):
    ap = argparse.ArgumentParser(prog="cosmos-rl", description="launch a cosmos-rl job on this node")
    ap.add_argument("--config", required=True)
    ap.add_argument("--url", default=None, help="address of an already running controller (host:port)")
    ap.add_argument("--port", type=int, default=None)
    ap.add_argument("--policy", type=int, default=None, help="number of policy replicas")
    ap.add_argument("--rollout", type=int, default=None, help="number of rollout replicas")
    ap.add_argument("--reference", type=int, default=None, help="number of reference (teacher) replicas")
    ap.add_argument("--p2r-ratio", type=str, default=None, help="policy:rollout replica ratio, e.g. 1:2; the node's "
                                                                "GPUs are divided accordingly")
    ap.add_argument("--log-dir", default=None)
    ap.add_argument("--num-workers", type=int, default=1, help="number of nodes of the job")
    ap.add_argument("--worker-idx", type=int, default=0, help="index of this node")
    ap.add_argument("--node-ip-list", default=None, help="semicolon separated node addresses (multi-node)")
    ap.add_argument("--rdzv-port", type=int, default=29345)
    ap.add_argument("--gpus-per-node", type=int, default=None,
                    help="GPUs of every node of the job (default: what this node shows); with --cpu it is the number "
                         "of ranks one node hosts")
    ap.add_argument("--cpu", action="store_true", help="run every replica on CPU (gloo); for plumbing tests")
    ap.add_argument("--share-gpus", action="store_true",
                    help="let replicas wrap around the node's GPUs when the job asks for more than there are (several "
                         "replicas then share a GPU; for functional tests on small machines, not for performance)")
    ap.add_argument("--tolerate-replica-failures", action="store_true",
                    help="a replica that exits abnormally does not take the job down: the controller reaps it after "
                         "its heartbeat stops and the remaining replicas carry on (elastic jobs)")
    ap.add_argument("--no-controller", action="store_true")
    ap.add_argument("script", nargs="?", default=None)
    ap.add_argument("script_args", nargs=argparse.REMAINDER)
    return ap.parse_args(argv)


def gpus_per_replica(par) -> int:
    """tp * dp_replicate * pp * cp * dp_shard (dp_shard -1/0 counts as 1 until the world size is known)."""
    return par.tp_size * max(par.dp_replicate_size, 1) * par.pp_size * par.cp_size * max(par.dp_shard_size, 1)


def replica_counts(config: Config, args, n_gpus: int) -> Tuple[int, int, int]:
    is_sft = config.train.train_policy.type == "sft"
    n_policy = args.policy if args.policy is not None else config.policy.parallelism.n_init_replicas
    n_rollout = 0 if is_sft else (args.rollout if args.rollout is not None else
                                  config.rollout.parallelism.n_init_replicas)
    n_ref = args.reference if args.reference is not None else (
        config.distillation.parallelism.n_init_replicas if config.distillation.enable else 0)
    if args.p2r_ratio and not is_sft and n_gpus > 0:
        p, r = (int(x) for x in args.p2r_ratio.split(":"))
        gp, gr = gpus_per_replica(config.policy.parallelism), gpus_per_replica(config.rollout.parallelism)
        unit = p * gp + r * gr
        k = max(1, n_gpus // unit)
        n_policy, n_rollout = p * k, r * k
    if config.mode == "colocated":
        if n_policy != n_rollout and n_rollout != 0:
            raise ValueError("colocated mode needs as many rollout replicas as policy replicas")
    if config.mode == "colocated_separated":
        # separate policy and rollout processes on the SAME GPUs (weights reach the rollout process through a
        # CUDA IPC mapping of the policy's buffer): replicas pair up one to one on equal GPU counts
        gp, gr = gpus_per_replica(config.policy.parallelism), gpus_per_replica(config.rollout.parallelism)
        if n_policy != n_rollout or gp != gr:
            raise ValueError("colocated_separated mode needs as many rollout replicas as policy replicas, on the same "
                             f"number of GPUs each (got {n_policy} x {gp} and {n_rollout} x {gr})")
    return n_policy, n_rollout, n_ref


def place_replicas(n_policy: int, n_rollout: int, n_ref: int, config: Config, n_gpus: int, colocated: bool,
                   share: bool = False) -> List[Dict]:
    """Assign GPU ids of this node to replicas, policies first. Colocated replicas share the policy's GPUs. With
    ``share`` the ids wrap around instead of running out (``--share-gpus``)."""
    out, next_gpu = [], 0
    sizes = {"policy": gpus_per_replica(config.policy.parallelism),
             "rollout": gpus_per_replica(config.rollout.parallelism),
             "reference": gpus_per_replica(config.distillation.parallelism)}
    policy_gpus: List[List[int]] = []
    for role, n in (("policy", n_policy), ("rollout", n_rollout), ("reference", n_ref)):
        for i in range(n):
            k = sizes[role]
            if colocated and role == "rollout" and i < len(policy_gpus):
                gpus = policy_gpus[i][:k]
            else:
                gpus = list(range(next_gpu, next_gpu + k))
                next_gpu += k
                if share and n_gpus:
                    if k > n_gpus:
                        raise ValueError(f"a {role} replica needs {k} GPUs, this node has {n_gpus}")
                    gpus = [g % n_gpus for g in gpus]
                elif n_gpus and next_gpu > n_gpus:
                    raise ValueError(f"job needs more than the {n_gpus} GPUs of this node "
                                     f"({role} replica {i} wants GPUs {gpus})")
            if role == "policy":
                policy_gpus.append(gpus)
            out.append({"role": role, "index": i, "gpus": gpus, "nproc": k})
    return out


def plan_nodes(n_policy: int, n_rollout: int, n_ref: int, config: Config, gpus_per_node: int) -> List[List[Dict]]:
    """Place every replica of the job on the nodes of the job; every node's launcher computes the same plan and starts
    its own row (cosmos_rl/launcher/utility.py:584-760 does the same walk).

    Roles are placed in the order policy, rollout, reference. A replica that fits a node takes the next free GPUs of
    the current node, or starts the next node when they do not suffice. A replica larger than a node spans
    ``gpus / gpus_per_node`` whole nodes (it must divide), starting on a fresh node; each of those nodes runs one
    ``torchrun`` of the replica with ``nnodes`` / ``node_rank`` and the first node of the span as the rendezvous host.
    In ``colocated_separated`` mode the rollout replicas restart at node 0, GPU 0 (they share the policies' GPUs).
    Entries: ``role, index, ordinal`` (replica number over the whole job, fixes the rendezvous port), ``gpus, nproc,
    nnodes, node_rank, rdzv_node``."""
    G = gpus_per_node
    if G <= 0:
        raise ValueError("gpus_per_node must be positive")
    sizes = {"policy": gpus_per_replica(config.policy.parallelism),
             "rollout": gpus_per_replica(config.rollout.parallelism),
             "reference": gpus_per_replica(config.distillation.parallelism)}
    nodes: List[List[Dict]] = [[]]
    node, gpu, ordinal = 0, 0, 0

    def row(i: int) -> List[Dict]:
        while len(nodes) <= i:
            nodes.append([])
        return nodes[i]

    for role, n in (("policy", n_policy), ("rollout", n_rollout), ("reference", n_ref)):
        if role == "rollout" and config.mode == "colocated_separated":
            node, gpu = 0, 0
        k = sizes[role]
        for i in range(n):
            ordinal += 1
            if k > G:
                if k % G:
                    raise ValueError(f"a {role} replica of {k} GPUs does not divide into nodes of {G}")
                if gpu > 0:
                    node, gpu = node + 1, 0
                span = k // G
                for j in range(span):
                    row(node + j).append({"role": role, "index": i, "ordinal": ordinal, "gpus": list(range(G)),
                                          "nproc": G, "nnodes": span, "node_rank": j, "rdzv_node": node})
                node += span
                continue
            if gpu + k > G:
                node, gpu = node + 1, 0
            row(node).append({"role": role, "index": i, "ordinal": ordinal, "gpus": list(range(gpu, gpu + k)),
                              "nproc": k, "nnodes": 1, "node_rank": 0, "rdzv_node": node})
            gpu += k
    return nodes


def reserve_port(port: Optional[int]) -> Tuple[socket.socket, int]:
    """Bind the controller's listening socket here and hand the descriptor to the controller process, so the
    port cannot be taken by someone else between choosing it and serving on it."""
    s = socket.socket(socket.AF_INET, socket.SOCK_STREAM)
    s.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
    s.bind(("0.0.0.0", port or 0))
    s.listen(128)
    s.set_inheritable(True)
    return s, s.getsockname()[1]


def wait_for_url(url: str, timeout_s: float = 120.0) -> None:
    import requests
    t0 = time.time()
    while time.time() - t0 < timeout_s:
        try:
            if requests.get(url + "/api/meta", timeout=2).status_code == 200:
                return
        except Exception:
            pass
        time.sleep(0.2)
    raise TimeoutError(f"controller at {url} did not come up within {timeout_s:.0f} s")


def is_coordinated_controller_exit(returncode: Optional[int]) -> bool:
    """The controller terminates itself with SIGTERM after every replica has checked out: that is success."""
    return returncode in (0, -signal.SIGTERM, 128 + signal.SIGTERM)


def main(argv=None) -> int:
    args = parse_args(argv)
    raw = load_toml(args.config)
    config = Config.from_dict(raw)
    try:
        import torch
        n_gpus = 0 if args.cpu else torch.cuda.device_count()
    except Exception:
        n_gpus = 0
    per_node = args.gpus_per_node or n_gpus
    n_policy, n_rollout, n_ref = replica_counts(config, args, per_node * max(1, args.num_workers))
    ips = args.node_ip_list.split(";") if args.node_ip_list else []
    if args.num_workers > 1:
        # a job of several nodes: --policy / --rollout count the replicas of the WHOLE job, every node's launcher
        # derives the same plan and starts its own row of it
        plan = plan_nodes(n_policy, n_rollout, n_ref, config, per_node)
        if len(plan) > args.num_workers:
            raise ValueError(f"the job needs {len(plan)} nodes of {per_node} GPUs, --num-workers is {args.num_workers}")
        if any(e["nnodes"] > 1 for row in plan for e in row) and len(ips) < len(plan):
            raise ValueError("a replica spans several nodes: --node-ip-list must name every node of the job")
        placement = plan[args.worker_idx] if args.worker_idx < len(plan) else []
    else:
        placement = place_replicas(n_policy, n_rollout, n_ref, config, n_gpus,
                                   config.mode in ("colocated", "colocated_separated"), share=args.share_gpus)
    log_dir = None
    if args.log_dir:
        log_dir = os.path.join(args.log_dir, time.strftime("logs_%Y%m%d-%H%M%S"))
        os.makedirs(log_dir, exist_ok=True)
        latest = os.path.join(args.log_dir, "logs_latest")
        tmp = latest + f".tmp{os.getpid()}"
        os.symlink(os.path.basename(log_dir), tmp)
        os.replace(tmp, latest)

    if raw.get("train", {}).get("timestamp") == "auto":
        # a fresh sub-folder per launch, stamped once here so that every process of the job sees the same path
        # (the reference stamps whenever train.timestamp is empty, cosmos_rl/policy/config/__init__.py:1883-1897;
        # here an empty value keeps output_dir as written, which is what a resumed job needs)
        raw["train"]["timestamp"] = time.strftime("%Y%m%d%H%M%S")
        raw["train"]["output_dir"] = os.path.join(raw["train"].get("output_dir", "./outputs"), raw["train"]["timestamp"])
    # the job file the controller serves carries the replica counts actually launched
    raw.setdefault("policy", {}).setdefault("parallelism", {})["n_init_replicas"] = max(n_policy, 1)
    raw.setdefault("rollout", {}).setdefault("parallelism", {})["n_init_replicas"] = max(n_rollout, 1)
    tmp_cfg = tempfile.NamedTemporaryFile("w", suffix=".toml", delete=False)
    tmp_cfg.write(dump_toml(raw))
    tmp_cfg.close()

    procs: List[Tuple[str, subprocess.Popen]] = []
    env_base = dict(os.environ)
    env_base.setdefault("NCCL_CUMEM_ENABLE", "0")
    script = [args.script] + list(args.script_args) if args.script else None

    def spawn(name: str, cmd: List[str], env: Dict[str, str], pass_fds=()):
        out = open(os.path.join(log_dir, f"{name}.log"), "w") if log_dir else None
        p = subprocess.Popen(cmd, env=env, stdout=out or None, stderr=subprocess.STDOUT if out else None,
                             pass_fds=pass_fds)
        procs.append((name, p))
        return p

    if config.mode == "colocated" and config.train.train_policy.type != "sft":
        # policy, rollout and the controller logic share one process (and one set of weights): no controller
        # process, no rollout replicas (cosmos_rl/colocated/rl_worker.py:41-229)
        env = dict(env_base, COSMOS_ROLE="Colocated", COSMOS_CONFIG=tmp_cfg.name)
        if args.cpu or not n_gpus:
            env["CUDA_VISIBLE_DEVICES"] = ""
        target = script if script else ["-m", "cosmos_rl_b200.launcher.worker_entry"]
        p = spawn("colocated_0", [sys.executable] + target, env)
        try:
            rc = p.wait()
        except KeyboardInterrupt:
            p.terminate()
            rc = p.wait()
        os.unlink(tmp_cfg.name)
        return rc

    controller = None
    if args.url:
        host = args.url
    elif args.worker_idx > 0:
        # a further node of the job: the controller lives on node 0 at the agreed port
        if not (ips and args.port):
            raise ValueError("a node with --worker-idx > 0 needs --url, or --node-ip-list together with --port")
        host = f"{ips[0]}:{args.port}"
        wait_for_url(f"http://{host}", timeout_s=600.0)
    else:
        sock, port = reserve_port(args.port)
        host = f"127.0.0.1:{port}"
        if not args.no_controller and args.worker_idx == 0:
            env = dict(env_base, COSMOS_ROLE="Controller", COSMOS_CONTROLLER_LISTEN_FD=str(sock.fileno()),
                       COSMOS_CONTROLLER_SELF_TERMINATE="1")
            cmd = [sys.executable] + (script if script else ["-m", "cosmos_rl_b200.dispatcher.run_web_panel"]) + \
                  ["--config", tmp_cfg.name, "--port", str(port)]
            controller = spawn("controller", cmd, env, pass_fds=(sock.fileno(),))
            wait_for_url(f"http://{host}")
        sock.close()
    ctrl_hosts = host if not ips else ";".join(f"{ip}:{host.split(':')[1]}" for ip in ips[:1])

    rdzv = args.rdzv_port
    for rep in placement:
        env = dict(env_base, COSMOS_ROLE=rep["role"].capitalize(), COSMOS_CONTROLLER_HOST=ctrl_hosts,
                   COSMOS_REPLICA_TAG=f"{rep['role']}_{rep['index']}")
        if args.num_workers > 1:
            env["COSMOS_NODE_INDEX"] = str(args.worker_idx)
        if rep["gpus"] and n_gpus:
            env["CUDA_VISIBLE_DEVICES"] = ",".join(str(g) for g in rep["gpus"])
        elif args.cpu or not n_gpus:
            env["CUDA_VISIBLE_DEVICES"] = ""
        if config.mode != "colocated_separated":
            env.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")
        module = {"policy": "cosmos_rl_b200.policy.train", "rollout": "cosmos_rl_b200.rollout.rollout_entry",
                  "reference": "cosmos_rl_b200.reference.reference_entry"}[rep["role"]]
        target = script if script else ["-m", module]
        rdzv += 1
        nnodes, master, port_ = rep.get("nnodes", 1), "127.0.0.1", rdzv
        if "ordinal" in rep:
            port_ = args.rdzv_port + rep["ordinal"]          # the same port on every node of the replica's span
        if nnodes > 1 and rep["rdzv_node"] != args.worker_idx:
            master = ips[rep["rdzv_node"]]
        cmd = [sys.executable, "-m", "torch.distributed.run", f"--nnodes={nnodes}",
               f"--nproc-per-node={max(1, rep['nproc'])}", "--master-addr", master, "--master-port", str(port_)]
        if nnodes > 1:
            cmd += [f"--node-rank={rep['node_rank']}"]
        cmd += target if script else ["--module", module]
        spawn(f"{rep['role']}_{rep['index']}", cmd, env)

    policy_procs = [p for n, p in procs if n.startswith("policy")]

    def forward(signum, _frame):
        for p in policy_procs:
            try:
                p.send_signal(signum)
            except Exception:
                pass

    for name in config.train.signal_to_handle:
        sig = getattr(signal, name, None)
        if sig is not None:
            signal.signal(sig, forward)

    # supervise: a failing replica or controller takes the job down; the controller's own SIGTERM is success
    rc = 0
    lost = set()
    try:
        while True:
            alive = False
            for name, p in procs:
                code = p.poll()
                if code is None:
                    alive = True
                    continue
                if name == "controller":
                    if not is_coordinated_controller_exit(code):
                        logger.error("controller exited with %s", code)
                        rc = code or 1
                        raise KeyboardInterrupt
                elif code != 0:
                    if args.tolerate_replica_failures:
                        if name not in lost:
                            lost.add(name)
                            logger.warning("%s exited with %s; the job continues without it", name, code)
                        continue
                    logger.error("%s exited with %s", name, code)
                    rc = code
                    raise KeyboardInterrupt
            workers_alive = any(p.poll() is None for n, p in procs if n != "controller")
            if not workers_alive:
                break
            time.sleep(0.5)
    except KeyboardInterrupt:
        pass
    finally:
        deadline = time.time() + 10
        for name, p in procs:
            if p.poll() is None and (name != "controller" or rc != 0 or time.time() > deadline):
                p.terminate()
        for name, p in procs:
            try:
                p.wait(timeout=15)
            except subprocess.TimeoutExpired:
                p.kill()
        os.unlink(tmp_cfg.name)
    return rc


if __name__ == "__main__":
    sys.exit(main())
