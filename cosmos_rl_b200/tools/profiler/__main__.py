"""``python -m cosmos_rl_b200.tools.profiler analyze logs/*.log``: summarise ``[Trace]`` lines of a run and
``check_nccl``: a preflight that reports what the collective stack of this box looks like
(cosmos_rl/tools/profiler/README.md:17-60)."""
import argparse
import glob
import json
import sys

from ...utils.trace import parse_lines, summarize


def analyze(paths):
    recs = []
    for pat in paths:
        for p in glob.glob(pat):
            with open(p, errors="replace") as f:
                recs.extend(parse_lines(f))
    table = summarize(recs)
    print(f"{'worker:op':50s} {'count':>7s} {'total s':>10s} {'mean ms':>10s} {'max ms':>10s}")
    for k, s in sorted(table.items(), key=lambda kv: -kv[1]["total"]):
        print(f"{k:50s} {s['count']:7d} {s['total']:10.3f} {s['mean'] * 1e3:10.2f} {s['max'] * 1e3:10.2f}")
    return table


def check_nccl():
    import torch
    info = {"torch": torch.__version__, "cuda": torch.version.cuda, "gpus": torch.cuda.device_count()}
    try:
        info["nccl"] = ".".join(str(x) for x in torch.cuda.nccl.version())
    except Exception as e:
        info["nccl"] = f"unavailable: {e}"
    if torch.cuda.device_count() > 1:
        info["p2p"] = [[torch.cuda.can_device_access_peer(i, j) if i != j else True
                        for j in range(torch.cuda.device_count())] for i in range(torch.cuda.device_count())]
    print(json.dumps(info, indent=2))
    return info


def main(argv=None):
    ap = argparse.ArgumentParser(prog="cosmos_rl_b200.tools.profiler")
    sub = ap.add_subparsers(dest="cmd", required=True)
    a = sub.add_parser("analyze")
    a.add_argument("logs", nargs="+")
    sub.add_parser("check_nccl")
    args = ap.parse_args(argv)
    if args.cmd == "analyze":
        analyze(args.logs)
    else:
        check_nccl()


if __name__ == "__main__":
    main()
