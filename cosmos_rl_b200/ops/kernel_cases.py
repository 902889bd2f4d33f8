"""Small, self-contained launches of each sm_100a kernel for timing and profiling.

    python -m cosmos_rl_b200.ops.kernel_cases <case> [--iters N]

Every case uses inputs larger than the 126 MB L2 (so DRAM figures mean something) but at most a few GB,
launches the kernel ``--iters`` times after 3 warm-up launches, times the launches with CUDA events and
prints achieved bandwidth / FLOP rate next to the measured machine peaks (``MEASURED_PEAKS.json`` at the
repository root when present, else 6.65 TB/s and 1.59 PFLOP/s).
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys

import torch

from . import functional as F
from . import native, optim


def peaks():
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    p = os.path.join(root, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["hbm_gbs"] * 1e9, d["bf16_tflops"] * 1e12, "measured"
    return 6.65e12, 1.59e15, "fallback"


def timed(fn, iters: int) -> float:
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters / 1e3


def timed_graph(fn, iters: int, inner: int = 8) -> float:
    """Device time per call of ``fn`` when ``inner`` calls are replayed from one CUDA graph (no host launch cost
    between kernels, which is how the decode step runs them)."""
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        for _ in range(2):
            fn()
    torch.cuda.current_stream().wait_stream(s)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for _ in range(inner):
            fn()
    return timed(g.replay, iters) / inner


def report(name: str, seconds: float, nbytes: float = 0.0, flops: float = 0.0) -> None:
    bw, fl, kind = peaks()
    line = f"{name}: {seconds * 1e6:.1f} us"
    if nbytes:
        line += f" | {nbytes / seconds / 1e9:.0f} GB/s = {nbytes / seconds / bw:.2f} of {kind} HBM copy bandwidth"
    if flops:
        line += f" | {flops / seconds / 1e12:.0f} TFLOP/s = {flops / seconds / fl:.2f} of {kind} cuBLAS bf16"
    print(line, flush=True)


def bf(*shape, scale=1.0):
    return (torch.randn(*shape, device="cuda") * scale).to(torch.bfloat16)


def case_gemm(iters):
    M, N, K = 8192, 8192, 4096
    a, b = bf(M, K), bf(N, K)
    c = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    t = timed(lambda: F.gemm_nt(a, b, out=c), iters)
    report(f"gemm_bf16_nt {M}x{N}x{K}", t, flops=2.0 * M * N * K)


def case_gemm_shapes(iters):
    """Every dense projection of the Qwen2.5-7B block on 8192 tokens (forward, input gradient, weight gradient) and
    the lm_head-sized GEMM: the CTA-pair kernel, the single-CTA kernel and the library GEMM side by side."""
    T, H, I, Q = 8192, 3584, 18944, 4608
    shapes = [("qkv fwd", T, Q, H, 0, 0), ("o fwd", T, H, H, 0, 0), ("gate_up fwd", T, 2 * I, H, 0, 0),
              ("down fwd", T, H, I, 0, 0), ("qkv dgrad", T, H, Q, 0, 1), ("gate_up dgrad", T, H, 2 * I, 0, 1),
              ("down dgrad", T, I, H, 0, 1), ("qkv wgrad", Q, H, T, 1, 1), ("gate_up wgrad", 2 * I, H, T, 1, 1),
              ("down wgrad", H, I, T, 1, 1), ("square 8192x8192x4096", 8192, 8192, 4096, 0, 0)]
    _, fl, kind = peaks()
    for name, M, N, K, a_mn, b_mn in shapes:
        a = bf(K, M) if a_mn else bf(M, K)
        b = bf(K, N) if b_mn else bf(N, K)
        c = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
        tp = timed(lambda: F.gemm(a, b, a_mn=bool(a_mn), b_mn=bool(b_mn), out=c, path=2), iters)
        ts = timed(lambda: F.gemm(a, b, a_mn=bool(a_mn), b_mn=bool(b_mn), out=c, path=1), iters)
        at = a.t() if a_mn else a
        bt = b if b_mn else b.t()
        tl = timed(lambda: torch.matmul(at, bt, out=c), iters)
        fl_ = 2.0 * M * N * K
        print(f"{name} {M}x{N}x{K}: pair {tp * 1e6:.0f} us = {fl_ / tp / 1e12:.0f} TFLOP/s ({fl_ / tp / fl:.2f} of {kind} "
              f"cuBLAS peak) | single-CTA {ts * 1e6:.0f} us = {fl_ / ts / 1e12:.0f} | library {tl * 1e6:.0f} us = "
              f"{fl_ / tl / 1e12:.0f} | pair/library time {tp / tl:.2f}", flush=True)
        del a, b, c


def case_gemm_pair(iters):
    """One shape on the CTA-pair kernel (profiling target)."""
    M, N, K = 8192, 8192, 4096
    a, b = bf(M, K), bf(N, K)
    c = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    t = timed(lambda: F.gemm(a, b, out=c, path=2), iters)
    report(f"gemm_bf16 CTA pairs {M}x{N}x{K}", t, flops=2.0 * M * N * K)


def case_decode_gemms(iters):
    """The four projections of a Qwen2.5-7B block and the lm_head at a decode batch of 128 rows: weight-streaming
    split-K kernel (with its fused reductions) against the library GEMM. Bytes = the weight matrix, read once."""
    Bm, H, I, Q, V = 128, 3584, 18944, 4608, 152064
    x, act, o = bf(Bm, H), bf(Bm, I), bf(Bm, H)
    res = bf(Bm, H)
    nw = torch.ones(H, dtype=torch.bfloat16, device="cuda")
    # several copies of each weight so that consecutive launches do not find it in L2
    n_copies = 4
    ws = {"qkv": [bf(Q, H, scale=0.02) for _ in range(n_copies)], "o": [bf(H, H, scale=0.02) for _ in range(n_copies)],
          "gate_up": [bf(2 * I, H, scale=0.02) for _ in range(n_copies)],
          "down": [bf(H, I, scale=0.02) for _ in range(n_copies)], "lm_head": [bf(V, H, scale=0.02) for _ in range(2)]}
    bq = bf(Q)
    pos = torch.arange(Bm, device="cuda", dtype=torch.int64)
    slots = torch.arange(Bm, device="cuda", dtype=torch.int32)
    cache = torch.zeros(2, 2, 4, 128, 128, dtype=torch.bfloat16, device="cuda")
    k = [0]

    def rot(name):
        k[0] += 1
        return ws[name][k[0] % len(ws[name])]

    cases = [
        ("qkv + bias + rope + kv append", Q * H, lambda: F.skinny_qkv_rope_append(x, rot("qkv"), bq, pos, slots, 1e6, 28, 4, 128, cache, True),
         lambda: torch.nn.functional.linear(x, rot("qkv"), bq)),
        ("o_proj + residual + rmsnorm", H * H, lambda: F.skinny_linear_residual_rmsnorm(o, rot("o"), res, nw, 1e-6),
         lambda: torch.nn.functional.linear(o, rot("o"))),
        ("gate_up + swiglu", 2 * I * H, lambda: F.skinny_gate_up_swiglu(x, rot("gate_up")),
         lambda: torch.nn.functional.linear(x, rot("gate_up"))),
        ("down_proj + residual + rmsnorm", H * I, lambda: F.skinny_linear_residual_rmsnorm(act, rot("down"), res, nw, 1e-6),
         lambda: torch.nn.functional.linear(act, rot("down"))),
        ("lm_head", V * H, lambda: F.gemm_skinny(x, rot("lm_head")), lambda: torch.nn.functional.linear(x, rot("lm_head"))),
    ]
    bw, _, kind = peaks()
    for name, nel, ours, lib in cases:
        to = timed_graph(ours, iters)
        tl = timed_graph(lib, iters)
        nbytes = 2.0 * nel
        print(f"decode M={Bm} {name}: ours {to * 1e6:.1f} us = {nbytes / to / 1e9:.0f} GB/s ({nbytes / to / bw:.2f} of {kind} "
              f"HBM copy) | library GEMM alone {tl * 1e6:.1f} us = {nbytes / tl / 1e9:.0f} GB/s", flush=True)


def case_gemm_fp8(iters):
    M, N, K = 8192, 8192, 8192
    a, b = bf(M, K), bf(N, K, scale=0.05)
    aq, sa = F.quant_fp8_block(a, 1)
    bq, sb = F.quant_fp8_block(b, 128)
    t = timed(lambda: F.gemm_fp8_block(aq, sa, bq, sb), iters)
    report(f"gemm_fp8_block (1x128 / 128x128 scales) {M}x{N}x{K}", t, flops=2.0 * M * N * K)
    t = timed(lambda: F.quant_fp8_block(a, 1), iters)
    report(f"quant_fp8 1x128 activations {M}x{K}", t, nbytes=M * K * 3.0)


def case_fp8_train(iters):
    """A projection of the Qwen2.5-7B block (gate_up: 3584 -> 37888) forward + backward on 8192 tokens: the three
    GEMMs on the block-scaled fp8 kernel (with the quantisation and transposes they need) against bf16 cuBLAS."""
    M, N, K = 8192, 37888, 3584
    go = bf(M, N)

    def run(w):
        x = bf(M, K).requires_grad_(True)
        w.grad = None
        F.linear_maybe_fp8(x, w).backward(go)

    w16 = bf(N, K, scale=0.03).requires_grad_(True)
    t16 = timed(lambda: run(w16), iters)
    report(f"linear fwd+bwd bf16 (cuBLAS) {M}x{N}x{K}", t16, flops=6.0 * M * N * K)
    w8 = bf(N, K, scale=0.03).requires_grad_(True)
    w8._fp8_train = True
    t8 = timed(lambda: run(w8), iters)
    report(f"linear fwd+bwd fp8 block-scaled (incl. quantisation, transposes) {M}x{N}x{K}", t8, flops=6.0 * M * N * K)
    print(f"fp8 / bf16 time: {t8 / t16:.2f}", flush=True)


def case_moe(iters):
    """One MoE layer of the Qwen3-30B-A3B architecture: 128 experts, top-8, hidden 2048, expert FFN 768."""
    from . import moe
    T, H, I, E, k = 16384, 2048, 768, 128, 8
    x = bf(T, H).requires_grad_(True)
    wgu = bf(E, 2 * I, H, scale=0.02).requires_grad_(True)
    wd = bf(E, H, I, scale=0.02).requires_grad_(True)
    logits = torch.randn(T, E, device="cuda")
    t = timed(lambda: moe.route_topk(logits, k), iters)
    report(f"moe route_topk T={T} E={E} k={k}", t, nbytes=T * E * 4.0)
    probs, idx = moe.route_topk(logits, k)
    flops_fwd = 2.0 * T * k * H * 3 * I
    with torch.no_grad():
        t = timed(lambda: moe.moe_experts(x, probs, idx, wgu, wd), iters)
    report(f"moe experts fwd (permute + grouped GEMM + SwiGLU + grouped GEMM + combine) T={T}", t, flops=flops_fwd)
    y = moe.moe_experts(x, probs, idx, wgu, wd)
    g = torch.randn_like(y)
    t = timed(lambda: torch.autograd.grad(y, (x, wgu, wd), g, retain_graph=True), iters)
    report(f"moe experts bwd (dgrad + wgrad grouped GEMMs, recomputed SwiGLU) T={T}", t, flops=2 * flops_fwd)


def case_logprob(iters):
    T, V, H = 4096, 152064, 3584
    h, w = bf(T, H), bf(V, H, scale=0.02)
    lab = torch.randint(0, V, (T,), device="cuda")
    t = timed(lambda: F.fused_logprob(h, w, lab, 1.0), iters)
    report(f"lmhead_logprob fwd T={T} V={V} H={H}", t, flops=2.0 * T * V * H)


def case_dlogits(iters):
    T, V, H = 4096, 32768, 3584
    h = bf(T, H).requires_grad_(True)
    w = bf(V, H, scale=0.02).requires_grad_(True)
    lab = torch.randint(0, V, (T,), device="cuda")

    def run():
        lp, ent = F.fused_logprob(h, w, lab, 1.0)
        lp.sum().backward()
        h.grad = None
        w.grad = None
    t = timed(run, iters)
    report(f"lmhead_logprob fwd+bwd T={T} V={V} H={H}", t, flops=8.0 * T * V * H)


def case_decode(iters):
    B, hq, hkv, d, P, L = 128, 28, 4, 128, 128, 1000
    pages = B * 8 + 1
    cache = bf(pages, 2, hkv, P, d)
    bt = (torch.arange(B * 8, device="cuda", dtype=torch.int32) + 1).view(B, 8)
    lens = torch.full((B,), L, dtype=torch.int32, device="cuda")
    q = bf(B, hq, d)
    t = timed(lambda: F.paged_decode(q, cache, bt, lens, v_transposed=True), iters)
    report(f"paged_decode_tc B={B} hq={hq} hkv={hkv} len={L}", t, nbytes=B * 8 * P * hkv * d * 2 * 2)


def case_reshard(iters):
    from ..rollout.weight_sync import PeerWeightSync
    rows, cols = 16384, 16384
    src = bf(rows * cols)
    dst = torch.empty_like(src)
    plan = [[0, 0, cols, 0, cols, rows, cols]]
    ws = PeerWeightSync(dst, plan, {0: src.data_ptr()})
    t = timed(ws.pull, iters)
    report(f"reshard_pull (local source) {rows}x{cols} bf16", t, nbytes=2.0 * rows * cols * 2)


def case_reshard_fp8(iters):
    """Weight-sync pull fused with 128x128 block-scaled fp8 quantisation (local source)."""
    import torch.nn as nn
    from ..parallel.flat import FlatParams
    from ..rollout.weight_sync import Fp8WeightStore, PeerWeightSync
    rows, cols = 16384, 16384
    with torch.device("meta"):
        lin = nn.Linear(cols, rows, bias=False)
    flat = FlatParams(lin, torch.bfloat16, torch.device("cuda"), with_grad=False)
    src = bf(rows * cols)
    store = Fp8WeightStore(flat, skip=())
    ws = PeerWeightSync(flat.data, [[0, 0, cols, 0, cols, rows, cols]], {0: src.data_ptr()}, fp8=store)
    assert ws.n_quant == 1
    t = timed(ws.pull, iters)
    report(f"reshard_pull + fp8 128x128 quantisation (local source) {rows}x{cols}", t, nbytes=3.0 * rows * cols)


def case_quant(iters):
    R, C = 16384, 16384
    w = bf(R, C)
    t = timed(lambda: F.quant_fp8_block(w, 128), iters)
    report(f"quant_fp8_block 128x128 {R}x{C}", t, nbytes=R * C * 3.0)


def case_quant_mxfp4(iters):
    """bf16 -> mxfp4 with the tensor-core scale layout, shape of one gpt-oss style expert stack (512 MB in)."""
    R, C = 32768, 8192
    w = bf(R, C)
    t = timed(lambda: F.quant_mxfp4(w, True), iters)
    report(f"quant_mxfp4 (swizzled scales) {R}x{C}", t, nbytes=R * C * (2.0 + 0.5 + 1.0 / 32))
    q, sf = F.quant_mxfp4(w, True)
    t = timed(lambda: F.dequant_mxfp4(q, sf, True), iters)
    report(f"dequant_mxfp4 {R}x{C}", t, nbytes=R * C * (2.0 + 0.5 + 1.0 / 32))


def case_rmsnorm(iters):
    T, H = 65536, 3584
    x, r, w = bf(T, H), bf(T, H), bf(H)
    t = timed(lambda: F.rms_norm(x, w, 1e-6, r), iters)
    report(f"rmsnorm_fwd(+residual) T={T} H={H}", t, nbytes=T * H * 2.0 * 4)
    xg = x.clone().requires_grad_(True)
    wg = w.clone().requires_grad_(True)
    y, _ = F.rms_norm(xg, wg, 1e-6)
    g = torch.randn_like(y)
    t = timed(lambda: torch.autograd.grad(y, (xg, wg), g, retain_graph=True), iters)
    report(f"rmsnorm_bwd T={T} H={H}", t, nbytes=T * H * 2.0 * 3)


def case_swiglu(iters):
    T, I = 32768, 18944
    gu = bf(T, 2 * I)
    t = timed(lambda: F.swiglu(gu), iters)
    report(f"swiglu_fwd T={T} I={I}", t, nbytes=T * I * 2.0 * 3)


def case_rope(iters):
    T, hq, hkv, d = 65536, 28, 4, 128
    qkv = bf(T, (hq + 2 * hkv) * d)
    pos = torch.arange(T, device="cuda") % 4096
    t = timed(lambda: F.rope_qkv_(qkv, pos, hq, hkv, d, 1e6), iters)
    report(f"rope_qkv T={T}", t, nbytes=T * (hq + hkv) * d * 2.0 * 2)


def case_adamw(iters):
    n = 1 << 26
    master = torch.randn(n, device="cuda")
    m, v = torch.zeros_like(master), torch.zeros_like(master)
    g = bf(n, scale=0.01)
    shadow = master.to(torch.bfloat16)
    coef = torch.ones(1, device="cuda")
    t = timed(lambda: optim.adamw_flat(master, m, v, g, shadow, lr=1e-4, beta1=0.9, beta2=0.999, eps=1e-8,
                                       weight_decay=0.01, step=3, grad_scale=coef), iters)
    report(f"adamw_flat n={n}", t, nbytes=n * (12 + 2 + 12 + 2.0))


def case_sample(iters):
    B, V = 512, 152064
    logits = torch.randn(B, V, device="cuda")
    temp = torch.ones(B, device="cuda")
    t = timed(lambda: F.sample(logits, temp, None, None, seed=1, offset=2), iters)
    report(f"sample B={B} V={V} (no truncation: 3 passes over the row, 2 served by L2)", t, nbytes=B * V * 4.0)


def case_flash_small(iters):
    """Profiling-sized variant of ``flash`` (4 sequences x 2048 tokens)."""
    case_flash(iters, B=4, L=2048, library=False)


def case_flash(iters, B=16, L=4096, library=True):
    """Packed causal attention forward + backward, Qwen2.5-7B head layout: 16 sequences x 4096 tokens."""
    from . import attention
    hq, hkv, d = 28, 4, 128
    T = B * L
    qkv = bf(T, (hq + 2 * hkv) * d)
    q, k, v = qkv.split([hq * d, hkv * d, hkv * d], dim=-1)
    q, k, v = q.unflatten(-1, (hq, d)), k.unflatten(-1, (hkv, d)), v.unflatten(-1, (hkv, d))
    cu = torch.arange(0, T + 1, L, device="cuda", dtype=torch.int32)
    flops = 4.0 * B * hq * d * L * L / 2            # causal: half of the score matrix
    t = timed(lambda: attention.flash_fwd(q, k, v, cu, cu, L, 1.0 / math.sqrt(d)), iters)
    report(f"flash_fwd tcgen05 B={B} L={L} hq={hq} hkv={hkv}", t, flops=flops)
    if library:
        from flash_attn import flash_attn_varlen_func
        t = timed(lambda: flash_attn_varlen_func(q, k, v, cu, cu, L, L, causal=True), iters)
        report(f"flash_attn library fwd (same shape)", t, flops=flops)
    out, lse = attention.flash_fwd(q, k, v, cu, cu, L, 1.0 / math.sqrt(d))
    go = torch.randn_like(out)
    t = timed(lambda: attention.flash_bwd(go, q, k, v, out, lse, cu, L, 1.0 / math.sqrt(d)), iters)
    report(f"flash_bwd tcgen05 (same shape, incl. delta pre-pass and dQ cast)", t, flops=2.5 * flops)
    if library:
        t = timed(lambda: attention.flash_bwd_library(go, q, k, v, out, lse, cu, L, 1.0 / math.sqrt(d)), iters)
        report(f"flash_attn library bwd (same shape)", t, flops=2.5 * flops)
    assert native.read_status(q.device) == 0


CASES = {"gemm_shapes": case_gemm_shapes, "gemm_pair": case_gemm_pair, "decode_gemms": case_decode_gemms, "quant_mxfp4": case_quant_mxfp4, "fp8_train": case_fp8_train, "reshard_fp8": case_reshard_fp8, "moe": case_moe, "gemm_fp8": case_gemm_fp8, "flash": case_flash, "flash_small": case_flash_small, "gemm": case_gemm, "logprob": case_logprob, "dlogits": case_dlogits, "decode": case_decode,
         "reshard": case_reshard, "quant": case_quant, "rmsnorm": case_rmsnorm, "swiglu": case_swiglu,
         "rope": case_rope, "adamw": case_adamw, "sample": case_sample}


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=sorted(CASES) + ["all"])
    ap.add_argument("--iters", type=int, default=10)
    a = ap.parse_args(argv)
    torch.manual_seed(0)
    for name in (sorted(CASES) if a.case == "all" else [a.case]):
        CASES[name](a.iters)
        native.read_status(torch.device("cuda", torch.cuda.current_device()))
        torch.cuda.empty_cache()


if __name__ == "__main__":
    main()
