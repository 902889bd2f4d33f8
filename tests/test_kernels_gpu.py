"""Numerics of every sm_100a kernel against the fp32 PyTorch statements in ops/reference.py."""
import math

import pytest
import torch

from cosmos_rl_b200.ops import functional as F
from cosmos_rl_b200.ops import native, reference as R

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _bf16(*shape, scale=1.0):
    return (torch.randn(*shape, device=DEV) * scale).to(torch.bfloat16)


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (300, 1000, 520), (1024, 3584, 3584),
                                   (77, 128, 64), (4096, 152, 1024)])
def test_gemm_bf16_nt(M, N, K):
    torch.manual_seed(0)
    a, b = _bf16(M, K), _bf16(N, K)
    c = F.gemm_nt(a, b)
    native.read_status(a.device)
    ref = a.float() @ b.float().t()
    err = (c.float() - ref).abs().max().item()
    tol = 2e-2 * math.sqrt(K) + 1e-2 * ref.abs().max().item()
    assert err < tol, (err, tol)
    # tight check against a bf16-rounded fp32 result
    assert torch.allclose(c.float(), ref.to(torch.bfloat16).float(), rtol=2e-2, atol=1e-2 * math.sqrt(K))


def test_gemm_fp32_accumulate():
    torch.manual_seed(1)
    a, b = _bf16(256, 512), _bf16(384, 512)
    out = torch.ones(256, 384, dtype=torch.float32, device=DEV)
    F.gemm_nt(a, b, out=out, accumulate=True)
    native.read_status(a.device)
    ref = a.float() @ b.float().t() + 1.0
    assert torch.allclose(out, ref, rtol=1e-3, atol=1e-2)


@pytest.mark.parametrize("T,V,H,temp", [(100, 1000, 128, 1.0), (257, 5000, 256, 0.7), (1024, 32000, 512, 1.0)])
def test_fused_logprob_fwd_bwd(T, V, H, temp):
    torch.manual_seed(2)
    h = _bf16(T, H).requires_grad_(True)
    w = _bf16(V, H, scale=0.05).requires_grad_(True)
    labels = torch.randint(0, V, (T,), device=DEV)
    labels[::7] = -100
    lp, ent = F.fused_logprob(h, w, labels, temp)
    native.read_status(h.device)
    hr = h.detach().float().requires_grad_(True)
    wr = w.detach().float().requires_grad_(True)
    lpr, entr = R.logprob_entropy(hr, wr, labels, temp)
    assert torch.allclose(lp, lpr, rtol=1e-3, atol=2e-3), (lp - lpr).abs().max()
    assert torch.allclose(ent, entr, rtol=1e-3, atol=2e-3), (ent - entr).abs().max()
    g1 = torch.randn(T, device=DEV)
    g2 = torch.randn(T, device=DEV) * 0.1
    (lp * g1 + ent * g2).sum().backward()
    native.read_status(h.device)
    (lpr * g1 + entr * g2).sum().backward()
    assert torch.allclose(h.grad.float(), hr.grad, rtol=5e-2, atol=5e-2 * hr.grad.abs().max().item())
    assert torch.allclose(w.grad.float(), wr.grad, rtol=5e-2, atol=5e-2 * wr.grad.abs().max().item())


@pytest.mark.parametrize("T,H", [(33, 256), (1000, 3584), (64, 8192)])
@pytest.mark.parametrize("with_res", [False, True])
def test_rmsnorm(T, H, with_res):
    torch.manual_seed(3)
    x = _bf16(T, H).requires_grad_(True)
    w = (1 + 0.1 * torch.randn(H, device=DEV)).to(torch.bfloat16).requires_grad_(True)
    res = _bf16(T, H).requires_grad_(True) if with_res else None
    y, ro = F.rms_norm(x, w, 1e-6, res)
    xr = x.detach().float().requires_grad_(True)
    wr = w.detach().float().requires_grad_(True)
    rr = res.detach().float().requires_grad_(True) if with_res else None
    h = (xr + rr).to(torch.bfloat16).float() if with_res else xr
    if with_res:
        # straight-through for the bf16 rounding of the residual stream
        h = (xr + rr) + (h - (xr + rr)).detach()
    yr = h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + 1e-6) * wr
    assert torch.allclose(y.float(), yr, rtol=2e-2, atol=2e-2)
    gy = torch.randn_like(yr)
    loss = (y.float() * gy).sum()
    lossr = (yr * gy).sum()
    if with_res:
        gr = torch.randn_like(yr)
        loss = loss + (ro.float() * gr).sum()
        lossr = lossr + (h * gr).sum()
    loss.backward()
    lossr.backward()
    assert torch.allclose(x.grad.float(), xr.grad, rtol=3e-2, atol=3e-2)
    assert torch.allclose(w.grad.float(), wr.grad, rtol=3e-2, atol=3e-2 * wr.grad.abs().max().item())
    if with_res:
        assert torch.allclose(res.grad.float(), rr.grad, rtol=3e-2, atol=3e-2)


def test_rope_qkv_fwd_bwd():
    torch.manual_seed(4)
    T, hq, hkv, d = 50, 4, 2, 128
    base = _bf16(T, (hq + 2 * hkv) * d)
    pos = torch.randint(0, 4000, (T,), device=DEV)
    a = base.clone().requires_grad_(True)
    out = F.rope_qkv_(a * 1.0, pos, hq, hkv, d, 1e6)
    b = base.detach().cpu().float().requires_grad_(True)
    outr = F.rope_qkv_(b, pos.cpu(), hq, hkv, d, 1e6)
    assert torch.allclose(out.float().cpu(), outr, rtol=2e-2, atol=2e-2)
    g = torch.randn_like(outr)
    (out.float() * g.to(DEV)).sum().backward()
    (outr * g).sum().backward()
    assert torch.allclose(a.grad.float().cpu(), b.grad, rtol=2e-2, atol=2e-2)


def test_swiglu():
    torch.manual_seed(5)
    gu = _bf16(300, 2 * 1024).requires_grad_(True)
    y = F.swiglu(gu)
    gr = gu.detach().float().requires_grad_(True)
    yr = R.swiglu(gr)
    assert torch.allclose(y.float(), yr, rtol=2e-2, atol=2e-2)
    g = torch.randn_like(yr)
    (y.float() * g).sum().backward()
    (yr * g).sum().backward()
    assert torch.allclose(gu.grad.float(), gr.grad, rtol=3e-2, atol=3e-2)


def test_adamw_and_clip():
    from cosmos_rl_b200.ops import optim
    torch.manual_seed(6)
    n = 100003
    master = torch.randn(n, device=DEV)
    m = torch.zeros(n, device=DEV)
    v = torch.zeros(n, device=DEV)
    shadow = master.to(torch.bfloat16)
    mr, mm, vv = master.clone(), m.clone(), v.clone()
    for step in range(1, 4):
        grad = (torch.randn(n, device=DEV) * 0.1).to(torch.bfloat16)
        norm, coef = optim.grad_norm_and_clip([grad], 1.0)
        ref_norm = grad.float().norm()
        assert abs(norm.item() - ref_norm.item()) < 1e-2 * ref_norm.item()
        optim.adamw_flat(master, m, v, grad, shadow, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01,
                         step=step, grad_scale=coef)
        R.adamw_step(mr, mm, vv, grad, 1e-3, 0.9, 0.999, 1e-8, 0.01, step, grad_scale=min(1.0, 1.0 / (ref_norm.item() + 1e-6)))
    assert torch.allclose(master, mr, rtol=1e-4, atol=1e-5)
    assert torch.allclose(shadow.float(), mr.to(torch.bfloat16).float(), rtol=1e-2, atol=1e-2)


def test_sampling_distribution_and_logprob():
    torch.manual_seed(7)
    B, V = 64, 1000
    logits = torch.randn(1, V, device=DEV).repeat(B, 1) * 2
    temp = torch.full((B,), 0.8, device=DEV)
    counts = torch.zeros(V, device=DEV)
    n_rounds = 200
    for i in range(n_rounds):
        toks, lps = F.sample(logits, temp, None, None, seed=123, offset=i)
        counts.index_add_(0, toks, torch.ones(B, device=DEV))
    p = torch.softmax(logits[0] / 0.8, -1)
    emp = counts / counts.sum()
    assert (emp - p).abs().sum().item() < 0.15  # total variation small with 12800 draws
    lsm = torch.log_softmax(logits[0] / 0.8, -1)
    assert torch.allclose(lps, lsm[toks], rtol=1e-4, atol=1e-4)
    # greedy
    toks, _ = F.sample(logits, torch.zeros(B, device=DEV), None, None, seed=1, offset=0)
    assert (toks == logits[0].argmax()).all()
    # top-k / top-p restrict the support
    topk = torch.full((B,), 5, dtype=torch.int32, device=DEV)
    allowed = set(torch.topk(logits[0], 5).indices.tolist())
    for i in range(20):
        toks, _ = F.sample(logits, temp, None, topk, seed=5, offset=i)
        assert set(toks.tolist()) <= allowed
    topp = torch.full((B,), 0.5, device=DEV)
    sp, si = torch.sort(p, descending=True)
    ncut = int((sp.cumsum(0) < 0.5).sum()) + 1
    allowed = set(si[:ncut + 1].tolist())
    for i in range(20):
        toks, _ = F.sample(logits, temp, topp, None, seed=9, offset=i)
        assert set(toks.tolist()) <= allowed


@pytest.mark.parametrize("hq,hkv,d", [(28, 4, 128), (8, 8, 128), (16, 2, 64)])
def test_paged_decode_and_append(hq, hkv, d):
    torch.manual_seed(8)
    B, page_size, n_pages = 5, 16, 64
    cache = torch.zeros(n_pages, 2, hkv, page_size, d, dtype=torch.bfloat16, device=DEV)
    seq_lens = torch.tensor([1, 17, 100, 160, 33], dtype=torch.int32, device=DEV)
    max_pages = 12
    perm = torch.randperm(n_pages, device=DEV)[: B * max_pages].view(B, max_pages).to(torch.int32)
    # append all tokens through the kernel
    ks, vs, slots = [], [], []
    for b in range(B):
        L = int(seq_lens[b])
        ks.append(_bf16(L, hkv, d))
        vs.append(_bf16(L, hkv, d))
        t = torch.arange(L, device=DEV)
        slots.append(perm[b, t // page_size].long() * page_size + t % page_size)
    k, v, slot = torch.cat(ks), torch.cat(vs), torch.cat(slots).to(torch.int32)
    F.kv_append(k, v, cache, slot)
    cache_ref = torch.zeros_like(cache).cpu()
    R.kv_append(k.cpu(), v.cpu(), cache_ref, slot.cpu())
    assert torch.equal(cache.cpu(), cache_ref)
    q = _bf16(B, hq, d)
    ref = R.paged_decode(q.cpu(), cache_ref, perm.cpu(), seq_lens.cpu())
    for nsplit in (1, 4):
        out = F.paged_decode(q, cache, perm, seq_lens, nsplit=nsplit)
        assert torch.allclose(out.float().cpu(), ref.float(), rtol=2e-2, atol=2e-2), nsplit


@pytest.mark.parametrize("R_,C", [(256, 384), (300, 200), (128, 128)])
def test_quant_fp8(R_, C):
    torch.manual_seed(9)
    w = _bf16(R_, C)
    q, s = F.quant_fp8_block(w, 128)
    qr, sr = R.quant_fp8_block(w.cpu(), 128, 128)
    assert torch.allclose(s.cpu(), sr, rtol=1e-5)
    deq = R.dequant_fp8_block(q.cpu(), s.cpu())
    assert (deq - w.cpu().float()).abs().max() <= 0.07 * w.abs().max().item()
    assert (q.cpu().float() - qr.float()).abs().max() <= 32  # at most one e4m3 ulp at the top binade
    qa, sa = F.quant_fp8_block(w, 1)
    deqa = R.dequant_fp8_block(qa.cpu(), sa.cpu(), 1, 128)
    assert (deqa - w.cpu().float()).abs().max() <= 0.07 * w.abs().max().item()


@pytest.mark.parametrize("hq,hkv", [(28, 4), (8, 8), (64, 8), (4, 4)])
def test_paged_decode_tensor_core(hq, hkv):
    """tcgen05 decode kernel (V stored transposed, 128-token pages) against the fp32 statement."""
    torch.manual_seed(10)
    d, P, B, n_pages, max_pages = 128, 128, 7, 64, 6
    cache = torch.zeros(n_pages, 2, hkv, P, d, dtype=torch.bfloat16, device=DEV)
    seq_lens = torch.tensor([1, 127, 128, 129, 500, 768, 300], dtype=torch.int32, device=DEV)
    perm = torch.stack([torch.randperm(n_pages - 1, device=DEV)[:max_pages] + 1 for _ in range(B)]).to(torch.int32)
    ks, vs, slots = [], [], []
    for b in range(B):
        L = int(seq_lens[b])
        ks.append(_bf16(L, hkv, d))
        vs.append(_bf16(L, hkv, d))
        t = torch.arange(L, device=DEV)
        slots.append(perm[b, t // P].long() * P + t % P)
    k, v, slot = torch.cat(ks), torch.cat(vs), torch.cat(slots).to(torch.int32)
    F.kv_append(k, v, cache, slot, v_transposed=True)
    cache_ref = torch.zeros_like(cache).cpu()
    R.kv_append(k.cpu(), v.cpu(), cache_ref, slot.cpu(), v_transposed=True)
    assert torch.equal(cache.cpu(), cache_ref)
    q = _bf16(B, hq, d)
    ref = R.paged_decode(q.cpu(), cache_ref, perm.cpu(), seq_lens.cpu(), v_transposed=True)
    for nsplit in (1, 3):
        out = F.paged_decode(q, cache, perm, seq_lens, nsplit=nsplit, v_transposed=True)
        native.read_status(q.device)
        err = (out.float().cpu() - ref.float()).abs().max().item()
        assert err < 3e-2, (nsplit, err)


@pytest.mark.parametrize("a_mn,b_mn", [(False, True), (True, True), (True, False)])
@pytest.mark.parametrize("M,N,K", [(256, 512, 384), (300, 200, 520), (1024, 3584, 2048)])
def test_gemm_operand_layouts(a_mn, b_mn, M, N, K):
    """dgrad (B stored [K, N]) and wgrad (both stored [K, *]) forms against fp32 matmul."""
    torch.manual_seed(11)
    K8 = K
    a = _bf16(K8, (M + 7) // 8 * 8)[:, :M] if a_mn else _bf16(M, K8)
    b = _bf16(K8, (N + 7) // 8 * 8)[:, :N] if b_mn else _bf16(N, K8)
    out = F.gemm(a, b, a_mn=a_mn, b_mn=b_mn)
    native.read_status(a.device)
    af = a.float().t() if a_mn else a.float()
    bf_ = b.float().t() if b_mn else b.float()
    ref = af @ bf_.t()
    assert torch.allclose(out.float(), ref, rtol=2e-2, atol=1e-2 * math.sqrt(K)), (out.float() - ref).abs().max()


def test_linear_tc_matches_torch_linear():
    torch.manual_seed(12)
    x = _bf16(512, 1024).requires_grad_(True)
    w = _bf16(768, 1024, scale=0.05).requires_grad_(True)
    b = _bf16(768).requires_grad_(True)
    y = F.linear_tc(x, w, b)
    native.read_status(x.device)
    g = _bf16(512, 768)
    y.backward(g)
    native.read_status(x.device)
    xr, wr, br = (t.detach().float().requires_grad_(True) for t in (x, w, b))
    yr = torch.nn.functional.linear(xr, wr, br)
    yr.backward(g.float())
    assert torch.allclose(y.float(), yr, rtol=2e-2, atol=0.3)
    assert torch.allclose(x.grad.float(), xr.grad, rtol=2e-2, atol=0.3)
    assert torch.allclose(w.grad.float(), wr.grad, rtol=2e-2, atol=0.5)
    # second backward accumulates into the existing .grad inside the GEMM epilogue
    y2 = F.linear_tc(x.detach(), w, None)
    y2.backward(g)
    assert torch.allclose(w.grad.float(), 2 * wr.grad, rtol=3e-2, atol=1.0)


def test_moe_router_topk():
    from cosmos_rl_b200.ops import moe
    torch.manual_seed(13)
    T, E, k = 777, 128, 8
    logits = torch.randn(T, E, device=DEV) * 2
    counts = torch.zeros(E, dtype=torch.int32, device=DEV)
    p, i = moe.route_topk(logits, k, True, counts)
    pr, ir = moe.route_topk_reference(logits, k, True)
    assert torch.equal(i.long().sort(-1).values, ir.long().sort(-1).values)
    assert torch.allclose(p.sort(-1).values, pr.sort(-1).values, rtol=1e-4, atol=1e-6)
    assert torch.equal(counts.long(), torch.bincount(ir.flatten().long(), minlength=E))


@pytest.mark.parametrize("T,H,I,E,k", [(300, 256, 128, 8, 2), (1024, 2048, 768, 16, 8), (64, 512, 256, 32, 4)])
def test_moe_experts_fwd_bwd(T, H, I, E, k):
    from cosmos_rl_b200.ops import moe
    torch.manual_seed(14)
    x = _bf16(T, H).requires_grad_(True)
    wgu = _bf16(E, 2 * I, H, scale=0.05).requires_grad_(True)
    wd = _bf16(E, H, I, scale=0.05).requires_grad_(True)
    logits = torch.randn(T, E, device=DEV)
    probs, idx = moe.route_topk(logits, k, True)
    probs = probs.clone().requires_grad_(True)
    out = moe.moe_experts(x, probs, idx, wgu, wd)
    native.read_status(x.device)
    xr, pr, wgur, wdr = (t.detach().float().requires_grad_(True) for t in (x, probs, wgu, wd))
    ref = moe.moe_experts_reference(xr, pr, idx, wgur, wdr)
    scale = ref.abs().max().item()
    assert torch.allclose(out.float(), ref, rtol=3e-2, atol=3e-2 * scale), (out.float() - ref).abs().max()
    g = _bf16(T, H)
    out.backward(g)
    native.read_status(x.device)
    ref.backward(g.float())
    for name, a, b in (("dx", x.grad, xr.grad), ("dprob", probs.grad, pr.grad), ("dwgu", wgu.grad, wgur.grad),
                       ("dwd", wd.grad, wdr.grad)):
        s = b.abs().max().item()
        assert torch.allclose(a.float(), b, rtol=5e-2, atol=5e-2 * s), (name, (a.float() - b).abs().max().item(), s)


def test_rope_separate_qk_autograd_on_views():
    """q / k that are views of another tensor (the per-head-norm path of Qwen3) must work under autograd."""
    torch.manual_seed(15)
    T, hq, hkv, d = 40, 4, 2, 128
    qb = _bf16(T * hq, d).requires_grad_(True)
    kb = _bf16(T * hkv, d).requires_grad_(True)
    pos = torch.randint(0, 3000, (T,), device=DEV)
    q, k = F.apply_rope((qb * 1.0).view(T, hq, d), (kb * 1.0).view(T, hkv, d), pos, 1e6)
    qr = qb.detach().float().cpu().requires_grad_(True)
    kr = kb.detach().float().cpu().requires_grad_(True)
    qe, ke = R.apply_rope(qr.view(T, hq, d), kr.view(T, hkv, d), pos.cpu(), 1e6)
    assert torch.allclose(q.float().cpu(), qe, rtol=2e-2, atol=2e-2)
    (q.float().sum() + 2 * k.float().sum()).backward()
    (qe.sum() + 2 * ke.sum()).backward()
    assert torch.allclose(qb.grad.float().cpu(), qr.grad, rtol=2e-2, atol=2e-2)
    assert torch.allclose(kb.grad.float().cpu(), kr.grad, rtol=2e-2, atol=2e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("over", [
    {}, {"kl_beta": 0.05}, {"kl_beta": 0.05, "unbiased_kl_estimate": True}, {"aipo_rho": 1.1},
    {"use_decoupled_loss": True, "behav_imp_weight_cap": 1.3, "kl_beta": 0.01},
    {"loss_type": "seq-mean-token-mean", "off_policy_masking_delta": 0.05},
    {"loss_type": "seq-mean-token-sum", "epsilon_high": 0.28, "lower_bound_ratio": 1.2},
])
def test_fused_grpo_loss_matches_op_by_op(over):
    from cosmos_rl_b200.policy import loss as L
    torch.manual_seed(3)
    n, n_seq = 5000, 37
    dev = torch.device("cuda")
    base = torch.randn(n, device=dev) - 2.0
    old = base + 0.25 * torch.randn(n, device=dev)
    old[::17] = base[::17]                               # exact ties: ratio == 1
    old[5] = base[5] + 30.0                              # clamp region
    ref = base + 0.1 * torch.randn(n, device=dev)
    roll = old + 0.2 * torch.randn(n, device=dev)
    seq_ids = torch.sort(torch.randint(0, n_seq, (n,), device=dev)).values
    A = torch.randn(n_seq, device=dev)[seq_ids]
    ent = torch.rand(n, device=dev)
    cfg = L.GrpoLossConfig(**over)
    res = {}
    for fused in (False, True):
        L.USE_FUSED_KERNEL = fused
        lp = base.clone().requires_grad_(True)
        loss, m = L.grpo_loss(lp, old, A, seq_ids, n_seq, cfg, ref_logprob=ref, rollout_logprob=roll, entropy=ent)
        loss.backward()
        res[fused] = (loss.detach(), lp.grad.clone(), {k: v.detach() for k, v in m.items()})
    L.USE_FUSED_KERNEL = True
    (l0, g0, m0), (l1, g1, m1) = res[False], res[True]
    assert torch.allclose(l0, l1, rtol=1e-4, atol=1e-6), (l0, l1)
    assert torch.allclose(g0, g1, rtol=1e-4, atol=1e-8), (g0 - g1).abs().max()
    for k in m0:
        assert torch.allclose(m0[k].float(), m1[k].float(), rtol=1e-4, atol=1e-6), k


@pytest.mark.gpu
@pytest.mark.parametrize("lens,hq,hkv", [([128], 2, 1), ([300, 17, 129, 1000], 4, 2), ([2048, 512], 28, 4),
                                         ([1, 1, 5], 8, 8)])
def test_flash_attention_forward_and_lse(lens, hq, hkv):
    from cosmos_rl_b200.ops import attention
    torch.manual_seed(11)
    d, T = 128, sum(lens)
    qkv = torch.randn(T, (hq + 2 * hkv) * d, device="cuda").to(torch.bfloat16)
    q, k, v = qkv.split([hq * d, hkv * d, hkv * d], dim=-1)         # strided views, as the model passes them
    q, k, v = q.unflatten(-1, (hq, d)), k.unflatten(-1, (hkv, d)), v.unflatten(-1, (hkv, d))
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device="cuda")
    scale = 1.0 / math.sqrt(d)
    out, lse = attention.flash_fwd(q, k, v, cu, cu, max(lens), scale)
    torch.cuda.synchronize()
    assert native.read_status(q.device) == 0
    ref = R.varlen_attention(q.float(), k.float(), v.float(), cu, scale)
    assert torch.allclose(out.float(), ref, atol=2e-2, rtol=2e-2), (out.float() - ref).abs().max()
    # log-sum-exp of the scaled scores per (head, token)
    g = hq // hkv
    for b in range(len(lens)):
        s0, s1 = int(cu[b]), int(cu[b + 1])
        qs, ks = q[s0:s1].float(), k[s0:s1].float().repeat_interleave(g, dim=1)
        sc = torch.einsum("qhd,khd->hqk", qs, ks) * scale
        sc = sc.masked_fill(torch.ones(s1 - s0, s1 - s0, device="cuda").triu(1).bool(), float("-inf"))
        assert torch.allclose(lse[:, s0:s1], torch.logsumexp(sc, -1), atol=2e-2, rtol=1e-3)


@pytest.mark.gpu
def test_flash_attention_prefix_aligned_queries():
    """Queries aligned to the end of a longer key sequence (prefill on top of cached keys, CP chunks)."""
    from cosmos_rl_b200.ops import attention
    torch.manual_seed(12)
    d, hq, hkv = 128, 4, 2
    lq, lk = [100, 256], [356, 300]
    q = torch.randn(sum(lq), hq, d, device="cuda").to(torch.bfloat16)
    k = torch.randn(sum(lk), hkv, d, device="cuda").to(torch.bfloat16)
    v = torch.randn(sum(lk), hkv, d, device="cuda").to(torch.bfloat16)
    cq = torch.tensor([0, 100, 356], dtype=torch.int32, device="cuda")
    ck = torch.tensor([0, 356, 656], dtype=torch.int32, device="cuda")
    scale = 1.0 / math.sqrt(d)
    out, _ = attention.flash_fwd(q, k, v, cq, ck, 256, scale)
    assert native.read_status(q.device) == 0
    for b in range(2):
        qs = q[int(cq[b]):int(cq[b + 1])].float()
        ks = k[int(ck[b]):int(ck[b + 1])].float().repeat_interleave(2, dim=1)
        vs = v[int(ck[b]):int(ck[b + 1])].float().repeat_interleave(2, dim=1)
        sc = torch.einsum("qhd,khd->hqk", qs, ks) * scale
        nq, nk = qs.shape[0], ks.shape[0]
        mask = torch.arange(nk, device="cuda")[None, :] > (torch.arange(nq, device="cuda")[:, None] + nk - nq)
        ref = torch.einsum("hqk,khd->qhd", torch.softmax(sc.masked_fill(mask, float("-inf")), -1), vs)
        got = out[int(cq[b]):int(cq[b + 1])].float()
        assert torch.allclose(got, ref, atol=2e-2, rtol=2e-2), (got - ref).abs().max()


@pytest.mark.gpu
@pytest.mark.parametrize("lens,hq,hkv", [([200, 56], 4, 2), ([128], 1, 1), ([300, 17, 129, 700], 14, 2),
                                         ([1, 5, 1500], 8, 8)])
def test_flash_attention_autograd_matches_reference(lens, hq, hkv):
    torch.manual_seed(13)
    d, T = 128, sum(lens)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device="cuda")
    qkv = torch.randn(T, (hq + 2 * hkv) * d, device="cuda").to(torch.bfloat16).requires_grad_(True)
    q, k, v = qkv.split([hq * d, hkv * d, hkv * d], dim=-1)         # strided views, as the model passes them
    go = torch.randn(T, hq, d, device="cuda").to(torch.bfloat16)
    F.varlen_attention(q.unflatten(-1, (hq, d)), k.unflatten(-1, (hkv, d)), v.unflatten(-1, (hkv, d)), cu,
                       max(lens)).backward(go)
    torch.cuda.synchronize()
    assert native.read_status(qkv.device) == 0
    ref = qkv.detach().float().requires_grad_(True)
    rq, rk, rv = ref.split([hq * d, hkv * d, hkv * d], dim=-1)
    R.varlen_attention(rq.unflatten(-1, (hq, d)), rk.unflatten(-1, (hkv, d)), rv.unflatten(-1, (hkv, d)), cu,
                       1.0 / math.sqrt(d)).backward(go.float())
    err = (qkv.grad.float() - ref.grad).abs().max().item()
    assert err <= 3e-2 * ref.grad.abs().max().item() + 2e-2, err


@pytest.mark.gpu
@pytest.mark.parametrize("lq,lk,hq,hkv", [([200, 56], None, 4, 2), ([300, 130], [77, 200], 4, 4), ([64], [333], 2, 1)])
def test_bidirectional_attention_self_and_cross(lq, lk, hq, hkv):
    """Non-causal mode of the attention kernels: every query sees all keys of its sequence, the key sequence may be
    shorter or longer than the query sequence (cross-attention)."""
    torch.manual_seed(14)
    d = 128
    cum = lambda l: torch.tensor([0] + list(torch.tensor(l).cumsum(0)), dtype=torch.int32, device="cuda")
    cq = cum(lq)
    ck = cq if lk is None else cum(lk)
    lk = lq if lk is None else lk
    q = torch.randn(sum(lq), hq, d, device="cuda").to(torch.bfloat16).requires_grad_(True)
    k = torch.randn(sum(lk), hkv, d, device="cuda").to(torch.bfloat16).requires_grad_(True)
    v = torch.randn(sum(lk), hkv, d, device="cuda").to(torch.bfloat16).requires_grad_(True)
    go = torch.randn(sum(lq), hq, d, device="cuda").to(torch.bfloat16)
    out = F.full_attention(q, k, v, cq, ck, max(lq), max(lk))
    out.backward(go)
    torch.cuda.synchronize()
    assert native.read_status(q.device) == 0
    rq, rk, rv = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    ref = R.varlen_attention(rq, rk, rv, cq, 1.0 / math.sqrt(d), causal=False, cu_k=ck)
    ref.backward(go.float())
    assert torch.allclose(out.float(), ref, atol=2e-2, rtol=2e-2), (out.float() - ref).abs().max()
    for got, want in ((q.grad, rq.grad), (k.grad, rk.grad), (v.grad, rv.grad)):
        err = (got.float() - want).abs().max().item()
        assert err <= 3e-2 * want.abs().max().item() + 2e-2, err


@pytest.mark.gpu
@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (300, 520, 1040), (1024, 3584, 3584), (17, 256, 4096)])
def test_gemm_fp8_block_scaled(M, N, K):
    torch.manual_seed(5)
    a = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    a[:, : K // 2] *= 8.0                                  # different scales along K: exercises the promotion
    b = (torch.randn(N, K, device="cuda") * 0.05).to(torch.bfloat16)
    aq, sa = F.quant_fp8_block(a, 1)
    bq, sb = F.quant_fp8_block(b, 128)
    got = F.gemm_fp8_block(aq, sa, bq, sb)
    torch.cuda.synchronize()
    assert native.read_status(a.device) == 0
    ref = R.dequant_fp8_block(aq, sa, 1, 128) @ R.dequant_fp8_block(bq, sb, 128, 128).t()   # same quantised inputs
    err = (got.float() - ref).abs().max().item()
    assert err <= 1e-2 * ref.abs().max().item() + 1e-3, err
    full = a.float() @ b.float().t()                       # and fp8 itself is close to the bf16 product
    assert (got.float() - full).abs().mean().item() <= 0.05 * full.abs().mean().item()
    y = F.fp8_linear(a, bq, sb)
    assert torch.equal(y, got)


@pytest.mark.gpu
@pytest.mark.parametrize("hq,hkv,n", [(28, 4, 4), (8, 8, 8), (64, 8, 3), (28, 4, 8)])
def test_paged_decode_shared_prefix_groups(hq, hkv, n):
    """Groups of n sequences share their first pages; the prefix pass + suffix pass + merge must equal plain
    attention over each sequence's whole block table."""
    torch.manual_seed(14)
    d, P, max_pages, max_shared = 128, 128, 8, 5
    groups = [(3, [400, 385, 500, 700, 384 + 1, 600, 900, 1000]), (0, [5, 100, 128, 129, 300, 1, 7, 64]),
              (5, [641, 700, 1024, 800, 650, 900, 1000, 777])]
    B = len(groups) * n
    n_pages = 1 + len(groups) * (5 + n * max_pages)
    cache = torch.zeros(n_pages, 2, hkv, P, d, dtype=torch.bfloat16, device=DEV)
    free = list(range(1, n_pages))
    bt = torch.zeros(B, max_pages, dtype=torch.int32)
    lens, pref = [], []
    for gi, (shared, ls) in enumerate(groups):
        shared_pages = [free.pop() for _ in range(shared)]
        for j in range(n):
            L = ls[j]
            own = [free.pop() for _ in range(max_pages - shared)]
            bt[gi * n + j] = torch.tensor(shared_pages + own)
            lens.append(L)
            pref.append(shared)
    # fill every page that any sequence can see with random K/V (shared pages hold the same data for the group)
    used = sorted(set(bt.flatten().tolist()))
    for pg in used:
        cache[pg, 0] = _bf16(hkv, P, d)
        cache[pg, 1] = _bf16(hkv, d, P)             # V slabs are stored transposed
    bt_d = bt.to(DEV)
    seq_lens = torch.tensor(lens, dtype=torch.int32, device=DEV)
    prefix = torch.tensor(pref, dtype=torch.int32, device=DEV)
    q = _bf16(B, hq, d)
    ref = R.paged_decode(q.cpu(), cache.cpu(), bt, seq_lens.cpu(), v_transposed=True)
    out = F.paged_decode(q, cache, bt_d, seq_lens, nsplit=1, v_transposed=True, prefix_pages=prefix, group=n,
                         max_shared=max_shared)
    torch.cuda.synchronize()
    assert native.read_status(q.device) == 0
    err = (out.float().cpu() - ref.float()).abs().max().item()
    assert err < 3e-2, err
    # a retired member (prefix 0) must not disturb the others
    prefix2 = prefix.clone()
    prefix2[0] = 0
    out2 = F.paged_decode(q, cache, bt_d, seq_lens, nsplit=1, v_transposed=True, prefix_pages=prefix2, group=n,
                          max_shared=max_shared)
    assert native.read_status(q.device) == 0
    assert (out2[1:].float().cpu() - ref[1:].float()).abs().max().item() < 3e-2


@pytest.mark.gpu
def test_dit_bf16_on_gpu_matches_fp32_reference():
    """Diffusion transformer with head_dim 128: self- and cross-attention run the non-causal tcgen05 kernels."""
    from cosmos_rl_b200.models.dit import DiT, DiTArgs
    torch.manual_seed(0)
    a = DiTArgs(in_channels=4, patch_size=(1, 2, 2), dim=256, n_layers=2, n_heads=2, head_dim=128, ffn_dim=512,
                text_dim=128, freq_dim=64)
    ref = DiT(a)
    ref.init_weights(0)
    with torch.no_grad():
        for n, p in ref.named_parameters():
            if "modulation" in n or n.startswith("patch_out"):
                p.normal_(0, 0.05)
    z, t, text = torch.randn(2, 4, 2, 16, 16), torch.tensor([0.2, 0.8]), torch.randn(2, 9, 128)
    mask = torch.tensor([[1] * 9, [1] * 4 + [0] * 5], dtype=torch.bool)
    want = ref(z, t, text, mask)
    want.square().mean().backward()
    import copy
    gpu = copy.deepcopy(ref).to("cuda", torch.bfloat16)
    gpu.zero_grad()
    got = gpu(z.cuda().to(torch.bfloat16), t.cuda(), text.cuda().to(torch.bfloat16), mask.cuda())
    got.square().mean().backward()
    torch.cuda.synchronize()
    assert native.read_status(torch.device("cuda")) == 0
    assert (got.float().cpu() - want).abs().max() < 0.05 * want.abs().max() + 0.02
    g_ref, g_gpu = ref.layers[0].qkv.weight.grad, gpu.layers[0].qkv.weight.grad.float().cpu()
    assert torch.nn.functional.cosine_similarity(g_ref.flatten(), g_gpu.flatten(), dim=0) > 0.98


@pytest.mark.gpu
@pytest.mark.parametrize("family", ["qwen2_5_vl", "internvl", "qwen3_vl_moe"])
def test_native_vision_language_models_bf16_on_gpu_match_fp32_reference(family):
    """The native vision-language families on the GPU in bf16 (decoder with head_dim 128 on the tcgen05 attention and
    GEMM kernels, vision towers with the head sizes of the public checkpoints) against the same weights in fp32 on the
    CPU: logits of a packed batch with two images, and the gradient that reaches the vision tower."""
    import copy
    torch.manual_seed(0)
    if family == "qwen2_5_vl":
        from cosmos_rl_b200.models.qwen2_5_vl import Qwen25VL, Qwen25VLArgs, VisionArgs
        a = Qwen25VLArgs(vocab_size=2048, dim=512, n_layers=2, n_heads=4, n_kv_heads=2, ffn_dim=1024, rope_theta=1e6,
                         qkv_bias=True, model_type="qwen2_5_vl", mrope_section=[16, 24, 24], image_token_id=2000)
        a.vision = VisionArgs(depth=3, hidden_size=160, num_heads=2, intermediate_size=216, out_hidden_size=512,
                              window_size=56, fullatt_block_indexes=[1])
        ref = Qwen25VL(a)
        grids = torch.tensor([[1, 6, 4], [1, 4, 8]])
        mm = {"pixel_values": torch.randn(56, 3 * 2 * 14 * 14), "image_grid_thw": grids}
        n_img, probe = (6, 8), lambda m: m.visual.blocks[0].qkv.weight
    elif family == "internvl":
        from cosmos_rl_b200.models.internvl import InternViTArgs, InternVL, InternVLArgs
        a = InternVLArgs(vocab_size=2048, dim=512, n_layers=2, n_heads=4, n_kv_heads=2, ffn_dim=1024, rope_theta=1e6,
                         qkv_bias=True, model_type="internvl", image_token_id=2000)
        a.vision = InternViTArgs(hidden_size=128, num_hidden_layers=2, num_attention_heads=2, intermediate_size=256,
                                 image_size=56, patch_size=14)
        ref = InternVL(a)
        mm = {"pixel_values": torch.randn(3, 3, 56, 56)}
        n_img, probe = (8, 4), lambda m: m.visual.blocks[0].q_proj.weight
    else:
        from cosmos_rl_b200.models.qwen3_vl_moe import Qwen3VisionArgs, Qwen3VLMoE, Qwen3VLMoEArgs
        a = Qwen3VLMoEArgs(vocab_size=2048, dim=512, n_layers=3, n_heads=4, n_kv_heads=2, head_dim=128, ffn_dim=512,
                           rope_theta=5e6, qkv_bias=False, qk_norm=True, model_type="qwen3_vl_moe", n_experts=8, top_k=2,
                           moe_ffn_dim=256, mrope_section=[24, 20, 20], image_token_id=2000)
        a.vision = Qwen3VisionArgs(depth=3, hidden_size=144, num_heads=2, intermediate_size=256, out_hidden_size=512,
                                   num_position_embeddings=64, deepstack_visual_indexes=[0, 2])
        ref = Qwen3VLMoE(a)
        grids = torch.tensor([[1, 6, 4], [1, 4, 8]])
        mm = {"pixel_values": torch.randn(56, 3 * 2 * 16 * 16), "image_grid_thw": grids}
        n_img, probe = (6, 8), lambda m: m.visual.blocks[0].qkv.weight
    ref = ref.float()
    with torch.no_grad():
        for n, p in ref.named_parameters():
            if p.dim() > 1:
                p.normal_(0, 0.05)
            else:                               # norm weights 1, layer scales 0.1, biases 0
                p.fill_(1.0 if "norm" in n and not n.endswith("_b") else (0.1 if "scale" in n else 0.0))
        for n, p in ref.named_parameters():
            if n.endswith("mlp.gate.weight"):   # decisive routing: bf16 rounding must not flip the chosen experts
                p.normal_(0, 1.0)
    g = torch.Generator().manual_seed(1)
    seq1 = torch.randint(0, 1900, (40,), generator=g).tolist()
    seq2 = torch.randint(0, 1900, (25,), generator=g).tolist()
    seq1[5:5] = [2000] * n_img[0]
    seq2[3:3] = [2000] * n_img[1]
    ids = torch.tensor(seq1 + seq2)
    cu = torch.tensor([0, len(seq1), len(seq1) + len(seq2)], dtype=torch.int32)
    ref.mm_inputs = mm
    want = ref.logits(ref(ids, ref.get_position_ids(cu, ids.numel()), cu, len(seq1)))
    want.square().mean().backward()
    gpu = copy.deepcopy(ref).to("cuda", torch.bfloat16)
    gpu.zero_grad()
    gpu.mm_inputs = {k: v.cuda() if k == "pixel_values" else v for k, v in mm.items()}
    cu_g = cu.cuda()
    got = gpu.logits(gpu(ids.cuda(), gpu.get_position_ids(cu_g, ids.numel()), cu_g, len(seq1)))
    got.square().mean().backward()
    torch.cuda.synchronize()
    assert native.read_status(torch.device("cuda")) == 0
    err = (got.float().cpu() - want).abs().amax(dim=1)              # per token
    tol = 0.06 * want.abs().max() + 0.03
    if family == "qwen3_vl_moe":       # a token whose second and third expert are nearly tied may still flip
        # the router's bf16 logits put the second and third expert of some tokens within rounding of each other in
        # at least one of the three blocks: those tokens take another expert than the fp32 model and differ by O(1)
        assert (err < tol).float().mean() > 0.7 and err.median() < tol / 3, (family, float(err.max()), float(err.median()))
    else:
        assert err.max() < tol, (family, err.max(), want.abs().max())
    g_ref, g_gpu = probe(ref).grad, probe(gpu).grad.float().cpu()
    cos = torch.nn.functional.cosine_similarity(g_ref.flatten(), g_gpu.flatten(), dim=0)
    assert cos > (0.6 if family == "qwen3_vl_moe" else 0.97), (family, float(cos))   # routing flips change which experts a token trains


@pytest.mark.gpu
@pytest.mark.parametrize("rows,cols,swizzle", [(128, 128, False), (300, 2880, True), (1, 32, True), (257, 96, False)])
def test_mxfp4_quant_matches_reference_bit_for_bit(rows, cols, swizzle):
    torch.manual_seed(9)
    w = (torch.randn(rows, cols, device="cuda") * torch.logspace(-3, 2, rows, device="cuda")[:, None]).to(torch.bfloat16)
    w[0, :32] = 0                                          # an all-zero block takes the smallest scale
    if rows > 2:
        w[2, :8] = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, -5.0], device="cuda") * 4   # ties, amax 20 -> scale 4
        w[2, 8:32] = 0
    q, sf = F.quant_mxfp4(w, swizzle)
    rq, rsf = R.quant_mxfp4(w, swizzle)
    assert torch.equal(q, rq) and torch.equal(sf, rsf)
    back = F.dequant_mxfp4(q, sf, swizzle)
    assert torch.equal(back.float(), R.dequant_mxfp4(rq, rsf, swizzle).to(torch.bfloat16).float())
    # error bound: the grid's largest gap is 2 scales (half of it when rounding), and a block maximum just under
    # 8 scales saturates at 6 scales
    blk = w.float().view(rows, cols // 32, 32)
    scale = torch.exp2(torch.floor(torch.log2(blk.abs().amax(-1).clamp_min(1e-30))) - 2)
    assert ((back.float().view(rows, cols // 32, 32) - blk).abs() <= scale[..., None] * 2.0 + 1e-30).all()


@pytest.mark.gpu
@pytest.mark.parametrize("M,N,K", [(1024, 4608, 3584), (304, 256, 1040)])
def test_fp8_training_linear_on_gpu(M, N, K):
    """All three GEMMs of a projection on the block-scaled fp8 kernel against the exact fp32 products."""
    torch.manual_seed(6)
    x = torch.randn(M, K, device="cuda").to(torch.bfloat16).requires_grad_(True)
    w = (torch.randn(N, K, device="cuda") * 0.03).to(torch.bfloat16).requires_grad_(True)
    w._fp8_train = True
    go = torch.randn(M, N, device="cuda").to(torch.bfloat16)
    y = F.linear_maybe_fp8(x, w)
    y.backward(go)
    torch.cuda.synchronize()
    assert native.read_status(x.device) == 0
    xr, wr = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    (xr @ wr.t()).backward(go.float())
    rel = lambda a, b: ((a.float() - b).norm() / b.norm()).item()
    assert rel(y.detach(), (xr @ wr.t()).detach()) < 0.05
    assert rel(x.grad, xr.grad) < 0.05 and rel(w.grad, wr.grad) < 0.05


# ---------------------------------------------------------------------------------------------------------
# CTA-pair GEMM (cta_group::2), its epilogues, and the decode-sized split-K GEMM with fused reductions
# ---------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("path", [1, 2])
@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (512, 768, 256), (300, 1000, 520), (77, 136, 64),
                                   (1024, 3584, 3584), (2048, 4608, 1024), (129, 128, 4096)])
def test_gemm_both_kernels(path, M, N, K):
    torch.manual_seed(20)
    a, b = _bf16(M, K), _bf16(N, K)
    c = F.gemm(a, b, path=path)
    native.read_status(a.device)
    ref = a.float() @ b.float().t()
    assert torch.allclose(c.float(), ref, rtol=2e-2, atol=1e-2 * math.sqrt(K)), (c.float() - ref).abs().max()


@pytest.mark.parametrize("a_mn,b_mn", [(False, True), (True, True), (True, False)])
def test_gemm_pair_kernel_operand_layouts(a_mn, b_mn):
    torch.manual_seed(21)
    M, N, K = 640, 904, 1096
    a = _bf16(K, M) if a_mn else _bf16(M, K)
    b = _bf16(K, N) if b_mn else _bf16(N, K)
    for out_dtype in (torch.bfloat16, torch.float32):
        out = F.gemm(a, b, a_mn=a_mn, b_mn=b_mn, path=2, out_dtype=out_dtype)
        native.read_status(a.device)
        ref = (a.float().t() if a_mn else a.float()) @ (b.float() if b_mn else b.float().t())
        assert torch.allclose(out.float(), ref, rtol=2e-2, atol=1e-2 * math.sqrt(K)), (out.float() - ref).abs().max()


def test_gemm_pair_kernel_bias_accumulate_and_swiglu():
    torch.manual_seed(22)
    M, N, K = 520, 1280, 768
    a, b = _bf16(M, K), _bf16(N, K, scale=0.05)
    bias = _bf16(N)
    ref = a.float() @ b.float().t()
    y = F.gemm(a, b, bias=bias, path=2)
    assert torch.allclose(y.float(), ref + bias.float(), rtol=2e-2, atol=0.1)
    # accumulate: C += A B^T by TMA reduce-add, fp32 and bf16
    acc = torch.full((M, N), 2.0, dtype=torch.float32, device=DEV)
    F.gemm(a, b, out=acc, accumulate=True, path=2)
    assert torch.allclose(acc, ref + 2.0, rtol=1e-3, atol=2e-2)
    acc16 = torch.full((M, N), 2.0, dtype=torch.bfloat16, device=DEV)
    F.gemm(a, b, out=acc16, accumulate=True, path=2)
    assert torch.allclose(acc16.float(), ref + 2.0, rtol=3e-2, atol=0.15)
    # SwiGLU epilogue on a fused gate/up weight
    I = N // 2
    g, u = ref[:, :I], ref[:, I:]
    z = F.gemm(a, b, swiglu=True)
    native.read_status(a.device)
    assert z.shape == (M, I)
    assert torch.allclose(z.float(), torch.nn.functional.silu(g) * u, rtol=3e-2, atol=0.05)


@pytest.mark.parametrize("M,N,K", [(128, 4608, 3584), (100, 3584, 3584), (8, 1024, 18944), (256, 3584, 1024),
                                   (200, 1000, 520), (128, 152064, 512)])
def test_gemm_skinny_matches_fp32(M, N, K):
    torch.manual_seed(23)
    x, w = _bf16(M, K), _bf16(N, K, scale=0.05)
    bias = _bf16(N)
    y = F.gemm_skinny(x, w, bias=bias)
    native.read_status(x.device)
    ref = x.float() @ w.float().t() + bias.float()
    assert torch.allclose(y.float(), ref, rtol=2e-2, atol=2e-2 * math.sqrt(K) * 0.05 + 0.05), (y.float() - ref).abs().max()


def test_skinny_fused_reductions():
    torch.manual_seed(24)
    M, H, I = 96, 1024, 2816
    hq, hkv, d, P = 6, 2, 128, 128
    x = _bf16(M, H)
    # o_proj / down_proj form: projection + residual + RMSNorm
    w = _bf16(H, I, scale=0.03)
    act = _bf16(M, I)
    res = _bf16(M, H)
    nw = (1.0 + 0.1 * torch.randn(H, device=DEV)).to(torch.bfloat16)
    y, res_out = F.skinny_linear_residual_rmsnorm(act, w, res, nw, 1e-6)
    native.read_status(x.device)
    r_ref = act.float() @ w.float().t() + res.float()
    assert torch.allclose(res_out.float(), r_ref, rtol=2e-2, atol=0.1)
    rr = res_out.float()
    y_ref = rr * torch.rsqrt(rr.pow(2).mean(-1, keepdim=True) + 1e-6) * nw.float()
    assert torch.allclose(y.float(), y_ref, rtol=2e-2, atol=2e-2)
    # gate/up form: SwiGLU in the GEMM epilogue
    wgu = _bf16(2 * I, H, scale=0.03)
    z = F.skinny_gate_up_swiglu(x, wgu)
    gu = x.float() @ wgu.float().t()
    assert torch.allclose(z.float(), torch.nn.functional.silu(gu[:, :I]) * gu[:, I:], rtol=3e-2, atol=0.05)
    # qkv form: bias + RoPE + cache append against the separate kernels
    wqkv = _bf16((hq + 2 * hkv) * d, H, scale=0.03)
    bqkv = _bf16((hq + 2 * hkv) * d)
    pos = torch.randint(0, 4000, (M,), device=DEV, dtype=torch.int64)
    n_pages = 8
    slots = torch.randperm(n_pages * P, device=DEV)[:M].to(torch.int32)
    slots[5] = -1
    for vt in (False, True):
        cache = torch.zeros(n_pages, 2, hkv, P, d, dtype=torch.bfloat16, device=DEV)
        q = F.skinny_qkv_rope_append(x, wqkv, bqkv, pos, slots, 1e6, hq, hkv, d, cache, vt)
        native.read_status(x.device)
        qkv_ref = (x.float() @ wqkv.float().t() + bqkv.float()).to(torch.bfloat16)
        q_ref, k_ref, v_ref = qkv_ref.split([hq * d, hkv * d, hkv * d], dim=-1)
        q_ref, k_ref = R.apply_rope(q_ref.reshape(M, hq, d).float(), k_ref.reshape(M, hkv, d).float(), pos, 1e6)
        assert torch.allclose(q.float(), q_ref.float(), rtol=2e-2, atol=3e-2), (q.float() - q_ref.float()).abs().max()
        cache_ref = torch.zeros_like(cache)
        R.kv_append(k_ref.to(torch.bfloat16), v_ref.reshape(M, hkv, d), cache_ref, slots, vt)
        assert torch.allclose(cache.float(), cache_ref.float(), rtol=2e-2, atol=3e-2)


def test_linear_product_path_runs_own_gemm():
    """The projection entry point of the models must reach this library's GEMM for bf16 CUDA tensors, in training
    (autograd) and inference (wide and decode-sized batches)."""
    torch.manual_seed(25)
    w = _bf16(768, 1024, scale=0.05).requires_grad_(True)
    b = _bf16(768).requires_grad_(True)
    for M in (64, 512):
        x = _bf16(M, 1024).requires_grad_(True)
        before = native.LAUNCHES[0]
        y = F.linear_maybe_fp8(x, w, b)
        assert native.LAUNCHES[0] > before
        y.float().sum().backward()
        ref = torch.nn.functional.linear(x.detach().float(), w.detach().float(), b.detach().float())
        assert torch.allclose(y.float(), ref, rtol=2e-2, atol=0.2)
        with torch.no_grad():
            before = native.LAUNCHES[0]
            y2 = F.linear_maybe_fp8(x, w, b)
            assert native.LAUNCHES[0] > before
            assert torch.allclose(y2.float(), ref, rtol=2e-2, atol=0.2)
    native.read_status(w.device)


def test_bounded_waits_run_out_report_status_and_release_tensor_memory():
    """Failure detection on the device, without a fault: a wait on a flag that nothing sets runs into its (short)
    limit, the kernel records ST_TIMEOUT_PEER_FLAG in the status word, frees what it holds and returns; the host
    reads the code, and the next tensor-core launch on the same context works (its TMEM allocation would block
    forever if the timed-out kernel had kept its columns)."""
    from cosmos_rl_b200.parallel import peer
    from cosmos_rl_b200.parallel.tp_fused import FusedTP
    dev = torch.device("cuda", torch.cuda.current_device())
    native.read_status(dev)
    # 1. the plain flag-wait kernel
    buf = peer.PeerBuffer(256, dev)
    peer.flag_wait(buf.ptr, 1, dev, limit_s=0.002)
    with pytest.raises(native.NativeError, match="peer flag"):
        native.read_status(dev)
    assert native.read_status(dev) == 0                      # reading the code re-arms the status word
    buf.free()
    # 2. the fused GEMM + all-reduce kernel (tcgen05 pipeline + side warps waiting for the other rank's arrivals)
    torch.manual_seed(30)
    M, N, K = 256, 512, 256
    a, w = _bf16(M, K), _bf16(N, K, scale=0.05)
    ctx = FusedTP.with_silent_peers(2, dev, M, N, wait_s=0.002)
    out = ctx.gemm_all_reduce(a, w)
    torch.cuda.synchronize()
    with pytest.raises(native.NativeError, match="peer flag"):
        native.read_status(dev)
    ctx.free_silent()
    del out
    # 3. the context is intact and no tensor memory leaked: ordinary GEMMs (both kernels) still run and are right
    ref = a.float() @ w.float().t()
    for path in (1, 2):
        c = F.gemm(a, w, path=path)
        assert torch.allclose(c.float(), ref, rtol=2e-2, atol=0.2)
    assert native.read_status(dev) == 0


def test_activation_offload_prefetches_and_keeps_gradients():
    """Saved activations go to pinned host memory in forward; in backward the copies of the tensors needed next are
    already enqueued when they are asked for (no host-side wait), and the gradients equal the resident run."""
    from torch import nn
    from cosmos_rl_b200.utils.activation_offloading import OffloadActivations
    torch.manual_seed(31)
    net = nn.Sequential(*[m for _ in range(6) for m in (nn.Linear(512, 512), nn.GELU())]).cuda()
    x = torch.randn(2048, 512, device=DEV, requires_grad=True)
    net(x).pow(2).sum().backward()
    ref = [p.grad.clone() for p in net.parameters()]
    gx = x.grad.clone()
    net.zero_grad()
    x.grad = None
    ctx = OffloadActivations(min_bytes=1 << 16, params={p.untyped_storage().data_ptr() for p in net.parameters()})
    with ctx:
        y = net(x).pow(2).sum()
    assert ctx.bytes_offloaded > 0 and len(ctx.stash) >= 6
    y.backward()
    torch.cuda.synchronize()
    assert ctx.n_prefetched >= len(ref) // 2 - 2, ctx.n_prefetched          # most fetches were issued ahead of their use
    assert not ctx.stash and not ctx.inflight
    for a, p in zip(ref, net.parameters()):
        assert torch.allclose(a, p.grad, rtol=1e-4, atol=1e-4)
    assert torch.allclose(gx, x.grad, rtol=1e-4, atol=1e-4)
