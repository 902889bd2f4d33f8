"""Multi-process CPU (gloo) tests of the parallel strategies: context parallelism, pipeline parallelism."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from cosmos_rl_b200.models.gpt import GPT, GPTArgs


def _tiny():
    return GPTArgs(vocab_size=512, dim=64, n_layers=2, n_heads=4, n_kv_heads=2, ffn_dim=128, qkv_bias=True,
                   model_type="qwen2")


def _spawn(fn, world, tmp_path, *args):
    store = str(tmp_path / "store")
    mp.spawn(fn, args=(world, store) + args, nprocs=world, join=True)


def _init(rank, world, store):
    dist.init_process_group("gloo", init_method=f"file://{store}", rank=rank, world_size=world)
    torch.manual_seed(0)


def _cp_worker(rank, world, store, mode):
    from cosmos_rl_b200.parallel.context_parallel import ContextParallel, local_cu_seqlens
    _init(rank, world, store)
    m = GPT(_tiny())
    m.init_weights(0)
    lens = [8, 20, 4]
    cu = torch.tensor([0, 8, 28, 32])
    if mode == "ring-zigzag-long":                         # four ranks: lengths have to be multiples of 2 * 4
        mode, lens, cu = "ring-zigzag", [8, 16, 8], torch.tensor([0, 8, 24, 32])
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, 512, (32,), generator=g)
    labels = torch.randint(0, 512, (32,), generator=g)
    pos = m.get_position_ids(cu, 32)
    # full model on every rank (the oracle)
    lp_full, _ = m.logprobs(m(ids, pos, cu, max(lens)), labels)
    lp_full.sum().backward()
    ref_grads = [p.grad.clone() for p in m.parameters()]
    m.zero_grad()
    cp = ContextParallel(dist.group.WORLD, world, rank, mode)
    m.attach_context_parallel(cp)
    lcu = local_cu_seqlens(cu, world)
    h = m(cp.shard(ids, cu), cp.shard(pos, cu), lcu, max(lens) // world)
    lp, _ = m.logprobs(h, cp.shard(labels, cu))
    assert torch.allclose(lp, cp.shard(lp_full.detach(), cu), atol=1e-5), (lp - cp.shard(lp_full.detach(), cu)).abs().max()
    lp.sum().backward()
    for p, r in zip(m.parameters(), ref_grads):
        gsum = p.grad.clone()
        dist.all_reduce(gsum)
        assert torch.allclose(gsum, r, atol=2e-5), (gsum - r).abs().max()
    dist.destroy_process_group()


@pytest.mark.parametrize("mode", ["kv-gather", "ulysses", "ring", "ring-zigzag"])
def test_context_parallel_matches_full_model(tmp_path, mode):
    _spawn(_cp_worker, 2, tmp_path, mode)


def test_zigzag_ring_on_four_ranks_and_its_layout(tmp_path):
    """Four ranks, eight chunks per sequence: every rank holds chunks r and 7 - r, and the model matches the unsplit
    one. (Sequence lengths of the worker are multiples of 8.)"""
    from cosmos_rl_b200.parallel.context_parallel import split_for_cp
    x, cu = torch.arange(24), torch.tensor([0, 16, 24])
    assert split_for_cp(x, cu, 2, 0, zigzag=True).tolist() == [0, 1, 2, 3, 12, 13, 14, 15, 16, 17, 22, 23]
    assert split_for_cp(x, cu, 2, 1, zigzag=True).tolist() == [4, 5, 6, 7, 8, 9, 10, 11, 18, 19, 20, 21]
    _spawn(_cp_worker, 4, tmp_path, "ring-zigzag-long")


def test_ring_attention_on_four_ranks(tmp_path):
    """K/V chunks pass three hops, their gradients four; chunks from the future are skipped."""
    _spawn(_cp_worker, 4, tmp_path, "ring")


def _pp_worker(rank, world, store):
    import copy
    from cosmos_rl_b200.parallel.pipeline import MicroBatch, PipelineStage, schedule_1f1b
    _init(rank, world, store)
    full = GPT(_tiny())
    full.init_weights(0)
    a = copy.deepcopy(full.args)
    a.pp_size, a.pp_rank = world, rank
    stage = GPT(a)
    sd = full.state_dict()
    off = stage.layer_offset
    with torch.no_grad():
        for name, p in stage.named_parameters():
            src = name
            if name.startswith("layers."):
                idx, rest = name[len("layers."):].split(".", 1)
                src = f"layers.{int(idx) + off}.{rest}"
            p.copy_(sd[src])
    g = torch.Generator().manual_seed(3)
    mbs, ref_loss = [], 0.0
    for lens in ([5, 9], [12], [3, 3, 4]):
        T = sum(lens)
        cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)))
        ids = torch.randint(0, 512, (T,), generator=g)
        labels = torch.randint(0, 512, (T,), generator=g)
        mbs.append(MicroBatch(ids, full.get_position_ids(cu, T), cu, max(lens), labels))

    def loss_fn(model):
        return lambda hidden, mb: -model.logprobs(hidden, mb.extra)[0].mean() / len(mbs)

    for mb in mbs:
        l = loss_fn(full)(full(mb.input_ids, mb.position_ids, mb.cu_seqlens, mb.max_seqlen), mb)
        l.backward()
        ref_loss += l.item()
    ref = {n: p.grad for n, p in full.named_parameters()}
    runner = PipelineStage(stage, dist.group.WORLD, rank, world, a.dim, torch.float32, torch.device("cpu"))
    losses = runner.run(mbs, loss_fn(stage))
    if rank == world - 1:
        assert abs(sum(x.item() for x in losses) - ref_loss) < 1e-5
    for name, p in stage.named_parameters():
        src = name
        if name.startswith("layers."):
            idx, rest = name[len("layers."):].split(".", 1)
            src = f"layers.{int(idx) + off}.{rest}"
        assert torch.allclose(p.grad, ref[src], atol=1e-5), (name, (p.grad - ref[src]).abs().max())
    # every forward precedes its backward and the number of in-flight micro-batches never exceeds the depth
    for s in range(4):
        steps, live = schedule_1f1b(s, 4, 8), 0
        for kind, i in steps:
            live += 1 if kind == "F" else -1
            assert 0 <= live <= 4 - s
        assert sorted(i for k, i in steps if k == "F") == list(range(8)) == sorted(i for k, i in steps if k == "B")
    dist.destroy_process_group()


def test_pipeline_1f1b_matches_full_model(tmp_path):
    _spawn(_pp_worker, 2, tmp_path)


def _pp_interleaved_worker(rank, world, store):
    """Two ranks, two model chunks each (virtual stages 0..3 of a four-block model), five micro-batches (a short
    last group): losses and gradients of the interleaved schedule equal the unsplit model; the forward-only pass
    returns its results in micro-batch order."""
    import copy
    from cosmos_rl_b200.parallel.pipeline import MicroBatch, PipelineStage
    _init(rank, world, store)
    base = _tiny()
    base.n_layers = 4
    full = GPT(base)
    full.init_weights(0)
    sd = full.state_dict()
    chunks = []
    for c in range(2):
        a = copy.deepcopy(full.args)
        a.pp_size, a.pp_rank = 2 * world, c * world + rank
        m = GPT(a)
        with torch.no_grad():
            for name, p in m.named_parameters():
                src = name
                if name.startswith("layers."):
                    idx, rest = name[len("layers."):].split(".", 1)
                    src = f"layers.{int(idx) + m.layer_offset}.{rest}"
                p.copy_(sd[src])
        chunks.append(m)
    g = torch.Generator().manual_seed(3)
    mbs, ref_loss = [], 0.0
    for lens in ([5, 9], [12], [3, 3, 4], [7], [2, 6]):
        T = sum(lens)
        cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)))
        ids = torch.randint(0, 512, (T,), generator=g)
        labels = torch.randint(0, 512, (T,), generator=g)
        mbs.append(MicroBatch(ids, full.get_position_ids(cu, T), cu, max(lens), labels))

    def loss_fn(model):
        return lambda hidden, mb: -model.logprobs(hidden, mb.extra)[0].mean() / len(mbs)

    per_mb = []
    for mb in mbs:
        l = loss_fn(full)(full(mb.input_ids, mb.position_ids, mb.cu_seqlens, mb.max_seqlen), mb)
        l.backward()
        per_mb.append(l.item())
    ref = {n: p.grad for n, p in full.named_parameters()}
    back = dist.new_group(list(range(world)))
    runner = PipelineStage(chunks, dist.group.WORLD, rank, world, base.dim, torch.float32, torch.device("cpu"),
                           schedule="Interleaved1F1B", back_group=back)
    head = chunks[-1]
    losses = runner.run(mbs, loss_fn(head))
    if rank == world - 1:
        assert abs(sum(x.item() for x in losses) - sum(per_mb)) < 1e-5
    else:
        assert losses == []
    for m in chunks:
        for name, p in m.named_parameters():
            src = name
            if name.startswith("layers."):
                idx, rest = name[len("layers."):].split(".", 1)
                src = f"layers.{int(idx) + m.layer_offset}.{rest}"
            assert torch.allclose(p.grad, ref[src], atol=1e-5), (name, (p.grad - ref[src]).abs().max())
    outs = runner.forward_only(mbs, lambda h, mb: loss_fn(head)(h, mb).item())
    if rank == world - 1:
        assert all(abs(a - b) < 1e-5 for a, b in zip(outs, per_mb)), (outs, per_mb)
    dist.destroy_process_group()


def test_pipeline_interleaved_1f1b_matches_full_model(tmp_path):
    """Several stages per rank (cosmos_rl/utils/pipelining/pipelining_utils.py:170-260)."""
    _spawn(_pp_interleaved_worker, 2, tmp_path)


def test_interleaved_schedule_properties():
    """Every (micro-batch, chunk) runs forward once and backward once, forward first; the schedule completes for
    awkward micro-batch counts; the bubble shrinks with the number of chunks."""
    from cosmos_rl_b200.parallel.pipeline import schedule_interleaved_1f1b, simulate_schedule
    for P, V, M in ((2, 2, 5), (4, 3, 5), (4, 2, 8), (5, 4, 12), (3, 1, 7)):
        for s in range(P):
            steps = schedule_interleaved_1f1b(s, P, M, V)
            seen = set()
            for kind, i, c in steps:
                if kind == "F":
                    assert (i, c) not in seen
                    seen.add((i, c))
                else:
                    assert (i, c) in seen
            assert len(steps) == 2 * M * V and len(seen) == M * V
        simulate_schedule(lambda r: schedule_interleaved_1f1b(r, P, M, V), P, M, V)       # raises on a deadlock
    b1 = simulate_schedule(lambda r: schedule_interleaved_1f1b(r, 4, 8, 1), 4, 8, 1)["bubble"]
    b2 = simulate_schedule(lambda r: schedule_interleaved_1f1b(r, 4, 8, 2), 4, 8, 2)["bubble"]
    b4 = simulate_schedule(lambda r: schedule_interleaved_1f1b(r, 4, 8, 4), 4, 8, 4)["bubble"]
    assert b1 > b2 > b4 and b1 > 0.25 and b4 < 0.1, (b1, b2, b4)


def _failure_worker(rank, world, store_path):
    """Host-side failure injection: rank 1 leaves between two steps (no collective in flight); rank 0's next
    collective ends with CommTimeout within its limit, the communicator is aborted and a smaller one is built."""
    import time
    from datetime import timedelta
    from cosmos_rl_b200.parallel import dyncomm
    store = dist.FileStore(store_path, world)
    events = []
    dyncomm.add_phase_observer(lambda name, phase, info: events.append((name, phase)))
    comm = dyncomm.DynComm("policy-mesh-v1", store, rank, world, torch.device("cpu"), timeout_s=2.0)
    t = torch.ones(4) * (rank + 1)
    comm.all_reduce(t)                                   # step 1: everybody is here
    assert torch.equal(t, torch.full((4,), 3.0))
    store.set(f"step1_done_{rank}", b"1")
    if rank == 1:
        store.wait(["step1_done_0"], timedelta(seconds=20))
        return                                           # rank 1 "dies" cleanly between steps
    store.wait(["step1_done_1"], timedelta(seconds=20))
    time.sleep(0.2)
    t0 = time.time()
    with pytest.raises(dyncomm.CommTimeout):
        comm.all_reduce(torch.ones(4))                   # step 2: the peer never joins
    assert time.time() - t0 < 15.0
    assert comm.aborted and "policy-mesh-v1" not in dyncomm.live_comms()
    assert ("policy-mesh-v1", "abort") in events
    with pytest.raises(dyncomm.CommTimeout):
        comm.all_reduce(torch.ones(4))                   # an aborted communicator refuses further work at once
    solo = dyncomm.DynComm("policy-mesh-v2", store, 0, 1, torch.device("cpu"), timeout_s=2.0)   # mesh rebuilt
    x = torch.ones(4)
    solo.all_reduce(x)
    assert torch.equal(x, torch.ones(4))
    solo.destroy()


def test_rank_leaving_between_steps_times_out_and_mesh_is_rebuilt(tmp_path):
    mp.spawn(_failure_worker, args=(2, str(tmp_path / "fstore")), nprocs=2, join=True)


def _watchdog_worker(rank, world, store_path):
    """A block deadline shorter than the per-operation limit: the watchdog's timer aborts the communicator under a
    receive whose sender never sends, and the block ends with CommTimeout. The stream form polls a probe and aborts
    when the enqueued work does not finish; a drain that runs out aborts the named communicators and says so."""
    import time
    from datetime import timedelta
    from cosmos_rl_b200.parallel import dyncomm
    store = dist.FileStore(store_path, world)
    comm = dyncomm.DynComm("p2r-a", store, rank, world, torch.device("cpu"), timeout_s=30.0)
    x = torch.ones(2)
    comm.all_reduce(x)
    if rank == 1:
        store.wait(["rank0_done"], timedelta(seconds=60))        # stays alive, sends nothing
        return
    t0 = time.time()
    with pytest.raises(dyncomm.CommTimeout):
        with dyncomm.watchdog(timeout_s=1.0) as ctx:
            comm.recv(torch.empty(2), 1)
    assert time.time() - t0 < 10.0 and comm.aborted and comm in ctx.comms
    # stream form: healthy block leaves the communicator alone
    solo = dyncomm.DynComm("solo-a", store, 0, 1, torch.device("cpu"), timeout_s=5.0)
    with dyncomm.watchdog(timeout_s=1.0, wait_stream=True, stream=lambda: True):
        solo.all_reduce(torch.ones(2))
    assert not solo.aborted
    # stream form: the device work never finishes
    t0 = time.time()
    with pytest.raises(dyncomm.CommTimeout):
        with dyncomm.watchdog(timeout_s=0.5, wait_stream=True, stream=lambda: False):
            solo.all_reduce(torch.ones(2))
    assert 0.4 < time.time() - t0 < 5.0 and solo.aborted
    # bounded drain
    a = dyncomm.DynComm("solo-b", store, 0, 1, torch.device("cpu"), timeout_s=5.0)
    b = dyncomm.DynComm("solo-c", store, 0, 1, torch.device("cpu"), timeout_s=5.0)
    assert dyncomm.bounded_drain_or_abort(lambda: True, 0.2, "test") and not a.aborted
    assert not dyncomm.bounded_drain_or_abort(lambda: False, 0.2, "test", comms=[a])
    assert a.aborted and not b.aborted
    assert not dyncomm.bounded_drain_or_abort(lambda: False, 0.2, "test")
    assert b.aborted and dyncomm.live_comms() == []
    assert a.async_error() is None
    store.set("rank0_done", b"1")


def test_watchdog_block_deadline_stream_deadline_and_bounded_drain(tmp_path):
    mp.spawn(_watchdog_worker, args=(2, str(tmp_path / "wstore")), nprocs=2, join=True)


def _tp_worker(rank, world, store, qk_norm, seq_parallel=False):
    """Tensor-parallel training step == unsharded model: log-probs and (gathered) gradients."""
    import copy
    from cosmos_rl_b200.models import hf_io
    from cosmos_rl_b200.parallel.tp import TensorParallel
    _init(rank, world, store)
    base = _tiny()
    if qk_norm:
        base.qk_norm, base.qkv_bias, base.model_type = True, False, "qwen3"
    full = GPT(base)
    full.init_weights(0)
    a = copy.deepcopy(full.args)
    a.tp_size, a.tp_rank = world, rank
    shard = GPT(a)
    cfg = full.args.to_hf_config()
    state = hf_io.hf_state_dict(full, cfg)
    hf_io.load_hf_state(shard, lambda k: state[k], state, cfg, world, rank)
    shard.tp = TensorParallel(dist.group.WORLD, world, rank)
    shard.tp.sequence_parallel = seq_parallel        # 21 tokens on 2 ranks: exercises the padding sequence too
    shard.tp.keep_gathered = not qk_norm             # one variant keeps the gathered rows, the other gathers again
    if seq_parallel:
        shard.gradient_checkpointing = "swiglu"
    g = torch.Generator().manual_seed(2)
    cu = torch.tensor([0, 9, 21])
    ids = torch.randint(0, 512, (21,), generator=g)
    labels = torch.randint(0, 512, (21,), generator=g)
    pos = full.get_position_ids(cu, 21)
    lp_full, ent_full = full.logprobs(full(ids, pos, cu, 12), labels)
    lp_full.sum().backward()
    lp, ent = shard.logprobs(shard(ids, pos, cu, 12), labels)
    assert torch.allclose(lp, lp_full.detach(), atol=1e-4), (lp - lp_full).abs().max()
    assert torch.allclose(ent, ent_full.detach(), atol=1e-4)
    lp.sum().backward()
    # replicated parameters (norms) carry the full gradient on every rank; sharded ones carry their slice
    ref = dict(full.named_parameters())
    checked = 0
    for name, p in shard.named_parameters():
        r = ref[name].grad
        if p.shape == r.shape:
            assert torch.allclose(p.grad, r, atol=2e-4), (name, (p.grad - r).abs().max())
            checked += 1
    assert checked >= 5
    down = dict(shard.named_parameters())["layers.0.mlp.down_proj.weight"]
    cols = ref["layers.0.mlp.down_proj.weight"].grad.chunk(world, dim=1)[rank]
    assert torch.allclose(down.grad, cols, atol=2e-4)
    dist.destroy_process_group()


@pytest.mark.parametrize("qk_norm", [False, True])
def test_tensor_parallel_training_matches_full_model(tmp_path, qk_norm):
    _spawn(_tp_worker, 2, tmp_path, qk_norm)


@pytest.mark.parametrize("qk_norm", [False, True])
def test_sequence_parallel_training_matches_full_model(tmp_path, qk_norm):
    """Residual stream, norms and the embedding output hold T/tp rows per rank; same log-probs and gradients."""
    _spawn(_tp_worker, 2, tmp_path, qk_norm, True)


def _ep_worker(rank, world, store):
    """Expert-parallel MoE layer (all-to-all dispatch) == the same layer with every expert local."""
    import copy
    from cosmos_rl_b200.models.qwen3_moe import ARCHS, MoEFeedForward
    _init(rank, world, store)
    a = copy.deepcopy(ARCHS["tiny-qwen3-moe"])
    a.aux_loss_coeff = 0.0
    torch.manual_seed(0)
    full = MoEFeedForward(a)
    for p in full.parameters():
        torch.nn.init.normal_(p, std=0.05)
    b = copy.deepcopy(a)
    b.ep_size, b.ep_rank = world, rank
    local = MoEFeedForward(b)
    El = a.n_experts // world
    with torch.no_grad():
        local.gate.weight.copy_(full.gate.weight)
        local.w_gate_up.copy_(full.w_gate_up[rank * El:(rank + 1) * El])
        local.w_down.copy_(full.w_down[rank * El:(rank + 1) * El])
    local.ep_group = dist.group.WORLD
    g = torch.Generator().manual_seed(10 + rank)          # every rank has its own tokens
    x = torch.randn(11 + rank, a.dim, generator=g)
    xf = x.clone().requires_grad_(True)
    yf = full(xf)
    yf.pow(2).sum().backward()
    xl = x.clone().requires_grad_(True)
    yl = local(xl)
    assert torch.allclose(yl, yf.detach(), atol=1e-5), (yl - yf).abs().max()
    yl.pow(2).sum().backward()
    assert torch.allclose(xl.grad, xf.grad, atol=1e-5)
    # expert gradients: the local experts received tokens from both ranks; compare with the sum over ranks
    want = full.w_down.grad[rank * El:(rank + 1) * El].clone()
    others = [torch.zeros_like(full.w_down.grad) for _ in range(world)]
    dist.all_gather(others, full.w_down.grad)
    want = sum(o[rank * El:(rank + 1) * El] for o in others)
    assert torch.allclose(local.w_down.grad, want, atol=1e-5), (local.w_down.grad - want).abs().max()
    dist.destroy_process_group()


def test_expert_parallel_moe_matches_local_experts(tmp_path):
    _spawn(_ep_worker, 2, tmp_path)


def _zero_worker(rank, world, store):
    """Sharded flat AdamW (optimizer state split over dp ranks, library collectives) == unsharded AdamW on the
    averaged gradient."""
    from cosmos_rl_b200.ops import reference as R
    from cosmos_rl_b200.parallel.flat import FlatParams
    from cosmos_rl_b200.policy.optim import FlatAdamW
    _init(rank, world, store)
    m = GPT(_tiny())
    flat = FlatParams(m, torch.float32, torch.device("cpu"), shard_multiple=world)
    m.init_weights(0)
    opt = FlatAdamW(flat, lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, max_grad_norm=1.0,
                    dp_group=dist.group.WORLD)
    from cosmos_rl_b200.utils.ema import ShardEMA
    ema = ShardEMA(opt, decay=0.5)
    w = flat.data.clone()
    ema_full = w.clone()
    mm, vv = torch.zeros_like(w), torch.zeros_like(w)
    for step in range(1, 4):
        g = torch.Generator().manual_seed(100 * step + rank)
        flat.grad.copy_(torch.randn(flat.total, generator=g) * 0.01)
        gs = [torch.zeros_like(flat.grad) for _ in range(world)]
        dist.all_gather(gs, flat.grad)
        avg = torch.stack(gs).mean(0)
        norm = opt.step()
        assert abs(norm.item() - avg.norm().item()) < 1e-5
        R.adamw_step(w, mm, vv, avg, 1e-2, 0.9, 0.95, 1e-8, 0.1, step, grad_scale=min(1.0, 1.0 / (avg.norm().item() + 1e-6)))
        assert torch.allclose(flat.data, w, atol=1e-6), (flat.data - w).abs().max()
        ema.step(step - 1)
        d = min(step / (9 + step), 0.5)
        ema_full = d * ema_full + (1 - d) * w
    # the average lives on the shard; swapping it in gathers it into every rank's live buffer and back out again
    assert ema.shard.numel() == flat.total // world
    with ema.swapped_in():
        assert torch.allclose(flat.data, ema_full, atol=1e-6)
    assert torch.allclose(flat.data, w, atol=1e-6)
    dist.destroy_process_group()


def test_sharded_flat_adamw_matches_unsharded(tmp_path):
    _spawn(_zero_worker, 2, tmp_path)


def _ep_train_worker(rank, world, store):
    """Training with expert parallelism: experts live in a rank-local tail of the flat buffer (full optimizer state,
    no reduction), everything else is reduced and sharded as usual. Two optimizer steps must reproduce plain AdamW on
    the unsharded model fed with both ranks' data."""
    import copy
    from cosmos_rl_b200.models.qwen3_moe import ARCHS, MoEFeedForward, Qwen3MoE
    from cosmos_rl_b200.ops import reference as R
    from cosmos_rl_b200.parallel.flat import FlatParams
    from cosmos_rl_b200.policy.optim import FlatAdamW
    _init(rank, world, store)
    a = copy.deepcopy(ARCHS["tiny-qwen3-moe"])
    a.vocab_size, a.aux_loss_coeff = 512, 0.0
    ref = Qwen3MoE(a)
    ref.init_weights(0)
    rflat = FlatParams(ref, torch.float32, torch.device("cpu"))
    b = copy.deepcopy(a)
    b.ep_size, b.ep_rank = world, rank
    ep = Qwen3MoE(b)
    is_expert = lambda n: n.endswith("w_gate_up") or n.endswith("w_down")
    flat = FlatParams(ep, torch.float32, torch.device("cpu"), shard_multiple=world, local_filter=is_expert)
    assert flat.total > flat.shared_total and flat.shared_total % world == 0
    El = a.n_experts // world
    rp = dict(ref.named_parameters())
    with torch.no_grad():
        for n, p in ep.named_parameters():
            p.copy_(rp[n][rank * El:(rank + 1) * El] if is_expert(n) else rp[n])
    for mod in ep.modules():
        if isinstance(mod, MoEFeedForward):
            mod.ep_group = dist.group.WORLD
    hp = dict(lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, max_grad_norm=0.5)
    opt = FlatAdamW(flat, dp_group=dist.group.WORLD, **hp)
    w = rflat.data.clone()
    mm, vv = torch.zeros_like(w), torch.zeros_like(w)
    data = []
    for r in range(world):
        g = torch.Generator().manual_seed(50 + r)
        n = 14 + 5 * r
        data.append((torch.randint(0, 512, (n,), generator=g), torch.randint(0, 512, (n,), generator=g),
                     torch.tensor([0, n])))
    loss_of = lambda model, d: -model.logprobs(model(d[0], torch.arange(d[0].numel()), d[2], int(d[0].numel())), d[1])[0].mean()
    for step in range(1, 3):
        rflat.zero_grad()
        (sum(loss_of(ref, d) for d in data) / world).backward()
        gn = rflat.grad.double().norm().item()  # the fp32 CPU norm of a long vector is off by 3e-4
        R.adamw_step(w, mm, vv, rflat.grad, 1e-2, 0.9, 0.95, 1e-8, 0.1, step, grad_scale=min(1.0, 0.5 / (gn + 1e-6)))
        rflat.data.copy_(w)
        flat.zero_grad()
        loss_of(ep, data[rank]).backward()
        norm = opt.step()
        assert abs(norm.item() - gn) < 1e-4 * max(1.0, gn), (norm.item(), gn)
        for n, p in ep.named_parameters():
            want = rp[n][rank * El:(rank + 1) * El] if is_expert(n) else rp[n]
            # Adam divides by |g|: elements whose gradient is near eps amplify reduction-order noise, a wiring error is ~lr
            assert torch.allclose(p, want, atol=5e-4), (step, n, (p - want).abs().max())
    dist.destroy_process_group()


def test_expert_parallel_training_matches_unsharded_adamw(tmp_path):
    _spawn(_ep_train_worker, 2, tmp_path)


def _ep_trainer_worker(rank, world, store, out_dir):
    """The SFT trainer with ``policy.parallelism.ep_size = dp_shard_size = 2``: experts are split over the ranks,
    the loss falls, and the replicated parameters stay bit-identical on both ranks."""
    from cosmos_rl_b200.config import Config
    from cosmos_rl_b200.parallel.dims import ParallelDims
    from cosmos_rl_b200.policy.trainer.sft_trainer import SFTTrainer
    _init(rank, world, store)
    cfg = Config.from_dict({
        "policy": {"model_name_or_path": "tiny-qwen3-moe", "model_max_length": 64, "model_gradient_checkpointing": False,
                   "parallelism": {"dp_shard_size": 2, "ep_size": 2, "tp_size": 1}},
        "train": {"seed": 0, "optm_lr": 2e-3, "optm_warmup_steps": 0, "output_dir": out_dir,
                  "train_policy": {"type": "sft", "trainer_type": "sft", "mini_batch": 2},
                  "ckpt": {"enable_checkpoint": False}},
    })
    dims = ParallelDims.from_config_parallelism(cfg.policy.parallelism, world, rank, torch.device("cpu"))
    dims.build_groups()
    tr = SFTTrainer(cfg, dims, device=torch.device("cpu"))
    tr.model_load_from_hf()
    a = tr.model.args
    assert a.ep_size == 2 and a.ep_rank == rank and tr.flat.total > tr.flat.shared_total
    V = a.vocab_size
    g = torch.Generator().manual_seed(10 + rank)
    batch = [{"input_ids": torch.randint(0, V, (n,), generator=g).tolist()} for n in (12, 9, 15, 7)]
    losses = [tr.step_training(batch, total_steps=10, train_step=i + 1)["train/loss_avg"] for i in range(4)]
    assert losses[-1] < losses[0] - 0.05, losses
    shared = tr.flat.data[:tr.flat.shared_total].clone()
    both = [torch.empty_like(shared) for _ in range(world)]
    dist.all_gather(both, shared)
    assert torch.equal(both[0], both[1])
    tail = tr.flat.data[tr.flat.shared_total:].clone()
    tails = [torch.empty_like(tail) for _ in range(world)]
    dist.all_gather(tails, tail)
    assert not torch.equal(tails[0], tails[1])                       # each rank owns different experts
    dist.destroy_process_group()


def test_sft_trainer_with_expert_parallelism(tmp_path):
    _spawn(_ep_trainer_worker, 2, tmp_path, str(tmp_path))


def _hsdp_worker(rank, world, store):
    """HSDP on 4 ranks (dp_replicate 2 x dp_shard 2) and DDP (dp_replicate 4): the update equals plain AdamW on the
    gradient averaged over all four ranks, and every rank ends with identical parameters."""
    from cosmos_rl_b200.ops import reference as R
    from cosmos_rl_b200.parallel.dims import ParallelDims
    from cosmos_rl_b200.parallel.flat import FlatParams
    from cosmos_rl_b200.policy.optim import FlatAdamW
    _init(rank, world, store)
    for rep, shard in ((2, 2), (4, 1)):
        dims = ParallelDims(dp_replicate=rep, dp_shard=shard, world_size=world, global_rank=rank,
                            device=torch.device("cpu"))
        dims.build_groups()
        m = GPT(_tiny())
        flat = FlatParams(m, torch.float32, torch.device("cpu"), shard_multiple=shard)
        m.init_weights(0)
        opt = FlatAdamW(flat, lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, max_grad_norm=1.0,
                        dp_group=dims.group("dp_shard") if shard > 1 else None,
                        replicate_group=dims.group("dp_replicate"))
        w = flat.data.clone()
        mm, vv = torch.zeros_like(w), torch.zeros_like(w)
        for step in range(1, 3):
            g = torch.Generator().manual_seed(100 * step + rank)
            flat.grad.copy_(torch.randn(flat.total, generator=g) * 0.01)
            gs = [torch.zeros_like(flat.grad) for _ in range(world)]
            dist.all_gather(gs, flat.grad)
            avg = torch.stack(gs).mean(0)
            n = avg.double().norm().item()
            norm = opt.step()
            assert abs(norm.item() - n) < 1e-5, (rep, shard, norm.item(), n)
            R.adamw_step(w, mm, vv, avg, 1e-2, 0.9, 0.95, 1e-8, 0.1, step, grad_scale=min(1.0, 1.0 / (n + 1e-6)))
            assert torch.allclose(flat.data, w, atol=1e-4), (rep, shard, (flat.data - w).abs().max())   # updates are ~1e-2
    dist.destroy_process_group()


def test_hsdp_and_ddp_match_unsharded_adamw(tmp_path):
    _spawn(_hsdp_worker, 4, tmp_path)


def _tp_trainer_worker(rank, world, store, out_dir):
    """The SFT trainer with tp_size = 2 (sequence-parallel plan): same losses, gradient norms and resulting weights as
    the single-process trainer on the same batches."""
    from cosmos_rl_b200.config import Config
    from cosmos_rl_b200.models import hf_io
    from cosmos_rl_b200.parallel.dims import ParallelDims
    from cosmos_rl_b200.policy.trainer.sft_trainer import SFTTrainer
    _init(rank, world, store)

    def cfg(tp):
        return Config.from_dict({
            "policy": {"model_name_or_path": "tiny-qwen2", "model_max_length": 64, "model_gradient_checkpointing": False,
                       "parallelism": {"tp_size": tp, "dp_shard_size": 1}},
            "b200": {"sequence_parallel": True},
            "train": {"seed": 0, "optm_lr": 1e-3, "optm_warmup_steps": 0, "output_dir": out_dir, "optm_grad_norm_clip": 0.5,
                      "train_policy": {"type": "sft", "trainer_type": "sft", "mini_batch": 4},
                      "ckpt": {"enable_checkpoint": False}}})
    dims = ParallelDims.from_config_parallelism(cfg(2).policy.parallelism, world, rank, torch.device("cpu"))
    dims.build_groups()
    tr = SFTTrainer(cfg(2), dims, device=torch.device("cpu"))
    assert tr.model.tp.sequence_parallel and tr.optimizer.tp_replicated.any()
    ref = SFTTrainer(cfg(1), ParallelDims(world_size=1, device=torch.device("cpu")), device=torch.device("cpu"))
    ref.model_load_from_hf()
    hf_cfg = ref.model.args.to_hf_config()
    state = hf_io.hf_state_dict(ref.model, hf_cfg)
    hf_io.load_hf_state(tr.model, lambda k: state[k], state, hf_cfg, world, rank)
    tr.optimizer.refresh_master_from_params()
    tr.weights_ready = True
    g = torch.Generator().manual_seed(3)
    batch = [{"input_ids": torch.randint(0, 32000, (n,), generator=g).tolist()} for n in (12, 9, 15, 7)]
    for i in range(3):
        a = tr.step_training(batch, total_steps=10, train_step=i + 1)
        b = ref.step_training(batch, total_steps=10, train_step=i + 1)
        assert abs(a["train/loss_avg"] - b["train/loss_avg"]) < 1e-4, (i, a["train/loss_avg"], b["train/loss_avg"])
        assert abs(a["train/grad_norm"] - b["train/grad_norm"]) < 1e-3 * b["train/grad_norm"], (i, a["train/grad_norm"], b["train/grad_norm"])
    want = hf_io.hf_state_dict(ref.model, hf_cfg)
    probe = GPT(tr.model.args)
    hf_io.load_hf_state(probe, lambda k: want[k], want, hf_cfg, world, rank)      # reference weights, this rank's slices
    for (n, p), (_, q) in zip(tr.model.named_parameters(), probe.named_parameters()):
        assert torch.allclose(p, q, atol=5e-4), (n, (p - q).abs().max())
    dist.destroy_process_group()


def test_sft_trainer_with_tensor_and_sequence_parallelism(tmp_path):
    _spawn(_tp_trainer_worker, 2, tmp_path, str(tmp_path))


def _cp_trainer_worker(rank, world, store, out_dir, mode):
    """SFT and GRPO trainers with cp_size = 2: same loss, gradient norm and weights as single-process trainers."""
    from cosmos_rl_b200.config import Config
    from cosmos_rl_b200.dispatcher.data.schema import Rollout
    from cosmos_rl_b200.parallel.dims import ParallelDims
    from cosmos_rl_b200.policy.trainer.grpo_trainer import GRPOTrainer
    from cosmos_rl_b200.policy.trainer.sft_trainer import SFTTrainer
    _init(rank, world, store)

    def cfg(cp, kind):
        return Config.from_dict({
            "policy": {"model_name_or_path": "tiny-qwen2", "model_max_length": 64, "model_gradient_checkpointing": False,
                       "parallelism": {"cp_size": cp, "dp_shard_size": 1, "tp_size": 1}},
            "b200": {"cp_mode": mode},
            "train": {"seed": 0, "optm_lr": 1e-3, "optm_warmup_steps": 0, "output_dir": out_dir, "optm_grad_norm_clip": 0.5,
                      "train_policy": {"type": kind, "trainer_type": kind, "mini_batch": 4},
                      "ckpt": {"enable_checkpoint": False}}})
    cpu = torch.device("cpu")
    dims = ParallelDims.from_config_parallelism(cfg(2, "sft").policy.parallelism, world, rank, cpu)
    dims.build_groups()
    one = ParallelDims(world_size=1, device=cpu)
    g = torch.Generator().manual_seed(3)
    batch = [{"input_ids": torch.randint(0, 32000, (n,), generator=g).tolist()} for n in (12, 9, 15, 7)]
    tr, ref = SFTTrainer(cfg(2, "sft"), dims, device=cpu), SFTTrainer(cfg(1, "sft"), one, device=cpu)
    for t in (tr, ref):
        t.model_load_from_hf()                                   # same seed: identical weights
    assert tr.model.layers[0].self_attn.cp.mode == mode
    for i in range(2):
        a = tr.step_training(batch, total_steps=10, train_step=i + 1)
        b = ref.step_training(batch, total_steps=10, train_step=i + 1)
        assert abs(a["train/loss_avg"] - b["train/loss_avg"]) < 1e-4, (a["train/loss_avg"], b["train/loss_avg"])
        assert abs(a["train/grad_norm"] - b["train/grad_norm"]) < 1e-3 * b["train/grad_norm"]
    assert torch.allclose(tr.flat.data, ref.flat.data, atol=5e-4)
    # GRPO: rollouts with behaviour log-probs (exercises the sharding of per-token side inputs)
    ros = []
    for i in range(4):
        n = [6, 11, 4, 9][i]
        toks = torch.randint(0, 32000, (n,), generator=g).tolist()
        ros.append(Rollout(prompt=torch.randint(0, 32000, (5 + i,), generator=g).tolist(), completion=toks,
                           advantage=[0.5, -1.0, 1.5, -0.2][i], reward=float(i),
                           completion_token_ids=[[t] for t in toks], completion_logprobs=[[-10.3 - 0.01 * j] for j in range(n)]))
    gt, gref = GRPOTrainer(cfg(2, "grpo"), dims, device=cpu), GRPOTrainer(cfg(1, "grpo"), one, device=cpu)
    for t in (gt, gref):
        t.model_load_from_hf()
        t.tp_cfg.use_rollout_logprobs_for_loss = True
    a = gt.step_training(ros, 1, 10)
    b = gref.step_training(ros, 1, 10)
    assert abs(a["train/grad_norm"] - b["train/grad_norm"]) < 1e-3 * b["train/grad_norm"], (a["train/grad_norm"], b["train/grad_norm"])
    assert torch.allclose(gt.flat.data, gref.flat.data, atol=5e-4)
    dist.destroy_process_group()


@pytest.mark.parametrize("mode", ["kv-gather", "ring", "ring-zigzag"])
def test_trainers_with_context_parallelism(tmp_path, mode):
    _spawn(_cp_trainer_worker, 2, tmp_path, str(tmp_path), mode)


def _pp_trainer_worker(rank, world, store, out_dir):
    """SFT and GRPO trainers with pp_size = 2 (1F1B over the packed mini-batches): same loss, gradient norm and
    weights as the single-process trainers."""
    from cosmos_rl_b200.config import Config
    from cosmos_rl_b200.dispatcher.data.schema import Rollout
    from cosmos_rl_b200.models import hf_io
    from cosmos_rl_b200.parallel.dims import ParallelDims
    from cosmos_rl_b200.policy.trainer.grpo_trainer import GRPOTrainer
    from cosmos_rl_b200.policy.trainer.sft_trainer import SFTTrainer
    _init(rank, world, store)

    def cfg(pp, kind):
        return Config.from_dict({
            "policy": {"model_name_or_path": "tiny-qwen2", "model_max_length": 64, "model_gradient_checkpointing": False,
                       "parallelism": {"pp_size": pp, "dp_shard_size": 1, "tp_size": 1, "pp_micro_batch_size": 2,
                                       "pp_schedule": "GPipe" if kind == "sft" else "1F1B"}},
            "train": {"seed": 0, "optm_lr": 1e-3, "optm_warmup_steps": 0, "output_dir": out_dir, "optm_grad_norm_clip": 0.5,
                      "train_policy": {"type": kind, "trainer_type": kind, "mini_batch": 2},
                      "ckpt": {"enable_checkpoint": False}}})
    cpu = torch.device("cpu")
    dims = ParallelDims.from_config_parallelism(cfg(2, "sft").policy.parallelism, world, rank, cpu)
    dims.build_groups()
    one = ParallelDims(world_size=1, device=cpu)

    def same_weights(stage_tr, ref_tr):
        hf_cfg = ref_tr.model.args.to_hf_config()
        state = hf_io.hf_state_dict(ref_tr.model, hf_cfg)
        hf_io.load_hf_state(stage_tr.model, lambda k: state[k], state, hf_cfg)
        stage_tr.optimizer.refresh_master_from_params()
        stage_tr.weights_ready = True

    def check_weights(stage_tr, ref_tr):
        ref_p = dict(ref_tr.model.named_parameters())
        off = stage_tr.model.layer_offset
        for n, p in stage_tr.model.named_parameters():
            if n.startswith("layers."):
                i, rest = n[len("layers."):].split(".", 1)
                n = f"layers.{int(i) + off}.{rest}"
            assert torch.allclose(p, ref_p[n], atol=5e-4), (n, (p - ref_p[n]).abs().max())

    g = torch.Generator().manual_seed(3)
    batch = [{"input_ids": torch.randint(0, 32000, (n,), generator=g).tolist()} for n in (12, 9, 15, 7, 10, 6)]
    tr, ref = SFTTrainer(cfg(2, "sft"), dims, device=cpu), SFTTrainer(cfg(1, "sft"), one, device=cpu)
    ref.model_load_from_hf()
    same_weights(tr, ref)
    assert len(tr.model.layers) == 1 and (tr.model.embed_tokens is None) == (rank == 1)
    for i in range(2):
        a = tr.step_training(batch, total_steps=10, train_step=i + 1)          # 3 micro-batches through 2 stages
        b = ref.step_training(batch, total_steps=10, train_step=i + 1)
        assert abs(a["train/loss_avg"] - b["train/loss_avg"]) < 1e-4, (a["train/loss_avg"], b["train/loss_avg"])
        assert abs(a["train/grad_norm"] - b["train/grad_norm"]) < 1e-3 * b["train/grad_norm"]
    check_weights(tr, ref)
    assert abs(tr.step_validation(batch)["val/loss"] - ref.step_validation(batch)["val/loss"]) < 1e-4
    ros = []
    for i in range(4):
        n = [6, 11, 4, 9][i]
        ros.append(Rollout(prompt=torch.randint(0, 32000, (5 + i,), generator=g).tolist(),
                           completion=torch.randint(0, 32000, (n,), generator=g).tolist(),
                           advantage=[0.5, -1.0, 1.5, -0.2][i], reward=float(i)))
    gt, gref = GRPOTrainer(cfg(2, "grpo"), dims, device=cpu), GRPOTrainer(cfg(1, "grpo"), one, device=cpu)
    gref.model_load_from_hf()
    same_weights(gt, gref)
    for t in (gt, gref):
        t.tp_cfg.mu_iterations = 2                         # old log-probs come from the forward-only pipeline pass
    a, b = gt.step_training(ros, 1, 10), gref.step_training(ros, 1, 10)
    assert abs(a["train/grad_norm"] - b["train/grad_norm"]) < 1e-3 * b["train/grad_norm"], (a["train/grad_norm"], b["train/grad_norm"])
    assert abs(a["train/loss_avg"] - b["train/loss_avg"]) < 1e-5
    assert set(b) <= set(a) and abs(a["train/clip_frac"] - b["train/clip_frac"]) < 1e-6      # metrics reach every stage
    check_weights(gt, gref)
    dist.destroy_process_group()


def test_trainers_with_pipeline_parallelism(tmp_path):
    _spawn(_pp_trainer_worker, 2, tmp_path, str(tmp_path))


def _combo_worker(rank, world, store, out_dir, axis):
    """Four ranks: dp_shard 2 combined with tp 2, cp 2 or pp 2 through the SFT trainer. Each data-parallel rank trains
    on its half of the batch; losses, gradient norm and weights must equal the single-process trainer on all of it.
    ``axis`` of the form "tp+cp" combines two model-parallel axes instead (no data parallelism: every rank sees the
    whole batch)."""
    from cosmos_rl_b200.config import Config
    from cosmos_rl_b200.models import hf_io
    from cosmos_rl_b200.parallel.dims import ParallelDims
    from cosmos_rl_b200.policy.trainer.sft_trainer import SFTTrainer
    _init(rank, world, store)

    def cfg(par):
        return Config.from_dict({
            "policy": {"model_name_or_path": "tiny-qwen2", "model_max_length": 64, "model_gradient_checkpointing": False,
                       "parallelism": dict({"tp_size": 1, "cp_size": 1, "pp_size": 1, "dp_shard_size": 1}, **par)},
            "train": {"seed": 0, "optm_lr": 1e-3, "optm_warmup_steps": 0, "output_dir": out_dir, "optm_grad_norm_clip": 0.5,
                      "train_policy": {"type": "sft", "trainer_type": "sft", "mini_batch": 2},
                      "ckpt": {"enable_checkpoint": False}}})
    cpu = torch.device("cpu")
    two = axis.split("+")
    n_dp = 2 if len(two) == 1 else 1
    c = cfg(dict({a + "_size": 2 for a in two}, dp_shard_size=n_dp))
    dims = ParallelDims.from_config_parallelism(c.policy.parallelism, world, rank, cpu)
    dims.build_groups()
    tr = SFTTrainer(c, dims, device=cpu)
    ref = SFTTrainer(cfg({}), ParallelDims(world_size=1, device=cpu), device=cpu)
    ref.model_load_from_hf()
    hf_cfg = ref.model.args.to_hf_config()
    state = hf_io.hf_state_dict(ref.model, hf_cfg)
    hf_io.load_hf_state(tr.model, lambda k: state[k], state, hf_cfg, dims.tp, dims.tp_coord)
    tr.optimizer.refresh_master_from_params()
    g = torch.Generator().manual_seed(3)
    batch = [{"input_ids": torch.randint(0, 32000, (n,), generator=g).tolist()} for n in (12, 9, 15, 7, 10, 6, 8, 14)]
    mine = batch[dims.dp_shard_coord::n_dp]                                # this data-parallel rank's samples
    for i in range(2):
        a = tr.step_training(mine, total_steps=10, train_step=i + 1)
        b = ref.step_training(batch, total_steps=10, train_step=i + 1)
        loss = torch.tensor(a["train/loss_avg"])
        if n_dp > 1:
            dist.all_reduce(loss, group=dims.group("dp_shard"))            # each dp rank reports its share of the sum
        assert abs(loss.item() / n_dp - b["train/loss_avg"]) < 1e-4, (axis, loss.item() / n_dp, b["train/loss_avg"])
        assert abs(a["train/grad_norm"] - b["train/grad_norm"]) < 2e-3 * b["train/grad_norm"], (axis, a["train/grad_norm"], b["train/grad_norm"])
    want = hf_io.hf_state_dict(ref.model, hf_cfg)
    probe = GPT(tr.model.args)
    hf_io.load_hf_state(probe, lambda k: want[k], want, hf_cfg, dims.tp, dims.tp_coord)
    for (n, p), (_, q) in zip(tr.model.named_parameters(), probe.named_parameters()):
        assert torch.allclose(p, q, atol=5e-4), (axis, n, (p - q).abs().max())
    dist.destroy_process_group()


@pytest.mark.parametrize("axis", ["tp", "cp", "pp"])
def test_data_parallel_combined_with_model_parallel_axes(tmp_path, axis):
    _spawn(_combo_worker, 4, tmp_path, str(tmp_path), axis)


@pytest.mark.parametrize("axis", ["tp+cp", "tp+pp", "cp+pp"])
def test_two_model_parallel_axes_combined(tmp_path, axis):
    """tp x cp (context exchange inside a tensor-parallel group's heads), tp x pp and cp x pp on four ranks match the
    single-process trainer (the reference composes its axes through one mesh: cosmos_rl/utils/parallelism.py:82-578)."""
    _spawn(_combo_worker, 4, tmp_path, str(tmp_path), axis)


def _force_save_worker(rank, world, store):
    """Only rank 1 saw the forwarded signal: both ranks must agree to save on this step, and nobody on the next."""
    import threading
    from cosmos_rl_b200.policy.worker.rl_worker import agree_force_save
    _init(rank, world, store)
    ev = threading.Event()
    if rank == 1:
        ev.set()
    assert agree_force_save(ev, world) is True
    assert not ev.is_set()
    # the following collective of the "training step" still pairs up on both ranks
    t = torch.tensor([float(rank + 1)])
    dist.all_reduce(t)
    assert t.item() == 3.0
    assert agree_force_save(ev, world) is False
    dist.destroy_process_group()


def test_force_save_flag_is_agreed_by_all_ranks_every_step(tmp_path):
    _spawn(_force_save_worker, 2, tmp_path)


def _ep_sub_worker(rank, world, store, out_dir):
    """Four ranks, ``dp_shard_size = 4`` with ``ep_size = 2``: ranks {0, 1} and {2, 3} each hold all experts between
    them, ranks {0, 2} and {1, 3} hold the same experts. Every rank trains on its quarter of the batch; loss, gradient
    norm and weights (experts included) must equal the single-process trainer on the whole batch."""
    from cosmos_rl_b200.config import Config
    from cosmos_rl_b200.models import hf_io
    from cosmos_rl_b200.models.base import ModelRegistry
    from cosmos_rl_b200.parallel.dims import ParallelDims
    from cosmos_rl_b200.policy.trainer.sft_trainer import SFTTrainer
    _init(rank, world, store)

    def cfg(par):
        return Config.from_dict({
            "policy": {"model_name_or_path": "tiny-qwen3-moe", "model_max_length": 64,
                       "model_gradient_checkpointing": False,
                       "parallelism": dict({"tp_size": 1, "dp_shard_size": 1, "ep_size": 1}, **par)},
            "train": {"seed": 0, "optm_lr": 1e-3, "optm_warmup_steps": 0, "output_dir": out_dir, "optm_grad_norm_clip": 0.5,
                      "train_policy": {"type": "sft", "trainer_type": "sft", "mini_batch": 2, "aux_loss_coeff": 0.0},
                      "ckpt": {"enable_checkpoint": False}}})
    cpu = torch.device("cpu")
    c = cfg({"dp_shard_size": 4, "ep_size": 2})
    dims = ParallelDims.from_config_parallelism(c.policy.parallelism, world, rank, cpu)
    dims.build_groups()
    tr = SFTTrainer(c, dims, device=cpu)
    assert tr.model.args.ep_size == 2 and tr.model.args.ep_rank == rank % 2
    assert dist.get_world_size(dims.group("ep")) == 2 and dist.get_world_size(dims.group("ep_replica")) == 2
    ref = SFTTrainer(cfg({}), ParallelDims(world_size=1, device=cpu), device=cpu)
    ref.model_load_from_hf()
    hf_cfg = ref.model.args.to_hf_config()
    state = hf_io.hf_state_dict(ref.model, hf_cfg)
    hf_io.load_hf_state(tr.model, lambda k: state[k], state, hf_cfg, 1, 0)
    tr.optimizer.refresh_master_from_params()
    V = ref.model.args.vocab_size
    g = torch.Generator().manual_seed(3)
    batch = [{"input_ids": torch.randint(0, V, (n,), generator=g).tolist()} for n in (12, 9, 15, 7, 10, 6, 8, 14)]
    mine = batch[rank::4]
    for i in range(2):
        a = tr.step_training(mine, total_steps=10, train_step=i + 1)
        b = ref.step_training(batch, total_steps=10, train_step=i + 1)
        loss = torch.tensor(a["train/loss_avg"])
        dist.all_reduce(loss, group=dims.group("dp_shard"))
        assert abs(loss.item() / 4 - b["train/loss_avg"]) < 2e-4, (loss.item() / 4, b["train/loss_avg"])
        assert abs(a["train/grad_norm"] - b["train/grad_norm"]) < 5e-3 * b["train/grad_norm"], \
            (a["train/grad_norm"], b["train/grad_norm"])
    want = hf_io.hf_state_dict(ref.model, hf_cfg)
    got = hf_io.hf_state_dict(tr.model, hf_cfg)
    assert len(got) < len(want)                                     # this rank exports only the experts it owns
    for k, v in got.items():
        assert torch.allclose(v, want[k], atol=5e-4), (k, (v - want[k]).abs().max())
    dist.destroy_process_group()


def test_expert_parallel_inside_a_larger_dp_shard_group(tmp_path):
    _spawn(_ep_sub_worker, 4, tmp_path, str(tmp_path))


def _split_load_worker(rank, world, store, ckpt):
    """Two data-parallel ranks load one multi-file checkpoint: each reads the tensor bytes of its own files only and
    receives the rest by broadcast; both end up with the full, identical model."""
    from cosmos_rl_b200.models import hf_io
    from cosmos_rl_b200.parallel.dims import ParallelDims
    _init(rank, world, store)
    dims = ParallelDims(dp_shard=2, world_size=2, global_rank=rank, device=torch.device("cpu"))
    dims.build_groups()
    m = GPT(_tiny())
    hf_io.load_hf_weights(m, ckpt, dims)
    st = m._hf_load_stats
    assert st["read_bytes"] > 0 and st["recv_bytes"] > 0
    total = torch.tensor([float(st["read_bytes"])])
    dist.all_reduce(total)
    n_bytes = sum(p.numel() * 4 for p in m.parameters())          # the checkpoint is fp32: every byte read once
    assert abs(total.item() - n_bytes) < 1e-6 * n_bytes, (total.item(), n_bytes)
    ref = GPT(_tiny())
    ref.init_weights(5)
    for (n, p), (_, q) in zip(m.named_parameters(), ref.named_parameters()):
        assert torch.equal(p, q), n
    dist.destroy_process_group()


def test_checkpoint_files_are_split_between_data_parallel_ranks(tmp_path, monkeypatch):
    from cosmos_rl_b200.models import hf_io
    m = GPT(_tiny())
    m.init_weights(5)
    monkeypatch.setattr(hf_io, "MAX_SHARD_BYTES", 64 * 1024)       # several files
    out = str(tmp_path / "ckpt")
    hf_io.export_safetensors(m, m.args.to_hf_config(), out)
    assert len([f for f in os.listdir(out) if f.endswith(".safetensors")]) >= 3
    _spawn(_split_load_worker, 2, tmp_path, out)


def _shard_params_worker(rank, world, store, out_dir, ckpt_mode):
    """Parameter-sharded data parallelism on two ranks: every rank holds half of every unit (embedding, block, final
    norm + head), units are gathered around their use and their gradients reduce-scattered after their backward.
    Losses, gradient norm and weights after two optimizer steps equal the single-process trainer on the whole batch;
    with full-block recomputation the same holds; gathers and reductions are counted."""
    from cosmos_rl_b200.config import Config
    from cosmos_rl_b200.parallel.dims import ParallelDims
    from cosmos_rl_b200.policy.trainer.sft_trainer import SFTTrainer
    _init(rank, world, store)

    def cfg(par, **b200):
        return Config.from_dict({
            "policy": {"model_name_or_path": "tiny-qwen2", "model_max_length": 64,
                       "model_gradient_checkpointing": ckpt_mode != "none",
                       "parallelism": dict({"tp_size": 1, "cp_size": 1, "pp_size": 1, "dp_shard_size": 1}, **par)},
            "b200": dict({"recompute": ckpt_mode}, **b200),
            "train": {"seed": 0, "optm_lr": 1e-3, "optm_warmup_steps": 0, "output_dir": out_dir, "optm_grad_norm_clip": 0.5,
                      "train_policy": {"type": "sft", "trainer_type": "sft", "mini_batch": 2},
                      "ckpt": {"enable_checkpoint": False}}})
    cpu = torch.device("cpu")
    c = cfg({"dp_shard_size": 2}, shard_params=True)
    dims = ParallelDims.from_config_parallelism(c.policy.parallelism, world, rank, cpu)
    dims.build_groups()
    tr = SFTTrainer(c, dims, device=cpu)
    ref = SFTTrainer(cfg({}), ParallelDims(world_size=1, device=cpu), device=cpu)
    tr.model_load_from_hf()                                # same seed: both start from the same weights
    ref.model_load_from_hf()
    sp = tr.flat
    assert sp.sharded and sp.n_shard * 2 == sp.total and tr.optimizer.master.numel() == sp.n_shard
    full0 = sp.gather_full()
    for (n, q) in ref.model.named_parameters():
        assert torch.equal(sp.view(n, full0), q), n
    g = torch.Generator().manual_seed(3)
    batch = [{"input_ids": torch.randint(0, 32000, (n,), generator=g).tolist()} for n in (12, 9, 15, 7, 10, 6, 8, 14)]
    mine = batch[rank::2]
    for i in range(2):
        g0 = sp.n_gathers
        a = tr.step_training(mine, total_steps=10, train_step=i + 1)
        b = ref.step_training(batch, total_steps=10, train_step=i + 1)
        loss = torch.tensor(a["train/loss_avg"])
        dist.all_reduce(loss)
        assert abs(loss.item() / 2 - b["train/loss_avg"]) < 1e-4, (loss.item() / 2, b["train/loss_avg"])
        assert abs(a["train/grad_norm"] - b["train/grad_norm"]) < 2e-3 * b["train/grad_norm"]
        assert sp.n_gathers - g0 >= 2 * len(sp.units)      # every unit fetched for forward and again for backward
    assert sp.n_reduces >= 2 * len(sp.units)
    full = sp.gather_full()
    for (n, q) in ref.model.named_parameters():
        assert torch.allclose(sp.view(n, full), q, atol=5e-4), (n, (sp.view(n, full) - q).abs().max())
    # export reads the whole model through a transient full copy; the shards are untouched afterwards
    before = sp.data.clone()
    with sp.materialized() as whole:
        assert torch.equal(whole, full)
        assert tr.model.layers[0].self_attn.o_proj.weight.data_ptr() >= whole.data_ptr()
    assert torch.equal(sp.data, before)
    dist.destroy_process_group()


@pytest.mark.parametrize("ckpt_mode", ["none", "full", "swiglu"])
def test_parameter_sharded_training_matches_unsharded(tmp_path, ckpt_mode):
    """The reference shards parameters per block with FSDP2 (cosmos_rl/policy/model/gpt/parallelize.py:366-423)."""
    _spawn(_shard_params_worker, 2, tmp_path, str(tmp_path), ckpt_mode)


def _collective_sync_worker(rank, world, store):
    """Two policy ranks (data-parallel copies) and two rollout ranks (tensor parallel 2): the rectangles of the
    resharding plan travel by grouped send / recv, every group matched by a group of the same composition on the other
    side; the rollout ranks end up with exactly their tensor-parallel slices."""
    import copy
    from cosmos_rl_b200.models import hf_io
    from cosmos_rl_b200.parallel.flat import FlatParams
    from cosmos_rl_b200.parallel.reshard import build_plan, model_parts, shard_info
    from cosmos_rl_b200.rollout.weight_sync import CollectiveWeightSync
    _init(rank, world, store)
    full = GPT(_tiny())
    full.init_weights(4)
    cfg = full.args.to_hf_config()
    state = hf_io.hf_state_dict(full, cfg)
    cpu = torch.device("cpu")
    is_policy = rank < 2
    a = copy.deepcopy(full.args)
    if not is_policy:
        a.tp_size, a.tp_rank = 2, rank - 2
    m = GPT(a)
    hf_io.load_hf_state(m, lambda k: state[k], state, cfg, a.tp_size, a.tp_rank)
    flat = FlatParams(m, torch.float32, cpu, with_grad=False)
    want = flat.data.clone()
    if not is_policy:
        flat.data.zero_()
    infos = [None] * world
    dist.all_gather_object(infos, {"policy": is_policy, "info": shard_info(rank, model_parts(m, flat), flat.total)})
    pol = [e["info"] for e in infos if e["policy"]]
    plans = {r: build_plan(pol, infos[r]["info"]) for r in (2, 3)}
    assert {d[0] for pl in plans.values() for d in pl} == {0, 1}          # both copies serve rectangles
    ident = {r: r for r in range(world)}
    coll = CollectiveWeightSync(None, ident, ident, batch=7)              # several chunks per pair
    if is_policy:
        coll.send(flat.data, [[r, d] for r, pl in sorted(plans.items()) for d in pl if d[0] == rank])
    else:
        coll.recv(flat.data, plans[rank])
        for name, p in m.named_parameters():
            ref = torch.as_strided(want, p.shape, p.stride(), p.storage_offset())
            assert torch.equal(p.data, ref), name
    dist.barrier()
    dist.destroy_process_group()


def test_collective_weight_sync_between_two_policy_and_two_rollout_ranks(tmp_path):
    _spawn(_collective_sync_worker, 4, tmp_path)


def _vlm_tp_worker(rank, world, store, out_dir):
    """Native Qwen2.5-VL through the SFT trainer with tensor parallelism 2: the decoder is sharded like any GPT, the
    vision tower is replicated; samples carry pixels and placeholder tokens. Loss, gradient norm and the weights after
    two steps equal the single-process trainer."""
    from cosmos_rl_b200.config import Config
    from cosmos_rl_b200.models import hf_io
    from cosmos_rl_b200.models.qwen2_5_vl import Qwen25VL
    from cosmos_rl_b200.parallel.dims import ParallelDims
    from cosmos_rl_b200.policy.trainer.sft_trainer import SFTTrainer
    _init(rank, world, store)

    def cfg(par):
        return Config.from_dict({
            "policy": {"model_name_or_path": "tiny-qwen2.5-vl", "model_max_length": 128, "model_gradient_checkpointing": False,
                       "parallelism": dict({"tp_size": 1, "cp_size": 1, "pp_size": 1, "dp_shard_size": 1}, **par)},
            "train": {"seed": 0, "optm_lr": 1e-3, "optm_warmup_steps": 0, "output_dir": out_dir, "optm_grad_norm_clip": 0.5,
                      "train_policy": {"type": "sft", "trainer_type": "sft", "mini_batch": 2},
                      "ckpt": {"enable_checkpoint": False}}})
    cpu = torch.device("cpu")
    c = cfg({"tp_size": 2})
    dims = ParallelDims.from_config_parallelism(c.policy.parallelism, world, rank, cpu)
    dims.build_groups()
    tr = SFTTrainer(c, dims, device=cpu)
    ref = SFTTrainer(cfg({}), ParallelDims(world_size=1, device=cpu), device=cpu)
    assert type(tr.model) is Qwen25VL and type(ref.model) is Qwen25VL
    ref.model_load_from_hf()
    hf_cfg = ref.model.args.to_hf_config()
    state = hf_io.hf_state_dict(ref.model, hf_cfg)
    hf_io.load_hf_state(tr.model, lambda k: state[k], state, hf_cfg, dims.tp, dims.tp_coord)
    tr.optimizer.refresh_master_from_params()
    g = torch.Generator().manual_seed(11)
    IMG = ref.model.args.image_token_id

    def sample(n_text, h, w):
        ids = torch.randint(0, 30000, (n_text,), generator=g).tolist()
        n_img = (h // 2) * (w // 2)
        return {"input_ids": ids[:3] + [IMG] * n_img + ids[3:],
                "pixel_values": torch.randn(h * w, 3 * 2 * 14 * 14, generator=g), "image_grid_thw": torch.tensor([[1, h, w]])}
    batch = [sample(9, 4, 6), sample(12, 6, 4), sample(7, 8, 4), sample(10, 4, 4)]
    w0 = ref.model.visual.blocks[0].qkv.weight.detach().clone()
    for i in range(2):
        a = tr.step_training(batch, total_steps=10, train_step=i + 1)
        b = ref.step_training(batch, total_steps=10, train_step=i + 1)
        assert abs(a["train/loss_avg"] - b["train/loss_avg"]) < 1e-4, (a["train/loss_avg"], b["train/loss_avg"])
        assert abs(a["train/grad_norm"] - b["train/grad_norm"]) < 2e-3 * b["train/grad_norm"], (a["train/grad_norm"], b["train/grad_norm"])
    want = hf_io.hf_state_dict(ref.model, hf_cfg)
    probe = Qwen25VL(tr.model.args)
    hf_io.load_hf_state(probe, lambda k: want[k], want, hf_cfg, dims.tp, dims.tp_coord)
    for (n, p), (_, q) in zip(tr.model.named_parameters(), probe.named_parameters()):
        assert torch.allclose(p, q, atol=5e-4), (n, (p - q).abs().max())
    assert (ref.model.visual.blocks[0].qkv.weight - w0).abs().max() > 0           # the tower trained
    # weight-sync plan: every tensor of the rollout side (tp 1) is covered by the two policy ranks
    from cosmos_rl_b200.parallel.flat import FlatParams
    from cosmos_rl_b200.parallel.reshard import build_plan, model_parts, shard_info
    infos = [None] * world
    dist.all_gather_object(infos, shard_info(rank, model_parts(tr.model, tr.flat), tr.flat.total))
    plan = build_plan(infos, shard_info(0, model_parts(ref.model, ref.flat), ref.flat.total))
    assert sum(d[5] * d[6] for d in plan) == sum(p.numel() for p in ref.model.parameters())
    dist.destroy_process_group()


def test_native_vlm_trains_with_tensor_parallelism(tmp_path):
    """The reference's native VLM families carry parallel plans and a weight-sync map
    (cosmos_rl/policy/model/qwen2_5_vl/__init__.py:566, weight_mapper.py)."""
    _spawn(_vlm_tp_worker, 2, tmp_path, str(tmp_path))


def _pp_interleaved_trainer_worker(rank, world, store, out_dir):
    """SFT and GRPO trainers with pp_size = 2 and two model chunks per rank (``pp_schedule = "Interleaved1F1B"``,
    ``b200.pp_chunks = 2``): a four-block model, rank 0 holds blocks 0 and 2, rank 1 holds blocks 1 and 3. Loss,
    gradient norm and weights equal the single-process trainers; checkpoint names follow the block map."""
    import copy
    from cosmos_rl_b200.config import Config
    from cosmos_rl_b200.dispatcher.data.schema import Rollout
    from cosmos_rl_b200.models import hf_io
    from cosmos_rl_b200.parallel.dims import ParallelDims
    from cosmos_rl_b200.policy.trainer.grpo_trainer import GRPOTrainer
    from cosmos_rl_b200.policy.trainer.sft_trainer import SFTTrainer
    _init(rank, world, store)
    arch = copy.deepcopy(_tiny())
    arch.n_layers = 4
    model_cfg = arch.to_hf_config()

    def cfg(pp, kind):
        par = {"pp_size": pp, "dp_shard_size": 1, "tp_size": 1, "pp_micro_batch_size": 2,
               "pp_schedule": "Interleaved1F1B" if pp > 1 else "1F1B"}
        return Config.from_dict({
            "policy": {"model_name_or_path": "four-block", "model_max_length": 64, "model_gradient_checkpointing": False,
                       "parallelism": par},
            "custom": {"model_config": model_cfg}, "b200": {"pp_chunks": 2 if pp > 1 else 1},
            "train": {"seed": 0, "optm_lr": 1e-3, "optm_warmup_steps": 0, "output_dir": out_dir, "optm_grad_norm_clip": 0.5,
                      "train_policy": {"type": kind, "trainer_type": kind, "mini_batch": 2},
                      "ckpt": {"enable_checkpoint": False}}})
    cpu = torch.device("cpu")
    dims = ParallelDims.from_config_parallelism(cfg(2, "sft").policy.parallelism, world, rank, cpu)
    dims.build_groups()
    one = ParallelDims(world_size=1, device=cpu)

    def same_weights(stage_tr, ref_tr):
        hf_cfg = ref_tr.model.args.to_hf_config()
        state = hf_io.hf_state_dict(ref_tr.model, hf_cfg)
        hf_io.load_hf_state(stage_tr.model, lambda k: state[k], state, hf_cfg)
        stage_tr.optimizer.refresh_master_from_params()
        stage_tr.weights_ready = True

    def check_weights(stage_tr, ref_tr):
        ref_p = dict(ref_tr.model.named_parameters())
        for n, p in stage_tr.model.named_parameters():
            if n.startswith("layers."):
                i, rest = n[len("layers."):].split(".", 1)
                n = f"layers.{stage_tr.model.layer_map[int(i)]}.{rest}"
            assert torch.allclose(p, ref_p[n], atol=5e-4), (n, (p - ref_p[n]).abs().max())

    g = torch.Generator().manual_seed(3)
    batch = [{"input_ids": torch.randint(0, 512, (n,), generator=g).tolist()} for n in (12, 9, 15, 7, 10, 6, 8, 11, 5, 13)]
    tr, ref = SFTTrainer(cfg(2, "sft"), dims, device=cpu), SFTTrainer(cfg(1, "sft"), one, device=cpu)
    ref.model_load_from_hf()
    same_weights(tr, ref)
    assert tr.model.layer_map == ([0, 2] if rank == 0 else [1, 3]) and tr.pipeline.n_chunks == 2
    for i in range(2):
        a = tr.step_training(batch, total_steps=10, train_step=i + 1)          # 5 micro-batches, 4 virtual stages
        b = ref.step_training(batch, total_steps=10, train_step=i + 1)
        assert abs(a["train/loss_avg"] - b["train/loss_avg"]) < 1e-4, (a["train/loss_avg"], b["train/loss_avg"])
        assert abs(a["train/grad_norm"] - b["train/grad_norm"]) < 1e-3 * b["train/grad_norm"]
    check_weights(tr, ref)
    assert abs(tr.step_validation(batch)["val/loss"] - ref.step_validation(batch)["val/loss"]) < 1e-4
    names = set(hf_io.hf_state_dict(tr.model, tr.model.args.to_hf_config()))
    want = "model.layers.2.mlp.down_proj.weight" if rank == 0 else "model.layers.3.mlp.down_proj.weight"
    assert want in names and ("model.layers.1.mlp.down_proj.weight" in names) == (rank == 1)
    ros = []
    for i in range(4):
        n = [6, 11, 4, 9][i]
        ros.append(Rollout(prompt=torch.randint(0, 512, (5 + i,), generator=g).tolist(),
                           completion=torch.randint(0, 512, (n,), generator=g).tolist(),
                           advantage=[0.5, -1.0, 1.5, -0.2][i], reward=float(i)))
    gt, gref = GRPOTrainer(cfg(2, "grpo"), dims, device=cpu), GRPOTrainer(cfg(1, "grpo"), one, device=cpu)
    gref.model_load_from_hf()
    same_weights(gt, gref)
    for t in (gt, gref):
        t.tp_cfg.mu_iterations = 2
    a, b = gt.step_training(ros, 1, 10), gref.step_training(ros, 1, 10)
    assert abs(a["train/grad_norm"] - b["train/grad_norm"]) < 1e-3 * b["train/grad_norm"], (a["train/grad_norm"], b["train/grad_norm"])
    assert abs(a["train/loss_avg"] - b["train/loss_avg"]) < 1e-5
    check_weights(gt, gref)
    dist.destroy_process_group()


def test_trainers_with_interleaved_pipeline_chunks(tmp_path):
    _spawn(_pp_interleaved_trainer_worker, 2, tmp_path, str(tmp_path))
