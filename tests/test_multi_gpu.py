"""Peer-memory communication on 2, 4 and 8 GPUs of one box (child processes, NCCL for the
bootstrap, NVLS off, plain peer loads/stores in the kernels).  Cases that depend on the number of
ranks (a rank with two neighbours exists only from 3 ranks up) run at every size the box offers."""
import os
import socket
import tempfile
import traceback

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _need_gpus(n):
    if not torch.cuda.is_available() or torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")


WORLDS = [2, 4, 8]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _entry(rank, world, port, fn, out_dir):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                      LOCAL_RANK=str(rank), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    try:
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
        res = fn(rank, world)
        torch.save(res, os.path.join(out_dir, f"{rank}.pt"))
        dist.barrier()
        dist.destroy_process_group()
    except Exception:
        traceback.print_exc()
        raise


def _run(fn, world=2):
    port = _free_port()
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_entry, args=(world, port, fn, d), nprocs=world, join=True)
        return [torch.load(os.path.join(d, f"{r}.pt"), weights_only=False) for r in range(world)]


def _mailbox_case(rank, world):
    import torch.distributed as dist
    from megalodon_b200.parallel.symm import PeerMailbox, PeerTimeout, SymmetricRegion
    dev = torch.device("cuda", rank)
    slot = 4096
    region = SymmetricRegion(PeerMailbox.bytes_needed(slot, 2), None, dev)
    box = PeerMailbox(region, rank - 1 if rank > 0 else None, rank + 1 if rank + 1 < world else None, slot,
                      n_slots=2, timeout_s=0.5)
    ok = True
    # forward messages 0 -> 1 and gradients 1 -> 0, more than there are slots
    for k in range(5):
        if rank == 0:
            box.send(torch.full((1000,), float(k), device=dev), "fwd")
            back = torch.empty(37, device=dev, dtype=torch.bfloat16)       # odd size: exercises padding
            box.recv(back, "bwd")
            ok = ok and bool((back.float() == -k).all())
        else:
            got = torch.empty(1000, device=dev)
            box.recv(got, "fwd")
            ok = ok and bool((got == k).all())
            box.send(torch.full((37,), -float(k), device=dev, dtype=torch.bfloat16), "bwd")
        torch.cuda.synchronize()
        box.check()
    dist.barrier()
    # a receive that nothing answers runs into its time limit and reports it; the context survives
    timed_out = False
    if rank == 1:
        junk = torch.empty(16, device=dev)
        box.recv(junk, "fwd")
        torch.cuda.synchronize()
        try:
            box.check()
        except PeerTimeout as e:
            timed_out = "receive" in str(e) and "timed out" in str(e)
    box.reset()                              # collective: flags, sequence numbers and the abort record start over
    if rank == 0:
        box.send(torch.arange(16.0, device=dev), "fwd")
    else:
        late = torch.empty(16, device=dev)
        box.recv(late, "fwd")
        torch.cuda.synchronize()
        box.check()
        ok = ok and bool((late == torch.arange(16.0, device=dev)).all())
    torch.cuda.synchronize()
    return ok, timed_out


def test_peer_mailbox_two_gpus():
    _need_gpus(2)
    res = _run(_mailbox_case)
    assert all(r[0] for r in res)
    assert res[1][1], "the unanswered receive should have reported a timeout"


def _line_case(rank, world):
    """A line of `world` ranks: every layer's state goes rank to rank forward, every gradient back,
    more rounds than slots.  Then rank 0 withholds one message: the whole line must be out after ONE
    wait ran its time, and `reset()` must bring it back."""
    import time
    import torch.distributed as dist
    from megalodon_b200.parallel.symm import AbortRecord, PeerMailbox, PeerTimeout, SymmetricRegion
    dev = torch.device("cuda", rank)
    slot, n_slots, timeout_s = 8192, 2, 1.0
    region = SymmetricRegion(PeerMailbox.bytes_needed(slot, n_slots), None, dev)
    box = PeerMailbox(region, rank - 1 if rank > 0 else None, rank + 1 if rank + 1 < world else None, slot,
                      n_slots=n_slots, timeout_s=timeout_s)
    box.poison_slots = True              # every slot is overwritten with NaNs once read: a stale read would show
    ok = True

    def forward(k, withhold=False):
        val = torch.full((2000,), float(k), device=dev)
        if rank > 0:
            box.recv(val, "fwd")
            val = val + 1
        if rank + 1 < world and not withhold:
            box.send(val, "fwd")
        return val

    def backward(k):
        g = torch.full((37,), -float(k), device=dev, dtype=torch.bfloat16)
        if rank + 1 < world:
            box.recv(g, "bwd")
            g = g - 1
        if rank > 0:
            box.send(g, "bwd")
        return g

    for k in range(9):
        v = forward(k)
        g = backward(k)
        ok = ok and bool((v == k + rank).all()) and bool((g.float() == -k - (world - 1 - rank)).all())
    torch.cuda.synchronize()
    box.check()
    dist.barrier()
    # fault made on the host: rank 0 does not launch one send
    t0 = time.time()
    forward(100, withhold=(rank == 0))
    backward(100)
    torch.cuda.synchronize()
    waited = time.time() - t0
    report = ""
    try:
        box.check()
    except PeerTimeout as e:
        report = str(e)
    tripped = AbortRecord.get(dev).tripped()             # host-only look at the pinned mirror
    box.reset()
    v = forward(7)
    g = backward(7)
    torch.cuda.synchronize()
    box.check()
    ok = ok and bool((v == 7 + rank).all()) and bool((g.float() == -7 - (world - 1 - rank)).all())
    return ok, waited, report, tripped, timeout_s


@pytest.mark.parametrize("world", WORLDS)
def test_mailbox_line_with_middle_ranks_and_one_timeout_for_the_whole_line(world):
    _need_gpus(world)
    res = _run(_line_case, world)
    timeout_s = res[0][4]
    for r, (ok, waited, report, tripped, _) in enumerate(res):
        assert ok, f"rank {r}: wrong payload"
        assert report, f"rank {r} did not learn of the failure"
        assert tripped, f"rank {r}: pinned mirror of the abort record not set"
        # one wait ran its time (rank 1's); nobody may have waited for two
        assert waited < 1.9 * timeout_s + 1.0, f"rank {r} waited {waited:.2f} s"
    assert "timed out" in res[1][2] and "receive" in res[1][2] and "forward" in res[1][2], res[1][2]
    for r in range(2, world):
        # told by the neighbour's poison, or its own equally long wait ran out in the same instant (every
        # rank of the line started waiting together); never two waits in a row (checked above)
        assert "poisoned" in res[r][2] or "timed out" in res[r][2], res[r][2]


def _allreduce_case(rank, world):
    import torch.distributed as dist
    from megalodon_b200.parallel.symm import SymmetricAllReduce, SymmetricRegion
    dev = torch.device("cuda", rank)
    bucket = 1 << 20
    region = SymmetricRegion(SymmetricAllReduce.bytes_needed(bucket, world), None, dev)
    ar = SymmetricAllReduce(region, bucket, timeout_s=5.0)
    out = {}
    for dtype in (torch.bfloat16, torch.float32):
        torch.manual_seed(100 + rank)
        ts = [torch.randn(n, device=dev).to(dtype) for n in (1000, 700001, 64)]      # spans several buckets
        ref = [t.clone() for t in ts]
        for t in ref:
            dist.all_reduce(t)
        acc = torch.zeros((), dtype=torch.float64, device=dev)
        ar.all_reduce_(ts, sumsq=acc)
        torch.cuda.synchronize()
        ar.check()
        dist.all_reduce(acc)
        want = sum(t.double().pow(2).sum() for t in ts)
        err = max((a.float() - b.float()).abs().max().item() for a, b in zip(ts, ref))
        out[str(dtype)] = (err, abs(acc.item() - want.item()) / want.item())
    return out


@pytest.mark.parametrize("world", WORLDS)
def test_symmetric_allreduce(world):
    _need_gpus(world)
    res = _run(_allreduce_case, world)
    for r in res:
        assert r["torch.bfloat16"][0] < 5e-2 and r["torch.bfloat16"][1] < 1e-3, r
        assert r["torch.float32"][0] < 1e-5 and r["torch.float32"][1] < 1e-5, r


def _train_case(rank, world):
    from megalodon_b200.config import ModelConf, OptimConf
    from megalodon_b200.models.mega import build_model
    from megalodon_b200.optim import build_optimizer
    from megalodon_b200.ops import cuda_ops
    from megalodon_b200.parallel import initialize_model_parallel
    from megalodon_b200.parallel.chunk_parallel import set_handoff_transport
    from megalodon_b200.parallel.symm import enable_peer_transport
    from megalodon_b200.utils import clip_grad_norm_, set_random_seed
    initialize_model_parallel(1, world)
    cfg = ModelConf(num_layers=2, model_dim=256, num_heads=2, z_dim=128, value_dim=512, ffn_hidden_dim=512,
                    cema_ndim=16, chunk_size=128, vocab_size=512, swiglu=True, norm_num_groups=16,
                    efficient_attn="fused", layerwise_ckpt=True)
    toks = torch.randint(0, 512, (2, 128 * max(4, world) + 1), generator=torch.Generator().manual_seed(0)).cuda()
    x, y = toks[:, :-1], toks[:, 1:]
    curves = {}
    for transport in ("nccl", "p2p"):
        set_random_seed(0)
        set_handoff_transport("nccl")
        model = build_model(cfg, "bf16", False, True)
        if transport == "p2p":
            box, reducer = enable_peer_transport(model, max_batch=2, n_slots=4, allreduce_bucket_mb=1, timeout_s=20.0)
        opt, sched = build_optimizer(model, OptimConf(lr=3e-3, warmup=2), 20, "bf16")
        curve = []
        for _ in range(4):
            loss = model(x, targets=y)[0].mean()
            loss.backward()
            model.grad_all_reduce()
            norm = clip_grad_norm_(model, 1.0)
            opt.step(); sched.step(); opt.zero_grad()
            curve.append((loss.item(), float(norm)))
        if transport == "p2p":
            box.check()
            reducer.check()
        cuda_ops.check_kernel_errors()
        curves[transport] = curve
    set_handoff_transport("nccl")
    return curves


@pytest.mark.parametrize("world", WORLDS)
def test_chunk_parallel_training_over_peer_memory_matches_nccl(world):
    _need_gpus(world)
    res = _run(_train_case, world)
    for r in res:
        for (l0, n0), (l1, n1) in zip(r["nccl"], r["p2p"]):
            assert abs(l0 - l1) < 5e-2, r
            assert abs(n0 - n1) < 0.15 * max(1.0, n0), r


def _tp_case(rank, world):
    import torch.distributed as dist
    from megalodon_b200.parallel import initialize_model_parallel, get_model_parallel_group
    from megalodon_b200.parallel.tp_comm import TensorParallelWorkspace
    from megalodon_b200.ops import cuda_ops
    initialize_model_parallel(world, 1)
    dev = torch.device("cuda", rank)
    group = get_model_parallel_group()
    M, K, N = 384, 512, 768
    ws = TensorParallelWorkspace(group, dev, max_tokens=M, part_features=max(K, N) // world, timeout_s=10.0)
    g = torch.Generator(device="cpu").manual_seed(0)
    x_full = torch.randn(M, K, generator=g).bfloat16().to(dev)
    w = (torch.randn(N, K, generator=g) * 0.05).bfloat16().to(dev)
    out = {}
    # all-gather -> GEMM: every rank holds a K-slice of x
    x_part = x_full[:, rank * (K // world):(rank + 1) * (K // world)].contiguous()
    for trial in range(3):
        y, _ = ws.ag_gemm(x_part, w)
    ref = x_full.float() @ w.float().t()
    out["ag"] = (y.float() - ref).abs().max().item() / ref.abs().max().item()
    # GEMM -> reduce-scatter: every rank holds a K-slice of x and of w, the sum is split over N
    w_part = w[:, rank * (K // world):(rank + 1) * (K // world)].contiguous()
    for trial in range(3):
        y_rs = ws.gemm_rs(x_part, w_part)
    ref_rs = ref[:, rank * (N // world):(rank + 1) * (N // world)]
    out["rs"] = (y_rs.float() - ref_rs).abs().max().item() / ref.abs().max().item()
    torch.cuda.synchronize()
    ws.check()
    cuda_ops.check_kernel_errors()
    return out


def test_fused_tensor_parallel_gemms_two_gpus():
    _need_gpus(2)
    for r in _run(_tp_case):
        assert r["ag"] < 2e-2 and r["rs"] < 2e-2, r


def _tp_model_case(rank, world):
    from megalodon_b200.config import ModelConf
    from megalodon_b200.models.mega import build_model
    from megalodon_b200.ops import cuda_ops
    from megalodon_b200.parallel import initialize_model_parallel
    from megalodon_b200.parallel.tp_comm import disable_tp_fused, enable_tp_fused
    from megalodon_b200.utils import set_random_seed
    initialize_model_parallel(world, 1)
    cfg = ModelConf(num_layers=2, model_dim=512, num_heads=2, z_dim=256, value_dim=1024, ffn_hidden_dim=1024,
                    cema_ndim=16, chunk_size=128, vocab_size=512, swiglu=True, norm_num_groups=16,
                    efficient_attn="fused")
    toks = torch.randint(0, 512, (2, 257), generator=torch.Generator().manual_seed(0)).cuda()
    x, y = toks[:, :-1], toks[:, 1:]
    res = {}
    for fused in (False, True):
        set_random_seed(0)
        model = build_model(cfg, "bf16", False, True, materialize_fp32_grads=True)
        if fused:
            ws = enable_tp_fused(model, max_tokens=512, timeout_s=20.0)
        loss = model(x, targets=y)[0].mean()
        loss.backward()
        model.finish_backward()
        grads = torch.cat([p.grad.flatten() for p in model.parameters()])
        if fused:
            torch.cuda.synchronize()
            ws.check()
            disable_tp_fused()
        cuda_ops.check_kernel_errors()
        res[fused] = (loss.item(), grads.float().cpu())
    return res


def test_model_parallel_training_with_fused_collectives_matches_nccl():
    _need_gpus(2)
    for r in _run(_tp_model_case):
        (l0, g0), (l1, g1) = r[False], r[True]
        assert abs(l0 - l1) < 2e-2, (l0, l1)
        rel = (g0 - g1).norm() / (g0.norm() + 1e-6)
        assert rel < 5e-2, rel


def _fsdp_rs_case(rank, world):
    from megalodon_b200.config import ModelConf, OptimConf
    from megalodon_b200.models.mega import build_model
    from megalodon_b200.optim import build_optimizer
    from megalodon_b200.ops import cuda_ops
    from megalodon_b200.parallel import initialize_model_parallel
    from megalodon_b200.parallel.symm import enable_peer_reduce_scatter
    from megalodon_b200.utils import clip_grad_norm_, set_random_seed
    initialize_model_parallel(1, 1)            # data parallel = world
    cfg = ModelConf(num_layers=2, model_dim=256, num_heads=2, z_dim=128, value_dim=512, ffn_hidden_dim=512,
                    cema_ndim=16, chunk_size=128, vocab_size=512, swiglu=True, norm_num_groups=16,
                    efficient_attn="fused")
    toks = torch.randint(0, 512, (2 * world, 257), generator=torch.Generator().manual_seed(0))
    toks = toks[rank * 2:(rank + 1) * 2].cuda()
    x, y = toks[:, :-1], toks[:, 1:]
    curves = {}
    for fused in (False, True):
        set_random_seed(0)
        model = build_model(cfg, "bf16", False, True)
        if fused:
            rs = enable_peer_reduce_scatter(model, timeout_s=20.0)
        opt, sched = build_optimizer(model, OptimConf(lr=3e-3, warmup=2), 20, "bf16")
        curve = []
        for _ in range(4):
            loss = model(x, targets=y)[0].mean()
            loss.backward()
            model.grad_all_reduce()
            norm = clip_grad_norm_(model, 1.0)
            opt.step(); sched.step(); opt.zero_grad()
            curve.append((loss.item(), float(norm)))
        if fused:
            torch.cuda.synchronize()
            rs.check()
        cuda_ops.check_kernel_errors()
        curves[fused] = curve
    return curves


@pytest.mark.parametrize("world", WORLDS)
def test_fsdp_with_peer_memory_reduce_scatter_matches_nccl(world):
    _need_gpus(world)
    for r in _run(_fsdp_rs_case, world):
        for (l0, n0), (l1, n1) in zip(r[False], r[True]):
            assert abs(l0 - l1) < 5e-2, r
            assert abs(n0 - n1) < 0.1 * max(1.0, n0), r


def _fsdp_rs_adamw_case(rank, world):
    """No clipping: NCCL reduce-scatter + separate AdamW kernel vs the update fused into the
    peer-memory reduce-scatter kernel."""
    from megalodon_b200.config import ModelConf, OptimConf
    from megalodon_b200.models.mega import build_model
    from megalodon_b200.optim import build_optimizer
    from megalodon_b200.ops import cuda_ops
    from megalodon_b200.parallel import initialize_model_parallel
    from megalodon_b200.parallel.symm import enable_peer_reduce_scatter
    from megalodon_b200.utils import set_random_seed
    initialize_model_parallel(1, 1)
    cfg = ModelConf(num_layers=2, model_dim=256, num_heads=2, z_dim=128, value_dim=512, ffn_hidden_dim=512,
                    cema_ndim=16, chunk_size=128, vocab_size=512, swiglu=True, norm_num_groups=16,
                    efficient_attn="fused")
    toks = torch.randint(0, 512, (4, 257), generator=torch.Generator().manual_seed(0))
    toks = toks[rank * 2:(rank + 1) * 2].cuda()
    x, y = toks[:, :-1], toks[:, 1:]
    out = {}
    for fused in (False, True):
        set_random_seed(0)
        model = build_model(cfg, "bf16", False, True)
        opt, sched = build_optimizer(model, OptimConf(lr=3e-3, warmup=2, clip=0.0), 20, "bf16")
        rs = None
        if fused:
            rs = enable_peer_reduce_scatter(model, timeout_s=20.0)
            assert opt.fuse_with_reduce_scatter() > 0
        curve = []
        for _ in range(4):
            loss = model(x, targets=y)[0].mean()
            loss.backward()
            model.grad_all_reduce()
            model.finish_backward()
            opt.step(); sched.step(); opt.zero_grad()
            curve.append(loss.item())
        if fused:
            torch.cuda.synchronize()
            rs.check()
        cuda_ops.check_kernel_errors()
        shard = torch.cat([p.detach().float().reshape(-1)[:4096] for p in model.parameters()])
        out[fused] = (curve, shard.cpu())
    return out


def test_fsdp_reduce_scatter_fused_with_adamw_matches_separate_kernels():
    _need_gpus(2)
    for r in _run(_fsdp_rs_adamw_case):
        (c0, s0), (c1, s1) = r[False], r[True]
        for l0, l1 in zip(c0, c1):
            assert abs(l0 - l1) < 5e-2, (c0, c1)
        assert c1[-1] < c1[0], c1                       # it actually trains
        assert (s0 - s1).abs().max().item() < 2e-2, (s0 - s1).abs().max().item()


def test_benchmark_restarts_on_nccl_after_a_host_made_rank_failure():
    """Rank 1 of a two-GPU benchmark run raises on the host between two warm-up steps (nothing of it in
    flight).  Rank 0's next bounded peer wait runs out, both ranks restart themselves with the NCCL
    transport, meet at the new rendezvous port and finish; the result line says what happened."""
    _need_gpus(2)
    import json
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MEGALODON_B200_BENCH_FAIL_AT="1:0",
               MEGALODON_B200_PEER_TIMEOUT_S="2")
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "MEGALODON_B200_BENCH_RESTARTED"):
        env.pop(k, None)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", str(_free_port()), os.path.join(root, "bench.py"), "--gpus", "2", "--steps", "2",
           "--warmup", "3", "--layers", "2", "--seq-len", "16384", "--step-timeout-s", "60"]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-3000:]
    line = [l for l in res.stdout.splitlines() if l.startswith("{")][-1]
    out = json.loads(line)
    assert "transport_fallback" in out["config"], out["config"]
    assert "nccl" in out["config"]["parallelism"]
    assert out["value"] > 0 and out["config"]["final_loss"] == out["config"]["final_loss"]
    assert "restarting with --transport nccl" in res.stderr


def _small_collective_case(rank, world):
    import torch.distributed as dist
    from megalodon_b200.parallel.symm import SmallCollective
    dev = torch.device("cuda", rank)
    sc = SmallCollective(None, dev, max_bytes=1 << 18, timeout_s=5.0)
    ok = True
    g = torch.Generator(device=dev).manual_seed(100 + rank)
    # eager: sums and gathers of several shapes, against NCCL
    for shape in [(1, 1, 4096), (4, 1, 512), (16, 1, 2048), (3, 1, 8)]:
        x = torch.randn(shape, device=dev, generator=g).bfloat16()
        ref = x.float().clone()
        dist.all_reduce(ref)
        got = sc.all_reduce(x)
        ok = ok and torch.allclose(got.float(), ref, atol=0.06, rtol=0.02)
        parts = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(parts, x)
        ok = ok and torch.equal(sc.all_gather_last_dim(x), torch.cat(parts, dim=-1))
    # every rank holds the same bits
    x = torch.randn(8, 1, 1024, device=dev, generator=g).bfloat16()
    mine = sc.all_reduce(x)
    parts = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(parts, mine)
    ok = ok and all(torch.equal(p, mine) for p in parts)
    # captured: three collectives per replay, inputs rewritten between replays
    a = torch.zeros(4, 1, 1024, device=dev, dtype=torch.bfloat16)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, capture_error_mode="thread_local"):
        s1 = sc.all_reduce(a)
        s2 = sc.all_gather_last_dim(s1 * 0.5)
        s3 = sc.all_reduce(s2[..., :512].contiguous())
    for it in range(6):
        a.copy_(torch.full_like(a, float(rank + 1 + it)))
        graph.replay()
        torch.cuda.synchronize()
        total = sum(r + 1 + it for r in range(world))
        ok = ok and bool((s1.float() == total).all()) and bool((s2.float() == 0.5 * total).all())
        ok = ok and bool((s3.float() == 0.5 * total * world).all())
    # eager calls after the replays continue the same epoch sequence
    got = sc.all_reduce(torch.ones(2, 1, 64, device=dev, dtype=torch.bfloat16))
    ok = ok and bool((got.float() == world).all())
    torch.cuda.synchronize()
    sc.check()
    return ok


@pytest.mark.parametrize("world", WORLDS)
def test_small_collectives_eager_and_graph_replayed(world):
    _need_gpus(world)
    assert all(_run(_small_collective_case, world))


def _tp_graph_decode_case(rank, world):
    from megalodon_b200.config import ModelConf
    from megalodon_b200.decoding import DecodeSession
    from megalodon_b200.models.mega import build_model
    from megalodon_b200.ops import cuda_ops
    from megalodon_b200.parallel import initialize_model_parallel
    from megalodon_b200.utils import init_cache, set_random_seed
    initialize_model_parallel(world, 1)
    cfg = ModelConf(num_layers=2, model_dim=256, num_heads=2, z_dim=128, value_dim=512, ffn_hidden_dim=512,
                    cema_ndim=16, chunk_size=128, vocab_size=512, swiglu=True, norm_num_groups=16,
                    efficient_attn="fused")
    set_random_seed(0)
    model = build_model(cfg, "bf16", False, False)
    model.eval()
    inner = model._wrapped
    B = 2
    prompt = torch.randint(0, 512, (B, 128 + 120), generator=torch.Generator().manual_seed(1)).cuda()
    with torch.no_grad():
        cache = init_cache(B, inner, torch.bfloat16, device=prompt.device)
        _, cache = model(prompt[:, :128], cache=cache)
        logits, cache = model(prompt[:, 128:], cache=cache)
        sess = DecodeSession(model, B, torch.bfloat16)
        sess.load_cache(cache)
        tok = logits[:, -1].argmax(-1)
        worst = 0.0
        for _ in range(14):                       # crosses the chunk boundary at 128
            ref, cache = model(tok.view(B, 1), cache=cache)
            got = sess.step(tok)
            worst = max(worst, (ref[:, -1] - got).abs().max().item())
            tok = ref[:, -1].argmax(-1)
        torch.cuda.synchronize()
        cuda_ops.check_kernel_errors()
    return worst, sess._graph is not None


def test_tensor_parallel_decode_replays_from_a_cuda_graph():
    _need_gpus(2)
    for worst, captured in _run(_tp_graph_decode_case):
        assert captured, "the tensor-parallel step was not captured"
        assert worst < 0.2, worst
