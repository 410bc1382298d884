"""Headline benchmark: Megalodon-7B training throughput (tokens/s) at 32K context.

    python bench.py --gpus N --steps K --warmup W            # this framework
    python bench.py --impl reference ...                      # the unmodified reference, if installable

One sequence of 32768 tokens per step (global batch 1).  With N GPUs the
sequence is split over a chunk-parallel group of size N (4096-token chunks,
CEMA / TimestepNorm state handed from rank to rank) and parameters, gradients
and optimiser state are sharded over the same group; with N = 1 the whole
sequence runs on one GPU, layer-checkpointed and fed chunk by chunk.  So the
total work per step is fixed ("strong" scaling).  A step is: host->device copy
of the tokens, forward, cross-entropy, backward, gradient reduction, global-norm
clipping, AdamW (fp32 master weights + moments), and a device->host read of the
loss.

Two timed regions, both with CUDA events on the compute stream, max over ranks:
`value` - K steps with the batch already resident on the device; `e2e` - K steps
including the per-step H2D copy from pinned memory and the D2H loss read.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

# before CUDA initialises: peer-waiting kernels must never be held up by a lazy kernel load
os.environ.setdefault("CUDA_MODULE_LOADING", "EAGER")
os.environ.setdefault("CUDA_DEVICE_MAX_CONNECTIONS", "32")    # one hardware queue per stream in use
# growable segments: the step allocates 154 GB of 180; fixed-size segments left 17 GB reserved but unusable
os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "Megalodon-7B train tokens/s @32K ctx"


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--ckpt-layers", type=int, default=None,
                    help="checkpoint only the first K layers (default: 27 at N=1, 8 at N=2, none from N=4)")
    ap.add_argument("--kernel-profile", default=None,
                    help="after the timed regions, run one more step under torch.profiler and write a per-kernel "
                         "summary to this path (rank number appended); never part of a reported number")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--seq-len", type=int, default=32768)
    ap.add_argument("--model", default="mega7B_32k")
    ap.add_argument("--layers", type=int, default=None, help="override depth (debugging only; marks the run invalid)")
    ap.add_argument("--gemm", default=None, choices=[None, "tcgen05", "tcgen05_1cta", "cublas"])
    ap.add_argument("--no-ckpt", action="store_true")
    ap.add_argument("--recompute-scores", action="store_true",
                    help="attention keeps row maxima instead of probabilities for backward (memory for time)")
    ap.add_argument("--composition", default="fused", choices=["fused", "library"],
                    help="library: the same model and step as a composition of library calls inside this framework "
                         "(cuBLAS products, materialised matmul + softmax attention, NCCL hand-off / all-gather / "
                         "reduce-scatter) - a context number for the fused paths, NOT the reference")
    ap.add_argument("--transport", default="peer", choices=["peer", "nccl"],
                    help="N > 1: 'peer' moves the chunk hand-off, the parameter gathers and the gradient "
                         "reduce-scatter through peer memory with this package's kernels; 'nccl' keeps every fused "
                         "compute kernel but moves those three through NCCL.  A 'peer' run whose bounded peer wait "
                         "or step watchdog fires restarts itself ONCE with 'nccl' and says so in its result line")
    ap.add_argument("--step-timeout-s", type=float, default=150.0,
                    help="a rank whose host makes no step progress for this long dumps its Python stacks and the "
                         "device's abort record to stderr and exits non-zero (the launcher then stops the others)")
    return ap.parse_args()


class StepWatchdog:
    """Host-side guard of the benchmark loop.  A daemon thread looks at two things once a second:
    the time since the main thread last finished enqueuing a step, and the pinned mirror of the
    device's abort record (set by the first kernel whose bounded wait on a peer ran out).  Either one
    ends the process with a report instead of leaving N GPUs waiting for the collective timeout."""

    def __init__(self, rank: int, timeout_s: float, abort_record=None, restart_argv=None):
        self.rank, self.timeout_s, self.abort = rank, timeout_s, abort_record
        self.restart_argv = restart_argv      # set: a failure restarts this rank with the NCCL transport
        self.last = time.time()
        self.where = "start"
        self._stop = False
        threading.Thread(target=self._run, daemon=True).start()

    def progress(self, where: str) -> None:
        self.last = time.time()
        self.where = where
        if os.environ.get("MEGALODON_B200_BENCH_VERBOSE"):
            print(f"[rank {self.rank}] {time.strftime('%H:%M:%S')} {where}", file=sys.stderr, flush=True)

    def stop(self) -> None:
        self._stop = True

    def _leave(self, code: int, why: str) -> None:
        """End this rank: with a restart command line, replace the process by one that uses the NCCL
        transport (every rank's watchdog sees the same stalled step and does the same; they meet again at
        a new rendezvous port, since the first store still holds the keys of the first process group);
        without one, exit non-zero so that the launcher stops the other ranks."""
        if self.restart_argv is None:
            os._exit(code)
        env = dict(os.environ)
        env["MEGALODON_B200_BENCH_RESTARTED"] = f"{why} (rank {self.rank}, after '{self.where}')"[:300]
        env["MASTER_PORT"] = str(int(env.get("MASTER_PORT", "29500")) + 1)
        env["TORCHELASTIC_USE_AGENT_STORE"] = "False"
        print(f"[rank {self.rank}] restarting with --transport nccl: {why}", file=sys.stderr, flush=True)
        sys.stdout.flush()
        # every descriptor but the standard three is marked close-on-exec (the driver's device files among
        # them), so that this process' device memory is released when its successor takes over; marking,
        # not closing, because the other threads of this process run until the exec
        import fcntl
        for name in os.listdir("/proc/self/fd"):
            try:
                if int(name) > 2:
                    fcntl.fcntl(int(name), fcntl.F_SETFD, fcntl.FD_CLOEXEC)
            except (OSError, ValueError):
                pass
        os.execve(sys.executable, [sys.executable] + self.restart_argv, env)

    def _run(self):
        import faulthandler
        tripped_at = None
        while not self._stop:
            time.sleep(1.0)
            if self.abort is not None and self.abort.tripped():
                if tripped_at is None:
                    tripped_at = time.time()
                    from megalodon_b200.parallel.symm import describe_abort
                    print(f"[rank {self.rank}] peer wait failed after '{self.where}': "
                          f"{describe_abort(self.abort.host.tolist())}", file=sys.stderr, flush=True)
                elif time.time() - tripped_at > 20.0:      # the main thread had its chance to raise
                    self._leave(4, "a bounded wait on a peer ran out")
            if time.time() - self.last > self.timeout_s:
                print(f"[rank {self.rank}] no progress for {self.timeout_s:.0f} s after '{self.where}'; stacks:",
                      file=sys.stderr, flush=True)
                faulthandler.dump_traceback(file=sys.stderr, all_threads=True)
                self._leave(3, f"no step progress for {self.timeout_s:.0f} s")


class ClockSampler:
    """Samples SM clock / power / throttle reasons of one GPU with nvidia-smi while active."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.rows = []
        self.proc = None
        self.since = 0.0

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            if time.time() >= self.since:
                self.rows.append([c.strip() for c in line.split(",")])

    def count_from_now(self):
        """Drop what was sampled so far: the sampler is started during the warm-up (the start of the
        `nvidia-smi` process and its first driver queries stay out of the timed steps) and only samples
        taken inside the timed regions are reported."""
        self.since = time.time()
        self.rows.clear()

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 7:
                continue
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except ValueError:
                continue
            for name, flag in zip(names, r[3:7]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def reference_arm(args):
    """The reference cannot be run here: its extension does not compile against
    torch 2.11 and it imports fairscale and apex, neither installable offline."""
    why = ("reference not installable offline: `pip install --no-index` of the unmodified source fails "
           "(csrc/ops/attention_kernel.cu uses at::Context::alertCuBLASConfigNotDeterministic, removed from "
           "torch 2.11) and its model imports fairscale + apex, which are not in the wheelhouse")
    ref_root = os.path.join(ROOT, "baseline", "_ref")
    if os.path.isdir(os.path.join(ref_root, "megalodon")):
        # an install exists: drive it through the reference's own API (baseline/reference_driver.py)
        try:
            sys.path.insert(0, os.path.join(ROOT, "baseline"))
            import reference_driver
            out = reference_driver.run(args, ref_root)
            if out is not None:
                out["metric"] = METRIC
                out["vs_baseline"] = None
                print(json.dumps(out))
            return
        except Exception as e:  # noqa: BLE001
            why = f"reference installed but does not run: {type(e).__name__}: {e}"[:300]
    if int(os.environ.get("RANK", "0")) == 0:          # one line per job, also when launched as N ranks
        print(json.dumps({"impl": "reference", "unavailable": why}))


def step_roofline(cfg, seq_len: int, world: int, ms_per_step: float) -> dict:
    """Matrix-product arithmetic of one step against the measured cuBLAS throughput: forward + backward
    of every layer and the vocabulary projection, plus the recomputed forward of the checkpointed layers."""
    from megalodon_b200.utils.profiling import measured_peaks, model_flops_per_token
    base = model_flops_per_token(cfg, with_recompute=False)            # forward + backward per token
    n_ckpt = 0 if not cfg.layerwise_ckpt else (cfg.num_layers if cfg.ckpt_layers is None else cfg.ckpt_layers)
    vocab = cfg.vocab_size if cfg.output_size == -1 else cfg.output_size
    layer_fwd = (base - 6.0 * cfg.model_dim * vocab) / 3.0 / cfg.num_layers   # one layer's forward per token
    flops_step = (base + n_ckpt * layer_fwd) * seq_len
    pk = measured_peaks()
    per_gpu = flops_step / world / (ms_per_step / 1e3)
    return {"pflop_per_step": round(flops_step / 1e15, 3),
            "achieved_tflops_per_gpu": round(per_gpu / 1e12, 1),
            "fraction_of_sustained_cublas": round(per_gpu / (pk["bf16_tflops_sustained"] * 1e12), 3),
            "fraction_of_burst_cublas": round(per_gpu / (pk["bf16_tflops"] * 1e12), 3),
            "peaks": pk["source"]}


_WATCHDOG = []       # the running benchmark's watchdog, for the handler of an exception that escapes run()


def main():
    args = parse()
    if args.impl == "reference":
        reference_arm(args)
        return
    try:
        run(args)
    except Exception as e:  # noqa: BLE001 - a peer-transport run gets its one restart on NCCL
        if not _WATCHDOG or _WATCHDOG[0].restart_argv is None or "OutOfMemory" in type(e).__name__:
            raise               # (running out of memory has nothing to do with the transport)
        import traceback
        traceback.print_exc()
        _WATCHDOG[0]._leave(5, f"{type(e).__name__}: {e}"[:200])


def run(args):

    import torch
    import torch.distributed as dist
    from megalodon_b200.config import OptimConf
    from megalodon_b200.data.dataloader import SyntheticTokens
    from megalodon_b200.models.mega import ModelStore, build_model
    from megalodon_b200.optim import build_optimizer
    from megalodon_b200.ops import cuda_ops
    from megalodon_b200.parallel import init_torch_distributed, initialize_model_parallel
    from megalodon_b200.utils import clip_grad_norm_, set_random_seed
    import dataclasses

    world = int(os.environ.get("WORLD_SIZE", "1"))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun for N > 1"
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    rank = 0
    if world > 1:
        # a collective that takes minutes is a failure here: end the job rather than occupy N GPUs
        info = init_torch_distributed(timeout=300)
        rank = info.global_rank
        initialize_model_parallel(1, world)
    if args.gemm:
        cuda_ops.set_gemm_backend(args.gemm)
    library = args.composition == "library"
    if library:
        cuda_ops.set_gemm_backend("cublas")

    cfg = dataclasses.replace(ModelStore[args.model])
    if args.layers is not None:
        cfg.num_layers = args.layers
    if library:
        cfg.efficient_attn = None             # matmul + softmax with the scores written out
    local_len = args.seq_len // world
    chunks_local = local_len // cfg.chunk_size
    # One GPU holds the whole 32K sequence only with layer checkpointing.  Activations cost about 1 GB
    # per layer and 4096-token chunk, optimiser state 137 GB / N: from two chunks per GPU down (N >= 4)
    # everything fits in 180 GB without recomputation.
    cfg.layerwise_ckpt = (not args.no_ckpt) and chunks_local > 2
    if args.ckpt_layers is not None:
        cfg.ckpt_layers = args.ckpt_layers
    elif chunks_local == 8:
        # N = 1: 138 GB of optimiser state and 7.6 GB of activations per un-checkpointed layer; measured peaks
        # with growable segments: 28 checkpointed layers 153.6 GB, 26 168.8 GB, 25 176.4 GB (of 178.4)
        cfg.ckpt_layers = 27
    elif chunks_local == 4:
        # N = 2: state 86 GB + 2.7 GB of activations per un-checkpointed layer.  Measured with growable
        # segments and the parameter gathers in peer memory: 16 checkpointed layers 130.6 GB and 1410 ms,
        # 8 layers 161.0 GB and 1292 ms, 4 layers out of memory.  The NCCL transport holds 9 GB more
        # (gather and reduce-scatter staging), so a restarted run goes back to 16.
        cfg.ckpt_layers = 8 if (args.transport == "peer" and not os.environ.get("MEGALODON_B200_BENCH_RESTARTED")
                                and not library) else 16
    if library and cfg.layerwise_ckpt and args.ckpt_layers is None:
        # the materialised fp32 scores add about 3 GB per un-checkpointed layer and 32K tokens
        cfg.ckpt_layers = 32 if chunks_local == 8 else 24
    if args.recompute_scores:
        # keeping the row maxima instead of the attention probabilities frees 0.54 GB per un-checkpointed
        # layer and 16K tokens; the extra score pass costs 54 us per layer and chunk in backward
        cuda_ops.set_attention_recompute_scores(True)
    set_random_seed(1234)
    model = build_model(cfg, "bf16", fp32_reduce_scatter=False, reshard_after_forward=False,
                        shard_over_chunk_group=True)
    model._wrapped.seq_microbatch_chunks = 1
    model.defer_grad_clip = True      # clipping coefficient is applied inside the fused AdamW kernel
    restarted = os.environ.get("MEGALODON_B200_BENCH_RESTARTED")
    peer = world > 1 and not library and args.transport == "peer" and not restarted
    if world > 1 and not peer:
        mailbox, abort_record = None, None    # NCCL send / recv, all-gather and reduce-scatter
    elif world > 1:
        # CEMA / TimestepNorm state goes from rank to rank through peer memory, not NCCL send/recv
        from megalodon_b200.parallel.symm import enable_peer_transport
        from megalodon_b200.parallel.symm import AbortRecord
        peer_timeout = float(os.environ.get("MEGALODON_B200_PEER_TIMEOUT_S", "10"))
        mailbox, _ = enable_peer_transport(model, max_batch=1, n_slots=8, timeout_s=peer_timeout)
        abort_record = AbortRecord.get(torch.device("cuda", local_rank))
    else:
        abort_record = None
    restart_argv = None
    if peer:
        restart_argv = [os.path.abspath(__file__)] + [a for a in sys.argv[1:]] + ["--transport", "nccl"]
    dog = StepWatchdog(rank, args.step_timeout_s, abort_record, restart_argv)
    _WATCHDOG.append(dog)
    opt, sched = build_optimizer(model, OptimConf(lr=1e-4, warmup=10, clip=1.0), 1000, "bf16")
    data = SyntheticTokens(cfg.vocab_size, 1, args.seq_len, seed=0)
    n_params = sum(p.numel() for p in model.parameters()) * (world if world > 1 else 1)

    def step(x_host, y_host, read_loss: bool):
        x = x_host.cuda(non_blocking=True)
        y = y_host.cuda(non_blocking=True)
        tok_loss, _ = model(x, targets=y)
        loss = tok_loss.mean()
        loss.backward()
        model.grad_all_reduce()
        clip_grad_norm_(model, 1.0)
        opt.step()
        sched.step()
        opt.zero_grad()
        return loss.item() if read_loss else loss

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def peer_failure(e):
        # every rank's record is poisoned by the first failure, so every rank comes through here
        print(f"[rank {rank}] {e}", file=sys.stderr, flush=True)
        dog._leave(4, "a bounded wait on a peer ran out")

    def check_peers():
        # a bounded device-side wait that ran out shows up here instead of slowing every later step
        cuda_ops.check_kernel_errors()
        if abort_record is not None:
            try:
                abort_record.check()
            except Exception as e:  # noqa: BLE001 - PeerTimeout: every rank restarts on the NCCL transport
                peer_failure(e)

    def peers_ok_so_far():
        # host-only look at the pinned mirror of the abort record: costs nothing inside a timed region
        if abort_record is not None and abort_record.tripped():
            torch.cuda.synchronize()
            check_peers()

    # The last two warm-up steps are enqueued back to back like the steps of the first timed region (no
    # host synchronisation between them): with side streams (N > 1) the caching allocator only reaches its
    # steady state once the host runs ahead of the device - blocks released on another stream are not yet
    # reusable - and that one-time growth (0.1 - 0.5 s) belongs to the warm-up, not to a timed step.
    synced = max(1, args.warmup - 2)
    tail = None
    sampler = ClockSampler(local_rank)
    for i in range(args.warmup):
        x, y = next(data)
        if i == args.warmup - 1:
            sampler.start()
        if i < synced:
            last = step(x, y, True)
            torch.cuda.synchronize()
            check_peers()
            dog.progress(f"warm-up step {i} done, loss {last:.4f}")
            if peer and os.environ.get("MEGALODON_B200_BENCH_FAIL_AT") == f"{rank}:{i}":
                # failure drill, made on the host between two steps (nothing of this rank in flight): this
                # rank raises, the others find out when their next bounded peer wait runs out
                raise RuntimeError(f"injected host failure on rank {rank} after warm-up step {i}")
        else:
            tail = step(x.cuda(), y.cuda(), False)
            dog.progress(f"warm-up step {i} enqueued")
    torch.cuda.synchronize()
    check_peers()
    if tail is not None:
        last = tail.item()
        dog.progress(f"warm-up done, loss {last:.4f}")

    if sampler.proc is None:
        sampler.start()

    # ---- region 1: batch resident on the device
    x, y = next(data)
    xd, yd = x.cuda(), y.cuda()
    barrier()
    sampler.count_from_now()
    launches0 = cuda_ops.count_launches()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    marks = []           # per step: events at the phase boundaries (recording an event costs no device time)

    def mark():
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        return ev

    e0.record()
    for i in range(args.steps):
        peers_ok_so_far()
        dog.progress(f"timed step {i} being enqueued")
        m = [mark()]
        tok_loss, _ = model(xd, targets=yd)
        loss = tok_loss.mean()
        m.append(mark())
        loss.backward()
        m.append(mark())
        model.grad_all_reduce()
        clip_grad_norm_(model, 1.0)
        m.append(mark())
        opt.step()
        sched.step()
        opt.zero_grad()
        m.append(mark())
        marks.append(m)
    e1.record()
    barrier()
    dev_ms = e0.elapsed_time(e1)
    launches = cuda_ops.count_launches() - launches0
    steps_ms = [marks[i][0].elapsed_time(marks[i][4]) for i in range(args.steps)]
    phase_names = ["forward", "backward", "grad_reduce_clip", "optimizer"]
    phases = {n: sum(m[i].elapsed_time(m[i + 1]) for m in marks) / args.steps for i, n in enumerate(phase_names)}

    # ---- region 2: end to end (H2D of the tokens from pinned memory, D2H of the loss, every step)
    barrier()
    e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_wall = time.perf_counter()
    e2.record()
    for i in range(args.steps):
        x, y = next(data)
        last = step(x, y, True)
        peers_ok_so_far()
        dog.progress(f"end-to-end step {i} done")
    e3.record()
    barrier()
    e2e_ms = e2.elapsed_time(e3)
    wall_ms = (time.perf_counter() - t_wall) * 1e3
    clocks = sampler.stop()
    check_peers()
    dog.progress("timed regions done")

    if args.kernel_profile:
        import collections
        from torch.profiler import ProfilerActivity, profile
        barrier()
        p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            p0.record()
            step(x, y, False)
            p1.record()
            torch.cuda.synchronize()
        agg = collections.defaultdict(lambda: [0.0, 0])
        spans = []
        for e in prof.events():
            if e.device_type == torch.autograd.DeviceType.CUDA:
                agg[e.name][0] += e.device_time
                agg[e.name][1] += 1
                spans.append((e.time_range.start, e.time_range.end))
        spans.sort()
        busy, cur_s, cur_e = 0.0, None, None          # union of kernel intervals = time the GPU was not idle
        for a, b in spans:
            if cur_e is None or a > cur_e:
                if cur_e is not None:
                    busy += cur_e - cur_s
                cur_s, cur_e = a, b
            else:
                cur_e = max(cur_e, b)
        if cur_e is not None:
            busy += cur_e - cur_s
        tot = sum(v[0] for v in agg.values())
        with open(f"{args.kernel_profile}.rank{rank}", "w") as f:
            f.write(f"step (CUDA events, under the profiler) {p0.elapsed_time(p1):.1f} ms; sum of kernel times "
                    f"{tot / 1e3:.1f} ms; GPU busy (union of kernel intervals) {busy / 1e3:.1f} ms\n")
            for name, (t, n) in sorted(agg.items(), key=lambda kv: -kv[1][0])[:45]:
                f.write(f"{t / 1e3:9.2f} ms {100 * t / tot:5.1f}% {n:6d}x {t / n:9.1f} us  {name[:120]}\n")

    if world > 1:
        t = torch.tensor([dev_ms, e2e_ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dev_ms, e2e_ms = t.tolist()
    if rank == 0:
        tokens = args.seq_len * args.steps
        value = tokens / (dev_ms / 1e3)
        out = {
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": dev_ms / args.steps, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "impl": "ours" if not library else "library-composition (cuBLAS + NCCL + materialised attention in this framework; not the reference)",
            "config": {
                "model": f"{args.model} (L{cfg.num_layers} D{cfg.model_dim} H{cfg.num_heads} z{cfg.z_dim} "
                         f"v{cfg.value_dim} ffn{cfg.ffn_hidden_dim} swiglu N{cfg.cema_ndim} chunk{cfg.chunk_size} "
                         f"V{cfg.vocab_size}), {n_params / 1e9:.2f}B params",
                "global_batch": 1, "seq_len": args.seq_len,
                "parallelism": f"cp{world}" + (("+zero3_over_cp+p2p_handoff+gathering_gemm" if peer else "+zero3_over_cp+nccl")
                                               if world > 1 else ""),
                "activation_checkpointing": (False if not cfg.layerwise_ckpt else
                                             ("all layers" if cfg.ckpt_layers is None else f"first {cfg.ckpt_layers} layers")),
                "optimizer": "AdamW fp32 master+moments, clip 1.0",
                "gemm_backend": cuda_ops.gemm_backend(),
                "l2": "working set (17 GB bf16 weights + activations) streams through L2 every step; no flush needed",
                "final_loss": last,
            },
            "clocks": clocks,
            "e2e": {"value": tokens / (e2e_ms / 1e3), "unit": "tokens/s", "ms_per_step": e2e_ms / args.steps,
                    "wall_ms_per_step": wall_ms / args.steps,
                    "h2d_bytes_per_step": 2 * args.seq_len * 8, "d2h_bytes_per_step": 4},
            "gpu_launches": launches,
            "peak_mem_gb_rank0": {"allocated": round(torch.cuda.max_memory_allocated() / 2 ** 30, 1),
                                  "reserved": round(torch.cuda.max_memory_reserved() / 2 ** 30, 1)},
            "phases_ms_rank0": {k: round(v, 1) for k, v in phases.items()},
            "steps_ms_rank0": [round(v, 1) for v in steps_ms],
        }
        try:
            out["roofline"] = step_roofline(cfg, args.seq_len, world, dev_ms / args.steps)
        except Exception as e:  # noqa: BLE001 - never lose the result line over the derived figures
            out["roofline"] = {"error": repr(e)[:200]}
        if restarted:
            out["config"]["transport_fallback"] = ("the peer-memory transport failed and the run restarted itself "
                                                   "with NCCL for hand-off, gathers and reduce-scatter: " + restarted)
        if args.layers is not None:
            out["invalid"] = "reduced depth (debug run)"
        print(json.dumps(out))
    dog.progress("result printed")
    if world > 1:
        dist.barrier()
        dog.progress("final barrier passed")
        dist.destroy_process_group()
    dog.stop()


if __name__ == "__main__":
    main()
