#!/usr/bin/env python
"""Benchmark of the Mega EMA layer path: fused TimestepNorm -> EMA forward, tokens/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload c4|c1] [--scaling weak|strong]

One "step" is one pass of the hot path over one batch of seeded synthetic input.  The default
workload is BASELINE config 4: bf16 x of shape (B=64, L=32768, D=2048), per-feature
TimestepNorm (weight=1, bias=0, eps=1e-5, prior count 2) followed by the causal ndim=16 EMA.
Under torchrun every rank runs the same per-rank batch on its own seed ("weak", the default)
or a 1/N shard of the global batch ("strong"); no collective sits on the data path.

Prints ONE JSON line (rank 0).  `value` = whole-job tokens/s with inputs resident in HBM,
timed with CUDA events, max over ranks.  `e2e` = the same metric through the host-buffer API
(pinned host input -> device -> kernel -> pinned host output inside the timed region).
`roofline` compares algorithmic bytes (2 * D * sizeof(elem) per token) per launch with the
measured HBM copy peak.  `cpu_baseline` times the reference's CPU path (its TimestepNorm C++
op from oracle/_ref when built, and the oracle's restatement of its FFT convolution) on a
bounded sample.  `--impl reference` prints that CPU measurement as its own line.
"""
import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (B, L, D, dtype)   fused TimestepNorm -> causal EMA
    "c4": (64, 32768, 2048, "bf16"),
    "c1": (16, 4096, 1024, "bf16"),
    "tiny": (4, 2048, 256, "bf16"),
}
# side workloads (BASELINE configs 0, 2 and the decode half of config 4): own JSON line, N=1 only
AUX_WORKLOADS = ("c0", "c2", "c3", "decode", "cema", "train", "c4n", "c1n", "c4pad")
# side workloads measured after the headline run and reported under its "aux" key (N = 1 only)
AUX_IN_HEADLINE = ("c0", "c1", "c2", "c3", "c4n", "c4pad", "cema", "train", "decode")
NDIM = 16
FALLBACK_HBM_GBS = 6650.0
CPU_DETAIL = {
    "reference+port": "TimestepNorm: the reference's own compiled CPU operator (oracle/_ref); EMA: the oracle's "
                      "port of the reference's torch.fft flow (the reference's Python cannot travel)",
    "port": "TimestepNorm and EMA through the oracle's port of the reference's CPU flow",
}


def make_ema_params(gen, dim, ndim):
    import torch
    alpha = torch.randn(dim, ndim, 1, generator=gen) * 0.2
    delta = torch.randn(dim, ndim, 1, generator=gen) * 0.2
    val = torch.ones(ndim, 1)
    val[1::2] = -1.0
    beta = torch.randn(dim, ndim, 1, generator=gen) * 0.02 + val
    gamma = torch.randn(dim, ndim, generator=gen)
    omega = torch.randn(dim, generator=gen)
    return alpha, delta, beta, gamma, omega


def hbm_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons of one GPU while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self, t0, t1):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        rows = [l for (t, l) in self.lines if t0 - 0.05 <= t <= t1 + 0.15] or [l for (_, l) in self.lines]
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in rows:
            f = [v.strip() for v in r.split(",")]
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except Exception:
                continue
            for n, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------ CPU reference arm
def cpu_reference_step_factory(dim, length, sample_b, sample_d):
    """Builds the reference's CPU path on a bounded sample: TimestepNorm through the
    reference's own C++ op (oracle/_ref) when it is built, else the oracle port, followed by
    the EMA through the oracle's restatement of the reference's FFT convolution."""
    import torch
    from oracle import mega_oracle as O
    from oracle.build_ref import load_ref
    ref = load_ref()
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    gen = torch.Generator().manual_seed(4321)
    x = torch.randn(sample_b, length, sample_d, generator=gen).to(torch.bfloat16)
    prm = make_ema_params(gen, sample_d, NDIM)
    pc = torch.full((sample_b,), 2, dtype=torch.int64)
    pm = torch.zeros(sample_b, sample_d, dtype=torch.bfloat16)
    pv = torch.ones(sample_b, sample_d, dtype=torch.bfloat16)
    gamma = torch.ones(sample_d, dtype=torch.bfloat16)
    beta = torch.zeros(sample_d, dtype=torch.bfloat16)
    kind = "reference+port" if ref is not None else "port"

    def step():
        with torch.no_grad():
            if ref is not None:
                xn = ref.ops.timestep_norm_fwd(x, pc, pm, pv, gamma, beta, None, 1e-5)[0]
            else:
                xn = O.timestep_norm(x, pc, pm.float(), pv.float(), gamma.float(), beta.float(), None)[0]
            y = O.ema_forward_fft(xn.transpose(1, 2).contiguous(), *prm)
        return y

    return step, kind, cores


def time_cpu(step, steps, warmup):
    for _ in range(warmup):
        step()
    ts = []
    for _ in range(steps):
        t0 = time.perf_counter()
        step()
        ts.append(time.perf_counter() - t0)
    return sum(ts) / len(ts)


def reference_gpu_leg(L, D):
    """Informative: the reference's own GPU path for the EMA on this workload's shape, through its
    CUDA operators compiled unmodified by ``oracle/build_ref.py --cuda`` and the lines of its Python
    flow restated here (base_moving_average.py:137-172; fused_ops/fftconv.py:13-27,45-61: its
    shared-memory FFT kernel up to L = 8192, torch.fft beyond).  The TimestepNorm half is absent:
    the reference's chunked CUDA kernel (L >= 256) does not launch on sm_100 ("too many resources
    requested for launch").  Returns a dict for the JSON line, or None without a GPU / the build."""
    import torch
    if not torch.cuda.is_available():
        return None
    from oracle.build_ref import load_ref_cuda
    mod = load_ref_cuda()
    if mod is None:
        return {"unavailable": "oracle/_ref/mega_ref_cuda.so not built"}
    R = mod.ops
    try:
        dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
        bsz = 8
        gen = torch.Generator().manual_seed(4321)
        alpha, delta, beta, gamma, omega = [t.to(dev) for t in make_ema_params(gen, D, NDIM)]
        x = torch.randn(bsz, D, L, device=dev, dtype=torch.bfloat16)
        n = L if (L & (L - 1)) == 0 else (1 << L.bit_length())

        def step():
            with torch.no_grad():
                p = torch.sigmoid(alpha)
                q = torch.polar(1.0 - p * torch.sigmoid(delta), torch.zeros_like(p))
                g = torch.complex(gamma * beta.squeeze(-1), torch.zeros_like(gamma)) * (1.0 / NDIM) ** 0.5
                w, _, _ = R.ema_parameters_fwd(p, q.log(), g, None, L)
                if 32 <= L <= 8192:
                    y, _ = R.fftconv_fwd(x, torch.fft.rfft(w.float(), 2 * n))
                else:
                    x_f = torch.fft.rfft(x.float(), n=2 * n)
                    k_f = torch.fft.rfft(w, n=2 * n, norm="forward")
                    y = torch.fft.irfft(x_f * k_f, n=2 * n, norm="forward")[..., :L].to(x.dtype)
                return y + x * omega.view(D, 1).to(x.dtype)

        for _ in range(2):
            step()
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(3):
            step()
        e1.record()
        torch.cuda.synchronize(dev)
        ms = e0.elapsed_time(e1) / 3
        return {"value": bsz * L / (ms * 1e-3), "unit": "tokens/s", "ms_per_step": ms,
                "what": "EMA only (no TimestepNorm: the reference's kernel does not launch on sm_100 for L >= 256), "
                        "B=%d L=%d D=%d bf16 on one GPU" % (bsz, L, D)}
    except Exception as exc:  # a reference kernel that does not run here is reported, not fatal
        return {"unavailable": str(exc).splitlines()[0][:200]}


def run_reference(args, B, L, D, dtype_name):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    sample_b, sample_d = min(B, os.cpu_count() or 1), min(D, 64)
    step, kind, cores = cpu_reference_step_factory(D, L, sample_b, sample_d)
    sec = time_cpu(step, max(1, args.steps), max(0, args.warmup))
    tokens = sample_b * L * (sample_d / D)
    val = tokens / sec
    sample = "B=%d, L=%d, %d of %d channels per step (tokens scaled by the channel fraction)" % (
        sample_b, L, sample_d, D)
    line = {
        "impl": "reference", "metric": "mega_ema_layer_tokens_per_s", "value": val, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3,
        "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None, "dtype": dtype_name,
        "data": "synthetic",
        "config": {"workload": workload_name(args, B, L, D, dtype_name), "ndim": NDIM,
                   "path": "reference CPU path: TimestepNorm C++ op + torch.fft convolution"},
        "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": cores, "kind": kind, "sample": sample,
                         "detail": CPU_DETAIL[kind]},
        "reference_scope": "one host's CPU cores, rank 0 only: the number does not grow with --gpus",
        "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    gpu = reference_gpu_leg(L, D)
    if gpu is not None:
        line["reference_gpu"] = gpu
    print(json.dumps(line), flush=True)


def batch_shard(batch, rank, world):
    """Contiguous [lo, hi) slice of the batch owned by `rank` (strong scaling)."""
    base, rem = divmod(batch, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


def job_throughput(tokens_per_rank, world, steps, total_ms):
    """Whole-job tokens/s: all ranks' tokens over the slowest rank's time."""
    return tokens_per_rank * world * steps / (total_ms * 1e-3)


# DRAM bytes per token of the tensor-core kernel (segmented 64-channel form, TimestepNorm -> EMA), from an ncu
# capture of one launch of the current kernel at B=40, L=8192, D=2048: dram__bytes_read.sum 1355.64 MB +
# dram__bytes_write.sum 1330.40 MB for 40 x 8192 tokens (1.0006 of the algorithmic 8192 B per token).  The
# traffic grows with the tokens of a launch.
NCU_DRAM_BYTES_PER_TOKEN_D2048_BF16 = (1355.64e6 + 1330.40e6) / (40 * 8192)
# The unsegmented 56-channel form (what a shard of 32 sequences or fewer runs), captured at B=32, L=4096, D=2048:
# 539.26 MB + 490.85 MB for 32 x 4096 tokens (0.96 of the algorithmic bytes: the tail of the output is still in
# L2 when the kernel ends).
NCU_DRAM_BYTES_PER_TOKEN_D2048_BF16_PLAIN = (539.26e6 + 490.85e6) / (32 * 4096)


def workload_name(args, B, L, D, dtype_name):
    return "%s: TimestepNorm+MultiHeadEMA causal fwd, B=%d L=%d D=%d %s per rank (%s scaling)" % (
        args.workload, B, L, D, dtype_name, args.scaling)


# ------------------------------------------------------------------ GPU arm
def run_ours(args, B, L, D, dtype_name):
    import torch
    import torch.distributed as dist
    import fairseq_apollo_b200 as M

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    if args.scaling == "strong":
        lo, hi = batch_shard(B, rank, world)
        Bl = hi - lo
    else:
        Bl = B
    dtype = torch.bfloat16 if dtype_name == "bf16" else torch.float32
    es = 2 if dtype_name == "bf16" else 4

    gen = torch.Generator().manual_seed(1238 + rank)
    prm = [t.to(dev) for t in make_ema_params(gen, D, NDIM)]
    norm = M.TimestepNorm(D, prior_count=2).to(dev).eval()
    move = M.MultiHeadEMA(D, ndim=NDIM).to(dev).eval()
    with torch.no_grad():
        for dst, src in zip((move.alpha, move.delta, move.beta, move.gamma, move.omega), prm):
            dst.copy_(src)
    dgen = torch.Generator(device=dev).manual_seed(1238 + rank)
    x = torch.empty(Bl, L, D, dtype=dtype, device=dev)
    for b in range(Bl):
        x[b] = torch.randn(L, D, generator=dgen, device=dev, dtype=torch.float32 if L * D < (1 << 26) else dtype).to(dtype)
    p, q, g = move.coeffs()
    p, q = p.squeeze(-1).contiguous(), q.squeeze(-1).contiguous()
    pc = norm.prior_count.expand(Bl).contiguous()
    pm = torch.zeros(Bl, D, device=dev)
    pv = torch.ones(Bl, D, device=dev)
    gamma = torch.ones(D, device=dev)
    beta = torch.zeros(D, device=dev)
    y = torch.empty_like(x)
    cnt = torch.empty(Bl, dtype=torch.int64, device=dev)
    mo = torch.empty(Bl, D, device=dev)
    vo = torch.empty(Bl, D, device=dev)
    from fairseq_apollo_b200 import _lib
    lib = _lib.lib()
    if args.tile:
        _lib.set_option(2, args.tile)
    stream = torch.cuda.current_stream()

    def step(xi=x, yi=y, bl=Bl):
        _lib.check(lib.mega_tsn_ema_fwd(
            xi.data_ptr(), yi.data_ptr(), None, 1 if dtype_name == "bf16" else 0, bl, L, D,
            *xi.stride(), *yi.stride(), pc.data_ptr(), pm.data_ptr(), pv.data_ptr(), gamma.data_ptr(),
            beta.data_ptr(), 1e-5, cnt.data_ptr(), mo.data_ptr(), vo.data_ptr(), p.data_ptr(), q.data_ptr(),
            g.data_ptr(), move.omega.data_ptr(), NDIM, None, None, None, 0, stream.cuda_stream), "tsn_ema_fwd")

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    sampler = ClockSampler(local) if rank == 0 else None
    if sampler:
        sampler.start()
        time.sleep(0.25)
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    l0 = M.launch_count()
    barrier()
    t0 = time.time()
    evs[0].record(stream)
    for i in range(args.steps):
        step()
        evs[i + 1].record(stream)
    barrier()
    t1 = time.time()
    launches = M.launch_count() - l0
    kernel_name = _lib.last_kernel()
    clocks = sampler.stop(t0, t1) if sampler else None
    total_ms = evs[0].elapsed_time(evs[-1])
    per_step = [evs[i].elapsed_time(evs[i + 1]) for i in range(args.steps)]
    tm = torch.tensor([total_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(tm, op=dist.ReduceOp.MAX)
    total_ms = float(tm.item())
    value = job_throughput(Bl * L, world, args.steps, total_ms)

    # ---- end-to-end through host buffers: pinned host x -> device -> kernel -> pinned host y
    # The per-rank batch streams through in slices on three streams (H2D, compute, D2H).  The host
    # side holds the whole per-rank batch (input and output) in pinned memory; if the host cannot
    # pin that much, one pinned slice stands in for every slice (same bytes moved, said in the note).
    sl = max(1, min(Bl, args.e2e_slice))
    nsl = (Bl + sl - 1) // sl
    whole_host_batch = True
    try:
        hx_all = torch.empty(nsl * sl, L, D, dtype=dtype).pin_memory()
        hy_all = torch.empty(nsl * sl, L, D, dtype=dtype).pin_memory()
        for i in range(nsl):
            n = min(sl, Bl - i * sl)
            hx_all[i * sl:i * sl + n].copy_(x[i * sl:i * sl + n])
    except Exception:  # noqa: BLE001 - not enough pinnable host memory
        whole_host_batch = False
        hx_all = torch.empty(sl, L, D, dtype=dtype).pin_memory()
        hy_all = torch.empty(sl, L, D, dtype=dtype).pin_memory()
        hx_all.copy_(x[:sl].cpu())
    hxs = [hx_all[i * sl:(i + 1) * sl] if whole_host_batch else hx_all for i in range(nsl)]
    hys = [hy_all[i * sl:(i + 1) * sl] if whole_host_batch else hy_all for i in range(nsl)]
    dx = [torch.empty(sl, L, D, dtype=dtype, device=dev) for _ in range(2)]
    dy = [torch.empty(sl, L, D, dtype=dtype, device=dev) for _ in range(2)]
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    pc_s = pc[:sl].contiguous()

    def e2e_step():
        ev_in = [torch.cuda.Event() for _ in range(nsl)]
        ev_k = [torch.cuda.Event() for _ in range(nsl)]
        ev_out = [torch.cuda.Event() for _ in range(nsl)]
        for i in range(nsl):
            k = i & 1
            with torch.cuda.stream(s_in):
                if i >= 2:
                    s_in.wait_event(ev_k[i - 2])          # buffer k consumed by the kernel
                dx[k].copy_(hxs[i], non_blocking=True)
                ev_in[i].record(s_in)
            stream.wait_event(ev_in[i])
            if i >= 2:
                stream.wait_event(ev_out[i - 2])          # output buffer k drained
            _lib.check(lib.mega_tsn_ema_fwd(
                dx[k].data_ptr(), dy[k].data_ptr(), None, 1 if dtype_name == "bf16" else 0, sl, L, D,
                *dx[k].stride(), *dy[k].stride(), pc_s.data_ptr(), pm.data_ptr(), pv.data_ptr(), gamma.data_ptr(),
                beta.data_ptr(), 1e-5, cnt.data_ptr(), mo.data_ptr(), vo.data_ptr(), p.data_ptr(), q.data_ptr(),
                g.data_ptr(), move.omega.data_ptr(), NDIM, None, None, None, 0, stream.cuda_stream), "tsn_ema_fwd")
            ev_k[i].record(stream)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_k[i])
                hys[i].copy_(dy[k], non_blocking=True)
                ev_out[i].record(s_out)
        stream.wait_stream(s_out)
        stream.wait_stream(s_in)

    e2e_steps = max(1, min(args.steps, args.e2e_steps))
    e2e_step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(e2e_steps):
        e2e_step()
    e1.record(stream)
    barrier()
    em = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(em, op=dist.ReduceOp.MAX)
    e2e_tokens = nsl * sl * L * world * e2e_steps
    e2e_val = e2e_tokens / (float(em.item()) * 1e-3)
    bytes_dir = nsl * sl * L * D * es

    # ---- verification (outside every timed region): the first sequence's first 4096 positions
    # through the streamed SIMT kernel (a different implementation of the same entry point) against
    # the timed kernel's output, and the end-to-end output in host memory against the device one;
    # every rank's result is gathered to rank 0 (the only collective of the run besides timing).
    step()
    torch.cuda.synchronize()
    vl = min(L, 4096)
    xv, yv = x[:1, :vl].contiguous(), torch.empty(1, vl, D, dtype=dtype, device=dev)
    _lib.set_option(1, 1)
    try:
        step(xv, yv, 1)
    finally:
        _lib.set_option(1, 0)
    ref = yv.float()
    rel = float((y[:1, :vl].float() - ref).norm() / ref.norm())
    e2e_rel = 0.0   # (a slice may run a different tile form than the whole batch: compared within the tolerance)
    if whole_host_batch:
        n = min(sl, Bl)
        ys = y[:n].float()
        e2e_rel = float((hy_all[:n].to(dev).float() - ys).norm() / ys.norm())
        del ys
    chk = torch.tensor([rel, e2e_rel], device=dev, dtype=torch.float64)
    outs = [chk]
    if world > 1:
        outs = [torch.empty_like(chk) for _ in range(world)]
        dist.all_gather(outs, chk)
    verify = {"max_rel_l2_vs_simt_kernel": max(float(o[0]) for o in outs), "tolerance": 1e-2,
              "max_rel_l2_e2e_host_output_vs_device_output": max(float(o[1]) for o in outs)}
    verify["ok"] = (verify["max_rel_l2_vs_simt_kernel"] < 1e-2
                    and verify["max_rel_l2_e2e_host_output_vs_device_output"] < 1e-2)
    del hx_all, hy_all, hxs, hys, dx, dy

    aux = None
    if rank == 0 and world == 1 and not args.no_aux:
        del x, y
        torch.cuda.empty_cache()
        aux = aux_summary(5, 3)
    if rank == 0:
        peak, peak_kind = hbm_peak()
        kern_ms = sum(per_step) / len(per_step)
        alg_bytes = 2.0 * D * es * Bl * L
        achieved = alg_bytes / (kern_ms * 1e-3) / 1e9
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            sample_b, sample_d = min(Bl, os.cpu_count() or 1), min(D, 64)
            cstep, kind, cores = cpu_reference_step_factory(D, L, sample_b, sample_d)
            sec = time_cpu(cstep, 3, 1)
            cpu = {"value": sample_b * L * (sample_d / D) / sec, "unit": "tokens/s", "cores": cores,
                   "kind": kind, "detail": CPU_DETAIL[kind],
                   "sample": "B=%d, L=%d, %d of %d channels, 3 timed passes (tokens scaled by the channel fraction)"
                             % (sample_b, L, sample_d, D)}
        line = {
            "metric": "mega_ema_layer_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": total_ms / args.steps,
            "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None, "dtype": dtype_name,
            "data": "synthetic",
            "config": {"workload": workload_name(args, Bl, L, D, dtype_name), "ndim": NDIM,
                       "global_batch": Bl * world, "l2": "inputs (%.1f GiB per rank) exceed the 126 MB L2"
                       % (Bl * L * D * es / 2**30), "parallelism": "batch shards, no data-path collective"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak,
                         "traffic": ((NCU_DRAM_BYTES_PER_TOKEN_D2048_BF16 if "segmented" in kernel_name
                                      else NCU_DRAM_BYTES_PER_TOKEN_D2048_BF16_PLAIN) * Bl * L
                                     if (D == 2048 and dtype_name == "bf16") else None),
                         "traffic_note": "ncu dram__bytes_read.sum + dram__bytes_write.sum of one launch of this "
                                         "kernel form (segmented: at B=40, L=8192; unsegmented: at B=32, L=4096; "
                                         "D=2048), scaled by the tokens of a launch",
                         "peak_kind": peak_kind,
                         "kernel": kernel_name, "algorithmic_bytes_per_launch": alg_bytes,
                         "kernel_ms": kern_ms},
            "cpu_baseline": cpu,
            "e2e": {"value": e2e_val, "unit": "tokens/s", "h2d_bytes_per_step": bytes_dir * world,
                    "d2h_bytes_per_step": bytes_dir * world, "steps": e2e_steps,
                    "note": ("the whole per-rank batch lives in pinned host memory (input and output); slices of %d "
                             "sequences stream H2D -> kernel -> D2H on 3 streams" % sl) if whole_host_batch else
                            ("host could not pin the whole batch: one pinned slice of %d sequences is sent and "
                             "received %d times per step (same bytes over PCIe)" % (sl, nsl))},
            "gpu_launches": int(launches),
            "clocks": clocks,
            "verify": verify,
            "aux": aux,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def aux_workload(workload, steps, warm):
    """One side workload (configs 0, 1, 2, the decode loop, the complex layer, a training step, the
    two-output form): CUDA-event timing of the module calls on GPU 0; returns the JSON line as a dict."""
    import torch
    import fairseq_apollo_b200 as M
    from fairseq_apollo_b200 import _lib
    args = argparse.Namespace(workload=workload)
    dev = torch.device("cuda", torch.cuda.current_device())
    gen = torch.Generator().manual_seed(1234)
    peak, peak_kind = hbm_peak()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def timed(fn, steps, warm):
        for _ in range(warm):
            fn()
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(2 * steps)]
        for i in range(steps):
            flush.zero_()
            ev[2 * i].record()
            fn()
            ev[2 * i + 1].record()
        torch.cuda.synchronize()
        ts = sorted(ev[2 * i].elapsed_time(ev[2 * i + 1]) for i in range(steps))
        return ts[len(ts) // 2]

    steps, warm = max(steps, 5), max(warm, 3)
    l0 = M.launch_count()
    kernel = None
    if args.workload == "train":
        # forward + backward of TimestepNorm -> EMA on the config-1 shape through the modules' autograd
        # Functions; compulsory traffic: x read twice, y written, dy read, dx written = 5 passes
        L, B, D = 4096, 16, 1024
        ema = M.MultiHeadEMA(D, ndim=NDIM).to(dev).train()
        norm = M.TimestepNorm(D, prior_count=2).to(dev).train()
        x = torch.randn(B, L, D, generator=gen).to(dev).bfloat16().requires_grad_(True)
        dy = torch.randn(B, L, D, generator=gen).to(dev).bfloat16()

        def train_step():
            for prm in list(ema.parameters()) + list(norm.parameters()) + [x]:
                prm.grad = None
            M.timestep_norm_ema(norm, ema, x).backward(dy)
        ms = timed(train_step, steps, warm)
        tokens, bytes_alg, name, dt = B * L, 5.0 * B * L * D * 2, "train: TimestepNorm+MultiHeadEMA fwd+bwd bf16 L=4096 B=16 D=1024", "bf16"
    with torch.no_grad():
        if args.workload == "train":
            pass
        elif args.workload == "cema":
            # the reference's default moving layer on the config-4 shape at B=16: fused TimestepNorm -> complex EMA
            L, B, D = 32768, 16, 2048
            x = torch.empty(B, L, D, dtype=torch.bfloat16, device=dev)
            for b in range(B):
                x[b] = torch.randn(L, D, device=dev, dtype=torch.bfloat16)
            ema = M.MultiHeadComplexEMA(D, ndim=NDIM).to(dev).eval()
            norm = M.TimestepNorm(D, prior_count=2).to(dev).eval()
            ms = timed(lambda: M.timestep_norm_ema(norm, ema, x), steps, warm)
            tokens, bytes_alg, name, dt = B * L, 2.0 * B * L * D * 2, "cema: TimestepNorm+MultiHeadComplexEMA causal fwd bf16 L=32768 B=16 D=2048", "bf16"
        elif args.workload == "c3":
            # BASELINE config 3: one Mega decoder block (this package's MovingAverageGatedAttention on the fused
            # kernels, projections on cuBLAS) + the normalised feed-forward network, bf16, random init;
            # token ids uniform over a 32k vocabulary into a random embedding scaled by sqrt(D)
            L, B, D, Z, H, FF, C = 8192, 8, 1024, 256, 2048, 2048, 1024
            emb = (torch.randn(32000, D, generator=gen) * D ** -0.5).to(dev).bfloat16()
            ids = torch.randint(0, 32000, (B, L), generator=gen).to(dev)
            x = (emb[ids] * math.sqrt(D)).contiguous()
            blk = M.MovingAverageGatedAttention(D, Z, H, NDIM, chunk_size=C, moving_layer='ema', moving_act='silu',
                                                rel_pos_bias='rotary', efficient_attn=True).to(dev).bfloat16().eval()
            ln = torch.nn.LayerNorm(D).to(dev).bfloat16()
            fc1, fc2 = torch.nn.Linear(D, FF).to(dev).bfloat16(), torch.nn.Linear(FF, D, bias=False).to(dev).bfloat16()

            def layer():
                h = blk(x)[0]
                return h + fc2(torch.nn.functional.silu(fc1(ln(h))))
            ms = timed(layer, steps, warm)
            ms_ema = timed(lambda: M.timestep_norm_ema(blk.norm, blk.move, x, None, None, 'silu', return_normed=True),
                           steps, warm)
            ms_blk = timed(lambda: blk(x), steps, warm)
            extra = {"ms_layer": ms, "ms_block": ms_blk, "ms_fused_norm_ema_part": ms_ema,
                     "share_of_layer_in_fused_norm_ema": ms_ema / ms,
                     "note": "projections, attention GEMMs and the feed-forward network are cuBLAS (library GEMMs); "
                             "the norm -> EMA -> SiLU, the gates and the attention softmax are this library's kernels"}
            # compulsory traffic of the norm -> EMA part only (x in, mx and xn out); the layer as a whole is GEMM-bound
            tokens, bytes_alg, dt = B * L, 3.0 * B * L * D * 2 * (ms / ms_ema), "bf16"
            name = "c3: Mega decoder block + NFFN fwd bf16 L=8192 B=8 D=1024 z=256 h=2048 ffn=2048 chunk=1024"
        elif args.workload == "c4pad":
            # config 4's shape with right padding of 0-25 % per sequence (padded batches are the reference's normal case)
            L, B, D = 32768, 64, 2048
            x = torch.empty(B, L, D, dtype=torch.bfloat16, device=dev)
            for b in range(B):
                x[b] = torch.randn(L, D, device=dev, dtype=torch.bfloat16)
            mask = torch.zeros(B, L, dtype=torch.bool)
            for b in range(B):
                n = int(torch.rand((), generator=gen).item() * 0.25 * L)
                if n:
                    mask[b, L - n:] = True
            mask = mask.to(dev)
            ema = M.MultiHeadEMA(D, ndim=NDIM).to(dev).eval()
            norm = M.TimestepNorm(D, prior_count=2).to(dev).eval()
            ms = timed(lambda: M.timestep_norm_ema(norm, ema, x, mask), steps, warm)
            tokens, bytes_alg, dt = B * L, 2.0 * B * L * D * 2, "bf16"
            name = "c4pad: TimestepNorm+MultiHeadEMA causal fwd bf16 L=32768 B=64 D=2048, 0-25% right padding"
        elif args.workload == "c1":
            L, B, D = 4096, 16, 1024
            x = torch.randn(B, L, D, generator=gen).to(dev).bfloat16()
            ema = M.MultiHeadEMA(D, ndim=NDIM).to(dev).eval()
            norm = M.TimestepNorm(D, prior_count=2).to(dev).eval()
            ms = timed(lambda: M.timestep_norm_ema(norm, ema, x), steps, warm)
            tokens, bytes_alg, name, dt = B * L, 2.0 * B * L * D * 2, "c1: TimestepNorm+MultiHeadEMA causal fwd bf16 L=4096 B=16 D=1024", "bf16"
        elif args.workload in ("c4n", "c1n"):
            # configs 4 and 1 as the Mega block calls the pair: the normalised activations are a second
            # output (they feed the value projection), so the compulsory traffic is 3 x D x 2 B per token
            L, B, D = (32768, 64, 2048) if args.workload == "c4n" else (4096, 16, 1024)
            x = torch.empty(B, L, D, dtype=torch.bfloat16, device=dev)
            for b in range(B):
                x[b] = torch.randn(L, D, device=dev, dtype=torch.bfloat16)
            ema = M.MultiHeadEMA(D, ndim=NDIM).to(dev).eval()
            norm = M.TimestepNorm(D, prior_count=2).to(dev).eval()
            ms = timed(lambda: M.timestep_norm_ema(norm, ema, x, None, None, 'silu', return_normed=True), steps, warm)
            tokens, bytes_alg, dt = B * L, 3.0 * B * L * D * 2, "bf16"
            name = "%s: TimestepNorm+MultiHeadEMA(+SiLU) fwd returning the normalised activations too, bf16 L=%d B=%d D=%d" % (
                args.workload, L, B, D)
        elif args.workload == "c0":
            L, B, D = 1024, 8, 512
            x = torch.randn(L, B, D, generator=gen).to(dev)           # time-major, viewed as (B, D, L)
            ema = M.MultiHeadEMA(D, ndim=NDIM).to(dev).eval()
            mask = torch.zeros(B, L, dtype=torch.bool)
            for b in range(B):
                n = int(torch.rand((), generator=gen).item() * 0.25 * L)
                if n:
                    mask[b, L - n:] = True
            mask = mask.to(dev)
            ms = timed(lambda: ema.forward_time_major(x, mask), steps, warm)
            tokens, bytes_alg, name, dt = B * L, 2.0 * B * L * D * 4, "c0: MultiHeadEMA fwd fp32 L=1024 B=8 D=512, 0-25% padding", "f32"
        elif args.workload == "c2":
            L, B, D = 16384, 32, 256
            x = torch.randn(B, D, L, generator=gen).to(dev)
            ema = M.MultiHeadEMA(D, ndim=NDIM, bidirectional=True).to(dev).eval()
            norm = M.SequenceNorm(D).to(dev).eval()
            mask = torch.zeros(B, L, dtype=torch.bool)
            for b in range(B):
                n = int(torch.rand((), generator=gen).item() * 0.5 * L)
                if n:
                    mask[b, L - n:] = True
            mask = mask.to(dev)
            ms = timed(lambda: M.sequence_norm_ema(norm, ema, x, mask), steps, warm)
            tokens, bytes_alg, name, dt = B * L, 2.0 * B * L * D * 4, "c2: SequenceNorm + bidirectional MultiHeadEMA fwd fp32 L=16384 B=32 D=256, 0-50% padding", "f32"
        else:  # decode: 1024 single-token steps, state seeded from a 4096-token prefix
            B, D, T = 64, 2048, 1024
            ema = M.MultiHeadEMA(D, ndim=NDIM).to(dev).eval()
            norm = M.TimestepNorm(D, prior_count=2).to(dev).eval()
            st = {}
            M.timestep_norm_ema(norm, ema, torch.randn(B, 4096, D, generator=gen).to(dev).bfloat16(), None, st)
            xs = torch.randn(T, B, 1, D, generator=gen).to(dev).bfloat16()

            def loop():
                for t in range(T):
                    M.timestep_norm_ema(norm, ema, xs[t], None, st)
            ms_module = timed(loop, 3, 1) / T
            # the same step captured once in a CUDA graph and replayed (device-side cost of a step)
            sx = xs[0].clone()
            torch.cuda.synchronize()
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr):
                M.timestep_norm_ema(norm, ema, sx, None, st)

            def replay():
                for _ in range(T):
                    gr.replay()
            kernel = _lib.last_kernel()
            ms = timed(replay, 3, 1) / T
            extra = {"module_call_us_per_step": ms_module * 1e3, "graph_replay_us_per_step": ms * 1e3}
            tokens, bytes_alg, name, dt = B, 2.0 * B * D * NDIM * 4 + 2.0 * B * D * 2, "decode: TimestepNorm+EMA single-token step, B=64 D=2048 ndim=16, state fp32", "bf16"
    launches = M.launch_count() - l0
    if args.workload not in ("decode", "c3"):
        extra = None
    if args.workload != "decode":
        kernel = _lib.last_kernel()
    torch.cuda.synchronize()
    del flush
    line = {"extra": extra, "kernel": kernel, "metric": "mega_ema_layer_tokens_per_s", "value": tokens / (ms * 1e-3), "unit": "tokens/s", "n_gpus": 1,
            "steps": steps, "warmup": warm, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": dt, "data": "synthetic",
            "config": {"workload": name, "ndim": NDIM, "l2": "256 MiB scratch written between timed calls"},
            "roofline": {"bound": "hbm", "achieved": bytes_alg / (ms * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                         "frac": bytes_alg / (ms * 1e-3) / 1e9 / peak, "traffic": None, "peak_kind": peak_kind},
            "gpu_launches": int(launches)}
    return line


def run_aux(args):
    import torch
    torch.cuda.set_device(0)
    print(json.dumps(aux_workload(args.workload, args.steps, args.warmup)), flush=True)


def aux_summary(steps, warm):
    """The side workloads, measured in this process after the headline run: one entry each with the
    time per step, tokens/s, the fraction of the HBM peak (algorithmic bytes) and the kernel family
    that ran.  A workload that fails is reported with its error, not dropped."""
    import gc
    import torch
    out = {}
    for w in AUX_IN_HEADLINE:
        try:
            r = aux_workload(w, steps, warm)
            out[w] = {"ms": r["ms_per_step"], "tokens_per_s": r["value"], "roofline_frac": r["roofline"]["frac"],
                      "achieved_gbs": r["roofline"]["achieved"], "kernel": r.get("kernel"),
                      "workload": r["config"]["workload"]}
            if r.get("extra"):
                out[w].update(r["extra"])
        except Exception as exc:  # noqa: BLE001 - reported in the line
            out[w] = {"error": str(exc).splitlines()[0][:200]}
        gc.collect()
        torch.cuda.empty_cache()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c4", choices=sorted(WORKLOADS) + list(AUX_WORKLOADS))
    ap.add_argument("--scaling", default="strong", choices=["weak", "strong"],
                    help="strong (default): the workload's batch is sharded over the ranks, as BASELINE config 4 "
                         "defines the multi-GPU run (B=64 -> 32/16/8 per GPU); weak: every rank runs the full batch")
    ap.add_argument("--no-aux", action="store_true", help="skip the side workloads reported under 'aux'")
    ap.add_argument("--batch", type=int, default=0, help="override the per-rank batch")
    ap.add_argument("--length", type=int, default=0, help="override the sequence length (profiling aid)")
    ap.add_argument("--e2e-slice", type=int, default=8)
    ap.add_argument("--e2e-steps", type=int, default=3)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--tile", type=int, default=0, help="force a tensor-core tile form (tuning aid; 0 = automatic)")
    args = ap.parse_args()
    if args.workload in AUX_WORKLOADS:
        return run_aux(args)
    B, L, D, dtype_name = WORKLOADS[args.workload]
    if args.batch:
        B = args.batch
    if args.length:
        L = args.length
    if args.impl == "reference":
        run_reference(args, B, L, D, dtype_name)
    else:
        run_ours(args, B, L, D, dtype_name)


if __name__ == "__main__":
    main()
