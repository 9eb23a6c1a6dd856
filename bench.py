#!/usr/bin/env python3
"""Benchmark of the sparse-attention forward hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

Workload (``config.workload``): the long-sequence causal sliding-window case,
B=1, N=65536, H=8, d_head=64, 64 taps, bf16, Q/K/V ~ N(0,1)*0.5 from a seed
(synthetic: the reference benchmarks on torch.randn as well).  One step is one
forward over the whole sequence.  With N GPUs the sequence is cut into N
contiguous chunks (strong scaling); the edge tiles of every chunk read the 63
K/V rows they need from the neighbouring GPU inside the kernel (``--halo nccl``
exchanges them by send/recv instead).  Steps are independent forwards over
rotating input sets; they are captured in CUDA graphs and alternate over two
streams (``--lanes``), each with its own output buffer.
``--workload block|longformer|orderbook|dense|backward|fp32|refwindow`` time the other configurations on one GPU
(refwindow: the reference's default window_size = 64, i.e. keys i-64 .. i+64, at the headline shape; with
``--head-dim`` and ``--dtype fp32`` it and ``backward`` run other head widths and the reference's own precision);
each forward workload compares sampled row blocks of its last timed launch with the CPU oracle after the timed region.

Prints ONE JSON line.  ``value`` is tokens/s with inputs resident in HBM, timed
with CUDA events over exactly K steps (max over ranks); ``e2e`` is the same
metric through the host-buffer entry point with pinned host tensors, copies
inside the timed region; ``roofline`` relates the kernel's algorithmic bytes
(read Q, K, V once, write O once = 4096 B per token) to measured HBM bandwidth;
``cpu_baseline`` times the CPU oracle (a port of the reference's C++ path) on
this box's host cores.  ``--impl reference`` times the reference's own compiled
CPU engine instead.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

B, SEQ, H, D, TAPS = 1, 65536, 8, 64, 64
SEED = 2
WORKLOAD = f"causal sliding-window fwd B={B} N={SEQ} H={H} d={D} taps={TAPS} bf16"
BYTES_PER_TOKEN = 4 * H * D * 2          # read Q,K,V + write O, bf16
METRIC = "sparse-attn fwd tokens/s @N=64K,w=64,bf16"
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of each window kernel on this
# workload, from ncu captures of those launches, per token
NCU_TRAFFIC_PER_TOKEN = {"umma_band": (201.378e6 + 41.432e6) / 65536, "mma_window": (201.354e6 + 49.839e6) / 65536}


def measured_peak_gbs():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


def measured_peak_tflops():
    """Dense bf16 GEMM throughput of this pool's GPUs (the burst figure: the kernel is timed alone)."""
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["bf16_tflops"]), "measured"
        except Exception:
            pass
    return 1590.0, "fallback"


# ---- clocks during the timed region ------------------------------------------------

class ClockSampler:
    """Polls SM clock and throttle reasons of one GPU through NVML from a thread."""

    def __init__(self, index: int, period_s: float = 0.0002):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
            self._period = period_s
        except Exception:
            self._nv = None

    def _loop(self):
        nv = self._nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4),
        }
        while not self._stop.is_set():
            try:
                self.samples.append((time.perf_counter(), nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM)))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
                for k, bit in names.items():
                    if mask & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            time.sleep(self._period)

    def start(self):
        if self._nv is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()

    def count_between(self, t0, t1):
        return sum(1 for (t, _) in list(self.samples) if t0 <= t <= t1)

    def stop(self, t0=None, t1=None):
        if self._thread is not None:
            self._stop.set()
            self._thread.join()
        inside = [m for (t, m) in self.samples if t0 is None or (t0 <= t <= t1)]
        use = inside or [m for (_, m) in self.samples]
        med = sorted(use)[len(use) // 2] if use else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples_in_timed_region": len(inside)}


# ---- CPU arms -------------------------------------------------------------------------

def make_inputs_cpu(n_tokens: int):
    import torch
    g = torch.Generator().manual_seed(SEED)
    mk = lambda: (torch.randn(B, n_tokens, H, D, generator=g) * 0.5).to(torch.bfloat16)
    return mk(), mk(), mk()


def cpu_baseline_port(budget_s: float = 20.0):
    """The oracle (C port of ma_core.cpp:160-246, OpenMP over rows) on all host cores."""
    from oracle import oracle as O
    n = SEQ
    q, k, v = (t.float().numpy() for t in make_inputs_cpu(n))
    pat = O.OraclePattern.causal_taps(TAPS)
    O.sparse_attention(q[:, :1024], k[:, :1024], v[:, :1024], pat)  # warm the thread pool
    t0 = time.perf_counter()
    passes = 0
    while True:
        O.sparse_attention(q, k, v, pat)
        passes += 1
        dt = time.perf_counter() - t0
        if dt > 3.0 or passes >= 5 or dt * (passes + 1) / passes > budget_s:
            break
    return {"value": B * n * passes / dt, "unit": "tokens/s", "cores": O.num_threads(), "kind": "port",
            "sample": f"full workload ({n} tokens x {H} heads), {passes} pass(es), fp32 upcast of the bf16 inputs"}


def _ref_worker(args):
    a, b, half = args
    import numpy as np
    from oracle import oracle as O
    m = O.reference_module()
    lo, hi = max(0, a - half), min(_REF_IN[0].shape[1], b + half)
    ts = []
    for x in _REF_IN:
        sl = np.ascontiguousarray(x[:, lo:hi])
        t = m.create_tensor(list(sl.shape))
        t.copy_from_numpy(sl)
        ts.append(t)
    out = np.asarray(m.compute_sparse_attention(ts[0], ts[1], ts[2], half).to_numpy())
    return float(out[:, a - lo:b - lo].sum())


_REF_IN = None


def reference_arm(steps: int, warmup: int):
    """The reference's own compiled CPU engine (oracle/_ref, module ma_core) on the
    host cores.  It is single-threaded and only knows the two-sided window
    [i-w, i+w], so it runs w=32 (65 keys per row, the work of 64 causal taps) on a
    prefix of the sequence, cut into row chunks (each with its 32-row halo) that a
    process pool spreads over every core."""
    global _REF_IN
    import multiprocessing as mp
    from oracle import oracle as O
    cores = os.cpu_count() or 1
    half = TAPS // 2
    kind = "reference" if O.reference_module() is not None else "port"
    if kind == "port":
        r = cpu_baseline_port()
        ms = B * SEQ / r["value"] * 1e3
        return r["value"], ms, r
    # calibrate on one small chunk, then size the per-step sample to a few seconds
    n_cal = 512
    _REF_IN = tuple(t.float().numpy() for t in make_inputs_cpu(SEQ))
    t0 = time.perf_counter()
    _ref_worker((0, n_cal, half))
    per_tok = (time.perf_counter() - t0) / n_cal
    target_s = max(0.5, min(4.0, 150.0 / max(1, steps + warmup)))
    n_sample = int(min(SEQ, max(cores * 256, target_s * cores / per_tok)))
    n_sample -= n_sample % cores
    per = max(1, n_sample // cores)
    tasks = [(a, min(n_sample, a + per), half) for a in range(0, n_sample, per)]
    ctx = mp.get_context("fork")
    with ctx.Pool(cores) as pool:
        for _ in range(warmup):
            pool.map(_ref_worker, tasks)
        t0 = time.perf_counter()
        for _ in range(steps):
            pool.map(_ref_worker, tasks)
        dt = time.perf_counter() - t0
    val = B * n_sample * steps / dt
    info = {"value": val, "unit": "tokens/s", "cores": cores, "kind": "reference",
            "sample": f"first {n_sample} of {SEQ} tokens x {H} heads per step, fp32, reference window +-{half} "
                      f"(65 keys/row; the engine has no causal mode), {len(tasks)} row chunks over {cores} processes"}
    return val, dt / steps * 1e3, info


# ---- GPU arm --------------------------------------------------------------------------

def gpu_arm(args):
    import torch
    import torch.distributed as dist
    from ma_transformer_b200 import _native as nat
    from ma_transformer_b200 import sparse_attention_cuda as ext
    from ma_transformer_b200.patterns import PatternSpec
    from ma_transformer_b200.sharded import PeerHaloAttention, SequenceShardedAttention

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch multi-GPU runs with torch.distributed.run (one rank per GPU)")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a GPU: the library has no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    spec = PatternSpec.causal_window(TAPS)
    rows = SEQ // world
    q_cpu, k_cpu, v_cpu = make_inputs_cpu(SEQ)
    a, b = rank * rows, (rank + 1) * rows

    # Rotating input sets so that consecutive steps never find their inputs in L2.
    per_rank_bytes = rows * BYTES_PER_TOKEN
    n_sets = max(2, -(-(2 * 126 * 2 ** 20) // per_rank_bytes) + 1)
    sets = []
    sharded = peer = None
    if world == 1:
        for s in range(n_sets):
            sets.append(tuple(t.to(dev).roll(s, dims=1).contiguous() for t in (q_cpu, k_cpu, v_cpu)))
    elif args.halo == "nccl":
        # halo rows exchanged by send/recv into an extended K/V buffer before the edge tiles run
        sharded = SequenceShardedAttention(spec, SEQ)
        for s in range(n_sets):
            q = q_cpu[:, a:b].to(dev).roll(s, dims=1).contiguous()
            k_ext = sharded.alloc_kv(B, H, D, torch.bfloat16, dev)
            v_ext = sharded.alloc_kv(B, H, D, torch.bfloat16, dev)
            sharded.chunk_view(k_ext).copy_(k_cpu[:, a:b].to(dev).roll(s, dims=1))
            sharded.chunk_view(v_ext).copy_(v_cpu[:, a:b].to(dev).roll(s, dims=1))
            sets.append((q, k_ext, v_ext))
    else:
        # each rank holds only its chunk; edge tiles read the neighbour's rows in place over NVLink
        peer = PeerHaloAttention(spec, SEQ)
        for s in range(n_sets):
            q, k, v = (t[:, a:b].to(dev).roll(s, dims=1).contiguous() for t in (q_cpu, k_cpu, v_cpu))
            sets.append((q, peer.register(k, v)))
    # one output buffer per lane: steps are independent forwards, and two lanes (streams) let
    # the tail of one step overlap the head of the next, as concurrent requests would
    n_lanes = max(1, args.lanes)
    outs = [torch.empty(B, rows, H, D, dtype=torch.bfloat16, device=dev) for _ in range(n_lanes)]
    out = outs[0]
    launches = [0]

    def step(i, out=out):
        if sharded is not None:
            q, k, v = sets[i % n_sets]
            sharded.forward(q, k, v, out=out)
            front, back = sharded.edge_rows()
            return 1 + (1 if front else 0) + (1 if back else 0)
        if peer is not None:
            q, shard = sets[i % n_sets]
            peer.forward(q, shard, out=out)
        else:
            q, k, v = sets[i % n_sets]
            ext.forward_pattern(q, k, v, spec, out=out)
        return 1

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # the clock sampler runs from before the warm-up (its first NVML calls take milliseconds);
    # only the samples that fall inside the timed region are used
    sampler = ClockSampler(local)
    sampler.start()
    for i in range(args.warmup):
        step(i)
    barrier()

    # Launch-bound at 8 GPUs (a shard's forward is a few microseconds): the steps are captured in
    # CUDA graphs: one graph of about 24 steps (whole passes over the input sets), replayed, plus
    # one graph with the K mod 24 steps left over, so exactly K steps run.
    use_graph = args.graph and sharded is None
    if use_graph:
        # steps per captured round: whole passes over the input sets, about 24 steps, never more than K
        round_len = n_sets * max(1, min(-(-24 // n_sets), args.steps // n_sets))
        side = torch.cuda.Stream()
        lanes = [side] + [torch.cuda.Stream() for _ in range(n_lanes - 1)]
        side.wait_stream(torch.cuda.current_stream())
        rounds, rest = divmod(args.steps, round_len)

        def capture(n_steps):
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                for ln in lanes[1:]:
                    ln.wait_stream(side)            # fork
                for s in range(n_steps):
                    with torch.cuda.stream(lanes[s % n_lanes]):
                        step(s, outs[s % n_lanes])
                for ln in lanes[1:]:
                    side.wait_stream(ln)            # join
            return graph

        with torch.cuda.stream(side):
            round_graph = capture(round_len)
            rest_graph = capture(rest) if rest else None   # the K mod round_len steps left over
        torch.cuda.current_stream().wait_stream(side)
        round_graph.replay()      # one untimed round warms the instantiated graphs
        barrier()

    # the timed region can be a few milliseconds: let the sampling thread in more often than the
    # interpreter's default 5 ms switch interval
    switch_interval = sys.getswitchinterval()
    sys.setswitchinterval(1e-4)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t_host0 = time.perf_counter()
    ev0.record()
    if use_graph:
        rounds, rest = divmod(args.steps, round_len)
        for _ in range(rounds):
            round_graph.replay()
        if rest_graph is not None:
            rest_graph.replay()
        launches[0] = args.steps
    else:
        for i in range(args.steps):
            launches[0] += step(args.warmup + i)
    ev1.record()
    while not ev1.query():      # wait in the interpreter, not inside a blocking call, so that the
        time.sleep(0)           # clock-sampling thread runs while the timed steps execute
    t_host1 = time.perf_counter()
    barrier()
    # If the timed region was still too short for the sampler, keep the identical load running
    # (untimed) until it has three samples, at most 50 ms, so that clocks and throttle reasons are
    # read under the load that was timed.
    extended = False
    # (only where a step holds no collective: every rank decides this for itself)
    if (use_graph or world == 1) and sampler.count_between(t_host0, t_host1) < 3:
        extended = True
        t_end = time.perf_counter() + 0.05
        i = 0
        while time.perf_counter() < t_end and sampler.count_between(t_host0, time.perf_counter()) < 3:
            if use_graph:
                round_graph.replay()
            else:
                step(args.warmup + args.steps + i)
                i += 1
            torch.cuda.synchronize()     # one round at a time: nothing queues up behind the check
        torch.cuda.synchronize()
        t_host1 = time.perf_counter()
    clocks = sampler.stop(t_host0, t_host1)
    sys.setswitchinterval(switch_interval)
    if extended:
        clocks["sampled"] = "timed steps plus up to 50 ms of the same steps continued untimed (the timed region was shorter than the sampler's reach)"
    ms = torch.tensor([ev0.elapsed_time(ev1)], device=dev)
    n_launch = torch.tensor([launches[0]], device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        dist.all_reduce(n_launch, op=dist.ReduceOp.SUM)
    ms_total = float(ms.item())
    ms_per_step = ms_total / args.steps
    value = B * SEQ / (ms_per_step * 1e-3)
    status = nat.device_status()
    kernel_name = nat.last_kernel()     # the device leg's kernel (the chunked end-to-end leg below may pick another)

    # ---- after the timed region: this rank's first and last 128 output rows (the first ones need the
    # previous shard's halo rows) of one more forward over input set 0 against the CPU oracle ----
    import numpy as np
    from oracle import oracle as O
    step(0, out)
    torch.cuda.synchronize()
    worst = 0.0
    for lo_row in (a, (a + b) // 2, b - 128):
        k_lo = max(0, lo_row - (TAPS - 1))
        pat = O.OraclePattern.causal_taps(TAPS)
        pat.q_offset = lo_row - k_lo
        want = O.sparse_attention(q_cpu[:, lo_row:lo_row + 128].float().numpy(), k_cpu[:, k_lo:lo_row + 128].float().numpy(),
                                  v_cpu[:, k_lo:lo_row + 128].float().numpy(), pat)
        got = out[:, lo_row - a:lo_row - a + 128].float().cpu().numpy()
        worst = max(worst, float(np.abs(got - want).max()))
    worst_t = torch.tensor([worst], device=dev)
    if world > 1:
        dist.all_reduce(worst_t, op=dist.ReduceOp.MAX)
    worst = float(worst_t.item())
    if not worst <= 2e-2:
        raise SystemExit(f"parity check after the timed region failed: max-abs {worst} > 2e-2")
    parity = {"rows_checked": 3 * 128 * world, "max_abs_vs_oracle": worst, "tolerance": 2e-2, "ok": True}

    # ---- end to end: pinned host tensors in, host tensor out, per rank its chunk plus halo ----
    if args.no_e2e:   # profiling runs: the device-resident leg only
        if rank == 0:
            print(json.dumps({"metric": METRIC, "value": value, "ms_per_step": ms_per_step, "n_gpus": world,
                              "clocks": clocks, "note": "device leg only (--no-e2e)"}), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return
    lo = max(0, a - (TAPS - 1))
    hq, hk, hv = (t[:, lo:b].contiguous().pin_memory() for t in (q_cpu, k_cpu, v_cpu))
    ho = torch.empty_like(hq).pin_memory()
    e2e_steps = max(3, min(args.steps, 20))
    for _ in range(2):
        ext.forward_host(hq, hk, hv, spec, device=local, out=ho)
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        ext.forward_host(hq, hk, hv, spec, device=local, out=ho)
    torch.cuda.synchronize()
    e2e_s = torch.tensor([time.perf_counter() - t0], device=dev)
    if world > 1:
        dist.all_reduce(e2e_s, op=dist.ReduceOp.MAX)
    e2e_val = B * SEQ * e2e_steps / float(e2e_s.item())
    h2d = 3 * hq.numel() * 2 * world
    d2h = ho.numel() * 2 * world

    if rank == 0:
        peak, peak_kind = measured_peak_gbs()
        achieved = per_rank_bytes / (ms_per_step * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": WORKLOAD, "sharding": (f"sequence x{world}, {TAPS - 1}-row K/V halo, " + ("read in place from the neighbour GPU by the kernel" if peer is not None else "64 rows exchanged by NCCL send/recv")) if world > 1 else "none",
                       "launch": f"CUDA graphs, steps alternate over {n_lanes} streams" if use_graph else "one host launch per kernel",
                       "l2": f"{n_sets} rotating input sets of {per_rank_bytes >> 20} MiB per GPU (> 126 MB L2 between reuses)"},
            "clocks": clocks,
            "e2e": {"value": e2e_val, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "steps": e2e_steps, "api": "sparse_attention_cuda.forward_host (mat_sparse_attn_fwd_host)"},
            "gpu_launches": int(n_launch.item()),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": NCU_TRAFFIC_PER_TOKEN.get(kernel_name, NCU_TRAFFIC_PER_TOKEN["umma_band"]) * rows,
                         "peak_source": f"{peak_kind} HBM copy bandwidth",
                         "kernel": kernel_name, "bytes_per_launch_algorithmic": per_rank_bytes},
            "parity_check": parity, "device_status": status,
        }
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline_port()
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def sampled_parity(out, q, k, v, spec, starts, rows=128, tol=2e-2):
    """After the timed region: a few blocks of output rows of the LAST timed launch against the CPU oracle
    (the checker, never the thing measured).  q, k, v, out: device tensors [B, S, H, 64]; each block of
    ``rows`` query rows runs against the whole key axis of its batch item, so window, block layout, global
    keys and rows at global positions are all covered.  Raises if a block is off by more than ``tol``."""
    import numpy as np
    from oracle import oracle as O
    kinds = {0: O.WINDOW, 1: O.BLOCK, 2: O.LONGFORMER}
    worst, n, scale_ref = 0.0, 0, 0.0
    for b, a in starts:
        a = max(0, min(a, q.shape[1] - rows))
        pat = O.OraclePattern(kind=kinds[spec.kind], left=spec.left, right=spec.right, dilation=spec.dilation,
                              causal=spec.causal, block=spec.block, blk_rowptr=spec.blk_rowptr,
                              blk_colidx=spec.blk_colidx, global_idx=spec.global_idx, q_offset=a)
        want = O.sparse_attention(q[b:b + 1, a:a + rows].float().cpu().numpy(), k[b:b + 1].float().cpu().numpy(),
                                  v[b:b + 1].float().cpu().numpy(), pat)
        got = out[b:b + 1, a:a + rows].float().cpu().numpy()
        worst = max(worst, float(np.abs(got - want).max()))
        scale_ref = max(scale_ref, float(np.abs(want).max()))
        n += rows
    if tol is None:     # fp32: max|gpu - oracle| / max|oracle| <= 1e-5
        rel = worst / max(scale_ref, 1e-30)
        if not rel <= 1e-5:
            raise SystemExit(f"parity check after the timed region failed: fp32 rel-err {rel} > 1e-5")
        return {"rows_checked": n, "rel_err_vs_oracle": rel, "tolerance": 1e-5, "ok": True}
    if not worst <= tol:
        raise SystemExit(f"parity check after the timed region failed: max-abs {worst} > {tol}")
    return {"rows_checked": n, "max_abs_vs_oracle": worst, "tolerance": tol, "ok": True}


def other_workload_arm(args):
    """Device-resident timing of the block-sparse (cfg-3) and Longformer (cfg-4) configurations on
    one GPU: same timing rules as the headline arm (events, warm-up, rotating input sets), one JSON
    line with the HBM roofline of the algorithmic bytes and the executed tensor-core FLOP rate."""
    import numpy as np
    import torch
    from ma_transformer_b200 import _native as nat
    from ma_transformer_b200 import sparse_attention_cuda as ext
    from ma_transformer_b200.patterns import PatternSpec, band_random_block_layout

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    g = torch.Generator().manual_seed(SEED)
    if args.workload == "orderbook":
        # cfg-5: the whole order-book transformer forward (library GEMMs around the native attention)
        from ma_transformer_b200.layers.orderbook_model import OrderBookTransformer, synthetic_ticks
        Bw, S = 16, 8192
        torch.manual_seed(SEED)
        model = OrderBookTransformer().eval().to(dev).to(torch.bfloat16)
        ticks = synthetic_ticks(Bw, S, seed=SEED)
        ticks = ((ticks - ticks.mean(dim=(0, 1))) / (ticks.std(dim=(0, 1)) + 1e-6)).to(dev).to(torch.bfloat16)
        qkv = [torch.randn(Bw, S, 4, 64, generator=g).to(torch.bfloat16).to(dev) for _ in range(3)]
        out = torch.empty_like(qkv[0])

        def timed(fn, n):
            for _ in range(args.warmup):
                fn()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(n):
                fn()
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) / n

        with torch.no_grad():
            ms_model = timed(lambda: model(ticks), args.steps)
            ms_attn = timed(lambda: ext.forward_pattern(*qkv, model.pattern, out=out), args.steps)
        torch.cuda.synchronize()
        parity = sampled_parity(out, *qkv, model.pattern, [(0, 0), (Bw - 1, S - 128), (Bw // 2, S // 2 - 64)])
        peak, peak_kind = measured_peak_gbs()
        attn_bytes = 4 * Bw * S * 4 * 64 * 2
        print(json.dumps({
            "metric": "order-book transformer fwd tokens/s (orderbook)", "value": Bw * S / (ms_model * 1e-3),
            "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_model,
            "higher_is_better": True, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"ticks [{Bw},{S},40] -> Linear(40,256) -> 4 pre-LN blocks (4 heads x 64, "
                                   "64 causal taps dilation 2, GELU FFN 1024) -> Linear(256,3), random-init weights"},
            "attention": {"ms_per_layer": ms_attn, "share_of_forward": 4 * ms_attn / ms_model, "kernel": nat.last_kernel(),
                          "roofline": {"bound": "hbm", "achieved": attn_bytes / (ms_attn * 1e-3) / 1e9, "peak": peak,
                                       "unit": "GB/s", "frac": attn_bytes / (ms_attn * 1e-3) / 1e9 / peak,
                                       "peak_source": f"{peak_kind} HBM copy bandwidth"}},
            "parity_check": parity, "device_status": nat.device_status()}), flush=True)
        return
    if args.workload == "fp32":
        # the reference's own precision: the small configuration that also runs on the reference's CPU engine
        # (B=1, H=4, N=1024, d=64, 32 causal taps) and the long-sequence shape in fp32 (N=65536, H=8, 64 taps)
        peak, peak_kind = measured_peak_gbs()
        lines = []
        for tag, Bw, S, Hw, taps, n_sets in (("cfg-1", 1, 1024, 4, 32, 64), ("64K", 1, 65536, 8, 64, 2)):
            spec = PatternSpec.causal_window(taps)
            nbytes = 4 * Bw * S * Hw * 64 * 4
            sets = [tuple(torch.randn(Bw, S, Hw, 64, generator=g).to(dev) for _ in range(3)) for _ in range(n_sets)]
            out = torch.empty_like(sets[0][0])
            reps = args.steps * (50 if S <= 4096 else 1)
            for i in range(max(args.warmup, 3)):
                ext.forward_pattern(*sets[i % n_sets], spec, out=out)
            torch.cuda.synchronize()
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ev0.record()
            for i in range(reps):
                ext.forward_pattern(*sets[i % n_sets], spec, out=out)
            ev1.record()
            torch.cuda.synchronize()
            ms = ev0.elapsed_time(ev1) / reps
            last = sets[(reps - 1) % n_sets]
            parity = sampled_parity(out, *last, spec, [(0, 0), (0, S - 128), (0, S // 2)], tol=None)
            achieved = nbytes / (ms * 1e-3) / 1e9
            lines.append({"shape": f"{tag}: B={Bw} N={S} H={Hw} d=64 taps={taps} fp32", "ms_per_step": ms,
                          "tokens_per_s": Bw * S / (ms * 1e-3), "kernel": nat.last_kernel(),
                          "l2": f"{n_sets} rotating input sets of {nbytes >> 20} MiB" +
                                (" (the whole set fits L2: an L2-resident figure)" if n_sets * nbytes < 126e6 else ""),
                          "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                                       "frac": achieved / peak, "peak_source": f"{peak_kind} HBM copy bandwidth",
                                       "bytes_per_launch_algorithmic": nbytes},
                          "parity_check": parity})
        print(json.dumps({"metric": "sparse-attn fwd tokens/s (fp32)", "value": lines[1]["tokens_per_s"], "unit": "tokens/s",
                          "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": lines[1]["ms_per_step"],
                          "higher_is_better": True, "dtype": "f32", "data": "synthetic",
                          "config": {"workload": lines[1]["shape"]}, "shapes": lines,
                          "device_status": nat.device_status()}), flush=True)
        return
    if args.workload == "backward":
        # backward of the headline window (64 causal taps at the cfg-2 shape): dQ, dK, dV from Q, K, V, dO
        # (--head-dim, --dtype: other head widths at the same 512 columns per token, the reference's precision;
        # --left / --right given together with one of them: another window)
        Dw = args.head_dim
        tdt = torch.bfloat16 if args.dtype == "bf16" else torch.float32
        esz = 2 if args.dtype == "bf16" else 4
        Bw, S, Hw = B, SEQ, H * 64 // Dw
        other = Dw != 64 or args.dtype != "bf16"
        spec = PatternSpec(left=args.left, right=args.right) if other and (args.left, args.right) != (64, 64) \
            else PatternSpec.causal_window(TAPS)
        nbytes = 7 * Bw * S * Hw * Dw * esz      # four tensors read once, three written once
        sets = [tuple((torch.randn(Bw, S, Hw, Dw, generator=g) * 0.5).to(tdt).to(dev) for _ in range(4))
                for _ in range(3)]
        for i in range(args.warmup):
            ext.backward_pattern(*sets[i % 3], spec)
        torch.cuda.synchronize()
        sampler = ClockSampler(0)
        sampler.start()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        ev0.record()
        for i in range(args.steps):
            ext.backward_pattern(*sets[i % 3], spec)
        ev1.record()
        torch.cuda.synchronize()
        clocks = sampler.stop(t0, time.perf_counter())
        ms = ev0.elapsed_time(ev1) / args.steps
        peak, peak_kind = measured_peak_gbs()
        achieved = nbytes / (ms * 1e-3) / 1e9
        print(json.dumps({
            "metric": "sparse-attn bwd tokens/s (backward)", "value": Bw * S / (ms * 1e-3), "unit": "tokens/s",
            "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "dtype": "bf16" if args.dtype == "bf16" else "f32", "data": "synthetic",
            "config": {"workload": f"sliding-window bwd B={Bw} N={S} H={Hw} d={Dw} taps -{spec.left}..+{spec.right} {args.dtype}",
                       "l2": "3 rotating input sets"},
            "clocks": clocks, "kernel": nat.last_kernel(),
            "gpu_launches": (2 if nat.last_kernel() == "bwd_window_mma" else 3) * args.steps,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_source": f"{peak_kind} HBM copy bandwidth", "bytes_per_launch_algorithmic": nbytes,
                         # dram bytes of the two passes, from an ncu capture of one backward (headline shape only)
                         "traffic": None if other else 322e6 + 375e6,
                         "note": "per backward (rows pass and cols pass; a dV and a dK pass for fp32 and other head widths)"},
            "device_status": nat.device_status()}), flush=True)
        return
    Dw = 64
    if args.workload == "block":
        Bw, S, Hw = 4, 16384, 8
        rp, ci = band_random_block_layout(S // 64, 4, 2, seed=SEED)
        spec = PatternSpec.block_sparse(64, rp, ci, causal=True)
        flops = Bw * Hw * int(rp[-1]) * 4 * 64 ** 3
        name = f"block-sparse fwd B={Bw} N={S} H={Hw} d=64 block=64 band4+2 random causal bf16"
    elif args.workload == "refwindow":
        # the window every unmodified caller of the reference gets: window_size = 64, keys i-64 .. i+64
        # (src/layers/ma_core_bridge.py:259), at the headline shape; --left / --right / --dilation change it
        # (--head-dim changes the head width at the same bytes per token: H * d stays 512)
        Dw = args.head_dim
        Bw, S, Hw = B, SEQ, H * 64 // Dw
        spec = PatternSpec(left=args.left, right=args.right, dilation=args.dilation)
        flops = Bw * Hw * S * (args.left + args.right + 1) * 4 * Dw
        name = (f"window fwd B={Bw} N={S} H={Hw} d={Dw} taps -{args.left}..+{args.right}"
                + (f" dilation {args.dilation}" if args.dilation > 1 else "") + f" {args.dtype}")
    elif args.workload == "dense":
        # the reference's dense_forward (every query over every key), the tensor-bound end of the path
        Bw, S, Hw = 2, 8192, 8
        spec = PatternSpec(left=S, right=S)
        flops = Bw * Hw * 4 * S * S * 64
        name = f"dense fwd B={Bw} N={S} H={Hw} d=64 bf16"
    else:
        Bw, S, Hw = 2, 32768, 12
        glob = torch.randperm(S, generator=g)[:32].sort().values.numpy()
        spec = PatternSpec.longformer(64, 64, glob)
        flops = Bw * Hw * (S * 129 + 2 * 32 * S) * 4 * 64
        name = f"Longformer fwd B={Bw} N={S} H={Hw} d=64 window +-64, 32 global tokens bf16"
    f32 = args.workload == "refwindow" and args.dtype == "fp32"
    nbytes = 4 * Bw * S * Hw * Dw * (4 if f32 else 2)
    sets = [tuple(torch.randn(Bw, S, Hw, Dw, generator=g).to(torch.float32 if f32 else torch.bfloat16).to(dev)
                  for _ in range(3)) for _ in range(2)]
    out = torch.empty_like(sets[0][0])
    for i in range(args.warmup):
        ext.forward_pattern(*sets[i % 2], spec, out=out)
    torch.cuda.synchronize()
    sampler = ClockSampler(0)
    sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    ev0.record()
    for i in range(args.steps):
        ext.forward_pattern(*sets[i % 2], spec, out=out)
    ev1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop(t0, time.perf_counter())
    ms = ev0.elapsed_time(ev1) / args.steps
    peak, peak_kind = measured_peak_gbs()
    achieved = nbytes / (ms * 1e-3) / 1e9
    # the output of the last timed launch, a few row blocks against the oracle
    last = sets[(args.steps - 1) % 2]
    starts = [(0, 0), (Bw - 1, S - 128), (Bw // 2, S // 2 - 64), (0, S // 4 + 64)]
    if args.workload == "longformer":
        starts += [(0, int(glob[0]) - 64), (Bw - 1, int(glob[-1]) - 64)]      # blocks that hold a global position
    parity = sampled_parity(out, *last, spec, starts, tol=None if f32 else 2e-2)
    if args.workload == "dense":
        tpeak, tkind = measured_peak_tflops()
        tf = flops / (ms * 1e-3) / 1e12
        print(json.dumps({
            "metric": "dense attention fwd tokens/s (dense)", "value": Bw * S / (ms * 1e-3), "unit": "tokens/s",
            "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "dtype": "bf16", "data": "synthetic", "config": {"workload": name, "l2": "2 rotating input sets"},
            "clocks": clocks, "kernel": nat.last_kernel(),
            "roofline": {"bound": "tensor", "achieved": tf, "peak": tpeak, "unit": "TFLOP/s", "frac": tf / tpeak,
                         "peak_source": f"{tkind} dense bf16 GEMM throughput", "flop_per_launch_algorithmic": flops},
            "parity_check": parity, "device_status": nat.device_status()}), flush=True)
        return
    print(json.dumps({
        "metric": f"sparse-attn fwd tokens/s ({args.workload})", "value": Bw * S / (ms * 1e-3), "unit": "tokens/s",
        "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "dtype": "f32" if f32 else "bf16", "data": "synthetic", "config": {"workload": name, "l2": "2 rotating input sets"},
        "clocks": clocks, "kernel": nat.last_kernel(),
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "peak_source": f"{peak_kind} HBM copy bandwidth", "bytes_per_launch_algorithmic": nbytes},
        "tensor": {"useful_flop_per_step": flops, "tflops": flops / (ms * 1e-3) / 1e12},
        "parity_check": parity, "device_status": nat.device_status()}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="window", choices=["window", "block", "longformer", "orderbook", "dense", "backward", "fp32", "refwindow"],
                    help="window = the headline configuration; block / longformer / orderbook / dense = one-GPU timing "
                         "of the block-sparse, Longformer, order-book-transformer and dense configurations")
    ap.add_argument("--left", type=int, default=64, help="refwindow: taps before the query")
    ap.add_argument("--right", type=int, default=64, help="refwindow: taps after the query")
    ap.add_argument("--dilation", type=int, default=1, help="refwindow: dilation")
    ap.add_argument("--head-dim", type=int, default=64, choices=[16, 32, 64, 128, 256, 512],
                    help="refwindow, backward: head width (the number of heads changes with it, 512 columns per token)")
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp32"],
                    help="refwindow, backward: element type (fp32 is the reference's own precision)")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="device-resident leg only (for profiler captures)")
    ap.add_argument("--halo", default="peer", choices=["peer", "nccl"],
                    help="N>1: edge tiles read the neighbour's rows in place (peer), or send/recv exchange (nccl)")
    ap.add_argument("--no-graph", dest="graph", action="store_false", help="launch every step from the host")
    ap.add_argument("--lanes", type=int, default=2,
                    help="streams the captured steps alternate over (each with its own output buffer)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    if args.impl == "reference":
        if int(os.environ.get("RANK", "0")) != 0:
            return
        steps, warmup = max(1, args.steps), args.warmup
        val, ms, info = reference_arm(steps, warmup)
        ran = (f"{WORKLOAD}; run by the reference's CPU engine in fp32 as its two-sided window +-{TAPS // 2} "
               f"(65 keys per row: the engine has no causal mode)") if info["kind"] == "reference" else WORKLOAD
        print(json.dumps({
            "impl": "reference", "metric": METRIC, "value": val, "unit": "tokens/s", "n_gpus": args.gpus,
            "steps": steps, "warmup": warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": {"workload": ran},
            "cpu_baseline": info,
            "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        }), flush=True)
        return
    if args.workload != "window":
        other_workload_arm(args)
        return
    gpu_arm(args)


if __name__ == "__main__":
    main()
