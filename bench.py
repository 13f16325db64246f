"""Benchmark: BERT-base fp16, batch 1, sequence 128, one CUDA graph per forward.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one forward of the compiled schedule.  Rank 0 prints ONE JSON line,
kept short; ``--details FILE`` additionally writes the long per-kernel tables
(grid, block, registers and buffer sets of every microbenchmark cell, every
in-model function, the replica rows, the same-method comparison) as JSON.

* ``value`` / ``ms_per_step``: latency of one graph replay with the inputs already
  in device memory, per-step CUDA events, L2 flushed (a 256 MiB write) between
  steps, mean over exactly K steps, max over ranks.
* ``e2e``: the same forward through the public call ``compiled(*host_inputs)``:
  pinned host inputs are copied in, the graph replayed, the result copied back
  to pinned host memory, host wall clock around each step (device drained at the
  end of every step).
* ``roofline``: the fused-kernel microbenchmarks (LayerNorm, causal softmax,
  bias+GELU+residual, fp16), timed live as CUDA graphs of launches over rotating
  buffer sets totalling more than four times L2.  The object describes the
  *lowest* of the three batch-32 cells; ``cells`` gives all three and
  ``fused_kernels`` all nine (batch 1, 8, 32).  ``traffic`` is the DRAM byte
  count of an ncu capture of the same function (looked up by symbol: a kernel
  that has changed since the capture reports null).
* ``cpu_baseline``: the reference's own CPU path (``mlc.compile`` with
  ``Config(backend="torch")`` on the copy of the reference under
  ``oracle/_ref``) timed on this host's cores on the same workload; where that
  copy is absent, the CPU oracle (a port) stands in and ``kind`` says so.
* ``config.replicas``: BERT-base and GPT-2 small, fp16 and bf16, batch 32 split
  32/N per GPU as independent replicas.  ``seq_per_s`` = 32 / the slowest rank's
  mean replay time; ``e2e_seq_per_s`` = 32 / the wall time from a common barrier
  to the moment every rank holds its output shard in pinned host memory (host
  shard -> device, replay, device -> host).
* ``config.same_method``: the reference's stock Triton build and this backend
  compiled from the same model object through ``mlc.compile`` in this process,
  timed alternately with the reference's own method (20 warm-ups, median of 50
  event-timed calls, ``mlc/bench/runner.py:84-104``).  N = 1 only; bench-only --
  Triton is not part of the product.

With N > 1 (torchrun) every rank runs an independent replica; there is no
data-path collective, only barriers and a max of the timings.
``--impl reference`` times the reference's CPU path alone on rank 0.
"""

from __future__ import annotations

import argparse
import json
import os
import pathlib
import statistics
import sys
import threading
import time

ROOT = pathlib.Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))
os.environ.setdefault("MLC_CACHE_DIR", str(ROOT / ".mlc_cache"))

import torch  # noqa: E402

WORKLOAD = "bert-base fp16 b1 s128, one CUDA graph per forward"
METRIC = "bert_base_fp16_b1_s128_latency"
#: what both arms state about the workload (the reference arm prints exactly these)
STATIC_CONFIG = {"workload": WORKLOAD, "accumulate": "f32", "batch": 1, "seq_len": 128,
                 "kernels_scheduled": 200}

#: dram__bytes_read.sum + dram__bytes_write.sum per launch, by function symbol,
#: from `ncu --set full` captures of the batch-32 microbenchmarks.  Written
#: lines that are still dirty in the 126 MB L2 when the kernel ends are not in
#: the figure, so it can be below the algorithmic bytes.
NCU_TRAFFIC: dict[str, int] = {
    "mlcb_red_4357894e362b": 6302720,              # LayerNorm [4096, 768]: 6,302,720 read + 0 written
    "mlcb_red_68614aa18ce2": 12623616,             # causal softmax [49152, 128]: 12,623,616 + 0
    "mlcb_pw_9dd2f6a63b0f": 50347008 + 1423104,    # bias+GELU+residual [4096, 3072]
}


def _peaks() -> tuple[float, str]:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


# --------------------------------------------------------------------------
# clocks
# --------------------------------------------------------------------------

class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while a region runs.
    Read-only: no setting of the GPU is touched."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown",
               0x4: "sw_power_cap", 0x80: "hw_power_brake", 0x2: "applications_clocks",
               0x100: "display_clocks"}

    def __init__(self, index: int, period: float = 0.005):
        self.index, self.period = index, period
        self.samples: list[int] = []
        self.reasons: set[str] = set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _loop(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(self.period)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self) -> dict:
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


# --------------------------------------------------------------------------
# pieces
# --------------------------------------------------------------------------

def _compiled(name: str, batch: int, dtype, dev, **cfg):
    from mlc_compiler_b200 import Config, models
    from mlc_compiler_b200.executor import CompiledModel
    from mlc_compiler_b200.frontend import load_schedule

    sched = load_schedule(models.schedule_name(name, batch, dtype))
    model, inputs = models.build(name, batch, dtype=dtype)
    return CompiledModel(sched, model, Config(**cfg), dev), inputs, sched


class L2Flush:
    def __init__(self, dev, mib: int = 256):
        self.buf = torch.empty(mib << 20, dtype=torch.uint8, device=dev)

    def __call__(self):
        self.buf.fill_(1)


def time_replays(cm, dev_inputs, steps: int, warmup: int, flush) -> list[float]:
    """Per-step device time of one replay, inputs resident, L2 flushed between."""
    cm(*dev_inputs)
    for _ in range(warmup):
        flush()
        cm.replay()
    torch.cuda.synchronize()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    for i in range(steps):
        flush()
        starts[i].record()
        cm.replay()
        ends[i].record()
    torch.cuda.synchronize()
    return [s.elapsed_time(e) for s, e in zip(starts, ends)]


def time_end_to_end(cm, host_inputs, steps: int, warmup: int, flush) -> tuple[list[float], int, int]:
    """Host wall clock of copy-in, replay, copy-out, per step."""
    pinned = [t.contiguous().pin_memory() for t in host_inputs]
    out = cm(*pinned)
    host_out = torch.empty(out.shape, dtype=out.dtype).pin_memory()
    h2d = sum(t.numel() * t.element_size() for t in pinned)
    d2h = host_out.numel() * host_out.element_size()
    times = []
    for i in range(warmup + steps):
        flush()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        out = cm(*pinned)
        host_out.copy_(out, non_blocking=True)
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        if i >= warmup:
            times.append((t1 - t0) * 1e3)
    return times, h2d, d2h


def micro_roofline(dev, peak_gbs: float, batches=(1, 8, 32), launches: int = 64,
                   only: str | None = None, branches: int = 0, **cfg_kw) -> list[dict]:
    """Each fused-kernel microbenchmark as a CUDA graph of ``launches`` launches
    cycling over buffer sets whose total size exceeds 4x L2, so every launch
    reads and writes HBM.  The launches form one chain (each waits for the one
    before it, as consecutive kernels of a model do): ``us_per_launch`` therefore
    includes the fixed latency of a dependent launch.  With ``branches`` > 1 the
    batch-32 rows also report the same launches captured over that many parallel
    graph branches (``branches_us`` / ``branches_frac``): independent launches
    overlapping each other's ramp-up and drain, i.e. the rate the kernel streams
    at once that latency is hidden."""
    from mlc_compiler_b200 import Config, models
    from mlc_compiler_b200.frontend import load_schedule
    from mlc_compiler_b200.runtime import CudaRuntime

    l2 = 126 << 20
    rows = []
    for name in ("micro-layernorm", "micro-softmax", "micro-gelu"):
        for b in batches:
            if only and only != f"{name}:{b}":
                continue
            sched = load_schedule(models.schedule_name(name, b, torch.float16))
            k = sched.generated()[0]
            rt = CudaRuntime(sched, Config(**cfg_kw), dev)
            spec = rt.generated.launch[k.name]
            model, inputs = models.build(name, b, dtype=torch.float16)
            table = dict(model.named_parameters(remove_duplicate=False))
            table.update(dict(model.named_buffers(remove_duplicate=False)))
            big = [n for n in set(k.reads()) | set(k.writes()) if n not in sched.params]
            per_set = sum(sched.buffers[n].nbytes for n in big)
            sets = max(2, min(4096, -(-4 * l2 // per_set)))
            n_launch = max(launches, sets)
            fixed = {n: table[o].detach().to(dev, getattr(torch, sched.buffers[n].dtype))
                     .contiguous().reshape(-1) for n, o in sched.params.items()
                     if n in k.reads()}
            bound = []
            for s in range(sets):
                bufs = dict(fixed)
                for v, t in zip(sched.inputs, inputs):
                    bufs[v.buffer] = t.to(dev).reshape(-1).clone()
                for n in big:
                    if n not in bufs:
                        bufs[n] = torch.empty(sched.buffers[n].numel, device=dev,
                                              dtype=getattr(torch, sched.buffers[n].dtype))
                # consecutive generated kernels on one stream: what the executor's
                # "chain" policy launches programmatically
                bound.append(rt.bind(k, bufs, 1 if (rt.chain or rt.flags) else 0)[0])
            side = torch.cuda.Stream(device=dev)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for f in bound:
                    f()
            torch.cuda.current_stream().wait_stream(side)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                for i in range(n_launch):
                    bound[i % sets]()
            for _ in range(3):
                g.replay()
            torch.cuda.synchronize()
            reps = 10
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            for _ in range(reps):
                g.replay()
            e.record()
            torch.cuda.synchronize()
            us = s.elapsed_time(e) * 1e3 / (reps * n_launch)
            gbs = spec.alg_bytes / us / 1e3
            info = rt.kernel_info(k.name)
            extra = {}
            if branches > 1 and b == 32 and sets >= branches:
                g2 = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g2):
                    main = torch.cuda.current_stream()
                    lanes = [main] + [torch.cuda.Stream(device=dev) for _ in range(branches - 1)]
                    for ln in lanes[1:]:
                        ln.wait_stream(main)
                    for i in range(n_launch):
                        with torch.cuda.stream(lanes[i % branches]):
                            bound[i % sets]()
                    for ln in lanes[1:]:
                        main.wait_stream(ln)
                for _ in range(3):
                    g2.replay()
                torch.cuda.synchronize()
                s.record()
                for _ in range(reps):
                    g2.replay()
                e.record()
                torch.cuda.synchronize()
                us2 = s.elapsed_time(e) * 1e3 / (reps * n_launch)
                extra = {"branches": branches, "branches_us": round(us2, 3),
                         "branches_frac": round(spec.alg_bytes / us2 / 1e3 / peak_gbs, 4)}
                del g2
            rows.append({**extra, "kernel": name, "batch": b, "symbol": rt.generated.symbol[k.name],
                         "alg_bytes": spec.alg_bytes,
                         "us_per_launch": round(us, 3), "gbs": round(gbs, 1),
                         "frac": round(gbs / peak_gbs, 4), "grid": spec.grid, "block": spec.block,
                         "registers": info["registers"],
                         "buffer_sets": sets, "set_bytes": per_set,
                         "launches_per_graph": n_launch,
                         "hbm_resident": bool(sets * per_set >= 4 * l2)})
            del bound, g
    return rows


def in_model_families(cm, dev_inputs, peak_gbs: float, reps: int = 20) -> list[dict]:
    """Device time of each distinct generated function inside the BERT step: one
    bound launch of it replayed ``reps`` times inside a CUDA graph (in place, so
    it runs out of L2 and is launch-bound at batch 1; reported for context)."""
    cm(*dev_inputs)
    torch.cuda.synchronize()
    table = cm.launch_table
    groups: dict[str, list[str]] = {}
    for name, row in table.items():
        groups.setdefault(row["symbol"], []).append(name)
    out = []
    for sym, names in groups.items():
        kind, fn = cm._bound[names[0]]
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            fn()
        torch.cuda.current_stream().wait_stream(side)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(reps):
                fn()
        g.replay()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(5):
            g.replay()
        e.record()
        torch.cuda.synchronize()
        us = s.elapsed_time(e) * 1e3 / (5 * reps)
        ab = table[names[0]]["alg_bytes"]
        out.append({"symbol": sym, "kernel": cm.executed_schedule.kernel(names[0]).summary().split(": ", 1)[1][:70],
                    "launches_per_forward": len(names), "us_per_launch": round(us, 3),
                    "alg_bytes": ab, "gbs": round(ab / us / 1e3, 1),
                    "frac": round(ab / us / 1e3 / peak_gbs, 4), "l2_resident": True})
    out.sort(key=lambda r: -r["us_per_launch"] * r["launches_per_forward"])
    return out


# --------------------------------------------------------------------------
# the reference's CPU path (and the port that stands in where it is absent)
# --------------------------------------------------------------------------

def _host_threads() -> int:
    # torchrun pins OMP_NUM_THREADS=1; the baseline is meant to use every host core
    try:
        torch.set_num_threads(max(1, len(os.sched_getaffinity(0))))
    except (AttributeError, RuntimeError):
        pass
    return torch.get_num_threads()


def reference_cpu_times(steps: int, warmup: int) -> tuple[list[float], int, str, str]:
    """``(per-step ms, threads, kind, sample)`` of BERT-base fp16 b1 on the host
    cores: the reference's torch backend behind ``mlc.compile`` when the copy under
    ``oracle/_ref`` is there (kind "reference"), else the CPU oracle (kind "port")."""
    from mlc_compiler_b200 import models

    sys.path.insert(0, str(ROOT / "oracle"))
    cores = _host_threads()
    model, inputs = models.build("bert-base", 1, dtype=torch.float16)
    try:
        import ref as reference_copy
        reference_copy.activate()
        import mlc
        from mlc.config import Config as RefConfig
    except ImportError:
        mlc = None
    if mlc is not None:
        compiled = mlc.compile(model, inputs, RefConfig(backend="torch", cuda_graphs=False),
                               device="cpu")
        run = lambda: compiled(*inputs)                                   # noqa: E731
        kind = "reference"
        sample = ("whole forwards of mlc.compile(..., Config(backend='torch', cuda_graphs=False), "
                  "device='cpu'), perf_counter per call")
    else:
        import kir_oracle as oracle
        from mlc_compiler_b200.frontend import load_schedule

        sched = load_schedule("bert-base_b1_s128_float16")
        table = dict(model.named_parameters(remove_duplicate=False))
        table.update(dict(model.named_buffers(remove_duplicate=False)))
        buffers = oracle.allocate(sched, table, inputs)
        run = lambda: oracle.run_schedule(sched, table, inputs, buffers=buffers)   # noqa: E731
        kind = "port"
        sample = "whole forwards of the same 200-kernel schedule on the CPU oracle"
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        run()
        if i >= warmup:
            times.append((time.perf_counter() - t0) * 1e3)
    return times, cores, kind, f"{steps} {sample}"


def run_reference(args) -> int:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    steps, warmup = max(1, min(args.steps, 100)), max(0, args.warmup)
    times, cores, kind, sample = reference_cpu_times(steps, warmup)
    ms = statistics.mean(times)
    line = {
        "impl": "reference", "metric": METRIC, "value": round(ms, 4), "unit": "ms",
        "n_gpus": args.gpus, "steps": steps, "warmup": warmup, "ms_per_step": round(ms, 4),
        "median_ms": round(statistics.median(times), 4),
        "higher_is_better": False, "scaling": "weak", "vs_baseline": None, "dtype": "f16",
        "data": "synthetic", "config": dict(STATIC_CONFIG, device="cpu"),
        "cpu_baseline": {"value": round(ms, 4), "unit": "ms", "cores": cores, "kind": kind,
                         "sample": sample},
        "e2e": {"value": round(ms, 4), "unit": "ms", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))
    return 0


# --------------------------------------------------------------------------
# same-method comparison with the reference's Triton build (bench-only)
# --------------------------------------------------------------------------

def same_method_comparison(dev, rounds: int = 5, batches=(1,)) -> dict:
    """Compile one model object three ways through the reference's public
    ``mlc.compile`` -- its stock Triton backend; this backend under the reference's
    own executor (``install()``); this backend with this package's executor
    (``install(native_executor=True)``) -- and time them alternately with the
    reference's method: 20 warm-up calls, then the median of 50 event-timed calls
    of ``compiled(*inputs)``, no L2 flush (``mlc/bench/runner.py:84-104``).
    Returns milliseconds (median over ``rounds`` rounds) per model."""
    sys.path.insert(0, str(ROOT / "oracle"))
    out: dict = {"method": f"mlc.compile on one model object; 20 warm-ups then median of 50 "
                           f"event-timed calls, no L2 flush; {rounds} alternating rounds, median"}
    try:
        import ref as reference_copy
        reference_copy.activate()
        import mlc
        import triton  # noqa: F401
        from mlc.config import Config as RefConfig
    except ImportError as e:
        out["unavailable"] = f"{type(e).__name__}: {e}"
        return out
    import mlc_compiler_b200 as mb
    from mlc_compiler_b200 import models

    def timed(fn, inputs) -> float:
        for _ in range(20):
            fn(*inputs)
        torch.cuda.synchronize()
        ts = []
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for _ in range(50):
            s.record()
            fn(*inputs)
            e.record()
            e.synchronize()
            ts.append(s.elapsed_time(e))
        return statistics.median(ts)

    for name, batch in [(n, b) for n in ("bert-base", "gpt2-small") for b in batches]:
        key = name.replace("-", "_") + f"_b{batch}"
        try:
            model, inputs = models.build(name, batch, dtype=torch.float16)
            model = model.to(dev)
            inputs = tuple(t.to(dev) for t in inputs)
            mb.uninstall()
            arms = {"triton_ref": mlc.compile(model, inputs, RefConfig(), device=dev)}
            if arms["triton_ref"].backend != "triton":
                raise RuntimeError(f"reference chose backend {arms['triton_ref'].backend!r}")
            mb.install()
            arms["ours_ref_executor"] = mlc.compile(model, inputs, RefConfig(), device=dev)
            mb.install(native_executor=True)
            arms["ours"] = mlc.compile(model, inputs, RefConfig(), device=dev)
            mb.uninstall()
            want = arms["triton_ref"](*inputs).float()
            err = {a: float((c(*inputs).float() - want).abs().max()) for a, c in arms.items()}
            samples = {a: [] for a in arms}
            for _ in range(rounds):
                for a, c in arms.items():
                    samples[a].append(timed(c, inputs))
            out[key] = {f"{a}_ms": round(statistics.median(v), 4) for a, v in samples.items()}
            out[key]["max_abs_diff_vs_triton"] = round(max(err.values()), 5)
            del arms
        except Exception as e:           # Triton may fail to JIT on a given stack
            mb.uninstall()
            out[key] = {"unavailable": f"{type(e).__name__}: {str(e)[:160]}"}
    return out


# --------------------------------------------------------------------------
# replicas: batch 32 split over the ranks
# --------------------------------------------------------------------------

def replica_rows(group, dev, steps: int, flush, cfg_kw, combos=None) -> list[dict]:
    """Batch 32 split 32/N per GPU as independent replicas, for each model and
    dtype: device-timed replays and the end-to-end variant from pinned host
    shards to pinned host outputs, both between common barriers."""
    from mlc_compiler_b200.replicas import shard_inputs, split_throughput
    from mlc_compiler_b200 import models

    per_gpu = 32 // group.world
    rows = []
    for name, dt in combos or [(m, d) for m in ("bert-base", "gpt2-small")
                               for d in (torch.float16, torch.bfloat16)]:
        cm, _, sched = _compiled(name, per_gpu, dt, dev, **cfg_kw)
        # the whole batch of 32 as the host sees it; this rank takes its contiguous share
        _, full = models.build_inputs(name, 32, dtype=dt)
        mine = [t.contiguous().pin_memory() for t in shard_inputs(full, group.world, group.rank)]
        dev_in = [t.to(dev) for t in mine]
        ms = statistics.mean(time_replays(cm, dev_in, steps, 3, flush))
        thr = split_throughput(group, 32, ms, dev)
        out = cm(*mine)
        host_out = torch.empty(out.shape, dtype=out.dtype).pin_memory()
        e2e = []
        for i in range(2 + steps):
            flush()
            barrier(group)
            t0 = time.perf_counter()
            out = cm(*mine)
            host_out.copy_(out, non_blocking=True)
            torch.cuda.synchronize()
            wall = group.max((time.perf_counter() - t0) * 1e3, dev)   # last rank to finish
            if i >= 2:
                e2e.append(wall)
        e2e_ms = statistics.mean(e2e)
        rows.append({"model": name, "dtype": str(dt).split(".")[-1].replace("float", "f"),
                     "per_gpu_batch": per_gpu, "seq_per_s": round(thr["seq_per_s"], 1),
                     "ms_slowest": round(thr["ms_per_forward"], 4),
                     "e2e_seq_per_s": round(32 / (e2e_ms / 1e3), 1), "e2e_ms": round(e2e_ms, 3),
                     "arena_mb_per_gpu": round(sched.arena_bytes / 2 ** 20, 2),
                     "launches": len(cm.executed_schedule)})
        del cm, host_out, out
    return rows


# --------------------------------------------------------------------------

def barrier(group) -> None:
    group.barrier()
    torch.cuda.synchronize()


def _write_details(details: dict, path: str | None) -> str | None:
    if not path:
        return None
    out = pathlib.Path(path)
    try:
        out.parent.mkdir(parents=True, exist_ok=True)
        out.write_text(json.dumps(details, indent=1))
        return str(path)
    except OSError:
        return None


def _parse_cfg(pairs) -> dict:
    kw = dict(kv.split("=") for kv in pairs)
    return {k: (v == "True" if v in ("True", "False") else int(v) if v.lstrip("-").isdigit() else v)
            for k, v in kw.items()}


def run_ours(args) -> int:
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the generated kernels have no CPU path")
    from mlc_compiler_b200.replicas import ReplicaGroup

    local = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    group = ReplicaGroup.from_env(backend="nccl", device=dev)
    rank, world = group.rank, group.world
    peak, peak_kind = _peaks()
    steps, warmup = max(1, args.steps), max(3, args.warmup)
    cfg_kw = _parse_cfg(args.cfg)

    if args.section == "families":
        fcm, fin, fs = _compiled(args.model, args.batch, getattr(torch, args.dtype), dev, **cfg_kw)
        fdev = [t.to(dev) for t in fin]
        fam = in_model_families(fcm, fdev, peak)
        lat = statistics.median(time_replays(fcm, fdev, 50, 10, lambda: None))
        print(json.dumps({"model": args.model, "batch": args.batch, "dtype": args.dtype,
                          "median_ms_no_flush": round(lat, 5), "kernels": len(fs),
                          "generated_us": round(sum(r["us_per_launch"] * r["launches_per_forward"]
                                                    for r in fam), 1), "families": fam}))
        return 0
    if args.section == "replicas":
        rows = replica_rows(group, dev, max(5, steps // 4), L2Flush(dev), cfg_kw)
        if rank == 0:
            print(json.dumps({"replicas": rows, "n_gpus": world, "l2": "flushed between steps"}))
        group.close()
        return 0
    if args.section == "same-method":
        batches = tuple(int(b) for b in args.batches.split(","))
        print(json.dumps(same_method_comparison(dev, batches=batches)))
        return 0
    if args.section == "compare":
        # this backend alone, timed as the reference's harness does (mlc/bench/runner.py:84-112):
        # median of 50 event-timed calls of compiled(*inputs) after 20 warm-ups, no flush
        rows = []
        for name, tag in (("bert-base", ""), ("gpt2-small", ""), ("gpt2-small", "ref")):
            for dt in ("float16", "bfloat16"):
                for b in (1, 8, 32):
                    if tag and dt != "float16":
                        continue
                    from mlc_compiler_b200 import Config, models
                    from mlc_compiler_b200.executor import CompiledModel
                    from mlc_compiler_b200.frontend import load_schedule, schedule_path
                    stem = models.schedule_name(name, b, getattr(torch, dt), tag=tag)
                    if not schedule_path(stem).exists():
                        continue
                    sch = load_schedule(stem)
                    model, inputs = models.build(name, b, dtype=getattr(torch, dt),
                                                 **sch.meta.get("variant", {}))
                    cmx = CompiledModel(sch, model, Config(**cfg_kw), dev)
                    di = [t.to(dev) for t in inputs]
                    for _ in range(20):
                        cmx(*di)
                    torch.cuda.synchronize()
                    ts = []
                    for _ in range(50):
                        s0, e0 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                        s0.record()
                        cmx(*di)
                        e0.record()
                        e0.synchronize()
                        ts.append(s0.elapsed_time(e0))
                    rows.append({"model": stem, "kernels": len(sch), "median_ms": round(statistics.median(ts), 4),
                                 "p10_ms": round(sorted(ts)[5], 4),
                                 "arena_mb": round(sch.arena_bytes / 2**20, 2),
                                 "peak_alloc_mb": round(torch.cuda.max_memory_allocated(dev) / 2**20, 1)})
                    del cmx
        print(json.dumps({"compare": rows, "cfg": cfg_kw}))
        return 0
    if args.section == "micro":
        rows = micro_roofline(dev, peak, only=args.only, branches=args.branches, **cfg_kw)
        print(json.dumps({"fused_kernels": rows, "cfg": cfg_kw}))
        return 0

    cm, host_inputs, sched = _compiled("bert-base", 1, torch.float16, dev, **cfg_kw)
    dev_inputs = [t.to(dev) for t in host_inputs]
    flush = L2Flush(dev)
    cm(*dev_inputs)
    torch.cuda.synchronize()

    barrier(group)
    with ClockSampler(local) as clocks:
        t_wall = time.perf_counter()
        per_step = time_replays(cm, dev_inputs, steps, warmup, flush)
        barrier(group)
        wall = time.perf_counter() - t_wall
    ms = group.max(statistics.mean(per_step), dev)
    med = group.max(statistics.median(per_step), dev)

    if args.section == "model":
        if rank == 0:
            print(json.dumps({"metric": METRIC, "value": round(ms, 5), "unit": "ms",
                              "steps": steps, "warmup": warmup, "cfg": cfg_kw}))
        return 0
    e2e_times, h2d, d2h = time_end_to_end(cm, host_inputs, steps, warmup, flush)
    e2e_ms = group.max(statistics.mean(e2e_times), dev)

    # GPT-2 small fp16 b1 beside the headline, same timing
    gcm, gin, gsched = _compiled("gpt2-small", 1, torch.float16, dev, **cfg_kw)
    gdev = [t.to(dev) for t in gin]
    gpt_ms = group.max(statistics.mean(time_replays(gcm, gdev, max(10, steps // 4), 3, flush)), dev)
    del gcm

    # batch 32 split over the ranks, independent replicas, both models, both narrow dtypes
    replicas = replica_rows(group, dev, max(5, steps // 4), flush, cfg_kw)

    config = dict(STATIC_CONFIG)
    config.update({
        "launched": len(cm.executed_schedule), "generated": cm.generated_launches,
        "arena_kib": round(sched.arena_bytes / 1024, 1),
        "l2": "flushed between steps",
        "graph_streams": cm.cfg.graph_streams, "dependent_policy": str(cm.dependent_policy),
        "parallelism": f"{world} independent replicas, no collectives",
        "gpt2_small_fp16_b1_ms": round(gpt_ms, 5),
        "replicas": {"global_batch": 32, "per_gpu_batch": 32 // world,
                     "cols": ["model", "dtype", "seq_per_s", "e2e_seq_per_s", "arena_mb_per_gpu",
                              "launches"],
                     "rows": [[r["model"], r["dtype"], r["seq_per_s"], r["e2e_seq_per_s"],
                               r["arena_mb_per_gpu"], r["launches"]] for r in replicas]},
    })
    line = {
        "metric": METRIC, "value": round(ms, 5), "unit": "ms", "n_gpus": world, "steps": steps,
        "warmup": warmup, "ms_per_step": round(ms, 5), "median_ms": round(med, 5),
        "higher_is_better": False, "scaling": "weak", "vs_baseline": None, "dtype": "f16",
        "data": "synthetic", "config": config,
        "e2e": {"value": round(e2e_ms, 5), "unit": "ms", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "timing": "host wall clock, drained per step"},
        # generated kernels launched inside the timed region, all ranks together
        "gpu_launches": cm.generated_launches * steps * world,
        "clocks": clocks.summary(),
        "timed_region_wall_s": round(wall, 3),
    }

    if rank == 0:
        details: dict = {"line": line, "replicas": replicas}
        micro = micro_roofline(dev, peak, batches=(1, 8, 32), branches=args.branches, **cfg_kw)
        cells = [r for r in micro if r["batch"] == 32]
        low = min(cells, key=lambda r: r["frac"])
        line["roofline"] = {
            "bound": "hbm", "achieved": low["gbs"], "peak": peak, "unit": "GB/s",
            "frac": low["frac"], "traffic": NCU_TRAFFIC.get(low["symbol"]),
            "kernel": f"{low['kernel']} b32 fp16 {low['symbol']} {low['grid']}x{low['block']}, "
                      "lowest b32 cell, chain of dependent launches",
            "alg_bytes_per_launch": low["alg_bytes"], "us_per_launch": low["us_per_launch"],
            "peak_source": peak_kind,
            "cells": {f"{r['kernel'][6:]}_b32": {"frac": r["frac"], "us": r["us_per_launch"],
                                                 "symbol": r["symbol"],
                                                 "traffic": NCU_TRAFFIC.get(r["symbol"]),
                                                 "branches4_frac": r.get("branches_frac")}
                      for r in cells}}
        line["fused_kernels"] = [[r["kernel"][6:], r["batch"], r["us_per_launch"], r["frac"]]
                                 for r in micro]
        details["fused_kernels"] = micro
        details["in_model"] = in_model_families(cm, dev_inputs, peak)
        gen_us = sum(r["us_per_launch"] * r["launches_per_forward"] for r in details["in_model"])
        config["generated_us_per_step"] = round(gen_us, 1)
        if world == 1 and not args.no_cpu:
            times, cores, kind, sample = reference_cpu_times(10, 1)
            line["cpu_baseline"] = {"value": round(statistics.mean(times), 3), "unit": "ms",
                                    "cores": cores, "kind": kind, "sample": sample}
        if world == 1 and not args.no_triton:
            sm = same_method_comparison(dev)
            details["same_method"] = sm
            bert = sm.get("bert_base_b1", {})
            gpt = sm.get("gpt2_small_b1", {})
            config["triton_ref_ms"] = bert.get("triton_ref_ms")
            config["ours_same_method_ms"] = bert.get("ours_ms")
            config["same_method"] = {
                "cols": ["triton_ref_ms", "ours_ref_executor_ms", "ours_ms"],
                "bert_base_b1": [bert.get(c) for c in ("triton_ref_ms", "ours_ref_executor_ms", "ours_ms")],
                "gpt2_small_b1": [gpt.get(c) for c in ("triton_ref_ms", "ours_ref_executor_ms", "ours_ms")]}
            note = sm.get("unavailable") or bert.get("unavailable") or gpt.get("unavailable")
            if note:
                config["triton_note"] = note
        written = _write_details(details, args.details)
        if written:
            line["details"] = written
    barrier(group)
    if rank == 0:
        print(json.dumps(line, separators=(",", ":")))
    group.close()
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=("ours", "reference"))
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-triton", action="store_true",
                    help="skip the same-method comparison with the reference's Triton build")
    ap.add_argument("--section", default="all",
                    choices=("all", "micro", "model", "families", "compare", "replicas", "same-method"),
                    help="'micro' prints only the fused-kernel microbenchmark table, "
                         "'model' only the device-timed BERT step (both for profiling)")
    ap.add_argument("--model", default="bert-base")
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--dtype", default="float16")
    ap.add_argument("--only", default=None, metavar="KERNEL:BATCH",
                    help="with --section micro: one row, e.g. micro-gelu:8")
    ap.add_argument("--details", default=None, metavar="FILE",
                    help="also write the long per-kernel tables to this JSON file")
    ap.add_argument("--batches", default="1", help="with --section same-method: e.g. 1,8,32")
    ap.add_argument("--branches", type=int, default=4,
                    help="parallel graph branches of the extra batch-32 microbenchmark figure (0 = skip)")
    ap.add_argument("--cfg", action="append", default=[], metavar="KEY=VALUE",
                    help="override a Config field (e.g. dependent_launch=True)")
    args = ap.parse_args()
    return run_reference(args) if args.impl == "reference" else run_ours(args)


if __name__ == "__main__":
    raise SystemExit(main())
