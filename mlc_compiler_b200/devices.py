"""Device profile for the cost model: the B200 entry the reference lacks.

The reference prices fusion decisions from a per-device table
(``mlc/devices.py:107-141``) that stops at Hopper; an unknown GPU silently gets
A100 constants (``:141,161-165``).  This module supplies the Blackwell entry
and a calibration that measures the three constants on the device itself
through this backend's own runtime (the reference's probe is a Triton kernel,
``mlc/bench/calibrate.py:46-59``):

* streaming copy bandwidth (a generated 128-bit copy kernel over a buffer
  larger than L2),
* launch overhead, eager and inside a CUDA graph (an empty-ish kernel),
* fp32 throughput (a dependent FMA chain per thread, many independent threads).

From those it derives the reference's cost-model fields: ``flops_per_byte``,
``launch_overhead_bytes`` and ``graph_launch_overhead_bytes``
(``mlc/config.py:36-52``).
"""

from __future__ import annotations

from dataclasses import dataclass

from .config import Config


@dataclass(frozen=True)
class DeviceProfile:
    name: str
    #: sustained streaming copy bandwidth, bytes/s (read + write)
    bandwidth: float
    #: fp32 FMA throughput, FLOP/s
    fp32_flops: float
    #: seconds per eager launch / per captured graph node
    launch_s: float
    graph_launch_s: float
    source: str = "table"

    @property
    def flops_per_byte(self) -> float:
        return self.fp32_flops / self.bandwidth

    @property
    def launch_overhead_bytes(self) -> float:
        return self.launch_s * self.bandwidth

    @property
    def graph_launch_overhead_bytes(self) -> float:
        return self.graph_launch_s * self.bandwidth

    def to_config(self, base: Config | None = None) -> Config:
        """The reference's ``DeviceProfile.to_config`` (``mlc/devices.py:71-76``)."""
        base = base or Config()
        return base.replace(flops_per_byte=self.flops_per_byte,
                            launch_overhead_bytes=self.launch_overhead_bytes,
                            graph_launch_overhead_bytes=self.graph_launch_overhead_bytes)


#: B200 (sm_100, 148 SMs, 1965 MHz boost): 148 x 128 lanes x 2 x 1.965 GHz = 74.5 TFLOP/s fp32
#: nominal.  The entry holds what :func:`calibrate` measures on a B200 (180 GB HBM3e,
#: 1 kW): 6.2-6.5 TB/s streaming copy, 67 TFLOP/s on the FMA chain, 5.7 us per
#: eager launch from Python, 0.53 us per node of a captured chain.
B200 = DeviceProfile(name="NVIDIA B200", bandwidth=6.459e12, fp32_flops=67.2e12,
                     launch_s=5.7e-6, graph_launch_s=0.55e-6)

TABLE = {"b200": B200}


def profile_for(device_name: str) -> DeviceProfile | None:
    key = device_name.lower()
    for tag, prof in TABLE.items():
        if tag in key:
            return prof
    return None


def config_for(device_name: str, base: Config | None = None) -> Config:
    """``base`` with the cost-model fields of the named device, as the reference's
    ``config_for`` (``mlc/devices.py:168-170``); a device without an entry keeps
    ``base`` unchanged (the reference's A100 defaults)."""
    prof = profile_for(device_name)
    return prof.to_config(base) if prof is not None else (base or Config())


def register_with_reference() -> bool:
    """Put the B200 entry at the head of the reference's own device table
    (``mlc/devices.py:107-134``), so that ``mlc.devices.profile_for`` -- which its
    bench harness prices fusion with (``mlc/bench/runner.py:158-161``) -- returns
    Blackwell constants on a B200 instead of the A100 fallback for an unknown
    device.  Returns False when the reference is not importable."""
    try:
        import importlib

        ref = importlib.import_module("mlc.devices")
    except ImportError:
        return False
    unregister_from_reference()
    ref.TABLE.insert(0, ("B200", ref.DeviceProfile(
        name=B200.name, bandwidth=B200.bandwidth, fp32_flops=B200.fp32_flops,
        launch_overhead=B200.launch_s, graph_launch_overhead=B200.graph_launch_s,
        l2_bytes=126 * 1024 ** 2, total_memory=180 * 1024 ** 3)))
    return True


def use_cuda_probe_in_reference() -> bool:
    """Give the reference's calibration (``mlc/bench/calibrate.py:141-168``) this
    package's CUDA fp32 probe in place of its Triton kernel (``:46-59,119-138``),
    so that ``python -m mlc.bench --calibrate`` measures all four constants on a
    machine without Triton.  Separate from :func:`register_with_reference`
    because importing ``mlc.bench.calibrate`` imports Triton where it is present,
    which ``install()`` must not do.  Returns False when the reference is absent."""
    import importlib

    try:
        cal = importlib.import_module("mlc.bench.calibrate")
    except ImportError:
        return False
    if not hasattr(cal, "_mlcb_saved_fp32_probe"):
        cal._mlcb_saved_fp32_probe = cal.measure_fp32_throughput
    cal.measure_fp32_throughput = measure_fp32_throughput
    return True


def unregister_from_reference() -> None:
    try:
        import importlib

        ref = importlib.import_module("mlc.devices")
    except ImportError:
        return
    ref.TABLE[:] = [(k, p) for k, p in ref.TABLE if k != "B200"]
    import sys

    cal = sys.modules.get("mlc.bench.calibrate")
    if cal is not None and hasattr(cal, "_mlcb_saved_fp32_probe"):
        cal.measure_fp32_throughput = cal._mlcb_saved_fp32_probe
        del cal._mlcb_saved_fp32_probe


# --------------------------------------------------------------------------
# calibration (needs a CUDA device)
# --------------------------------------------------------------------------

_PROBES = r"""
extern "C" __global__ void __launch_bounds__(256) mlcb_probe_copy(const uint4* __restrict__ src,
                                                                uint4* __restrict__ dst, long long n) {
    long long i = (long long)blockIdx.x * 256 + threadIdx.x;
    const long long stride = (long long)gridDim.x * 256;
    for (; i < n; i += stride) dst[i] = src[i];
}
extern "C" __global__ void mlcb_probe_empty(float* p) {
    if (p == nullptr) p[0] = 0.0f;
}
extern "C" __global__ void __launch_bounds__(256) mlcb_probe_fma(float* out, int iters) {
    float a = 1.0f + threadIdx.x * 1e-6f, b = 0.999f, c = 1e-3f;
    float x0 = a, x1 = a + 1.0f, x2 = a + 2.0f, x3 = a + 3.0f;
    for (int i = 0; i < iters; ++i) {
        x0 = fmaf(x0, b, c); x1 = fmaf(x1, b, c); x2 = fmaf(x2, b, c); x3 = fmaf(x3, b, c);
    }
    if (x0 + x1 + x2 + x3 == -1.0f) out[0] = x0;
}
"""


def measure_fp32_throughput(device="cuda", n: int = 1 << 20, chain: int = 512) -> float:
    """fp32 operations per second of pointwise code on ``device``: ``n`` threads
    each run four independent chains of ``chain`` fused multiply-adds.  Same
    signature and meaning as the reference's probe
    (``mlc/bench/calibrate.py:119-138``), which is a Triton kernel; this one is
    CUDA C++ compiled and launched through the C ABI, and ``install()`` puts it in
    the reference's place."""
    import ctypes

    import torch

    from .runtime import LoadedModule, _check, compile_source

    dev = torch.device(device)
    index = dev.index if dev.index is not None else torch.cuda.current_device()
    with torch.cuda.device(index):
        mod = LoadedModule(compile_source(_PROBES), index)
        buf = torch.zeros(16, device=torch.device("cuda", index))
        iters = max(1, int(chain) * 4)
        grid = max(1, int(n) // 256)
        arr = (ctypes.c_uint64 * 2)(buf.data_ptr(), iters)
        kernel = mod.kernel("mlcb_probe_fma")

        def launch():
            stream = torch.cuda.current_stream(index).cuda_stream
            _check(mod.lib, mod.lib.mlcb_launch(kernel, grid, 256, 0, arr, 2, stream, 0), "mlcb_probe_fma")

        for _ in range(3):
            launch()
        torch.cuda.synchronize(index)
        s_, e_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 10
        s_.record()
        for _ in range(reps):
            launch()
        e_.record()
        torch.cuda.synchronize(index)
        seconds = s_.elapsed_time(e_) * 1e-3 / reps
    return grid * 256 * 4 * 2 * iters / seconds


def calibrate(device="cuda", quick: bool = False) -> DeviceProfile:
    """Measure the profile on ``device`` with CUDA events."""
    import ctypes

    import torch

    from .runtime import LoadedModule, _check, compile_source

    dev = torch.device(device)
    index = dev.index if dev.index is not None else torch.cuda.current_device()
    torch.cuda.set_device(index)
    mod = LoadedModule(compile_source(_PROBES), index)
    lib = mod.lib
    stream = torch.cuda.current_stream().cuda_stream

    def launch(sym, grid, block, *vals):
        arr = (ctypes.c_uint64 * len(vals))(*vals)
        _check(lib, lib.mlcb_launch(mod.kernel(sym), grid, block, 0, arr, len(vals), stream, 0), sym)

    def timed(fn, reps):
        fn()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(reps):
            fn()
        e.record()
        torch.cuda.synchronize()
        return s.elapsed_time(e) * 1e-3 / reps

    n_bytes = (256 if quick else 1024) << 20
    src = torch.empty(n_bytes, dtype=torch.uint8, device=dev)
    dst = torch.empty_like(src)
    n_vec = n_bytes // 16
    sm = torch.cuda.get_device_properties(index).multi_processor_count
    t = timed(lambda: launch("mlcb_probe_copy", sm * 16, 256, src.data_ptr(), dst.data_ptr(), n_vec),
              5 if quick else 20)
    bandwidth = 2 * n_bytes / t

    buf = torch.zeros(16, device=dev)
    eager = timed(lambda: launch("mlcb_probe_empty", 1, 32, buf.data_ptr()), 2000)
    g = torch.cuda.CUDAGraph()
    nodes = 500
    with torch.cuda.graph(g):
        cs = torch.cuda.current_stream().cuda_stream
        arr = (ctypes.c_uint64 * 1)(buf.data_ptr())
        for _ in range(nodes):
            _check(lib, lib.mlcb_launch(mod.kernel("mlcb_probe_empty"), 1, 32, 0, arr, 1, cs, 0), "probe")
    graph = timed(g.replay, 20) / nodes

    iters = 2048 if quick else 8192
    # iters is a by-value int parameter; the shim passes 8-byte slots, the low 4 are read
    tf = timed(lambda: launch("mlcb_probe_fma", sm * 8, 256, buf.data_ptr(), iters), 5)
    flops = sm * 8 * 256 * 4 * 2 * iters / tf
    return DeviceProfile(name=torch.cuda.get_device_name(index), bandwidth=bandwidth,
                         fp32_flops=flops, launch_s=eager, graph_launch_s=graph, source="measured")


def report(measured: DeviceProfile, table: DeviceProfile | None = None) -> str:
    rows = [f"device            {measured.name} ({measured.source})",
            f"copy bandwidth    {measured.bandwidth / 1e9:8.1f} GB/s",
            f"fp32 throughput   {measured.fp32_flops / 1e12:8.2f} TFLOP/s",
            f"launch            {measured.launch_s * 1e6:8.2f} us eager, "
            f"{measured.graph_launch_s * 1e6:.2f} us per graph node",
            f"flops_per_byte    {measured.flops_per_byte:8.2f}",
            f"launch_overhead_bytes        {measured.launch_overhead_bytes:12.0f}",
            f"graph_launch_overhead_bytes  {measured.graph_launch_overhead_bytes:12.0f}"]
    if table is not None:
        rows.append(f"table entry       {table.bandwidth / 1e9:.0f} GB/s, {table.fp32_flops / 1e12:.1f} TFLOP/s, "
                    f"{table.launch_s * 1e6:.1f}/{table.graph_launch_s * 1e6:.1f} us")
    return "\n".join(rows)
