"""B200 device profile: constants are physical, and convert to cost-model fields."""

import pytest
import torch

from mlc_compiler_b200 import Config, devices


def test_table_entry_is_physical():
    p = devices.profile_for("NVIDIA B200")
    assert p is devices.B200
    assert 4e12 < p.bandwidth < 8.1e12          # below nominal HBM3e, above Hopper
    assert 50e12 < p.fp32_flops < 90e12
    assert 0 < p.graph_launch_s < p.launch_s < 20e-6
    assert devices.profile_for("NVIDIA A40") is None


def test_profile_converts_to_cost_model_fields():
    cfg = devices.B200.to_config(Config(pointwise_block=512))
    assert cfg.pointwise_block == 512
    assert cfg.flops_per_byte == pytest.approx(devices.B200.fp32_flops / devices.B200.bandwidth)
    assert cfg.launch_overhead_bytes == pytest.approx(devices.B200.launch_s * devices.B200.bandwidth)
    # replaying a graph is cheaper than launching eagerly, so merging two kernels
    # only to save a launch is worth less with capture on
    assert cfg.effective_launch_bytes == cfg.graph_launch_overhead_bytes < cfg.launch_overhead_bytes


@pytest.mark.gpu
def test_calibration_measures_sane_constants():
    m = devices.calibrate("cuda:0", quick=True)
    assert m.source == "measured"
    assert 2e12 < m.bandwidth < 9e12
    assert 20e12 < m.fp32_flops < 120e12
    assert 0.2e-6 < m.graph_launch_s < 10e-6 and 0.5e-6 < m.launch_s < 60e-6
    assert "flops_per_byte" in devices.report(m, devices.B200)


# ---- the profile is wired into the reference (needs the reference) -----------------

import pathlib  # noqa: E402
import sys  # noqa: E402

sys.path.insert(0, str(pathlib.Path(__file__).resolve().parent.parent / "oracle"))
import ref as reference_copy  # noqa: E402

needs_reference = pytest.mark.skipif(reference_copy.path() is None, reason="reference not present")


def test_config_for_keeps_unknown_devices_on_the_defaults():
    base = Config(pointwise_block=256)
    assert devices.config_for("NVIDIA A40", base) is base
    cfg = devices.config_for("NVIDIA B200", base)
    assert cfg.pointwise_block == 256 and cfg.flops_per_byte == pytest.approx(devices.B200.flops_per_byte)


@needs_reference
def test_install_adds_the_b200_to_the_reference_device_table():
    reference_copy.activate()
    import mlc.devices as ref_devices
    import mlc_compiler_b200 as mb

    assert not any(k == "B200" for k, _ in ref_devices.TABLE)
    mb.install()
    try:
        key, prof = ref_devices.TABLE[0]
        assert key == "B200"
        cfg = prof.to_config()
        ours = devices.B200.to_config()
        assert cfg.flops_per_byte == pytest.approx(ours.flops_per_byte)
        assert cfg.launch_overhead_bytes == pytest.approx(ours.launch_overhead_bytes)
        assert cfg.graph_launch_overhead_bytes == pytest.approx(ours.graph_launch_overhead_bytes)
        mb.install()                                   # idempotent
        assert sum(k == "B200" for k, _ in ref_devices.TABLE) == 1
    finally:
        mb.uninstall()
    assert not any(k == "B200" for k, _ in ref_devices.TABLE)


@needs_reference
@pytest.mark.parametrize("name,batch,dtype", [("encoder-block", 1, torch.float32),
                                              ("micro-layernorm", 8, torch.float16),
                                              ("micro-softmax", 8, torch.float16),
                                              ("micro-gelu", 8, torch.float16)])
def test_b200_cost_constants_leave_the_shipped_schedules_unchanged(name, batch, dtype):
    """The fusion and recompute decisions of the benchmark models are far from the
    margin: pricing them for a B200 (10.4 FLOP/B, 3.6 MB per captured launch)
    instead of the reference's A100 default (20 FLOP/B, 1.1 MB) yields the same
    kernels, byte for byte -- which is why one set of shipped schedules serves both.
    (``python -m mlc_compiler_b200.schedules.capture --check-profile`` runs the same
    comparison over every shipped configuration.)"""
    reference_copy.activate()
    from mlc_compiler_b200 import capture_schedule, kir, models

    model, inputs = models.build(name, batch, dtype=dtype)
    a = capture_schedule(model, inputs, Config())
    b = capture_schedule(model, inputs, devices.B200.to_config())
    assert kir.dumps(a) == kir.dumps(b)
    shipped = kir.dumps(__import__("mlc_compiler_b200").load_schedule(
        models.schedule_name(name, batch, dtype)))
    fresh = kir.loads(kir.dumps(b))
    assert [k.summary() for k in fresh.kernels] == [k.summary() for k in kir.loads(shipped).kernels]


@needs_reference
def test_cuda_probe_takes_the_place_of_the_reference_triton_probe():
    reference_copy.activate()
    import mlc_compiler_b200 as mb

    assert devices.use_cuda_probe_in_reference()
    import mlc.bench.calibrate as cal

    assert cal.measure_fp32_throughput is devices.measure_fp32_throughput
    mb.install()
    mb.uninstall()                                   # restores the reference's own probe
    assert cal.measure_fp32_throughput is not devices.measure_fp32_throughput


@pytest.mark.gpu
@needs_reference
def test_reference_calibration_runs_on_the_cuda_probe():
    """``mlc.bench.calibrate.calibrate`` -- the reference's own routine -- with its
    fp32 probe replaced: all four constants measured, none taken from the table."""
    reference_copy.activate()
    import mlc_compiler_b200 as mb

    mb.install()
    try:
        assert devices.use_cuda_probe_in_reference()
        import mlc.bench.calibrate as cal

        prof = cal.calibrate("cuda:0", quick=True)
        assert prof.source == "measured"
        assert 20e12 < prof.fp32_flops < 120e12
        assert 2e12 < prof.bandwidth < 9e12
        cfg = prof.to_config()
        assert 3 < cfg.flops_per_byte < 40
    finally:
        mb.uninstall()
