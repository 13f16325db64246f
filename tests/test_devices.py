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
