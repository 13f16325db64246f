"""Graph-branch planning: physical dependencies, level ordering, relaxed arena."""

import itertools

import pytest

from conftest import load_tiny
from mlc_compiler_b200 import concurrency as C
from mlc_compiler_b200.frontend import load_schedule

NAMES = ["bert-base_b1_s128_float16", "gpt2-small_b1_s128_float16", "bert-base_b8_s128_float16"]


def _ancestors(deps):
    anc = []
    for j, ds in enumerate(deps):
        a = set()
        for p in ds:
            a |= anc[p] | {p}
        anc.append(a)
    return anc


@pytest.mark.parametrize("name", NAMES)
def test_every_physical_conflict_is_ordered(name):
    """Two kernels that touch the same bytes (one of them writing) are never
    left unordered, in the original order and after relaxation."""
    for s in (load_schedule(name), C.relax(load_schedule(name))):
        deps = C.dependencies(s)
        anc = _ancestors(deps)
        R = [C._ranges(s, k.reads()) for k in s.kernels]
        W = [C._ranges(s, k.writes()) for k in s.kernels]
        for i, j in itertools.combinations(range(len(s.kernels)), 2):
            if C._overlap(W[i], R[j]) or C._overlap(R[i], W[j]) or C._overlap(W[i], W[j]):
                assert i in anc[j], (s.kernels[i].name, s.kernels[j].name)


@pytest.mark.parametrize("name", NAMES)
def test_relaxed_schedule_keeps_kernels_and_respects_data_order(name):
    s = load_schedule(name)
    r = C.relax(s)
    assert sorted(k.name for k in r.kernels) == sorted(k.name for k in s.kernels)
    written = set(s.params) | {v.buffer for v in s.inputs}
    for k in r.kernels:                      # every read is of something already produced
        assert all(b in written for b in k.reads()), k.name
        written |= set(k.writes())
    assert r.arena_bytes % 256 == 0 and all(o % 256 == 0 for o in r.plan.offsets.values())
    assert set(r.plan.offsets) == set(s.plan.offsets)


def test_bert_projections_become_parallel_branches():
    s = load_schedule("bert-base_b1_s128_float16")
    serial = C.critical_path(C.dependencies(s))
    relaxed = C.relax(s)
    deps = C.dependencies(relaxed)
    assert C.critical_path(deps) <= serial - 40       # 2 of 3 projections per layer leave the chain
    plan = C.assign_streams(deps, 4)
    assert plan.forked >= 40 and max(plan.stream) <= 3
    for j, ws in enumerate(plan.waits):               # waits only ever look backwards
        assert all(p < j and plan.stream[p] != plan.stream[j] and p in plan.signals for p in ws)


def test_single_stream_plan_is_the_serial_chain():
    s = load_schedule("gpt2-small_b1_s128_float16")
    plan = C.assign_streams(C.dependencies(s), 1)
    assert plan.forked == 0 and not any(plan.waits)


def test_eager_schedules_are_left_alone():
    s = load_tiny("block__no_fusion__float32")["schedule"]
    assert C.relax(s) is s
