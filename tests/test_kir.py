"""Kernel IR: JSON round trip, index arithmetic, shipped schedules."""

import itertools

import pytest

from conftest import load_tiny, tiny_cases
from mlc_compiler_b200 import kir
from mlc_compiler_b200.frontend import SCHEDULE_DIR, load_schedule


@pytest.mark.parametrize("stem", tiny_cases()[::3])
def test_json_round_trip(stem):
    s = load_tiny(stem)["schedule"]
    text = kir.dumps(s)
    assert kir.dumps(kir.loads(text)) == text


def test_special_constants_survive():
    for v in (float("inf"), float("-inf"), 1e-12, -3.4028234663852886e+38, 0.1):
        e = kir.Call("add", (kir.Load(0), kir.Const(v)))
        back = kir._dec_expr(kir._enc_expr(e))
        assert back == e
    nan = kir._dec_expr(kir._enc_expr(kir.Const(float("nan"))))
    assert nan.value != nan.value


def test_index_offsets_match_definition():
    ax = kir.Axis("idx", 98304, ((128, 768, 64), (12, 64, 8192), (64, 1, 1)))
    m = kir.IndexMap((ax,), 5)
    for i in (0, 1, 63, 64, 767, 768, 98303):
        want = 5 + (i // 768 % 128) * 64 + (i // 64 % 12) * 8192 + (i % 64)
        assert m.offset(idx=i) == want
    lo, hi = m.bounds()
    assert lo == 5 and hi == 5 + 127 * 64 + 11 * 8192 + 63


def test_shipped_schedules_load_and_have_expected_shape():
    names = sorted(p.name[:-8] for p in SCHEDULE_DIR.glob("*.json.gz"))
    assert "bert-base_b1_s128_float16" in names and "gpt2-small_b1_s128_float16" in names
    bert = load_schedule("bert-base_b1_s128_float16")
    # the composition the reference publishes for BERT-base at batch 1
    assert bert.counts() == {"extern": 100, "pointwise": 63, "reduction": 37}
    gpt = load_schedule("gpt2-small-ref_b1_s128_float16")
    assert gpt.counts() == {"extern": 75, "reduction": 37, "pointwise": 36}
    for s in (bert, gpt):
        assert s.plan.mode == "arena" and s.arena_bytes % 256 == 0
        for off in s.plan.offsets.values():
            assert off % 256 == 0


def test_arena_plan_never_overlaps_live_buffers():
    """Two planned buffers alive at the same kernel never share a byte."""
    s = load_schedule("bert-base_b1_s128_float16")
    first, last = {}, {}
    for i, k in enumerate(s.kernels):
        for b in k.writes():
            first.setdefault(b, i)
            last[b] = max(last.get(b, i), i)
        for b in k.reads():
            last[b] = max(last.get(b, i), i)
    planned = [b for b in s.plan.offsets if b in first]
    for a, b in itertools.combinations(planned, 2):
        if last[a] < first[b] or last[b] < first[a]:
            continue
        oa, ob = s.plan.offsets[a], s.plan.offsets[b]
        na, nb = s.buffers[a].nbytes, s.buffers[b].nbytes
        assert oa + na <= ob or ob + nb <= oa, (a, b)
