"""Dependency analysis of a schedule and assignment of kernels to capture streams.

The reference captures its launch sequence on one stream, so the CUDA graph is
a chain: 200 nodes for BERT-base, each waiting for the one before
(``mlc/runtime/executor.py:286-307``).  At batch 1 every node is latency-bound
and the chain *is* the latency.  Many neighbours in the chain are independent,
though -- the query, key and value projections of a layer with their bias
kernels, the three embedding gathers, the mask kernel -- and a graph with
forked branches lets the hardware overlap them.

Kernels are kept exactly as scheduled (same cuBLAS calls, same generated
kernels, same arena); only the edges of the graph change.  Because planned
buffers share arena bytes, dependencies are computed on *physical* byte ranges,
not buffer names: kernel j must follow every earlier kernel that wrote a range
j reads (RAW), read a range j writes (WAR) or wrote a range j writes (WAW).
That makes any execution order consistent with the edges equivalent to the
serial order, including with respect to arena reuse.
"""

from __future__ import annotations

from dataclasses import dataclass, field

from . import kir

Range = tuple[str, int, int]  # (space, begin, end): "arena" or a buffer name


def _ranges(schedule: kir.Schedule, names) -> list[Range]:
    offsets = schedule.plan.offsets if schedule.plan.mode == "arena" else {}
    out = []
    for n in names:
        spec = schedule.buffers[n]
        off = offsets.get(n) if spec.plannable else None
        if off is None:
            out.append((n, 0, max(1, spec.nbytes)))
        else:
            out.append(("arena", off, off + max(1, spec.nbytes)))
    return out


def _overlap(a: list[Range], b: list[Range]) -> bool:
    for sa, lo_a, hi_a in a:
        for sb, lo_b, hi_b in b:
            if sa == sb and lo_a < hi_b and lo_b < hi_a:
                return True
    return False


def dependencies(schedule: kir.Schedule) -> list[list[int]]:
    """For every kernel, the indices of the earlier kernels it must wait for,
    transitively reduced (a predecessor implied by another one is dropped)."""
    reads = [_ranges(schedule, k.reads()) for k in schedule.kernels]
    writes = [_ranges(schedule, k.writes()) for k in schedule.kernels]
    n = len(schedule.kernels)
    ancestors = [0] * n          # bitsets
    deps: list[list[int]] = []
    for j in range(n):
        direct = []
        for i in range(j - 1, -1, -1):
            if (_overlap(writes[i], reads[j]) or _overlap(reads[i], writes[j])
                    or _overlap(writes[i], writes[j])):
                direct.append(i)
        keep, covered = [], 0
        for i in direct:                      # latest first
            if not (covered >> i) & 1:
                keep.append(i)
                covered |= ancestors[i] | (1 << i)
        ancestors[j] = covered
        deps.append(sorted(keep))
    return deps


@dataclass
class StreamPlan:
    """Which capture stream each kernel goes to and which earlier kernels it has
    to wait for across streams."""

    stream: list[int]
    waits: list[list[int]]                      # cross-stream predecessors per kernel
    signals: set[int] = field(default_factory=set)  # kernels that need a completion event
    n_streams: int = 1

    @property
    def forked(self) -> int:
        return sum(1 for s in self.stream if s != 0)


def assign_streams(deps: list[list[int]], n_streams: int) -> StreamPlan:
    """Greedy list scheduling in schedule order.  A kernel continues the stream
    of a predecessor that is still that stream's tail (stream 0 preferred);
    otherwise it takes the stream that has been idle longest.  Placing a kernel
    behind an unrelated tail only adds an ordering, never removes one."""
    n = len(deps)
    n_streams = max(1, n_streams)
    tail = [-1] * n_streams                    # last kernel placed on each stream
    stream = [0] * n
    waits: list[list[int]] = [[] for _ in range(n)]
    signals: set[int] = set()
    for j in range(n):
        cands = [stream[p] for p in deps[j] if tail[stream[p]] == p]
        if cands:
            s = 0 if 0 in cands else cands[0]
        elif not deps[j] and tail[0] == -1:
            s = 0
        else:
            # no predecessor is a tail: fork.  Prefer an unused stream, then the
            # one whose tail is oldest (least likely to still be running).
            s = min(range(n_streams), key=lambda t: tail[t])
        stream[j] = s
        for p in deps[j]:
            if stream[p] != s:
                waits[j].append(p)
                signals.add(p)
        tail[s] = j
    return StreamPlan(stream, waits, signals, n_streams)


def critical_path(deps: list[list[int]], cost: list[float] | None = None) -> float:
    """Length of the longest dependency chain (unit cost per kernel by default):
    a lower bound on the number of serial launch latencies."""
    n = len(deps)
    cost = cost or [1.0] * n
    dist = [0.0] * n
    for j in range(n):
        dist[j] = cost[j] + max((dist[p] for p in deps[j]), default=0.0)
    return max(dist, default=0.0)


# --------------------------------------------------------------------------
# exposing the concurrency the serial plan hides
# --------------------------------------------------------------------------

def data_levels(schedule: kir.Schedule) -> list[int]:
    """Level of each kernel in the *data* dependency DAG (by buffer name, arena
    aliasing ignored): 0 for kernels that read only parameters and inputs,
    otherwise one more than the deepest producer (or earlier reader/writer of a
    buffer it overwrites)."""
    last_writer: dict[str, int] = {}
    readers: dict[str, list[int]] = {}
    level: list[int] = []
    for j, k in enumerate(schedule.kernels):
        lv = 0
        for b in k.reads():
            if b in last_writer:
                lv = max(lv, level[last_writer[b]] + 1)
        for b in k.writes():
            if b in last_writer:
                lv = max(lv, level[last_writer[b]] + 1)
            for r in readers.get(b, ()):
                lv = max(lv, level[r] + 1)
        level.append(lv)
        for b in k.reads():
            readers.setdefault(b, []).append(j)
        for b in k.writes():
            last_writer[b] = j
            readers[b] = []
    return level


def _align(n: int, to: int = 256) -> int:
    return (n + to - 1) // to * to


def relax(schedule: kir.Schedule) -> kir.Schedule:
    """A schedule with the same kernels, ordered by data level, and an arena
    re-packed so that buffers of kernels which may now overlap in time do not
    share bytes.

    The packing is the reference planner's (``mlc/passes/memory_planning.py:
    92-175``: live range per buffer, largest first, lowest offset that clears
    every conflicting buffer already placed, 256-byte alignment), with live
    ranges measured in levels instead of schedule positions: a buffer is live
    from its writer's level to its last reader's level, inclusive, and graph
    outputs stay live to the end.  Unplanned (eager) schedules are returned
    unchanged.
    """
    if schedule.plan.mode != "arena":
        return schedule
    level = data_levels(schedule)
    order = sorted(range(len(schedule.kernels)), key=lambda j: (level[j], j))
    out = kir.Schedule(name=schedule.name, kernels=[schedule.kernels[j] for j in order],
                       buffers=schedule.buffers, inputs=schedule.inputs,
                       outputs=schedule.outputs, params=schedule.params, meta=dict(schedule.meta))
    first: dict[str, int] = {}
    last: dict[str, int] = {}
    for j, k in enumerate(schedule.kernels):
        for b in k.writes():
            first.setdefault(b, level[j])
            last[b] = max(last.get(b, level[j]), level[j])
        for b in k.reads():
            last[b] = max(last.get(b, level[j]), level[j])
    horizon = max(level, default=0) + 1
    for v in schedule.outputs:
        last[v.buffer] = horizon
    ranges = []
    for name, spec in schedule.buffers.items():
        if spec.plannable and name in first and name in schedule.plan.offsets:
            ranges.append((name, first[name], last.get(name, first[name]), _align(spec.nbytes)))
    placed: list[tuple[int, tuple]] = []
    offsets: dict[str, int] = {}
    total = 0
    for r in sorted(ranges, key=lambda r: (-r[3], r[1], r[0])):
        name, lo, hi, size = r
        conflicts = sorted((off, p) for off, p in placed if not (p[2] < lo or hi < p[1]))
        offset = 0
        for off, p in conflicts:
            if off >= offset + size:
                break
            offset = max(offset, _align(off + p[3]))
        offsets[name] = offset
        placed.append((offset, r))
        total = max(total, offset + size)
    # two buffers live at a common level never share a byte
    for i, (oa, a) in enumerate(placed):
        for ob, b in placed[i + 1:]:
            if not (a[2] < b[1] or b[2] < a[1]) and oa < ob + b[3] and ob < oa + a[3]:
                raise AssertionError(f"relaxed arena overlaps {a[0]} and {b[0]}")
    peak = 0
    for lv in range(horizon + 1):
        peak = max(peak, sum(r[3] for r in ranges if r[1] <= lv <= r[2]))
    out.plan = kir.ArenaPlan(mode="arena", arena_bytes=total, offsets=offsets, peak_bytes=peak,
                             total_bytes=schedule.plan.total_bytes)
    return out
