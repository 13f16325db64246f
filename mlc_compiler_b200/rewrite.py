"""Schedule rewrites applied by the executor before code generation.

``forward_into_consumers`` removes a class of kernels the reference's fusion
pass cannot: a pointwise producer whose only readers are pointwise kernels that
read it *at a different index* -- typically ``mm + bias`` over ``[B*T, D]``
followed, at batch > 1, by the ``clone`` that lays the heads out as
``[B, H, T, D/H]`` (or transposed for K).  The reference refuses to fuse them
because one iteration would need a value another iteration computed
(``reads_are_local``, ``mlc/lower.py:117-155``), and so launches the bias kernel,
writes ``[B*T, D]``, and reads it straight back in the copy.  Every element of
the producer is independent, however, so the consumer can simply *recompute*
the producer's expression at the index it wants: compose the consumer's read
map with each producer operand's map, inline the body, drop the producer.  The
copy then reads the matmul output directly and the intermediate buffer is never
written (36 launches and 36 round trips through memory fewer per BERT-base
forward at batch > 1).  Results are bit-identical: the inlined value is rounded
to the intermediate's dtype exactly where the store used to round it.

Composition is done on the ``(size, out_stride, in_stride)`` terms.  The
consumer's map turns its index into digits ``d_k`` with weights ``s_k``
(``x = base + sum d_k s_k``); a producer operand's term ``((x / o) % n) * s``
selects the digits whose weight lies in ``[o, o n)``.  When every digit falls
wholly inside, below or above that window (and the base cannot carry across
it) the composite is again a list of terms; otherwise the rewrite is skipped
for that producer.
"""

from __future__ import annotations

import math

from . import kir
from .kir import Call, Cast, Load, Ref


class _NoCompose(Exception):
    pass


def compose(outer: kir.IndexMap, inner: kir.IndexMap, inner_numel: int) -> kir.IndexMap:
    """Map ``idx_c -> inner(outer(idx_c))`` where ``outer`` yields a position in
    the producer's flat iteration space and ``inner`` is one of its operands."""
    if len(outer.axes) != 1 or len(inner.axes) > 1:
        raise _NoCompose
    ax = outer.axes[0]
    digits = sorted(ax.terms, key=lambda t: t[2])
    reach = 0
    for n, _, s in digits:                       # non-overlapping mixed radix
        if s <= 0 or s < reach:
            raise _NoCompose
        reach = s * n
    new_terms: list[tuple[int, int, int]] = []
    base = inner.base
    terms = inner.axes[0].terms if inner.axes else ()
    for n, o, s in terms:
        top = o * n
        modulo = top != inner_numel              # the outermost term carries no '%'
        low_max = outer.base % o
        mid = outer.base // o
        mid = mid % n if modulo else mid
        inside_max = mid
        for nk, ok, sk in digits:
            if sk * nk <= o:
                low_max += (nk - 1) * sk
            elif sk % o == 0 and (not modulo or sk * nk <= top):
                new_terms.append((nk, ok, (sk // o) * s))
                inside_max += (nk - 1) * (sk // o)
            elif modulo and sk % top == 0:
                continue
            else:
                raise _NoCompose
        if low_max >= o or (modulo and inside_max >= n):
            raise _NoCompose
        base += mid * s
    new_terms = [t for t in new_terms if t[2] != 0]
    new_terms.sort(key=lambda t: -t[1])
    return kir.IndexMap((kir.Axis(ax.var, ax.numel, tuple(new_terms)),), base)


def _rename(e, prefix: str, slot_map: dict[int, int]):
    if isinstance(e, Load):
        return Load(slot_map[e.slot])
    if isinstance(e, Ref):
        return Ref(prefix + e.name)
    if isinstance(e, Call):
        return Call(e.fn, tuple(_rename(a, prefix, slot_map) for a in e.args))
    if isinstance(e, Cast):
        return Cast(_rename(e.x, prefix, slot_map), e.dtype)
    return e


def _identity_output(k: kir.PointwiseKernel) -> bool:
    if len(k.outputs) != 1:
        return False
    m = k.outputs[0].index
    return (m.base == 0 and len(m.axes) == 1
            and m.axes[0].terms in (((k.numel, 1, 1),), ()) and (k.numel > 1 or not m.axes[0].terms))


def _next_prefix(consumer: kir.PointwiseKernel) -> int:
    used = {nm.split("_", 1)[0] for nm, _ in consumer.body if nm.startswith("f") and "_" in nm}
    n = 0
    while f"f{n}" in used:
        n += 1
    return n


def _inline(producer: kir.PointwiseKernel, consumer: kir.PointwiseKernel):
    """``consumer`` with every read of the producer's buffer replaced by the
    producer's expression; raises ``_NoCompose`` when a map does not compose."""
    x = producer.outputs[0]
    inputs = list(consumer.inputs)
    body: list[tuple[str, object]] = []
    replace: dict[int, object] = {}
    drop: list[int] = []
    n = _next_prefix(consumer)
    for j, arg in enumerate(consumer.inputs):
        if arg.buffer != x.buffer:
            continue
        prefix = f"f{n}_"
        n += 1
        slot_map: dict[int, int] = {}
        for i, a in enumerate(producer.inputs):
            m = compose(arg.index, a.index, producer.numel)
            for q, have in enumerate(inputs):
                if have.buffer == a.buffer and have.dtype == a.dtype and have.index == m and q not in drop:
                    slot_map[i] = q
                    break
            else:
                inputs.append(kir.Operand(a.name, a.buffer, a.dtype, m))
                slot_map[i] = len(inputs) - 1
        for name, e in producer.body:
            body.append((prefix + name, _rename(e, prefix, slot_map)))
        value = _rename(producer.out_expr[x.name], prefix, slot_map)
        # what the consumer used to load: the value rounded to the buffer's dtype,
        # widened again if that dtype is a narrow float
        value = Cast(value, x.dtype)
        if x.dtype in kir.NARROW_FLOATS:
            value = Cast(value, "float32")
        replace[j] = value
        drop.append(j)
    if not drop:
        return consumer
    # renumber the remaining loads
    keep = [q for q in range(len(inputs)) if q not in drop]
    renum = {old: new for new, old in enumerate(keep)}

    def fix(e):
        if isinstance(e, Load):
            if e.slot in replace:
                return fix(replace[e.slot])
            return Load(renum[e.slot])
        if isinstance(e, Call):
            return Call(e.fn, tuple(fix(a) for a in e.args))
        if isinstance(e, Cast):
            return Cast(fix(e.x), e.dtype)
        return e

    new_body = [(nm, fix(e)) for nm, e in body] + [(nm, fix(e)) for nm, e in consumer.body]
    out_expr = {nm: fix(e) for nm, e in consumer.out_expr.items()}
    return kir.PointwiseKernel(consumer.name, consumer.space, [inputs[q] for q in keep],
                               list(consumer.outputs), new_body, out_expr,
                               list(producer.ops) + list(consumer.ops))


def forward_into_consumers(schedule: kir.Schedule, max_body: int = 32,
                           max_consumers: int = 4, replan: bool = True) -> kir.Schedule:
    """Inline eligible pointwise producers into their pointwise consumers and
    drop them.  Returns a new schedule (kernels keep their names; the dropped
    producer's buffer stays in the table, unused).

    A consumer now reads the producer's operands, which the original arena plan
    considered dead by then.  With ``replan`` the arena is re-packed afterwards
    from the new live ranges (``concurrency.relax``); without it a producer is
    only forwarded when no kernel up to its last consumer reuses its operands'
    bytes."""
    kernels = list(schedule.kernels)
    outputs = {v.buffer for v in schedule.outputs}
    changed = True
    while changed:
        changed = False
        for pi, p in enumerate(kernels):
            if not isinstance(p, kir.PointwiseKernel) or not _identity_output(p):
                continue
            x = p.outputs[0]
            if x.buffer in outputs or not schedule.buffers[x.buffer].plannable:
                continue
            if len(p.body) > max_body or x.buffer in p.reads():
                continue
            readers = [ci for ci, c in enumerate(kernels) if ci != pi and x.buffer in c.reads()]
            writers = [ci for ci, c in enumerate(kernels) if ci != pi and x.buffer in c.writes()]
            if not readers or writers or len(readers) > max_consumers or min(readers) < pi:
                continue
            if not all(isinstance(kernels[ci], kir.PointwiseKernel) for ci in readers):
                continue
            # never make a consumer move more bytes than the load it replaces
            heavy = sum(min(a.index.distinct_elements(), p.numel) * kir.ITEMSIZE[a.dtype]
                        for a in p.inputs)
            if heavy > schedule.buffers[x.buffer].nbytes + 65536:
                continue
            # a producer operand must still hold the same data when the consumer runs
            stable = True
            for a in p.inputs:
                for ci in range(pi + 1, max(readers) + 1):
                    if a.buffer in kernels[ci].writes():
                        stable = False
            if not stable or (not replan and _arena_clobbered(schedule, kernels, p, pi, max(readers))):
                continue
            try:
                new = {ci: _inline(p, kernels[ci]) for ci in readers}
            except _NoCompose:
                continue
            for ci, c in new.items():
                kernels[ci] = c
            del kernels[pi]
            changed = True
            break
    if len(kernels) == len(schedule.kernels):
        return schedule
    out = kir.Schedule(name=schedule.name, kernels=kernels, buffers=schedule.buffers,
                       inputs=schedule.inputs, outputs=schedule.outputs, params=schedule.params,
                       plan=schedule.plan, meta=dict(schedule.meta))
    return _replanned(out) if replan else out


def _arena_clobbered(schedule, kernels, p, pi: int, last_reader: int) -> bool:
    """True when the arena bytes of one of the producer's operands are reused by a
    kernel that runs before the last consumer: reading the operand later would
    then see someone else's data."""
    if schedule.plan.mode != "arena":
        return False
    off = schedule.plan.offsets

    def span(b):
        if b in off and schedule.buffers[b].plannable:
            return off[b], off[b] + schedule.buffers[b].nbytes
        return None

    for a in p.inputs:
        sa = span(a.buffer)
        if sa is None:
            continue
        for ci in range(pi + 1, last_reader + 1):
            for b in kernels[ci].writes():
                sb = span(b)
                if sb is not None and b != a.buffer and sa[0] < sb[1] and sb[0] < sa[1]:
                    return True
    return False


# --------------------------------------------------------------------------
# copies after an extern: let the extern write the copy's layout itself
# --------------------------------------------------------------------------

#: externs whose ``out=`` may be any strided matrix (cuBLAS takes a leading
#: dimension and a batch stride, so ATen hands such a destination straight on)
_STRIDED_OUT = ("aten.mm.default", "aten.bmm.default", "aten.addmm.default")


def _pure_copy(k) -> bool:
    if not isinstance(k, kir.PointwiseKernel) or len(k.inputs) != 1 or len(k.outputs) != 1:
        return False
    e = k.out_expr[k.outputs[0].name]
    # widening and back is the identity; float64 -> float32 -> float64 is not
    while isinstance(e, Cast) and k.inputs[0].dtype in kir.FLOAT_DTYPES and (
            e.dtype == k.inputs[0].dtype
            or (e.dtype == "float32" and k.inputs[0].dtype in ("float16", "bfloat16", "float32"))):
        e = e.x
    return (not k.body and isinstance(e, Load) and k.inputs[0].dtype == k.outputs[0].dtype
            and k.inputs[0].buffer != k.outputs[0].buffer)


def _destination_strides(view: kir.View, copy: kir.PointwiseKernel) -> tuple[int, ...] | None:
    """Strides ``T`` such that element ``i`` of the extern's (dense) result lands
    where the copy would have put it: ``dst[sum i_j T_j] = src[sum i_j S_j]``.
    Exists when every dimension of the result is exactly one digit of the copy's
    read map; a dimension the copy splits into two digits with unrelated
    destination strides (heads and batch at batch > 1) has no single stride."""
    src, dst = copy.inputs[0].index, copy.outputs[0].index
    n = view.numel
    if (src.base or dst.base or len(src.axes) != 1 or len(dst.axes) != 1 or copy.numel != n
            or dst.axes[0].terms != ((n, 1, 1),) or view.offset != 0):
        return None
    digits = {s: (size, o) for size, o, s in src.axes[0].terms}
    if len(digits) != len(src.axes[0].terms) or math.prod(z for z, _ in digits.values()) != n:
        return None
    strides = []
    used = 0
    for size, s in zip(view.shape, view.strides):
        if size == 1:
            strides.append(s)
            continue
        if digits.get(s, (0, 0))[0] != size:
            return None
        strides.append(digits[s][1])
        used += 1
    return tuple(strides) if used == len(digits) else None


def write_through_copies(schedule: kir.Schedule, replan: bool = True) -> kir.Schedule:
    """Drop a pure copy that only re-lays an extern's result, by handing the
    extern the copy's layout as its strided ``out=``.

    At batch 1 the context matmul produces ``[H, T, D/H]`` and a ``clone``
    permutes it to ``[T, H, D/H]`` for the output projection: one launch per
    layer that moves no information.  ``bmm`` writes any matrix layout with a
    leading dimension and a batch stride, so it can store ``[H, T, D/H]`` with
    strides ``(D/H, D, 1)`` directly into the clone's buffer.  Values are
    unchanged (a copy is exact); the op and its inputs are unchanged.  At
    batch > 1 the clone splits the batched-heads dimension in two and no
    strided view expresses it, so the copy stays."""
    kernels = list(schedule.kernels)
    finals = {v.buffer for v in schedule.outputs}
    dropped = False
    for ei in range(len(kernels)):
        e = kernels[ei]
        if not isinstance(e, kir.ExternKernel) or e.op not in _STRIDED_OUT or len(e.outputs) != 1:
            continue
        x = e.outputs[0]
        spec = schedule.buffers[x.buffer]
        if x.buffer in finals or not spec.plannable or x.numel != spec.numel:
            continue
        if any(s != d for s, d in zip(x.strides, _dense_strides(x.shape))):
            continue
        touching = [ci for ci, c in enumerate(kernels)
                    if ci != ei and c is not None and (x.buffer in c.reads() or x.buffer in c.writes())]
        if len(touching) != 1 or touching[0] < ei or not _pure_copy(kernels[touching[0]]):
            continue
        ci = touching[0]
        c = kernels[ci]
        y = c.outputs[0]
        strides = _destination_strides(x, c)
        if strides is None or x.buffer in e.reads() or y.buffer in e.reads():
            continue
        # the destination must not be touched between the extern and the copy
        if any(k is not None and (y.buffer in k.reads() or y.buffer in k.writes())
               for k in kernels[ei + 1:ci]):
            continue
        # ATen wants a matrix it can give cuBLAS: unit stride on one of the last two
        # dimensions, the other at least as long as the row it steps over
        if not _blas_layout(x.shape, strides):
            continue
        kernels[ei] = kir.ExternKernel(e.name, e.op, e.args, e.kwargs,
                                       [kir.View(y.name, y.buffer, x.shape, strides, 0)])
        kernels[ci] = None
        dropped = True
    if not dropped:
        return schedule
    out = kir.Schedule(name=schedule.name, kernels=[k for k in kernels if k is not None],
                       buffers=schedule.buffers, inputs=schedule.inputs, outputs=schedule.outputs,
                       params=schedule.params, plan=schedule.plan, meta=dict(schedule.meta))
    return _replanned(out) if replan else out


def _dense_strides(shape) -> tuple[int, ...]:
    out, run = [], 1
    for n in reversed(shape):
        out.append(run)
        run *= n
    return tuple(reversed(out))


def _blas_layout(shape, strides) -> bool:
    if len(shape) < 2:
        return False
    (m, n), (sm, sn) = shape[-2:], strides[-2:]
    return (sn == 1 and sm >= max(1, n)) or (sm == 1 and sn >= max(1, m))


def _replanned(out: kir.Schedule) -> kir.Schedule:
    from .concurrency import relax

    live = out.live_buffers()
    out.plan = kir.ArenaPlan(out.plan.mode, out.plan.arena_bytes,
                             {b: o for b, o in out.plan.offsets.items() if b in live},
                             out.plan.peak_bytes, out.plan.total_bytes,
                             out.plan.alloc_at, out.plan.free_at)
    return relax(out)


# --------------------------------------------------------------------------
# bias epilogue (opt-in: it changes how a matmul is dispatched)
# --------------------------------------------------------------------------

def _col_only(m: kir.IndexMap, n_cols: int, var: str) -> bool:
    """``m`` reads element ``column`` of a length-``n_cols`` vector."""
    if m.base != 0:
        return False
    terms = [t for a in m.axes for t in a.terms]
    if len(terms) != 1 or terms[0] != (n_cols, 1, 1):
        return False
    return all(a.var == var or not a.terms for a in m.axes)


def _row_major(m: kir.IndexMap, rows: int, cols: int) -> bool:
    """``m`` addresses a contiguous ``[rows, cols]`` matrix at ``(row, column)``."""
    if m.base != 0:
        return False
    if len(m.axes) == 1:                                   # flat idx
        return m.axes[0].terms == ((rows * cols, 1, 1),)
    by = {a.var: a.terms for a in m.axes}
    return by.get("row") == ((rows, 1, cols),) and by.get("col") == ((cols, 1, 1),)


def _strip_bias_add(e, x_slot: int, b_slot: int):
    """``e`` with the first ``add(Load(x), Load(b))`` (either order) replaced by
    ``Load(x)``; returns ``(new expression, replaced?)``."""
    if isinstance(e, Call):
        if e.fn == "add" and len(e.args) == 2 and all(isinstance(a, Load) for a in e.args) \
                and {e.args[0].slot, e.args[1].slot} == {x_slot, b_slot}:
            return Load(x_slot), True
        out, hit = [], False
        for a in e.args:
            if hit:
                out.append(a)
            else:
                na, hit = _strip_bias_add(a, x_slot, b_slot)
                out.append(na)
        return Call(e.fn, tuple(out)), hit
    if isinstance(e, Cast):
        x, hit = _strip_bias_add(e.x, x_slot, b_slot)
        return Cast(x, e.dtype), hit
    return e, False


def _drop_slot(k, slot: int):
    """Kernel ``k`` without input ``slot`` (which nothing reads any more)."""
    renum = {old: new for new, old in enumerate(i for i in range(len(k.inputs)) if i != slot)}

    def fix(e):
        if isinstance(e, Load):
            return Load(renum[e.slot])
        if isinstance(e, Call):
            return Call(e.fn, tuple(fix(a) for a in e.args))
        if isinstance(e, Cast):
            return Cast(fix(e.x), e.dtype)
        return e

    inputs = [a for i, a in enumerate(k.inputs) if i != slot]
    out_expr = {n: fix(e) for n, e in k.out_expr.items()}
    if isinstance(k, kir.PointwiseKernel):
        return kir.PointwiseKernel(k.name, k.space, inputs, list(k.outputs),
                                   [(n, fix(e)) for n, e in k.body], out_expr, list(k.ops))
    steps = [kir.Reduce(s.name, s.kind, fix(s.expr)) if isinstance(s, kir.Reduce)
             else kir.Bind(s.name, fix(s.expr)) for s in k.steps]
    return kir.ReductionKernel(k.name, k.row_space, k.reduce_space, inputs, list(k.outputs), steps,
                               out_expr, set(k.row_outputs), k.two_pass, list(k.ops))


def fold_bias_into_matmul(schedule: kir.Schedule) -> kir.Schedule:
    """Turn ``mm`` followed by a generated kernel that starts with ``+ bias`` into
    ``addmm`` (cuBLASLt bias epilogue) and remove the add from the kernel; a
    kernel that was *only* the bias add disappears and the matmul writes its
    output directly.

    Not applied by default: the matmul is then no longer dispatched as the
    reference dispatches it, and the bias is added to the fp32 accumulator
    before the single rounding instead of after a first rounding to the buffer
    dtype (a difference of at most one unit in the last place of fp16/bf16).
    """
    kernels = list(schedule.kernels)
    outputs = {v.buffer for v in schedule.outputs}
    i = 0
    changed = False
    while i < len(kernels):
        e = kernels[i]
        i += 1
        if not (isinstance(e, kir.ExternKernel) and e.op == "aten.mm.default" and not e.kwargs
                and len(e.args) == 2 and all(isinstance(a, kir.View) for a in e.args)
                and len(e.outputs) == 1):
            continue
        x = e.outputs[0]
        if x.buffer in outputs or len(x.shape) != 2 or x.offset != 0 \
                or tuple(x.strides) != (x.shape[1], 1):
            continue
        rows, cols = x.shape
        readers = [j for j, k in enumerate(kernels) if x.buffer in k.reads()]
        if len(readers) != 1 or readers[0] < i:
            continue
        j = readers[0]
        p = kernels[j]
        if isinstance(p, kir.ExternKernel):
            continue
        var = "idx" if isinstance(p, kir.PointwiseKernel) else "col"
        x_slots = [q for q, a in enumerate(p.inputs) if a.buffer == x.buffer]
        if len(x_slots) != 1 or not _row_major(p.inputs[x_slots[0]].index, rows, cols):
            continue
        xs = x_slots[0]
        done = False
        for bs, b in enumerate(p.inputs):
            spec = schedule.buffers[b.buffer]
            if bs == xs or spec.kind != "param" or spec.numel != cols or b.dtype != p.inputs[xs].dtype \
                    or not _col_only(b.index, cols, var):
                continue
            # the add must be the only use of both operands
            exprs = ([ex for _, ex in p.body] if isinstance(p, kir.PointwiseKernel)
                     else [s.expr for s in p.steps]) + list(p.out_expr.values())
            uses_x = sum(1 for ex in exprs for sub in kir.walk(ex)
                         if isinstance(sub, Load) and sub.slot == xs)
            uses_b = sum(1 for ex in exprs for sub in kir.walk(ex)
                         if isinstance(sub, Load) and sub.slot == bs)
            if uses_x != 1 or uses_b != 1:
                continue
            hit = False

            def strip(ex):
                nonlocal hit
                if hit:
                    return ex
                new, h = _strip_bias_add(ex, xs, bs)
                hit = hit or h
                return new

            if isinstance(p, kir.PointwiseKernel):
                body = [(n, strip(ex)) for n, ex in p.body]
                out_expr = {n: strip(ex) for n, ex in p.out_expr.items()}
                q = kir.PointwiseKernel(p.name, p.space, list(p.inputs), list(p.outputs), body,
                                        out_expr, list(p.ops))
            else:
                steps = [kir.Reduce(s.name, s.kind, strip(s.expr)) if isinstance(s, kir.Reduce)
                         else kir.Bind(s.name, strip(s.expr)) for s in p.steps]
                out_expr = {n: strip(ex) for n, ex in p.out_expr.items()}
                q = kir.ReductionKernel(p.name, p.row_space, p.reduce_space, list(p.inputs),
                                        list(p.outputs), steps, out_expr, set(p.row_outputs),
                                        p.two_pass, list(p.ops))
            if not hit:
                continue
            q = _drop_slot(q, bs)
            bias_view = kir.View(b.name, b.buffer, (cols,), (1,), 0)
            target = x
            # a kernel that was nothing but the bias add: let the matmul write its output
            if isinstance(q, kir.PointwiseKernel) and len(q.outputs) == 1 and len(q.inputs) == 1:
                o = q.outputs[0]
                sole = q.out_expr[o.name]
                while isinstance(sole, Ref):
                    sole = dict(q.body).get(sole.name, sole)
                    if isinstance(sole, Ref):
                        break
                plain = isinstance(sole, Load) or (isinstance(sole, Cast) and isinstance(sole.x, Load)
                                                   and sole.dtype == o.dtype)
                if plain and o.dtype == schedule.buffers[x.buffer].dtype \
                        and _row_major(o.index, rows, cols) and o.buffer not in outputs:
                    target = kir.View(o.name, o.buffer, (rows, cols), (cols, 1), 0)
                    q = None
            kernels[i - 1] = kir.ExternKernel(e.name, "aten.addmm.default",
                                              [bias_view, e.args[0], e.args[1]], {}, [target])
            if q is None:
                del kernels[j]
            else:
                kernels[j] = q
            changed = done = True
            break
        if not done:
            continue
    if not changed:
        return schedule
    from .concurrency import relax

    out = kir.Schedule(name=schedule.name, kernels=kernels, buffers=schedule.buffers,
                       inputs=schedule.inputs, outputs=schedule.outputs, params=schedule.params,
                       plan=schedule.plan, meta=dict(schedule.meta))
    if out.plan.mode == "arena":
        live = out.live_buffers()
        out.plan = kir.ArenaPlan(out.plan.mode, out.plan.arena_bytes,
                                 {b: o for b, o in out.plan.offsets.items() if b in live},
                                 out.plan.peak_bytes, out.plan.total_bytes)
        out = relax(out)
    return out


# --------------------------------------------------------------------------
# embeddings: gather the table row inside the kernel that consumes it
# --------------------------------------------------------------------------

def _constant_fill(k) -> int | None:
    """The integer a kernel fills its single output with, if that is all it does."""
    if (isinstance(k, kir.PointwiseKernel) and not k.inputs and _identity_output(k)):
        e = k.out_expr[k.outputs[0].name]
        while isinstance(e, Cast):
            e = e.x
        if isinstance(e, kir.Const) and isinstance(e.value, int) and not isinstance(e.value, bool):
            return int(e.value)
    return None


def _token_map(a: kir.Operand, width: int, rows: int):
    """For an operand that reads ``[tokens, width]`` rows whole (``col`` walks one
    row, ``row`` picks the token): the map ``row -> token`` as a one-axis map."""
    col, row = a.index.axis("col"), a.index.axis("row")
    if (a.index.base or len(a.index.axes) != 2 or col is None or row is None
            or col.terms != ((width, 1, 1),)):
        return None
    terms = []
    for size, o, s in row.terms:
        if s % width:
            return None
        terms.append((size, o, s // width))
    return kir.IndexMap((kir.Axis("row", rows, tuple(terms)),))


def fold_embeddings(schedule: kir.Schedule, replan: bool = True) -> kir.Schedule:
    """Drop ``aten.embedding`` calls whose result only feeds row reductions, by
    letting the reduction fetch the table row itself.

    BERT's embedding LayerNorm reads three ``[tokens, D]`` arrays that three
    library gathers have just written (word, position and token-type rows; the
    token-type ids come from a ``full_like(0)`` kernel); GPT-2's first LayerNorm
    reads two.  A row reduction already loads each row as ``base + row_offset +
    col``: taking ``row_offset`` from ``table_row[ids[row]]`` instead of from the
    row number costs one 8-byte load per row and removes the gather, its launch
    and the round trip of ``tokens x D`` elements through memory.  Ids that a
    kernel fills with a constant become a plain broadcast row of the table and
    the fill disappears as well.  The values read are the same table entries, so
    results are bit-identical; an id outside the table reads a clamped row where
    the library call would have raised a device assertion."""
    kernels: list = list(schedule.kernels)
    finals = {v.buffer for v in schedule.outputs}
    changed = False
    for ei, e in enumerate(kernels):
        if not isinstance(e, kir.ExternKernel) or e.op != "aten.embedding.default":
            continue
        if len(e.args) < 2 or len(e.outputs) != 1:
            continue
        table, ids, x = e.args[0], e.args[1], e.outputs[0]
        if not (isinstance(table, kir.View) and isinstance(ids, kir.View)):
            continue
        if len(table.shape) != 2 or table.strides != (table.shape[1], 1) or table.shape[1] < 2:
            continue
        n_table, width = table.shape
        spec = schedule.buffers[x.buffer]
        if (x.buffer in finals or not spec.plannable or x.offset or x.numel != spec.numel
                or x.strides != _dense_strides(x.shape) or x.numel != ids.numel * width):
            continue
        if schedule.buffers[ids.buffer].dtype not in ("int64", "int32"):
            continue
        users = [ci for ci, c in enumerate(kernels) if c is not None and ci != ei
                 and (x.buffer in c.reads() or x.buffer in c.writes())]
        if not users or min(users) < ei or not all(
                isinstance(kernels[ci], kir.ReductionKernel) and x.buffer not in kernels[ci].writes()
                for ci in users):
            continue
        # ids and table must still hold the same data when the last consumer runs
        if any(c is not None and (ids.buffer in c.writes() or table.buffer in c.writes())
               for c in kernels[ei + 1:max(users) + 1]):
            continue
        fill = None
        writers = [c for c in kernels[:ei] if c is not None and ids.buffer in c.writes()]
        if len(writers) == 1:
            fill = _constant_fill(writers[0])
            if fill is not None and writers[0].numel != schedule.buffers[ids.buffer].numel:
                fill = None
        # token t of the ids view -> element of the ids buffer
        dims: list[list[int]] = []                 # innermost first, dense neighbours merged
        for size, stride in zip(reversed(ids.shape), reversed(ids.strides)):
            if size == 1:
                continue
            if dims and stride == dims[-1][0] * dims[-1][1]:
                dims[-1][0] *= size
            else:
                dims.append([size, stride])
        run, inner_terms = 1, []
        for size, stride in dims:
            inner_terms.append((size, run, stride))
            run *= size
        ids_map = kir.IndexMap((kir.Axis("idx", ids.numel, tuple(reversed(inner_terms))),), ids.offset)

        new: dict[int, kir.ReductionKernel] = {}
        try:
            for ci in users:
                c = kernels[ci]
                inputs = list(c.inputs)
                if c.n_cols != width:
                    raise _NoCompose
                for slot, a in enumerate(c.inputs):
                    if a.buffer != x.buffer:
                        continue
                    tok = _token_map(a, width, c.n_rows)
                    if tok is None or a.dtype != schedule.buffers[table.buffer].dtype:
                        raise _NoCompose
                    if fill is not None:
                        at = min(max(fill, 0), n_table - 1)
                        inputs[slot] = kir.Operand(table.name, table.buffer, a.dtype, kir.IndexMap(
                            (kir.Axis("row", c.n_rows, ()), kir.Axis("col", width, ((width, 1, 1),))),
                            table.offset + at * width))
                        continue
                    where = compose(tok, ids_map, ids.numel)
                    id_operand = kir.Operand(ids.name, ids.buffer, schedule.buffers[ids.buffer].dtype,
                                             kir.IndexMap((where.axes[0], kir.Axis("col", width, ())),
                                                          where.base))
                    for q, have in enumerate(inputs):
                        if (have.buffer, have.dtype, have.index, have.via) == \
                                (id_operand.buffer, id_operand.dtype, id_operand.index, None):
                            id_slot = q
                            break
                    else:
                        inputs.append(id_operand)
                        id_slot = len(inputs) - 1
                    inputs[slot] = kir.Operand(table.name, table.buffer, a.dtype, kir.IndexMap(
                        (kir.Axis("row", n_table, ((n_table, 1, width),)),
                         kir.Axis("col", width, ((width, 1, 1),))), table.offset), (id_slot, n_table))
                new[ci] = kir.ReductionKernel(c.name, c.row_space, c.reduce_space, inputs,
                                              list(c.outputs), list(c.steps), dict(c.out_expr),
                                              set(c.row_outputs), c.two_pass,
                                              ["embedding"] + list(c.ops))
        except _NoCompose:
            continue
        for ci, c in new.items():
            kernels[ci] = c
        kernels[ei] = None
        changed = True
    if not changed:
        return schedule
    # fills nobody reads any more
    for pi, p in enumerate(kernels):
        if p is not None and _constant_fill(p) is not None:
            b = p.outputs[0].buffer
            if b not in finals and not any(c is not None and c is not p and b in c.reads()
                                           for c in kernels):
                kernels[pi] = None
    out = kir.Schedule(name=schedule.name, kernels=[k for k in kernels if k is not None],
                       buffers=schedule.buffers, inputs=schedule.inputs, outputs=schedule.outputs,
                       params=schedule.params, plan=schedule.plan, meta=dict(schedule.meta))
    return _replanned(out) if replan else out


# --------------------------------------------------------------------------
# batch > 1: sequence-first storage around the attention matmuls
# --------------------------------------------------------------------------

_ROWWISE = {"aten.mm.default": 0, "aten.addmm.default": 1}      # op -> position of the row operand


def _rows_independent(k) -> bool:
    """A matmul whose result row ``i`` depends on row ``i`` of its row operand and
    on nothing else that varies with ``i``: ``mm``, and ``addmm`` whose ``self`` is
    the same for every row (a bias vector, a ``[1, F]`` row, a stride-0 broadcast).
    Only then may the rows of operand and result be permuted together;
    ``addmm(residual[R, F], x, w)`` adds a different row of ``self`` to every result
    row and must keep its order."""
    if not (isinstance(k, kir.ExternKernel) and k.op in _ROWWISE and len(k.outputs) == 1):
        return False
    if k.op == "aten.addmm.default":
        bias = k.args[0]
        if isinstance(bias, kir.View):
            return len(bias.shape) < 2 or bias.shape[0] == 1 or bias.strides[0] == 0
    return True


def _whole_dense(schedule, v) -> bool:
    return (isinstance(v, kir.View) and v.offset == 0 and v.strides == _dense_strides(v.shape)
            and v.numel == schedule.buffers[v.buffer].numel)


def _movable(schedule, buffer: str, finals) -> bool:
    return buffer not in finals and schedule.buffers[buffer].plannable


def output_major(k: kir.PointwiseKernel, order=None) -> kir.PointwiseKernel:
    """``k`` iterating in the order its first output is stored.

    A pointwise kernel may visit its elements in any order.  The frontend numbers
    them by the output's *logical* shape; once a buffer has been given another
    physical layout that numbering can leave no operand contiguous along the
    innermost iteration digit, and the emitter would fall back to one element per
    access.  The iteration index is cut at every boundary any operand's map uses,
    the resulting digits are re-ordered by the output's stride, and every map is
    rewritten for the new numbering (adjacent digits an operand walks densely are
    fused again).  ``order`` (a permutation of the digits, innermost first, or a
    function of their count returning one) overrides the choice; tests use it to
    scramble a kernel."""
    operands = list(k.inputs) + list(k.outputs)
    if not k.outputs or any(len(a.index.axes) != 1 or a.via is not None for a in operands):
        return k
    numel = k.numel
    cuts = {1, numel}
    for a in operands:
        for n, o, _ in a.index.axes[0].terms:
            cuts.add(o)
            cuts.add(o * n)
    edges = sorted(cuts)
    if any(hi % lo for lo, hi in zip(edges, edges[1:])):
        return k
    digits = [(hi // lo, lo) for lo, hi in zip(edges, edges[1:])]          # (size, weight), innermost first

    def strides(a):
        out = []
        for size, lo in digits:
            st = 0
            for n, o, s_ in a.index.axes[0].terms:
                if o <= lo and lo * size <= o * n and lo % o == 0:
                    st = s_ * (lo // o)
            out.append(st)
        return out

    if order is None:
        key = strides(k.outputs[0])
        if any(st == 0 for st in key):
            return k
        order = sorted(range(len(digits)), key=lambda j: key[j])            # innermost first
    elif callable(order):
        order = order(len(digits))
    if list(order) == list(range(len(digits))):
        return k
    weight, w = {}, 1
    for j in order:
        weight[j] = w
        w *= digits[j][0]

    def rebuilt(a):
        st = strides(a)
        terms = []                                                          # innermost first
        for j in order:
            n, sj = digits[j][0], st[j]
            if sj == 0:
                continue
            if terms and terms[-1][1] * terms[-1][0] == weight[j] and terms[-1][2] * terms[-1][0] == sj:
                terms[-1] = (terms[-1][0] * n, terms[-1][1], terms[-1][2])
            else:
                terms.append((n, weight[j], sj))
        return kir.Operand(a.name, a.buffer, a.dtype, kir.IndexMap(
            (kir.Axis(a.index.axes[0].var, numel, tuple(reversed(terms))),), a.index.base))

    space = tuple(digits[j][0] for j in reversed(order))
    return kir.PointwiseKernel(k.name, space, [rebuilt(a) for a in k.inputs],
                               [rebuilt(a) for a in k.outputs], k.body, k.out_expr, k.ops)


def sequence_first(schedule: kir.Schedule, replan: bool = True) -> kir.Schedule:
    """Store the operands and the result of the attention ``bmm`` calls as
    ``[T, B, H, D/H]`` instead of ``[B, H, T, D/H]`` when the batch is larger
    than one.

    ``bmm`` has one batch dimension with one stride.  With tokens stored
    batch-first the merged layout ``[B, T, H, D/H]`` the output projection wants
    has no such stride for ``(b, h)``, which is why the exporter puts a ``clone``
    after the context matmul (and transposing clones in front of it).  With
    tokens stored sequence-first, ``(b, h)`` is contiguous with stride ``D/H``
    both in the head layout and in the merged layout: ``bmm`` reads and writes
    ``[T, B, H, D/H]`` through plain strided views, the context ``clone`` becomes
    the identity and disappears (``read_through_copies``), and the key copy no
    longer transposes.  The output projection then sees its rows in ``(t, b)``
    order -- a matmul treats rows independently -- and the generated kernel that
    consumes its result reads row ``(b, t)`` at ``(t B + b)``.  Only buffers
    between the head copies and that kernel move; every index map and view on
    them is rewritten with ``layout.remap``, and a buffer whose uses cannot all be
    rewritten keeps its layout."""
    from . import layout as L

    kernels = list(schedule.kernels)
    finals = {v.buffer for v in schedule.outputs}
    writer = {}
    for k in kernels:
        for b in k.writes():
            writer.setdefault(b, []).append(k)

    # anchor: bmm -> pure copy -> row operand of a matmul
    anchor = None
    for k in kernels:
        if not _rows_independent(k):
            continue
        a = k.args[_ROWWISE[k.op]]
        if not (_whole_dense(schedule, a) and len(a.shape) == 2):
            continue
        w = writer.get(a.buffer, [])
        if len(w) != 1 or not _pure_copy(w[0]):
            continue
        src = writer.get(w[0].inputs[0].buffer, [])
        if len(src) != 1 or not (isinstance(src[0], kir.ExternKernel) and src[0].op == "aten.bmm.default"):
            continue
        ctx = src[0].outputs[0]
        if not (_whole_dense(schedule, ctx) and len(ctx.shape) == 3 and ctx.numel == a.numel):
            continue
        G, T, Dh = ctx.shape
        R, F = a.shape
        if F % Dh or G % (F // Dh) or (G // (F // Dh)) * T != R:
            continue
        anchor = (G // (F // Dh), T, F // Dh)
        break
    if anchor is None or anchor[0] == 1:
        return schedule
    B, T, H = anchor

    tables: dict[str, list] = {}

    def propose(buffer, digits):
        if not _movable(schedule, buffer, finals):
            return
        if buffer in tables and tables[buffer] != digits:
            tables[buffer] = None                                # two roles, two layouts: leave it
        else:
            tables.setdefault(buffer, digits)

    for k in kernels:
        if not isinstance(k, kir.ExternKernel):
            continue
        if k.op == "aten.bmm.default":
            for v in list(k.args[:2]) + list(k.outputs):
                if not (_whole_dense(schedule, v) and len(v.shape) == 3):
                    continue
                G, M, N = v.shape
                if G != B * H or (M == T) == (N == T):
                    continue
                order = (2, 0, 1, 3) if M == T else (3, 0, 1, 2)
                propose(v.buffer, L.dense_digits((B, H, M, N), order))
    # a generated kernel's result that only feeds pure copies into moved bmm operands
    # (the bias add in front of the head copies): stored [T, B, H, J, D/H] -- J = 3 for a
    # fused q/k/v projection -- (b, h) is one stride for each of the J slices, the
    # copies become re-addressable and ``read_through_copies`` drops them
    readers: dict[str, list] = {}
    for k in kernels:
        for b in k.reads():
            readers.setdefault(b, []).append(k)
    for y in [b for b, d in tables.items() if d]:
        w = writer.get(y, [])
        if len(w) != 1 or not _pure_copy(w[0]):
            continue
        x = w[0].inputs[0].buffer
        spec = schedule.buffers[x]
        made = writer.get(x, [])
        if (x in tables or len(made) != 1 or spec.numel % (B * T * H) or not all(
                _pure_copy(r) and tables.get(r.outputs[0].buffer) for r in readers.get(x, []))):
            continue
        Dh = schedule.buffers[y].numel // (B * T * H)
        J, rem = divmod(spec.numel, B * T * H * Dh)
        if rem or J < 1:
            continue
        if not isinstance(made[0], kir.ExternKernel):
            propose(x, L.dense_digits((B, T, J, H, Dh), (1, 0, 3, 2, 4)))
        elif J == 1 and _rows_independent(made[0]):
            # written by a matmul itself (bias folded into it): a library call cannot
            # interleave columns, but its rows can come in (t, b) order if its row
            # operand does
            a, out = made[0].args[_ROWWISE[made[0].op]], made[0].outputs[0]
            if (_whole_dense(schedule, a) and _whole_dense(schedule, out) and len(a.shape) == 2
                    and a.shape[0] == B * T and not any(
                        isinstance(w_, kir.ExternKernel) for w_ in writer.get(a.buffer, []))):
                propose(x, L.dense_digits((B, T, out.shape[1]), (1, 0, 2)))
                propose(a.buffer, L.dense_digits((B, T, a.shape[1]), (1, 0, 2)))
    # matmuls fed by a copy of a moved bmm result: row operand and result move together
    for k in kernels:
        if _rows_independent(k):
            a, out = k.args[_ROWWISE[k.op]], k.outputs[0]
            if not (_whole_dense(schedule, a) and _whole_dense(schedule, out) and len(a.shape) == 2
                    and a.shape[0] == B * T and out.shape[0] == B * T):
                continue
            w = writer.get(a.buffer, [])
            if len(w) == 1 and _pure_copy(w[0]) and tables.get(w[0].inputs[0].buffer):
                propose(a.buffer, L.dense_digits((B, T, a.shape[1]), (1, 0, 2)))
                propose(out.buffer, L.dense_digits((B, T, out.shape[1]), (1, 0, 2)))
    tables = {b: d for b, d in tables.items() if d}

    def rowwise_pair(k):
        if _rows_independent(k):
            return k.args[_ROWWISE[k.op]], k.outputs[0]
        return None

    def rewrite_kernel(k):
        """``k`` with every use of a moved buffer re-addressed (raises NoRemap)."""
        if isinstance(k, kir.ExternKernel):
            pair = rowwise_pair(k)
            keep = set()
            if pair and pair[0].buffer in tables and pair[1].buffer in tables \
                    and _whole_dense(schedule, pair[0]) and _whole_dense(schedule, pair[1]) \
                    and all(len(v.shape) == 2 and v.shape[0] == B * T and tables[v.buffer] ==
                            L.dense_digits((B, T, v.shape[1]), (1, 0, 2)) for v in pair):
                keep = {id(pair[0]), id(pair[1])}                # the same row permutation on both sides

            def fix(a):
                if isinstance(a, kir.View):
                    if a.buffer in tables and id(a) not in keep:
                        return L.remap_view(a, a.buffer, tables[a.buffer])
                    return a
                if isinstance(a, (list, tuple)):
                    return type(a)(fix(x) for x in a)
                return a
            if pair and not keep and (pair[0].buffer in tables) != (pair[1].buffer in tables):
                raise L.NoRemap("row operand and result of a matmul must move together")
            return kir.ExternKernel(k.name, k.op, [fix(a) for a in k.args],
                                    {n: fix(a) for n, a in k.kwargs.items()},
                                    [fix(o) for o in k.outputs])
        touched = [a for a in list(k.inputs) + list(k.outputs) if a.buffer in tables]
        if not touched:
            return k

        def op(a):
            if a.buffer not in tables:
                return a
            if a.via is not None:
                raise L.NoRemap("gathered operand")
            return kir.Operand(a.name, a.buffer, a.dtype, L.remap_index(a.index, tables[a.buffer]))
        if isinstance(k, kir.PointwiseKernel):
            return output_major(kir.PointwiseKernel(k.name, k.space, [op(a) for a in k.inputs],
                                                    [op(a) for a in k.outputs], k.body, k.out_expr,
                                                    k.ops))
        return kir.ReductionKernel(k.name, k.row_space, k.reduce_space, [op(a) for a in k.inputs],
                                   [op(a) for a in k.outputs], k.steps, k.out_expr, k.row_outputs,
                                   k.two_pass, k.ops)

    # a buffer whose uses cannot all be re-addressed keeps its layout; so does its partner
    for _ in range(len(tables) + 1):
        bad = None
        for k in kernels:
            try:
                rewrite_kernel(k)
            except L.NoRemap:
                used = [b for b in list(k.reads()) + list(k.writes()) if b in tables]
                bad = used
                break
        if bad is None:
            break
        for b in bad:
            tables.pop(b, None)
    else:
        return schedule
    if not tables:
        return schedule
    out = kir.Schedule(name=schedule.name, kernels=[rewrite_kernel(k) for k in kernels],
                       buffers=schedule.buffers, inputs=schedule.inputs, outputs=schedule.outputs,
                       params=schedule.params, plan=schedule.plan, meta=dict(schedule.meta))
    return _replanned(out) if replan else out


def read_through_copies(schedule: kir.Schedule, replan: bool = True) -> kir.Schedule:
    """Drop a pure copy whose result is only read by library calls, by pointing
    their views at the copy's source (the input-side twin of
    ``write_through_copies``).  After ``sequence_first`` the context ``clone`` is
    such a copy, and an identity at that."""
    from . import layout as L

    kernels: list = list(schedule.kernels)
    finals = {v.buffer for v in schedule.outputs}
    dropped = False
    for ci, c in enumerate(kernels):
        if c is None or not _pure_copy(c):
            continue
        x, y = c.inputs[0], c.outputs[0]
        if y.buffer in finals or not schedule.buffers[y.buffer].plannable:
            continue
        users = [ki for ki, k in enumerate(kernels) if k is not None and ki != ci
                 and (y.buffer in k.reads() or y.buffer in k.writes())]
        if not users or min(users) < ci or not all(
                isinstance(kernels[ki], kir.ExternKernel) and y.buffer not in kernels[ki].writes()
                for ki in users):
            continue
        if any(k is not None and x.buffer in k.writes() for k in kernels[ci + 1:max(users) + 1]):
            continue
        try:
            src = kir.IndexMap(x.index.axes, 0)
            digits = L.copy_digits(src, y.index, forward=False)

            def fix(a):
                if isinstance(a, kir.View):
                    if a.buffer != y.buffer:
                        return a
                    v = L.remap_view(a, x.buffer, digits)
                    v = kir.View(v.name, v.buffer, v.shape, v.strides, v.offset + x.index.base)
                    if len(v.shape) >= 2 and not _blas_layout(v.shape, v.strides):
                        raise L.NoRemap("not a matrix a BLAS call takes without copying")
                    return v
                if isinstance(a, (list, tuple)):
                    return type(a)(fix(e) for e in a)
                return a
            new = {ki: kir.ExternKernel(kernels[ki].name, kernels[ki].op,
                                        [fix(a) for a in kernels[ki].args],
                                        {n: fix(a) for n, a in kernels[ki].kwargs.items()},
                                        list(kernels[ki].outputs)) for ki in users}
        except L.NoRemap:
            continue
        for ki, k in new.items():
            kernels[ki] = k
        kernels[ci] = None
        dropped = True
    if not dropped:
        return schedule
    out = kir.Schedule(name=schedule.name, kernels=[k for k in kernels if k is not None],
                       buffers=schedule.buffers, inputs=schedule.inputs, outputs=schedule.outputs,
                       params=schedule.params, plan=schedule.plan, meta=dict(schedule.meta))
    return _replanned(out) if replan else out


# --------------------------------------------------------------------------
# sibling pointwise kernels: one launch for several independent maps
# --------------------------------------------------------------------------

def _renumbered(e, slot_offset: int, prefix: str):
    if isinstance(e, Load):
        return Load(e.slot + slot_offset)
    if isinstance(e, kir.Ref):
        return kir.Ref(prefix + e.name)
    if isinstance(e, Call):
        return Call(e.fn, tuple(_renumbered(a, slot_offset, prefix) for a in e.args))
    if isinstance(e, Cast):
        return Cast(_renumbered(e.x, slot_offset, prefix), e.dtype)
    return e


def _merged(members: list) -> kir.PointwiseKernel:
    inputs, outputs, body, out_expr, ops = [], [], [], {}, []
    for j, m in enumerate(members):
        off, pre = len(inputs), f"m{j}_"
        inputs += list(m.inputs)
        outputs += list(m.outputs)
        body += [(pre + n, _renumbered(e, off, pre)) for n, e in m.body]
        for a in m.outputs:
            out_expr[a.name] = _renumbered(m.out_expr[a.name], off, pre)
        ops += list(m.ops)
    last = members[-1]
    return kir.PointwiseKernel(last.name, last.space, inputs, outputs, body, out_expr, ops)


def fuse_siblings(schedule: kir.Schedule, replan: bool = True, limit: int = 4) -> kir.Schedule:
    """Run pointwise kernels that share an iteration space and do not depend on
    each other as one launch (BERT's q, k and v bias adds: 36 launches -> 12).

    Members keep their own operands, bodies and stores; the fused kernel is placed
    where the last member was, which is legal when nothing between the first and
    the last member touches a member's output or overwrites a member's input.
    Values are unchanged.  Off by default: the members already run as parallel
    branches of the graph, and joining them makes the fused launch wait for the
    slowest producer (see ``Config.fuse_siblings`` for the measurement)."""
    kernels = list(schedule.kernels)
    finals = {v.buffer for v in schedule.outputs}
    used: set[int] = set()
    groups: list[list[int]] = []
    for i, k in enumerate(kernels):
        if i in used or not isinstance(k, kir.PointwiseKernel) or len(k.outputs) != 1:
            continue
        group = [i]
        out_names = {a.name for a in k.outputs}
        for j in range(i + 1, min(len(kernels), i + 12)):
            c = kernels[j]
            if len(group) >= limit:
                break
            if j in used or not isinstance(c, kir.PointwiseKernel) or len(c.outputs) != 1:
                continue
            if c.space != k.space or c.ops != k.ops or len(c.inputs) != len(k.inputs) \
                    or [a.dtype for a in c.inputs + c.outputs] != [a.dtype for a in k.inputs + k.outputs] \
                    or c.outputs[0].name in out_names or c.outputs[0].buffer in finals:
                continue
            members = [kernels[g] for g in group]
            writes = {b for m in members for b in m.writes()}
            reads = {b for m in members for b in m.reads()}
            if (set(c.reads()) & writes) or (set(c.writes()) & (writes | reads)):
                continue
            # nothing in between may touch what the earlier members write, nor overwrite
            # what they read: they now run at position j
            between = [kernels[t] for t in range(group[0] + 1, j) if t not in group]
            if any((set(b.reads()) | set(b.writes())) & writes or set(b.writes()) & reads
                   for b in between):
                continue
            group.append(j)
            out_names.add(c.outputs[0].name)
        if len(group) > 1 and not any(kernels[g].outputs[0].buffer in finals for g in group):
            groups.append(group)
            used.update(group)
    if not groups:
        return schedule
    for group in groups:
        kernels[group[-1]] = _merged([kernels[g] for g in group])
        for g in group[:-1]:
            kernels[g] = None
    out = kir.Schedule(name=schedule.name, kernels=[k for k in kernels if k is not None],
                       buffers=schedule.buffers, inputs=schedule.inputs, outputs=schedule.outputs,
                       params=schedule.params, plan=schedule.plan, meta=dict(schedule.meta))
    return _replanned(out) if replan else out


def prepare(schedule: kir.Schedule, cfg) -> kir.Schedule:
    """Every rewrite ``cfg`` enables, in the order the executor applies them.
    Only arena-planned schedules are rewritten: the rewrites change live ranges
    and re-pack the arena afterwards."""
    if schedule.plan.mode != "arena":
        return schedule
    work = schedule
    if getattr(cfg, "bias_epilogue", False):
        work = fold_bias_into_matmul(work)
    if getattr(cfg, "sequence_first", True):
        moved = sequence_first(work)
        if moved is not work:
            work = read_through_copies(moved)
    if getattr(cfg, "forward_into_copies", True):
        work = forward_into_consumers(work)
    if getattr(cfg, "write_through_copies", True):
        work = write_through_copies(work)
    if getattr(cfg, "fold_embeddings", True):
        work = fold_embeddings(work)
    if getattr(cfg, "fuse_siblings", False):
        work = fuse_siblings(work)
    return work
