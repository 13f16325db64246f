"""Row-reduction kernels: LayerNorm, softmax and every other fused row statistic.

Replaces ``_emit_persistent`` and ``_emit_streamed``
(``mlc/codegen/triton_reduction.py:147-274``).  The reference gives every row
one Triton program whose column block is the next power of two (a 768-wide row
runs 1024 lanes with a quarter of them masked, and 128 LayerNorm rows occupy 128
programs whatever the machine).  Here a row is owned by a *group* of G threads,
G a power of two chosen from the row length and the row count:

* G <= 32: the group is a slice of a warp, several rows share a warp and a CTA,
  and a reduction is a shuffle butterfly -- no shared memory, no barrier;
* G  > 32: one CTA per row, butterfly per warp plus one shared-memory hop.

Each thread owns packs of V consecutive columns (128-bit accesses) at a stride
of G packs, so a warp-wide access is fully coalesced.  In the *persistent* form
the row is loaded once into registers and every step runs over it
(two reductions cost two butterflies and no extra traffic).  In the *streamed*
form (``two_pass``) the row does not fit: each reduction becomes a loop over the
row that recomputes the column-varying values it needs, a max followed by a sum
of ``exp(x - max)`` is fused into one online pass with a *per-row* running
maximum, as the torch reference backend does (``torch_backend.py:196-225``), and
a final loop stores the element outputs.

Steps are ordered and a later step may read any earlier result
(``mlc/kernels.py:117-134``): the walk below closes a phase at every ``Reduce``.
Values that do not vary along the column axis -- reduction results, values
derived only from them, operands indexed by row alone -- are scalars held once
per thread; lanes outside the row contribute nothing to a reduction, which is
the identity for every kind.
"""

from __future__ import annotations

from dataclasses import dataclass, field

from .. import kir
from ..kir import Bind, Reduce
from . import expr as X
from .indexing import (Access, check_bounds, classify, needs_64bit, pow2_ceil,
                       render_offset)
from .pointwise import (LaunchSpec, algorithmic_bytes, dependent_release, loads_ahead_of_wait,
                        pick_vector, store_code)

_OP = {"sum": "mlcb_op_sum", "prod": "mlcb_op_prod", "max": "mlcb_op_max", "min": "mlcb_op_min"}

#: machine shape the launch geometry is sized for (B200: 148 SMs)
SM_COUNT = 148


def _identity(kind: str, dtype: str) -> str:
    t = X.REG_T[dtype]
    if kind == "sum":
        return f"(({t})0)"
    if kind == "prod":
        return f"(({t})1)"
    hi = kind == "min"
    if dtype == "float64":
        return "MLCB_INF_D" if hi else "MLCB_NINF_D"
    if X.is_float(dtype):
        return "MLCB_INF_F" if hi else "MLCB_NINF_F"
    if dtype == "bool":
        return "true" if hi else "false"
    bits = kir.ITEMSIZE[dtype] * 8
    if dtype == "uint8":
        return "((unsigned char)255)" if hi else "((unsigned char)0)"
    if hi:
        return f"(({t}){(1 << (bits - 1)) - 1}LL)"
    return f"(({t})(-{(1 << (bits - 1)) - 1}LL - 1))"


def _acc_dtype(rdt: str) -> str:
    """dtype the partial is carried in: narrow floats accumulate in fp32."""
    return "float32" if rdt in kir.NARROW_FLOATS else rdt


@dataclass
class Geometry:
    V: int       # columns per pack
    P: int       # packs per row
    G: int       # threads per row
    NP: int      # packs per thread
    block: int   # threads per CTA
    rpb: int     # rows per CTA
    grid: int
    masked: bool  # some (thread, q) slots fall outside the row

    @property
    def cta_row(self) -> bool:
        return self.G > 32


def plan_geometry(n_rows: int, n_cols: int, operands, cfg, streamed: bool,
                  alg_bytes: int = 0) -> Geometry:
    V = pick_vector(operands, n_cols)
    wide = int(getattr(cfg, "wide_reduction_bytes", 0) or 0)
    if wide and alg_bytes >= wide and not streamed:
        V2 = pick_vector(operands, n_cols, cap_bytes=32)
        if V2 > V and all(classify(a.index, "col", V2).width == V2 for a in operands):
            V = V2
    P = n_cols // V
    want_np = max(1, int(getattr(cfg, "reduction_packs_per_thread", 2)))
    if streamed:
        # eight packs per lane per pass, at least a warp unless the row is shorter
        G = min(1024, max(min(32, pow2_ceil(P)), pow2_ceil((P + 7) // 8)))
        G = min(G, 256) if n_rows >= 4 * SM_COUNT else G
    else:
        # Prefer a slice of one warp (no shared memory, no barrier) with about
        # want_np packs per lane; go to a CTA per row only when a warp would need
        # more than max_np packs per lane.
        max_np = max(want_np, int(getattr(cfg, "reduction_max_packs", 8)))
        G = min(32, pow2_ceil((P + want_np - 1) // want_np))
        if (P + G - 1) // G > max_np:
            G = min(1024, pow2_ceil((P + 3) // 4))
        # small problems: spread each row over more lanes until the machine is
        # covered, as long as every lane still has a pack
        while G < 1024 and G * 2 <= pow2_ceil(P) and n_rows * G < SM_COUNT * 128:
            G *= 2
    forced = int(getattr(cfg, "reduction_group", 0) or 0)
    if forced:
        G = min(1024, pow2_ceil(forced))
    NP = (P + G - 1) // G
    if G > 32:
        block, rpb = G, 1
    else:
        rpb = max(1, 128 // G)
        # keep at least two CTAs per SM in flight before packing more rows per CTA
        while rpb > max(1, 32 // G) and (n_rows + rpb - 1) // rpb < 2 * SM_COUNT:
            rpb //= 2
        want_rows = int(getattr(cfg, "reduction_rows_per_cta", 0) or 0)
        if want_rows:
            rpb = max(max(1, 32 // G), min(1024 // G, pow2_ceil(want_rows)))
        block = G * rpb
    grid = (n_rows + rpb - 1) // rpb
    return Geometry(V, P, G, NP, block, rpb, grid, masked=(NP * G != P))


# --------------------------------------------------------------------------
# analysis shared by both forms
# --------------------------------------------------------------------------

def varying_steps(k: kir.ReductionKernel) -> set[str]:
    """Bind names whose value is a vector over the column axis (same rule as
    ``varies_by_column``, ``mlc/codegen/reduction_schedule.py:95-110``)."""
    col_slots = {i for i, a in enumerate(k.inputs) if a.index.varies_along("col")}
    vec: set[str] = set()
    for s in k.steps:
        if isinstance(s, Reduce):
            continue
        if (kir.expr_loads(s.expr) & col_slots) or (kir.expr_refs(s.expr) & vec):
            vec.add(s.name)
    return vec


class _Ctx:
    """Bookkeeping for one kernel emission."""

    def __init__(self, k: kir.ReductionKernel, geo: Geometry, it: str, stable=frozenset(), cfg=None):
        self.k, self.geo, self.it = k, geo, it
        #: input slots whose buffer nothing writes: loadable before the wait
        self.ahead = {i for i, a in enumerate(k.inputs) if a.buffer in stable and a.via is None} \
            if loads_ahead_of_wait(geo.grid, geo.block, cfg) else set()
        self.elide = X.store_only_casts([(s.name, s.expr) for s in k.steps if isinstance(s, Bind)],
                                        {n: e for n, e in k.out_expr.items()
                                         if n not in k.row_outputs},
                                        [a for a in k.outputs if a.name not in k.row_outputs])
        # a temp also read by a Reduce or a row output must keep its rounding
        for s in k.steps:
            if isinstance(s, Reduce):
                self.elide -= kir.expr_refs(s.expr)
        for n in k.row_outputs:
            self.elide -= kir.expr_refs(k.out_expr[n])
        self.lines: list[str] = []
        self.vec = varying_steps(k)
        self.scalars: dict[str, X.Val] = {}   # rendered row scalars (binds + reduces)

    def emit(self, s: str = "") -> None:
        self.lines.append(s)


def resident_ctas(geo: "Geometry", cfg, row_registers: int = 0) -> int:
    """CTAs per SM the compiler is told to keep resident (``__launch_bounds__``),
    i.e. the cap on registers per thread.

    The floor keeps 512 threads per SM (at most 128 registers each); without it
    ptxas aims far lower and serialises the row's loads, or spills.  On top of
    that, a launch that *can* be resident all at once should be: when the grid
    needs ``n`` CTAs per SM for one wave, ``n`` is requested as long as every
    thread keeps 64 registers or what the row itself occupies
    (``row_registers``), whichever is more.  LayerNorm over [4096, 768] with its
    gain and bias held across the wait is the case in point: left alone ptxas
    takes 80 registers, six CTAs fit an SM and 1024 CTAs need a second, nearly
    empty wave (4.4 us); told to fit seven it uses 64 and the launch is one wave
    (3.7 us)."""
    forced = int(getattr(cfg, "reduction_min_ctas", 0) or 0)
    if forced:
        return forced
    base = max(1, min(16, 512 // geo.block))
    need = -(-geo.grid // SM_COUNT)
    budget = max(64, row_registers)
    cap = min(2048 // geo.block, 65536 // (geo.block * budget))
    return max(base, min(need, cap))


def _signature(k, name: str, block: int, cfg=None, resident: int | None = None) -> str:
    aliased = {a.buffer for a in k.inputs} & {a.buffer for a in k.outputs}
    params = []
    for i, a in enumerate(k.inputs):
        r = "" if a.buffer in aliased else " __restrict__"
        params.append(f"const {X.STORAGE_T[a.dtype]}*{r} in{i}")
    for i, a in enumerate(k.outputs):
        r = "" if a.buffer in aliased else " __restrict__"
        params.append(f"{X.STORAGE_T[a.dtype]}*{r} out{i}")
    # the second bound keeps at least 512 threads resident per SM, which caps the
    # allocation at 128 registers per thread; without it ptxas aims far lower and
    # serialises the row's loads (or spills)
    if resident is None:
        resident = int(getattr(cfg, "reduction_min_ctas", 0) or 0) or max(1, min(16, 512 // block))
    return (f'extern "C" __global__ void __launch_bounds__({block}, {resident}) '
            f'{name}({", ".join(params)}) {{')


def _row_setup(c: _Ctx, n_rows: int, n_red: int) -> None:
    g, it = c.geo, c.it
    if g.cta_row:
        c.emit(f"    const int lane = threadIdx.x;")
        c.emit(f"    const {it} row = blockIdx.x;")
        c.emit(f"    __shared__ unsigned long long mlcb_red[{max(1, n_red)} * 32];")
        c.emit("    const bool live = true;")
    else:
        c.emit(f"    const int lane = threadIdx.x % {g.G};")
        c.emit(f"    {it} row = ({it})blockIdx.x * {g.rpb} + threadIdx.x / {g.G};")
        if n_rows % g.rpb != 0:
            # surplus groups shadow the last row so that shuffles stay convergent
            c.emit(f"    const bool live = row < {n_rows};")
            c.emit(f"    if (!live) row = {n_rows - 1};")
        else:
            c.emit("    const bool live = true;")


def _scalar_loads(c: _Ctx, ahead: bool, out: list | None = None) -> list[X.Val | None]:
    """Operands indexed by row alone: one scalar load per row
    (``triton_reduction.py:103-110``).  Called twice: for the operands that may be
    read before the grid-dependency wait (``ahead``), then for the rest."""
    if out is None:
        out = [None] * len(c.k.inputs)
    for i, a in enumerate(c.k.inputs):
        if a.index.varies_along("col") or (i in c.ahead) != ahead:
            continue
        st, rt = X.STORAGE_T[a.dtype], X.REG_T[a.dtype]
        off = render_offset(a.index, {"row": "row"}, skip=("col",))
        c.emit(f"    const {rt} s{i} = mlcb_load1<{st}>(in{i} + ({off}));  // {a.name} (per row)")
        out[i] = X.Val(f"s{i}", X.promoted_load_dtype(a.dtype), True, False)
    return out


def _finish_reduce(c: _Ctx, r: Reduce, acc_dt: str, rdt: str, ordinal: int) -> None:
    g = c.geo
    t = X.REG_T[acc_dt]
    if g.cta_row:
        nw = g.G // 32
        red = (f"mlcb_cta_reduce<{_OP[r.kind]}, {nw}, {t}>(acc_{r.name}, "
               f"reinterpret_cast<{t}*>(mlcb_red + {ordinal} * 32))")
    else:
        red = f"mlcb_group_reduce<{_OP[r.kind]}, {g.G}, {t}>(acc_{r.name})"
    if rdt in kir.NARROW_FLOATS:
        red = X.convert(red, "float32", rdt)
    c.emit(f"    const {X.REG_T[rdt]} {r.name} = {red};")
    c.scalars[r.name] = X.Val(r.name, rdt, True, False)


def _row_offsets(c: _Ctx, operands, prefix: str, ahead: bool | None = None) -> None:
    """``ahead`` selects the inputs loadable before the wait (True), the others
    (False) or all (None); output offsets are plain arithmetic and go first."""
    for i, a in enumerate(operands):
        if prefix == "in" and not a.index.varies_along("col"):
            continue
        if prefix == "in" and ahead is not None and (i in c.ahead) != ahead:
            continue
        if prefix == "out" and a.name in c.k.row_outputs:
            continue                               # stored once per row, at its own offset
        row = "row"
        if prefix == "in" and a.via is not None:
            # row gather: the table row is the integer operand `slot` holds for this
            # row, clamped so that a bad id reads a wrong row, never out of bounds
            slot, table_rows = a.via
            row = f"in{i}_id"
            c.emit(f"    const {c.it} {row} = ({c.it})mlcb_clamp_index((long long)s{slot}, "
                   f"{table_rows});  // {a.name}[{c.k.inputs[slot].name}]")
        off = render_offset(a.index, {"row": row}, skip=("col",))
        c.emit(f"    const {c.it} {prefix}{i}_r = {off};")


def _col_off(a, var: str) -> str:
    return render_offset(a.index, {"col": var}, skip=("row", "base"))


# --------------------------------------------------------------------------
# persistent form
# --------------------------------------------------------------------------

def _emit_persistent(k: kir.ReductionKernel, cfg, name: str, stable=frozenset()) -> tuple[str, LaunchSpec]:
    operands = [a for a in k.inputs if a.index.varies_along("col")] + [
        a for a in k.outputs if a.name not in k.row_outputs]
    geo = plan_geometry(k.n_rows, k.n_cols, operands or k.inputs + k.outputs, cfg, False,
                        algorithmic_bytes(k.inputs, k.outputs, k.n_rows * k.n_cols))
    V, G, NP = geo.V, geo.G, geo.NP
    extents = [k.n_rows * max(1, k.n_cols)] + [a.index.bounds()[1] + 1
                                               for a in k.inputs + k.outputs]
    it = "i64" if needs_64bit(*extents) else "int"
    c = _Ctx(k, geo, it, stable, cfg)
    reduces = k.reduces
    n_phases = len(reduces) + 1

    c.emit("")      # the signature: written once the row's register footprint is known
    c.emit(f"    // persistent: {k.n_rows} rows x {k.n_cols} cols; {G} lanes per row, "
           f"{NP} packs of {V} per lane, {geo.rpb} rows per CTA, grid {geo.grid}")
    _row_setup(c, k.n_rows, len(reduces))
    _row_offsets(c, k.outputs, "out")
    _row_offsets(c, k.inputs, "in", ahead=True)
    scalar_in = _scalar_loads(c, True)
    mark_ahead = len(c.lines)      # packed loads of stable operands are spliced in here
    c.emit("    MLCB_GRID_WAIT();")
    if getattr(cfg, "trigger_early", False) and dependent_release(geo.grid, geo.block, cfg):
        c.emit(dependent_release(geo.grid, geo.block, cfg))
    _scalar_loads(c, False, scalar_in)
    _row_offsets(c, k.inputs, "in", ahead=False)

    # ---- which phase defines / uses each column-varying value -------------
    phase_of: dict[str, int] = {}
    p = 0
    for s in k.steps:
        phase_of[s.name] = p
        if isinstance(s, Reduce):
            p += 1
    last_use: dict[str, int] = {}
    load_first: dict[int, int] = {}
    load_last: dict[int, int] = {}

    def note(e, ph):
        for nm in kir.expr_refs(e):
            last_use[nm] = max(last_use.get(nm, -1), ph)
        for sl in kir.expr_loads(e):
            load_first.setdefault(sl, ph)
            load_first[sl] = min(load_first[sl], ph)
            load_last[sl] = max(load_last.get(sl, -1), ph)

    for s in k.steps:
        if isinstance(s, Reduce) or s.name in c.vec:
            note(s.expr, phase_of[s.name])
    # An element output is stored in the first phase that has everything its
    # expression reads (GPT-2's LayerNorm also emits the residual sum it normalises:
    # stored as soon as it exists, that row stops occupying registers through both
    # reductions).  An output that aliases an input keeps the last phase.
    reduce_names = {s.name for s in k.steps if isinstance(s, Reduce)}
    in_place = {a.buffer for a in k.inputs} & {a.buffer for a in k.outputs}
    store_phase: dict[str, int] = {}
    for a in k.outputs:
        if a.name not in k.row_outputs:
            ready = max([phase_of[nm] + (1 if nm in reduce_names else 0)
                         for nm in kir.expr_refs(k.out_expr[a.name])] + [0])
            store_phase[a.name] = n_phases - 1 if a.buffer in in_place else ready
            note(k.out_expr[a.name], store_phase[a.name])

    # ---- operand access plans ---------------------------------------------
    acc_in: dict[int, Access] = {}
    for i, a in enumerate(k.inputs):
        if a.index.varies_along("col"):
            acc_in[i] = classify(a.index, "col", V)
    acc_out: dict[int, Access] = {}
    for i, a in enumerate(k.outputs):
        if a.name not in k.row_outputs:
            ac = classify(a.index, "col", V)
            acc_out[i] = ac if ac.mode == "contig" else Access("contig", 1)

    packed_in = {i for i, ac in acc_in.items() if ac.width > 1}
    kept = {nm for nm in c.vec if last_use.get(nm, -1) > phase_of[nm]}
    kept_decl: dict[str, str] = {}
    # registers the row itself occupies: one row in its register type per value that
    # is alive across the same reduction (at least one) and working room
    words = lambda dt: max(1, kir.ITEMSIZE[dt] // 4) if dt not in kir.NARROW_FLOATS else 1   # noqa: E731
    width = max([words(X.promoted_load_dtype(k.inputs[i].dtype)) for i in packed_in] or [1])
    live_rows = max([sum(1 for nm in kept if phase_of[nm] <= b < last_use[nm])
                     for b in range(n_phases)] + [1])
    row_regs = NP * V * width * live_rows + 16

    # Stable operands read as whole packs are fetched before the wait as packed words
    # (a quarter of the registers of the widened form) and widened where first used.
    # The words are held across the reductions, so they are only taken while the launch
    # still fits the machine in one wave with them: operands wanted last (LayerNorm's
    # gain and bias, whose load would otherwise start after the reductions) go first,
    # operands of the first phase -- needed together with the row itself -- last.
    # (A prefetch.global.L1 of the same addresses instead, holding no register, was
    # measured and is far slower on large launches: [4096, 768] 8.1 us against 3.6 us.)
    candidates = sorted((i for i in packed_in if i in c.ahead and i in load_first
                         and acc_in[i].mode == "contig" and acc_in[i].width == V),
                        key=lambda i: (-load_first[i], i))
    need = -(-geo.grid // SM_COUNT)
    budget = 65536 // (geo.block * need) if need * geo.block <= 2048 else 255
    raw_in: list[int] = []
    for i in candidates:
        cost = NP * max(1, V * kir.ITEMSIZE[k.inputs[i].dtype] // 4)
        if row_regs + cost <= max(budget, 64) or getattr(cfg, "hoist_stable_loads", True) == "all":
            raw_in.append(i)
            row_regs += cost
    raw_in.sort()
    if raw_in:
        pre = []
        for i in raw_in:
            pre.append(f"    mlcb_pack<{X.STORAGE_T[k.inputs[i].dtype]}, {V}> w{i}[{NP}];"
                       f"  // {k.inputs[i].name}: read ahead of the wait")
        pre.append("#pragma unroll")
        pre.append(f"    for (int q = 0; q < {NP}; ++q) {{")
        pre.append(f"        const int c0 = (lane + q * {G}) * {V};")
        guard = f"if (c0 < {k.n_cols}) " if geo.masked else ""
        for i in raw_in:
            a = k.inputs[i]
            pre.append(f"        {guard}mlcb_load_raw<{X.STORAGE_T[a.dtype]}, {V}>(in{i} + in{i}_r + "
                       f"({_col_off(a, 'c0')}), w{i}[q]);")
        pre.append("    }")
        c.lines[mark_ahead:mark_ahead] = pre
    c.lines[0] = _signature(k, name, geo.block, cfg, resident_ctas(geo, cfg, row_regs))
    for i in sorted(packed_in):
        if i in load_first:
            c.emit(f"    {X.REG_T[k.inputs[i].dtype]} v{i}[{NP}][{V}];  // {k.inputs[i].name}")

    def load_vals(in_loop_gather: bool) -> list[X.Val | None]:
        vals: list[X.Val | None] = []
        for i, a in enumerate(k.inputs):
            if scalar_in[i] is not None:
                vals.append(scalar_in[i])
            elif i in packed_in:
                ac = acc_in[i]
                code = f"v{i}[q][j]" if ac.mode == "contig" else f"v{i}[q][j / {ac.width}]"
                vals.append(X.Val(code, X.promoted_load_dtype(a.dtype), True, True))
            else:
                vals.append(X.Val(f"g{i}", X.promoted_load_dtype(a.dtype), True, True))
        return vals

    loads = load_vals(True)
    vec_vals: dict[str, X.Val] = {}

    def refs_now() -> dict[str, X.Val]:
        d = dict(c.scalars)
        d.update(vec_vals)
        return d

    pending: list = list(k.steps)
    pos = 0
    for ph in range(n_phases):
        # steps of this phase: up to and including the next Reduce
        phase_steps = []
        while pos < len(pending):
            s = pending[pos]
            pos += 1
            phase_steps.append(s)
            if isinstance(s, Reduce):
                break
        red = phase_steps[-1] if phase_steps and isinstance(phase_steps[-1], Reduce) else None

        # row scalars of this phase first: they depend on scalars only
        for s in phase_steps:
            if isinstance(s, Bind) and s.name not in c.vec:
                v = X.render(s.expr, loads, refs_now())
                c.emit(f"    const {X.REG_T[v.dtype]} {s.name} = {v.code};")
                c.scalars[s.name] = X.Val(s.name, v.dtype, v.dim, False)

        vbinds = [s for s in phase_steps if isinstance(s, Bind) and s.name in c.vec]
        stores = [(i, a) for i, a in enumerate(k.outputs) if store_phase.get(a.name) == ph]
        first_loads = sorted(i for i in acc_in if load_first.get(i) == ph and i in packed_in)
        gathers = sorted(i for i in acc_in if i not in packed_in
                         and load_first.get(i, 99) <= ph <= load_last.get(i, -1))
        if not (vbinds or red is not None or stores or first_loads):
            continue

        # declare arrays for values this phase defines and a later one reads
        pre_vals = dict(vec_vals)
        acc_dt = rdt = None
        if red is not None:
            probe = dict(c.scalars)
            probe.update(pre_vals)
            tmp_refs = dict(probe)
            for s in vbinds:
                v = X.render_bind(s.name, s.expr, loads, tmp_refs, c.elide)
                tmp_refs[s.name] = X.Val(s.name, v.dtype, v.dim, True)
            rv = X.render(red.expr, loads, tmp_refs)
            rdt = X.reduce_type(red.kind, rv.dtype)
            acc_dt = _acc_dtype(rdt)
            c.emit(f"    {X.REG_T[acc_dt]} acc_{red.name} = {_identity(red.kind, acc_dt)};")
        # types of kept values are needed before the loop to declare their arrays
        tmp_refs = dict(c.scalars)
        tmp_refs.update(pre_vals)
        for s in vbinds:
            v = X.render_bind(s.name, s.expr, loads, tmp_refs, c.elide)
            tmp_refs[s.name] = X.Val(s.name, v.dtype, v.dim, True)
            if s.name in kept:
                c.emit(f"    {X.REG_T[v.dtype]} a_{s.name}[{NP}][{V}];")
        out_regs = [(i, a) for i, a in stores if acc_out[i].width > 1]

        c.emit("#pragma unroll")
        c.emit(f"    for (int q = 0; q < {NP}; ++q) {{")
        if geo.masked or first_loads or stores or gathers:
            c.emit(f"        const int c0 = (lane + q * {G}) * {V};")
        ind = "        "
        if geo.masked:
            c.emit(f"        if (c0 < {k.n_cols}) {{")
            ind = "            "
        for i in first_loads:
            a, ac = k.inputs[i], acc_in[i]
            st = X.STORAGE_T[a.dtype]
            if ac.mode == "bcast":
                # one element per run of ac.width columns
                for r_, cc in enumerate(range(0, V, ac.width)):
                    c.emit(f"{ind}v{i}[q][{r_}] = mlcb_load1<{st}>(in{i} + in{i}_r + "
                           f"({_col_off(a, f'(c0 + {cc})')}));")
            elif i in raw_in:
                c.emit(f"{ind}mlcb_unpack<{st}, {V}>(w{i}[q], v{i}[q]);")
            elif ac.width == V:
                c.emit(f"{ind}mlcb_load<{st}, {V}>(in{i} + in{i}_r + ({_col_off(a, 'c0')}), v{i}[q]);")
            else:
                for cc in range(0, V, ac.width):
                    c.emit(f"{ind}mlcb_load_at<{st}, {ac.width}, {V}>(in{i} + in{i}_r + "
                           f"({_col_off(a, f'(c0 + {cc})')}), v{i}[q], {cc});")
        for i, a in out_regs:
            c.emit(f"{ind}{X.REG_T[a.dtype]} o{i}[{V}];")
        if vbinds or red is not None or stores or gathers:
            c.emit(f"#pragma unroll")
            c.emit(f"{ind}for (int j = 0; j < {V}; ++j) {{")
            in2 = ind + "    "
            if gathers or any(acc_out[i].width == 1 for i, _ in stores):
                c.emit(f"{in2}const int col = c0 + j;")
            for i in gathers:
                a = k.inputs[i]
                c.emit(f"{in2}const {X.REG_T[a.dtype]} g{i} = mlcb_load1<{X.STORAGE_T[a.dtype]}>"
                       f"(in{i} + in{i}_r + ({_col_off(a, 'col')}));  // {a.name}")
            local = dict(c.scalars)
            local.update(pre_vals)
            for s in vbinds:
                v = X.render_bind(s.name, s.expr, loads, local, c.elide)
                c.emit(f"{in2}const {X.REG_T[v.dtype]} {s.name} = {v.code};")
                local[s.name] = X.Val(s.name, v.dtype, v.dim, True)
                if s.name in kept:
                    c.emit(f"{in2}a_{s.name}[q][j] = {s.name};")
                    vec_vals[s.name] = X.Val(f"a_{s.name}[q][j]", v.dtype, v.dim, True)
            if red is not None:
                rv = X.render(red.expr, loads, local)
                x = X.convert(rv.code, rv.dtype, acc_dt) if rv.dtype not in kir.NARROW_FLOATS \
                    else rv.code
                t = X.REG_T[acc_dt]
                c.emit(f"{in2}acc_{red.name} = {_OP[red.kind]}::f<{t}>(acc_{red.name}, {x});")
            for i, a in stores:
                v = X.render(k.out_expr[a.name], loads, local)
                code = store_code(v, a.dtype)
                if acc_out[i].width > 1:
                    c.emit(f"{in2}o{i}[j] = {code};  // {a.name}")
                else:
                    c.emit(f"{in2}if (live) mlcb_store1<{X.STORAGE_T[a.dtype]}>(out{i} + out{i}_r + "
                           f"({_col_off(a, 'col')}), {code});  // {a.name}")
            c.emit(f"{ind}}}")
        for i, a in out_regs:
            ac, st = acc_out[i], X.STORAGE_T[a.dtype]
            if ac.width == V:
                c.emit(f"{ind}if (live) mlcb_store<{st}, {V}>(out{i} + out{i}_r + "
                       f"({_col_off(a, 'c0')}), o{i});")
            else:
                for cc in range(0, V, ac.width):
                    c.emit(f"{ind}if (live) mlcb_store_at<{st}, {ac.width}, {V}>(out{i} + out{i}_r + "
                           f"({_col_off(a, f'(c0 + {cc})')}), o{i}, {cc});")
        if geo.masked:
            c.emit("        }")
        c.emit("    }")
        if red is not None:
            _finish_reduce(c, red, acc_dt, rdt, reduces.index(red))
        if ph == 0 and not getattr(cfg, "trigger_early", False) \
                and dependent_release(geo.grid, geo.block, cfg, registers=row_regs):
            c.emit(dependent_release(geo.grid, geo.block, cfg, registers=row_regs))

    _row_stores(c, loads)
    c.emit("}")
    spec = LaunchSpec(grid=geo.grid, block=geo.block, vector=V,
                      alg_bytes=algorithmic_bytes(k.inputs, k.outputs, k.n_rows * k.n_cols))
    return "\n".join(c.lines), spec


def _row_stores(c: _Ctx, loads) -> None:
    """Outputs that live in row space: written once per row by the group's first
    lane (``triton_reduction.py:113-131``)."""
    k = c.k
    for i, a in enumerate(k.outputs):
        if a.name not in k.row_outputs:
            continue
        v = X.render(k.out_expr[a.name], loads, dict(c.scalars))
        off = render_offset(a.index, {"row": "row"}, skip=("col",))
        c.emit(f"    if (live && lane == 0) mlcb_store1<{X.STORAGE_T[a.dtype]}>(out{i} + ({off}), "
               f"{store_code(v, a.dtype)});  // {a.name} (per row)")


# --------------------------------------------------------------------------
# streamed form
# --------------------------------------------------------------------------

@dataclass
class Pass:
    """One traversal of the row (same partition as ``plan_passes``,
    ``mlc/codegen/reduction_schedule.py:150-209``)."""

    binds: list = field(default_factory=list)
    reduces: list = field(default_factory=list)
    stores: list = field(default_factory=list)
    online: tuple | None = None  # (max_step, sum_step, value expr)


def _dependencies(steps) -> dict[str, set[str]]:
    """name -> steps it needs, not looking behind a reduction (its result is a
    scalar that survives the pass that made it)."""
    by = {s.name: s for s in steps}
    memo: dict[str, set[str]] = {}

    def go(nm: str) -> set[str]:
        if nm in memo:
            return memo[nm]
        memo[nm] = set()
        out: set[str] = set()
        s = by.get(nm)
        if s is not None:
            for r in kir.expr_refs(s.expr):
                out.add(r)
                if not isinstance(by.get(r), Reduce):
                    out |= go(r)
        memo[nm] = out
        return out

    return {s.name: go(s.name) for s in steps}


def detect_online_softmax(k: kir.ReductionKernel):
    """A max whose only job is to shift the argument of a summed exponential."""
    rs = k.reduces
    if len(rs) != 2 or rs[0].kind != "max" or rs[1].kind != "sum":
        return None
    # the fused pass carries its running max and sum in fp32; a float64 row keeps
    # the two separate passes, which accumulate in float64 like the persistent form
    if any(a.dtype == "float64" for a in list(k.inputs) + list(k.outputs)) or any(
            isinstance(e, kir.Cast) and e.dtype == "float64"
            for s in k.steps for e in kir.walk(s.expr)):
        return None
    by = {s.name: s for s in k.steps}

    def resolve(e):
        while isinstance(e, kir.Ref) and isinstance(by.get(e.name), Bind):
            e = by[e.name].expr
        return e

    body = resolve(rs[1].expr)
    if not (isinstance(body, kir.Call) and body.fn == "exp"):
        return None
    inner = resolve(body.args[0])
    if not (isinstance(inner, kir.Call) and inner.fn == "sub"):
        return None
    shifted, sub = resolve(inner.args[0]), inner.args[1]
    if not (isinstance(sub, kir.Ref) and sub.name == rs[0].name):
        return None
    if shifted != resolve(rs[0].expr):
        return None
    return (rs[0], rs[1], rs[0].expr)


def plan_passes(k: kir.ReductionKernel) -> list[Pass]:
    deps = _dependencies(k.steps)
    vec = varying_steps(k)
    by = {s.name: s for s in k.steps}
    order = [s.name for s in k.steps]
    online = detect_online_softmax(k)

    def vbinds(needed: set[str]) -> list:
        return [by[n] for n in order if n in needed and isinstance(by[n], Bind) and n in vec]

    passes: list[Pass] = []
    rs = k.reduces
    i = 0
    while i < len(rs):
        r = rs[i]
        if online is not None and r is online[0]:
            passes.append(Pass(binds=vbinds(deps[r.name]), reduces=[online[0], online[1]],
                               online=online))
            i += 2
            continue
        passes.append(Pass(binds=vbinds(deps[r.name] | {r.name}), reduces=[r]))
        i += 1
    elem = [a.name for a in k.outputs if a.name not in k.row_outputs]
    if elem:
        needed: set[str] = set()
        for nm in elem:
            for ref in kir.expr_refs(k.out_expr[nm]):
                needed.add(ref)
                needed |= deps.get(ref, set())
        passes.append(Pass(binds=vbinds(needed), stores=elem))
    return passes


def _emit_streamed(k: kir.ReductionKernel, cfg, name: str, stable=frozenset()) -> tuple[str, LaunchSpec]:
    operands = [a for a in k.inputs if a.index.varies_along("col")] + [
        a for a in k.outputs if a.name not in k.row_outputs]
    geo = plan_geometry(k.n_rows, k.n_cols, operands or k.inputs + k.outputs, cfg, True)
    V, G = geo.V, geo.G
    extents = [k.n_rows * max(1, k.n_cols)] + [a.index.bounds()[1] + 1
                                               for a in k.inputs + k.outputs]
    it = "i64" if needs_64bit(*extents) else "int"
    c = _Ctx(k, geo, it, stable, cfg)
    passes = plan_passes(k)
    reduces = k.reduces
    by_reduce = {r.name: p for p in passes for r in p.reduces}

    c.emit(_signature(k, name, geo.block, cfg))
    c.emit(f"    // streamed: {k.n_rows} rows x {k.n_cols} cols, {len(passes)} passes over the row; "
           f"{G} lanes per row, packs of {V}, {geo.rpb} rows per CTA, grid {geo.grid}")
    _row_setup(c, k.n_rows, len(reduces) + 1)
    _row_offsets(c, k.outputs, "out")
    _row_offsets(c, k.inputs, "in", ahead=True)
    scalar_in = _scalar_loads(c, True)
    c.emit("    MLCB_GRID_WAIT();")
    _scalar_loads(c, False, scalar_in)
    _row_offsets(c, k.inputs, "in", ahead=False)
    if dependent_release(geo.grid, geo.block, cfg):
        c.emit(dependent_release(geo.grid, geo.block, cfg))

    acc_in = {i: classify(a.index, "col", V) for i, a in enumerate(k.inputs)
              if a.index.varies_along("col")}
    acc_out = {}
    for i, a in enumerate(k.outputs):
        if a.name not in k.row_outputs:
            ac = classify(a.index, "col", V)
            acc_out[i] = ac if ac.mode == "contig" else Access("contig", 1)

    def load_vals() -> list[X.Val]:
        vals = []
        for i, a in enumerate(k.inputs):
            if scalar_in[i] is not None:
                vals.append(scalar_in[i])
                continue
            ac = acc_in[i]
            dt = X.promoted_load_dtype(a.dtype)
            if ac.width > 1:
                code = f"v{i}[j]" if ac.mode == "contig" else f"v{i}[j / {ac.width}]"
                vals.append(X.Val(code, dt, True, True))
            else:
                vals.append(X.Val(f"g{i}", dt, True, True))
        return vals

    loads = load_vals()

    def pass_slots(p: Pass) -> list[int]:
        used: set[int] = set()
        for b in p.binds:
            used |= kir.expr_loads(b.expr)
        if p.online is not None:
            used |= kir.expr_loads(p.online[2])
        else:
            for r in p.reduces:
                used |= kir.expr_loads(r.expr)
        for nm in p.stores:
            used |= kir.expr_loads(k.out_expr[nm])
        return sorted(used & set(acc_in))

    def emit_pass(p: Pass) -> None:
        slots = pass_slots(p)
        online = p.online
        # result types first (needed to declare accumulators)
        probe = dict(c.scalars)
        for b in p.binds:
            v = X.render_bind(b.name, b.expr, loads, probe, c.elide)
            probe[b.name] = X.Val(b.name, v.dtype, v.dim, True)
        accs = {}
        if online is not None:
            c.emit("    // online softmax: running max and rescaled sum in one pass")
            c.emit("    float run_m = MLCB_NINF_F, run_l = 0.0f;")
        else:
            for r in p.reduces:
                rv = X.render(r.expr, loads, probe)
                rdt = X.reduce_type(r.kind, rv.dtype)
                adt = _acc_dtype(rdt)
                accs[r.name] = (adt, rdt)
                c.emit(f"    {X.REG_T[adt]} acc_{r.name} = {_identity(r.kind, adt)};")
        c.emit(f"    for (int c0 = lane * {V}; c0 < {k.n_cols}; c0 += {G * V}) {{")
        ind = "        "
        for i in slots:
            a, ac = k.inputs[i], acc_in[i]
            st, rt = X.STORAGE_T[a.dtype], X.REG_T[a.dtype]
            if ac.width <= 1:
                continue
            if ac.mode == "bcast":
                c.emit(f"{ind}{rt} v{i}[{V // ac.width}];")
                for r_, cc in enumerate(range(0, V, ac.width)):
                    c.emit(f"{ind}v{i}[{r_}] = mlcb_load1<{st}>(in{i} + in{i}_r + "
                           f"({_col_off(a, f'(c0 + {cc})')}));")
            elif ac.width == V:
                c.emit(f"{ind}{rt} v{i}[{V}]; mlcb_load<{st}, {V}>(in{i} + in{i}_r + "
                       f"({_col_off(a, 'c0')}), v{i});")
            else:
                c.emit(f"{ind}{rt} v{i}[{V}];")
                for cc in range(0, V, ac.width):
                    c.emit(f"{ind}mlcb_load_at<{st}, {ac.width}, {V}>(in{i} + in{i}_r + "
                           f"({_col_off(a, f'(c0 + {cc})')}), v{i}, {cc});")
        stores = [(i, a) for i, a in enumerate(k.outputs) if a.name in p.stores]
        for i, a in stores:
            if acc_out[i].width > 1:
                c.emit(f"{ind}{X.REG_T[a.dtype]} o{i}[{V}];")
        if online is not None:
            c.emit(f"{ind}float xs[{V}];")
        c.emit("#pragma unroll")
        c.emit(f"{ind}for (int j = 0; j < {V}; ++j) {{")
        in2 = ind + "    "
        gathers = [i for i in slots if acc_in[i].width <= 1]
        if gathers or any(acc_out[i].width == 1 for i, _ in stores):
            c.emit(f"{in2}const int col = c0 + j;")
        for i in gathers:
            a = k.inputs[i]
            c.emit(f"{in2}const {X.REG_T[a.dtype]} g{i} = mlcb_load1<{X.STORAGE_T[a.dtype]}>"
                   f"(in{i} + in{i}_r + ({_col_off(a, 'col')}));  // {a.name}")
        local = dict(c.scalars)
        for b in p.binds:
            v = X.render_bind(b.name, b.expr, loads, local, c.elide)
            c.emit(f"{in2}const {X.REG_T[v.dtype]} {b.name} = {v.code};")
            local[b.name] = X.Val(b.name, v.dtype, v.dim, True)
        if online is not None:
            xv = X.render(online[2], loads, local)
            c.emit(f"{in2}xs[j] = {X.convert(xv.code, xv.dtype, 'float32')};")
        else:
            for r in p.reduces:
                adt, _ = accs[r.name]
                rv = X.render(r.expr, loads, local)
                x = rv.code if rv.dtype in kir.NARROW_FLOATS else X.convert(rv.code, rv.dtype, adt)
                c.emit(f"{in2}acc_{r.name} = {_OP[r.kind]}::f<{X.REG_T[adt]}>(acc_{r.name}, {x});")
        for i, a in stores:
            v = X.render(k.out_expr[a.name], loads, local)
            code = store_code(v, a.dtype)
            if acc_out[i].width > 1:
                c.emit(f"{in2}o{i}[j] = {code};  // {a.name}")
            else:
                c.emit(f"{in2}if (live) mlcb_store1<{X.STORAGE_T[a.dtype]}>(out{i} + out{i}_r + "
                       f"({_col_off(a, 'col')}), {code});  // {a.name}")
        c.emit(f"{ind}}}")
        if online is not None:
            # m' = max(m, max(pack)); l' = l * exp(m - m') + sum(exp(x - m')).
            # A lane that has only met -inf keeps l = 0 and never evaluates
            # exp(-inf - -inf).
            ex = "mlcb_exp_fast" if X._FAST else "expf"
            c.emit(f"{ind}float pm = xs[0];")
            c.emit("#pragma unroll")
            c.emit(f"{ind}for (int j = 1; j < {V}; ++j) pm = mlcb_max<float>(pm, xs[j]);")
            c.emit(f"{ind}const float nm = mlcb_max<float>(run_m, pm);")
            c.emit(f"{ind}if (nm != MLCB_NINF_F) {{")
            c.emit(f"{ind}    float ps = 0.0f;")
            c.emit("#pragma unroll")
            c.emit(f"{ind}    for (int j = 0; j < {V}; ++j) ps += {ex}(xs[j] - nm);")
            c.emit(f"{ind}    run_l = run_l * ((run_m == MLCB_NINF_F) ? 0.0f : {ex}(run_m - nm)) + ps;")
            c.emit(f"{ind}    run_m = nm;")
            c.emit(f"{ind}}}")
        for i, a in stores:
            ac, st = acc_out[i], X.STORAGE_T[a.dtype]
            if ac.width == V and V > 1:
                c.emit(f"{ind}if (live) mlcb_store<{st}, {V}>(out{i} + out{i}_r + "
                       f"({_col_off(a, 'c0')}), o{i});")
            elif ac.width > 1:
                for cc in range(0, V, ac.width):
                    c.emit(f"{ind}if (live) mlcb_store_at<{st}, {ac.width}, {V}>(out{i} + out{i}_r + "
                           f"({_col_off(a, f'(c0 + {cc})')}), o{i}, {cc});")
        c.emit("    }")
        if online is not None:
            mx, sm, _ = online
            nred = len(reduces)
            if geo.cta_row:
                nw = G // 32
                c.emit(f"    const float {mx.name} = mlcb_cta_reduce<mlcb_op_max, {nw}, float>(run_m, "
                       f"reinterpret_cast<float*>(mlcb_red + 0 * 32));")
            else:
                c.emit(f"    const float {mx.name} = mlcb_group_reduce<mlcb_op_max, {G}, float>(run_m);")
            c.emit(f"    const float scaled_l = (run_m == MLCB_NINF_F) ? 0.0f : "
                   f"run_l * {'mlcb_exp_fast' if X._FAST else 'expf'}(run_m - {mx.name});")
            if geo.cta_row:
                c.emit(f"    const float {sm.name} = mlcb_cta_reduce<mlcb_op_sum, {nw}, float>(scaled_l, "
                       f"reinterpret_cast<float*>(mlcb_red + 1 * 32));")
            else:
                c.emit(f"    const float {sm.name} = mlcb_group_reduce<mlcb_op_sum, {G}, float>(scaled_l);")
            c.scalars[mx.name] = X.Val(mx.name, "float32", True, False)
            c.scalars[sm.name] = X.Val(sm.name, "float32", True, False)
        else:
            for r in p.reduces:
                adt, rdt = accs[r.name]
                _finish_reduce(c, r, adt, rdt, reduces.index(r))

    done: set[int] = set()
    for s in k.steps:
        if isinstance(s, Reduce):
            p = by_reduce[s.name]
            if id(p) in done:
                continue
            done.add(id(p))
            emit_pass(p)
        elif s.name not in c.vec:
            v = X.render(s.expr, loads, dict(c.scalars))
            c.emit(f"    const {X.REG_T[v.dtype]} {s.name} = {v.code};")
            c.scalars[s.name] = X.Val(s.name, v.dtype, v.dim, False)
    for p in passes:
        if p.stores and not p.reduces:
            emit_pass(p)
    _row_stores(c, loads)
    c.emit("}")
    traffic = algorithmic_bytes(k.inputs, k.outputs, k.n_rows * k.n_cols)
    spec = LaunchSpec(grid=geo.grid, block=geo.block, vector=V, alg_bytes=traffic)
    return "\n".join(c.lines), spec


def emit_reduction(k: kir.ReductionKernel, cfg, buffers: dict[str, kir.BufferSpec] | None = None,
                   name: str | None = None, stable=frozenset()) -> tuple[str, LaunchSpec]:
    if buffers is not None:
        for a in list(k.inputs) + list(k.outputs):
            check_bounds(a.index, buffers[a.buffer].numel, f"{k.name}:{a.name}")
    for i, a in enumerate(k.inputs):
        if a.via is None:
            continue
        slot, table_rows = a.via
        ids = k.inputs[slot]
        ax = a.index.axis("row")
        if (ids.index.varies_along("col") or ids.dtype not in ("int64", "int32")
                or ax is None or ax.numel != table_rows or not a.index.varies_along("col")):
            raise ValueError(f"{k.name}:{a.name}: malformed row gather")
    if any(a.via is not None for a in k.outputs):
        raise ValueError(f"{k.name}: outputs cannot be gathered")
    name = name or k.name
    with X.math_mode(X.wants_fast_math(k, cfg)):
        return (_emit_streamed(k, cfg, name, stable) if k.two_pass
                else _emit_persistent(k, cfg, name, stable))
