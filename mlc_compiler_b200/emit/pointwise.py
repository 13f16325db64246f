"""Pointwise kernels: one thread owns one pack of V consecutive flat indices.

Replaces ``emit_pointwise`` (``mlc/codegen/triton_backend.py:206-254``).  Where
the Triton form is a flat scalar ``idx = pid * BLOCK + arange`` and trusts the
compiler to find vector accesses, this emitter decides them: V is the number of
elements of the *narrowest* operand that fill 128 bits, every operand gets the
widest access its index map proves legal (``indexing.classify``), and the body
is straight-line code over ``V`` lanes held in registers.  A broadcast operand
such as a bias row (``idx % 768``) is still one packed load per thread because
768 is a multiple of V; a gather such as the head-merge copy
(``(idx / 768) * 64 + ((idx / 64) % 12) * 8192 + idx % 64``) keeps 128-bit
accesses because every coefficient is a multiple of V.
"""

from __future__ import annotations

from dataclasses import dataclass

from .. import kir
from . import expr as X
from .indexing import Access, check_bounds, classify, needs_64bit, pow2_ceil, render_offset


@dataclass
class LaunchSpec:
    """Grid and block of one launch; everything else is baked into the source.
    Counterpart of the reference's ``LaunchSpec`` (``triton_backend.py:105-112``)."""

    grid: int
    block: int
    smem: int = 0
    #: descriptive, for reports: elements per thread-pack and algorithmic bytes
    vector: int = 1
    alg_bytes: int = 0

    def as_dict(self) -> dict:
        return {"grid": (self.grid,), "block": self.block, "smem": self.smem,
                "vector": self.vector, "alg_bytes": self.alg_bytes}


def algorithmic_bytes(inputs, outputs, iter_numel: int) -> int:
    """Distinct elements addressed per operand x itemsize (broadcast operands
    counted once), the figure the roofline report divides by kernel time."""
    total = 0
    for a in inputs:
        total += min(a.index.distinct_elements(), iter_numel) * kir.ITEMSIZE[a.dtype]
    for a in outputs:
        total += min(a.index.distinct_elements(), iter_numel) * kir.ITEMSIZE[a.dtype]
    return total


def single_wave(grid: int, block: int, sms: int = 148, threads_per_sm: int = 1024,
                slack: float = 1.0) -> bool:
    """Whether every CTA of the launch can be resident at once (1024 threads per
    SM assumed unless the caller knows the kernel's footprint).  Only such
    launches release their dependents early: a dependent grid that becomes
    resident while later waves of its predecessor are still waiting for SM slots
    takes those slots and just sits at its wait."""
    return grid * block <= sms * threads_per_sm * slack


def dependent_release(grid: int, block: int, cfg, indent: str = "    ",
                      registers: int = 0) -> str | None:
    """The line that releases the next launch (``griddepcontrol.launch_dependents``),
    or None.  ``Config.dependent_trigger``: 0 never; 1 launches that fit the
    machine in one wave; 2 every launch.  A caller that can estimate the kernel's
    ``registers`` per thread gets the residency that follows from them, and up to
    half a wave of excess: the causal softmax over [49152, 128] (32 registers, 1.3
    waves at 2048 threads per SM) runs 5.65 us per launch releasing its dependent
    against 5.80 us not; the 4-wave bias+GELU+residual launch loses 10 % doing so."""
    policy = int(getattr(cfg, "dependent_trigger", 1))
    if policy == 2:
        return f"{indent}MLCB_GRID_TRIGGER();"
    if policy == 1:
        if registers:
            resident = min(2048, 65536 // max(32, registers)) // block * block
            ok = single_wave(grid, block, threads_per_sm=max(block, resident), slack=1.5)
        else:
            ok = single_wave(grid, block)
        if ok:
            return f"{indent}MLCB_GRID_TRIGGER();"
    return None


def loads_ahead_of_wait(grid: int, block: int, cfg) -> bool:
    """Whether a launch fetches its parameters before the grid-dependency wait
    (``Config.hoist_stable_loads``: False never, "all" always, True only when the
    whole launch is resident at once).  CTAs of a later wave start long after the
    predecessor has finished, so for them there is nothing to overlap and the
    packed words held across the wait only cost registers: BERT-base at batch 32
    runs 1.2 % slower with every launch hoisted, 2.5 % faster at batch 1 where all
    launches are a fraction of a wave."""
    mode = getattr(cfg, "hoist_stable_loads", True)
    return bool(mode) and (mode == "all" or single_wave(grid, block))


def pick_vector(operands, numel: int, cap_bytes: int = 16) -> int:
    smallest = min((kir.ITEMSIZE[a.dtype] for a in operands), default=4)
    v = max(1, cap_bytes // smallest)
    while v > 1 and numel % v != 0:
        v //= 2
    return v


def _chunks(acc: Access, v: int):
    return range(0, v, acc.width)


def emit_pointwise(k: kir.PointwiseKernel, cfg, buffers: dict[str, kir.BufferSpec] | None = None,
                   name: str | None = None, stable=frozenset()) -> tuple[str, LaunchSpec]:
    """``stable`` names buffers whose contents are fixed before the first launch
    (parameters nothing writes); their loads are issued ahead of the
    grid-dependency wait."""
    with X.math_mode(X.wants_fast_math(k, cfg)):
        return _emit_pointwise(k, cfg, buffers, name, stable)


def _emit_pointwise(k, cfg, buffers, name, stable=frozenset()) -> tuple[str, LaunchSpec]:
    name = name or k.name
    numel = k.numel
    operands = list(k.inputs) + list(k.outputs)
    if any(a.via is not None for a in operands):
        raise ValueError(f"{k.name}: row gathers are only emitted for reduction inputs")
    if buffers is not None:
        for a in operands:
            check_bounds(a.index, buffers[a.buffer].numel, f"{k.name}:{a.name}")

    V = pick_vector(operands, numel)
    tile = plan_tile(k, V)
    if tile is not None:
        return _emit_tiled(k, cfg, name, V, tile)
    # large streaming kernels use 256-bit accesses (two 128-bit packs per thread)
    wide = int(getattr(cfg, "wide_access_bytes", 0) or 0)
    if wide and algorithmic_bytes(k.inputs, k.outputs, numel) >= wide:
        V2 = pick_vector(operands, numel, cap_bytes=32)
        if V2 > V and all(classify(a.index, "idx", V2).width == V2 for a in operands):
            V = V2
    packs = numel // V
    extents = [numel] + [a.index.bounds()[1] + 1 for a in operands]
    it = "i64" if needs_64bit(*extents) else "int"

    block_cap = max(32, pow2_ceil(max(1, int(getattr(cfg, "pointwise_block", 1024))) // V))
    block = max(32, min(1024, block_cap, pow2_ceil(packs)))
    grid = (packs + block - 1) // block
    guard = packs % block != 0

    aliased = {a.buffer for a in k.inputs} & {a.buffer for a in k.outputs}
    params = []
    for i, a in enumerate(k.inputs):
        r = "" if a.buffer in aliased else " __restrict__"
        params.append(f"const {X.STORAGE_T[a.dtype]}*{r} in{i}")
    for i, a in enumerate(k.outputs):
        r = "" if a.buffer in aliased else " __restrict__"
        params.append(f"{X.STORAGE_T[a.dtype]}*{r} out{i}")

    L: list[str] = []
    L.append(f'extern "C" __global__ void __launch_bounds__({block}, {max(1, min(16, 512 // block))}) '
             f'{name}({", ".join(params)}) {{')
    L.append(f"    // pointwise {list(k.space)} = {numel} elements, {V} per thread, "
             f"{grid} x {block} threads")
    L.append(f"    const {it} pack = ({it})blockIdx.x * {block} + threadIdx.x;")
    if guard:
        L.append(f"    if (pack >= {packs}) return;")
    L.append(f"    const {it} i0 = pack * {V};")

    names = {"idx": "idx"}
    at_i0 = {"idx": "i0"}
    loads: list[X.Val] = []
    inner: list[str] = []   # per-element loads placed inside the lane loop
    early: list[str] = []   # loads of stable operands: issued before the wait
    after: list[str] = []   # everything that may read a predecessor's output
    need_idx = False
    hoist = loads_ahead_of_wait(grid, block, cfg)
    for i, a in enumerate(k.inputs):
        acc = classify(a.index, "idx", V)
        st, rt = X.STORAGE_T[a.dtype], X.REG_T[a.dtype]
        vdt = X.promoted_load_dtype(a.dtype)
        ahead = hoist and a.buffer in stable
        if acc.mode == "bcast" and acc.width == V:
            (early if ahead else after).append(
                f"    const {rt} v{i} = mlcb_load1<{st}>(in{i} + ({render_offset(a.index, at_i0)}));"
                f"  // {a.name}")
            loads.append(X.Val(f"v{i}", vdt))
        elif acc.mode == "contig" and acc.width == V and V > 1:
            if ahead:
                # the packed words travel across the wait; widened where the others are
                early.append(f"    mlcb_pack<{st}, {V}> w{i}; mlcb_load_raw<{st}, {V}>(in{i} + "
                             f"({render_offset(a.index, at_i0)}), w{i});  // {a.name}")
                after.append(f"    {rt} v{i}[{V}]; mlcb_unpack<{st}, {V}>(w{i}, v{i});")
            else:
                after.append(f"    {rt} v{i}[{V}]; mlcb_load<{st}, {V}>(in{i} + "
                             f"({render_offset(a.index, at_i0)}), v{i});  // {a.name}")
            loads.append(X.Val(f"v{i}[j]", vdt))
        elif acc.mode == "contig" and acc.width > 1:
            after.append(f"    {rt} v{i}[{V}];  // {a.name}: runs of {acc.width}")
            for c in _chunks(acc, V):
                off = render_offset(a.index, {"idx": f"(i0 + {c})"})
                after.append(f"    mlcb_load_at<{st}, {acc.width}, {V}>(in{i} + ({off}), v{i}, {c});")
            loads.append(X.Val(f"v{i}[j]", vdt))
        else:
            need_idx = True
            inner.append(f"        const {rt} v{i} = mlcb_load1<{st}>(in{i} + ({render_offset(a.index, names)}));"
                         f"  // {a.name}")
            loads.append(X.Val(f"v{i}", vdt))
    L += early
    L.append("    MLCB_GRID_WAIT();")
    if getattr(cfg, "trigger_early", False) and dependent_release(grid, block, cfg):
        L.append(dependent_release(grid, block, cfg))
    # operands a predecessor may have written first: their latency is the critical path
    L += [ln for ln in after if "mlcb_unpack" not in ln] + [ln for ln in after if "mlcb_unpack" in ln]

    out_acc = []
    for i, a in enumerate(k.outputs):
        acc = classify(a.index, "idx", V)
        if acc.mode != "contig":
            acc = Access("contig", 1)
        out_acc.append(acc)
        if acc.width > 1:
            L.append(f"    {X.REG_T[a.dtype]} o{i}[{V}];")
        else:
            need_idx = True

    if not getattr(cfg, "trigger_early", False) and dependent_release(grid, block, cfg):
        L.append(dependent_release(grid, block, cfg))
    L.append("#pragma unroll")
    L.append(f"    for (int j = 0; j < {V}; ++j) {{")
    if need_idx:
        L.append(f"        const {it} idx = i0 + j;")
    L += inner
    refs: dict[str, X.Val] = {}
    elide = X.store_only_casts(k.body, k.out_expr, k.outputs)
    for temp, e in k.body:
        v = X.render_bind(temp, e, loads, refs, elide)
        L.append(f"        const {X.REG_T[v.dtype]} {temp} = {v.code};")
        refs[temp] = X.Val(temp, v.dtype, v.dim)
    for i, a in enumerate(k.outputs):
        v = X.render(k.out_expr[a.name], loads, refs)
        code = store_code(v, a.dtype)
        if out_acc[i].width > 1:
            L.append(f"        o{i}[j] = {code};  // {a.name}")
        else:
            L.append(f"        mlcb_store1<{X.STORAGE_T[a.dtype]}>(out{i} + ({render_offset(a.index, names)}), {code});"
                     f"  // {a.name}")
    L.append("    }")
    for i, a in enumerate(k.outputs):
        acc = out_acc[i]
        st = X.STORAGE_T[a.dtype]
        if acc.width == V and V > 1:
            L.append(f"    mlcb_store<{st}, {V}>(out{i} + ({render_offset(a.index, at_i0)}), o{i});")
        elif acc.width > 1:
            for c in _chunks(acc, V):
                off = render_offset(a.index, {"idx": f"(i0 + {c})"})
                L.append(f"    mlcb_store_at<{st}, {acc.width}, {V}>(out{i} + ({off}), o{i}, {c});")
    L.append("}")

    spec = LaunchSpec(grid=grid, block=block, vector=V,
                      alg_bytes=algorithmic_bytes(k.inputs, k.outputs, numel))
    return "\n".join(L), spec


def store_code(v: X.Val, out_dtype: str) -> str:
    """Register value handed to a store of ``out_dtype``.  The store itself
    rounds a float register to fp16/bf16, so a float32 (or already narrow)
    value is passed through rather than rounded twice, and a value that is
    known to be ``round(x)`` to this same dtype is stored as ``x``."""
    if out_dtype in kir.NARROW_FLOATS:
        if v.unrounded is not None and v.unrounded[1] == out_dtype:
            return v.unrounded[0]
        if v.dtype in ("float32", out_dtype):
            return v.code
        return X.convert(v.code, v.dtype, "float32")
    return X.convert(v.code, v.dtype, out_dtype)


# --------------------------------------------------------------------------
# transposing kernels: V x V register tiles
# --------------------------------------------------------------------------

@dataclass
class Tile:
    """A second iteration digit ``r`` along which some operands are contiguous
    while the outputs are contiguous along the innermost digit ``t``."""

    n0: int        # size of the innermost digit t (out_stride 1)
    nr: int        # size of digit r
    o_r: int       # out_stride of digit r
    along_r: dict  # input slot -> True if the operand also varies along t
    along_t: dict  # input slot -> Access (contig / bcast, width V)


def plan_tile(k: kir.PointwiseKernel, V: int) -> Tile | None:
    """Decide whether ``k`` is a transposing kernel that can run on V x V
    register tiles: every operand is 128-bit contiguous either along the
    innermost iteration digit (all outputs are) or along one other digit."""
    if V < 2 or not k.inputs or not k.outputs:
        return None
    numel = k.numel
    along_t: dict[int, Access] = {}
    gathers: list[int] = []
    for i, a in enumerate(k.inputs):
        acc = classify(a.index, "idx", V)
        if acc.width == V:
            along_t[i] = acc
        else:
            gathers.append(i)
    if not gathers:
        return None
    for a in k.outputs:
        acc = classify(a.index, "idx", V)
        if acc.mode != "contig" or acc.width != V:
            return None
    digit = None
    with_t: dict[int, bool] = {}
    n0 = None
    for i in gathers:
        a = k.inputs[i]
        ax = a.index.axis("idx")
        if ax is None:
            return None
        unit = [t for t in ax.terms if t[2] == 1 and t[1] != 1]
        if len(unit) != 1:
            return None
        nr, o_r, _ = unit[0]
        if digit is None:
            digit = (nr, o_r)
        elif digit != (nr, o_r):
            return None
        if a.index.base % V:
            return None
        t_terms = [t for t in ax.terms if t[1] == 1]
        if len(t_terms) > 1:
            return None
        for t in ax.terms:
            if t is unit[0]:
                continue
            if t[2] % V:                      # keeps every run along r 16-byte aligned
                return None
            if t not in t_terms and t[1] % V:
                return None
        if t_terms:
            if n0 is None:
                n0 = t_terms[0][0]
            elif n0 != t_terms[0][0]:
                return None
        with_t[i] = bool(t_terms)
    nr, o_r = digit
    if n0 is None:
        n0 = o_r          # nothing fixes the t digit: take everything below r
    if o_r % n0 or nr % (8 * V) or n0 % (4 * V) or numel % (o_r * nr):
        return None
    # operands contiguous along t must see runs that do not straddle the digit
    for i, acc in along_t.items():
        if acc.mode == "bcast" and acc.width != V:
            return None
    return Tile(n0=n0, nr=nr, o_r=o_r, along_r=with_t, along_t=along_t)


def _emit_tiled(k: kir.PointwiseKernel, cfg, name: str, V: int, tile: Tile) -> tuple[str, LaunchSpec]:
    """One thread owns a V x V tile: V consecutive values of digit r by V
    consecutive values of the innermost digit t.  Operands contiguous along r are
    fetched with V packed loads (one per t), operands and outputs contiguous
    along t with one packed access per r; the transpose between the two happens
    in registers, by indexing.  Lanes are laid out 4 along t by 8 along r so that
    a warp-wide access covers whole 64- and 128-byte segments in both
    directions: no shared memory, no barrier, no partially used sector."""
    numel = k.numel
    n0, nr, o_r = tile.n0, tile.nr, tile.o_r
    operands = list(k.inputs) + list(k.outputs)
    extents = [numel] + [a.index.bounds()[1] + 1 for a in operands]
    it = "i64" if needs_64bit(*extents) else "int"
    micro = numel // (V * V)
    block = 128
    while block > 32 and micro % block:
        block //= 2
    grid = (micro + block - 1) // block
    WT, WR, M = n0 // (4 * V), nr // (8 * V), o_r // n0

    aliased = {a.buffer for a in k.inputs} & {a.buffer for a in k.outputs}
    params = []
    for i, a in enumerate(k.inputs):
        r = "" if a.buffer in aliased else " __restrict__"
        params.append(f"const {X.STORAGE_T[a.dtype]}*{r} in{i}")
    for i, a in enumerate(k.outputs):
        r = "" if a.buffer in aliased else " __restrict__"
        params.append(f"{X.STORAGE_T[a.dtype]}*{r} out{i}")

    L: list[str] = []
    L.append(f'extern "C" __global__ void __launch_bounds__({block}, {max(1, min(16, 512 // block))}) '
             f'{name}({", ".join(params)}) {{')
    L.append(f"    // transposing pointwise {list(k.space)} = {numel} elements; {V}x{V} register tile per "
             f"thread over digits r=({nr} @ {o_r}) and t=({n0} @ 1); {grid} x {block} threads")
    L.append(f"    const {it} micro = ({it})blockIdx.x * {block} + threadIdx.x;")
    if micro % block:
        L.append(f"    if (micro >= {micro}) return;")
    L.append(f"    const int lane = (int)(micro % 32);")
    L.append(f"    const {it} w = micro / 32;")
    L.append(f"    const {it} t_oct = (w % {WT}) * 4 + (lane % 4);")
    L.append(f"    const {it} r_oct = ((w / {WT}) % {WR}) * 8 + (lane / 4);")
    L.append(f"    const {it} rest = w / {WT * WR};")
    L.append(f"    const {it} base_idx = t_oct * {V} + (rest % {M}) * {n0} + r_oct * {V * o_r} "
             f"+ (rest / {M}) * {o_r * nr};")
    L.append("    MLCB_GRID_WAIT();")

    loads: list[X.Val | None] = [None] * len(k.inputs)
    for i, a in enumerate(k.inputs):
        st, rt = X.STORAGE_T[a.dtype], X.REG_T[a.dtype]
        vdt = X.promoted_load_dtype(a.dtype)
        if i in tile.along_r:
            if tile.along_r[i]:
                L.append(f"    {rt} g{i}[{V}][{V}];  // {a.name}: contiguous along r")
                L.append("#pragma unroll")
                L.append(f"    for (int j = 0; j < {V}; ++j) mlcb_load<{st}, {V}>(in{i} + "
                         f"({render_offset(a.index, {'idx': '(base_idx + j)'})}), g{i}[j]);")
                loads[i] = X.Val(f"g{i}[j][i]", vdt)
            else:
                L.append(f"    {rt} g{i}[{V}]; mlcb_load<{st}, {V}>(in{i} + "
                         f"({render_offset(a.index, {'idx': 'base_idx'})}), g{i});  // {a.name}: along r only")
                loads[i] = X.Val(f"g{i}[i]", vdt)
    if dependent_release(grid, block, cfg):
        L.append(dependent_release(grid, block, cfg))
    L.append("#pragma unroll")
    L.append(f"    for (int i = 0; i < {V}; ++i) {{")
    L.append(f"        const {it} i0 = base_idx + i * {o_r};")
    at_i0 = {"idx": "i0"}
    for i, a in enumerate(k.inputs):
        if i not in tile.along_t:
            continue
        acc = tile.along_t[i]
        st, rt = X.STORAGE_T[a.dtype], X.REG_T[a.dtype]
        vdt = X.promoted_load_dtype(a.dtype)
        if acc.mode == "bcast":
            L.append(f"        const {rt} v{i} = mlcb_load1<{st}>(in{i} + ({render_offset(a.index, at_i0)}));"
                     f"  // {a.name}")
            loads[i] = X.Val(f"v{i}", vdt)
        else:
            L.append(f"        {rt} v{i}[{V}]; mlcb_load<{st}, {V}>(in{i} + ({render_offset(a.index, at_i0)}), v{i});"
                     f"  // {a.name}")
            loads[i] = X.Val(f"v{i}[j]", vdt)
    for i, a in enumerate(k.outputs):
        L.append(f"        {X.REG_T[a.dtype]} o{i}[{V}];")
    L.append("#pragma unroll")
    L.append(f"        for (int j = 0; j < {V}; ++j) {{")
    refs: dict[str, X.Val] = {}
    elide = X.store_only_casts(k.body, k.out_expr, k.outputs)
    for temp, e in k.body:
        v = X.render_bind(temp, e, loads, refs, elide)
        L.append(f"            const {X.REG_T[v.dtype]} {temp} = {v.code};")
        refs[temp] = X.Val(temp, v.dtype, v.dim)
    for i, a in enumerate(k.outputs):
        v = X.render(k.out_expr[a.name], loads, refs)
        L.append(f"            o{i}[j] = {store_code(v, a.dtype)};  // {a.name}")
    L.append("        }")
    for i, a in enumerate(k.outputs):
        L.append(f"        mlcb_store<{X.STORAGE_T[a.dtype]}, {V}>(out{i} + ({render_offset(a.index, at_i0)}), o{i});")
    L.append("    }")
    L.append("}")
    spec = LaunchSpec(grid=grid, block=block, vector=V,
                      alg_bytes=algorithmic_bytes(k.inputs, k.outputs, numel))
    return "\n".join(L), spec
