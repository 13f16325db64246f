"""Seeded random kernel IR for differential tests of the emitter.

Builds pointwise and reduction kernels out of the whole scalar function table,
with random strided / broadcast / sliced operand views, mixed dtypes, mid-body
casts and boolean logic.  Every kernel comes with input buffers drawn so that
all functions stay in their domain (no log of a negative, no division by ~0),
which keeps the comparison meaningful: the oracle and the CUDA kernel must then
agree to the parity bar on every element.
"""

from __future__ import annotations

import math
import random

import torch

from mlc_compiler_b200 import kir

FLOATS = ("float32", "float16", "bfloat16")


class Gen:
    def __init__(self, seed: int):
        #: a second stream decides which inputs are parameters and which reductions get
        #: a second element output, so that the kernels themselves stay what they were
        import random as _random
        self.side = _random.Random(seed * 7919 + 13)
        #: input buffers declared as parameters (nothing writes them): the emitter loads
        #: those ahead of the grid-dependency wait
        self.params: list[str] = []
        self.r = random.Random(seed)
        self.g = torch.Generator().manual_seed(seed)

    # -- operand views ---------------------------------------------------------
    def view(self, space: tuple[int, ...], var: str | None = None):
        """(terms-by-dim, buffer numel, base): a random layout of ``space`` --
        contiguous, permuted, padded, sliced, or broadcast along some dims."""
        r = self.r
        rank = len(space)
        order = list(range(rank))
        style = r.choice(["contig", "contig", "perm", "pad", "bcast"])
        if style == "perm":
            r.shuffle(order)
        pad = r.choice([1, 2, 8]) if style == "pad" else 1
        strides = [0] * rank
        acc = 1
        for d in reversed(order):
            if style == "bcast" and r.random() < 0.5 and rank > 1:
                strides[d] = 0
            else:
                strides[d] = acc
                acc *= space[d] * (pad if d == order[-1] else 1)
        if all(s == 0 for s in strides):
            strides[-1] = 1
            acc = space[-1]
        base = r.choice([0, 0, 0, 8, 3])
        numel = base + sum((n - 1) * s for n, s in zip(space, strides)) + 1
        return strides, numel, base

    def index_map(self, groups, strides, base) -> kir.IndexMap:
        """``groups`` = [(var, dims)], dims a list of (size, in_stride)."""
        axes = []
        for var, dims in groups:
            numel = math.prod(n for n, _ in dims) if dims else 1
            terms, out_stride = [], numel
            for n, s in dims:
                out_stride //= n
                if n != 1 and s != 0:
                    terms.append((n, out_stride, s))
            axes.append(kir.Axis(var, numel, tuple(terms)))
        return kir.IndexMap(tuple(axes), base)

    # -- expressions -----------------------------------------------------------
    def float_expr(self, leaves: list[kir.Expr], depth: int) -> kir.Expr:
        r = self.r
        if depth == 0 or r.random() < 0.2:
            return r.choice(leaves)
        a = self.float_expr(leaves, depth - 1)
        kind = r.random()
        if kind < 0.35:
            fn = r.choice(["tanh", "erf", "sigmoid", "sin", "cos", "neg", "abs", "floor", "exp_s",
                           "log_p", "sqrt_p", "rsqrt_p", "recip_p"])
            safe = kir.Call("add", (kir.Call("abs", (a,)), kir.Const(0.5)))
            if fn == "floor":
                # discontinuous: only on exactly representable arguments, so that a
                # last-bit difference between libm implementations cannot flip it
                return kir.Call("floor", (kir.Call("mul", (r.choice(leaves[:1] or leaves), kir.Const(4.0))),))
            return {
                "exp_s": kir.Call("exp", (kir.Call("mul", (kir.Call("tanh", (a,)), kir.Const(2.0))),)),
                "log_p": kir.Call("log", (safe,)), "sqrt_p": kir.Call("sqrt", (safe,)),
                "rsqrt_p": kir.Call("rsqrt", (safe,)), "recip_p": kir.Call("reciprocal", (safe,)),
            }.get(fn) or kir.Call(fn, (a,))
        b = self.float_expr(leaves, depth - 1) if r.random() < 0.7 else kir.Const(
            r.choice([0.5, 2.0, -1.25, 3.0, 8.0, 1]))
        if kind < 0.75:
            fn = r.choice(["add", "sub", "mul", "maximum", "minimum", "div_p", "pow_p"])
            if fn == "div_p":
                return kir.Call("div", (a, kir.Call("add", (kir.Call("abs", (b,)), kir.Const(0.75)))))
            if fn == "pow_p":
                return kir.Call("pow", (kir.Call("add", (kir.Call("abs", (a,)), kir.Const(0.5))),
                                        kir.Call("tanh", (b,))))
            return kir.Call(fn, (a, b))
        if kind < 0.9:
            # comparisons read inputs directly (exact on both sides), never computed values
            la = r.choice(self.inputs_only)
            lb = r.choice(self.inputs_only + [kir.Const(0.0), kir.Const(0.5)])
            cmp = kir.Call(r.choice(["gt", "lt", "ge", "le", "eq", "ne"]), (la, lb))
            if r.random() < 0.4:
                other = kir.Call(r.choice(["gt", "lt"]), (r.choice(self.inputs_only), kir.Const(0.0)))
                cmp = kir.Call(r.choice(["logical_and", "logical_or"]), (cmp, other))
                if r.random() < 0.5:
                    cmp = kir.Call("logical_not", (cmp,))
            return kir.Call("where", (cmp, a, b))
        return kir.Cast(kir.Cast(a, r.choice(["float16", "bfloat16"])), "float32")

    def tensor(self, numel: int, dtype: str) -> torch.Tensor:
        if dtype == "int64":
            return torch.randint(-9, 10, (numel,), generator=self.g)
        if dtype == "bool":
            return torch.rand(numel, generator=self.g) > 0.5
        t = torch.randn(numel, generator=self.g) * 1.5
        return t.to(kir.torch_dtype(dtype))

    # -- kernels -----------------------------------------------------------------
    def pointwise(self, name: str):
        r = self.r
        rank = r.randint(1, 3)
        space = tuple(r.choice([1, 2, 3, 4, 8, 16, 24]) for _ in range(rank))
        if math.prod(space) < 2:
            space = space[:-1] + (8,)
        dt = r.choice(FLOATS)
        buffers, specs, inputs = {}, {}, []
        for i in range(r.randint(1, 4)):
            idt = dt if r.random() < 0.8 else r.choice(FLOATS + ("int64",))
            strides, numel, base = self.view(space)
            bname = f"{name}_in{i}"
            is_param = self.side.random() < 0.4
            specs[bname] = kir.BufferSpec(bname, (numel,), idt, "param" if is_param else "input")
            if is_param:
                self.params.append(bname)
            buffers[bname] = self.tensor(numel, idt)
            m = self.index_map([("idx", list(zip(space, strides)))], strides, base)
            inputs.append(kir.Operand(bname, bname, idt, m))
        leaves = [kir.Load(i) if inputs[i].dtype != "int64" else kir.Cast(kir.Load(i), "float32")
                  for i in range(len(inputs))]
        self.inputs_only = list(leaves)
        body = []
        for t in range(r.randint(1, 4)):
            e = self.float_expr(leaves + [kir.Ref(n) for n, _ in body], r.randint(1, 3))
            body.append((f"t{t}", e))
        outs, out_expr = [], {}
        n = math.prod(space)
        for o in range(r.randint(1, 2)):
            odt = r.choice([dt, dt, "float32", "bool", "int64"])
            oname = f"{name}_out{o}"
            specs[oname] = kir.BufferSpec(oname, (n,), odt, "output")
            buffers[oname] = torch.zeros(n, dtype=kir.torch_dtype(odt))
            e = kir.Ref(r.choice(body)[0])
            if odt == "bool":
                e = kir.Call("gt", (r.choice(leaves), kir.Const(0.25)))
            elif odt == "int64":
                e = kir.Cast(kir.Call("floor", (kir.Call("mul", (r.choice(leaves), kir.Const(4.0))),)),
                             "int64")
            elif odt != "float32":
                e = kir.Cast(e, odt)
            outs.append(kir.Operand(oname, oname, odt,
                                    kir.IndexMap((kir.Axis("idx", n, ((n, 1, 1),) if n > 1 else ()),))))
            out_expr[oname] = e
        return kir.PointwiseKernel(name, space, inputs, outs, body, out_expr, ["fuzz"]), specs, buffers

    def reduction(self, name: str, streamed: bool):
        r = self.r
        rows = r.choice([1, 3, 5, 16, 33])
        cols = r.choice([4, 7, 24, 64, 100, 257] if not streamed else [24, 100, 257, 1100])
        dt = r.choice(FLOATS)
        buffers, specs, inputs = {}, {}, []
        for i in range(r.randint(1, 3)):
            kind = r.choice(["full", "full", "col", "row"]) if i else "full"
            bname = f"{name}_in{i}"
            if kind == "full":
                pad = r.choice([0, 0, 8])
                numel = rows * (cols + pad)
                m = self.index_map([("row", [(rows, cols + pad)]), ("col", [(cols, 1)])], None, 0)
            elif kind == "col":
                numel = cols
                m = self.index_map([("row", [(rows, 0)]), ("col", [(cols, 1)])], None, 0)
            else:
                numel = rows
                m = self.index_map([("row", [(rows, 1)]), ("col", [(cols, 0)])], None, 0)
            is_param = self.side.random() < 0.5
            specs[bname] = kir.BufferSpec(bname, (numel,), dt, "param" if is_param else "input")
            if is_param:
                self.params.append(bname)
            buffers[bname] = self.tensor(numel, dt)
            inputs.append(kir.Operand(bname, bname, dt, m))
        leaves = [kir.Load(i) for i in range(len(inputs))]
        self.inputs_only = list(leaves)
        steps = [kir.Bind("t0", self.float_expr(leaves, 2))]
        kind1 = r.choice(["sum", "max", "min"])
        steps.append(kir.Reduce("r1", kind1, kir.Ref("t0")))
        if kind1 == "max" and r.random() < 0.6:           # softmax shape
            steps += [kir.Bind("t2", kir.Call("sub", (kir.Ref("t0"), kir.Ref("r1")))),
                      kir.Bind("t3", kir.Call("exp", (kir.Ref("t2"),))),
                      kir.Reduce("r4", "sum", kir.Ref("t3")),
                      kir.Bind("t5", kir.Call("div", (kir.Ref("t3"), kir.Ref("r4"))))]
            final = "t5"
        else:
            steps += [kir.Bind("t2", kir.Call("div", (kir.Ref("r1"), kir.Const(float(cols))))),
                      kir.Bind("t3", kir.Call("sub", (kir.Ref("t0"), kir.Call("tanh", (kir.Ref("t2"),))))),
                      kir.Bind("t4", kir.Call("mul", (kir.Ref("t3"), kir.Ref("t3")))),
                      kir.Reduce("r5", "sum", kir.Ref("t4")),
                      kir.Bind("t6", kir.Call("mul", (kir.Ref("t3"), kir.Call("rsqrt", (
                          kir.Call("add", (kir.Call("div", (kir.Ref("r5"), kir.Const(float(cols)))),
                                           kir.Const(1e-5))),))))),
                      ]
            final = "t6"
        steps.append(kir.Bind("t9", kir.Cast(kir.Ref(final), dt)))
        elem = f"{name}_out0"
        specs[elem] = kir.BufferSpec(elem, (rows * cols,), dt, "output")
        buffers[elem] = torch.zeros(rows * cols, dtype=kir.torch_dtype(dt))
        outs = [kir.Operand(elem, elem, dt, self.index_map(
            [("row", [(rows, cols)]), ("col", [(cols, 1)])], None, 0))]
        out_expr = {elem: kir.Ref("t9")}
        if not streamed and self.side.random() < 0.4:
            # a second element output whose value exists before the first reduction
            # (the residual sum a LayerNorm also emits): stored in the first phase
            early = f"{name}_out2"
            specs[early] = kir.BufferSpec(early, (rows * cols,), dt, "output")
            buffers[early] = torch.zeros(rows * cols, dtype=kir.torch_dtype(dt))
            outs.append(kir.Operand(early, early, dt, self.index_map(
                [("row", [(rows, cols)]), ("col", [(cols, 1)])], None, 0)))
            steps.insert(1, kir.Bind("t0c", kir.Cast(kir.Ref("t0"), dt)))
            out_expr[early] = kir.Ref("t0c")
        row_outputs = set()
        if r.random() < 0.5:
            rname = f"{name}_out1"
            specs[rname] = kir.BufferSpec(rname, (rows,), "float32", "output")
            buffers[rname] = torch.zeros(rows)
            outs.append(kir.Operand(rname, rname, "float32", self.index_map(
                [("row", [(rows, 1)])], None, 0)))
            out_expr[rname] = kir.Ref("r1")
            row_outputs.add(rname)
        k = kir.ReductionKernel(name, (rows,), (cols,), inputs, outs, steps, out_expr, row_outputs,
                                streamed, ["fuzz"])
        return k, specs, buffers


def special_cases():
    """Hand-shaped kernels for the code paths random small shapes cannot reach:
    register-tile transposes, 256-bit accesses, narrow integer dtypes, fp64."""
    g = torch.Generator().manual_seed(5)
    kernels, specs, buffers = [], {}, {}

    def buf(name, numel, dtype, kind="input", fill=None):
        specs[name] = kir.BufferSpec(name, (numel,), dtype, kind)
        if fill is None:
            t = torch.zeros(numel, dtype=kir.torch_dtype(dtype))
        elif dtype in kir.FLOAT_DTYPES:
            t = (torch.randn(numel, generator=g) * 1.5).to(kir.torch_dtype(dtype))
        elif dtype == "uint8":
            t = torch.randint(0, 100, (numel,), generator=g).to(torch.uint8)
        else:
            t = torch.randint(-50, 50, (numel,), generator=g).to(kir.torch_dtype(dtype))
        buffers[name] = t
        return name

    def flat(n):
        return kir.IndexMap((kir.Axis("idx", n, ((n, 1, 1),)),))

    # 1/2: transposes [B, R, T] <- storage [B, T, R], with a t-contiguous addend and a per-r bias
    for tag, dt, (B, R, T) in (("tr16", "float16", (2, 128, 64)), ("trbf", "bfloat16", (3, 64, 96))):
        n = B * R * T
        x = buf(f"{tag}_x", n, dt, fill=1)
        y = buf(f"{tag}_y", n, dt, fill=1)
        b = buf(f"{tag}_b", R, dt, fill=1)
        o = buf(f"{tag}_o", n, dt, "output")
        ax = lambda terms: kir.IndexMap((kir.Axis("idx", n, terms),))
        k = kir.PointwiseKernel(
            tag, (B, R, T),
            [kir.Operand(x, x, dt, ax(((B, R * T, R * T), (R, T, 1), (T, 1, R)))),
             kir.Operand(y, y, dt, flat(n)),
             kir.Operand(b, b, dt, ax(((R, T, 1),)))],
            [kir.Operand(o, o, dt, flat(n))],
            [("t0", kir.Call("add", (kir.Load(0), kir.Load(2)))),
             ("t1", kir.Call("mul", (kir.Ref("t0"), kir.Call("tanh", (kir.Load(1),)))))],
            {o: kir.Cast(kir.Ref("t1"), dt)}, ["transpose"])
        kernels.append(k)

    # 3: 24 MB streaming kernel -> 256-bit accesses
    n = 1 << 22
    x, y, o = buf("wide_x", n, "float16", fill=1), buf("wide_y", n, "float16", fill=1), \
        buf("wide_o", n, "float16", "output")
    kernels.append(kir.PointwiseKernel(
        "wide", (n,), [kir.Operand(x, x, "float16", flat(n)), kir.Operand(y, y, "float16", flat(n))],
        [kir.Operand(o, o, "float16", flat(n))],
        [("t0", kir.Call("add", (kir.Load(0), kir.Call("mul", (kir.Load(1), kir.Const(2.0))))))],
        {o: kir.Cast(kir.Ref("t0"), "float16")}, ["wide"]))

    # 4: every narrow integer dtype in and out
    n = 1000
    for dt in ("int32", "int16", "int8", "uint8"):
        x = buf(f"i_{dt}_x", n, dt, fill=1)
        o = buf(f"i_{dt}_o", n, dt, "output")
        f = buf(f"i_{dt}_f", n, "float32", "output")
        kernels.append(kir.PointwiseKernel(
            f"ints_{dt}", (n,), [kir.Operand(x, x, dt, flat(n))],
            [kir.Operand(o, o, dt, flat(n)), kir.Operand(f, f, "float32", flat(n))],
            [("t0", kir.Call("abs", (kir.Load(0),))),
             ("t1", kir.Call("minimum", (kir.Ref("t0"), kir.Const(40)))),
             ("t2", kir.Call("mul", (kir.Cast(kir.Ref("t1"), "float32"), kir.Const(0.5))))],
            {o: kir.Cast(kir.Ref("t1"), dt), f: kir.Ref("t2")}, ["ints"]))

    # 5: fp64 pointwise + row reduction
    rows, cols = 7, 50
    x = buf("d_x", rows * cols, "float64", fill=1)
    o = buf("d_o", rows * cols, "float64", "output")
    r = buf("d_r", rows, "float64", "output")
    rc = kir.IndexMap((kir.Axis("row", rows, ((rows, 1, cols),)), kir.Axis("col", cols, ((cols, 1, 1),))))
    kernels.append(kir.ReductionKernel(
        "fp64", (rows,), (cols,), [kir.Operand(x, x, "float64", rc)],
        [kir.Operand(o, o, "float64", rc),
         kir.Operand(r, r, "float64", kir.IndexMap((kir.Axis("row", rows, ((rows, 1, 1),)),)))],
        [kir.Bind("t0", kir.Call("exp", (kir.Call("mul", (kir.Load(0), kir.Const(0.25))),))),
         kir.Reduce("r1", "sum", kir.Ref("t0")),
         kir.Bind("t2", kir.Call("div", (kir.Ref("t0"), kir.Ref("r1"))))],
        {o: kir.Ref("t2"), r: kir.Ref("r1")}, {r}, False, ["fp64"]))
    # 6: rows gathered from a table by id (ids strided, out of range at both ends,
    #    table at an offset), persistent and streamed, three dtypes
    for tag, dt, idt, two_pass, (rows, width, table_rows) in (
            ("gath16", "float16", "int64", False, (37, 96, 11)),
            ("gathbf", "bfloat16", "int32", False, (64, 256, 5)),
            ("gath32", "float32", "int64", True, (9, 2500, 7))):
        skip = 2 * width                                      # table starts two rows into its buffer
        tab = buf(f"{tag}_t", skip + table_rows * width, dt, fill=1)
        ids = buf(f"{tag}_i", 2 * rows, idt, fill=1)          # values in [-50, 50): some outside the table
        y = buf(f"{tag}_y", rows * width, dt, fill=1)
        o = buf(f"{tag}_o", rows * width, dt, "output")
        r = buf(f"{tag}_r", rows, "float32", "output")
        rc = kir.IndexMap((kir.Axis("row", rows, ((rows, 1, width),)),
                           kir.Axis("col", width, ((width, 1, 1),))))
        kernels.append(kir.ReductionKernel(
            tag, (rows,), (width,),
            [kir.Operand(tab, tab, dt, kir.IndexMap(
                (kir.Axis("row", table_rows, ((table_rows, 1, width),)),
                 kir.Axis("col", width, ((width, 1, 1),))), skip), (2, table_rows)),
             kir.Operand(y, y, dt, rc),
             kir.Operand(ids, ids, idt, kir.IndexMap(
                 (kir.Axis("row", rows, ((rows, 1, 2),)), kir.Axis("col", width, ())), 1))],
            [kir.Operand(o, o, dt, rc),
             kir.Operand(r, r, "float32", kir.IndexMap((kir.Axis("row", rows, ((rows, 1, 1),)),)))],
            [kir.Bind("t0", kir.Call("add", (kir.Load(0), kir.Call("mul", (kir.Load(1), kir.Const(0.5)))))),
             kir.Reduce("r1", "max", kir.Ref("t0")),
             kir.Bind("t2", kir.Call("sub", (kir.Ref("t0"), kir.Ref("r1")))),
             kir.Bind("t3", kir.Cast(kir.Ref("t2"), dt))],
            {o: kir.Ref("t3"), r: kir.Ref("r1")}, {r}, two_pass, ["embedding"]))
    return kir.Schedule("special", kernels, specs), buffers
