"""``python -m mlc_compiler_b200`` -- inspect shipped schedules and their CUDA source.

    python -m mlc_compiler_b200 list
    python -m mlc_compiler_b200 show bert-base_b1_s128_float16
    python -m mlc_compiler_b200 source bert-base_b1_s128_float16 --kernel k13
    python -m mlc_compiler_b200 run bert-base_b1_s128_float16        # needs a CUDA device
    python -m mlc_compiler_b200 calibrate                            # needs a CUDA device

Counterpart of the reference's ``show`` / ``source`` / ``run`` commands
(``mlc/__main__.py:60-133``) for hosts that hold serialised schedules rather
than the frontend.  ``source --kernel`` prints the CUDA function behind one
schedule kernel (the reference's own ``--kernel`` filter splits on
``@triton.jit`` and therefore cannot cut CUDA text).
"""

from __future__ import annotations

import argparse
import sys


def main(argv=None) -> int:
    from . import Config, kir
    from .emit import generate_module
    from .frontend import SCHEDULE_DIR, load_schedule

    ap = argparse.ArgumentParser(prog="python -m mlc_compiler_b200", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="command", required=True)
    sub.add_parser("list")
    for name in ("show", "source", "run"):
        p = sub.add_parser(name)
        p.add_argument("schedule", help="shipped schedule name or a path to a .json[.gz] file")
        p.add_argument("--rewritten", action="store_true",
                       help="after producer forwarding, as the executor launches it")
        if name == "source":
            p.add_argument("--kernel", default=None)
    sub.add_parser("calibrate")
    args = ap.parse_args(argv)

    if args.command == "list":
        for p in sorted(SCHEDULE_DIR.glob("*.json.gz")):
            print(p.name[:-8])
        return 0
    if args.command == "calibrate":
        from . import devices

        print(devices.report(devices.calibrate("cuda"), devices.B200))
        return 0

    sched = load_schedule(args.schedule)
    if args.rewritten:
        from .rewrite import prepare

        sched = prepare(sched, Config())
    if args.command == "show":
        print(sched.format())
        return 0
    if args.command == "source":
        mod = generate_module(sched, Config())
        if args.kernel is None:
            print(mod.source)
            return 0
        if args.kernel not in mod.symbol:
            named = next((k for k in sched.kernels if k.name == args.kernel), None)
            if isinstance(named, kir.ExternKernel):
                print(f"{args.kernel} is an extern kernel and has no generated source: "
                      f"{named.summary()}", file=sys.stderr)
            else:
                print(f"no kernel named {args.kernel!r}", file=sys.stderr)
            return 1
        print(mod.kernel_source(args.kernel), end="")
        return 0

    # run: execute once on the GPU and report latency
    import torch

    from . import models
    from .executor import CompiledModel

    m = sched.meta
    model, inputs = models.build(m["model"], m["batch"], dtype=kir.torch_dtype(m["dtype"]),
                                 **m.get("variant", {}))
    cm = CompiledModel(load_schedule(args.schedule), model, Config(), "cuda")
    dev_in = [t.cuda() for t in inputs]
    for _ in range(5):
        cm(*dev_in)
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(50):
        cm(*dev_in)
    e.record()
    torch.cuda.synchronize()
    with torch.no_grad():
        want = model.cuda()(*dev_in)
    err = float((cm(*dev_in).float() - want.float()).abs().max())
    print(f"{args.schedule}: {len(cm.executed_schedule)} kernels launched "
          f"({cm.generated_launches} generated), {s.elapsed_time(e) / 50:.4f} ms per call, "
          f"max |compiled - eager| = {err:.3e}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
