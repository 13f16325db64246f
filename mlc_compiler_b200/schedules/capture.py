"""Capture the benchmark schedules with the reference frontend.

    python -m mlc_compiler_b200.schedules.capture --reference /path/to/mlc-compiler

For every benchmark configuration this builds the model from
``mlc_compiler_b200.models`` (seeded synthetic weights), runs the reference's
capture + fusion + lowering + memory planning on it, and writes the resulting
kernel IR as ``<name>.json.gz`` beside this file.  The files are what machines
without the reference frontend load.

The fusion passes price their decisions with three cost-model constants
(``flops_per_byte``, ``launch_overhead_bytes``, ``graph_launch_overhead_bytes``,
``mlc/config.py:36-52``).  ``--profile b200`` (the default) takes them from this
package's B200 device profile, ``--profile default`` leaves the reference's A100
defaults; ``--check-profile`` captures every configuration both ways and reports
whether the schedules differ (they do not for any shipped configuration: every
fusion and recompute decision of these models is far from the margin, so the
files are valid under either profile).
"""

from __future__ import annotations

import argparse
import sys
import time

import torch


def configurations():
    """(file stem, model name, batch, dtype, variant kwargs[, Config overrides])."""
    out = []
    f16, bf16, f32 = torch.float16, torch.bfloat16, torch.float32
    out.append(("encoder-block_b1_s128_float32", "encoder-block", 1, f32, {}))
    for dt in (f16, bf16):
        for b in (1, 4, 8, 16, 32):
            if dt is bf16 and b == 1:
                pass
            out.append((None, "bert-base", b, dt, {}))
            out.append((None, "gpt2-small", b, dt, {}))
    out.append((None, "bert-base", 1, f32, {}))
    # the variant the reference itself ships: exact GELU, untied head
    out.append(("gpt2-small-ref_b1_s128_float16", "gpt2-small", 1, f16,
                {"gelu": "erf", "tied_head": False}))
    # every row longer than 64 streams (the reference's `--max-row 64` check)
    out.append(("bert-base-streamed_b1_s128_float16", "bert-base", 1, f16, {},
                {"max_persistent_row": 64}))
    out.append(("gpt2-small-streamed_b1_s128_float16", "gpt2-small", 1, f16, {},
                {"max_persistent_row": 64}))
    for dt in (f16, bf16):
        for b in (1, 8, 32):
            for m in ("micro-layernorm", "micro-softmax", "micro-gelu"):
                out.append((None, m, b, dt, {}))
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--reference", default=None, help="checkout of the reference (adds it to sys.path)")
    ap.add_argument("--only", default=None, help="substring filter on the file stem")
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--profile", choices=("b200", "default"), default="b200",
                    help="device profile the cost model is priced with")
    ap.add_argument("--check-profile", action="store_true",
                    help="capture each configuration with both profiles and report differences; "
                         "writes nothing")
    args = ap.parse_args(argv)
    if args.reference:
        sys.path.insert(0, args.reference)
        sys.dont_write_bytecode = True

    from mlc_compiler_b200 import devices, kir, models
    from mlc_compiler_b200.config import Config
    from mlc_compiler_b200.frontend import capture_schedule, schedule_path

    def priced(overrides, profile):
        base = Config(**overrides)
        return devices.B200.to_config(base) if profile == "b200" else base

    differing = 0
    for stem, name, batch, dtype, variant, *rest in configurations():
        overrides = rest[0] if rest else {}
        stem = stem or models.schedule_name(name, batch, dtype)
        if args.only and args.only not in stem:
            continue
        if args.check_profile:
            model, inputs = models.build(name, batch, dtype=dtype, **variant)
            a = capture_schedule(model, inputs, priced(overrides, "default"))
            b = capture_schedule(model, inputs, priced(overrides, "b200"))
            same = kir.dumps(a) == kir.dumps(b)
            differing += not same
            print(f"{stem}: {'identical' if same else f'DIFFERENT {a.counts()} vs {b.counts()}'}",
                  flush=True)
            continue
        path = schedule_path(stem)
        if path.exists() and not args.force:
            continue
        t0 = time.time()
        model, inputs = models.build(name, batch, dtype=dtype, **variant)
        sched = capture_schedule(model, inputs, priced(overrides, args.profile))
        sched.meta = {"model": name, "batch": batch, "seq": 128,
                      "dtype": str(dtype).replace("torch.", ""), "variant": variant,
                      "config": overrides, "cost_profile": args.profile}
        kir.dump(sched, path)
        print(f"{stem}: {len(sched)} kernels {sched.counts()} arena "
              f"{sched.arena_bytes / 1024:.1f} KiB  ({time.time() - t0:.1f}s)", flush=True)
    if args.check_profile:
        print(f"{differing} configuration(s) differ between the A100-default and the B200 profile")
        return 1 if differing else 0
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
