"""Capture the benchmark schedules with the reference frontend.

    python -m mlc_compiler_b200.schedules.capture --reference /path/to/mlc-compiler

For every benchmark configuration this builds the model from
``mlc_compiler_b200.models`` (seeded synthetic weights), runs the reference's
capture + fusion + lowering + memory planning on it with the default ``Config``,
and writes the resulting kernel IR as ``<name>.json.gz`` beside this file.  The
files are what machines without the reference frontend load.
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
    args = ap.parse_args(argv)
    if args.reference:
        sys.path.insert(0, args.reference)
        sys.dont_write_bytecode = True

    from mlc_compiler_b200 import kir, models
    from mlc_compiler_b200.config import Config
    from mlc_compiler_b200.frontend import capture_schedule, schedule_path

    for stem, name, batch, dtype, variant, *rest in configurations():
        overrides = rest[0] if rest else {}
        stem = stem or models.schedule_name(name, batch, dtype)
        if args.only and args.only not in stem:
            continue
        path = schedule_path(stem)
        if path.exists() and not args.force:
            continue
        t0 = time.time()
        model, inputs = models.build(name, batch, dtype=dtype, **variant)
        sched = capture_schedule(model, inputs, Config(**overrides))
        sched.meta = {"model": name, "batch": batch, "seq": 128,
                      "dtype": str(dtype).replace("torch.", ""), "variant": variant,
                      "config": overrides}
        kir.dump(sched, path)
        print(f"{stem}: {len(sched)} kernels {sched.counts()} arena "
              f"{sched.arena_bytes / 1024:.1f} KiB  ({time.time() - t0:.1f}s)", flush=True)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
