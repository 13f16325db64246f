"""The reference's own test files, unmodified, on a GPU with this backend installed.

``oracle/ref.py`` installs the reference (package and ``tests/``) under
``oracle/_ref``.  A child pytest runs the seven test files that exercise the
compiled path -- eager parity over ten models x six pass configurations
(rtol 1e-5 / atol 1e-6), bit-identity across configurations, streamed =
persistent, large-logit softmax, float64 known-answer variance and LayerNorm,
the fp16 bars, layout and memory-planning checks, the bench-shaped models -- with
CUDA as the default device and ``mlc_compiler_b200.install()`` in effect
(``tests/reference_suite_plugin.py``), once under the reference's executor and
once under this package's.

Every numerics test must pass.  The only tests allowed to fail are the ones
that read the generated module as Python/Triton *text*
(``ast.parse(generate_module(...))``, ``"tl.max(" in src``, ``"for _base" in src``,
``tl.where(cmask, ...)``, ``.to(tl.float32)``), which cannot hold for a CUDA C++
translation unit; what they check is covered here by ``tests/test_emit.py``.
"""

import os
import pathlib
import re
import subprocess
import sys

import pytest

sys.path.insert(0, str(pathlib.Path(__file__).resolve().parent.parent / "oracle"))
import ref as reference_copy  # noqa: E402

HERE = pathlib.Path(__file__).resolve().parent
FILES = ["test_correctness.py", "test_reduction_fusion.py", "test_dtypes.py", "test_fusion.py",
         "test_bench_models.py", "test_layout.py", "test_memory_planning.py"]
#: tests that inspect Triton source text (by function name)
READS_TRITON_TEXT = re.compile(
    r"test_generated_reduction_source_parses|test_persistent_source_has_no_loop|"
    r"test_streamed_source_loops_and_rescales|test_masked_reduce_uses_the_right_identity|"
    r"test_row_statistics_load_as_scalars|test_narrow_loads_promote_and_stores_cast_back|"
    r"test_every_model_compiles_and_generates_valid_source")

_root = reference_copy.path()
pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(_root is None or not (_root / "tests" / FILES[0]).exists(),
                                 reason="the reference's tests are not installed under oracle/_ref")]


@pytest.mark.parametrize("mode", ["dropin", "native"])
def test_reference_suite_passes_on_the_gpu_with_this_backend(mode, tmp_path):
    env = dict(os.environ, MLCB_SUITE_MODE=mode, PYTHONDONTWRITEBYTECODE="1",
               MLC_CACHE_DIR=str(tmp_path / "cache"),
               PYTHONPATH=os.pathsep.join([str(HERE), str(HERE.parent), os.environ.get("PYTHONPATH", "")]))
    cmd = [sys.executable, "-m", "pytest", *[str(_root / "tests" / f) for f in FILES],
           "-p", "reference_suite_plugin", "-p", "no:cacheprovider", "-q", "-rf"]
    r = subprocess.run(cmd, cwd=str(_root), env=env, capture_output=True, text=True, timeout=1500)
    out = r.stdout + r.stderr
    tally = re.search(r"\[mlcb-suite\] runtimes=(\d+) on_cuda=(\d+) generated_kernels=(\d+)", out)
    assert tally, out[-3000:]
    runtimes, on_cuda, kernels = map(int, tally.groups())
    assert runtimes == on_cuda and on_cuda >= 100 and kernels >= 500, tally.group(0)
    summary = re.search(r"(?:(\d+) failed, )?(\d+) passed", out)
    assert summary, out[-3000:]
    failed, passed = int(summary.group(1) or 0), int(summary.group(2))
    failures = re.findall(r"^FAILED (\S+)", out, flags=re.M)
    unexpected = [f for f in failures if not READS_TRITON_TEXT.search(f)]
    assert not unexpected, "\n".join(unexpected) + "\n" + out[-3000:]
    assert len(failures) == failed
    assert not re.search(r"\d+ errors? in ", out), out[-3000:]        # e.g. a collection error
    assert passed >= 370, (passed, failed)
