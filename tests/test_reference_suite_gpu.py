"""The reference's own test files, run against this library.

Two ways, both in a child process so that the reference's `tests/conftest.py` and module names do not mix with ours:

* `test_reference_tests_against_this_package`: the reference's tests/test_quantize.py and tests/test_gemm.py (whole
  files) and the stable-API part of tests/test_attention.py (test_flash_attn_gqa_and_kv_cache,
  test_flash_attn_rejects_bad_gqa_and_causal_shapes, lines 229-257) import `kernelforge` = THIS package.
* `test_integration_shim_under_the_reference_ops`: the reference's own kernelforge/{ops,quantize,modules}.py are
  used unchanged; the ctypes shim printed in INTEGRATION.md is extracted from that file verbatim and installed as
  `kernelforge._C` (the swap INTEGRATION.md describes), and the same reference tests run on top of it.

The reference's sources are not part of this repository.  Point KFB_REFERENCE_ROOT at a checkout of the reference
(a directory holding its `kernelforge/` and `tests/`); without it these tests are skipped.
"""

import os
import re
import shutil
import subprocess
import sys
from pathlib import Path

import pytest

from conftest import ROOT

pytestmark = pytest.mark.gpu

REF = os.environ.get("KFB_REFERENCE_ROOT", "")
needs_ref = pytest.mark.skipif(not (REF and (Path(REF) / "tests" / "test_gemm.py").exists()),
                               reason="KFB_REFERENCE_ROOT does not point at a checkout of the reference")

STABLE_ATTENTION = "test_flash_attn_gqa_and_kv_cache or test_flash_attn_rejects_bad_gqa_and_causal_shapes"


def _run(pythonpath: list[str], tests_dir: Path, extra_env: dict | None = None) -> str:
    env = dict(os.environ, PYTHONPATH=os.pathsep.join(pythonpath))
    env.update(extra_env or {})
    out = []
    for args in (["test_quantize.py", "test_gemm.py"], ["test_attention.py", "-k", STABLE_ATTENTION]):
        res = subprocess.run([sys.executable, "-m", "pytest", "-q", "-x", "-p", "no:cacheprovider", *args],
                             cwd=tests_dir, env=env, capture_output=True, text=True, timeout=1500)
        tail = "\n".join(res.stdout.strip().splitlines()[-15:])
        print(tail)
        assert res.returncode == 0, f"reference tests {args} failed:\n{tail}\n{res.stderr[-2000:]}"
        out.append(tail.splitlines()[-1])
    return " | ".join(out)


def _copy_tests(tmp_path: Path) -> Path:
    dst = tmp_path / "ref_tests"
    shutil.copytree(Path(REF) / "tests", dst)
    return dst


@needs_ref
def test_reference_tests_against_this_package(tmp_path):
    tests_dir = _copy_tests(tmp_path)
    # tests/test_attention.py names the reference's ablation kernels at import time (IMPLS, ATTN_V1_CONFIGS, ...);
    # they are out of scope here, so placeholders let the module import and only the stable-API tests are selected.
    (tests_dir / "conftest.py").write_text((tests_dir / "conftest.py").read_text() + '''

import kernelforge.ops as _ops
def _not_built(*a, **k):
    raise NotImplementedError("ablation kernel of the reference, not part of this library")
for _n in ("attn_naive", "flash_attn_v1", "flash_attn_v2", "flash_attn_v3", "flash_attn_v4"):
    if not hasattr(_ops, _n):
        setattr(_ops, _n, _not_built)
for _n in ("ATTN_V1_CONFIGS", "ATTN_V4_CONFIGS"):
    if not hasattr(_ops, _n):
        setattr(_ops, _n, ())
''')
    summary = _run([str(ROOT / "kernel-forge_b200")], tests_dir)
    print("reference tests against this package:", summary)


@needs_ref
def test_integration_shim_under_the_reference_ops(tmp_path):
    tests_dir = _copy_tests(tmp_path)
    pkg = tmp_path / "site" / "kernelforge"
    pkg.mkdir(parents=True)
    for name in ("__init__.py", "ops.py", "quantize.py", "modules.py", "bench_utils.py"):
        src = Path(REF) / "kernelforge" / name
        if src.exists():
            shutil.copy(src, pkg / name)
    text = (ROOT / "INTEGRATION.md").read_text()
    blocks = re.findall(r"```python\n(.*?)```", text, flags=re.S)
    shim = next(b for b in blocks if "def attn_v4" in b and "def int4_gemv" in b and "def int4_gemm" in b)
    (pkg / "_C.py").write_text(shim)   # `from kernelforge import _C` in the reference's ops.py now finds the shim
    lib_dir = str(ROOT / "kernel-forge_b200" / "kernelforge")
    ld = os.pathsep.join(p for p in (lib_dir, os.environ.get("LD_LIBRARY_PATH", "")) if p)
    summary = _run([str(tmp_path / "site")], tests_dir, {"LD_LIBRARY_PATH": ld})
    print("reference tests on the reference's ops.py + INTEGRATION.md shim:", summary)
