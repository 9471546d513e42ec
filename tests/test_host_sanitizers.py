"""The host library under AddressSanitizer and UndefinedBehaviorSanitizer.

`compute-sanitizer` is not available where this suite runs, and most of the library's own risk
sits in host code anyway: handle lifetimes, moved and consumed objects, operand tables, error
payloads.  `python loom_kernels_b200/build.py --asan` builds the library with both sanitizers;
this test runs the host-side suites (fake driver, no device) against that build in a child
process and fails on any report.
"""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def runtime_of(name):
    path = subprocess.run(["gcc", f"-print-file-name={name}"], capture_output=True,
                          text=True).stdout.strip()
    return path if os.path.isabs(path) and os.path.exists(path) else None


def test_host_suites_are_clean_under_asan_and_ubsan():
    asan, ubsan = runtime_of("libasan.so"), runtime_of("libubsan.so")
    if not asan or not ubsan:
        pytest.skip("the compiler's sanitizer runtimes are not installed")
    sys.path.insert(0, ROOT)
    from loom_kernels_b200 import build as lib_build
    library = lib_build.build(variant="asan")
    env = dict(os.environ, LD_PRELOAD=f"{asan}:{ubsan}", LOOM_B200_LIBRARY=library,
               ASAN_OPTIONS="detect_leaks=0:abort_on_error=0:exitcode=66",
               UBSAN_OPTIONS="print_stacktrace=1:halt_on_error=0")
    result = subprocess.run(
        [sys.executable, "-m", "pytest", "tests/test_host_runtime.py", "tests/test_host_prefill.py",
         "tests/test_oracle_contract.py", "-x", "-q", "-p", "no:cacheprovider"],
        cwd=ROOT, env=env, capture_output=True, text=True, timeout=1200)
    report = result.stdout + result.stderr
    assert "ERROR: AddressSanitizer" not in report, report[-4000:]
    assert "runtime error:" not in report, report[-4000:]
    assert result.returncode == 0, report[-4000:]
