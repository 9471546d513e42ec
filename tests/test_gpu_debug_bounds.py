"""The GPU suites against the checked build of the library.

`python loom_kernels_b200/build.py --debug-bounds` compiles the decode and append kernels with
every computed global index compared with the length of the operand it indexes (page-table
entries, query / output / LSE rows, workspace states, pool slots, page coordinates of the copies).
An index outside its operand would be recorded in the provider's status word (0x1000 | site) and
the access skipped; nothing traps.  This test runs the small decode and append cases, the guard
cases included (out-of-range pages, malformed page tables, duplicate slots), against that build
in a child process; the runs of those suites assert that their provider's status word is zero
after every call.  It is the stand-in for a memory checker where none can be run on the device.
"""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_decode_and_append_suites_leave_no_index_outside_its_operand():
    sys.path.insert(0, ROOT)
    from loom_kernels_b200 import build as lib_build
    library = lib_build.build(variant="debug-bounds")
    env = dict(os.environ, LOOM_B200_LIBRARY=library)
    result = subprocess.run(
        [sys.executable, "-m", "pytest", "tests/test_gpu_paged_decode.py",
         "tests/test_gpu_rope_append.py", "tests/test_gpu_state_merge.py",
         "tests/test_gpu_indices_capacity.py", "tests/test_gpu_graph.py", "-x", "-q",
         "-p", "no:cacheprovider"],
        cwd=ROOT, env=env, capture_output=True, text=True, timeout=1500)
    assert result.returncode == 0, (result.stdout + result.stderr)[-4000:]
    assert " passed" in result.stdout
