"""The checked build of the library (``-DB200_SDPA_DEBUG``, ``libb200_sdpa_checked.so``).

Every global store whose address a kernel computes from decoded indices, every scratch slot and
every tensor-memory column range is verified before use; a violation is reported through the status
word (``B200_SDPA_ERR_BOUNDS``) and the access skipped -- the device never traps.  Two things are
shown here: the report arrives (a self-test kernel offers the checker an index past its limit; no
real access is wrong and nothing faults), and the small-shape matrices of the parity, backward,
paged-decode, prefill-form and random-shape tests run under the checked build without one report
(``tests/conftest.py`` reads the status word after every test when ``B200_SDPA_CHECKED=1``).
"""

import ctypes as C
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CHECKED_LIB = os.path.join(ROOT, "torch_neuronx_b200", "libb200_sdpa_checked.so")

needs_checked = pytest.mark.skipif(not os.path.exists(CHECKED_LIB),
                                   reason="checked library not built (python -m torch_neuronx_b200.build --checked)")


@needs_checked
def test_a_violation_is_reported_and_nothing_faults():
    import torch

    from torch_neuronx_b200 import _lib

    lib = C.CDLL(CHECKED_LIB)
    lib.b200_sdpa_checked_build.restype = C.c_int
    lib.b200_sdpa_debug_selftest.restype = C.c_int
    lib.b200_sdpa_debug_selftest.argtypes = [C.c_int, C.c_void_p, C.c_void_p]
    assert lib.b200_sdpa_checked_build() == 1
    status = torch.zeros(4, dtype=torch.int32, device="cuda:0")
    rc = lib.b200_sdpa_debug_selftest(0, C.c_void_p(status.data_ptr()),
                                      C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    torch.cuda.synchronize()
    # code, site, the offending index, its limit: the in-range offer (site 9901) left no trace
    assert status.tolist() == [_lib.ERR_BOUNDS, 9902, 8, 8]
    # the context is intact
    assert torch.ones(8, device="cuda:0").sum().item() == 8.0
    # the normal build has the entry point but no checks to exercise
    normal = _lib.load()
    assert normal.b200_sdpa_checked_build() == 0
    assert normal.b200_sdpa_debug_selftest(0, C.c_void_p(status.data_ptr()), None) == _lib.ERR_UNSUPPORTED


@needs_checked
def test_small_shape_matrices_run_clean_under_the_checked_build():
    env = dict(os.environ, B200_SDPA_CHECKED="1")
    files = ["tests/test_gpu_parity.py", "tests/test_gpu_backward.py", "tests/test_gpu_paged.py",
             "tests/test_gpu_prefill_modes.py", "tests/test_gpu_fuzz.py"]
    res = subprocess.run([sys.executable, "-m", "pytest", "-x", "-q", "-m", "gpu", "-p", "no:cacheprovider"] + files,
                         cwd=ROOT, env=env, capture_output=True, text=True, timeout=1500)
    tail = (res.stdout + res.stderr)[-3000:]
    assert res.returncode == 0, tail
    assert " passed" in res.stdout, tail
