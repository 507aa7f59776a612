"""Host-side decisions of the kernel library that need no device: into how many parts the many-token
product cuts its K range (the launcher's plan runs with 148 SMs when it finds no GPU)."""
import ctypes

import pytest


@pytest.fixture(scope="module")
def lib():
    from pytriton_llama_b200.ops import build
    try:
        path = build.library_path()
    except build.BuildError as e:                      # no compiler on this machine
        pytest.skip(f"the kernel library cannot be built here: {e}")
    lib = ctypes.CDLL(str(path))
    lib.ptl_gemm_tc_k_parts.argtypes = [ctypes.c_int] * 3
    lib.ptl_gemm_tc_k_parts.restype = ctypes.c_int
    return lib


def test_parts_of_the_k_range(lib):
    parts = lib.ptl_gemm_tc_k_parts
    assert parts(64, 2048, 8192) == 1                  # few tokens: the other kernel path splits K over a cluster
    assert parts(2048, 2048, 8192) == 1                # 128 tiles fill the SMs
    assert parts(4096, 8192, 2048) == 1
    assert parts(300, 2048, 100) == 1                  # K no multiple of 8: not this kernel at all
    for m, n, k in [(128, 2048, 2048), (300, 2048, 8192), (1000, 1024, 1024), (65, 128, 4096)]:
        p = parts(m, n, k)
        assert 2 <= p <= 8, (m, n, k, p)
        assert -(-k // 64) // p >= 8 or p == 1, (m, n, k, p)      # at least 8 blocks of 64 values per part
    assert parts(300, 2048, 256) == 1                  # too short a K range to cut
