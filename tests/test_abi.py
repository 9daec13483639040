"""CPU-side checks of the C-ABI library: it loads, exports every function the header
declares, and refuses to work without a GPU instead of falling back."""
import ctypes as C
import re
from pathlib import Path

import pytest

from candy_b200 import abi

ROOT = Path(__file__).resolve().parent.parent


def declared_functions():
    names = []
    for header in sorted((ROOT / "include").glob("*.h")):
        text = re.sub(r"/\*.*?\*/", "", header.read_text(), flags=re.S)
        names += re.findall(r"\b(cq_[a-z0-9_]+)\s*\(", text)
    return sorted(set(names))


def test_header_declares_the_expected_surface():
    names = declared_functions()
    for must in ("cq_ctx_create", "cq_qmatmul", "cq_qmatmul_host", "cq_dequantize", "cq_quantize_rows",
                 "cq_quantize_q8_1", "cq_synchronize", "cq_malloc", "cq_memcpy_h2d", "cq_memcpy_d2h"):
        assert must in names


def test_library_loads_and_exports_every_declared_symbol():
    handle = abi.lib()
    for name in declared_functions():
        assert hasattr(handle, name), f"{name} is declared in include/*.h but not exported by libcandyq.so"


def test_python_binding_covers_every_declared_symbol():
    bound = set(abi.SIGNATURES) | set(abi._OTHER_RESTYPE)
    assert set(declared_functions()) <= bound


def test_status_strings_and_sizes():
    handle = abi.lib()
    assert handle.cq_status_string(0) == b"ok"
    assert b"invalid" in handle.cq_status_string(abi.ERR_INVALID_ARG)
    assert b"sm_100a" in handle.cq_version()
    assert handle.cq_blocks_bytes(abi.Q4_0, 4096, 4096) == 9437184
    assert handle.cq_blocks_bytes(abi.Q8_0, 4096, 4096) == 17825792
    assert handle.cq_blocks_bytes(abi.Q4_0, 4, 40) == 0
    assert handle.cq_blocks_bytes(5, 4, 64) == 0


def test_no_gpu_means_failure_not_fallback():
    if abi.device_count() > 0:
        pytest.skip("a GPU is present; the no-GPU behaviour is checked on CPU-only machines")
    ctx = C.c_void_p()
    assert abi.lib().cq_ctx_create(0, C.byref(ctx)) == abi.ERR_CUDA
    assert not ctx.value
    from candy_b200.backend import CudaDevice
    with pytest.raises(abi.CandyqError):
        CudaDevice(0)


def test_null_context_is_rejected():
    handle = abi.lib()
    assert handle.cq_synchronize(None) == abi.ERR_INVALID_ARG
    assert handle.cq_qmatmul(None, 2, 0, 0, None, 1, 32, 32, None, 1, None, 1) == abi.ERR_INVALID_ARG
