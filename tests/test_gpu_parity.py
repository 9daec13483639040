"""GPU parity tests: every result comes from libcandyq through its C ABI (ctypes) and is
checked against the CPU oracle.  Bars: bit-exact for bytes and dequantized weights;
max|y - y_ref| / max|y_ref| <= 1e-3 for f32 matmul outputs (tighter "expected" bounds are
asserted too, so a summation bug cannot hide inside the 1e-3 allowance)."""
import ctypes as C
from pathlib import Path

import numpy as np
import pytest

from helpers import REL_TOL, make_case, rel_err
from oracle import oracle_c as oc

pytestmark = pytest.mark.gpu

GOLDEN = Path(__file__).resolve().parent / "golden" / "qmatmul_small.npz"
QT_ORDERS = [(oc.Q4_0, 0), (oc.Q4_0, 1), (oc.Q8_0, 0)]


def bits(a):
    return np.asarray(a, dtype=np.float32).view(np.uint32)


def gpu_dequantize(device, qt, order, blocks):
    from candy_b200.backend import QStorage
    nb = blocks.size // oc.BLOCK_BYTES[qt]
    qs = QStorage.from_blocks(device, qt, order, 1, nb * 32, blocks)
    return qs.dequantize().data()


def gpu_qmatmul(device, qt, order, x, blocks, n, actmode=0):
    from candy_b200.backend import QStorage
    m, k = x.shape
    qs = QStorage.from_blocks(device, qt, order, n, k, blocks)
    xs = device.storage_from_slice(x)
    y = xs.matmul(qs, 1, m, n, k, actmode).data().reshape(m, n)
    device.synchronize()
    return y


# ---- dequantize: bit-exact ---------------------------------------------------------------
@pytest.mark.parametrize("qt,order", QT_ORDERS)
def test_dequantize_bit_exact_random_and_edge_scales(device, qt, order):
    rng = np.random.default_rng(100 + qt + order)
    bb = oc.BLOCK_BYTES[qt]
    nblk = 4099  # not a multiple of anything convenient
    blocks = rng.integers(0, 256, size=(nblk, bb), dtype=np.uint8)
    scales = [0x0000, 0x8000, 0x0001, 0x03FF, 0x0400, 0x7BFF, 0xFBFF, 0x7C00, 0xFC00, 0x7E00, 0x7C01, 0xFE01]
    for i, s in enumerate(scales):
        blocks[i, 0], blocks[i, 1] = s & 0xFF, s >> 8
    # keep the random scales finite so the bulk of the comparison is about values, not NaNs
    hi = blocks[len(scales):, 1]
    hi[(hi & 0x7C) == 0x7C] &= 0xBF
    got = gpu_dequantize(device, qt, order, blocks.reshape(-1))
    want = oc.dequantize(qt, order, blocks.reshape(-1))
    assert (bits(got) == bits(want)).all()


def test_dequantize_all_65536_scales(device):
    hs = np.arange(65536, dtype=np.uint16)
    blocks = np.zeros((65536, 18), dtype=np.uint8)
    blocks[:, 0], blocks[:, 1] = hs & 0xFF, hs >> 8
    blocks[:, 2:] = np.array([j | ((15 - j) << 4) for j in range(16)], dtype=np.uint8)
    for order in (0, 1):
        got = gpu_dequantize(device, oc.Q4_0, order, blocks.reshape(-1))
        assert (bits(got) == bits(oc.dequantize(oc.Q4_0, order, blocks.reshape(-1)))).all()


def test_dequantize_unaligned_output_and_empty(device):
    lib, ctx = device._lib, device.ctx
    rng = np.random.default_rng(5)
    blocks = rng.integers(0, 256, size=(33, 18), dtype=np.uint8)
    blocks[:, 1] &= 0x3F
    buf = device.upload_bytes(blocks)
    out = device.alloc(33 * 32 + 1)
    p = C.c_void_p(out.ptr.value + 4)  # 4-byte aligned only: scalar store path
    assert lib.cq_dequantize(ctx, oc.Q4_0, 0, buf.ptr, 33, p) == 0
    got = out.data()[1:]
    assert (bits(got) == bits(oc.dequantize(oc.Q4_0, 0, blocks))).all()
    assert lib.cq_dequantize(ctx, oc.Q4_0, 0, buf.ptr, 0, p) == 0  # empty input is a no-op


# ---- quantizers: byte-exact ----------------------------------------------------------------
@pytest.mark.parametrize("qt,order", QT_ORDERS)
def test_quantize_rows_byte_exact(device, qt, order):
    from candy_b200.backend import QStorage
    rng = np.random.default_rng(200 + qt + order)
    w = (rng.standard_normal((257, 416)) * 0.02).astype(np.float32)
    w[0, :32] = 0
    w[1, 32:64] = np.float32(1e-8)
    w[2, :] *= np.float32(1e3)
    w[3, 64], w[3, 65] = -0.5, 0.5
    w[4, 96], w[4, 97] = 0.5, -0.5
    w[5, :] = np.round(w[5, :] * 1000) / 8  # many exact ties for the rounding rules
    got = QStorage.quantize(device, qt, order, w).data()
    assert (got == oc.quantize(qt, order, w)).all()


def test_quantize_q8_1_byte_exact(device):
    from candy_b200.backend import RawBuffer
    rng = np.random.default_rng(7)
    x = rng.standard_normal((5, 1024)).astype(np.float32)
    x[1, 64:96] = 0
    x[2, :] *= 1e-3
    x[3, :] = np.round(x[3, :] * 4) / 4
    xs = device.storage_from_slice(x)
    out = RawBuffer(device, 5 * 32 * 36)
    device._check(device._lib.cq_quantize_q8_1(device.ctx, xs.ptr, 5, 1024, 1024, out.ptr), "q8_1")
    assert (out.data() == oc.quantize_q8_1(x)).all()


# ---- golden fixtures ---------------------------------------------------------------------
def test_golden_fixture_on_gpu(device):
    from candy_b200.backend import QStorage
    g = np.load(GOLDEN)
    w, x = g["w"], g["x"]
    n = w.shape[0]
    for qt, name in ((oc.Q4_0, "q4_0"), (oc.Q8_0, "q8_0")):
        for order in (0, 1):
            tag = f"{name}_o{order}"
            if f"{tag}_blocks" not in g:
                continue
            blocks = g[f"{tag}_blocks"]
            assert (QStorage.quantize(device, qt, order, w).data() == blocks).all()
            assert (bits(gpu_dequantize(device, qt, order, blocks)) == bits(g[f"{tag}_deq"])).all()
            for force_simple in (0, 1):
                device.set_option("gemv_force_simple", force_simple)
                y = gpu_qmatmul(device, qt, order, x, blocks, n)
                assert rel_err(y, g[f"{tag}_y"]) < 1e-4
            device.set_option("gemv_force_simple", 0)
            y8 = gpu_qmatmul(device, qt, order, x, blocks, n, actmode=1)
            assert rel_err(y8, g[f"{tag}_y_q8_1"]) < 2e-5


# ---- decode GEMV, f32 activations, against the CPU path ----------------------------------
STREAM_SHAPES = [  # (n, k): k % 256 == 0 -> streaming kernel
    (64, 256), (100, 512), (37, 1024), (300, 2048), (513, 4096), (1200, 4096), (200, 11008), (70, 8192), (33, 28672),
    (1, 4096), (7, 768), (149, 3584),
]
SIMPLE_SHAPES = [(5, 32), (9, 96), (17, 160), (40, 288), (31, 4128), (3, 64)]  # k % 256 != 0 -> plain kernel


@pytest.mark.parametrize("qt,order", QT_ORDERS)
@pytest.mark.parametrize("n,k", STREAM_SHAPES + SIMPLE_SHAPES)
def test_gemv_f32_matches_cpu_path(device, qt, order, n, k):
    w, x = make_case(1000 + n + k, n, k, 1)
    blocks = oc.quantize(qt, order, w)
    want = oc.qmatmul(qt, order, x, blocks, n, nthreads=8)
    got = gpu_qmatmul(device, qt, order, x, blocks, n)
    err = rel_err(got, want)
    assert err <= REL_TOL
    assert err < 1e-4, f"16-bit activations should stay near 1e-5, got {err}"


@pytest.mark.parametrize("qt,order", QT_ORDERS)
@pytest.mark.parametrize("m", [2, 3, 5, 8])
@pytest.mark.parametrize("n,k", [(130, 1024), (40, 288)])
def test_gemv_small_batches(device, qt, order, m, n, k):
    w, x = make_case(2000 + m + n, n, k, m)
    blocks = oc.quantize(qt, order, w)
    want = oc.qmatmul(qt, order, x, blocks, n, nthreads=8)
    got = gpu_qmatmul(device, qt, order, x, blocks, n)
    assert rel_err(got, want) < 1e-4


@pytest.mark.parametrize("qt,order", QT_ORDERS)
def test_streaming_and_plain_kernels_agree(device, qt, order):
    w, x = make_case(31, 777, 4096, 1)
    blocks = oc.quantize(qt, order, w)
    a = gpu_qmatmul(device, qt, order, x, blocks, 777)
    device.set_option("gemv_force_simple", 1)
    try:
        b = gpu_qmatmul(device, qt, order, x, blocks, 777)
    finally:
        device.set_option("gemv_force_simple", 0)
    assert rel_err(a, b) < 1e-4


@pytest.mark.parametrize("warps,stages,ctas", [(4, 2, 1), (8, 3, 2), (16, 8, 1), (12, 16, 1), (1, 4, 4)])
def test_gemv_result_does_not_depend_on_launch_geometry(device, warps, stages, ctas):
    w, x = make_case(77, 1000, 4096, 1)
    blocks = oc.quantize(oc.Q4_0, 0, w)
    want = oc.qmatmul(oc.Q4_0, 0, x, blocks, 1000, nthreads=8)
    device.set_option("gemv_warps", warps)
    device.set_option("gemv_stages", stages)
    device.set_option("gemv_ctas_per_sm", ctas)
    try:
        got = gpu_qmatmul(device, oc.Q4_0, 0, x, blocks, 1000)
    finally:
        device.set_option("gemv_warps", 8)
        device.set_option("gemv_stages", 8)
        device.set_option("gemv_ctas_per_sm", 0)
    assert rel_err(got, want) < 1e-4


@pytest.mark.parametrize("variant,bound", [(0, 1e-4), (1, 2e-5), (2, 1e-4), (3, 2e-5)])
@pytest.mark.parametrize("qt,order", QT_ORDERS)
@pytest.mark.parametrize("n,k", [(513, 4096), (200, 11008), (64, 256), (37, 1024)])
def test_gemv_decoder_variants(device, variant, bound, qt, order, n, k):
    """0: 16-bit block fixed point (default), 1: f32 FMA decoder, 2 / 3: two / three int8 slices."""
    w, x = make_case(4000 + n + k, n, k, 1)
    x[0, :32] *= 1e-4  # a block of small activations next to ordinary ones
    x[0, 40] = 37.5    # and one dominant value inside a block
    blocks = oc.quantize(qt, order, w)
    want = oc.qmatmul(qt, order, x, blocks, n, nthreads=8)
    device.set_option("gemv_variant", variant)
    try:
        got = gpu_qmatmul(device, qt, order, x, blocks, n)
    finally:
        device.set_option("gemv_variant", 0)
    err = rel_err(got, want)
    assert err <= REL_TOL and err < bound


def test_gemv_extreme_values_and_zero_rows(device):
    rng = np.random.default_rng(3)
    n, k = 96, 1024
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    w[0] = 0
    w[1] *= 1e4
    w[2, :32] = 1e-8
    x = rng.standard_normal((1, k)).astype(np.float32)
    x[0, :64] = 0
    x[0, 64:96] = 1e4
    for qt, order in QT_ORDERS:
        blocks = oc.quantize(qt, order, w)
        want = oc.qmatmul(qt, order, x, blocks, n)
        got = gpu_qmatmul(device, qt, order, x, blocks, n)
        assert rel_err(got, want) < 1e-4
        assert got[0, 0] == 0.0


# ---- BASELINE configs at full size ---------------------------------------------------------
def test_config1_q8_0_gemv_4096(device):
    rng = np.random.default_rng(0)
    x = rng.standard_normal((1, 4096)).astype(np.float32)
    w = (rng.standard_normal((4096, 4096)) * 0.02).astype(np.float32)
    blocks = oc.quantize(oc.Q8_0, 0, w)
    want = oc.qmatmul(oc.Q8_0, 0, x, blocks, 4096, nthreads=8)
    got = gpu_qmatmul(device, oc.Q8_0, 0, x, blocks, 4096)
    assert rel_err(got, want) < 1e-4


@pytest.mark.parametrize("n,k", [(4096, 4096), (11008, 4096), (4096, 11008), (32000, 4096)])
def test_config2_q4_0_gemv_sweep(device, n, k):
    from candy_b200.backend import QStorage
    rng = np.random.default_rng(0)
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    x = rng.standard_normal((1, k)).astype(np.float32)
    for order in (0, 1):
        blocks = oc.quantize(oc.Q4_0, order, w)
        # the GPU quantizer reproduces the oracle's bytes at full size too
        assert (QStorage.quantize(device, oc.Q4_0, order, w).data() == blocks).all()
        want = oc.qmatmul(oc.Q4_0, order, x, blocks, n, nthreads=8)
        got = gpu_qmatmul(device, oc.Q4_0, order, x, blocks, n)
        err = rel_err(got, want)
        assert err <= REL_TOL and err < 1e-4


# ---- Q8_1 activation mode against the reference CUDA arithmetic ---------------------------
@pytest.mark.parametrize("qt,order", QT_ORDERS)
@pytest.mark.parametrize("m,n,k", [(1, 300, 4096), (4, 64, 1024), (8, 33, 288)])
def test_gemv_q8_1_matches_reference_cuda_arithmetic(device, qt, order, m, n, k):
    w, x = make_case(3000 + m + n, n, k, m)
    blocks = oc.quantize(qt, order, w)
    want = oc.qmatmul(qt, order, x, blocks, n, nthreads=8, q8_1=True)
    got = gpu_qmatmul(device, qt, order, x, blocks, n, actmode=1)
    assert rel_err(got, want) < 1e-4
    cpu = oc.qmatmul(qt, order, x, blocks, n, nthreads=8)
    assert rel_err(got, cpu) < 5e-2  # int8 activations: percent-level distance from the CPU path


# ---- the host-buffer entry point and the layer mirror --------------------------------------
def test_qmatmul_host_buffers(device):
    lib, ctx = device._lib, device.ctx
    w, x = make_case(9, 512, 2048, 1)
    blocks = oc.quantize(oc.Q4_0, 0, w)
    wbuf = device.upload_bytes(blocks)
    y = np.empty((1, 512), dtype=np.float32)
    st = lib.cq_qmatmul_host(ctx, oc.Q4_0, 0, 0, x.ctypes.data_as(C.c_void_p), 1, 2048, wbuf.ptr, 512,
                             y.ctypes.data_as(C.c_void_p))
    assert st == 0
    assert rel_err(y, oc.qmatmul(oc.Q4_0, 0, x, blocks, 512)) < 1e-4


@pytest.mark.parametrize("m,n", [(1, 4096), (4, 1024), (1, 80000), (16, 512)])
def test_qmatmul_host_pinned_result_is_written_in_place(device, m, n):
    """A pinned result buffer gets the same bits as a pageable one, whether the kernel writes it directly (small
    results of the row-streaming kernels) or the call copies out (large results, m > 8, or the option off)."""
    lib, ctx = device._lib, device.ctx
    k = 1024
    w, x = make_case(21, n, k, m)
    blocks = oc.quantize(oc.Q4_0, 0, w)
    wbuf = device.upload_bytes(blocks)
    want = np.empty((m, n), dtype=np.float32)
    assert lib.cq_qmatmul_host(ctx, oc.Q4_0, 0, 0, x.ctypes.data_as(C.c_void_p), m, k, wbuf.ptr, n,
                               want.ctypes.data_as(C.c_void_p)) == 0
    py = C.c_void_p()
    assert lib.cq_malloc_host(ctx, 4 * m * n, C.byref(py)) == 0
    try:
        view = np.ctypeslib.as_array(C.cast(py, C.POINTER(C.c_float)), shape=(m, n))
        for zero_copy in (256 << 10, 0):
            assert lib.cq_ctx_set_option(ctx, b"host_zero_copy", zero_copy) == 0
            view[:] = np.nan
            assert lib.cq_qmatmul_host(ctx, oc.Q4_0, 0, 0, x.ctypes.data_as(C.c_void_p), m, k, wbuf.ptr, n, py) == 0
            assert np.array_equal(view, want)
    finally:
        lib.cq_ctx_set_option(ctx, b"host_zero_copy", 256 << 10)
        lib.cq_free_host(ctx, py)


def test_qlinear_forward_flattens_batch_dims(device):
    from candy_b200.backend import QLinear, QStorage
    rng = np.random.default_rng(4)
    w = (rng.standard_normal((48, 256)) * 0.02).astype(np.float32)
    x = rng.standard_normal((2, 3, 256)).astype(np.float32)
    qs = QStorage.quantize(device, oc.Q4_0, 0, w)
    y = QLinear(qs).forward(x)
    assert y.shape == (2, 3, 48)
    want = oc.qmatmul(oc.Q4_0, 0, x.reshape(6, 256), qs.data(), 48).reshape(2, 3, 48)
    assert rel_err(y, want) < 1e-4
    with pytest.raises(ValueError, match="input rank must be >= 2"):
        QLinear(qs).forward(np.zeros(256, dtype=np.float32))
    with pytest.raises(ValueError, match="inner dims mismatch"):
        QLinear(qs).forward(np.zeros((2, 128), dtype=np.float32))


def test_argument_errors_come_back_as_status_codes(device):
    from candy_b200 import abi
    lib, ctx = device._lib, device.ctx
    buf = device.alloc(4096)
    p = buf.ptr
    assert lib.cq_qmatmul(ctx, 2, 0, 0, None, 1, 64, 64, p, 4, p, 4) == abi.ERR_INVALID_ARG
    assert lib.cq_qmatmul(ctx, 2, 0, 0, p, 1, 48, 48, p, 4, p, 4) == abi.ERR_INVALID_ARG  # k % 32
    assert lib.cq_qmatmul(ctx, 2, 0, 0, p, 1, 64, 32, p, 4, p, 4) == abi.ERR_INVALID_ARG  # ldx < k
    assert lib.cq_qmatmul(ctx, 2, 0, 0, p, 1, 64, 64, p, 4, p, 2) == abi.ERR_INVALID_ARG  # ldy < n
    assert lib.cq_qmatmul(ctx, 5, 0, 0, p, 1, 64, 64, p, 4, p, 4) == abi.ERR_INVALID_ARG  # qtype (5 is no format of this library)
    assert lib.cq_qmatmul(ctx, 2, 7, 0, p, 1, 64, 64, p, 4, p, 4) == abi.ERR_INVALID_ARG  # order
    assert lib.cq_qmatmul(ctx, 2, 0, 9, p, 1, 64, 64, p, 4, p, 4) == abi.ERR_INVALID_ARG  # actmode
    assert b"ldy" in lib.cq_last_error(ctx) or b"actmode" in lib.cq_last_error(ctx)
    assert lib.cq_dequantize(ctx, 2, 0, p, -1, p) == abi.ERR_INVALID_ARG
    assert lib.cq_quantize_rows(ctx, 2, 0, p, 4, 40, p) == abi.ERR_INVALID_ARG
    device.synchronize()  # the context is still usable after rejected calls


def test_independent_gemv_launches_give_the_same_bits(device):
    """Option gemv_independent: launches that do not depend on one another skip the wait on the previous kernel and
    overlap it.  Three projections of one x into three buffers, with and without the option: equal results."""
    lib, ctx = device._lib, device.ctx
    k, ns = 4096, (4096, 1024, 11008)
    rng = np.random.default_rng(31)
    x = device.storage_from_slice(rng.standard_normal((1, k), dtype=np.float32))
    ws, ys = [], []
    for i, n in enumerate(ns):
        w, _ = make_case(700 + i, n, k, 1)
        ws.append(device.upload_bytes(oc.quantize(oc.Q4_0, 0, w)))
        ys.append(device.zeros(n))
    outs = {}
    for opt in (0, 1):
        device.set_option("gemv_independent", opt)
        try:
            for rep in range(3):
                for w, y, n in zip(ws, ys, ns):
                    assert lib.cq_qmatmul(ctx, oc.Q4_0, 0, 0, x.ptr, 1, k, k, w.ptr, n, y.ptr, n) == 0
            device.synchronize()
        finally:
            device.set_option("gemv_independent", 0)
        outs[opt] = [y.data().copy() for y in ys]
    for a, b in zip(outs[0], outs[1]):
        assert np.array_equal(a, b)
