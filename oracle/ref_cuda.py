"""Launches the reference's own CUDA kernels (test infrastructure).

`oracle/build_oracle.py:build_ref` compiles tensor/internal/cuda/kernels/quantized.cu of a
gocnn/candy checkout, from where it lies, into `_ref/quantized_sm100a.cubin`.  The reference has no
host code that launches these kernels, so the launch geometry below is derived from each kernel's
own index arithmetic (cited per function); only kernels and shapes whose every access was checked
against that arithmetic are launched.  Used by GPU tests to pin the oracle against code the
reference ships; never by the library.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

CUBIN = Path(__file__).resolve().parent / "_ref" / "quantized_sm100a.cubin"


class RefKernels:
    def __init__(self, device: int = 0):
        from cuda.bindings import driver as drv
        self.drv = drv
        self._ok(drv.cuInit(0))
        dev = self._ok(drv.cuDeviceGet(device))
        self.ctx = self._ok(drv.cuDevicePrimaryCtxRetain(dev))  # the context the runtime API (and libcandyq) uses
        self._ok(drv.cuCtxSetCurrent(self.ctx))
        self.mod = self._ok(drv.cuModuleLoadData(CUBIN.read_bytes()))
        self.fn = {}

    @staticmethod
    def _ok(res):
        err = res[0]
        if int(err) != 0:
            raise RuntimeError(f"CUDA driver error {err}")
        return res[1] if len(res) == 2 else res[1:] if len(res) > 2 else None

    def _get(self, name):
        if name not in self.fn:
            self.fn[name] = self._ok(self.drv.cuModuleGetFunction(self.mod, name.encode()))
        return self.fn[name]

    def _launch(self, name, grid, block, args, types, sync=True):
        self._ok(self.drv.cuCtxSetCurrent(self.ctx))
        self._ok(self.drv.cuLaunchKernel(self._get(name), grid[0], grid[1], grid[2], block[0], block[1], block[2], 0, 0,
                                         (tuple(args), tuple(types)), 0))
        if sync:
            self._ok(self.drv.cuCtxSynchronize())

    def timed_ms(self, fn) -> float:
        """Device time of the launches fn() enqueues on the default stream (CUDA events, synchronised on both sides)."""
        drv = self.drv
        self._ok(drv.cuCtxSetCurrent(self.ctx))
        e0, e1 = self._ok(drv.cuEventCreate(0)), self._ok(drv.cuEventCreate(0))
        self._ok(drv.cuCtxSynchronize())
        self._ok(drv.cuEventRecord(e0, 0))
        fn()
        self._ok(drv.cuEventRecord(e1, 0))
        self._ok(drv.cuEventSynchronize(e1))
        ms = self._ok(drv.cuEventElapsedTime(e0, e1))
        self._ok(drv.cuEventDestroy(e0))
        self._ok(drv.cuEventDestroy(e1))
        return float(ms)

    def dequantize(self, qname: str, blocks_ptr: int, y_ptr: int, nb32: int):
        """dequantize_block_q4_0_f32 / _q8_0_f32 (quantized.cu:838-867, :1149-1175): block i of the grid
        handles blocks 8i..8i+7 with 32 threads, guarded by ib < nb32."""
        self._launch(f"dequantize_block_{qname}_f32", ((nb32 + 7) // 8, 1, 1), (32, 1, 1), (blocks_ptr, y_ptr, nb32),
                     (C.c_void_p, C.c_void_p, C.c_int))

    def quantize_q8_1(self, x_ptr: int, out_ptr: int, k: int, rows: int, sync=True):
        """quantize_q8_1 (quantized.cu:3521-3558): block (256,1), grid (ceil(k/256), rows); k % 32 == 0 so
        the ix >= kx_padded guard retires whole warps."""
        assert k % 32 == 0
        self._launch("quantize_q8_1", ((k + 255) // 256, rows, 1), (256, 1, 1), (x_ptr, out_ptr, k, k),
                     (C.c_void_p, C.c_void_p, C.c_int, C.c_int), sync=sync)

    def mul_mat_vec_q8_1(self, qname: str, w_ptr: int, act_ptr: int, dst_ptr: int, k: int, n: int, sync=True):
        """mul_mat_vec_q4_0_q8_1_cuda1 / _q8_0_ (quantized.cu:2787-2880): one activation row, block (32,4),
        one weight row per CTA (rows_per_cuda_block = 1 for ncols_y = 1), grid = n rows."""
        self._launch(f"mul_mat_vec_{qname}_q8_1_cuda1", (n, 1, 1), (32, 4, 1), (w_ptr, act_ptr, dst_ptr, k, n, k, n),
                     (C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int), sync=sync)

    def dequantize_mul_mat_vec(self, qname: str, w_ptr: int, x_ptr: int, dst_ptr: int, k: int, n: int, sync=True):
        """dequantize_mul_mat_vec_q4_0_cuda / _q8_0_cuda (quantized.cu:1251-1345): f32 activations, one warp
        per row (block (32,1), grid n); each iteration covers 64 columns, so k % 64 == 0 is required."""
        assert k % 64 == 0
        self._launch(f"dequantize_mul_mat_vec_{qname}_cuda", (n, 1, 1), (32, 1, 1), (w_ptr, x_ptr, dst_ptr, k, n),
                     (C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int), sync=sync)
