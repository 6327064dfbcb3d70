"""Host-side mirror of the reference's atlas-quant crate (crates/atlas-quant/src/lib.rs):
Int8Tensor :32-88 and Int4Tensor :101-180, same fields and method names.  quantize() and
dequantize() run on the GPU through the C ABI and are bit-exact with the Rust code (round half
away from zero, multiply by the reciprocal scale, scale 1.0 for an all-zero row or block, even
index in the high nibble)."""
import ctypes as C

import numpy as np

from . import _ffi
from ._ffi import check
from .tensor import Context

INT4_BLOCK_SIZE = 64   # crates/atlas-quant/src/lib.rs:93


class Int8Tensor:
    def __init__(self, data, scales, rows, cols):
        self.data, self.scales, self.rows, self.cols = data, scales, rows, cols

    @classmethod
    def quantize(cls, t, ctx=None):
        t = np.asarray(t, dtype=np.float32)
        if t.ndim != 2:
            raise _ffi.AtlasError("Int8Tensor::quantize requires 2D tensor")
        ctx = ctx or Context.default()
        rows, cols = t.shape
        src = ctx.to_device(t)
        d = ctx.malloc(max(rows * cols, 16))
        s = ctx.malloc(max(rows * 4, 16))
        try:
            check(_ffi.lib().atlasx_quantize_int8(ctx.handle, src, rows, cols, d, s))
            data = ctx.download(d, (rows * cols,), np.int8)
            scales = ctx.download(s, (rows,), np.float32)
        finally:
            ctx.free(src); ctx.free(d); ctx.free(s)
        return cls(data, scales, rows, cols)

    def dequantize(self, ctx=None):
        ctx = ctx or Context.default()
        d = ctx.to_device(self.data); s = ctx.to_device(self.scales)
        o = ctx.malloc(max(self.rows * self.cols * 4, 16))
        try:
            check(_ffi.lib().atlasx_dequantize_int8(ctx.handle, d, s, self.rows, self.cols, o))
            out = ctx.download(o, (self.rows, self.cols), np.float32)
        finally:
            ctx.free(d); ctx.free(s); ctx.free(o)
        return out

    def memory_bytes(self):
        return self.data.size + self.scales.size * 4

    def compression_ratio(self):
        return self.rows * self.cols * 4 / self.memory_bytes()


class Int4Tensor:
    def __init__(self, data, scales, rows, cols, block_size):
        self.data, self.scales, self.rows, self.cols, self.block_size = data, scales, rows, cols, block_size

    @classmethod
    def quantize(cls, t, block_size=INT4_BLOCK_SIZE, ctx=None):
        t = np.asarray(t, dtype=np.float32)
        if t.ndim != 2:
            raise _ffi.AtlasError("Int4Tensor::quantize requires 2D tensor")
        ctx = ctx or Context.default()
        rows, cols = t.shape
        n = rows * cols
        nb = (n + block_size - 1) // block_size
        src = ctx.to_device(t)
        d = ctx.malloc(max((n + 1) // 2, 16))
        s = ctx.malloc(max(nb * 4, 16))
        try:
            check(_ffi.lib().atlasx_quantize_int4(ctx.handle, src, n, block_size, d, s))
            data = ctx.download(d, ((n + 1) // 2,), np.uint8)
            scales = ctx.download(s, (nb,), np.float32)
        finally:
            ctx.free(src); ctx.free(d); ctx.free(s)
        return cls(data, scales, rows, cols, block_size)

    def dequantize(self, ctx=None):
        ctx = ctx or Context.default()
        n = self.rows * self.cols
        d = ctx.to_device(self.data); s = ctx.to_device(self.scales)
        o = ctx.malloc(max(n * 4, 16))
        try:
            check(_ffi.lib().atlasx_dequantize_int4(ctx.handle, d, s, n, self.block_size, o))
            out = ctx.download(o, (self.rows, self.cols), np.float32)
        finally:
            ctx.free(d); ctx.free(s); ctx.free(o)
        return out

    def memory_bytes(self):
        return self.data.size + self.scales.size * 4

    def compression_ratio(self):
        return self.rows * self.cols * 4 / self.memory_bytes()
