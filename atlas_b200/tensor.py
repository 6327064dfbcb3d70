"""Host-side mirror of the GPU types of the reference's atlas-tensor crate
(crates/atlas-tensor/src/lib.rs): GpuMatrix :309-436, GpuVec :460-556, GpuRopeTables :662-693,
GpuKvCache :701-785 and the free functions :97-142,590-654 — same names, argument meaning and
results, over the sm_100a library.  Differences are additions only: int8/int4 weights,
a batch dimension and a bf16 option on the KV cache, multi-column sgemm_vec.

Unlike the reference there is no CPU branch: a missing device raises AtlasError.
"""
import ctypes as C

import numpy as np

from . import _ffi
from ._ffi import AtlasError, BF16, F32, INT4, INT8, check


class Context:
    """One GPU and one stream.  `Context.default()` plays the role of the reference's implicit
    stream-0 world."""
    _default = None

    def __init__(self, device=0):
        h = C.c_void_p()
        check(_ffi.lib().atlasx_ctx_create(int(device), C.byref(h)))
        self._h = h
        self.device = device

    @classmethod
    def default(cls):
        if cls._default is None:
            cls._default = Context(0)
        return cls._default

    @property
    def handle(self):
        return self._h

    def sync(self):
        check(_ffi.lib().atlasx_ctx_sync(self._h))

    @property
    def sm_count(self):
        return _ffi.lib().atlasx_ctx_sm_count(self._h)

    def set_gemv_impl(self, impl):
        """0 automatic, 1 plain 128-bit loads, 2 bulk-copy pipeline."""
        check(_ffi.lib().atlasx_ctx_set_gemv_impl(self._h, int(impl)))

    def poll_device_error(self):
        code = C.c_int(0)
        check(_ffi.lib().atlasx_ctx_poll_device_error(self._h, C.byref(code)))
        return code.value

    # raw device memory ---------------------------------------------------------------
    def malloc(self, nbytes):
        p = C.c_void_p()
        check(_ffi.lib().atlasx_malloc(self._h, int(nbytes), C.byref(p)))
        return p.value or 0

    def free(self, ptr):
        if ptr:
            check(_ffi.lib().atlasx_free(self._h, C.c_void_p(ptr)))

    def upload(self, ptr, arr):
        arr = np.ascontiguousarray(arr)
        check(_ffi.lib().atlasx_upload(self._h, C.c_void_p(ptr), arr.ctypes.data, arr.nbytes))

    def download(self, ptr, shape, dtype):
        out = np.empty(shape, dtype=dtype)
        check(_ffi.lib().atlasx_download(self._h, out.ctypes.data, C.c_void_p(ptr), out.nbytes))
        return out

    def to_device(self, arr):
        arr = np.ascontiguousarray(arr)
        p = self.malloc(max(arr.nbytes, 16))
        if arr.nbytes:
            self.upload(p, arr)
        return p

    def close(self):
        if self._h:
            _ffi.lib().atlasx_ctx_destroy(self._h)
            self._h = None
            if Context._default is self:
                Context._default = None


def cuda_available():
    return _ffi.cuda_available()


def device_sync():
    """device_sync(), :97-100."""
    _ffi.lib().atlas_sync()


class GpuVec:
    """Activation vector in HBM (f32).  Mirrors GpuVec :460-556 without the CPU mirror."""

    def __init__(self, ctx, ptr, length, owner=True):
        self.ctx, self.ptr, self.len, self._owner = ctx, ptr, int(length), owner

    @classmethod
    def zeros(cls, n, ctx=None):
        ctx = ctx or Context.default()
        p = ctx.malloc(max(4 * n, 16))
        check(_ffi.lib().atlasx_memset(ctx.handle, C.c_void_p(p), 0, 4 * n))
        return cls(ctx, p, n)

    @classmethod
    def from_slice(cls, data, ctx=None):
        ctx = ctx or Context.default()
        a = np.ascontiguousarray(data, dtype=np.float32).ravel()
        return cls(ctx, ctx.to_device(a), a.size)

    def download(self):
        return self.ctx.download(self.ptr, (self.len,), np.float32)

    def is_on_gpu(self):
        return True

    def gpu_ptr(self):
        return self.ptr

    def add_inplace(self, other):
        assert self.len == other.len
        check(_ffi.lib().atlasx_vec_add(self.ctx.handle, self.ptr, other.ptr, self.ptr, self.len))

    def rmsnorm_inplace(self, w, eps):
        assert self.len == w.len
        out = self.ctx.malloc(max(4 * self.len, 16))
        check(_ffi.lib().atlasx_rmsnorm(self.ctx.handle, self.ptr, w.ptr, out, self.len, float(eps)))
        old, self.ptr = self.ptr, out
        if self._owner:
            self.ctx.free(old)
        self._owner = True

    def __del__(self):
        try:
            if self._owner and self.ptr and self.ctx.handle:
                self.ctx.free(self.ptr)
        except Exception:
            pass
        self.ptr = 0


class GpuMatrix:
    """Weight matrix [rows=out × cols=in] resident in HBM.  Mirrors GpuMatrix :309-436."""

    def __init__(self, ctx, handle, rows, cols, dtype, keep=()):
        self.ctx, self._h, self.rows, self.cols, self.dtype = ctx, handle, rows, cols, dtype
        self._keep = keep

    @classmethod
    def upload(cls, data, rows, cols, ctx=None):
        ctx = ctx or Context.default()
        a = np.ascontiguousarray(data, dtype=np.float32)
        assert a.size == rows * cols
        h = C.c_void_p()
        check(_ffi.lib().atlasx_matrix_upload_f32(ctx.handle, a.ctypes.data, rows, cols, C.byref(h)))
        return cls(ctx, h, rows, cols, F32)

    @classmethod
    def upload_bf16(cls, data, rows, cols, ctx=None):
        ctx = ctx or Context.default()
        a = np.ascontiguousarray(data, dtype=np.uint16)
        assert a.size == rows * cols
        h = C.c_void_p()
        check(_ffi.lib().atlasx_matrix_upload_bf16(ctx.handle, a.ctypes.data, rows, cols, C.byref(h)))
        return cls(ctx, h, rows, cols, BF16)

    @classmethod
    def upload_int8(cls, q, ctx=None):
        """q: quant.Int8Tensor."""
        ctx = ctx or Context.default()
        h = C.c_void_p()
        d = np.ascontiguousarray(q.data, dtype=np.int8)
        s = np.ascontiguousarray(q.scales, dtype=np.float32)
        check(_ffi.lib().atlasx_matrix_upload_int8(ctx.handle, d.ctypes.data, s.ctypes.data, q.rows, q.cols, C.byref(h)))
        return cls(ctx, h, q.rows, q.cols, INT8)

    @classmethod
    def upload_int4(cls, q, scales_f16=False, ctx=None):
        """q: quant.Int4Tensor."""
        ctx = ctx or Context.default()
        h = C.c_void_p()
        d = np.ascontiguousarray(q.data, dtype=np.uint8)
        s = np.ascontiguousarray(q.scales, dtype=np.float32)
        check(_ffi.lib().atlasx_matrix_upload_int4(ctx.handle, d.ctypes.data, s.ctypes.data, q.rows, q.cols,
                                                   q.block_size, int(bool(scales_f16)), C.byref(h)))
        return cls(ctx, h, q.rows, q.cols, INT4)

    @classmethod
    def wrap(cls, dtype, data_ptr, scales_ptr, rows, cols, block_size=0, scales_f16=False, ctx=None, keep=()):
        """Adopt device arrays (not copied, not freed)."""
        ctx = ctx or Context.default()
        h = C.c_void_p()
        check(_ffi.lib().atlasx_matrix_wrap(ctx.handle, dtype, C.c_void_p(data_ptr), C.c_void_p(scales_ptr or 0),
                                            rows, cols, block_size, int(bool(scales_f16)), C.byref(h)))
        return cls(ctx, h, rows, cols, dtype, keep)

    def is_on_gpu(self):
        return True

    def is_bf16(self):
        return self.dtype == BF16

    @property
    def weight_bytes(self):
        return int(_ffi.lib().atlasx_matrix_bytes(self._h))

    def sgemm(self, rhs, k, n, out):
        """out[m×n] = self[m×k]·rhs[k×n] with host arrays; returns True (GPU was used)."""
        r = np.ascontiguousarray(rhs, dtype=np.float32)
        assert r.size == k * n and out.size == self.rows * n and out.dtype == np.float32
        check(_ffi.lib().atlasx_matrix_sgemm(self.ctx.handle, self._h, r.ctypes.data, k, n, out.ctypes.data))
        return True

    def sgemm_vec(self, x, n=1):
        """Device-to-device product; x holds [cols×n] row-major.  Returns a new GpuVec [rows×n]."""
        assert x.len == self.cols * n
        y = self.ctx.malloc(max(4 * self.rows * n, 16))
        try:
            check(_ffi.lib().atlasx_gemv(self.ctx.handle, self._h, x.ptr, n, y))
        except AtlasError:
            self.ctx.free(y)
            raise
        return GpuVec(self.ctx, y, self.rows * n)

    def gemv_into(self, x_ptr, y_ptr, n=1):
        check(_ffi.lib().atlasx_gemv(self.ctx.handle, self._h, x_ptr, n, y_ptr))

    def __del__(self):
        try:
            if self._h and self.ctx.handle:
                _ffi.lib().atlasx_matrix_free(self._h)
        except Exception:
            pass
        self._h = None


def silu_mul_gpu(gate, up):
    """silu_mul_gpu, :590-609."""
    assert gate.len == up.len
    out = GpuVec.zeros(gate.len, gate.ctx)
    check(_ffi.lib().atlasx_silu_mul(gate.ctx.handle, gate.ptr, up.ptr, out.ptr, gate.len))
    return out


def qk_norm_inplace_gpu(x, w, n_heads, head_dim, eps):
    """qk_norm_inplace_gpu, :633-654."""
    check(_ffi.lib().atlasx_qk_norm_inplace(x.ctx.handle, x.ptr, w.ptr, n_heads, head_dim, float(eps)))


def gpu_argmax(x):
    """Index of the maximum, with the tie rule of the CPU argmax that generate() uses
    (last of equal maxima, crates/atlas-model/src/lib.rs:2701-2706)."""
    out = C.c_int(0)
    check(_ffi.lib().atlasx_argmax(x.ctx.handle, x.ptr, x.len, C.byref(out)))
    return out.value


def rope_tables(head_dim, max_seq, theta, yarn=None):
    """RopeCache::new (crates/atlas-model/src/lib.rs:380-423) → (cos, sin) of shape [max_seq, head_dim/2]."""
    half = head_dim // 2
    cos = np.empty((max_seq, half), np.float32)
    sin = np.empty((max_seq, half), np.float32)
    y = yarn or {}
    check(_ffi.lib().atlasx_rope_tables_host(head_dim, max_seq, float(theta), 1 if yarn else 0,
                                             float(y.get("factor", 1.0)), int(y.get("orig_max_pos", 0)),
                                             float(y.get("beta_fast", 32.0)), float(y.get("beta_slow", 1.0)),
                                             cos.ctypes.data, sin.ctypes.data))
    return cos, sin


class GpuRopeTables:
    """GpuRopeTables, :662-693."""

    def __init__(self, cos, sin, max_seq, half_dim):
        self.cos, self.sin, self.max_seq, self.half_dim = cos, sin, max_seq, half_dim

    @classmethod
    def upload(cls, cos_flat, sin_flat, max_seq, half_dim, ctx=None):
        return cls(GpuVec.from_slice(cos_flat, ctx), GpuVec.from_slice(sin_flat, ctx), max_seq, half_dim)

    def apply_to(self, x, n_heads, head_dim, pos):
        check(_ffi.lib().atlasx_rope_apply(x.ctx.handle, x.ptr, self.cos.ptr, self.sin.ptr, n_heads, head_dim,
                                           int(pos), self.max_seq))


class GpuKvCache:
    """GpuKvCache, :701-785, with `batch` sequences and bf16 or f32 storage."""

    def __init__(self, max_seq, n_kv_heads, head_dim, dtype=BF16, batch=1, ctx=None):
        self.ctx = ctx or Context.default()
        h = C.c_void_p()
        check(_ffi.lib().atlasx_kvcache_create(self.ctx.handle, max_seq, n_kv_heads, head_dim, dtype, batch, C.byref(h)))
        self._h = h
        self.max_seq, self.n_kv_heads, self.head_dim, self.dtype, self.batch = max_seq, n_kv_heads, head_dim, dtype, batch

    @classmethod
    def new(cls, max_seq, n_kv_heads, head_dim, **kw):
        return cls(max_seq, n_kv_heads, head_dim, **kw)

    def ptrs(self):
        k, v, n = C.c_void_p(), C.c_void_p(), C.c_size_t()
        check(_ffi.lib().atlasx_kvcache_ptrs(self._h, C.byref(k), C.byref(v), C.byref(n)))
        return k.value, v.value, n.value

    def _pos(self, pos):
        p = np.ascontiguousarray(np.broadcast_to(np.asarray(pos, dtype=np.int32), (self.batch,)))
        return p

    def write(self, pos, new_k, new_v):
        p = self._pos(pos)
        check(_ffi.lib().atlasx_kvcache_write(self.ctx.handle, self._h, new_k.ptr, new_v.ptr, p.ctypes.data))

    def decode_attention(self, q, n_heads, pos, scale, window_size=0):
        p = self._pos(pos)
        out = GpuVec.zeros(self.batch * n_heads * self.head_dim, self.ctx)
        check(_ffi.lib().atlasx_decode_attention(self.ctx.handle, self._h, q.ptr, out.ptr, n_heads, p.ctypes.data,
                                                 float(scale), int(window_size)))
        return out

    def attention_bytes(self, n_heads, pos, window_size=0):
        p = self._pos(pos)
        return int(_ffi.lib().atlasx_decode_attention_bytes(self._h, n_heads, p.ctypes.data, int(window_size)))

    def reset(self):
        """No-op by design, as in the reference (:782-784): rows beyond pos are never read."""

    def __del__(self):
        try:
            if self._h and self.ctx.handle:
                _ffi.lib().atlasx_kvcache_free(self._h)
        except Exception:
            pass
        self._h = None
