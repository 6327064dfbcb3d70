"""GPU: atlasx_decode_attention_static — the attention entry point for hosts that may not
allocate device memory while serving (a fully pre-partitioned memory pool, a plugin living
inside another allocator, a loop where cudaMalloc's implicit synchronisation is unacceptable).
Its split-K scratch is a fixed array inside the library.  The output must equal that of the
regular entry point (atlasx_decode_attention, scratch in context memory) and that of the CPU
oracle within the 1e-3 attention tolerance of these tests, on two calls in a row: the second
call reuses the array the first one left behind.  Collected last so that a stop-at-first-failure run has already run
everything else."""
import ctypes as C
import math

import numpy as np
import pytest

from oracle import orc
from helpers import rel_err

pytestmark = pytest.mark.gpu


def _case(ab, nh, nkv, hd, max_seq, batch, dtype, positions, window, seed):
    from atlas_b200 import _ffi
    L = _ffi.lib()
    kv = ab.GpuKvCache(max_seq, nkv, hd, dtype=dtype, batch=batch)
    ctx = kv.ctx
    kp, vp, nbytes = kv.ptrs()
    n = nbytes // (2 if dtype == ab.BF16 else 4)
    fill = L.atlasx_fill_normal_bf16 if dtype == ab.BF16 else L.atlasx_fill_normal_f32
    _ffi.check(fill(ctx.handle, kp, n, seed, 1, 0, 1.0))
    _ffi.check(fill(ctx.handle, vp, n, seed, 2, 0, 1.0))
    q_host = orc.normal_f32(batch * nh * hd, seed, 3, 1.0)
    q = ab.GpuVec.from_slice(q_host)
    scale = 1.0 / math.sqrt(hd)
    want = kv.decode_attention(q, nh, positions, scale, window).download()
    # the regular entry point itself against the CPU oracle fed the same cache contents
    gen = (lambda st: orc.bf16_to_f32(orc.normal_bf16(n, seed, st, 1.0))) if dtype == ab.BF16 else (lambda st: orc.normal_f32(n, seed, st, 1.0))
    k_host, v_host = gen(1).reshape(batch, -1), gen(2).reshape(batch, -1)
    oracle = np.concatenate([orc.decode_attention(q_host[b * nh * hd:(b + 1) * nh * hd], k_host[b], v_host[b], nh, nkv, hd,
                                                  positions[b], scale, window) for b in range(batch)])
    assert rel_err(want, oracle) <= 1e-3
    out = ab.GpuVec.zeros(batch * nh * hd)
    pos = np.ascontiguousarray(positions, dtype=np.int32)
    stream = L.atlasx_ctx_stream(ctx.handle)
    for call in range(2):                                  # second call sees the first one's leftovers
        check_rc = L.atlasx_decode_attention_static(stream, dtype, kp, vp, max_seq, nkv, hd, batch, q.ptr, out.ptr, nh,
                                                    pos.ctypes.data, scale, window)
        _ffi.check(check_rc)
        got = out.download()
        assert np.all(np.isfinite(got)), call
        assert rel_err(got, want) <= 1e-3, call
        assert rel_err(got, oracle) <= 1e-3, call
        _ffi.check(L.atlasx_memset(ctx.handle, out.ptr, 0, 4 * out.len))
    return kv


def test_static_scratch_attention_matches_regular_entry_point():
    import atlas_b200 as ab
    # config-5 shape, bf16 cache, ragged positions, full and windowed
    _case(ab, 32, 8, 128, 4096, 4, ab.BF16, [4095, 1000, 17, 0], 0, 71)
    _case(ab, 32, 8, 128, 4096, 4, ab.BF16, [4095, 1000, 17, 0], 512, 72)
    # f32 cache, MHA, head_dim 64; then a shape that takes the scratch-free generic kernel
    _case(ab, 8, 8, 64, 512, 2, ab.F32, [511, 3], 0, 73)
    _case(ab, 6, 2, 48, 100, 1, ab.BF16, [99], 0, 74)


def test_static_scratch_limits_are_rejected():
    import atlas_b200 as ab
    from atlas_b200 import _ffi
    L = _ffi.lib()
    kv = ab.GpuKvCache(16, 1, 64, dtype=ab.BF16, batch=1)
    kp, vp, _ = kv.ptrs()
    q = ab.GpuVec.zeros(64)
    pos = np.zeros(5000, np.int32)
    stream = L.atlasx_ctx_stream(kv.ctx.handle)
    # batch beyond the fixed array
    rc = L.atlasx_decode_attention_static(stream, ab.BF16, kp, vp, 16, 1, 64, 5000, q.ptr, q.ptr, 1, pos.ctypes.data, 1.0, 0)
    assert rc != 0 and b"exceeds the fixed scratch" in L.atlasx_last_error()
    # batch × heads beyond the ticket area
    rc = L.atlasx_decode_attention_static(stream, ab.BF16, kp, vp, 16, 1, 64, 100, q.ptr, q.ptr, 64, pos.ctypes.data, 1.0, 0)
    assert rc != 0 and b"exceeds the fixed scratch" in L.atlasx_last_error()
    # position outside the cache
    pos[0] = 16
    rc = L.atlasx_decode_attention_static(stream, ab.BF16, kp, vp, 16, 1, 64, 1, q.ptr, q.ptr, 1, pos.ctypes.data, 1.0, 0)
    assert rc != 0
