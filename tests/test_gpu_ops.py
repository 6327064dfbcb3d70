"""GPU: the reference's kernel ABI (atlas_*) and the GpuVec/GpuMatrix mirror against the known
answers of the reference's own tests (crates/atlas-tensor/src/lib.rs:1097-1220,
crates/atlas-model/src/lib.rs:3826-3845) and against the CPU oracle."""
import ctypes as C
import math

import numpy as np
import pytest

from oracle import orc

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ab():
    import atlas_b200
    return atlas_b200


@pytest.fixture(scope="module")
def ctx(ab):
    return ab.Context.default()


def test_gpuvec_roundtrip_zeros_add(ab, ctx):
    v = ab.GpuVec.zeros(64)
    assert v.len == 64 and not v.download().any()
    data = np.arange(16, dtype=np.float32)
    assert np.array_equal(ab.GpuVec.from_slice(data).download(), data)
    a = ab.GpuVec.from_slice([1.0, 2.0, 3.0, 4.0]); b = ab.GpuVec.from_slice([0.5] * 4)
    a.add_inplace(b)
    assert np.allclose(a.download(), [1.5, 2.5, 3.5, 4.5])


def test_rmsnorm_known_answers(ab, ctx):
    x = ab.GpuVec.from_slice([1.0, 2.0, 3.0, 4.0]); w = ab.GpuVec.from_slice([1.0] * 4)
    x.rmsnorm_inplace(w, 1e-5)
    rms = math.sqrt(7.5)
    out = x.download()
    assert abs(out[0] - 1 / rms) < 1e-5 and abs(out[3] - 4 / rms) < 1e-5
    xs = ((np.arange(64, dtype=np.float32) + 1.0) * np.float32(0.01)).astype(np.float32)
    g = ab.GpuVec.from_slice(xs); g.rmsnorm_inplace(ab.GpuVec.from_slice(np.ones(64)), 1e-5)
    assert np.max(np.abs(g.download() - orc.rmsnorm(xs, np.ones(64, np.float32), 1e-5))) < 1e-6
    for n in (1, 3, 31, 33, 4096, 5000):
        xv = orc.normal_f32(n, 1, n, 1.0); wv = 1 + orc.normal_f32(n, 2, n, 0.1)
        g = ab.GpuVec.from_slice(xv); g.rmsnorm_inplace(ab.GpuVec.from_slice(wv), 1e-6)
        assert np.max(np.abs(g.download() - orc.rmsnorm(xv, wv, 1e-6))) < 2e-6 * max(1, np.abs(xv).max())


def test_silu_mul(ab, ctx):
    out = ab.silu_mul_gpu(ab.GpuVec.from_slice([0.0, 1.0, -1.0, 2.0]), ab.GpuVec.from_slice([1.0] * 4)).download()
    assert abs(out[0]) < 1e-6 and abs(out[1] - 0.7310586) < 1e-6
    g = orc.normal_f32(1376, 3, 1, 2.0); u = orc.normal_f32(1376, 3, 2, 1.0)
    ref = np.array([orc.silu(a) * b for a, b in zip(g, u)], np.float32)
    out = ab.silu_mul_gpu(ab.GpuVec.from_slice(g), ab.GpuVec.from_slice(u)).download()
    assert np.max(np.abs(out - ref)) < 1e-6


def test_sgemm_vec_all_ones_and_matmul_known_answer(ab, ctx):
    gm = ab.GpuMatrix.upload(np.ones(12, np.float32), 4, 3)
    assert np.allclose(gm.sgemm_vec(ab.GpuVec.from_slice([1.0, 1.0, 1.0]), 1).download(), 3.0)
    a = ab.GpuMatrix.upload(np.array([1, 2, 3, 4, 5, 6], np.float32), 2, 3)
    out = np.zeros(4, np.float32)
    assert a.sgemm(np.array([7, 8, 9, 10, 11, 12], np.float32), 3, 2, out)
    assert out.tolist() == [58.0, 64.0, 139.0, 154.0]


def test_bf16_gemv_parity_reference_case(ab, ctx):
    # crates/atlas-model/src/lib.rs:3887-3934
    M, K = 128, 256
    i = np.arange(M * K, dtype=np.int64)
    w = (((i * 6977 + 1231) % 10000).astype(np.float32) / np.float32(10000.0) - np.float32(0.5))
    k = np.arange(K, dtype=np.int64)
    x = ((k * 3571 + 421) % 10000).astype(np.float32) / np.float32(10000.0) - np.float32(0.5)
    w16 = (w.view(np.uint32) >> 16).astype(np.uint16)
    y_ref = orc.linear(w.reshape(M, K), x)
    gm = ab.GpuMatrix.upload_bf16(w16, M, K)
    assert gm.is_bf16() and gm.is_on_gpu()
    y = gm.sgemm_vec(ab.GpuVec.from_slice(x), 1).download()
    assert np.max(np.abs(y - y_ref)) / max(np.abs(y_ref).max(), 1e-6) < 0.01
    assert np.max(np.abs(y - orc.linear(w16.reshape(M, K), x))) / np.abs(y_ref).max() < 1e-5


def _legacy(ab):
    from atlas_b200 import _ffi
    return _ffi.lib()


def test_legacy_elementwise_symbols(ab, ctx):
    L = _legacy(ab)
    n = 1000
    a = orc.normal_f32(n, 4, 1); b = orc.normal_f32(n, 4, 2)
    da, db, do = ctx.to_device(a), ctx.to_device(b), ctx.malloc(4 * n)
    L.atlas_vec_add_f32(da, db, do, n); L.atlas_sync()
    assert np.array_equal(ctx.download(do, (n,), np.float32), a + b)
    L.atlas_scale_f32(da, 0.5, do, n); L.atlas_sync()
    assert np.array_equal(ctx.download(do, (n,), np.float32), a * np.float32(0.5))
    L.atlas_relu_f32(da, do, n); L.atlas_sync()
    assert np.array_equal(ctx.download(do, (n,), np.float32), np.maximum(a, 0))
    L.atlas_vram_copy_f32(da, do, n); L.atlas_sync()
    assert np.array_equal(ctx.download(do, (n,), np.float32), a)
    L.atlas_silu_mul_f32(da, db, do, n); L.atlas_sync()
    ref = np.array([orc.silu(x) * y for x, y in zip(a, b)], np.float32)
    assert np.max(np.abs(ctx.download(do, (n,), np.float32) - ref)) < 1e-6
    L.atlas_softmax_f32(da, do, 10, 100); L.atlas_sync()
    sm = ctx.download(do, (10, 100), np.float32)
    ref = np.stack([orc.softmax(a[r * 100:(r + 1) * 100]) for r in range(10)])
    assert np.max(np.abs(sm - ref)) < 1e-6 and np.allclose(sm.sum(1), 1, atol=1e-5)
    L.atlas_rmsnorm_f32(da, db, do, n, 1e-5); L.atlas_sync()
    assert np.max(np.abs(ctx.download(do, (n,), np.float32) - orc.rmsnorm(a, b, 1e-5))) < 1e-5
    for p in (da, db, do):
        ctx.free(p)


def test_legacy_rope_and_argmax(ab, ctx):
    L = _legacy(ab)
    x = np.array([1.0, 2.0, 3.0, 4.0], np.float32)
    dx = ctx.to_device(x)
    L.atlas_rope_apply_f32(dx, 0, 4, 10000.0); L.atlas_sync()
    assert np.allclose(ctx.download(dx, (4,), np.float32), x, atol=1e-6)       # identity at pos 0
    L.atlas_rope_apply_f32(dx, 3, 4, 10000.0); L.atlas_sync()
    cos, sin = orc.rope_tables(4, 4, 10000.0)
    assert np.max(np.abs(ctx.download(dx, (4,), np.float32) - orc.rope_apply(x, 4, cos[3], sin[3]))) < 1e-5
    # reference kernel rule: first of equal maxima, index written as a float
    v = np.zeros(5000, np.float32); v[[17, 4000]] = 3.0
    dv, do = ctx.to_device(v), ctx.malloc(16)
    L.atlas_gpu_argmax(dv, do, 5000); L.atlas_sync()
    assert ctx.download(do, (1,), np.float32)[0] == 17.0
    # generate()'s CPU rule: last of equal maxima
    assert ab.gpu_argmax(ab.GpuVec.from_slice(v)) == 4000
    assert ab.gpu_argmax(ab.GpuVec.from_slice(np.zeros(7))) == 6
    big = orc.normal_f32(100278, 9, 9); assert ab.gpu_argmax(ab.GpuVec.from_slice(big)) == orc.argmax(big)
    for p in (dx, dv, do):
        ctx.free(p)


def test_legacy_qk_norm_rope_kvwrite_attention(ab, ctx):
    """The reference call sequence of Attention::forward_token_gpu_full (:848-866) through the
    atlas_* symbols, f32 cache, against the oracle."""
    L = _legacy(ab)
    nh, nkv, hd, max_seq = 8, 2, 64, 64
    cos, sin = orc.rope_tables(hd, max_seq, 10000.0)
    dcos, dsin = ctx.to_device(cos), ctx.to_device(sin)
    kc = np.zeros((max_seq, nkv, hd), np.float32); vc = np.zeros_like(kc)
    dkc, dvc = ctx.to_device(kc), ctx.to_device(vc)
    qn = 1 + orc.normal_f32(nh * hd, 5, 1, 0.1); kn = 1 + orc.normal_f32(nkv * hd, 5, 2, 0.1)
    dqn, dkn = ctx.to_device(qn), ctx.to_device(kn)
    dout = ctx.malloc(4 * nh * hd)
    scale = 1.0 / math.sqrt(hd)
    for pos in range(40):
        q = orc.normal_f32(nh * hd, 6, pos); k = orc.normal_f32(nkv * hd, 7, pos); v = orc.normal_f32(nkv * hd, 8, pos)
        # oracle
        qo, ko = q.copy(), k.copy()
        for h in range(nh):
            qo[h * hd:(h + 1) * hd] = orc.rope_apply(orc.rmsnorm(q[h * hd:(h + 1) * hd], qn[h * hd:(h + 1) * hd], 1e-6), hd, cos[pos], sin[pos])
        for h in range(nkv):
            ko[h * hd:(h + 1) * hd] = orc.rope_apply(orc.rmsnorm(k[h * hd:(h + 1) * hd], kn[h * hd:(h + 1) * hd], 1e-6), hd, cos[pos], sin[pos])
        kc[pos] = ko.reshape(nkv, hd); vc[pos] = v.reshape(nkv, hd)
        dq, dk, dv = ctx.to_device(q), ctx.to_device(k), ctx.to_device(v)
        L.atlas_qk_norm_inplace(dq, dqn, nh, hd, 1e-6); L.atlas_qk_norm_inplace(dk, dkn, nkv, hd, 1e-6)
        L.atlas_rope_precomputed(dq, dcos, dsin, nh, hd, pos, max_seq); L.atlas_rope_precomputed(dk, dcos, dsin, nkv, hd, pos, max_seq)
        L.atlas_kv_cache_write(dkc, dvc, dk, dv, pos, nkv, hd)
        for window in (0, 5):
            L.atlas_decode_attention(dq, dkc, dvc, dout, nh, nkv, hd, pos, scale, window); L.atlas_sync()
            ref = orc.decode_attention(qo, kc, vc, nh, nkv, hd, pos, scale, window)
            got = ctx.download(dout, (nh * hd,), np.float32)
            assert np.max(np.abs(got - ref)) < 2e-5, (pos, window)
        assert np.max(np.abs(ctx.download(dq, (nh * hd,), np.float32) - qo)) < 1e-5
        for p in (dq, dk, dv):
            ctx.free(p)
    assert np.max(np.abs(ctx.download(dkc, kc.shape, np.float32) - kc)) < 1e-5


def test_legacy_quantisers_keep_reference_kernel_semantics(ab, ctx):
    """atlas_quantize_int8/int4 follow kernels/matmul.cu:166-237 (ties to even, reciprocal 0 for
    an all-zero row, one int4 scale per tensor), NOT atlas-quant."""
    L = _legacy(ab)
    w = np.array([[2.0, 1.0, -1.0, 0.5], [0, 0, 0, 0]], np.float32)       # 1·63.5 = 63.5 → 64 (even)
    dw, dq, ds = ctx.to_device(w), ctx.malloc(16), ctx.malloc(16)
    L.atlas_quantize_int8(dw, dq, ds, 2, 4)
    q = ctx.download(dq, (2, 4), np.int8); s = ctx.download(ds, (2,), np.float32)
    assert q.tolist() == [[127, 64, -64, 32], [0, 0, 0, 0]] and s[1] == 0.0
    x = np.array([7.0, -7.0, 3.5, 2.5, 1.0], np.float32)                   # trailing odd element dropped
    dx, d4, d4s = ctx.to_device(x), ctx.malloc(16), ctx.malloc(16)
    check = np.zeros(3, np.uint8); ctx.upload(d4, check)
    L.atlas_quantize_int4(dx, d4, d4s, 5)
    out = ctx.download(d4, (3,), np.uint8)
    assert out.tolist() == [(7 << 4) | 9, (4 << 4) | 2, 0]                 # 3.5→4 (even), 2.5→2 (even)
    for p in (dw, dq, ds, dx, d4, d4s):
        ctx.free(p)


def test_bounded_device_wait_expires_with_an_error_status_and_leaves_the_context_usable(ab):
    """Failure detection on the device: a wait for data that never arrives (a mailbox part whose
    sequence words nothing sets) runs out after its limit, the kernel returns, the error word reads
    3, and the same context computes correctly afterwards."""
    import ctypes as C
    import time
    from atlas_b200 import _ffi
    ctx = ab.Context.default()
    code = C.c_int(-1)
    t0 = time.time()
    _ffi.check(_ffi.lib().atlasx_comm_selftest_wait_expiry(ctx.handle, C.byref(code), 0))
    dt = time.time() - t0
    assert code.value == 3
    assert 1.5 <= dt <= 10.0
    # the error word was cleared by the poll and the context still works
    w = np.arange(32 * 64, dtype=np.float32).reshape(32, 64) / 100.0
    x = np.ones(64, np.float32)
    y = ab.GpuMatrix.upload(w, 32, 64, ctx=ctx).sgemm_vec(ab.GpuVec.from_slice(x, ctx=ctx)).download()
    assert np.allclose(y, w @ x, rtol=1e-5)
    assert _ffi.lib().atlasx_ctx_poll_device_error(ctx.handle, C.byref(code)) == 0 and code.value == 0
