"""GPU: split-K GQA decode attention over a bf16 or f32 KV cache against the CPU oracle fed the
identical (bf16-rounded) values — BASELINE config 5 shapes: 32 query heads, 8 KV heads,
head_dim 128, contexts 1k/8k/32k, batch 1/8/64, full and window-4096 masks.
Tolerance 1e-3 in the max-abs relative form."""
import math
import os

import numpy as np
import pytest

from oracle import orc
from helpers import rel_err

pytestmark = pytest.mark.gpu
TOL = 1e-3
G = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.fixture(scope="module")
def ab():
    import atlas_b200
    orc.set_threads(os.cpu_count() or 1)
    return atlas_b200


def fill_cache(ab, kv, rows, seed, keep=None):
    """Fill rows [0, rows) of every sequence of the cache from the seeded generator and return
    the values as f32 (exactly what the cache holds); `keep` limits the host copies to the
    sequences that will be checked (the others come back as None)."""
    from atlas_b200 import _ffi
    ctx = kv.ctx
    kptr, vptr, _ = kv.ptrs()
    per_seq = kv.max_seq * kv.n_kv_heads * kv.head_dim
    n = rows * kv.n_kv_heads * kv.head_dim
    ks, vs = [], []
    esz = 2 if kv.dtype == ab.BF16 else 4
    for b in range(kv.batch):
        for ptr, stream, acc in ((kptr, 2 * b, ks), (vptr, 2 * b + 1, vs)):
            dst = ptr + b * per_seq * esz
            host = keep is None or b in keep
            if kv.dtype == ab.BF16:
                _ffi.check(_ffi.lib().atlasx_fill_normal_bf16(ctx.handle, dst, n, seed, stream, 0, 1.0))
                acc.append(orc.bf16_to_f32(orc.normal_bf16(n, seed, stream, 1.0)) if host else None)
            else:
                _ffi.check(_ffi.lib().atlasx_fill_normal_f32(ctx.handle, dst, n, seed, stream, 0, 1.0))
                acc.append(orc.normal_f32(n, seed, stream, 1.0) if host else None)
    return ks, vs


def run_case(ab, nh, nkv, hd, ctx_len, batch, window, dtype, positions=None):
    max_seq = ctx_len
    kv = ab.GpuKvCache(max_seq, nkv, hd, dtype=dtype, batch=batch)
    check = list(range(batch)) if batch <= 8 else [0, batch // 2, batch - 1]
    ks, vs = fill_cache(ab, kv, ctx_len, 51, keep=check)
    q = orc.normal_f32(batch * nh * hd, 52, ctx_len, 1.0)
    pos = positions if positions is not None else [ctx_len - 1] * batch
    scale = 1.0 / math.sqrt(hd)
    out = kv.decode_attention(ab.GpuVec.from_slice(q), nh, pos, scale, window).download().reshape(batch, nh * hd)
    assert kv.ctx.poll_device_error() == 0
    for b in check:
        ref = orc.decode_attention(q[b * nh * hd:(b + 1) * nh * hd], ks[b], vs[b], nh, nkv, hd, pos[b], scale, window)
        assert rel_err(out[b], ref) <= TOL, (b, pos[b])
    return kv


@pytest.mark.parametrize("dtype_name", ["bf16", "f32"])
@pytest.mark.parametrize("ctx_len,batch", [(1024, 1), (1024, 8), (1024, 64), (8192, 1), (8192, 8), (32768, 1)])
@pytest.mark.parametrize("window", [0, 4096])
def test_config5_shapes(ab, dtype_name, ctx_len, batch, window):
    dtype = ab.BF16 if dtype_name == "bf16" else ab.F32
    run_case(ab, 32, 8, 128, ctx_len, batch, window, dtype)


@pytest.mark.parametrize("ctx_len", [8192, 32768])
@pytest.mark.parametrize("window", [0, 4096])
def test_config5_batch_64_long_contexts(ab, ctx_len, window):
    """The batch-64 cells of BASELINE config 5 at 8k and 32k context (2.1 GB and 8.6 GB each of bf16
    K and V): first, middle and last sequence against the oracle."""
    run_case(ab, 32, 8, 128, ctx_len, 64, window, ab.BF16)


def test_config5_largest(ab):
    """32k context × batch 8 (8.6 GB of bf16 cache): checked on three sequences."""
    run_case(ab, 32, 8, 128, 32768, 8, 4096, ab.BF16)
    run_case(ab, 32, 8, 128, 32768, 8, 0, ab.BF16)


@pytest.mark.parametrize("nh,nkv,hd", [(32, 32, 128), (8, 8, 64), (8, 2, 64), (4, 2, 16), (15, 5, 64), (6, 2, 128), (9, 3, 64),
                                       (16, 2, 128), (10, 2, 128), (14, 2, 128)])
def test_head_layouts(ab, nh, nkv, hd):
    """MHA (config 4), GQA groups of 1/2/3/4 and 5/7/8 (the two forms of the tensor-core kernel at head_dim 128),
    small and odd head_dim (generic kernel)."""
    for dtype in (ab.BF16, ab.F32):
        run_case(ab, nh, nkv, hd, 300, 2, 0, dtype, positions=[299, 57])


@pytest.mark.parametrize("window", [1, 8, 64])
def test_window_edges(ab, window):
    """pos = 0, window−1, window, window+1: the mask is pos − t ≥ window (matmul.cu:815)."""
    nh, nkv, hd = 8, 2, 64
    for pos in sorted({0, max(window - 1, 0), window, window + 1, 3 * window + 5}):
        run_case(ab, nh, nkv, hd, 3 * window + 6, 1, window, ab.BF16, positions=[pos])


def test_ragged_batch_positions(ab):
    run_case(ab, 32, 8, 128, 2048, 8, 0, ab.BF16, positions=[0, 1, 17, 500, 1023, 1024, 2000, 2047])
    run_case(ab, 32, 8, 128, 2048, 8, 100, ab.BF16, positions=[0, 99, 100, 101, 1023, 1024, 2000, 2047])


def test_kvcache_write_and_bf16_rounding(ab):
    nkv, hd, batch = 2, 64, 3
    for dtype in (ab.BF16, ab.F32):
        kv = ab.GpuKvCache(16, nkv, hd, dtype=dtype, batch=batch)
        k = orc.normal_f32(batch * nkv * hd, 53, 1); v = orc.normal_f32(batch * nkv * hd, 53, 2)
        pos = [0, 5, 15]
        kv.write(pos, ab.GpuVec.from_slice(k), ab.GpuVec.from_slice(v))
        kp, vp, nbytes = kv.ptrs()
        np_dt = np.uint16 if dtype == ab.BF16 else np.float32
        kc = kv.ctx.download(kp, (batch, 16, nkv * hd), np_dt); vc = kv.ctx.download(vp, (batch, 16, nkv * hd), np_dt)
        for b, p in enumerate(pos):
            want_k = k[b * nkv * hd:(b + 1) * nkv * hd]; want_v = v[b * nkv * hd:(b + 1) * nkv * hd]
            if dtype == ab.BF16:
                assert np.array_equal(kc[b, p], orc.f32_to_bf16_rne(want_k)) and np.array_equal(vc[b, p], orc.f32_to_bf16_rne(want_v))
            else:
                assert np.array_equal(kc[b, p], want_k) and np.array_equal(vc[b, p], want_v)
            other = [r for r in range(16) if r != p]
            assert not kc[b, other].any()               # GpuKvCache::new is zeroed; only pos was written
        with pytest.raises(ab.AtlasError):
            kv.write([0, 0, 16], ab.GpuVec.from_slice(k), ab.GpuVec.from_slice(v))


def test_golden_fixtures(ab):
    g = np.load(os.path.join(G, "attention.npz"))
    nh, nkv, hd = 8, 2, 64
    from atlas_b200 import _ffi
    for pos, window in [(0, 0), (37, 0), (37, 8), (7, 8), (8, 8)]:
        kv = ab.GpuKvCache(pos + 1, nkv, hd, dtype=ab.BF16)
        n = (pos + 1) * nkv * hd
        kp, vp, _ = kv.ptrs()
        _ffi.check(_ffi.lib().atlasx_fill_normal_bf16(kv.ctx.handle, kp, n, 23, 1, 0, 1.0))
        _ffi.check(_ffi.lib().atlasx_fill_normal_bf16(kv.ctx.handle, vp, n, 23, 2, 0, 1.0))
        q = orc.normal_f32(nh * hd, 23, 3, 1.0)
        out = kv.decode_attention(ab.GpuVec.from_slice(q), nh, pos, 1.0 / np.sqrt(hd), window).download()
        assert rel_err(out, g["p%d_w%d" % (pos, window)]) <= TOL


def test_softmax_weights_sum_to_one_property(ab):
    """With V ≡ 1 the output must be exactly 1 in every dimension whatever the context, split
    count and mask are (size-independent property at full size: 32k × batch 8)."""
    nh, nkv, hd, ctx_len, batch = 32, 8, 128, 32768, 8
    kv = ab.GpuKvCache(ctx_len, nkv, hd, dtype=ab.BF16, batch=batch)
    from atlas_b200 import _ffi
    kp, vp, nbytes = kv.ptrs()
    _ffi.check(_ffi.lib().atlasx_fill_normal_bf16(kv.ctx.handle, kp, nbytes // 2, 54, 1, 0, 1.0))
    ones = np.full(1 << 20, 0x3F80, np.uint16)
    dones = kv.ctx.to_device(ones)
    for off in range(0, nbytes, ones.nbytes):
        _ffi.check(_ffi.lib().atlasx_copy_dev(kv.ctx.handle, vp + off, dones, min(ones.nbytes, nbytes - off)))
    q = orc.normal_f32(batch * nh * hd, 54, 2, 1.0)
    for window in (0, 4096):
        out = kv.decode_attention(ab.GpuVec.from_slice(q), nh, [ctx_len - 1 - 1000 * b for b in range(batch)],
                                  1.0 / math.sqrt(hd), window).download()
        assert np.max(np.abs(out - 1.0)) < 1e-5
    kv.ctx.free(dones)
