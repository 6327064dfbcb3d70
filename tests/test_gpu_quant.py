"""GPU: atlas-quant formats on the device are bit-exact with the CPU oracle
(crates/atlas-quant/src/lib.rs:41-168), including ragged shapes, zero rows, exact .5 ties and
blocks that straddle rows."""
import hashlib
import os

import numpy as np
import pytest

from oracle import orc

pytestmark = pytest.mark.gpu
G = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


@pytest.fixture(scope="module")
def ab():
    import atlas_b200
    return atlas_b200


@pytest.mark.parametrize("rows,cols", [(1, 1), (3, 5), (7, 257), (16, 4096), (64, 11008), (2, 2)])
def test_int8_bit_exact(ab, rows, cols):
    w = orc.normal_f32(rows * cols, 31, rows * 7919 + cols, 0.02).reshape(rows, cols)
    w[0, :] = 0.0
    if rows > 1 and cols >= 2:
        w[1, 0], w[1, 1] = 2.0, 1.0          # 1·(127/2) = 63.5: half away from zero → 64
    q = ab.Int8Tensor.quantize(w)
    qo, so = orc.int8_quantize(w)
    assert np.array_equal(q.scales.view(np.uint32), so.view(np.uint32))
    assert np.array_equal(q.data.reshape(rows, cols), qo)
    assert np.array_equal(q.dequantize().view(np.uint32), orc.int8_dequantize(qo, so).view(np.uint32))
    assert q.memory_bytes() == rows * cols + 4 * rows


@pytest.mark.parametrize("rows,cols,block", [(1, 64, 64), (4, 128, 32), (3, 50, 32), (5, 33, 64), (2, 7, 4), (3, 5, 3),
                                              (16, 4096, 32), (8, 11008, 32), (8, 4096, 64)])
def test_int4_bit_exact(ab, rows, cols, block):
    w = orc.normal_f32(rows * cols, 32, rows * 7919 + cols + block, 0.02).reshape(rows, cols)
    w.ravel()[:min(block, w.size)] = 0.0
    if w.size > block + 2:
        w.ravel()[block], w.ravel()[block + 1] = 7.0, 3.5       # 3.5 → 4, an exact tie
    q = ab.Int4Tensor.quantize(w, block)
    qo, so = orc.int4_quantize(w, block)
    assert np.array_equal(q.scales.view(np.uint32), so.view(np.uint32))
    assert np.array_equal(q.data, qo)
    assert np.array_equal(q.dequantize().ravel().view(np.uint32), orc.int4_dequantize(qo, so, w.size, block).view(np.uint32))


def test_reference_roundtrip_cases(ab):
    # crates/atlas-quant/src/lib.rs:258-297
    t = np.array([[1.0, -2.0], [3.0, -4.0]], np.float32)
    q = ab.Int8Tensor.quantize(t)
    assert np.max(np.abs(q.dequantize() - t)) < 0.1
    assert ab.Int8Tensor.quantize(np.ones((128, 128), np.float32)).compression_ratio() > 3.5
    data = (np.arange(64, dtype=np.float32) * np.float32(0.1) - np.float32(3.0)).reshape(1, 64)
    q4 = ab.Int4Tensor.quantize(data, ab.INT4_BLOCK_SIZE)
    assert np.max(np.abs(q4.dequantize() - data)) < 0.5
    assert ab.Int4Tensor.quantize(np.ones((128, 128), np.float32), ab.INT4_BLOCK_SIZE).compression_ratio() > 7.0
    with pytest.raises(ab.AtlasError):
        ab.Int8Tensor.quantize(np.ones(4, np.float32))


def test_golden_fixtures(ab):
    g = np.load(os.path.join(G, "quant.npz"))
    for rows, cols, block in [(7, 257, 32), (16, 4096, 32), (5, 96, 64), (64, 11008, 32)]:
        w = orc.normal_f32(rows * cols, 21, rows * 100000 + cols, 0.02).reshape(rows, cols)
        w[0, :] = 0.0
        q8 = ab.Int8Tensor.quantize(w); q4 = ab.Int4Tensor.quantize(w, block)
        key = "%dx%d_b%d" % (rows, cols, block)
        assert sha(q8.data) == str(g[key + "_i8_sha"]) and sha(q8.scales) == str(g[key + "_s8_sha"])
        assert sha(q4.data) == str(g[key + "_i4_sha"]) and sha(q4.scales) == str(g[key + "_s4_sha"])


def test_full_size_checksum_of_checksums(ab):
    """BASELINE shapes at full size on the device: quantise 11008×4096 in row chunks and as a
    whole — per-row formats must not depend on how the matrix is cut (size-independent property),
    and a CPU-checked sample of rows must match bit for bit."""
    rows, cols = 11008, 4096
    ctx = ab.Context.default()
    from atlas_b200 import _ffi
    src = ctx.malloc(rows * cols * 4)
    _ffi.check(_ffi.lib().atlasx_fill_normal_f32(ctx.handle, src, rows * cols, 33, 1, 0, 0.02))
    d8, s8 = ctx.malloc(rows * cols), ctx.malloc(rows * 4)
    _ffi.check(_ffi.lib().atlasx_quantize_int8(ctx.handle, src, rows, cols, d8, s8))
    whole = ctx.download(d8, (rows, cols), np.int8); whole_s = ctx.download(s8, (rows,), np.float32)
    half = rows // 2
    _ffi.check(_ffi.lib().atlasx_quantize_int8(ctx.handle, src + half * cols * 4, rows - half, cols, d8, s8))
    part = ctx.download(d8, (rows - half, cols), np.int8)
    assert np.array_equal(part, whole[half:])
    sample = [0, 1, 4095, 5504, 11007]
    w = np.array([[orc.lib().orc_synth_normal(33, 1, r * cols + c) for c in range(0, cols, 512)] for r in sample], np.float32)
    host = ctx.download(src, (rows, cols), np.float32)
    assert np.array_equal(host[sample][:, ::512], (w * np.float32(0.02)).astype(np.float32))
    qo, so = orc.int8_quantize(host[sample])
    assert np.array_equal(qo, whole[sample]) and np.array_equal(so, whole_s[sample])
    d4, s4 = ctx.malloc(rows * cols // 2), ctx.malloc(rows * cols // 32 * 4)
    _ffi.check(_ffi.lib().atlasx_quantize_int4(ctx.handle, src, rows * cols, 32, d4, s4))
    q4 = ctx.download(d4, (rows, cols // 2), np.uint8); sc4 = ctx.download(s4, (rows, cols // 32), np.float32)
    q4o, s4o = orc.int4_quantize(host[sample], 32)
    assert np.array_equal(q4o.reshape(len(sample), -1), q4[sample]) and np.array_equal(s4o.reshape(len(sample), -1), sc4[sample])
    for p in (src, d8, s8, d4, s4):
        ctx.free(p)
