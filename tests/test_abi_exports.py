"""The shared library must load without a GPU and export every function that
include/atlas_kernels.h declares; the Python binding must cover the same set."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "atlas_kernels.h")


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(atlasx?_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_reference_abi():
    syms = declared_symbols()
    # the 19 functions crates/atlas-tensor/src/lib.rs:20-91 binds, plus the three quantisers
    # kernels/matmul.cu:559-578 exports
    for name in ["atlas_matmul_f32", "atlas_vec_add_f32", "atlas_scale_f32", "atlas_relu_f32", "atlas_softmax_f32",
                 "atlas_cuda_available", "atlas_cuda_device_count", "atlas_rmsnorm_f32", "atlas_rope_apply_f32",
                 "atlas_silu_mul_f32", "atlas_vram_copy_f32", "atlas_adamw_step", "atlas_sgemm_bf16_f32", "atlas_sync",
                 "atlas_qk_norm_inplace", "atlas_rope_precomputed", "atlas_kv_cache_write", "atlas_decode_attention",
                 "atlas_gpu_argmax", "atlas_quantize_int8", "atlas_dequantize_int8", "atlas_quantize_int4"]:
        assert name in syms, name


def test_library_exports_every_declared_symbol():
    from atlas_b200 import _ffi
    lib = ctypes.CDLL(_ffi.LIB_PATH)
    missing = [s for s in declared_symbols() if not hasattr(lib, s)]
    assert not missing, missing


def test_binding_covers_header():
    from atlas_b200 import _ffi
    assert sorted(_ffi.SIGNATURES) == declared_symbols()
    _ffi.lib()      # resolves every symbol with its signature


def test_static_archive_is_built():
    # the reference links `static=atlas_kernels` (crates/atlas-tensor/build.rs:104)
    from atlas_b200 import build
    assert os.path.exists(build.LIB_A)


def test_no_device_fails_loudly():
    import atlas_b200 as ab
    if os.path.exists("/dev/nvidiactl"):
        pytest.skip("a device is present")
    with pytest.raises(ab.AtlasError):
        ab.Context(0)
    assert ab.cuda_available() is False
