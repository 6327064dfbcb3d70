"""GPU: parity against the reference's OWN CUDA kernels (kernels/matmul.cu compiled unchanged
into oracle/_ref/libatlas_ref.so) driven through the reference's call sequence — the
'reference's own path on identical seeded inputs' of the task statement.
Skipped when that library was not built (it needs the reference checkout at build time)."""
import ctypes as C
import math
import os

import numpy as np
import pytest

from oracle import orc
import helpers
from helpers import rel_err

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref():
    if not os.path.exists(orc.REF_SO):
        pytest.skip("oracle/_ref/libatlas_ref.so not built")
    L = C.CDLL(orc.REF_SO)
    vp, ci, cf = C.c_void_p, C.c_int, C.c_float
    L.atlas_sgemm_bf16_f32.argtypes = [vp, vp, vp, ci, ci, ci]
    L.atlas_matmul_f32.argtypes = [vp, vp, vp, ci, ci, ci]
    L.atlas_decode_attention.argtypes = [vp, vp, vp, vp, ci, ci, ci, ci, cf, ci]
    L.atlas_sync.argtypes = []
    L.refgpu_model_new.restype = vp
    L.refgpu_model_new.argtypes = [ci, ci, ci, ci, ci, ci, ci, cf, cf, ci, vp]
    L.refgpu_model_free.argtypes = [vp]
    L.refgpu_set_tensor.argtypes = [vp, ci, ci, vp, ci]
    L.refgpu_upload_rope.argtypes = [vp, vp, vp]
    L.refgpu_reset.argtypes = [vp]
    L.refgpu_forward_one.restype = ci
    L.refgpu_forward_one.argtypes = [vp, C.c_uint32, vp]
    return L


@pytest.fixture(scope="module")
def ab():
    import atlas_b200
    orc.set_threads(os.cpu_count() or 1)
    return atlas_b200


@pytest.mark.parametrize("shape", [(4096, 4096), (11008, 4096), (4096, 11008), (100352, 4096)])
def test_bf16_gemv_vs_reference_sgemv_kernel(ab, ref, shape):
    """BASELINE config 2: compared against the reference sgemv_bf16_kernel output."""
    from atlas_b200 import _ffi
    M, K = shape
    ctx = ab.Context.default()
    w = ctx.malloc(M * K * 2)
    _ffi.check(_ffi.lib().atlasx_fill_normal_bf16(ctx.handle, w, M * K, 61, M + K, 0, 0.02))
    x = orc.normal_f32(K, 61, 5, 1.0)
    dx, dy_ref = ctx.to_device(x), ctx.malloc(M * 4)
    ctx.sync()
    ref.atlas_sgemm_bf16_f32(w, dx, dy_ref, M, 1, K); ref.atlas_sync()
    y_ref = ctx.download(dy_ref, (M,), np.float32)
    gm = ab.GpuMatrix.wrap(ab.BF16, w, 0, M, K)
    for impl in (1, 2):
        ctx.set_gemv_impl(impl)
        y = gm.sgemm_vec(ab.GpuVec(ctx, dx, K, owner=False), 1).download()
        assert rel_err(y, y_ref) <= 1e-3
    ctx.set_gemv_impl(0)
    for p in (w, dx, dy_ref):
        ctx.free(p)


@pytest.mark.parametrize("ctx_len,window", [(1024, 0), (8192, 0), (8192, 4096), (12000, 4096)])
def test_attention_vs_reference_decode_attention_kernel(ab, ref, ctx_len, window):
    """BASELINE config 5 against the reference decode_attention_kernel, fed an f32 cache that
    holds the identical bf16-rounded values.  The reference kernel keeps one score per position
    in shared memory without opting in to more than 48 KB, so it cannot run past ~12k positions;
    longer contexts are covered by the CPU oracle in test_gpu_attention.py."""
    nh, nkv, hd = 32, 8, 128
    ctx = ab.Context.default()
    n = ctx_len * nkv * hd
    k16 = orc.normal_bf16(n, 62, 1, 1.0); v16 = orc.normal_bf16(n, 62, 2, 1.0)
    q = orc.normal_f32(nh * hd, 62, 3, 1.0)
    kf, vf = ctx.to_device(orc.bf16_to_f32(k16)), ctx.to_device(orc.bf16_to_f32(v16))
    dq, dout = ctx.to_device(q), ctx.malloc(nh * hd * 4)
    scale = 1.0 / math.sqrt(hd)
    ctx.sync()
    ref.atlas_decode_attention(dq, kf, vf, dout, nh, nkv, hd, ctx_len - 1, scale, window); ref.atlas_sync()
    want = ctx.download(dout, (nh * hd,), np.float32)
    assert np.all(np.isfinite(want)) and np.abs(want).max() > 0
    kv = ab.GpuKvCache(ctx_len, nkv, hd, dtype=ab.BF16)
    kp, vp, _ = kv.ptrs()
    ctx.upload(kp, k16); ctx.upload(vp, v16)
    got = kv.decode_attention(ab.GpuVec(ctx, dq, nh * hd, owner=False), nh, ctx_len - 1, scale, window).download()
    assert rel_err(got, want) <= 1e-3
    for p in (kf, vf, dq, dout):
        ctx.free(p)


def _ref_model(ref, ctx, cfg, dev_tensors, layer_sliding, cos, sin, scale):
    windows = (C.c_int * cfg["n_layers"])(*[(cfg.get("sliding_window", 0) if (layer_sliding and layer_sliding[l]) else 0)
                                            for l in range(cfg["n_layers"])])
    h = ref.refgpu_model_new(cfg["vocab_size"], cfg["d_model"], cfg["n_layers"], cfg["n_heads"], cfg["n_kv_heads"],
                             cfg["ffn_hidden"], cfg["max_seq_len"], cfg["rms_norm_eps"], scale, cfg.get("post_norm", 0), windows)
    for (layer, which), (ptr, dt) in dev_tensors.items():
        assert ref.refgpu_set_tensor(h, layer, which, ptr, dt) == 0
    ref.refgpu_upload_rope(h, cos.ctypes.data, sin.ctypes.data)
    return h


def test_small_model_vs_reference_gpu_path(ab, ref):
    """Whole-model decode against the reference's GPU call sequence on a small OLMo-3-shaped
    model (f32 weights, f32 cache on both sides): tokens identical, |Δlogit| ≤ 1e-2."""
    cfg = dict(helpers.SMALL_SWA)
    w = helpers.synth_weights(cfg, seed=9, norm_jitter=0.1)
    ctx = ab.Context.default()
    dev = {}
    helpers.give(None, w, set_fn=lambda l, t, a: dev.__setitem__((l, t), (ctx.to_device(np.ascontiguousarray(a, np.float32)), 0)))
    hd = cfg["d_model"] // cfg["n_heads"]
    cos, sin = ab.rope_tables(hd, cfg["max_seq_len"], cfg["rope_theta"],
                              dict(factor=cfg["yarn_factor"], orig_max_pos=cfg["yarn_orig_max_pos"],
                                   beta_fast=cfg["yarn_beta_fast"], beta_slow=cfg["yarn_beta_slow"]))
    oc, osn = orc.rope_tables(hd, cfg["max_seq_len"], cfg["rope_theta"],
                              dict(factor=cfg["yarn_factor"], orig_max_pos=cfg["yarn_orig_max_pos"],
                                   beta_fast=cfg["yarn_beta_fast"], beta_slow=cfg["yarn_beta_slow"]))
    assert np.array_equal(cos, oc) and np.array_equal(sin, osn)
    scale = np.float32(1.0) / np.sqrt(np.float32(hd)) * np.float32(cfg["yarn_attn_factor"])
    h = _ref_model(ref, ctx, cfg, dev, helpers.SMALL_SWA_LAYERS, cos, sin, float(scale))
    m = helpers.cuda_model(cfg, w, helpers.SMALL_SWA_LAYERS, kv_dtype=ab.F32)
    prompt = orc.uniform_u32(16, 9, 1, cfg["vocab_size"])
    logits_ref = np.empty(cfg["vocab_size"], np.float32)
    seq = list(prompt)
    worst = 0.0
    for i in range(16 + 40):
        t = int(seq[i])
        assert ref.refgpu_forward_one(h, t, logits_ref.ctypes.data) == 0
        lg = m.forward_one_gpu(t)
        worst = max(worst, float(np.max(np.abs(lg - logits_ref))))
        if i >= 15:
            nxt = orc.argmax(logits_ref)
            assert nxt == orc.argmax(lg)
            seq.append(nxt)
    assert worst <= 1e-2
    ref.refgpu_model_free(h)
    for ptr, _ in dev.values():
        ctx.free(ptr)


def test_olmo3_7b_arch_vs_reference_gpu_path(ab, ref):
    """BASELINE config 4: OLMo-3-7B architecture, random init N(0,0.02) stored as bf16, 2048-token
    random prompt, 256 greedy tokens, against the reference's GPU call sequence on the same
    device tensors (the reference keeps an f32 KV cache).
      * f32 KV cache (the reference's format): free-running greedy tokens identical;
      * bf16 KV cache (an extension: half the cache traffic): teacher-forced on the reference's
        tokens.  Rounding K and V to 8 mantissa bits through 32 layers at 2k context moves the
        logits by ≈3e-2 (measured 2.8e-2), which is a property of the format, not of the kernels
        (the same kernels with the f32 cache pass the line above); asserted: |Δlogit| ≤ 5e-2 and
        the greedy choice agrees wherever the reference's top-1/top-2 gap exceeds twice the
        largest observed difference.
    ATLAS_C4_PROMPT shortens the prompt for a quick run."""
    from atlas_b200 import _ffi
    n_prompt = int(os.environ.get("ATLAS_C4_PROMPT", "2048"))
    n_new = 256
    mc = ab.ModelConfig.olmo3_actual_7b(max_seq_len=n_prompt + n_new + 8)
    ctx = ab.Context.default()
    L = _ffi.lib()
    d, f, V, hd = mc.d_model, mc.ffn_hidden, mc.vocab_size, 128
    dev = {}

    def mat(layer, which, rows, cols, stream):
        p = ctx.malloc(rows * cols * 2)
        _ffi.check(L.atlasx_fill_normal_bf16(ctx.handle, p, rows * cols, 0, stream, 0, 0.02))
        dev[(layer, which)] = (p, 1)
    mat(0, orc.T_EMBED, V, d, 1)
    mat(0, orc.T_LM_HEAD, V, d, 2)
    ones = ctx.to_device(np.ones(d, np.float32))
    dev[(0, orc.T_FINAL_NORM)] = (ones, 0)
    shapes = {"wq": (d, d), "wk": (d, d), "wv": (d, d), "wo": (d, d), "gate": (f, d), "up": (f, d), "down": (d, f)}
    for l in range(mc.n_layers):
        for name, tid in helpers.PER_LAYER:
            mat(l, tid, shapes[name][0], shapes[name][1], 1000 + l * 32 + tid)
        for tid in (orc.T_ATTN_NORM, orc.T_FFN_NORM, orc.T_Q_NORM, orc.T_K_NORM):
            dev[(l, tid)] = (ones, 0)

    def build(kv_dtype):
        m = ab.OlmoModel(mc, kv_dtype=kv_dtype, weight_format=ab.BF16)
        for (layer, which), (ptr, dt) in dev.items():
            m.set_tensor(layer, which, ptr, on_device=True, dtype=ab.BF16 if dt else ab.F32)
        m.init_gpu_resources()
        return m

    cos, sin = ab.rope_tables(hd, mc.max_seq_len, mc.rope_theta,
                              dict(factor=8.0, orig_max_pos=8192, beta_fast=32.0, beta_slow=1.0))
    scale = float(np.float32(1.0) / np.sqrt(np.float32(hd)) * np.float32(mc.rope_scaling.attn_factor))
    cfg = dict(vocab_size=V, d_model=d, n_layers=32, n_heads=32, n_kv_heads=32, ffn_hidden=f,
               max_seq_len=mc.max_seq_len, rms_norm_eps=mc.rms_norm_eps, post_norm=1, sliding_window=4096)
    h = _ref_model(ref, ctx, cfg, dev, [int(t == ab.LAYER_SLIDING) for t in mc.layer_types], cos, sin, scale)
    prompt = orc.uniform_u32(n_prompt, 0, 99, V)

    # reference: free-running greedy with the CPU argmax rule, logits kept for every step
    ref_logits = np.empty((n_new, V), np.float32)
    for t in prompt[:-1]:
        assert ref.refgpu_forward_one(h, int(t), None) == 0
    assert ref.refgpu_forward_one(h, int(prompt[-1]), ref_logits[0].ctypes.data) == 0
    ref_toks, margins = [], []
    for i in range(n_new):
        nxt = orc.argmax(ref_logits[i])
        top2 = np.partition(ref_logits[i], -2)[-2:]
        margins.append(float(top2[1] - top2[0]))
        ref_toks.append(nxt)
        if i + 1 < n_new:
            assert ref.refgpu_forward_one(h, nxt, ref_logits[i + 1].ctypes.data) == 0
    ref.refgpu_model_free(h)
    assert np.all(np.isfinite(ref_logits))

    # f32 cache: identical greedy tokens
    m = build(ab.F32)
    toks = m.generate(prompt, n_new, 0.0)
    first_diff = next((i for i in range(n_new) if toks[i] != ref_toks[i]), None)
    assert first_diff is None, "token %s differs (reference margin there %.3g, min margin %.3g)" % (
        first_diff, margins[first_diff], min(margins))
    del m

    # bf16 cache: teacher-forced logits
    m = build(ab.BF16)
    seq = list(prompt) + ref_toks
    worst, flips = 0.0, []
    for i in range(n_prompt - 1):
        m.forward_one_gpu(int(seq[i]), want_logits=False)
    for i in range(n_new):
        lg = m.forward_one_gpu(int(seq[n_prompt - 1 + i]))
        worst = max(worst, float(np.max(np.abs(lg - ref_logits[i]))))
        if orc.argmax(lg) != ref_toks[i]:
            flips.append(i)
    print("bf16 KV cache: max |dlogit| vs reference = %.4g, flips %s" % (worst, flips))
    assert worst <= 5e-2, worst
    for i in flips:
        assert margins[i] <= 2 * worst, "step %d flipped with margin %.3g > 2×%.3g" % (i, margins[i], worst)
    del m
    for ptr, _ in set(dev.values()):
        ctx.free(ptr)
