"""ctypes view of the CPU oracle (oracle/atlas_oracle.c) and of the reference's own CUDA
kernels built into oracle/_ref/libatlas_ref.so.

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the CPU-baseline
leg of the benchmark.  The product package never imports this module.
"""
import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "_build", "liboracle.so")
REF_SO = os.path.join(HERE, "_ref", "libatlas_ref.so")

# tensor ids shared by atlas_oracle.h and ref_gpu_harness.cu
T_EMBED, T_FINAL_NORM, T_LM_HEAD = 0, 1, 2
T_WQ, T_WK, T_WV, T_WO, T_GATE, T_UP, T_DOWN = 10, 11, 12, 13, 14, 15, 16
T_ATTN_NORM, T_FFN_NORM, T_Q_NORM, T_K_NORM = 17, 18, 19, 20


class OrcConfig(C.Structure):
    _fields_ = [
        ("vocab_size", C.c_int), ("d_model", C.c_int), ("n_layers", C.c_int),
        ("n_heads", C.c_int), ("n_kv_heads", C.c_int), ("ffn_hidden", C.c_int),
        ("max_seq_len", C.c_int), ("rope_theta", C.c_float), ("rms_norm_eps", C.c_float),
        ("sliding_window", C.c_int), ("rope_scaling", C.c_int), ("yarn_factor", C.c_float),
        ("yarn_orig_max_pos", C.c_int), ("yarn_attn_factor", C.c_float),
        ("yarn_beta_fast", C.c_float), ("yarn_beta_slow", C.c_float),
        ("post_norm", C.c_int), ("eos_token_id", C.c_int),
    ]


class OrcSampling(C.Structure):
    _fields_ = [("temperature", C.c_float), ("repetition_penalty", C.c_float), ("repetition_window", C.c_int),
                ("frequency_penalty", C.c_float), ("presence_penalty", C.c_float), ("top_p", C.c_float),
                ("top_k", C.c_int), ("min_p", C.c_float)]


def sampling(temperature=1.0, repetition_penalty=1.0, repetition_window=64, frequency_penalty=0.0, presence_penalty=0.0,
             top_p=1.0, top_k=0, min_p=0.0):
    """SamplingConfig (defaults of :1250-1263)."""
    return OrcSampling(temperature, repetition_penalty, repetition_window, frequency_penalty, presence_penalty, top_p, top_k, min_p)


def build(force=False):
    """Compile the CPU oracle (and the reference kernels when the checkout is present)."""
    if force or not os.path.exists(ORACLE_SO) or \
            os.path.getmtime(ORACLE_SO) < os.path.getmtime(os.path.join(HERE, "atlas_oracle.c")):
        subprocess.run(["make", "-C", HERE, "_build/liboracle.so"], check=True, capture_output=True)
    # the reference checkout: ATLAS_REF, else a `reference` directory beside this repository
    ref_src = os.environ.get("ATLAS_REF") or os.path.abspath(os.path.join(HERE, "..", "..", "reference"))
    if os.path.exists(os.path.join(ref_src, "kernels", "matmul.cu")):
        subprocess.run(["make", "-C", HERE, "ref", "REF=" + ref_src], check=True, capture_output=True)


_lib = None


def _p(a, ctype):
    return a.ctypes.data_as(C.POINTER(ctype))


def lib():
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(ORACLE_SO):
        build()
    L = C.CDLL(ORACLE_SO)
    u64, sz, f32p = C.c_uint64, C.c_size_t, C.POINTER(C.c_float)
    L.orc_mix64.restype = u64; L.orc_mix64.argtypes = [u64]
    L.orc_synth_normal.restype = C.c_float; L.orc_synth_normal.argtypes = [u64, u64, u64]
    L.orc_fill_normal_f32.argtypes = [f32p, sz, u64, u64, C.c_float]
    L.orc_fill_normal_bf16.argtypes = [C.POINTER(C.c_uint16), sz, u64, u64, C.c_float]
    L.orc_fill_uniform_u32.argtypes = [C.POINTER(C.c_uint32), sz, u64, u64, C.c_uint32]
    L.orc_pseudo_randn.argtypes = [f32p, sz, u64]
    L.orc_int8_quantize.argtypes = [f32p, sz, sz, C.POINTER(C.c_int8), f32p]
    L.orc_int8_dequantize.argtypes = [C.POINTER(C.c_int8), f32p, sz, sz, f32p]
    L.orc_int4_quantize.argtypes = [f32p, sz, sz, C.POINTER(C.c_uint8), f32p]
    L.orc_int4_dequantize.argtypes = [C.POINTER(C.c_uint8), f32p, sz, sz, f32p]
    L.orc_rmsnorm_inplace.argtypes = [f32p, f32p, sz, C.c_float]
    L.orc_silu.restype = C.c_float; L.orc_silu.argtypes = [C.c_float]
    L.orc_softmax_inplace.argtypes = [f32p, sz]
    L.orc_argmax.restype = sz; L.orc_argmax.argtypes = [f32p, sz]
    L.orc_rope_tables.argtypes = [C.c_int, C.c_int, C.c_float, C.c_int, C.c_float, C.c_int,
                                  C.c_float, C.c_float, f32p, f32p]
    L.orc_rope_apply.argtypes = [f32p, C.c_int, f32p, f32p]
    L.orc_linear_f32.argtypes = [f32p, f32p, f32p, sz, sz]
    L.orc_linear_bf16.argtypes = [C.POINTER(C.c_uint16), f32p, f32p, sz, sz]
    L.orc_gemm_f32.argtypes = [f32p, f32p, f32p, sz, sz, sz]
    L.orc_gemm_bf16.argtypes = [C.POINTER(C.c_uint16), f32p, f32p, sz, sz, sz]
    L.orc_decode_attention.argtypes = [f32p, f32p, f32p, f32p, C.c_int, C.c_int, C.c_int,
                                       C.c_int, C.c_float, C.c_int]
    L.orc_model_new.restype = C.c_void_p
    L.orc_model_new.argtypes = [C.POINTER(OrcConfig), C.POINTER(C.c_int)]
    L.orc_model_free.argtypes = [C.c_void_p]
    L.orc_model_set_tensor.restype = C.c_int
    L.orc_model_set_tensor.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_int]
    L.orc_model_init_reference_random.argtypes = [C.c_void_p]
    L.orc_model_set_kv_round_bf16.argtypes = [C.c_void_p, C.c_int]
    L.orc_model_reset.argtypes = [C.c_void_p]
    L.orc_model_pos.restype = C.c_int; L.orc_model_pos.argtypes = [C.c_void_p]
    L.orc_model_seed_context.argtypes = [C.c_void_p, C.c_int, u64]
    L.orc_forward_one.argtypes = [C.c_void_p, C.c_uint32, f32p, f32p]
    L.orc_generate_greedy.restype = C.c_int
    L.orc_generate_greedy.argtypes = [C.c_void_p, C.POINTER(C.c_uint32), C.c_int, C.c_int,
                                      C.POINTER(C.c_uint32), C.c_int, C.c_float, C.c_int,
                                      C.POINTER(C.c_uint32), C.c_int,
                                      C.POINTER(C.c_uint32), f32p, f32p]
    u32p = C.POINTER(C.c_uint32)
    L.orc_rng_from_seed.restype = u64; L.orc_rng_from_seed.argtypes = [u64]
    L.orc_rng_next_f32.restype = C.c_float; L.orc_rng_next_f32.argtypes = [C.POINTER(u64)]
    L.orc_apply_repetition_penalty.argtypes = [f32p, sz, u32p, C.c_int, C.c_float]
    L.orc_apply_frequency_penalty.argtypes = [f32p, sz, u32p, C.c_int, C.c_float]
    L.orc_apply_presence_penalty.argtypes = [f32p, sz, u32p, C.c_int, C.c_float]
    L.orc_apply_top_k.argtypes = [f32p, sz, sz]
    L.orc_apply_top_p.argtypes = [f32p, sz, C.c_float]
    L.orc_apply_min_p.argtypes = [f32p, sz, C.c_float]
    L.orc_sample_from_probs.restype = sz; L.orc_sample_from_probs.argtypes = [f32p, sz, C.c_float]
    L.orc_sample_token.restype = sz
    L.orc_sample_token.argtypes = [f32p, sz, C.POINTER(OrcSampling), C.c_int, u32p, C.c_int, u32p, C.c_int, C.POINTER(u64), f32p]
    L.orc_generate_sampling.restype = C.c_int
    L.orc_generate_sampling.argtypes = [C.c_void_p, u32p, C.c_int, C.c_int, C.POINTER(OrcSampling), u32p, C.c_int, u32p, C.c_int, u64, u32p]
    L.orc_set_threads.argtypes = [C.c_int]
    L.orc_get_threads.restype = C.c_int
    _lib = L
    return L


def set_threads(n):
    lib().orc_set_threads(int(n))


# ── synthetic data ──────────────────────────────────────────────────────────────
def normal_f32(n, seed, stream, std=1.0):
    out = np.empty(int(n), dtype=np.float32)
    lib().orc_fill_normal_f32(_p(out, C.c_float), out.size, seed, stream, std)
    return out


def normal_bf16(n, seed, stream, std=1.0):
    out = np.empty(int(n), dtype=np.uint16)
    lib().orc_fill_normal_bf16(_p(out, C.c_uint16), out.size, seed, stream, std)
    return out


def uniform_u32(n, seed, stream, modulo):
    out = np.empty(int(n), dtype=np.uint32)
    lib().orc_fill_uniform_u32(_p(out, C.c_uint32), out.size, seed, stream, modulo)
    return out


def pseudo_randn(n, seed):
    out = np.empty(int(n), dtype=np.float32)
    lib().orc_pseudo_randn(_p(out, C.c_float), out.size, seed)
    return out


def bf16_to_f32(u16):
    return (np.asarray(u16, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_rne(f):
    u = np.ascontiguousarray(f, dtype=np.float32).view(np.uint32).astype(np.uint64)
    u = u + 0x7FFF + ((u >> 16) & 1)
    return (u >> 16).astype(np.uint16)


# ── quant formats ───────────────────────────────────────────────────────────────
def int8_quantize(w):
    w = np.ascontiguousarray(w, dtype=np.float32)
    rows, cols = w.shape
    data = np.empty((rows, cols), dtype=np.int8)
    scales = np.empty(rows, dtype=np.float32)
    lib().orc_int8_quantize(_p(w, C.c_float), rows, cols, _p(data, C.c_int8), _p(scales, C.c_float))
    return data, scales


def int8_dequantize(data, scales):
    rows, cols = data.shape
    out = np.empty((rows, cols), dtype=np.float32)
    lib().orc_int8_dequantize(_p(data, C.c_int8), _p(scales, C.c_float), rows, cols, _p(out, C.c_float))
    return out


def int4_quantize(w, block):
    w = np.ascontiguousarray(w, dtype=np.float32)
    n = w.size
    data = np.zeros((n + 1) // 2, dtype=np.uint8)
    scales = np.empty((n + block - 1) // block, dtype=np.float32)
    lib().orc_int4_quantize(_p(w, C.c_float), n, block, _p(data, C.c_uint8), _p(scales, C.c_float))
    return data, scales


def int4_dequantize(data, scales, n, block):
    out = np.empty(int(n), dtype=np.float32)
    lib().orc_int4_dequantize(_p(data, C.c_uint8), _p(scales, C.c_float), n, block, _p(out, C.c_float))
    return out


# ── ops ─────────────────────────────────────────────────────────────────────────
def rmsnorm(x, w, eps):
    x = np.array(x, dtype=np.float32)
    w = np.ascontiguousarray(w, dtype=np.float32)
    lib().orc_rmsnorm_inplace(_p(x, C.c_float), _p(w, C.c_float), x.size, eps)
    return x


def silu(x):
    return float(lib().orc_silu(float(x)))


def softmax(x):
    x = np.array(x, dtype=np.float32)
    lib().orc_softmax_inplace(_p(x, C.c_float), x.size)
    return x


def argmax(x):
    x = np.ascontiguousarray(x, dtype=np.float32)
    return int(lib().orc_argmax(_p(x, C.c_float), x.size))


def rope_tables(head_dim, max_seq, theta, yarn=None):
    half = head_dim // 2
    cos = np.empty((max_seq, half), dtype=np.float32)
    sin = np.empty((max_seq, half), dtype=np.float32)
    if yarn is None:
        lib().orc_rope_tables(head_dim, max_seq, theta, 0, 1.0, 0, 1.0, 1.0, _p(cos, C.c_float), _p(sin, C.c_float))
    else:
        lib().orc_rope_tables(head_dim, max_seq, theta, 1, yarn["factor"], yarn["orig_max_pos"],
                              yarn["beta_fast"], yarn["beta_slow"], _p(cos, C.c_float), _p(sin, C.c_float))
    return cos, sin


def rope_apply(x, head_dim, cos_row, sin_row):
    x = np.array(x, dtype=np.float32)
    c = np.ascontiguousarray(cos_row, dtype=np.float32)
    s = np.ascontiguousarray(sin_row, dtype=np.float32)
    lib().orc_rope_apply(_p(x, C.c_float), head_dim, _p(c, C.c_float), _p(s, C.c_float))
    return x


def linear(W, x):
    """y = W·x with W f32 [out×in] or bf16 bits (uint16)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    out_dim, in_dim = W.shape
    y = np.empty(out_dim, dtype=np.float32)
    W = np.ascontiguousarray(W)
    if W.dtype == np.uint16:
        lib().orc_linear_bf16(_p(W, C.c_uint16), _p(x, C.c_float), _p(y, C.c_float), out_dim, in_dim)
    else:
        lib().orc_linear_f32(_p(W, C.c_float), _p(x, C.c_float), _p(y, C.c_float), out_dim, in_dim)
    return y


def gemm(W, X):
    """Y[out×n] = W[out×in]·X[in×n]."""
    X = np.ascontiguousarray(X, dtype=np.float32)
    out_dim, in_dim = W.shape
    n = X.shape[1]
    Y = np.empty((out_dim, n), dtype=np.float32)
    W = np.ascontiguousarray(W)
    if W.dtype == np.uint16:
        lib().orc_gemm_bf16(_p(W, C.c_uint16), _p(X, C.c_float), _p(Y, C.c_float), out_dim, n, in_dim)
    else:
        lib().orc_gemm_f32(_p(W, C.c_float), _p(X, C.c_float), _p(Y, C.c_float), out_dim, n, in_dim)
    return Y


def decode_attention(q, kc, vc, n_heads, n_kv, hd, pos, scale, window):
    q = np.ascontiguousarray(q, dtype=np.float32)
    kc = np.ascontiguousarray(kc, dtype=np.float32)
    vc = np.ascontiguousarray(vc, dtype=np.float32)
    out = np.empty(n_heads * hd, dtype=np.float32)
    lib().orc_decode_attention(_p(q, C.c_float), _p(kc, C.c_float), _p(vc, C.c_float), _p(out, C.c_float),
                               n_heads, n_kv, hd, pos, scale, window)
    return out


# ── sampling primitives (each returns a new array) ────────────────────────────────
class Rng:
    """Rng::from_seed + next_f32 (:1205-1215)."""

    def __init__(self, seed):
        self.state = C.c_uint64(lib().orc_rng_from_seed(int(seed)))

    def next_f32(self):
        return float(lib().orc_rng_next_f32(C.byref(self.state)))


def _u32(a):
    return np.ascontiguousarray(a, dtype=np.uint32)


def _apply(fn, logits, *args):
    l = np.array(logits, dtype=np.float32)
    fn(_p(l, C.c_float), l.size, *args)
    return l


def apply_repetition_penalty(logits, toks, theta):
    t = _u32(toks); return _apply(lib().orc_apply_repetition_penalty, logits, _p(t, C.c_uint32), t.size, theta)


def apply_frequency_penalty(logits, history, penalty):
    t = _u32(history); return _apply(lib().orc_apply_frequency_penalty, logits, _p(t, C.c_uint32), t.size, penalty)


def apply_presence_penalty(logits, history, penalty):
    t = _u32(history); return _apply(lib().orc_apply_presence_penalty, logits, _p(t, C.c_uint32), t.size, penalty)


def apply_top_k(logits, k):
    return _apply(lib().orc_apply_top_k, logits, int(k))


def apply_top_p(logits, p):
    return _apply(lib().orc_apply_top_p, logits, p)


def apply_min_p(logits, min_p):
    return _apply(lib().orc_apply_min_p, logits, min_p)


def sample_from_probs(probs, r):
    pr = np.ascontiguousarray(probs, dtype=np.float32)
    return int(lib().orc_sample_from_probs(_p(pr, C.c_float), pr.size, r))


def sample_token(last_logits, cfg, step, history, rng, suppress=(), want_probs=False):
    """One selection of generate_with_sampling (:1625-1710); rng is an orc.Rng (advanced by one draw)."""
    l = np.ascontiguousarray(last_logits, dtype=np.float32)
    sup, hist = _u32(suppress), _u32(history)
    probs = np.zeros(l.size, np.float32) if want_probs else None
    tok = int(lib().orc_sample_token(_p(l, C.c_float), l.size, C.byref(cfg), int(step), _p(sup, C.c_uint32), sup.size,
                                     _p(hist, C.c_uint32), hist.size, C.byref(rng.state),
                                     _p(probs, C.c_float) if probs is not None else None))
    return (tok, probs) if want_probs else tok


# ── model ───────────────────────────────────────────────────────────────────────
class OracleModel:
    """CPU twin of OlmoModel (forward_one / greedy generate)."""

    def __init__(self, cfg: dict, layer_sliding=None):
        c = OrcConfig()
        for k, _ in OrcConfig._fields_:
            if k in cfg:
                setattr(c, k, cfg[k])
        if "eos_token_id" not in cfg or cfg["eos_token_id"] is None:
            c.eos_token_id = -1
        self.cfg = c
        ls = None
        if layer_sliding is not None:
            ls = (C.c_int * c.n_layers)(*[int(v) for v in layer_sliding])
        self._h = lib().orc_model_new(C.byref(c), ls)
        self._keep = []

    def __del__(self):
        if getattr(self, "_h", None):
            lib().orc_model_free(self._h)
            self._h = None

    def set_tensor(self, layer, which, arr):
        arr = np.ascontiguousarray(arr)
        assert arr.dtype in (np.float32, np.uint16)
        self._keep.append(arr)
        rc = lib().orc_model_set_tensor(self._h, layer, which, arr.ctypes.data, 1 if arr.dtype == np.uint16 else 0)
        assert rc == 0

    def init_reference_random(self):
        lib().orc_model_init_reference_random(self._h)

    def set_kv_round_bf16(self, on):
        lib().orc_model_set_kv_round_bf16(self._h, int(bool(on)))

    def reset(self):
        lib().orc_model_reset(self._h)

    @property
    def pos(self):
        return lib().orc_model_pos(self._h)

    def seed_context(self, pos, seed=0):
        """Measurement aid: cache rows [0,pos) filled with seeded N(0,1) values, position set to pos."""
        lib().orc_model_seed_context(self._h, int(pos), int(seed))

    def forward_one(self, token, want_hidden=False):
        logits = np.empty(self.cfg.vocab_size, dtype=np.float32)
        hid = None
        if want_hidden:
            hid = np.empty((self.cfg.n_layers, self.cfg.d_model), dtype=np.float32)
        lib().orc_forward_one(self._h, int(token), _p(logits, C.c_float),
                              _p(hid, C.c_float) if hid is not None else None)
        return (logits, hid) if want_hidden else logits

    def generate_greedy(self, prompt, max_new, suppress=(), rep_penalty=1.0, rep_window=64, stops=(),
                        want_logits=False):
        prompt = np.ascontiguousarray(prompt, dtype=np.uint32)
        sup = np.ascontiguousarray(suppress, dtype=np.uint32)
        stp = np.ascontiguousarray(stops, dtype=np.uint32)
        out = np.zeros(max(max_new, 1), dtype=np.uint32)
        trace = np.zeros((max(max_new, 1), self.cfg.vocab_size), dtype=np.float32) if want_logits else None
        margins = np.zeros(max(max_new, 1), dtype=np.float32)
        n = lib().orc_generate_greedy(self._h, _p(prompt, C.c_uint32), prompt.size, max_new,
                                      _p(sup, C.c_uint32), sup.size, rep_penalty, rep_window,
                                      _p(stp, C.c_uint32), stp.size, _p(out, C.c_uint32),
                                      _p(trace, C.c_float) if trace is not None else None,
                                      _p(margins, C.c_float))
        if want_logits:
            return out[:n].copy(), trace[:n], margins[:n]
        return out[:n].copy()

    def generate_sampling(self, prompt, max_new, cfg, seed, suppress=(), stops=()):
        """generate_with_sampling (:1599-1732) with Rng::from_seed(seed) in place of the system time."""
        prompt, sup, stp = _u32(prompt), _u32(suppress), _u32(stops)
        out = np.zeros(max(max_new, 1), dtype=np.uint32)
        n = lib().orc_generate_sampling(self._h, _p(prompt, C.c_uint32), prompt.size, max_new, C.byref(cfg),
                                        _p(sup, C.c_uint32), sup.size, _p(stp, C.c_uint32), stp.size, int(seed), _p(out, C.c_uint32))
        return out[:n].copy()
