"""Host-side mirror of the decode surface of the reference's atlas-model crate
(crates/atlas-model/src/lib.rs): ModelConfig :58-329, SamplingConfig :1223-1295 and
OlmoModel {new, init_gpu_resources, reset, forward_one_gpu, generate, generate_with_sampling}
:1298-1732 — over the fused sm_100a decode step, greedy or with the sampling pipeline on the
device; there is no CPU fallback.
"""
import ctypes as C
from dataclasses import dataclass, field
from typing import List, Optional

import numpy as np

from . import _ffi
from ._ffi import AtlasError, BF16, F32, INT4, INT8, ModelConfigC, check
from .tensor import Context

LAYER_FULL, LAYER_SLIDING = 0, 1


@dataclass
class Yarn:
    """RopeScaling::Yarn, :40-53."""
    factor: float = 8.0
    orig_max_pos: int = 8192
    attn_factor: float = 1.0
    beta_fast: float = 32.0
    beta_slow: float = 1.0


@dataclass
class ModelConfig:
    vocab_size: int
    d_model: int
    n_layers: int
    n_heads: int
    n_kv_heads: int
    ffn_hidden: int
    max_seq_len: int
    rope_theta: float = 10000.0
    rms_norm_eps: float = 1e-5
    layer_types: List[int] = field(default_factory=list)     # empty = all full
    sliding_window: Optional[int] = None
    rope_scaling: Optional[Yarn] = None
    eos_token_id: Optional[int] = None
    # set by the loader in the reference (private fields there): OLMo-2/3 post-norm
    post_norm: bool = False

    def head_dim(self):
        return self.d_model // self.n_heads

    def kv_dim(self):
        return self.n_kv_heads * self.head_dim()

    @classmethod
    def tiny(cls):
        """:312-328"""
        return cls(256, 64, 2, 4, 2, 128, 128, 10000.0, 1e-5)

    @classmethod
    def olmo3_actual_7b(cls, max_seq_len=4096):
        """:253-269 plus what load_model_from_dir reads from config.json (:2367-2432, test :3534-3575):
        three sliding layers then one full, window 4096, YaRN factor 8."""
        return cls(100278, 4096, 32, 32, 32, 11008, max_seq_len, 500000.0, 1e-6,
                   layer_types=[LAYER_FULL if i % 4 == 3 else LAYER_SLIDING for i in range(32)],
                   sliding_window=4096,
                   rope_scaling=Yarn(8.0, 8192, 1.2079441541679836, 32.0, 1.0), post_norm=True)


@dataclass
class SamplingConfig:
    """:1223-1248"""
    temperature: float = 1.0
    repetition_penalty: float = 1.0
    repetition_window: int = 64
    frequency_penalty: float = 0.0
    presence_penalty: float = 0.0
    top_p: float = 1.0
    top_k: int = 0
    min_p: float = 0.0
    suppress_initial_tokens: List[int] = field(default_factory=list)

    @classmethod
    def olmo3(cls):
        """:1278-1294"""
        return cls(temperature=0.6, repetition_penalty=1.15, repetition_window=256, frequency_penalty=0.0,
                   presence_penalty=0.0, top_p=0.95, top_k=50, min_p=0.05, suppress_initial_tokens=[14023])


def sampling_struct(config: SamplingConfig):
    return _ffi.SamplingConfigC(config.temperature, config.repetition_penalty, config.repetition_window, config.frequency_penalty,
                                config.presence_penalty, config.top_p, config.top_k, config.min_p)


def sample_token(logits_dev, n, config: SamplingConfig, step, history, rng_state, ctx=None, probs_dev=None):
    """One selection of the sampling pipeline from `n` logits on the device (atlasx_sample_token).
    Returns (token, new rng state)."""
    ctx = ctx or Context.default()
    sup = np.ascontiguousarray(config.suppress_initial_tokens, dtype=np.uint32)
    hist = np.ascontiguousarray(history, dtype=np.uint32)
    st, tok = C.c_uint64(int(rng_state)), C.c_int(-1)
    check(_ffi.lib().atlasx_sample_token(ctx.handle, C.c_void_p(int(logits_dev)), int(n), C.byref(sampling_struct(config)), int(step),
                                         sup.ctypes.data, sup.size, hist.ctypes.data, hist.size, C.byref(st), C.byref(tok),
                                         C.c_void_p(int(probs_dev)) if probs_dev else None))
    return tok.value, st.value


class OlmoModel:
    """The GPU side of OlmoModel.  Weights are given tensor by tensor (set_tensor), then
    init_gpu_resources() builds RoPE tables, KV caches and the step graph."""

    def __init__(self, cfg: ModelConfig, ctx=None, kv_dtype=BF16, weight_format=None, int4_block=32,
                 tp_rank=0, tp_world=1):
        self.config = cfg
        self.ctx = ctx or Context.default()
        self.eos_token_id = cfg.eos_token_id
        self.extra_stop_tokens: List[int] = []
        self._weight_format = weight_format
        self._pending = []
        self._h = None
        self._kv_dtype, self._int4_block, self._tp = kv_dtype, int4_block, (tp_rank, tp_world)

    @staticmethod
    def config_struct(cfg, kv_dtype, weight_format, int4_block, tp_rank, tp_world):
        """(atlasx_model_config, layer_sliding array or None) for a ModelConfig."""
        c = ModelConfigC()
        c.vocab_size, c.d_model, c.n_layers = cfg.vocab_size, cfg.d_model, cfg.n_layers
        c.n_heads, c.n_kv_heads, c.ffn_hidden, c.max_seq_len = cfg.n_heads, cfg.n_kv_heads, cfg.ffn_hidden, cfg.max_seq_len
        c.rope_theta, c.rms_norm_eps = cfg.rope_theta, cfg.rms_norm_eps
        c.sliding_window = cfg.sliding_window or 0
        if cfg.rope_scaling is not None:
            y = cfg.rope_scaling
            c.rope_scaling, c.yarn_factor, c.yarn_orig_max_pos = 1, y.factor, y.orig_max_pos
            c.yarn_attn_factor, c.yarn_beta_fast, c.yarn_beta_slow = y.attn_factor, y.beta_fast, y.beta_slow
        c.post_norm = int(cfg.post_norm)
        c.eos_token_id = -1          # EOS is passed with the stop tokens at generate() time (it is a pub field there)
        c.kv_dtype, c.weight_format, c.int4_block = kv_dtype, weight_format, int4_block
        c.tp_rank, c.tp_world = tp_rank, tp_world
        sliding = None
        if cfg.layer_types:
            assert len(cfg.layer_types) == cfg.n_layers
            sliding = (C.c_int * cfg.n_layers)(*[int(t == LAYER_SLIDING) for t in cfg.layer_types])
        return c, sliding

    def _create(self, weight_format):
        cfg = self.config
        c, sliding = self.config_struct(cfg, self._kv_dtype, weight_format, self._int4_block, *self._tp)
        h = C.c_void_p()
        check(_ffi.lib().atlasx_model_create(self.ctx.handle, C.byref(c), sliding, C.byref(h)))
        self._h = h
        self._cfg_c = c

    def set_tensor(self, layer, which, data, on_device=False, dtype=None):
        """data: numpy f32 / uint16 (bf16 bits) FULL tensor, or a device pointer with dtype given.
        The storage format of the linear weights follows the first weight given (bf16 → W16A32,
        f32 → f32) unless weight_format was passed to the constructor."""
        if on_device:
            ptr, dt = int(data), dtype
        else:
            a = np.ascontiguousarray(data)
            if a.dtype == np.uint16:
                dt = BF16
            else:
                a = np.ascontiguousarray(a, dtype=np.float32); dt = F32
            ptr = a.ctypes.data
        if self._h is None:
            fmt = self._weight_format
            if fmt is None:
                fmt = dt
            self._create(fmt)
        check(_ffi.lib().atlasx_model_set_tensor(self._h, int(layer), int(which), C.c_void_p(ptr), dt, int(bool(on_device))))

    def init_gpu_resources(self, use_graph=True, use_pdl=True):
        """:1360-1386"""
        if self._h is None:
            raise AtlasError("no tensors were given")
        check(_ffi.lib().atlasx_model_set_options(self._h, int(use_graph), int(use_pdl)))
        check(_ffi.lib().atlasx_model_finalize(self._h))

    def time_classes(self, names, iters=32):
        """Device time per pass (ms), algorithmic bytes and launch count of the named launch classes
        replayed back to back as one graph (see atlasx_model_time_classes)."""
        L = _ffi.lib()
        mask = 0
        for i in range(32):
            nm = L.atlasx_model_class_name(i)
            if nm and nm.decode() in names:
                mask |= 1 << i
        ms, by, n = C.c_float(0), C.c_double(0), C.c_int(0)
        check(L.atlasx_model_time_classes(self._h, mask, int(iters), C.byref(ms), C.byref(by), C.byref(n)))
        return ms.value, by.value, n.value

    def set_prefill(self, chunk=16):
        """Prompt ingestion `chunk` tokens at a time (the reference's generate feeds one token per
        forward, :1611-1618).  Returns the chunk size in effect (1 = token by token)."""
        eff = C.c_int(0)
        check(_ffi.lib().atlasx_model_set_prefill(self._h, int(chunk), C.byref(eff)))
        return eff.value

    def set_options(self, use_graph=True, use_pdl=True):
        check(_ffi.lib().atlasx_model_set_options(self._h, int(use_graph), int(use_pdl)))

    def reset(self):
        """:1389-1392"""
        check(_ffi.lib().atlasx_model_reset(self._h))

    @property
    def pos(self):
        return _ffi.lib().atlasx_model_pos(self._h)

    def forward_one_gpu(self, token, want_logits=True):
        """:1463-1505 — returns logits [vocab_size] (host), or None when want_logits is False."""
        logits = np.empty(self.config.vocab_size, np.float32) if want_logits else None
        check(_ffi.lib().atlasx_model_forward_one(self._h, int(token), logits.ctypes.data if want_logits else None))
        return logits

    forward_one = forward_one_gpu

    def hidden(self, layer=None):
        """Residual stream after the last layer (or after `layer`) of the last forward."""
        out = np.empty(self.config.d_model, np.float32)
        if layer is None:
            check(_ffi.lib().atlasx_model_hidden(self._h, out.ctypes.data))
        else:
            check(_ffi.lib().atlasx_model_layer_hidden(self._h, int(layer), out.ctypes.data))
        return out

    def set_layer_hook(self, fn):
        """fn(layer_idx, hidden: float32 array) -> Optional[float], called for every layer of every
        forward (forward_one_gpu_hooked, :1524-1557; generate_with_sampling_hooked, :1745-1846).
        None detaches.  Returns the native callback object (kept alive by the model as well)."""
        if fn is None:
            check(_ffi.lib().atlasx_model_set_layer_hook(self._h, None, None))
            self._hook_cb = None
            return None
        d = self.config.d_model

        def trampoline(_user, layer, hidden, d_model, delta_out):
            r = fn(int(layer), np.ctypeslib.as_array(hidden, shape=(d_model,)))
            if r is None:
                return 0
            delta_out[0] = float(r)
            return 1
        cb = _ffi.LAYER_HOOK(trampoline)
        check(_ffi.lib().atlasx_model_set_layer_hook(self._h, C.cast(cb, C.c_void_p), None))
        self._hook_cb = cb
        return cb

    def deposits(self):
        """(token_id, total_delta, layers_fired) per token generated by the last generate call with a hook."""
        n = C.c_int(0)
        check(_ffi.lib().atlasx_model_deposits(self._h, None, None, None, 0, C.byref(n)))
        k = n.value
        tok, delta, fired = np.zeros(k, np.uint32), np.zeros(k, np.float32), np.zeros(k, np.uint32)
        if k:
            check(_ffi.lib().atlasx_model_deposits(self._h, tok.ctypes.data, delta.ctypes.data, fired.ctypes.data, k, C.byref(n)))
        return [(int(t), float(x), int(f)) for t, x, f in zip(tok, delta, fired)]

    def generate_streaming(self, prompt, max_new, config: "SamplingConfig", on_token, seed=None):
        """:1855-1965 — as generate_with_sampling, with on_token(token) called for every token right after
        it is emitted; a false return ends the generation there (no forward runs for that token)."""
        def trampoline(_user, tok):
            return 1 if on_token(int(tok)) else 0
        cb = _ffi.TOKEN_CALLBACK(trampoline)
        check(_ffi.lib().atlasx_model_set_token_callback(self._h, C.cast(cb, C.c_void_p), None))
        try:
            return self.generate_with_sampling(prompt, max_new, config, seed=seed)
        finally:
            check(_ffi.lib().atlasx_model_set_token_callback(self._h, None, None))

    def generate(self, prompt, max_new, temperature=0.0):
        """:1584-1590"""
        return self.generate_with_sampling(prompt, max_new, SamplingConfig(temperature=temperature))

    def generate_with_sampling(self, prompt, max_new, config: SamplingConfig, seed=None):
        """:1599-1732.  temperature ≤ 0: the greedy branch.  Otherwise the sampling pipeline runs on the
        device between steps (only the 4-byte token id is read back per step); the XorShift64 generator is
        seeded from the clock as the reference does, or from `seed` (Rng::from_seed) for repeatable runs."""
        if not (config.temperature <= 0.0 or config.temperature < 1e-6):
            return self._generate_sampling(prompt, max_new, config, seed)
        p = np.ascontiguousarray(prompt, dtype=np.uint32)
        sup = np.ascontiguousarray(config.suppress_initial_tokens, dtype=np.uint32)
        stop_list = list(self.extra_stop_tokens) + ([int(self.eos_token_id)] if self.eos_token_id is not None else [])
        stops = np.ascontiguousarray(stop_list, dtype=np.uint32)
        out = np.zeros(max(max_new, 1), np.uint32)
        n = C.c_int(0)
        check(_ffi.lib().atlasx_model_generate_greedy(
            self._h, p.ctypes.data, p.size, int(max_new), sup.ctypes.data, sup.size,
            float(config.repetition_penalty), int(config.repetition_window),
            stops.ctypes.data, stops.size, out.ctypes.data, C.byref(n)))
        return out[:n.value].tolist()

    def _generate_sampling(self, prompt, max_new, config, seed):
        p = np.ascontiguousarray(prompt, dtype=np.uint32)
        sup = np.ascontiguousarray(config.suppress_initial_tokens, dtype=np.uint32)
        stop_list = list(self.extra_stop_tokens) + ([int(self.eos_token_id)] if self.eos_token_id is not None else [])
        stops = np.ascontiguousarray(stop_list, dtype=np.uint32)
        out = np.zeros(max(max_new, 1), np.uint32)
        n = C.c_int(0)
        check(_ffi.lib().atlasx_model_generate_sampling(
            self._h, p.ctypes.data, p.size, int(max_new), C.byref(sampling_struct(config)), sup.ctypes.data, sup.size,
            stops.ctypes.data, stops.size, int(seed or 0), int(seed is None), out.ctypes.data, C.byref(n)))
        return out[:n.value].tolist()

    # measurement helpers -----------------------------------------------------------------
    def decode_timed(self, steps, lead=0):
        """Device time (ms) of `steps` greedy steps and their tokens; `lead` untimed steps run first."""
        ms = C.c_float(0)
        toks = np.zeros(lead + steps, np.uint32)
        check(_ffi.lib().atlasx_model_decode_timed(self._h, int(steps), int(lead), C.byref(ms), toks.ctypes.data))
        return ms.value, toks[lead:]

    def profile_step(self):
        n = 16
        launches = (C.c_int * n)(); ms = (C.c_float * n)(); by = (C.c_double * n)(); k = C.c_int(0)
        check(_ffi.lib().atlasx_model_profile_step(self._h, n, launches, ms, by, C.byref(k)))
        return {_ffi.lib().atlasx_model_class_name(i).decode(): dict(launches=launches[i], ms=ms[i], bytes=by[i])
                for i in range(k.value)}

    def step_bytes(self, pos):
        return float(_ffi.lib().atlasx_model_step_bytes(self._h, int(pos)))

    @property
    def launches_per_step(self):
        return _ffi.lib().atlasx_model_kernel_launches_per_step(self._h)

    def __del__(self):
        try:
            if self._h and self.ctx.handle:
                _ffi.lib().atlasx_model_free(self._h)
        except Exception:
            pass
        self._h = None
