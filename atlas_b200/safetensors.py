"""Host-side mirror of SafetensorsFile and the two model loaders of the reference's atlas-model
crate (crates/atlas-model/src/lib.rs: SafetensorsFile :2046-2240, load_model_from_safetensors
:2283-2360, load_model_from_dir :2437-2570) over the library's mapped-file reader: a BF16 tensor
reaches the device as the bytes it is stored as, each tensor-parallel rank reads only its part,
nothing is kept in host memory.
"""
import ctypes as C
import os
from dataclasses import dataclass
from typing import List, Sequence, Tuple

import numpy as np

from . import _ffi
from ._ffi import AUTO, AtlasError, BF16, F16, F32, LoadStatsC, check
from .model import LAYER_SLIDING, ModelConfig, OlmoModel
from .tensor import Context

_DTYPE_NAMES = {F32: "F32", BF16: "BF16", F16: "F16", -1: "?"}


@dataclass
class TensorDesc:
    """TensorDesc, :2052-2057 (offsets are not exposed: reads go through the mapping)."""
    name: str
    dtype: str
    shape: Tuple[int, ...]
    nbytes: int


class SafetensorsFile:
    def __init__(self, handle):
        self._h = handle

    @classmethod
    def open(cls, path):
        """:2071-2078 — the file is mapped; only the header is parsed."""
        h = C.c_void_p()
        check(_ffi.lib().atlasx_safetensors_open(os.fsencode(path), C.byref(h)))
        return cls(h)

    def close(self):
        if self._h:
            _ffi.lib().atlasx_safetensors_close(self._h)
            self._h = None

    __del__ = close

    def __len__(self):
        return _ffi.lib().atlasx_safetensors_count(self._h)

    def is_empty(self):
        return len(self) == 0

    def _desc(self, i):
        name, dt, nd, nb = C.c_char_p(), C.c_int(), C.c_int(), C.c_size_t()
        dims = (C.c_size_t * 4)()
        check(_ffi.lib().atlasx_safetensors_tensor(self._h, i, C.byref(name), C.byref(dt), C.byref(nd), dims, C.byref(nb)))
        return TensorDesc(name.value.decode(), _DTYPE_NAMES.get(dt.value, "?"), tuple(dims[k] for k in range(min(nd.value, 4))), nb.value)

    @property
    def tensors(self) -> List[TensorDesc]:
        return [self._desc(i) for i in range(len(self))]

    def tensor_names(self):
        return [t.name for t in self.tensors]

    def contains(self, name):
        return _ffi.lib().atlasx_safetensors_find(self._h, name.encode()) >= 0

    def get_desc(self, name):
        i = _ffi.lib().atlasx_safetensors_find(self._h, name.encode())
        return self._desc(i) if i >= 0 else None

    def _read(self, name, out_dtype, rows=None, cols=None):
        i = _ffi.lib().atlasx_safetensors_find(self._h, name.encode())
        if i < 0:
            raise AtlasError("tensor '%s' not found" % name)
        d = self._desc(i)
        esz = 4 if d.dtype == "F32" else 2
        n = d.nbytes // esz
        full_c = d.shape[-1] if d.shape else n
        full_r = n // full_c if full_c else 0
        r0, r1 = rows if rows is not None else (0, full_r)
        c0, c1 = cols if cols is not None else (0, full_c)
        out = np.empty((r1 - r0, c1 - c0), np.float32 if out_dtype == F32 else np.uint16)
        check(_ffi.lib().atlasx_safetensors_read(self._h, i, r0, r1, c0, c1, out_dtype, out.ctypes.data))
        return out

    def get_f32(self, name, rows=None, cols=None):
        """:2205-2240 — F32 as stored, BF16 and F16 converted; optional (start, stop) row / column ranges."""
        a = self._read(name, F32, rows, cols)
        return a if (rows or cols) else a.reshape(-1)

    def get_bf16(self, name, rows=None, cols=None):
        """:2187-2202 — raw bf16 bit patterns; fails for tensors of another dtype."""
        a = self._read(name, BF16, rows, cols)
        return a if (rows or cols) else a.reshape(-1)

    @staticmethod
    def build(path, tensors: Sequence[Tuple[str, Sequence[int], np.ndarray]]):
        """Write (name, shape, values) tensors: float32 arrays as F32, uint16 arrays as BF16 bit
        patterns.  Same header text as build_f32 (:2154-2185): keys in the order given, no spaces."""
        n = len(tensors)
        keep = []
        names = (C.c_char_p * n)(); dtypes = (C.c_int * n)(); nd = (C.c_int * n)()
        dims = (C.c_size_t * (4 * n))(*([1] * (4 * n))); data = (C.c_void_p * n)()
        for i, (name, shape, values) in enumerate(tensors):
            a = np.ascontiguousarray(values)
            if a.dtype != np.uint16:
                a = np.ascontiguousarray(a, dtype=np.float32)
            if int(np.prod(shape, dtype=np.int64)) != a.size or len(shape) > 4:
                raise AtlasError("shape %s does not match %d values" % (tuple(shape), a.size))
            keep.append(a)
            names[i] = name.encode(); dtypes[i] = BF16 if a.dtype == np.uint16 else F32; nd[i] = len(shape)
            for k, e in enumerate(shape):
                dims[4 * i + k] = int(e)
            data[i] = a.ctypes.data
        check(_ffi.lib().atlasx_safetensors_write(os.fsencode(path), n, names, dtypes, nd, dims, data))

    @staticmethod
    def build_f32(path, tensors):
        """:2154-2185, written to `path`."""
        SafetensorsFile.build(path, [(n, s, np.asarray(v, np.float32)) for n, s, v in tensors])


@dataclass
class LoadStats:
    seconds: float
    file_bytes_read: int
    bytes_uploaded: int
    peak_host_rss_bytes: int
    n_tensors_used: int
    post_norm: bool
    tied_lm_head: bool
    weight_format: int


def _adopt(cfg, ctx, handle, stats, kv_dtype, int4_block, tp):
    m = OlmoModel(cfg, ctx=ctx, kv_dtype=kv_dtype, weight_format=stats.weight_format, int4_block=int4_block,
                  tp_rank=tp[0], tp_world=tp[1])
    m._h = handle
    m.load_stats = LoadStats(stats.seconds, stats.file_bytes_read, stats.bytes_uploaded, stats.peak_host_rss_bytes,
                             stats.n_tensors_used, bool(stats.post_norm), bool(stats.tied_lm_head), stats.weight_format)
    cfg.post_norm = bool(stats.post_norm)
    return m


def load_model_from_safetensors(path, cfg: ModelConfig, ctx=None, kv_dtype=BF16, weight_format=AUTO, int4_block=32,
                                tp_rank=0, tp_world=1) -> OlmoModel:
    """:2283-2360.  `path` may also be a list of files (later files win for a repeated name).
    Returns a finalised model; model.load_stats reports time, bytes and peak host memory."""
    ctx = ctx or Context.default()
    paths = [path] if isinstance(path, (str, bytes, os.PathLike)) else list(path)
    arr = (C.c_char_p * len(paths))(*[os.fsencode(p) for p in paths])
    c, sliding = OlmoModel.config_struct(cfg, kv_dtype, weight_format, int4_block, tp_rank, tp_world)
    h, st = C.c_void_p(), LoadStatsC()
    check(_ffi.lib().atlasx_model_load_safetensors(ctx.handle, arr, len(paths), C.byref(c), sliding, C.byref(h), C.byref(st)))
    return _adopt(cfg, ctx, h, st, kv_dtype, int4_block, (tp_rank, tp_world))


def load_model_from_dir(directory, cfg: ModelConfig, ctx=None, kv_dtype=BF16, weight_format=AUTO, int4_block=32,
                        tp_rank=0, tp_world=1) -> OlmoModel:
    """:2437-2570 — config.json overlay (layer_types, sliding_window, rope_scaling, rope_theta,
    rms_norm_eps, eos_token_id), then the shards of model.safetensors.index.json or model.safetensors.
    The overlay is applied to `cfg` as well, so the caller sees the configuration in effect."""
    ctx = ctx or Context.default()
    cj = os.path.join(directory, "config.json")
    if os.path.exists(cj):
        patch_config_from_hf_json(cfg, cj)
    c, sliding = OlmoModel.config_struct(cfg, kv_dtype, weight_format, int4_block, tp_rank, tp_world)
    h, st = C.c_void_p(), LoadStatsC()
    check(_ffi.lib().atlasx_model_load_dir(ctx.handle, os.fsencode(directory), C.byref(c), sliding, C.byref(h), C.byref(st)))
    m = _adopt(cfg, ctx, h, st, kv_dtype, int4_block, (tp_rank, tp_world))
    m.eos_token_id = cfg.eos_token_id
    return m


def patch_config_from_hf_json(cfg: ModelConfig, config_path) -> ModelConfig:
    """:2367-2432, in place (and returned)."""
    from .model import Yarn
    c, _ = OlmoModel.config_struct(cfg, BF16, F32, 32, 0, 1)
    sliding = (C.c_int * max(cfg.n_layers, 1))()
    n_lt = C.c_int(0)
    check(_ffi.lib().atlasx_config_patch_from_json(os.fsencode(config_path), C.byref(c), sliding, C.byref(n_lt)))
    if n_lt.value > 0:
        cfg.layer_types = [LAYER_SLIDING if sliding[i] else 0 for i in range(min(n_lt.value, cfg.n_layers))]
    cfg.sliding_window = c.sliding_window or None
    if c.rope_scaling == 1:
        cfg.rope_scaling = Yarn(c.yarn_factor, c.yarn_orig_max_pos, c.yarn_attn_factor, c.yarn_beta_fast, c.yarn_beta_slow)
    cfg.rope_theta, cfg.rms_norm_eps = c.rope_theta, c.rms_norm_eps
    cfg.eos_token_id = c.eos_token_id if c.eos_token_id >= 0 else None
    return cfg
