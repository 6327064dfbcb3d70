"""Tensor-parallel partition of the decode path (no counterpart in the reference, which is
single-GPU).  One process per GPU; rank r of g keeps

  wq, wk, wv   rows of its heads           (column-parallel: no communication)
  wo           columns of its heads        (row-parallel: partial [d_model] → all-reduce)
  gate, up     rows r·ffn/g … (r+1)·ffn/g  (column-parallel)
  down         the matching columns        (row-parallel → all-reduce)
  lm_head      rows of a vocabulary padded to a multiple of g (all-gather of logits)
  q_norm/k_norm the slices of its heads; other norms, RoPE tables, embedding: replicated.

slice_of() states the same ranges the C++ loader applies (csrc/model.cu, set_tensor), so host
code and tests can shard reference tensors identically.
"""
from . import _ffi


def local_dims(cfg, world):
    hd = cfg.d_model // cfg.n_heads
    if cfg.n_heads % world or cfg.n_kv_heads % world or cfg.ffn_hidden % world:
        raise _ffi.AtlasError("heads, kv heads and ffn_hidden must divide by the tensor-parallel degree")
    return dict(head_dim=hd, q_rows=cfg.n_heads // world * hd, kv_rows=cfg.n_kv_heads // world * hd,
                ffn=cfg.ffn_hidden // world, vocab=(cfg.vocab_size + world - 1) // world)


def slice_of(cfg, which, rank, world):
    """(row_start, row_stop, col_start, col_stop) of the full tensor `which` kept by `rank`."""
    L = local_dims(cfg, world)
    d, hd = cfg.d_model, L["head_dim"]
    full = {_ffi.T_WQ: (cfg.n_heads * hd, d), _ffi.T_WK: (cfg.n_kv_heads * hd, d), _ffi.T_WV: (cfg.n_kv_heads * hd, d),
            _ffi.T_WO: (d, cfg.n_heads * hd), _ffi.T_GATE: (cfg.ffn_hidden, d), _ffi.T_UP: (cfg.ffn_hidden, d),
            _ffi.T_DOWN: (d, cfg.ffn_hidden), _ffi.T_LM_HEAD: (cfg.vocab_size, d), _ffi.T_EMBED: (cfg.vocab_size, d)}
    if which == _ffi.T_WQ:
        return rank * L["q_rows"], (rank + 1) * L["q_rows"], 0, d
    if which in (_ffi.T_WK, _ffi.T_WV):
        return rank * L["kv_rows"], (rank + 1) * L["kv_rows"], 0, d
    if which == _ffi.T_WO:
        return 0, d, rank * L["q_rows"], (rank + 1) * L["q_rows"]
    if which in (_ffi.T_GATE, _ffi.T_UP):
        return rank * L["ffn"], (rank + 1) * L["ffn"], 0, d
    if which == _ffi.T_DOWN:
        return 0, d, rank * L["ffn"], (rank + 1) * L["ffn"]
    if which == _ffi.T_LM_HEAD:
        return min(rank * L["vocab"], cfg.vocab_size), min((rank + 1) * L["vocab"], cfg.vocab_size), 0, d
    if which == _ffi.T_Q_NORM:
        return 0, 1, rank * L["q_rows"], (rank + 1) * L["q_rows"]
    if which == _ffi.T_K_NORM:
        return 0, 1, rank * L["kv_rows"], (rank + 1) * L["kv_rows"]
    r, c = full.get(which, (1, d))
    return 0, r, 0, c            # replicated


def init_comm(ctx, rank, world, broadcast_bytes):
    """Create the NCCL communicator of a context.  broadcast_bytes(buf: bytes|None) -> bytes must
    return rank 0's buffer on every rank (e.g. through torch.distributed or any other store)."""
    import ctypes as C
    ident = (C.c_ubyte * 128)()
    if rank == 0:
        _ffi.check(_ffi.lib().atlasx_comm_unique_id(ident))
    data = broadcast_bytes(bytes(ident) if rank == 0 else None)
    ident = (C.c_ubyte * 128)(*data)
    _ffi.check(_ffi.lib().atlasx_comm_init(ctx.handle, ident, rank, world))
