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


class StepGuard:
    """Host-side failure detection for a tensor-parallel group (no counterpart in the reference).

    The fused all-reduce makes every decode step a rendezvous of all ranks: a rank that raised,
    exited or simply never reached the step would leave the others waiting in their mailbox
    polls until the device-side limit.  The guard moves that discovery to the host, before the
    launch: every rank counts its steps in a shared key-value store (anything with the
    `add(key, n) -> int` call of torch.distributed's stores) and, before it launches step s,
    checks that every peer has announced step s too.  A peer that does not show up within
    `deadline_s`, or that said goodbye with leave(), ends the step with AtlasError on the ranks
    that are still there — no kernel or collective is in flight at that point, so the GPU and
    the context stay usable.
    """

    def __init__(self, store, rank, world, deadline_s=5.0, prefix="atlasx/tp"):
        self.store, self.rank, self.world = store, int(rank), int(world)
        self.deadline_s, self.prefix = float(deadline_s), prefix
        self.step = 0

    def _key(self, what, r):
        return "%s/%s/%d" % (self.prefix, what, r)

    def arrive(self):
        """Announce that this rank is about to run its next step; returns the step number."""
        self.step = int(self.store.add(self._key("step", self.rank), 1))
        return self.step

    def leave(self):
        """Announce that this rank runs no more steps (call between steps, nothing in flight)."""
        self.store.add(self._key("left", self.rank), 1)

    def check(self, poll_s=0.002):
        """Block until every peer has announced this rank's current step.  Raises AtlasError naming
        the ranks that left or did not arrive before the deadline."""
        import time
        t_end = time.monotonic() + self.deadline_s
        while True:
            late, gone = [], []
            for r in range(self.world):
                if r == self.rank:
                    continue
                if int(self.store.add(self._key("step", r), 0)) >= self.step:
                    continue
                (gone if int(self.store.add(self._key("left", r), 0)) > 0 else late).append(r)
            if gone:
                raise _ffi.AtlasError("tensor-parallel rank(s) %s left the group before step %d" % (gone, self.step))
            if not late:
                return
            if time.monotonic() >= t_end:
                raise _ffi.AtlasError("tensor-parallel rank(s) %s did not reach step %d within %.1f s"
                                      % (late, self.step, self.deadline_s))
            time.sleep(poll_s)

    def step_barrier(self):
        """arrive() + check(): call right before launching a step."""
        self.arrive()
        self.check()
        return self.step
