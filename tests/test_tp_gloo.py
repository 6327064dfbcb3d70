"""CPU, world_size 2 over gloo: the tensor-parallel partition (atlas_b200/tp.py, mirrored by the
C++ loader) reproduces the unsharded oracle when each rank computes on its slices and the
row-parallel partial sums are all-reduced — the data flow of bench.py --gpus N."""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close(); return p


def _worker(rank, world, port, out):
    sys.path.insert(0, ROOT); sys.path.insert(0, os.path.join(ROOT, "tests"))
    import torch
    import torch.distributed as dist
    from oracle import orc
    import helpers
    import atlas_b200 as ab
    from atlas_b200 import tp, _ffi
    os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    cfg = dict(helpers.SMALL_SWA, vocab_size=1001)          # odd vocabulary: padded shard
    mc = ab.ModelConfig(cfg["vocab_size"], cfg["d_model"], cfg["n_layers"], cfg["n_heads"], cfg["n_kv_heads"],
                        cfg["ffn_hidden"], cfg["max_seq_len"])
    w = helpers.synth_weights(cfg, seed=13, norm_jitter=0.1)
    L = tp.local_dims(mc, world)
    hd, d = L["head_dim"], cfg["d_model"]

    def cut(a, which):
        r0, r1, c0, c1 = tp.slice_of(mc, which, rank, world)
        return np.ascontiguousarray(a[r0:r1, c0:c1])

    def allreduce(v):
        t = torch.from_numpy(v.copy()); dist.all_reduce(t); return t.numpy()

    cos, sin = orc.rope_tables(hd, cfg["max_seq_len"], cfg["rope_theta"],
                               dict(factor=cfg["yarn_factor"], orig_max_pos=cfg["yarn_orig_max_pos"],
                                    beta_fast=cfg["yarn_beta_fast"], beta_slow=cfg["yarn_beta_slow"]))
    scale = np.float32(1.0 / np.sqrt(hd) * cfg["yarn_attn_factor"])
    nh, nkv = cfg["n_heads"] // world, cfg["n_kv_heads"] // world
    kc = [np.zeros((cfg["max_seq_len"], nkv * hd), np.float32) for _ in range(cfg["n_layers"])]
    vc = [np.zeros((cfg["max_seq_len"], nkv * hd), np.float32) for _ in range(cfg["n_layers"])]
    full = helpers.oracle_model(cfg, w, helpers.SMALL_SWA_LAYERS)
    toks = orc.uniform_u32(12, 13, 1, cfg["vocab_size"])
    worst = 0.0
    for pos, t in enumerate(toks):
        x = w["embed"][int(t)].copy()
        for l, Lw in enumerate(w["layers"]):
            q = orc.linear(cut(Lw["wq"], _ffi.T_WQ), x); k = orc.linear(cut(Lw["wk"], _ffi.T_WK), x)
            v = orc.linear(cut(Lw["wv"], _ffi.T_WV), x)
            qn = cut(Lw["q_norm"][None, :], _ffi.T_Q_NORM)[0]; kn = cut(Lw["k_norm"][None, :], _ffi.T_K_NORM)[0]
            for h in range(nh):
                q[h * hd:(h + 1) * hd] = orc.rope_apply(orc.rmsnorm(q[h * hd:(h + 1) * hd], qn[h * hd:(h + 1) * hd], 1e-6), hd, cos[pos], sin[pos])
            for h in range(nkv):
                k[h * hd:(h + 1) * hd] = orc.rope_apply(orc.rmsnorm(k[h * hd:(h + 1) * hd], kn[h * hd:(h + 1) * hd], 1e-6), hd, cos[pos], sin[pos])
            kc[l][pos] = k; vc[l][pos] = v
            window = cfg["sliding_window"] if helpers.SMALL_SWA_LAYERS[l] else 0
            a = orc.decode_attention(q, kc[l], vc[l], nh, nkv, hd, pos, scale, window)
            o = allreduce(orc.linear(cut(Lw["wo"], _ffi.T_WO), a))                     # row-parallel
            x = x + orc.rmsnorm(o, Lw["attn_norm"], cfg["rms_norm_eps"])
            g = orc.linear(cut(Lw["gate"], _ffi.T_GATE), x); u = orc.linear(cut(Lw["up"], _ffi.T_UP), x)
            hgu = np.array([orc.silu(a_) * b_ for a_, b_ in zip(g, u)], np.float32)
            dn = allreduce(orc.linear(cut(Lw["down"], _ffi.T_DOWN), hgu))              # row-parallel
            x = x + orc.rmsnorm(dn, Lw["ffn_norm"], cfg["rms_norm_eps"])
        xn = orc.rmsnorm(x, w["final_norm"], cfg["rms_norm_eps"])
        part = np.zeros(L["vocab"], np.float32)
        mine = cut(w["lm_head"], _ffi.T_LM_HEAD)
        part[:mine.shape[0]] = orc.linear(mine, xn)
        gathered = [torch.zeros(L["vocab"]) for _ in range(world)]
        dist.all_gather(gathered, torch.from_numpy(part))
        logits = torch.cat(gathered).numpy()[:cfg["vocab_size"]]
        ref = full.forward_one(int(t))
        worst = max(worst, float(np.max(np.abs(logits - ref))))
        assert orc.argmax(logits) == orc.argmax(ref)
    out.put((rank, worst))
    dist.destroy_process_group()


def test_two_rank_partition_matches_unsharded_oracle():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=240) for _ in procs]
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    assert all(w <= 1e-4 for _, w in res), res


def test_slices_cover_every_tensor_once():
    import atlas_b200 as ab
    from atlas_b200 import tp, _ffi
    mc = ab.ModelConfig.olmo3_actual_7b()
    for world in (1, 2, 4, 8):
        for which, shape in [(_ffi.T_WQ, (4096, 4096)), (_ffi.T_WO, (4096, 4096)), (_ffi.T_GATE, (11008, 4096)),
                             (_ffi.T_DOWN, (4096, 11008)), (_ffi.T_LM_HEAD, (100278, 4096))]:
            cover = np.zeros(shape, np.uint8)
            for r in range(world):
                r0, r1, c0, c1 = tp.slice_of(mc, which, r, world)
                cover[r0:r1, c0:c1] += 1
            assert (cover == 1).all()
        assert tp.local_dims(mc, world)["vocab"] * world >= mc.vocab_size
    with pytest.raises(ab.AtlasError):
        tp.local_dims(ab.ModelConfig(100, 96, 1, 3, 3, 64, 8), 2)


def _guard_worker(rank, world, port, store_port, scenario, out):
    """Failure made on the host, CPU ranks over gloo: rank 1 skips a step, or leaves between steps;
    rank 0 must get an error status within the deadline instead of entering the collective."""
    sys.path.insert(0, ROOT)
    import datetime
    import time
    import torch
    import torch.distributed as dist
    import atlas_b200 as ab
    from atlas_b200 import tp
    os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
    store = dist.TCPStore("127.0.0.1", store_port, world, rank == 0, timeout=datetime.timedelta(seconds=20))
    guard = tp.StepGuard(store, rank, world, deadline_s=1.0)
    done, err, waited = 0, "", 0.0
    try:
        for s in range(1, 7):
            if rank == 1 and s == 4:
                if scenario == "leave":
                    guard.leave()                   # between steps, nothing in flight
                else:
                    time.sleep(3.0)                 # never announces step 4 in time: "skips" it
                break
            t0 = time.monotonic()
            guard.step_barrier()
            waited = time.monotonic() - t0
            t = torch.ones(4) * (rank + 1)
            dist.all_reduce(t)                      # stands for the step's collective
            assert float(t[0]) == 3.0
            done = s
    except ab.AtlasError as e:
        err = str(e)
        waited = time.monotonic() - t0
    out.put((rank, done, err, waited))
    time.sleep(0.5 if rank == 0 else 0.0)           # rank 0 owns the store: let the peer finish its last reads
    # no destroy_process_group: it would be a collective with a rank that has gone


@pytest.mark.parametrize("scenario", ["skip", "leave"])
def test_step_guard_turns_a_missing_rank_into_an_error_within_the_deadline(scenario):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port, store_port = _free_port(), _free_port()
    procs = [ctx.Process(target=_guard_worker, args=(r, 2, port, store_port, scenario, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = dict((r, (done, err, waited)) for r, done, err, waited in [q.get(timeout=120) for _ in procs])
    for p in procs:
        p.join(60)
    done0, err0, waited0 = res[0]
    assert done0 == 3 and res[1][0] == 3                      # three good steps on both ranks
    if scenario == "leave":
        assert "left the group before step 4" in err0 and waited0 < 1.0     # learnt at once, no deadline needed
    else:
        assert "did not reach step 4 within" in err0 and 0.9 <= waited0 < 2.5
