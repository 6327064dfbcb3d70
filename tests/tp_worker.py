"""Worker of tests/test_gpu_tp.py: one rank of a tensor-parallel group on its own GPU.
Launched with torch.distributed.run; rank 0 writes the logits of every step to the given file."""
import ctypes as C
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT); sys.path.insert(0, os.path.join(ROOT, "tests"))


def main():
    out_path, kv, n_tok = sys.argv[1], sys.argv[2], int(sys.argv[3])
    import torch
    import torch.distributed as dist
    import helpers
    from oracle import orc
    import atlas_b200 as ab
    from atlas_b200 import _ffi
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    ctx = ab.Context(local)
    ident = (C.c_ubyte * 128)()
    if rank == 0:
        _ffi.check(_ffi.lib().atlasx_comm_unique_id(ident))
    t = torch.tensor(list(bytes(ident)), dtype=torch.uint8, device="cuda")
    dist.broadcast(t, 0)
    ident = (C.c_ubyte * 128)(*t.cpu().tolist())
    _ffi.check(_ffi.lib().atlasx_comm_init(ctx.handle, ident, rank, world))

    cfg = dict(helpers.HD128)
    w = helpers.synth_weights(cfg, seed=33, norm_jitter=0.1)
    mc = ab.ModelConfig(cfg["vocab_size"], cfg["d_model"], cfg["n_layers"], cfg["n_heads"], cfg["n_kv_heads"],
                        cfg["ffn_hidden"], cfg["max_seq_len"], cfg["rope_theta"], cfg["rms_norm_eps"],
                        layer_types=list(helpers.HD128_LAYERS), sliding_window=cfg["sliding_window"], post_norm=True)
    mc.rope_scaling = ab.Yarn(cfg["yarn_factor"], cfg["yarn_orig_max_pos"], cfg["yarn_attn_factor"],
                              cfg["yarn_beta_fast"], cfg["yarn_beta_slow"])
    # A first tensor-parallel model with fewer layers runs a few steps on the same context and is
    # freed: its sequence numbers stay behind in the peer mailboxes, and the model under test must
    # not take them for its own (the use counter belongs to the mailbox, not to a model).
    cfg0 = dict(cfg, n_layers=2)
    mc0 = ab.ModelConfig(cfg0["vocab_size"], cfg0["d_model"], 2, cfg0["n_heads"], cfg0["n_kv_heads"], cfg0["ffn_hidden"],
                         cfg0["max_seq_len"], cfg0["rope_theta"], cfg0["rms_norm_eps"], layer_types=[1, 0],
                         sliding_window=cfg0["sliding_window"], post_norm=True)
    m0 = ab.OlmoModel(mc0, ctx=ctx, kv_dtype=ab.F32, tp_rank=rank, tp_world=world)
    helpers.give(m0, dict(w, layers=w["layers"][:2]))
    m0.init_gpu_resources()
    for tk in range(9):
        m0.forward_one_gpu(tk)
    del m0
    if len(sys.argv) > 4:
        # from a safetensors file: each rank maps the file and reads only its rows / columns
        m = ab.load_model_from_safetensors(sys.argv[4], mc, ctx=ctx, kv_dtype=ab.F32 if kv == "f32" else ab.BF16,
                                           weight_format={"auto": ab.AUTO, "int8": ab.INT8, "int4": ab.INT4}[sys.argv[5]],
                                           tp_rank=rank, tp_world=world)
    else:
        m = ab.OlmoModel(mc, ctx=ctx, kv_dtype=ab.F32 if kv == "f32" else ab.BF16, tp_rank=rank, tp_world=world)
        helpers.give(m, w)                   # full tensors: the library keeps this rank's slices
        m.init_gpu_resources()
    toks = orc.uniform_u32(n_tok, 33, 1, cfg["vocab_size"])
    logits = np.stack([m.forward_one_gpu(int(tk)) for tk in toks])
    m.reset()
    gen = m.generate(toks[:4], 12, 0.0)
    dist.barrier()
    if rank == 0:
        np.savez(out_path, logits=logits, gen=np.asarray(gen, np.int64))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
