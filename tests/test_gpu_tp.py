"""Two GPUs, one process each: the tensor-parallel step (row-parallel GEMVs pushing their partial
sums into peer mailboxes, and the NCCL all-reduce it replaces) gives the logits and greedy tokens
of the single-GPU model and of the CPU oracle."""
import os
import socket
import subprocess
import sys

import numpy as np
import pytest

import helpers
from oracle import orc

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _gpu_count():
    try:
        import torch
        return torch.cuda.device_count()
    except Exception:
        return 0


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close(); return p


@pytest.mark.skipif(_gpu_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("peer", ["mailbox", "mailbox_reduce", "mailbox_fused", "mailbox_fused_gather", "nccl"])
@pytest.mark.parametrize("kv", ["f32", "bf16"])
def test_two_gpu_tensor_parallel_matches_single_gpu_and_oracle(tmp_path, kv, peer):
    import atlas_b200 as ab
    n_tok = 20
    out = str(tmp_path / "tp.npz")
    # who sums the mailbox parts: every consumer CTA (0), a kernel of its own (1), the consumer's first CTAs (2, the
    # default); and greedy selection over the ranks' local maxima (default) or over all-gathered logits
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", ATLASX_PEER_ALLREDUCE="0" if peer == "nccl" else "1",
               ATLASX_MAIL_REDUCE={"mailbox": "0", "mailbox_reduce": "1"}.get(peer, "2"),
               ATLASX_TP_SELECT="0" if peer == "mailbox_fused_gather" else "1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()),
           os.path.join(ROOT, "tests", "tp_worker.py"), out, kv, str(n_tok)]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=240)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    got = np.load(out)

    cfg = dict(helpers.HD128)
    w = helpers.synth_weights(cfg, seed=33, norm_jitter=0.1)
    one = helpers.cuda_model(cfg, w, helpers.HD128_LAYERS, kv_dtype=ab.F32 if kv == "f32" else ab.BF16)
    toks = orc.uniform_u32(n_tok, 33, 1, cfg["vocab_size"])
    ref = np.stack([one.forward_one_gpu(int(t)) for t in toks])
    tol = 1e-4 if kv == "f32" else 5e-3         # bf16 cache: a last-bit difference can flip a cached element's rounding
    assert np.max(np.abs(got["logits"] - ref)) <= tol
    o = helpers.oracle_model(cfg, w, helpers.HD128_LAYERS, kv_round_bf16=(kv == "bf16"))
    want = np.stack([o.forward_one(int(t)) for t in toks])
    assert np.max(np.abs(got["logits"] - want)) <= (1e-3 if kv == "f32" else 1e-2)
    one.reset()
    assert got["gen"].tolist() == one.generate(toks[:4], 12, 0.0)


@pytest.mark.skipif(_gpu_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("fmt", ["auto", "int8", "int4"])
def test_two_gpu_model_loaded_from_a_safetensors_file(tmp_path, fmt):
    """Each rank maps the same file and reads only its rows or columns (int8 weights that are split by
    columns are read whole, quantised, then cut): logits equal the single-GPU model built from the same
    tensors in the same storage format."""
    import atlas_b200 as ab
    from test_safetensors import hf_names
    n_tok = 12
    cfg = dict(helpers.HD128)
    w = helpers.synth_weights(cfg, seed=33, norm_jitter=0.1)
    path = str(tmp_path / "tp.safetensors")
    ab.SafetensorsFile.build(path, hf_names(cfg, w))
    out = str(tmp_path / "tp.npz")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()),
           os.path.join(ROOT, "tests", "tp_worker.py"), out, "f32", str(n_tok), path, fmt]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=240)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    got = np.load(out)
    code = {"auto": None, "int8": ab.INT8, "int4": ab.INT4}[fmt]
    one = helpers.cuda_model(cfg, w, helpers.HD128_LAYERS, kv_dtype=ab.F32, weight_format=code)
    toks = orc.uniform_u32(n_tok, 33, 1, cfg["vocab_size"])
    ref = np.stack([one.forward_one_gpu(int(t)) for t in toks])
    # quantised matrices see their input through two base-254 digits scaled by the largest element of the
    # vector THEY get: a rank's slice of a row-parallel input has its own scale, so the two models round the
    # activations differently (about 1e-5 of a product, a few 1e-4 on the logits after three layers)
    assert np.max(np.abs(got["logits"] - ref)) <= (1e-4 if fmt == "auto" else 5e-4)
