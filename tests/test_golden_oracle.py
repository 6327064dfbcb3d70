"""The committed golden vectors must be reproduced by the CPU oracle on any machine
(guards against a libm or compiler difference silently changing the checker)."""
import hashlib
import os

import numpy as np
import pytest

from oracle import orc
import helpers

G = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def test_quant_fixtures():
    g = np.load(os.path.join(G, "quant.npz"))
    for rows, cols, block in [(7, 257, 32), (16, 4096, 32), (5, 96, 64), (64, 11008, 32)]:
        w = orc.normal_f32(rows * cols, 21, rows * 100000 + cols, 0.02).reshape(rows, cols)
        w[0, :] = 0.0
        q8, s8 = orc.int8_quantize(w)
        q4, s4 = orc.int4_quantize(w, block)
        key = "%dx%d_b%d" % (rows, cols, block)
        assert sha(q8) == str(g[key + "_i8_sha"]) and sha(s8) == str(g[key + "_s8_sha"])
        assert sha(q4) == str(g[key + "_i4_sha"]) and sha(s4) == str(g[key + "_s4_sha"])
        if key + "_i8" in g:
            assert np.array_equal(q8, g[key + "_i8"]) and np.array_equal(q4, g[key + "_i4"])


def test_gemv_fixtures():
    g = np.load(os.path.join(G, "gemv.npz"))
    for m, k in [(64, 256), (48, 1376), (33, 200)]:
        w16 = orc.normal_bf16(m * k, 22, m * 10000 + k, 0.02).reshape(m, k)
        x = orc.normal_f32(k, 22, 7, 1.0)
        assert np.array_equal(orc.linear(w16, x), g["bf16_%dx%d" % (m, k)])


def test_attention_fixtures():
    g = np.load(os.path.join(G, "attention.npz"))
    nh, nkv, hd = 8, 2, 64
    for pos, window in [(0, 0), (37, 0), (37, 8), (7, 8), (8, 8)]:
        n = (pos + 1) * nkv * hd
        k = orc.bf16_to_f32(orc.normal_bf16(n, 23, 1, 1.0))
        v = orc.bf16_to_f32(orc.normal_bf16(n, 23, 2, 1.0))
        q = orc.normal_f32(nh * hd, 23, 3, 1.0)
        out = orc.decode_attention(q, k, v, nh, nkv, hd, pos, 1.0 / np.sqrt(hd), window)
        assert np.max(np.abs(out - g["p%d_w%d" % (pos, window)])) < 1e-6


@pytest.mark.parametrize("tag,rnd", [("c1_f32kv", False), ("c1_bf16kv", True)])
def test_c1_model_fixture(tag, rnd):
    g = np.load(os.path.join(G, "model.npz"))
    orc.set_threads(os.cpu_count() or 1)
    w = helpers.synth_weights(helpers.C1, seed=0)
    m = helpers.oracle_model(helpers.C1, w, kv_round_bf16=rnd)
    toks, logits, margins = m.generate_greedy(g["c1_prompt"], 64, want_logits=True)
    assert np.array_equal(toks, g[tag + "_tokens"])
    assert np.max(np.abs(logits[0] - g[tag + "_logits_step0"])) < 1e-5
    assert np.max(np.abs(logits[63] - g[tag + "_logits_step63"])) < 1e-5
    assert margins.min() > 5e-3


def test_swa_model_fixture():
    g = np.load(os.path.join(G, "model.npz"))
    w = helpers.synth_weights(helpers.SMALL_SWA, seed=5, norm_jitter=0.1)
    m = helpers.oracle_model(helpers.SMALL_SWA, w, helpers.SMALL_SWA_LAYERS)
    toks, logits, _ = m.generate_greedy(g["swa_prompt"], 40, want_logits=True)
    assert np.array_equal(toks, g["swa_f32kv_tokens"])
    assert np.max(np.abs(logits[39] - g["swa_f32kv_logits_step39"])) < 1e-5
