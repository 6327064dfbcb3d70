"""Shared test helpers: seeded synthetic models given identically to the CPU oracle and to the
CUDA library.  Test infrastructure only."""
import numpy as np

from oracle import orc

# tensor ids are the same numbers in the oracle and in the C ABI
PER_LAYER = [("wq", orc.T_WQ), ("wk", orc.T_WK), ("wv", orc.T_WV), ("wo", orc.T_WO),
             ("gate", orc.T_GATE), ("up", orc.T_UP), ("down", orc.T_DOWN)]

# BASELINE config 1: tiny OLMo-2-style decoder
C1 = dict(vocab_size=32000, d_model=512, n_layers=4, n_heads=8, n_kv_heads=8, ffn_hidden=1376,
          max_seq_len=128, rope_theta=10000.0, rms_norm_eps=1e-6, post_norm=1)

# a small GQA model with sliding-window layers and YaRN, shaped like OLMo-3 (S,S,S,F pattern)
SMALL_SWA = dict(vocab_size=1000, d_model=256, n_layers=4, n_heads=4, n_kv_heads=2, ffn_hidden=512,
                 max_seq_len=96, rope_theta=500000.0, rms_norm_eps=1e-6, post_norm=1,
                 sliding_window=8, rope_scaling=1, yarn_factor=8.0, yarn_orig_max_pos=32,
                 yarn_attn_factor=1.2079441541679836, yarn_beta_fast=32.0, yarn_beta_slow=1.0)
SMALL_SWA_LAYERS = [1, 1, 1, 0]

# head_dim 128 with two query heads per KV head: the shape class of the one-launch attention
HD128 = dict(vocab_size=2000, d_model=512, n_layers=3, n_heads=4, n_kv_heads=2, ffn_hidden=1024,
             max_seq_len=80, rope_theta=500000.0, rms_norm_eps=1e-6, post_norm=1,
             sliding_window=8, rope_scaling=1, yarn_factor=8.0, yarn_orig_max_pos=32,
             yarn_attn_factor=1.2079441541679836, yarn_beta_fast=32.0, yarn_beta_slow=1.0)
HD128_LAYERS = [1, 0, 1]


def shapes(cfg):
    d, hd = cfg["d_model"], cfg["d_model"] // cfg["n_heads"]
    kv = cfg["n_kv_heads"] * hd
    f = cfg["ffn_hidden"]
    return dict(wq=(d, d), wk=(kv, d), wv=(kv, d), wo=(d, d), gate=(f, d), up=(f, d), down=(d, f))


def synth_weights(cfg, seed=0, bf16=False, std=0.02, qk_norm=True, norm_jitter=0.0):
    """All tensors of a model from the seeded generator: stream id = layer·32 + tensor id.
    bf16=True returns uint16 bit patterns for the matrices (rounded to nearest even)."""
    gen = orc.normal_bf16 if bf16 else orc.normal_f32
    d, hd = cfg["d_model"], cfg["d_model"] // cfg["n_heads"]
    w = {"embed": gen(cfg["vocab_size"] * d, seed, 1, std).reshape(cfg["vocab_size"], d),
         "lm_head": gen(cfg["vocab_size"] * d, seed, 2, std).reshape(cfg["vocab_size"], d),
         "final_norm": _norm(d, seed, 3, norm_jitter), "layers": []}
    sh = shapes(cfg)
    for l in range(cfg["n_layers"]):
        L = {}
        for name, tid in PER_LAYER:
            r, c = sh[name]
            L[name] = gen(r * c, seed, 1000 + l * 32 + tid, std).reshape(r, c)
        L["attn_norm"] = _norm(d, seed, 1000 + l * 32 + orc.T_ATTN_NORM, norm_jitter)
        L["ffn_norm"] = _norm(d, seed, 1000 + l * 32 + orc.T_FFN_NORM, norm_jitter)
        if qk_norm:
            L["q_norm"] = _norm(cfg["n_heads"] * hd, seed, 1000 + l * 32 + orc.T_Q_NORM, norm_jitter)
            L["k_norm"] = _norm(cfg["n_kv_heads"] * hd, seed, 1000 + l * 32 + orc.T_K_NORM, norm_jitter)
        w["layers"].append(L)
    return w


def _norm(n, seed, stream, jitter):
    if jitter == 0.0:
        return np.ones(n, np.float32)
    return (np.float32(1.0) + orc.normal_f32(n, seed, stream, jitter)).astype(np.float32)


def give(model, w, set_fn=None):
    """Hand every tensor to a model exposing set_tensor(layer, which, array)."""
    st = set_fn or model.set_tensor
    st(0, orc.T_EMBED, w["embed"])
    st(0, orc.T_LM_HEAD, w["lm_head"])
    st(0, orc.T_FINAL_NORM, w["final_norm"])
    for l, L in enumerate(w["layers"]):
        for name, tid in PER_LAYER:
            st(l, tid, L[name])
        st(l, orc.T_ATTN_NORM, L["attn_norm"])
        st(l, orc.T_FFN_NORM, L["ffn_norm"])
        if "q_norm" in L:
            st(l, orc.T_Q_NORM, L["q_norm"])
            st(l, orc.T_K_NORM, L["k_norm"])


def oracle_model(cfg, w, layer_sliding=None, kv_round_bf16=False):
    m = orc.OracleModel(cfg, layer_sliding)
    give(m, w)
    m.set_kv_round_bf16(kv_round_bf16)
    return m


def cuda_model(cfg, w, layer_sliding=None, kv_dtype=None, weight_format=None, int4_block=32, ctx=None,
               use_graph=True, use_pdl=True):
    import atlas_b200 as ab
    mc = ab.ModelConfig(cfg["vocab_size"], cfg["d_model"], cfg["n_layers"], cfg["n_heads"], cfg["n_kv_heads"],
                        cfg["ffn_hidden"], cfg["max_seq_len"], cfg["rope_theta"], cfg["rms_norm_eps"],
                        layer_types=list(layer_sliding) if layer_sliding else [],
                        sliding_window=cfg.get("sliding_window") or None,
                        post_norm=bool(cfg.get("post_norm", 0)),
                        eos_token_id=cfg.get("eos_token_id"))
    if cfg.get("rope_scaling"):
        mc.rope_scaling = ab.Yarn(cfg["yarn_factor"], cfg["yarn_orig_max_pos"], cfg["yarn_attn_factor"],
                                  cfg["yarn_beta_fast"], cfg["yarn_beta_slow"])
    m = ab.OlmoModel(mc, ctx=ctx, kv_dtype=ab.BF16 if kv_dtype is None else kv_dtype,
                     weight_format=weight_format, int4_block=int4_block)
    give(m, w)
    m.init_gpu_resources(use_graph=use_graph, use_pdl=use_pdl)
    return m


def rel_err(a, b):
    """max|a−b| / max|b| — the form the reference's GEMV parity test uses
    (crates/atlas-model/src/lib.rs:3926-3933)."""
    a = np.asarray(a, np.float64); b = np.asarray(b, np.float64)
    return float(np.max(np.abs(a - b)) / max(np.max(np.abs(b)), 1e-6))
