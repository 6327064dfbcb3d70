"""GPU: models loaded straight from safetensors files (atlasx_model_load_safetensors / _load_dir)
give the tokens and logits of the same tensors handed over one by one, of the committed golden run
and of the CPU oracle."""
import json
import os

import numpy as np
import pytest

from oracle import orc
import helpers
from test_safetensors import hf_names

pytestmark = pytest.mark.gpu
G = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.fixture(scope="module")
def ab():
    import atlas_b200
    orc.set_threads(os.cpu_count() or 1)
    return atlas_b200


def _mc(ab, cfg, layers=None):
    mc = ab.ModelConfig(cfg["vocab_size"], cfg["d_model"], cfg["n_layers"], cfg["n_heads"], cfg["n_kv_heads"],
                        cfg["ffn_hidden"], cfg["max_seq_len"], cfg["rope_theta"], cfg["rms_norm_eps"],
                        layer_types=list(layers) if layers else [], sliding_window=cfg.get("sliding_window") or None)
    if cfg.get("rope_scaling"):
        mc.rope_scaling = ab.Yarn(cfg["yarn_factor"], cfg["yarn_orig_max_pos"], cfg["yarn_attn_factor"],
                                  cfg["yarn_beta_fast"], cfg["yarn_beta_slow"])
    return mc


def test_config1_from_file_yields_the_golden_tokens(ab, tmp_path):
    """BASELINE config 1 written as an F32 safetensors file (the reference's synthetic-file test,
    :3352-3386, at model scale) and loaded: the committed golden tokens of the oracle."""
    g = np.load(os.path.join(G, "model.npz"))
    w = helpers.synth_weights(helpers.C1, seed=0)
    p = str(tmp_path / "c1.safetensors")
    ab.SafetensorsFile.build(p, hf_names(helpers.C1, w))
    m = ab.load_model_from_safetensors(p, _mc(ab, helpers.C1), kv_dtype=ab.F32)
    s = m.load_stats
    assert s.post_norm and not s.tied_lm_head and s.weight_format == ab.F32
    assert s.n_tensors_used == 3 + 4 * 11 and s.bytes_uploaded == os.path.getsize(p) - 8 - _header_len(p)
    assert m.generate(g["c1_prompt"], 64, 0.0) == g["c1_f32kv_tokens"].tolist()


def _header_len(p):
    import struct
    return struct.unpack("<Q", open(p, "rb").read(8))[0]


@pytest.mark.parametrize("fmt", ["auto", "int8", "int4"])
def test_sharded_bf16_directory_with_config_json(ab, tmp_path, fmt):
    """A model directory as load_model_from_dir reads it (:2437-2570): config.json (layer types, window,
    YaRN, eps, eos), an index naming two shards, BF16 tensors.  The file's bytes reach the device as
    stored (auto → bf16) or are quantised while loading; logits equal the same tensors given one by one
    and stay within the bound of the oracle."""
    cfg = dict(helpers.SMALL_SWA)
    w = helpers.synth_weights(cfg, seed=63, bf16=True, norm_jitter=0.1)
    d = tmp_path / "model"; d.mkdir()
    tensors = hf_names(cfg, w)
    half = len(tensors) // 2
    ab.SafetensorsFile.build(str(d / "model-00001-of-00002.safetensors"), tensors[:half])
    ab.SafetensorsFile.build(str(d / "model-00002-of-00002.safetensors"), tensors[half:])
    json.dump({"metadata": {}, "weight_map": {t[0]: ("model-00001-of-00002.safetensors" if i < half else "model-00002-of-00002.safetensors")
                                              for i, t in enumerate(tensors)}}, open(d / "model.safetensors.index.json", "w"))
    json.dump({"layer_types": ["sliding_attention" if s else "full_attention" for s in helpers.SMALL_SWA_LAYERS],
               "sliding_window": cfg["sliding_window"], "rope_theta": cfg["rope_theta"], "rms_norm_eps": cfg["rms_norm_eps"],
               "eos_token_id": 7,
               "rope_scaling": {"rope_type": "yarn", "factor": cfg["yarn_factor"], "original_max_position_embeddings": cfg["yarn_orig_max_pos"],
                                "attention_factor": cfg["yarn_attn_factor"], "beta_fast": cfg["yarn_beta_fast"], "beta_slow": cfg["yarn_beta_slow"]}},
              open(d / "config.json", "w"))
    bare = ab.ModelConfig(cfg["vocab_size"], cfg["d_model"], cfg["n_layers"], cfg["n_heads"], cfg["n_kv_heads"],
                          cfg["ffn_hidden"], cfg["max_seq_len"])                # everything else comes from config.json
    code = {"auto": ab.AUTO, "int8": ab.INT8, "int4": ab.INT4}[fmt]
    m = ab.load_model_from_dir(str(d), bare, kv_dtype=ab.F32, weight_format=code)
    assert m.load_stats.weight_format == (ab.BF16 if fmt == "auto" else code) and m.load_stats.post_norm
    assert bare.layer_types == list(helpers.SMALL_SWA_LAYERS) and bare.sliding_window == cfg["sliding_window"] and m.eos_token_id == 7
    m.eos_token_id = None
    one_by_one = helpers.cuda_model(cfg, w, helpers.SMALL_SWA_LAYERS, kv_dtype=ab.F32, weight_format=None if fmt == "auto" else code)
    wf = {"embed": orc.bf16_to_f32(w["embed"]).reshape(w["embed"].shape), "final_norm": w["final_norm"],
          "lm_head": orc.bf16_to_f32(w["lm_head"]).reshape(w["lm_head"].shape), "layers": []}
    for L in w["layers"]:
        wf["layers"].append({k: (orc.bf16_to_f32(v).reshape(v.shape) if v.dtype == np.uint16 else v) for k, v in L.items()})
    if fmt != "auto":
        from test_gpu_model import _requantised
        wf = _requantised(wf, fmt)
    o = helpers.oracle_model(cfg, wf, helpers.SMALL_SWA_LAYERS)
    toks = orc.uniform_u32(20, 63, 1, cfg["vocab_size"])
    for t in toks:
        a = m.forward_one_gpu(int(t))
        assert np.array_equal(a, one_by_one.forward_one_gpu(int(t)))
        assert np.max(np.abs(a - o.forward_one(int(t)))) <= 1e-3


def test_tied_head_prenorm_names_and_f16_tensors(ab, tmp_path):
    """No lm_head.weight (lm_head = embedding, :2309-2312), Llama pre-norm names (input_layernorm, and
    post_attention_layernorm as the FFN norm when no post_feedforward_layernorm exists, :2330-2338),
    layers.N. prefix without `model.`, F16 tensors converted while loading, unknown tensors ignored."""
    cfg = dict(vocab_size=256, d_model=64, n_layers=2, n_heads=4, n_kv_heads=2, ffn_hidden=128,
               max_seq_len=64, rope_theta=10000.0, rms_norm_eps=1e-5, post_norm=0)
    w = helpers.synth_weights(cfg, seed=65, qk_norm=False, norm_jitter=0.2)
    half = lambda a: a.astype(np.float16)
    names = {"wq": "self_attn.q_proj", "wk": "self_attn.k_proj", "wv": "self_attn.v_proj", "wo": "self_attn.o_proj",
             "gate": "mlp.gate_proj", "up": "mlp.up_proj", "down": "mlp.down_proj",
             "attn_norm": "input_layernorm", "ffn_norm": "post_attention_layernorm"}
    entries, blob, wf = {}, b"", {"embed": half(w["embed"]).astype(np.float32), "final_norm": w["final_norm"], "layers": []}
    wf["lm_head"] = wf["embed"]

    def add(name, a, f16):
        nonlocal blob
        raw = half(a).tobytes() if f16 else a.astype(np.float32).tobytes()
        entries[name] = {"dtype": "F16" if f16 else "F32", "shape": list(a.shape), "data_offsets": [len(blob), len(blob) + len(raw)]}
        blob += raw
    add("tok_embeddings.weight", w["embed"], True)
    add("norm.weight", w["final_norm"], False)
    add("rotary.inv_freq", np.ones(8, np.float32), False)                   # ignored
    for l, L in enumerate(w["layers"]):
        Lf = {}
        for k, n in names.items():
            f16 = k not in ("attn_norm", "ffn_norm")
            add("layers.%d.%s.weight" % (l, n), L[k], f16)
            Lf[k] = half(L[k]).astype(np.float32) if f16 else L[k]
        wf["layers"].append(Lf)
    import struct
    p = str(tmp_path / "llama.safetensors")
    text = json.dumps(entries)
    open(p, "wb").write(struct.pack("<Q", len(text)) + text.encode() + blob)
    mc = ab.ModelConfig(256, 64, 2, 4, 2, 128, 64, 10000.0, 1e-5)
    m = ab.load_model_from_safetensors(p, mc, kv_dtype=ab.F32)
    assert m.load_stats.tied_lm_head and not m.load_stats.post_norm and m.load_stats.weight_format == ab.F32
    o = helpers.oracle_model(cfg, wf)
    for t in (7, 100, 255, 3):
        assert np.max(np.abs(m.forward_one_gpu(t) - o.forward_one(t))) <= 1e-4


def test_loader_errors(ab, tmp_path):
    cfg = dict(helpers.SMALL_SWA)
    w = helpers.synth_weights(cfg, seed=66)
    p = str(tmp_path / "bad.safetensors")
    t = hf_names(cfg, w)
    ab.SafetensorsFile.build(p, [x for x in t if "layers.2.mlp.down_proj" not in x[0]])
    with pytest.raises(ab.AtlasError, match="was not set"):
        ab.load_model_from_safetensors(p, _mc(ab, cfg, helpers.SMALL_SWA_LAYERS))
    wrong = dict(cfg, ffn_hidden=256)
    ab.SafetensorsFile.build(p, t)
    with pytest.raises(ab.AtlasError, match="the configuration expects"):
        ab.load_model_from_safetensors(p, _mc(ab, wrong, helpers.SMALL_SWA_LAYERS))
    with pytest.raises(ab.AtlasError, match="cannot open"):
        ab.load_model_from_dir(str(tmp_path / "nothing_here"), _mc(ab, cfg))
