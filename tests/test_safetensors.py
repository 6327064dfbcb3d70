"""CPU: the mapped safetensors reader/writer of the library (csrc/loader.cu behind
atlas_b200.safetensors) against the format the reference reads and writes
(crates/atlas-model/src/lib.rs: from_bytes :2081-2125, build_f32 :2154-2185, get_f32 :2205-2240,
f16_to_f32 :2243-2262) and its own known answers (:3156-3240).  No compute call: runs without a GPU."""
import json
import os
import struct

import numpy as np
import pytest

import atlas_b200 as ab
from atlas_b200 import _ffi, tp
from oracle import orc
import helpers


def test_writer_produces_the_reference_header_text(tmp_path):
    """build_f32 writes `"name":{"dtype":"F32","shape":[..],"data_offsets":[a,b]}` entries in the order
    given, comma-separated, no spaces, after an 8-byte little-endian header length."""
    p = str(tmp_path / "a.safetensors")
    w1 = np.arange(6, dtype=np.float32).reshape(2, 3)
    w2 = np.array([1.5, -2.0, 0.25], np.float32)
    w3 = np.array([7.0], np.float32)
    ab.SafetensorsFile.build_f32(p, [("layer.0.weight", [2, 3], w1), ("layer.1.bias", [3], w2), ("scalar", [1], w3)])
    raw = open(p, "rb").read()
    want = ('{"layer.0.weight":{"dtype":"F32","shape":[2,3],"data_offsets":[0,24]},'
            '"layer.1.bias":{"dtype":"F32","shape":[3],"data_offsets":[24,36]},'
            '"scalar":{"dtype":"F32","shape":[1],"data_offsets":[36,40]}}').encode()
    assert struct.unpack("<Q", raw[:8])[0] == len(want)
    assert raw[8:8 + len(want)] == want
    assert raw[8 + len(want):] == w1.tobytes() + w2.tobytes() + w3.tobytes()
    st = ab.SafetensorsFile.open(p)
    assert len(st) == 3 and not st.is_empty()
    assert st.tensor_names() == ["layer.0.weight", "layer.1.bias", "scalar"]
    assert st.contains("scalar") and not st.contains("nope")
    assert st.get_desc("layer.0.weight").shape == (2, 3) and st.get_desc("layer.1.bias").shape == (3,)
    assert np.array_equal(st.get_f32("layer.0.weight"), w1.reshape(-1))
    assert np.array_equal(st.get_f32("scalar"), w3)
    with pytest.raises(ab.AtlasError, match="not BF16"):
        st.get_bf16("scalar")
    with pytest.raises(ab.AtlasError, match="not found"):
        st.get_f32("nope")


def _handwritten(path, entries, data, metadata=True, spaces=True):
    """A file written the way other tools write it: spaces in the header, a __metadata__ entry."""
    hdr = {}
    if metadata:
        hdr["__metadata__"] = {"format": "pt"}
    hdr.update(entries)
    text = json.dumps(hdr) if spaces else json.dumps(hdr, separators=(",", ":"))
    text += " " * ((8 - len(text) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(text))); f.write(text.encode()); f.write(data)


def test_reader_known_answers_bf16_f16_and_foreign_headers(tmp_path):
    """bf16 1.0 = 0x3F80, −2.0 = 0xC000 (:3202-3240); f16 table 1.0, −1.0, ±0, 0.5, 65504, ±inf, NaN,
    smallest subnormal (:3156-3199)."""
    p = str(tmp_path / "b.safetensors")
    bf = np.array([0x3F80, 0xC000, 0x0000], np.uint16)
    f16 = np.array([0x3C00, 0xBC00, 0x0000, 0x8000, 0x3800, 0x7BFF, 0x7C00, 0xFC00, 0x7C01, 0x0001], np.uint16)
    i64 = np.arange(2, dtype=np.int64)
    data = bf.tobytes() + f16.tobytes() + i64.tobytes()
    _handwritten(p, {"y": {"dtype": "BF16", "shape": [3], "data_offsets": [0, 6]},
                     "x": {"dtype": "F16", "shape": [10], "data_offsets": [6, 26]},
                     "ids": {"dtype": "I64", "shape": [2], "data_offsets": [26, 42]}}, data)
    st = ab.SafetensorsFile.open(p)
    assert st.tensor_names() == ["y", "x", "ids"]                         # __metadata__ is skipped
    assert st.get_f32("y").tolist() == [1.0, -2.0, 0.0]
    assert st.get_bf16("y").tolist() == bf.tolist()
    x = st.get_f32("x")
    assert x[:3].tolist() == [1.0, -1.0, 0.0] and x[3] == 0.0 and np.signbit(x[3])
    assert x[4] == 0.5 and x[5] == 65504.0 and x[6] == np.inf and x[7] == -np.inf and np.isnan(x[8])
    assert x[9] == np.float32(2.0 ** -24)
    assert np.array_equal(x[:8], f16[:8].view(np.float16).astype(np.float32))
    with pytest.raises(ab.AtlasError, match="unsupported dtype: I64"):
        st.get_f32("ids")


def test_reader_rejects_damaged_files(tmp_path):
    p = str(tmp_path / "c.safetensors")
    open(p, "wb").write(b"\x01\x02")
    with pytest.raises(ab.AtlasError, match="too short"):
        ab.SafetensorsFile.open(p)
    open(p, "wb").write(struct.pack("<Q", 1000) + b"{}")
    with pytest.raises(ab.AtlasError, match="header truncated"):
        ab.SafetensorsFile.open(p)
    open(p, "wb").write(struct.pack("<Q", 5) + b"{nope")
    with pytest.raises(ab.AtlasError, match="header JSON"):
        ab.SafetensorsFile.open(p)
    _handwritten(p, {"w": {"dtype": "F32", "shape": [4]}}, b"\0" * 16)
    with pytest.raises(ab.AtlasError, match="missing data_offsets for w"):
        ab.SafetensorsFile.open(p)
    _handwritten(p, {"w": {"dtype": "F32", "shape": [4], "data_offsets": [0, 64]}}, b"\0" * 16)
    with pytest.raises(ab.AtlasError, match="outside the file"):
        ab.SafetensorsFile.open(p)
    _handwritten(p, {"w": {"dtype": "F32", "shape": [4], "data_offsets": [0.5, 16]}}, b"\0" * 16)
    with pytest.raises(ab.AtlasError, match="not non-negative integers"):
        ab.SafetensorsFile.open(p)
    _handwritten(p, {"w": {"dtype": "F32", "shape": [4], "data_offsets": [-4, 16]}}, b"\0" * 16)
    with pytest.raises(ab.AtlasError, match="not non-negative integers"):
        ab.SafetensorsFile.open(p)
    # a shape whose product wraps around 2^64 back to the element count must not pass for a match
    # (3 · 0xAAAAAAAAAAAAAAAB ≡ 1 modulo 2^64, so the wrapped product of this shape equals the four stored elements)
    _handwritten(p, {"w": {"dtype": "F32", "shape": [3, 0xAAAAAAAAAAAAAAAB, 4], "data_offsets": [0, 16]}}, b"\0" * 16)
    f = ab.SafetensorsFile.open(p)
    with pytest.raises(ab.AtlasError, match="shape and byte count disagree"):
        f.get_f32("w")
    with pytest.raises(ab.AtlasError, match="cannot open"):
        ab.SafetensorsFile.open(str(tmp_path / "missing.safetensors"))
    open(p, "wb").write(struct.pack("<Q", 2) + b"{}")
    assert ab.SafetensorsFile.open(p).is_empty()


def hf_names(cfg, w, bf16=False):
    """The tensors of a synthetic model under the names the loaders match (:2300-2346), post-norm layout."""
    out = [("model.embed_tokens.weight", w["embed"]), ("lm_head.weight", w["lm_head"]), ("model.norm.weight", w["final_norm"])]
    local = {"wq": "self_attn.q_proj", "wk": "self_attn.k_proj", "wv": "self_attn.v_proj", "wo": "self_attn.o_proj",
             "gate": "mlp.gate_proj", "up": "mlp.up_proj", "down": "mlp.down_proj",
             "attn_norm": "post_attention_layernorm", "ffn_norm": "post_feedforward_layernorm",
             "q_norm": "self_attn.q_norm", "k_norm": "self_attn.k_norm"}
    for l, L in enumerate(w["layers"]):
        for k, name in local.items():
            if k in L:
                out.append(("model.layers.%d.%s.weight" % (l, name), L[k]))
    return [(n, list(a.shape), a) for n, a in out]


@pytest.mark.parametrize("bf16", [False, True])
def test_round_trip_of_a_synthetic_model_and_rank_slices(tmp_path, bf16):
    """Every tensor of a synthetic model written and read back bit for bit — whole, and as the row or
    column ranges each tensor-parallel rank keeps (tp.slice_of)."""
    cfg = dict(helpers.SMALL_SWA)
    w = helpers.synth_weights(cfg, seed=61, bf16=bf16, norm_jitter=0.1)
    p = str(tmp_path / "m.safetensors")
    tensors = hf_names(cfg, w)
    ab.SafetensorsFile.build(p, tensors)
    st = ab.SafetensorsFile.open(p)
    assert st.tensor_names() == [t[0] for t in tensors]
    for name, shape, a in tensors:
        d = st.get_desc(name)
        assert d.shape == tuple(shape) and d.dtype == ("BF16" if a.dtype == np.uint16 else "F32")
        if a.dtype == np.uint16:
            assert np.array_equal(st.get_bf16(name), a.reshape(-1))
            assert np.array_equal(st.get_f32(name), orc.bf16_to_f32(a.reshape(-1)))
        else:
            assert np.array_equal(st.get_f32(name).view(np.uint32), a.reshape(-1).view(np.uint32))
    mc = ab.ModelConfig(cfg["vocab_size"], cfg["d_model"], cfg["n_layers"], cfg["n_heads"], cfg["n_kv_heads"],
                        cfg["ffn_hidden"], cfg["max_seq_len"])
    for which, name in ((_ffi.T_WQ, "self_attn.q_proj"), (_ffi.T_WK, "self_attn.k_proj"), (_ffi.T_WO, "self_attn.o_proj"),
                        (_ffi.T_GATE, "mlp.gate_proj"), (_ffi.T_DOWN, "mlp.down_proj")):
        key = {"self_attn.q_proj": "wq", "self_attn.k_proj": "wk", "self_attn.o_proj": "wo", "mlp.gate_proj": "gate", "mlp.down_proj": "down"}[name]
        full = w["layers"][1][key]
        for rank in range(2):
            r0, r1, c0, c1 = tp.slice_of(mc, which, rank, 2)
            get = st.get_bf16 if bf16 else st.get_f32
            part = get("model.layers.1.%s.weight" % name, rows=(r0, r1), cols=(c0, c1))
            assert np.array_equal(part, full[r0:r1, c0:c1])


def test_config_json_overlay(tmp_path):
    """patch_config_from_hf_json (:2367-2432): only present fields change; OLMo-3 values as in the
    reference's own test (:3523-3592)."""
    p = str(tmp_path / "config.json")
    json.dump({"layer_types": ["sliding_attention", "sliding_attention", "sliding_attention", "full_attention"],
               "sliding_window": 4096, "rope_theta": 500000, "rms_norm_eps": 1e-06, "eos_token_id": 100257,
               "max_position_embeddings": 65536,
               "rope_scaling": {"rope_type": "yarn", "factor": 8.0, "original_max_position_embeddings": 8192,
                                "attention_factor": 1.2079441541679836, "beta_fast": 32, "beta_slow": 1}}, open(p, "w"))
    cfg = ab.ModelConfig(100278, 4096, 4, 32, 32, 11008, 512)
    ab.patch_config_from_hf_json(cfg, p)
    assert cfg.layer_types == [ab.LAYER_SLIDING] * 3 + [ab.LAYER_FULL]
    assert cfg.sliding_window == 4096 and cfg.rope_theta == 500000.0 and cfg.eos_token_id == 100257
    assert abs(cfg.rms_norm_eps - 1e-6) < 1e-12 and cfg.max_seq_len == 512            # max_seq_len is the caller's
    y = cfg.rope_scaling
    assert (y.factor, y.orig_max_pos, y.beta_fast, y.beta_slow) == (8.0, 8192, 32.0, 1.0)
    assert abs(y.attn_factor - 1.2079441541679836) < 1e-6
    json.dump({"rope_theta": 10000.0}, open(p, "w"))
    cfg2 = ab.ModelConfig(256, 64, 2, 4, 2, 128, 128, rope_theta=1.0, rms_norm_eps=1e-5)
    ab.patch_config_from_hf_json(cfg2, p)
    assert cfg2.rope_theta == 10000.0 and abs(cfg2.rms_norm_eps - 1e-5) < 1e-12 and cfg2.rope_scaling is None
    assert cfg2.layer_types == [] and cfg2.eos_token_id is None
