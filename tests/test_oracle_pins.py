"""Pins the CPU oracle against every known answer the reference's own tests hold for the
decode path (file:line of web3guru888/ATLAS in each test) and against an independent
numpy restatement of the atlas-quant formats.  No GPU needed."""
import math

import numpy as np
import pytest

from oracle import orc


# ── atlas-tensor known answers ───────────────────────────────────────────────────
def test_matmul_known_answer():
    # crates/atlas-tensor/src/lib.rs:1097-1106
    a = np.array([[1, 2, 3], [4, 5, 6]], dtype=np.float32)
    b = np.array([[7, 8], [9, 10], [11, 12]], dtype=np.float32)
    c = orc.gemm(a, b)
    assert c.tolist() == [[58.0, 64.0], [139.0, 154.0]]


def test_silu_known_answer():
    # crates/atlas-tensor/src/lib.rs:1183-1194
    assert abs(orc.silu(0.0)) < 1e-3
    assert abs(orc.silu(1.0) - 0.7310586) < 1e-6


def test_rmsnorm_known_answer():
    # crates/atlas-tensor/src/lib.rs:1170-1181
    out = orc.rmsnorm([1, 2, 3, 4], [1, 1, 1, 1], 1e-5)
    rms = math.sqrt(7.5)
    assert abs(out[0] - 1.0 / rms) < 1e-3 and abs(out[3] - 4.0 / rms) < 1e-3
    # crates/atlas-model/src/lib.rs:3832-3844 (d=64 regression inputs)
    x = ((np.arange(64, dtype=np.float32) + 1.0) * np.float32(0.01)).astype(np.float32)
    out = orc.rmsnorm(x, np.ones(64, np.float32), 1e-5)
    ref = x / np.sqrt(np.mean(x.astype(np.float64) ** 2) + 1e-5)
    assert np.max(np.abs(out - ref)) < 1e-5


def test_rope_identity_at_pos0():
    # crates/atlas-tensor/src/lib.rs:1196-1206
    cos, sin = orc.rope_tables(4, 2, 10000.0)
    out = orc.rope_apply([1, 2, 3, 4], 4, cos[0], sin[0])
    assert np.allclose(out, [1, 2, 3, 4], atol=1e-6)


def test_all_ones_gemv():
    # crates/atlas-tensor/src/lib.rs:1208-1219
    y = orc.linear(np.ones((4, 3), np.float32), np.ones(3, np.float32))
    assert np.allclose(y, 3.0)


def test_bf16_bit_patterns():
    # crates/atlas-model/src/lib.rs:3202-3215
    L = orc.lib()
    assert L.orc_f32_to_bf16_trunc(orc.C.c_float(1.0)) == 0x3F80
    assert L.orc_f32_to_bf16_trunc(orc.C.c_float(-2.0)) == 0xC000
    assert L.orc_f32_to_bf16_trunc(orc.C.c_float(0.0)) == 0x0000
    assert orc.bf16_to_f32(np.array([0x3F80, 0xC000], np.uint16)).tolist() == [1.0, -2.0]


def test_bf16_gemv_parity_inputs():
    # crates/atlas-model/src/lib.rs:3887-3934: formula-generated W and x, bf16 by truncation,
    # bf16 GEMV within 1 % (max-abs relative form) of the f32 GEMV.
    M, K = 128, 256
    i = np.arange(M * K, dtype=np.int64)
    w = (((i * 6977 + 1231) % 10000).astype(np.float32) / np.float32(10000.0) - np.float32(0.5)).reshape(M, K)
    k = np.arange(K, dtype=np.int64)
    x = ((k * 3571 + 421) % 10000).astype(np.float32) / np.float32(10000.0) - np.float32(0.5)
    w16 = (w.view(np.uint32) >> 16).astype(np.uint16)
    y_ref = orc.linear(w, x)
    y16 = orc.linear(w16, x)
    rel = np.max(np.abs(y_ref - y16)) / max(np.max(np.abs(y_ref)), 1e-6)
    assert rel < 0.01


def test_softmax_sums_to_one():
    # crates/atlas-tensor/src/lib.rs:1108-1114
    p = orc.softmax([1, 2, 3])
    assert abs(float(p.sum()) - 1.0) < 1e-6


def test_argmax_takes_last_of_equal_maxima():
    # crates/atlas-model/src/lib.rs:2701-2706 — Iterator::max_by keeps the later element on Equal
    assert orc.argmax([1.0, 3.0, 3.0, 2.0]) == 2
    assert orc.argmax(np.zeros(7, np.float32)) == 6
    assert orc.argmax([5.0]) == 0


# ── atlas-quant ──────────────────────────────────────────────────────────────────
def _np_round_half_away(v):
    return np.sign(v) * np.floor(np.abs(v) + np.float32(0.5))


def _np_int8_quantize(w):
    """numpy restatement of Int8Tensor::quantize, crates/atlas-quant/src/lib.rs:52-61."""
    w = w.astype(np.float32)
    mx = np.max(np.abs(w), axis=1)
    s = np.where(mx > 0, mx / np.float32(127.0), np.float32(1.0)).astype(np.float32)
    inv = (np.float32(1.0) / s).astype(np.float32)
    v = (w * inv[:, None]).astype(np.float32)
    q = _np_round_half_away(np.clip(v, -127.0, 127.0)).astype(np.int8)
    return q, s


def _np_int4_quantize(w, block):
    """numpy restatement of Int4Tensor::quantize, crates/atlas-quant/src/lib.rs:118-144."""
    flat = w.astype(np.float32).ravel()
    n = flat.size
    nb = (n + block - 1) // block
    scales = np.empty(nb, np.float32)
    q = np.empty(n, np.int8)
    for b in range(nb):
        blk = flat[b * block:(b + 1) * block]
        mx = np.max(np.abs(blk)) if blk.size else np.float32(0)
        s = np.float32(mx / np.float32(7.0)) if mx > 0 else np.float32(1.0)
        scales[b] = s
        inv = np.float32(1.0) / s
        q[b * block:b * block + blk.size] = _np_round_half_away(np.clip((blk * inv).astype(np.float32), -7, 7)).astype(np.int8)
    nib = (q.astype(np.uint8) & 0x0F)
    if n % 2:
        nib = np.concatenate([nib, np.zeros(1, np.uint8)])
    data = ((nib[0::2] << 4) | nib[1::2]).astype(np.uint8)
    return data, scales


def test_int8_roundtrip_reference_case():
    # crates/atlas-quant/src/lib.rs:258-267
    t = np.array([[1.0, -2.0], [3.0, -4.0]], np.float32)
    q, s = orc.int8_quantize(t)
    assert q.tolist() == [[64, -127], [95, -127]]      # 1·(127/2)=63.5 rounds away from zero
    assert np.max(np.abs(orc.int8_dequantize(q, s) - t)) < 0.1


def test_int8_compression_ratio():
    # crates/atlas-quant/src/lib.rs:269-275 (bytes = rows·cols + 4·rows)
    rows = cols = 128
    assert rows * cols * 4 / (rows * cols + 4 * rows) > 3.5


def test_int4_roundtrip_reference_case():
    # crates/atlas-quant/src/lib.rs:277-289
    data = (np.arange(64, dtype=np.float32) * np.float32(0.1) - np.float32(3.0)).reshape(1, 64)
    q, s = orc.int4_quantize(data, 64)
    out = orc.int4_dequantize(q, s, 64, 64)
    assert np.max(np.abs(out - data.ravel())) < 0.5
    assert q.size == 32 and s.size == 1


def test_int4_compression_ratio():
    # crates/atlas-quant/src/lib.rs:291-297 (block 64)
    n = 128 * 128
    assert n * 4 / (n // 2 + (n // 64) * 4) > 7.0


def test_int4_nibble_layout():
    # even index → high nibble, odd → low; two's-complement nibbles (:133-141,149-153)
    w = np.array([[7.0, -7.0, 3.5, -3.5, 0.0, 1.0]], np.float32)
    q, s = orc.int4_quantize(w, 64)
    assert s[0] == np.float32(1.0)
    # 3.5 rounds away from zero to 4, −3.5 to −4
    assert q.tolist() == [(7 << 4) | (0x10 - 7), (4 << 4) | (0x10 - 4), (0 << 4) | 1]


@pytest.mark.parametrize("rows,cols", [(3, 5), (16, 64), (7, 257), (64, 4096)])
def test_int8_matches_numpy_restatement(rows, cols):
    w = orc.normal_f32(rows * cols, 11, rows * 1000 + cols, 0.02).reshape(rows, cols)
    w[0, :] = 0.0                       # all-zero row: scale 1.0
    if cols > 4:
        w[1, 0], w[1, 1] = 2.0, 1.0     # exact .5 tie: 1·(127/2) = 63.5
        w[1, 2:] *= 0.1
    q, s = orc.int8_quantize(w)
    qn, sn = _np_int8_quantize(w)
    assert np.array_equal(s.view(np.uint32), sn.view(np.uint32))
    assert np.array_equal(q, qn)
    assert s[0] == 1.0 and not q[0].any()


@pytest.mark.parametrize("rows,cols,block", [(1, 64, 64), (4, 128, 32), (3, 50, 32), (5, 33, 64), (2, 7, 4), (8, 4096, 32)])
def test_int4_matches_numpy_restatement(rows, cols, block):
    w = orc.normal_f32(rows * cols, 12, rows * 1000 + cols + block, 0.02).reshape(rows, cols)
    w.ravel()[:min(block, w.size)] = 0.0
    q, s = orc.int4_quantize(w, block)
    qn, sn = _np_int4_quantize(w, block)
    assert np.array_equal(s.view(np.uint32), sn.view(np.uint32))
    assert np.array_equal(q, qn)
    deq = orc.int4_dequantize(q, s, w.size, block)
    assert np.max(np.abs(deq - w.ravel())) <= np.max(s) * 0.5 + 1e-7


# ── RoPE / YaRN ──────────────────────────────────────────────────────────────────
def test_yarn_band_behaviour_olmo3():
    # crates/atlas-model/src/lib.rs:3393-3460
    hd, theta, factor, orig, bf, bs = 128, 500000.0, 8.0, 8192, 32.0, 1.0
    yarn = dict(factor=factor, orig_max_pos=orig, beta_fast=bf, beta_slow=bs)
    ycos, _ = orc.rope_tables(hd, 256, theta, yarn)
    scos, _ = orc.rope_tables(hd, 256, theta)
    two_pi = np.float32(2.0) * np.float32(math.pi)
    low = np.float32(orig) / (two_pi * np.float32(bs))
    high = np.float32(orig) / (two_pi * np.float32(bf))
    n_un = n_sc = 0
    pos = 100
    for i in range(hd // 2):
        base = np.float32(1.0) / np.float32(np.power(np.float32(theta), np.float32(2.0 * i / hd), dtype=np.float32))
        wl = two_pi / base
        if wl < high:
            assert abs(ycos[pos, i] - scos[pos, i]) < 1e-4
            n_un += 1
        elif wl > low:
            assert abs(ycos[pos, i] - math.cos(pos * float(base) / factor)) < 1e-4
            n_sc += 1
        assert np.isfinite(ycos[pos, i])
    assert n_un > 0 and n_sc > 0


def test_olmo3_layer_pattern_helper():
    # crates/atlas-model/src/lib.rs:3534-3575: three sliding layers then one full, ×8
    pattern = [0 if (i % 4) == 3 else 1 for i in range(32)]
    assert sum(pattern) == 24 and [i for i, s in enumerate(pattern) if not s] == list(range(3, 32, 4))


# ── tiny random-init model (OlmoModel::new with ModelConfig::tiny) ───────────────
TINY = dict(vocab_size=256, d_model=64, n_layers=2, n_heads=4, n_kv_heads=2, ffn_hidden=128,
            max_seq_len=128, rope_theta=10000.0, rms_norm_eps=1e-5, post_norm=0)


def _tiny(**over):
    cfg = dict(TINY); cfg.update(over)
    sliding = over.pop("_sliding", None) if "_sliding" in over else None
    m = orc.OracleModel(cfg, sliding)
    m.init_reference_random()
    return m


def test_pseudo_randn_range_and_determinism():
    # crates/atlas-model/src/lib.rs:2725-2732
    a = orc.pseudo_randn(1000, 7)
    assert np.array_equal(a, orc.pseudo_randn(1000, 7))
    assert a.min() >= -1.0 and a.max() <= 1.0 and abs(float(a.mean())) < 0.1
    # first value by hand: state = (7+12345)·6364136223846793005 + 1442695040888963407 mod 2^64
    st = ((7 + 12345) * 6364136223846793005 + 1442695040888963407) % (1 << 64)
    assert a[0] == np.float32(np.float32(np.float32(st >> 33) / np.float32(1 << 31)) * np.float32(2.0) - np.float32(1.0))


def test_reset_is_deterministic():
    # crates/atlas-model/src/lib.rs:3108-3123
    m = _tiny()
    m.forward_one(0); m.forward_one(1)
    m.reset(); l1 = m.forward_one(0)
    m.reset(); l2 = m.forward_one(0)
    assert np.max(np.abs(l1 - l2)) < 1e-6 and np.all(np.isfinite(l1)) and l1.size == 256


def test_swa_window_isolates_prior_tokens():
    # crates/atlas-model/src/lib.rs:3467-3493 and the counter-test :3497-3517
    def run(prefix, sliding):
        cfg = dict(TINY)
        if sliding:
            cfg["sliding_window"] = 1
        m = orc.OracleModel(cfg, [1, 1] if sliding else None)
        m.init_reference_random()
        for t in prefix:
            m.forward_one(t)
        return m.forward_one(30)
    assert np.max(np.abs(run([10, 20], True) - run([99, 77], True))) < 1e-5
    assert np.max(np.abs(run([10, 20], False) - run([99, 77], False))) > 1e-5


def test_generate_eos_and_suppress_semantics():
    # crates/atlas-model/src/lib.rs:2798-2828 (EOS not emitted) and :3000-3022 (suppress list)
    m = _tiny()
    full = m.generate_greedy([0, 1], 10)
    assert full.size == 10 and np.all(full < 256)
    cfg = dict(TINY, eos_token_id=int(full[0]))
    m2 = orc.OracleModel(cfg); m2.init_reference_random()
    assert m2.generate_greedy([0, 1], 10).size == 0
    # first occurrence of full[4] decides where generation stops
    first = int(np.where(full == full[4])[0][0])
    cfg = dict(TINY, eos_token_id=int(full[4]))
    m3 = orc.OracleModel(cfg); m3.init_reference_random()
    stopped = m3.generate_greedy([0, 1], 10)
    assert stopped.size == first and np.array_equal(stopped, full[:first])
    # extra stop tokens behave like EOS (:1718)
    m4 = _tiny()
    assert np.array_equal(m4.generate_greedy([0, 1], 10, stops=[int(full[4])]), full[:first])
    # suppressing the first greedy token changes it
    m5 = _tiny()
    t2 = m5.generate_greedy([0, 1], 5, suppress=[int(full[0])])
    assert t2[0] != full[0]
    # greedy decoding is repeatable across reset (crates/atlas-infer/src/engine.rs:361-369)
    assert np.array_equal(m.generate_greedy([0, 1], 10), full)


def test_empty_prompt_uses_zero_logits():
    # generate_with_sampling starts from vec![0.0; vocab] (:1609): with no prompt the first
    # token is argmax of all-equal logits, i.e. the last index.
    m = _tiny()
    out = m.generate_greedy([], 2)
    assert out[0] == 255


def test_synthetic_generator_statistics():
    z = orc.normal_f32(200000, 0, 1, 1.0)
    assert abs(float(z.mean())) < 0.01 and abs(float(z.std()) - 1.0) < 0.01
    assert np.abs(z).max() < 6.0
    assert np.array_equal(z[:100], orc.normal_f32(100, 0, 1, 1.0))
    assert not np.array_equal(z[:100], orc.normal_f32(100, 0, 2, 1.0))
    b = orc.normal_bf16(1000, 3, 4, 0.02)
    assert np.array_equal(b, orc.f32_to_bf16_rne(orc.normal_f32(1000, 3, 4, 0.02)))


# ── sampling: the reference's own unit expectations (crates/atlas-model/src/lib.rs:2846-2990) plus an
#    independent numpy restatement of every primitive ─────────────────────────────────────────────
def test_rng_xorshift_stream():
    # :2846-2866: values in range and not constant; and the exact stream, recomputed here with
    # Python integers: state = seed | 1; x ^= x << 13; x ^= x >> 7; x ^= x << 17 (64-bit);
    # value = (x >> 33) as f32 / 2^31
    rng = orc.Rng(42)
    x = 42 | 1
    seen = set()
    for _ in range(1000):
        x ^= (x << 13) & 0xFFFFFFFFFFFFFFFF
        x ^= x >> 7
        x ^= (x << 17) & 0xFFFFFFFFFFFFFFFF
        want = np.float32(np.float32(x >> 33) / np.float32(2 ** 31))
        v = rng.next_f32()
        assert v == float(want) and 0.0 <= v < 2.0
        seen.add(v)
    assert len(seen) > 900
    assert orc.Rng(0).state.value == 1                      # from_seed avoids the all-zero state


def test_sample_from_probs_basic():
    # :2869-2876
    probs = [0.1, 0.2, 0.3, 0.4]
    assert [orc.sample_from_probs(probs, r) for r in (0.0, 0.05, 0.15, 0.35, 0.95)] == [0, 0, 1, 2, 3]
    assert orc.sample_from_probs(probs, 1.5) == 3            # past the total: the last index (:2716)


def test_penalties_known_answers():
    # :2881-2900 repetition, :2961-2981 frequency and presence
    l = orc.apply_repetition_penalty([1.0, 2.0, 3.0, -1.0], [1, 3], 1.5)
    assert abs(l[1] - 1.333) < 0.01 and abs(l[3] + 1.5) < 0.01 and l[0] == 1.0 and l[2] == 3.0
    assert l[1] == np.float32(2.0) / np.float32(1.5) and l[3] == np.float32(-1.5)
    orig = [1.0, 2.0, 3.0, -1.0]
    assert orc.apply_repetition_penalty(orig, [0, 1, 2, 3], 1.0).tolist() == orig
    # a token seen twice in the window is penalised twice (:2582 loops over occurrences)
    assert orc.apply_repetition_penalty([4.0], [0, 0], 2.0)[0] == 1.0
    l = orc.apply_frequency_penalty([1.0, 2.0, 3.0], [1, 2, 1, 1], 0.5)            # counts (1,3), (2,1)
    assert abs(l[1] - 0.5) < 0.01 and abs(l[2] - 2.5) < 0.01 and l[0] == 1.0
    l = orc.apply_presence_penalty([1.0, 2.0, 3.0], [2, 0, 2], 0.5)                # seen {0, 2}
    assert abs(l[0] - 0.5) < 0.01 and l[1] == 2.0 and abs(l[2] - 2.5) < 0.01
    assert orc.apply_presence_penalty([1.0], [5, 9], 0.5)[0] == 1.0                # ids past the vocabulary are skipped


def test_top_k_top_p_min_p_known_answers():
    ninf = -np.inf
    # :2926-2944
    l = orc.apply_top_k([1.0, 5.0, 3.0, 2.0, 4.0], 3)
    assert l.tolist() == [ninf, 5.0, 3.0, ninf, 4.0]
    orig = [1.0, 5.0, 3.0, 2.0, 4.0]
    assert orc.apply_top_k(orig, 0).tolist() == orig and orc.apply_top_k(orig, 5).tolist() == orig
    # ties at the threshold: exactly k survive, the first ones in index order (:2670-2684)
    assert orc.apply_top_k([2.0, 7.0, 2.0, 2.0, 1.0], 3).tolist() == [2.0, 7.0, 2.0, ninf, ninf]
    # :2903-2923
    l = orc.apply_top_p([-1.0, 0.0, 0.7, 1.7], 0.5)
    assert l[3] > ninf and int(np.sum(l == ninf)) >= 1
    assert l.tolist() == [ninf, ninf, ninf, np.float32(1.7)]                       # p(token 3) ≈ 0.60 ≥ 0.5 alone
    assert np.all(orc.apply_top_p([1.0, 2.0, 3.0, 4.0], 1.0) > ninf)
    # :2947-2958
    l = orc.apply_min_p([10.0, 0.0, -5.0, 9.0], 0.1)
    assert l.tolist() == [10.0, ninf, ninf, 9.0]


def _np_pipeline(logits, cfg, step, history, suppress, r):
    """numpy restatement of the sampling branch (:1650-1710), written from the reference text
    independently of the C oracle: f32 throughout, sequential sums."""
    f = np.float32
    l = np.array(logits, dtype=np.float32)
    if step == 0:
        for t in suppress:
            if t < l.size:
                l[t] = -np.inf
    if cfg.repetition_penalty != 1.0 and len(history):
        for t in history[max(0, len(history) - cfg.repetition_window):]:
            if t < l.size:
                l[t] = l[t] / f(cfg.repetition_penalty) if l[t] > 0 else l[t] * f(cfg.repetition_penalty)
    if cfg.frequency_penalty != 0.0 and len(history):
        for t in dict.fromkeys(history):
            if t < l.size:
                l[t] = l[t] - f(cfg.frequency_penalty) * f(list(history).count(t))
    if cfg.presence_penalty != 0.0 and len(history):
        for t in sorted(set(history)):
            if t < l.size:
                l[t] = l[t] - f(cfg.presence_penalty)
    l = l / f(cfg.temperature)
    k = cfg.top_k
    if 0 < k < l.size:
        thr = np.sort(l)[::-1][k - 1]
        if np.sum(l >= thr) <= k:
            l[l < thr] = -np.inf
        else:
            need = k - int(np.sum(l > thr))
            ties = np.flatnonzero(l == thr)
            l[l < thr] = -np.inf
            l[ties[need:]] = -np.inf

    def seqsum(a):
        s = f(0.0)
        for v in a:
            s = f(s + v)
        return s
    if cfg.top_p < 1.0:
        e = np.exp((l - l.max()).astype(np.float32)).astype(np.float32)
        s = seqsum(e)
        if s > 0:
            pr = (e / s).astype(np.float32)
            order = sorted(range(l.size), key=lambda i: (-pr[i], i))
            cum, cut = f(0.0), l.size
            for j, i in enumerate(order):
                cum = f(cum + pr[i])
                if cum >= f(cfg.top_p):
                    cut = j + 1
                    break
            for i in order[cut:]:
                l[i] = -np.inf
    if cfg.min_p > 0.0:
        l[l < f(l.max() + np.log(f(cfg.min_p)))] = -np.inf
    e = np.exp((l - l.max()).astype(np.float32)).astype(np.float32)
    pr = (e * f(f(1.0) / seqsum(e))).astype(np.float32)
    cum = f(0.0)
    for i, p in enumerate(pr):
        cum = f(cum + p)
        if f(r) < cum:
            return i, pr
    return l.size - 1, pr


@pytest.mark.parametrize("case", ["olmo3", "plain", "penalties", "top_p_only", "min_p_only", "top_k_ties"])
def test_sampling_pipeline_matches_numpy_restatement(case):
    cfgs = {"olmo3": orc.sampling(0.6, 1.15, 256, 0.0, 0.0, 0.95, 50, 0.05),        # SamplingConfig::olmo3 (:1278-1294)
            "plain": orc.sampling(1.0), "penalties": orc.sampling(0.8, 1.3, 4, 0.2, 0.4, 1.0, 0, 0.0),
            "top_p_only": orc.sampling(1.2, top_p=0.7), "min_p_only": orc.sampling(0.9, min_p=0.2),
            "top_k_ties": orc.sampling(1.0, top_k=5)}
    cfg = cfgs[case]
    n = 997
    hist = [int(t) for t in orc.uniform_u32(40, 77, 1, 60)]
    for trial in range(25):
        logits = orc.normal_f32(n, 77, 10 + trial, 2.0)
        if case == "top_k_ties":
            logits = np.round(logits)                        # many exact ties around the k-th value
        rng = orc.Rng(1000 + trial)
        probe = orc.Rng(1000 + trial)
        r = probe.next_f32()
        step = 0 if trial % 5 == 0 else trial
        tok, probs = orc.sample_token(logits, cfg, step, hist[:trial * 2], rng, suppress=[3, 14023], want_probs=True)
        want_tok, want_probs = _np_pipeline(logits, cfg, step, hist[:trial * 2], [3, 14023], r)
        assert rng.state.value == probe.state.value          # exactly one draw
        # the survivor set is bit-exact; probabilities agree to a few ulp (numpy's exp vs libm's expf)
        assert np.array_equal(probs > 0, want_probs > 0)
        assert np.max(np.abs(probs - want_probs)) <= 1e-6
        assert tok == want_tok


def test_sampling_config_defaults_and_olmo3():
    # :2984-3010
    import atlas_b200 as ab
    c = ab.SamplingConfig()
    assert (c.repetition_penalty, c.top_p, c.top_k, c.min_p, c.temperature) == (1.0, 1.0, 0, 0.0, 1.0)
    c = ab.SamplingConfig.olmo3()
    assert abs(c.temperature - 0.6) < 0.01 and abs(c.repetition_penalty - 1.15) < 0.01 and abs(c.top_p - 0.95) < 0.01
    assert c.top_k == 50 and abs(c.min_p - 0.05) < 0.01 and c.repetition_window == 256 and c.frequency_penalty == 0.0
    assert c.suppress_initial_tokens == [14023]


def test_greedy_branch_of_sample_token_equals_generate_greedy():
    m = _tiny()
    want = m.generate_greedy([0, 1], 8, rep_penalty=1.3, rep_window=4)
    got = m.generate_sampling([0, 1], 8, orc.sampling(0.0, 1.3, 4), seed=5)
    assert np.array_equal(want, got)
    a = m.generate_sampling([0, 1], 12, orc.sampling(1.0, top_k=20), seed=5)
    b = m.generate_sampling([0, 1], 12, orc.sampling(1.0, top_k=20), seed=5)
    c = m.generate_sampling([0, 1], 12, orc.sampling(1.0, top_k=20), seed=6)
    assert np.array_equal(a, b) and not np.array_equal(a, c) and a.size == 12


def test_bf16_hi_lo_split_keeps_17_bits():
    """The tcgen05 products feed f32 values (tokens; dequantised int4 weights) to the tensor cores as two bf16 parts,
    hi = rne(v) and lo = rne(v − hi).  The parts add up to v within 2⁻¹⁷ relative — the bound the kernels' comments and
    the 2e-5 / 1e-4 tolerances of their GPU tests rest on."""
    rng = np.random.default_rng(7)
    v = (rng.standard_normal(400_000) * rng.choice([1e-3, 1.0, 37.5], 400_000)).astype(np.float32)
    hi = orc.bf16_to_f32(orc.f32_to_bf16_rne(v)).astype(np.float32)
    lo = orc.bf16_to_f32(orc.f32_to_bf16_rne((v - hi).astype(np.float32))).astype(np.float32)
    err = np.abs(v.astype(np.float64) - (hi.astype(np.float64) + lo.astype(np.float64))) / np.abs(v)
    assert err.max() <= 2.0 ** -16.9


def test_three_base_254_digits_keep_the_token_to_1e7_of_its_maximum():
    """The int8 tcgen05 product sees a token as three int8 digit planes in base 254 with one scale per token:
    x ≈ s · (q1 + q2/254 + q3/254²), s = max|x| / 127.  The same f32 arithmetic as the kernel, restated in numpy:
    every digit fits an int8 and the reconstruction is within 1.2e-7 · max|x| of x (half a third digit, 6.1e-8 · max|x|,
    plus the f32 rounding of x · 127 / max|x|, 6e-8 · |x|)."""
    rng = np.random.default_rng(11)
    x = rng.standard_normal(11008).astype(np.float32)
    x[3670] = np.float32(37.5)
    mx = np.float32(np.max(np.abs(x)))
    inv = np.float32(127.0) / mx
    t = np.clip(x * inv, np.float32(-127.0), np.float32(127.0)).astype(np.float32)
    q1 = np.rint(t).astype(np.float32)
    rr = ((t - q1) * np.float32(254.0)).astype(np.float32)
    q2 = np.rint(rr).astype(np.float32)
    q3 = np.rint(((rr - q2) * np.float32(254.0)).astype(np.float32)).astype(np.float32)
    for q in (q1, q2, q3):
        assert np.all(np.abs(q) <= 127)
    s = np.float64(mx) / 127.0
    rec = s * (q1.astype(np.float64) + q2.astype(np.float64) / 254.0 + q3.astype(np.float64) / 254.0 ** 2)
    assert np.max(np.abs(rec - x.astype(np.float64))) <= 1.2e-7 * float(mx)


def test_two_base_254_digits_per_group_of_32_keep_the_input_to_1_6e5_of_the_group_maximum():
    """The single-column int8 / int4 GEMV sees its input through TWO int8 digits in base 254 with one scale per group
    of 32 elements (x ≈ s · (q1 + q2/254), s = max|group| / 127): half a second digit is 1.55e-5 of the group's
    maximum, which is what the 1e-4 linearity bound of the GPU tests allows for."""
    rng = np.random.default_rng(12)
    x = rng.standard_normal(4096).astype(np.float32).reshape(-1, 32)
    x[5, 7] = np.float32(37.5)
    mx = np.max(np.abs(x), axis=1, keepdims=True).astype(np.float32)
    t = np.clip(x * (np.float32(127.0) / mx), np.float32(-127.0), np.float32(127.0)).astype(np.float32)
    q1 = np.rint(t).astype(np.float32)
    q2 = np.rint(((t - q1) * np.float32(254.0)).astype(np.float32)).astype(np.float32)
    assert np.all(np.abs(q1) <= 127) and np.all(np.abs(q2) <= 127)
    rec = (mx.astype(np.float64) / 127.0) * (q1.astype(np.float64) + q2.astype(np.float64) / 254.0)
    assert np.max(np.abs(rec - x.astype(np.float64)) / mx.astype(np.float64)) <= 1.6e-5
