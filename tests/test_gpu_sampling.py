"""GPU: the sampling pipeline on the device (atlasx_sample_token, atlasx_model_generate_sampling)
against the CPU oracle's restatement of generate_with_sampling
(crates/atlas-model/src/lib.rs:1599-1732, 2581-2717).  Bar: XorShift64 stream, surviving token set
and selected tokens identical; probabilities within 1e-6 (the last bits of expf)."""
import os

import numpy as np
import pytest

from oracle import orc
import helpers

pytestmark = pytest.mark.gpu

CASES = {
    "olmo3": dict(temperature=0.6, repetition_penalty=1.15, repetition_window=256, top_p=0.95, top_k=50, min_p=0.05),
    "plain": dict(temperature=1.0),
    "penalties": dict(temperature=0.8, repetition_penalty=1.3, repetition_window=4, frequency_penalty=0.2, presence_penalty=0.4),
    "top_p_only": dict(temperature=1.2, top_p=0.7),
    "min_p_only": dict(temperature=0.9, min_p=0.2),
    "top_k_ties": dict(temperature=1.0, top_k=5),
    "top_k_1": dict(temperature=0.7, top_k=1),
    "window_0": dict(temperature=1.0, repetition_penalty=1.5, repetition_window=0, presence_penalty=0.3),
}


@pytest.fixture(scope="module")
def ab():
    import atlas_b200
    orc.set_threads(os.cpu_count() or 1)
    return atlas_b200


def _run_case(ab, name, n, trials, seed0):
    kw = CASES[name]
    cfg_gpu = ab.SamplingConfig(suppress_initial_tokens=[3, 14023], **kw)
    cfg_cpu = orc.sampling(**kw)
    ctx = ab.Context.default()
    probs_dev = ctx.malloc(4 * n)
    hist_all = [int(t) for t in orc.uniform_u32(400, seed0, 1, min(n, 60))]
    for trial in range(trials):
        logits = orc.normal_f32(n, seed0, 10 + trial, 2.0)
        if name == "top_k_ties":
            logits = np.round(logits)
        if trial == 1:
            logits[5:9] = -np.inf                                  # masked entries in the input
        hist = hist_all[:trial * 7]
        step = 0 if trial % 3 == 0 else trial
        rng = orc.Rng(7000 + trial)
        state0 = rng.state.value
        want_tok, want_probs = orc.sample_token(logits, cfg_cpu, step, hist, rng, suppress=[3, 14023], want_probs=True)
        dl = ctx.to_device(logits)
        tok, state1 = ab.sample_token(dl, n, cfg_gpu, step, hist, state0, ctx=ctx, probs_dev=probs_dev)
        probs = ctx.download(probs_dev, (n,), np.float32)
        ctx.free(dl)
        assert state1 == rng.state.value, (name, trial)            # one draw, same stream
        assert np.array_equal(probs > 0, want_probs > 0), (name, trial)
        assert np.max(np.abs(probs - want_probs)) <= 1e-6, (name, trial)
        assert tok == want_tok, (name, trial)
    ctx.free(probs_dev)


@pytest.mark.parametrize("name", sorted(CASES))
def test_pipeline_small_vocabulary(ab, name):
    _run_case(ab, name, 997, 24, 81)


@pytest.mark.parametrize("name", ["olmo3", "plain", "top_p_only", "penalties"])
def test_pipeline_full_vocabulary(ab, name):
    """The benchmark model's vocabulary (100278); `plain` and `top_p_only` keep every token, so the
    sort and the sequential sums run over the whole vocabulary."""
    _run_case(ab, name, 100278, 4, 82)


def test_all_but_a_few_logits_masked_and_fallback_to_last_index(ab):
    n = 300
    ctx = ab.Context.default()
    cfg_gpu, cfg_cpu = ab.SamplingConfig(temperature=1.0, top_k=50), orc.sampling(1.0, top_k=50)
    logits = np.full(n, -np.inf, np.float32)
    logits[[7, 150, 299]] = [1.0, 2.0, 0.5]                       # fewer finite logits than k
    for seed in range(20):
        rng = orc.Rng(seed)
        s0 = rng.state.value
        want = orc.sample_token(logits, cfg_cpu, 5, [], rng)
        dl = ctx.to_device(logits)
        tok, s1 = ab.sample_token(dl, n, cfg_gpu, 5, [], s0, ctx=ctx)
        ctx.free(dl)
        assert tok == want and tok in (7, 150, 299) and s1 == rng.state.value


@pytest.mark.parametrize("name", ["olmo3", "penalties", "plain"])
def test_model_generation_with_sampling_matches_oracle(ab, name):
    """generate_with_sampling end to end on a small model: same seed, same tokens as the CPU oracle
    (logits agree to 1e-4, so a draw would have to land within that of a boundary to differ)."""
    cfg = dict(helpers.SMALL_SWA)
    w = helpers.synth_weights(cfg, seed=85, norm_jitter=0.1, std=0.08)
    prompt = orc.uniform_u32(9, 85, 1, cfg["vocab_size"])
    kw = CASES[name]
    m = helpers.cuda_model(cfg, w, helpers.SMALL_SWA_LAYERS, kv_dtype=ab.F32)
    o = helpers.oracle_model(cfg, w, helpers.SMALL_SWA_LAYERS)
    sup = [int(o.generate_greedy(prompt, 1)[0])]
    for seed in (11, 12, 13):
        got = m.generate_with_sampling(prompt, 30, ab.SamplingConfig(suppress_initial_tokens=sup, **kw), seed=seed)
        want = o.generate_sampling(prompt, 30, orc.sampling(**kw), seed, suppress=sup).tolist()
        assert got == want, (name, seed)
        assert len(got) == 30 and got[0] != sup[0]
    assert ab.Context.default().poll_device_error() == 0


def test_olmo3_defaults_through_the_engine_and_stop_tokens(ab):
    """SamplingConfig::olmo3() — the API's default — runs on the GPU path through InferEngine.generate;
    seeds repeat, the clock seed varies (the reference's own expectation, :2831-2843); EOS and stop
    tokens end a sampled run before being emitted; temperature 0 still takes the greedy branch."""
    cfg = dict(helpers.SMALL_SWA, vocab_size=20000)
    w = helpers.synth_weights(cfg, seed=86, norm_jitter=0.1, std=0.05)
    prompt = orc.uniform_u32(6, 86, 1, cfg["vocab_size"])
    m = helpers.cuda_model(cfg, w, helpers.SMALL_SWA_LAYERS, kv_dtype=ab.BF16)
    eng = ab.InferEngine(m)
    toks, deposits = eng.generate(prompt, 20, ab.SamplingConfig.olmo3())
    assert len(toks) == 20 and deposits == [] and all(0 <= t < 20000 for t in toks)
    c = ab.SamplingConfig(temperature=1.0)
    a = m.generate_with_sampling(prompt, 20, c, seed=5)
    assert a == m.generate_with_sampling(prompt, 20, c, seed=5)
    assert a != m.generate_with_sampling(prompt, 20, c, seed=6)
    assert m.generate_with_sampling(prompt, 20, c) != m.generate_with_sampling(prompt, 20, c)       # clock-seeded
    m.extra_stop_tokens = [a[7]]
    first = a.index(a[7])
    assert m.generate_with_sampling(prompt, 20, c, seed=5) == a[:first]
    m.extra_stop_tokens = []
    m.eos_token_id = a[0]
    assert m.generate_with_sampling(prompt, 20, c, seed=5) == []
    m.eos_token_id = None
    greedy = m.generate(prompt, 10, 0.0)
    assert m.generate_with_sampling(prompt, 10, ab.SamplingConfig(temperature=0.0)) == greedy
    assert m.generate_with_sampling([], 3, c, seed=9) == m.generate_with_sampling([], 3, c, seed=9)
