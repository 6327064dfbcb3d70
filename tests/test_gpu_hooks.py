"""GPU: the per-layer hook (StigmergicHook) on the GPU path.  Semantics from the reference:
on_layer(layer_idx, hidden) after every layer of every forward, prompt included
(forward_one_gpu_hooked, crates/atlas-model/src/lib.rs:1524-1557); one deposit per generated token
with the sum of the non-negative deltas and the number of layers that returned one
(generate_with_sampling_hooked :1745-1846; accumulate, crates/atlas-infer/src/hook.rs:60-67).
The hidden states the hook sees are checked against the CPU oracle layer by layer."""
import os

import numpy as np
import pytest

from oracle import orc
import helpers

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ab():
    import atlas_b200
    orc.set_threads(os.cpu_count() or 1)
    return atlas_b200


class Recorder:
    def __init__(self, n_layers):
        self.calls, self.n_layers = [], n_layers

    def on_layer(self, layer_idx, hidden):
        self.calls.append((layer_idx, np.array(hidden, copy=True)))
        if layer_idx % 2 == 1:
            return None                                   # odd layers do not fire
        return 0.5 * layer_idx - 0.6                      # layer 0: −0.6 (counts as 0), layer 2: +0.4


@pytest.mark.parametrize("fmt_kv", ["f32", "bf16"])
def test_hook_sees_every_layer_of_every_forward_and_deposits_add_up(ab, fmt_kv):
    cfg = dict(helpers.SMALL_SWA)
    L, d = cfg["n_layers"], cfg["d_model"]
    w = helpers.synth_weights(cfg, seed=91, norm_jitter=0.1)
    prompt = orc.uniform_u32(7, 91, 1, cfg["vocab_size"])
    kv = ab.F32 if fmt_kv == "f32" else ab.BF16
    m = helpers.cuda_model(cfg, w, helpers.SMALL_SWA_LAYERS, kv_dtype=kv)
    m.set_prefill(16)                                      # a hook turns chunked ingestion off again
    plain = m.generate(prompt, 9, 0.0)
    rec = Recorder(L)
    eng = ab.InferEngine(m).with_hook(rec)
    assert eng.has_hook()
    toks, deposits = eng.generate(prompt, 9, ab.SamplingConfig(temperature=0.0))
    assert toks == plain                                   # the tap does not change the computation
    assert len(rec.calls) == (len(prompt) + len(toks)) * L
    assert [c[0] for c in rec.calls] == list(range(L)) * (len(prompt) + len(toks))
    # every hidden state against the oracle, forward by forward, layer by layer
    o = helpers.oracle_model(cfg, w, helpers.SMALL_SWA_LAYERS, kv_round_bf16=(fmt_kv == "bf16"))
    tol = 1e-4 if fmt_kv == "f32" else 5e-3
    for i, t in enumerate(list(prompt) + toks):
        _, hid = o.forward_one(int(t), want_hidden=True)
        for l in range(L):
            got = rec.calls[i * L + l][1]
            assert got.shape == (d,) and np.max(np.abs(got - hid[l])) <= tol, (i, l)
    want_delta = sum(max(0.5 * l - 0.6, 0.0) for l in range(0, L, 2))
    assert [dp.token_id for dp in deposits] == toks
    assert all(dp.layers_fired == (L + 1) // 2 for dp in deposits)
    assert all(abs(dp.total_delta - want_delta) < 1e-6 for dp in deposits)
    # forward_one with the hook attached: L calls before it returns
    rec.calls.clear()
    lg = m.forward_one_gpu(3)
    assert len(rec.calls) == L and np.max(np.abs(rec.calls[-1][1] - m.hidden())) == 0.0
    assert np.max(np.abs(m.hidden(layer=1) - rec.calls[1][1])) == 0.0 and lg.size == cfg["vocab_size"]
    # detached: the zero-overhead path, no deposits
    eng.set_hook(None)
    rec.calls.clear()
    toks2, deposits2 = eng.generate(prompt, 9, ab.SamplingConfig(temperature=0.0))
    assert toks2 == plain and deposits2 == [] and rec.calls == [] and not eng.has_hook()


def test_hook_with_sampling_and_streaming(ab):
    cfg = dict(helpers.SMALL_SWA)
    w = helpers.synth_weights(cfg, seed=92, norm_jitter=0.1, std=0.08)
    prompt = orc.uniform_u32(5, 92, 1, cfg["vocab_size"])
    m = helpers.cuda_model(cfg, w, helpers.SMALL_SWA_LAYERS, kv_dtype=ab.F32)
    sc = ab.SamplingConfig(temperature=0.9, top_k=40, repetition_penalty=1.1)
    plain = m.generate_with_sampling(prompt, 12, sc, seed=4)

    class Norm(ab.StigmergicHook):
        def on_layer(self, layer_idx, hidden):
            return float(np.sqrt(np.mean(hidden * hidden))) if layer_idx == 3 else None
    eng = ab.InferEngine(m).with_hook(Norm())
    toks, deposits = eng.generate(prompt, 12, sc, seed=4)
    assert toks == plain and len(deposits) == 12
    assert all(dp.layers_fired == 1 and dp.total_delta > 0 for dp in deposits)
    seen = []
    n = eng.generate_streaming(prompt, 12, sc, lambda tok, dep: (seen.append((tok, dep.token_id)) or len(seen) < 5), seed=4)
    assert n == 5 and seen == [(t, t) for t in plain[:5]]
    # a stop token ends the run; the hooks of the forwards that did run are all delivered
    m.extra_stop_tokens = [plain[6]]
    toks, deposits = eng.generate(prompt, 12, sc, seed=4)
    cut = plain.index(plain[6])
    assert toks == plain[:cut] and [dp.token_id for dp in deposits] == toks


def test_streaming_without_a_hook_stops_the_generation_itself(ab):
    """engine.rs:181-190 / atlas-model :1855-1965: without a hook the tokens arrive while the run is going on, the
    deposit is None, and a false return ends the generation at once — the model has then processed the prompt and
    the tokens before the last one, nothing more."""
    cfg = dict(helpers.SMALL_SWA)
    w = helpers.synth_weights(cfg, seed=93, norm_jitter=0.1, std=0.08)
    prompt = orc.uniform_u32(6, 93, 1, cfg["vocab_size"])
    m = helpers.cuda_model(cfg, w, helpers.SMALL_SWA_LAYERS, kv_dtype=ab.F32)
    for sc, seed in ((ab.SamplingConfig(temperature=0.0), None), (ab.SamplingConfig(temperature=0.8, top_k=50), 7)):
        plain = m.generate_with_sampling(prompt, 10, sc, seed=seed)
        eng = ab.InferEngine(m)
        seen = []
        n = eng.generate_streaming(prompt, 10, sc, lambda tok, dep: (seen.append((tok, dep)) or len(seen) < 4), seed=seed)
        assert n == 4 and seen == [(t, None) for t in plain[:4]]
        assert m.pos == len(prompt) + 3                       # no forward ran for the token that ended the run
        # a callback that never says stop sees the whole run, and the callback is gone afterwards
        seen.clear()
        assert eng.generate_streaming(prompt, 10, sc, lambda tok, dep: seen.append(tok) or True, seed=seed) == len(plain)
        assert seen == plain
        assert m.generate_with_sampling(prompt, 10, sc, seed=seed) == plain
