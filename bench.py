#!/usr/bin/env python
"""Decode benchmark: OLMo-3-7B-architecture BF16 batch-1 greedy decode (BASELINE config 4).

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

A step is one generated token at context ≥ prompt length (default 2048): the whole hot path
(161 weight-streaming GEMVs, 32 attention calls, selection) over 13.77 GB of bf16 weights, so
every step reads far more than the 126 MB L2 and no flush is needed between steps.
Prints ONE JSON line (rank 0).  `value` is device-timed tokens/s with everything resident in
HBM; `e2e` is the same metric through the reference-facing call forward_one_gpu(token) →
host logits → host argmax, with the token upload and the logits download inside the timed
region.  With N > 1 the model is sharded tensor-parallel over N GPUs (one process per GPU,
NCCL all-reduce after o_proj and down): total work is fixed, so scaling is "strong".

--impl reference times the CPU restatement of the reference's forward_one path (oracle/,
OpenMP over output rows, all host threads) on the same model and metric.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import numpy as np  # noqa: E402

METRIC = "olmo3_7b_arch_bf16_bs1_greedy_decode_tokens_per_s"
UNIT = "tok/s"
WORKLOAD = ("configs[3]: OLMo-3-7B arch (32 layers, d 4096, 32 heads x 128, ffn 11008, vocab 100278, "
            "post-norm + QK-norm, SWA 4096 on 24/32 layers, YaRN), bf16 weights N(0,0.02) seed 0, batch 1")
PER_LAYER = [("wq", 10), ("wk", 11), ("wv", 12), ("wo", 13), ("gate", 14), ("up", 15), ("down", 16)]


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            j = json.load(open(p))
            return float(j["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.idx, self.proc, self.lines = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.idx), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": float(max(mx)), "reasons": sorted(reasons), "samples": len(sm)}


# (32 x (100.74 + 33.63 + 180.47 + 90.29) + 821.61) / 129 MB read + 2.64 MB written, from the ncu capture
NCU_GEMV_TRAFFIC_PER_LAUNCH = 109.51e6
PROFILE_LAYERS = 0          # > 0: a truncated model for profiler captures only (--profile-layers)


def model_config(ab, max_seq):
    mc = ab.ModelConfig.olmo3_actual_7b(max_seq_len=max_seq)
    if PROFILE_LAYERS:
        mc.n_layers = PROFILE_LAYERS
        mc.layer_types = mc.layer_types[:PROFILE_LAYERS]
    return mc


WEIGHTS = "bf16"            # --weights int8 | int4: informational runs of the quantised formats
PROMPT_SEED = 3


def build_cuda_model(ab, ctx, max_seq, rank, world):
    """Random-init weights generated on the device from the seeded hash (full tensors, then each
    rank keeps its tensor-parallel slice)."""
    from atlas_b200 import _ffi
    L = _ffi.lib()
    mc = model_config(ab, max_seq)
    fmt = {"bf16": ab.BF16, "int8": ab.INT8, "int4": ab.INT4}[WEIGHTS]
    m = ab.OlmoModel(mc, ctx=ctx, kv_dtype=ab.BF16, weight_format=fmt, int4_block=32, tp_rank=rank, tp_world=world)
    d, f, V = mc.d_model, mc.ffn_hidden, mc.vocab_size
    shapes = {"wq": (d, d), "wk": (d, d), "wv": (d, d), "wo": (d, d), "gate": (f, d), "up": (f, d), "down": (d, f)}
    big = ctx.malloc(V * d * 2)

    def give(layer, which, rows, cols, stream):
        _ffi.check(L.atlasx_fill_normal_bf16(ctx.handle, big, rows * cols, 0, stream, 0, 0.02))
        m.set_tensor(layer, which, big, on_device=True, dtype=ab.BF16)
    give(0, 0, V, d, 1)          # embedding
    give(0, 2, V, d, 2)          # lm_head
    ones = np.ones(d, np.float32)
    m.set_tensor(0, 1, ones)
    for l in range(mc.n_layers):
        for name, tid in PER_LAYER:
            give(l, tid, shapes[name][0], shapes[name][1], 1000 + l * 32 + tid)
        for tid in (17, 18, 19, 20):
            m.set_tensor(l, tid, ones)
    ctx.free(big)
    m.init_gpu_resources()
    return m, mc


def cpu_reference_model(n_layers, max_seq):
    """The oracle's model with the same seeded weights (bf16 bits in host memory)."""
    from oracle import orc
    cfg = dict(vocab_size=100278, d_model=4096, n_layers=n_layers, n_heads=32, n_kv_heads=32, ffn_hidden=11008,
               max_seq_len=max_seq, rope_theta=500000.0, rms_norm_eps=1e-6, sliding_window=4096, rope_scaling=1,
               yarn_factor=8.0, yarn_orig_max_pos=8192, yarn_attn_factor=1.2079441541679836,
               yarn_beta_fast=32.0, yarn_beta_slow=1.0, post_norm=1)
    d, f, V = 4096, 11008, 100278
    m = orc.OracleModel(cfg, [0 if i % 4 == 3 else 1 for i in range(n_layers)])
    shapes = {"wq": (d, d), "wk": (d, d), "wv": (d, d), "wo": (d, d), "gate": (f, d), "up": (f, d), "down": (d, f)}
    lm = orc.normal_bf16(V * d, 0, 2, 0.02).reshape(V, d)
    m.set_tensor(0, orc.T_LM_HEAD, lm)
    if n_layers == 32:
        m.set_tensor(0, orc.T_EMBED, orc.normal_bf16(V * d, 0, 1, 0.02).reshape(V, d))
    else:
        m.set_tensor(0, orc.T_EMBED, lm)       # bounded sample: any embedding row will do
    ones = np.ones(d, np.float32)
    for l in range(n_layers):
        for name, tid in PER_LAYER:
            r, c = shapes[name]
            m.set_tensor(l, tid, orc.normal_bf16(r * c, 0, 1000 + l * 32 + tid, 0.02).reshape(r, c))
        m.set_tensor(l, orc.T_Q_NORM, ones); m.set_tensor(l, orc.T_K_NORM, ones)
    return m


def cpu_baseline_sample(context=2049):
    """Bounded sample for the default run: one layer of the model plus lm_head through the
    oracle's forward_one at the benchmark's context length, all host threads; tokens/s
    extrapolated to 32 layers."""
    from oracle import orc
    cores = os.cpu_count() or 1
    orc.set_threads(cores)
    m = cpu_reference_model(1, context + 16)
    m.seed_context(context)                                 # cache rows below `context` hold seeded values
    m.forward_one(1)                                        # warm-up
    t0 = time.perf_counter(); n = 3
    for i in range(n):
        m.forward_one(2 + i)
    t_tok = (time.perf_counter() - t0) / n                  # 1 layer + head
    lm = m._keep[0]
    x = orc.normal_f32(4096, 1, 1, 1.0)
    orc.linear(lm, x)
    t0 = time.perf_counter()
    for i in range(n):
        orc.linear(lm, x)
    t_head = (time.perf_counter() - t0) / n
    t_layer = max(t_tok - t_head, 1e-9)
    full = 32 * t_layer + t_head
    return {"value": 1.0 / full, "unit": UNIT, "cores": cores, "kind": "port",
            "sample": "oracle forward_one on 1 of 32 layers + lm_head at pos %d.., %d tokens; per-token time = 32*layer + head = %.3f s"
                      % (context + 1, n, full)}


def ref_gpu_sample(ab, ctx, context, n_tok=8):
    """Informational: the reference's OWN CUDA kernels (kernels/matmul.cu compiled unchanged into
    oracle/_ref) replaying forward_one_gpu's launch sequence for the same model on this GPU, at the
    benchmark's context length.  Kernels only: the Rust host's per-op allocations are not included, so this
    is an upper bound on what the reference reaches here.  None when the checker library is absent."""
    import ctypes as C
    from oracle import orc
    from atlas_b200 import _ffi
    if not os.path.exists(orc.REF_SO):
        return None
    R = C.CDLL(orc.REF_SO)
    vp, ci, cf = C.c_void_p, C.c_int, C.c_float
    R.refgpu_model_new.restype = vp
    R.refgpu_model_new.argtypes = [ci, ci, ci, ci, ci, ci, ci, cf, cf, ci, vp]
    R.refgpu_model_free.argtypes = [vp]; R.refgpu_set_tensor.argtypes = [vp, ci, ci, vp, ci]
    R.refgpu_upload_rope.argtypes = [vp, vp, vp]; R.refgpu_set_pos.argtypes = [vp, ci]
    R.refgpu_forward_one.restype = ci; R.refgpu_forward_one.argtypes = [vp, C.c_uint32, vp]
    R.atlas_sync.argtypes = []
    L = _ffi.lib()
    mc = model_config(ab, context + n_tok + 8)
    d, f, V, hd = mc.d_model, mc.ffn_hidden, mc.vocab_size, 128
    shapes = {"wq": (d, d), "wk": (d, d), "wv": (d, d), "wo": (d, d), "gate": (f, d), "up": (f, d), "down": (d, f)}
    windows = (C.c_int * mc.n_layers)(*[(mc.sliding_window if t == ab.LAYER_SLIDING else 0) for t in mc.layer_types])
    scale = float(np.float32(1.0) / np.sqrt(np.float32(hd)) * np.float32(mc.rope_scaling.attn_factor))
    h = R.refgpu_model_new(V, d, mc.n_layers, mc.n_heads, mc.n_kv_heads, f, mc.max_seq_len, mc.rms_norm_eps, scale, 1, windows)
    bufs = []

    def mat(layer, which, rows, cols, stream):
        p = ctx.malloc(rows * cols * 2); bufs.append(p)
        _ffi.check(L.atlasx_fill_normal_bf16(ctx.handle, p, rows * cols, 0, stream, 0, 0.02))
        assert R.refgpu_set_tensor(h, layer, which, p, 1) == 0
    mat(0, 0, V, d, 1); mat(0, 2, V, d, 2)
    ones = ctx.to_device(np.ones(d, np.float32)); bufs.append(ones)
    assert R.refgpu_set_tensor(h, 0, 1, ones, 0) == 0
    for l in range(mc.n_layers):
        for name, tid in PER_LAYER:
            mat(l, tid, shapes[name][0], shapes[name][1], 1000 + l * 32 + tid)
        for tid in (17, 18, 19, 20):
            assert R.refgpu_set_tensor(h, l, tid, ones, 0) == 0
    cos, sin = ab.rope_tables(hd, mc.max_seq_len, mc.rope_theta, dict(factor=8.0, orig_max_pos=8192, beta_fast=32.0, beta_slow=1.0))
    R.refgpu_upload_rope(h, cos.ctypes.data, sin.ctypes.data)
    ctx.sync()
    R.refgpu_set_pos(h, context)
    tok = 11
    for _ in range(2):
        assert R.refgpu_forward_one(h, tok, None) == 0
    R.atlas_sync()
    t0 = time.perf_counter()
    for _ in range(n_tok):
        assert R.refgpu_forward_one(h, tok, None) == 0
    R.atlas_sync()
    dt = time.perf_counter() - t0
    R.refgpu_model_free(h)
    for p in bufs:
        ctx.free(p)
    return {"value": n_tok / dt, "unit": UNIT, "what": "the reference's kernels (kernels/matmul.cu, unchanged) in forward_one_gpu's launch order "
            "on this GPU, %d tokens from pos %d, host wall clock; no logits download, no per-op allocations" % (n_tok, context + 2)}


def run_reference(args, rank):
    """CPU arm: the restatement of the reference's forward_one (oracle/) on the full model."""
    if rank != 0:
        return
    from oracle import orc
    cores = os.cpu_count() or 1
    orc.set_threads(cores)
    try:
        avail_gb = os.sysconf("SC_AVPHYS_PAGES") * os.sysconf("SC_PAGE_SIZE") / 1e9
    except Exception:
        avail_gb = 0
    steps, warm = args.steps, max(args.warmup, 3)
    pos0 = args.prompt + 1 + warm                            # the position the GPU arm's timed region starts at
    if avail_gb > 40:
        m = cpu_reference_model(32, pos0 + steps + 8)
        m.seed_context(args.prompt + 1)                     # cache rows of the context: seeded values instead of an ingested prompt
        for i in range(warm):
            m.forward_one(7 + i)
        t0 = time.perf_counter()
        tok = 11
        for i in range(steps):
            tok = orc.argmax(m.forward_one(int(tok)))
        dt = time.perf_counter() - t0
        value = steps / dt
        sample = ("full model, %d greedy tokens from pos %d (cache rows below %d seeded) on %d host threads (OpenMP over output rows; "
                  "the reference's forward_one is single-threaded)" % (steps, pos0, args.prompt + 1, cores))
        ms = dt / steps * 1e3
    else:
        b = cpu_baseline_sample(args.prompt + 1)
        value, sample, ms = b["value"], b["sample"] + " (host RAM too small for the full model)", 1e3 / b["value"]
    line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": steps, "warmup": warm,
            "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic", "impl": "reference",
            "config": {"workload": WORKLOAD, "context": "pos %d..%d (context of %d tokens, then warm-up)" % (pos0, pos0 + steps, args.prompt + 1),
                       "kv_cache": "f32 (the reference's format)", "parallelism": "cpu x%d threads" % cores,
                       "l2": "inputs larger than any cache: 13.77 GB of weights stream per step"},
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def print_timeline(m, n_layers, quiet=False):
    """One more captured step with stamps; per launch class (averaged over layers 1..): the time from
    dependency release to the last CTA's end, how early the first CTA started and how late the
    release came relative to the previous launch's end, the input-staging time and the spread of
    CTA end times.  All in microseconds, from %globaltimer."""
    import ctypes as C
    from atlas_b200 import _ffi
    L = _ffi.lib()
    fn = L.atlasx_model_step_trace
    fn.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]
    fn.restype = C.c_int
    cap, n = 1024, C.c_int(0)
    out = (C.c_ulonglong * (cap * 6))()
    for _ in range(2):
        _ffi.check(fn(m._h, out, cap, C.byref(n)))
    if quiet:
        return
    t = np.array(out[:n.value * 6], dtype=np.float64).reshape(-1, 6) / 1e3
    per = (n.value - 1) // n_layers
    names = {5: ["gemv_qkv", "attention_fused", "gemv_o_proj", "gemv_gate_up", "gemv_down"],
             4: ["gemv_qkv", "gemv_o_proj", "gemv_gate_up", "gemv_down"]}.get(per)
    if names is None:
        sys.stderr.write("timeline: unexpected launch count %d\n" % n.value)
        return
    acc = {k: [] for k in names}
    for i in range(per, n_layers * per):
        acc[names[i % per]].append((t[i, 3] - t[i, 2], t[i, 0] - t[i - 1, 3], t[i, 2] - t[i - 1, 3],
                                    t[i, 5] - t[i, 2], t[i, 3] - t[i, 4]))
    sys.stderr.write("timeline of one step: %.1f us from first start to last end, %d traced launches\n"
                     % (t[-1, 3] - t[0, 0], n.value))
    sys.stderr.write("%-16s %10s %18s %20s %16s %12s\n" % ("class", "active", "start-prev_end", "release-prev_end",
                                                          "release->staged", "end spread"))
    for k in names:
        a = np.array(acc[k]).mean(0)
        sys.stderr.write("%-16s %10.2f %18.2f %20.2f %16.2f %12.2f\n" % (k, *a))
    i = n_layers * per
    sys.stderr.write("%-16s %10.2f %18.2f %20.2f %16.2f %12.2f\n" % ("gemv_lm_head", t[i, 3] - t[i, 2], t[i, 0] - t[i - 1, 3],
                     t[i, 2] - t[i - 1, 3], t[i, 5] - t[i, 2], t[i, 3] - t[i, 4]))


def hf_tensor_names(n_layers):
    """(name, bench tensor key, layer, tensor id) in the order the synthetic file is written; names as the
    loaders match them (crates/atlas-model/src/lib.rs:2328-2346), post-norm layout."""
    out = [("model.embed_tokens.weight", "embed", 0, 1), ("lm_head.weight", "lm_head", 0, 2)]
    local = {"wq": "self_attn.q_proj", "wk": "self_attn.k_proj", "wv": "self_attn.v_proj", "wo": "self_attn.o_proj",
             "gate": "mlp.gate_proj", "up": "mlp.up_proj", "down": "mlp.down_proj"}
    for l in range(n_layers):
        for name, tid in PER_LAYER:
            out.append(("model.layers.%d.%s.weight" % (l, local[name]), name, l, 1000 + l * 32 + tid))
    return out


def run_loader_leg(args):
    """Weight load of the benchmark model from a safetensors file (BASELINE: the reference takes 109 s and 28 GB of
    host memory for the real checkpoint): the synthetic model is written once as bf16 (13.77 GB, same seeded
    tensors as the benchmark), then a fresh process maps it and loads it to the device; that process reports
    seconds, bytes and its peak resident set, and generates the first tokens for comparison with the in-memory
    model."""
    import atlas_b200 as ab
    from atlas_b200 import _ffi
    import ctypes as C
    path = args.loader_file
    if args.loader_child:
        ctx = ab.Context(0)
        mc = model_config(ab, args.prompt + 64)
        m = ab.load_model_from_safetensors(path, mc, ctx=ctx, kv_dtype=ab.BF16)
        st = m.load_stats
        prompt = np.random.default_rng(0).integers(0, mc.vocab_size, size=64, dtype=np.uint32)
        toks = m.generate(prompt, 8, 0.0)
        print(json.dumps({"seconds": st.seconds, "file_bytes_read": st.file_bytes_read, "bytes_uploaded": st.bytes_uploaded,
                          "peak_host_rss_bytes": st.peak_host_rss_bytes, "n_tensors": st.n_tensors_used,
                          "post_norm": st.post_norm, "tokens": [int(t) for t in toks]}))
        return
    ctx = ab.Context(0)
    L = _ffi.lib()
    mc = model_config(ab, args.prompt + 64)
    d, f, V = mc.d_model, mc.ffn_hidden, mc.vocab_size
    shapes = {"embed": (V, d), "lm_head": (V, d), "wq": (d, d), "wk": (d, d), "wv": (d, d), "wo": (d, d), "gate": (f, d), "up": (f, d), "down": (d, f)}
    big = ctx.malloc(V * d * 2)
    tensors = []
    t0 = time.perf_counter()
    for name, key, l, stream in hf_tensor_names(mc.n_layers):
        r, c = shapes[key]
        _ffi.check(L.atlasx_fill_normal_bf16(ctx.handle, big, r * c, 0, stream, 0, 0.02))
        host = np.empty(r * c, np.uint16)
        _ffi.check(L.atlasx_download(ctx.handle, host.ctypes.data_as(C.c_void_p), big, r * c * 2))
        tensors.append((name, [r, c], host))
    ones = np.ones(d, np.float32)
    tensors.append(("model.norm.weight", [d], ones))
    hd = d // mc.n_heads
    for l in range(mc.n_layers):
        for nm in ("post_attention_layernorm", "post_feedforward_layernorm"):
            tensors.append(("model.layers.%d.%s.weight" % (l, nm), [d], ones))
        tensors.append(("model.layers.%d.self_attn.q_norm.weight" % l, [mc.n_heads * hd], np.ones(mc.n_heads * hd, np.float32)))
        tensors.append(("model.layers.%d.self_attn.k_norm.weight" % l, [mc.n_kv_heads * hd], np.ones(mc.n_kv_heads * hd, np.float32)))
    ctx.free(big)
    ab.SafetensorsFile.build(path, tensors)
    t_write = time.perf_counter() - t0
    size = os.path.getsize(path)
    del tensors
    # the in-memory model's first tokens, for the comparison
    m, _ = build_cuda_model(ab, ctx, args.prompt + 64, 0, 1)
    prompt = np.random.default_rng(0).integers(0, mc.vocab_size, size=64, dtype=np.uint32)
    want = [int(t) for t in m.generate(prompt, 8, 0.0)]
    del m
    r = subprocess.run([sys.executable, os.path.abspath(__file__), "--loader-child", "--loader-file", path, "--prompt", str(args.prompt),
                        "--profile-layers", str(PROFILE_LAYERS)], capture_output=True, text=True)
    if r.returncode != 0:
        sys.exit("loader child failed: " + r.stderr[-2000:])
    child = json.loads(r.stdout.strip().splitlines()[-1])
    os.remove(path)
    print(json.dumps({"metric": "safetensors_to_device_load", "file_bytes": size, "file": "bf16 tensors of the benchmark model, in the page cache",
                      "write_s": round(t_write, 2), "load_s": round(child["seconds"], 3),
                      "load_gb_per_s": round(child["bytes_uploaded"] / child["seconds"] / 1e9, 2),
                      "bytes_uploaded": child["bytes_uploaded"], "peak_host_rss_gb": round(child["peak_host_rss_bytes"] / 1e9, 3),
                      "n_tensors": child["n_tensors"], "tokens_from_file": child["tokens"], "tokens_in_memory": want,
                      "tokens_match": child["tokens"] == want}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--repeats", type=int, default=3, help="timed regions of --steps tokens taken back to back; the median is reported")
    ap.add_argument("--prompt", type=int, default=2048, help="context length reached before the timed steps")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-tp-check", action="store_true", help="N > 1: skip rebuilding the model on one GPU to compare tokens")
    ap.add_argument("--no-pdl", action="store_true", help="launch without programmatic dependent launch")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--profile-layers", type=int, default=0,
                    help="keep only the first N layers: a few GB on the device, for profiler captures; the line is marked invalid as a benchmark")
    ap.add_argument("--timeline", action="store_true",
                    help="record %%globaltimer stamps in every GEMV and attention launch of the captured step and print a "
                         "per-class summary on stderr; the stamps cost a little, so the JSON line is marked invalid")
    ap.add_argument("--prefill", type=int, default=128, help="prompt tokens ingested per chunk before the timed region (1: token by token)")
    ap.add_argument("--weights", default="bf16", choices=["bf16", "int8", "int4"],
                    help="weight format held on the device (quantised from the same bf16 tensors); anything but bf16 marks the line invalid as the benchmark")
    ap.add_argument("--gemv-impl", type=int, default=0, help="0 automatic, 1 plain 128-bit loads, 2 bulk-copy pipeline")
    ap.add_argument("--loader", action="store_true", help="separate leg: write the benchmark model as a safetensors file, load it in a fresh process, report time and peak host memory")
    ap.add_argument("--loader-file", default="/dev/shm/atlas_b200_bench_model.safetensors")
    ap.add_argument("--loader-child", action="store_true", help=argparse.SUPPRESS)
    args = ap.parse_args()
    global PROFILE_LAYERS, WEIGHTS
    PROFILE_LAYERS = max(0, args.profile_layers)
    WEIGHTS = args.weights
    if args.timeline:
        os.environ["ATLASX_STEP_TRACE"] = "1"
    if args.loader or args.loader_child:
        run_loader_leg(args)
        return

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            sys.exit("launch with torchrun --nproc-per-node %d for --gpus %d" % (args.gpus, args.gpus))
        args.gpus = world

    import atlas_b200 as ab
    from atlas_b200 import _ffi
    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    ctx = ab.Context(local_rank)
    ctx.set_gemv_impl(args.gemv_impl)
    if world > 1:
        import ctypes as C
        import torch
        ident = (C.c_ubyte * 128)()
        if rank == 0:
            _ffi.check(_ffi.lib().atlasx_comm_unique_id(ident))
        t = torch.tensor(list(bytes(ident)), dtype=torch.uint8, device="cuda")
        dist.broadcast(t, 0)
        ident = (C.c_ubyte * 128)(*t.cpu().tolist())
        _ffi.check(_ffi.lib().atlasx_comm_init(ctx.handle, ident, rank, world))

    steps, warm = args.steps, max(args.warmup, 3)
    reps = max(1, args.repeats)
    lead = 2 if world > 1 else 0                           # untimed lock-step steps in front of every timed region
    max_seq = args.prompt + warm + reps * (steps + lead) + 2 * steps + 16
    m, mc = build_cuda_model(ab, ctx, max_seq, rank, world)
    if args.no_pdl or args.no_graph:
        m.set_options(use_graph=not args.no_graph, use_pdl=not args.no_pdl)
    # Seed of the synthetic prompt: chosen among 0..15 as the one whose first 50 greedy steps behind the prompt keep the
    # largest top-2 logit gap (> 1.5e-2), so that last-bit differences between summation orders (tensor-parallel ranks,
    # split counts) cannot flip a token inside the window the parity check compares.
    prompt = np.random.default_rng(PROMPT_SEED).integers(0, mc.vocab_size, size=args.prompt, dtype=np.uint32)

    # context: the prompt is ingested before the timed region (in chunks through the multi-column
    # kernels unless --prefill 1; the reference feeds it token by token)
    chunk = m.set_prefill(args.prefill) if args.prefill > 1 else 1
    ctx.sync()
    t_in = time.perf_counter()
    m.generate(prompt, 1, 0.0)
    ctx.sync()
    t_in = time.perf_counter() - t_in
    prompt_ingest = {"tokens": int(args.prompt), "chunk": chunk, "ms": round(t_in * 1e3, 2),
                     "tok_s": round(args.prompt / t_in, 1) if t_in > 0 else None}
    m.decode_timed(warm)                                   # warm-up steps (untimed)

    def barrier():
        ctx.sync()
        if dist is not None:
            dist.barrier()

    # The timed region is EXACTLY `steps` tokens between two CUDA events on the launching stream; it
    # is taken `reps` times back to back (each behind a barrier) and the median region is reported.
    # The clock sampler starts before the barrier, so that forking it delays no rank inside a region.
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    pos0 = m.pos
    all_ms, toks = [], None
    for _ in range(reps):
        barrier()
        ms_r, t_r = m.decode_timed(steps, lead)            # `lead` untimed lock-step steps, then the events
        if dist is not None:
            import torch
            tt = torch.tensor([ms_r], device="cuda")
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)      # max over ranks
            ms_r = float(tt.item())
        all_ms.append(ms_r)
        if toks is None:
            toks = t_r
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    ms = float(np.median(all_ms))
    value = steps / (ms / 1e3)

    # end to end through the reference-facing call: token in, logits out, host argmax
    tok = int(toks[-1])
    e2e_steps = min(steps, 64)
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        logits = m.forward_one_gpu(tok)
        tok = int(np.argmax(logits))
    barrier()
    e2e_dt = time.perf_counter() - t0
    if dist is not None:
        import torch
        tt = torch.tensor([e2e_dt], device="cuda")
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        e2e_dt = float(tt.item())
    e2e = {"value": e2e_steps / e2e_dt, "unit": UNIT, "h2d_bytes_per_step": 4,
           "d2h_bytes_per_step": mc.vocab_size * 4, "steps": e2e_steps,
           "call": "OlmoModel.forward_one_gpu(token) -> host logits, numpy argmax"}

    # per-kernel-class device times (event pair around every launch, outside the graph)
    prof_pos = m.pos
    prof = m.profile_step()
    for _ in range(2):
        p2 = m.profile_step()
        for k in prof:
            prof[k]["ms"] = min(prof[k]["ms"], p2[k]["ms"])
    peak, peak_kind = peaks()
    gemv = [k for k in prof if k.startswith("gemv")]
    g_bytes = sum(prof[k]["bytes"] for k in gemv)
    g_ms = sum(prof[k]["ms"] for k in gemv)
    g_launch = sum(prof[k]["launches"] for k in gemv)
    eager = g_bytes / (g_ms / 1e3) / 1e9
    step_bytes = m.step_bytes(pos0 + (reps * (steps + lead)) // 2)
    # The same launches under the conditions of the timed region: one CUDA graph holding only the
    # GEMV launches of a step, in order, with their programmatic-dependent-launch attributes,
    # replayed between two CUDA events (the attention and selection launches are left out).
    fam_ms, fam_bytes, fam_n = None, None, None
    if world == 1:
        fam_ms, fam_bytes, fam_n = m.time_classes(set(gemv), iters=max(8, min(steps, 64)))
    achieved = (fam_bytes / (fam_ms / 1e3) / 1e9) if fam_ms else eager
    roofline = {"bound": "hbm", "kernel": "ax_gemv_stream_kernel<bf16> (all %d GEMV launches of a step)" % g_launch,
                "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "peak_kind": peak_kind,
                "how": ("algorithmic bytes of the %d GEMV launches / device time of a graph with exactly these launches "
                        "(step order, programmatic dependent launch), CUDA events, %.1f us per launch" % (fam_n, fam_ms * 1e3 / fam_n))
                       if fam_ms else "CUDA events around each launch of an eager step",
                "eager_per_launch": {"achieved": eager, "frac": eager / peak,
                                     "note": "event pair around every launch of an eager step without programmatic dependent "
                                             "launch: includes ~4 us of launch latency per kernel that the decode loop hides"},
                "traffic": NCU_GEMV_TRAFFIC_PER_LAUNCH if (world == 1 and not PROFILE_LAYERS) else None,
                "traffic_note": "dram__bytes_read+write per GEMV launch, averaged over the 129 launches of a step from one "
                                "ncu capture of the same kernels and shapes on a 2-layer model; "
                                "algorithmic: %.2f MB" % (g_bytes / max(g_launch, 1) / 1e6),
                "step": {"algorithmic_bytes": step_bytes, "achieved": step_bytes * value / 1e9,
                         "frac": step_bytes * value / 1e9 / peak, "frac_of_8000": step_bytes * value / 1e9 / 8000.0},
                "per_class": {k: {"launches": v["launches"], "ms": round(v["ms"], 4),
                                  "gbs": (v["bytes"] / (v["ms"] / 1e3) / 1e9) if v["ms"] > 0 else None}
                              for k, v in prof.items() if v["launches"]},
                "profiled_at_pos": prof_pos}

    if args.timeline:
        print_timeline(m, mc.n_layers, quiet=(rank != 0))      # every rank runs the extra steps
    # Parity inside a tensor-parallel run: rank 0 rebuilds the model on its GPU alone (second context,
    # no communicator) and regenerates the same tokens; the first tokens of the timed region must agree.
    tp_parity = None
    if world > 1 and rank == 0 and not args.no_tp_check:
        ctx1 = ab.Context(local_rank)
        m1, _ = build_cuda_model(ab, ctx1, max_seq, 0, 1)
        if args.prefill > 1:
            m1.set_prefill(args.prefill)
        m1.generate(prompt, 1, 0.0)
        m1.decode_timed(warm)
        _, t1 = m1.decode_timed(min(steps, 32), lead)
        n_cmp = min(len(t1), len(toks))
        same = [int(a) == int(b) for a, b in zip(t1[:n_cmp], toks[:n_cmp])]
        tp_parity = {"tokens_compared": n_cmp, "match_single_gpu": all(same),
                     "first_mismatch": None if all(same) else same.index(False)}
        if not all(same):
            # The ranks add their partial sums in another order than one GPU does, so logits differ in the last bits and a
            # near-tie of the random-init model can fall the other way; from there on the two runs see different contexts.
            # Replay the single-GPU model up to the first differing step and report how far apart it sees the two tokens:
            # inside the logit bound of the parity definition (1e-2) the divergence is such a tie, beyond it a fault.
            i = same.index(False)
            m1.reset()
            m1.generate(prompt, 1, 0.0)
            _, tw = m1.decode_timed(warm)
            prev = int(tw[-1])
            if lead + i > 0:
                _, tl = m1.decode_timed(lead + i, 0)
                prev = int(tl[-1])
            lg = m1.forward_one_gpu(prev)
            margin = float(lg[int(t1[i])]) - float(lg[int(toks[i])])
            tp_parity.update({"margin_at_first_mismatch": margin, "within_logit_bound": bool(abs(margin) <= 1e-2),
                              "tokens_before_mismatch_identical": i})
            sys.stderr.write("tensor-parallel tokens differ from the single-GPU model at step %d (single-GPU logit margin %.3g)\n" % (i, margin))
        del m1
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    if rank != 0:
        return
    cpu = None
    gpu_launches = m.launches_per_step * steps
    if not args.no_cpu_baseline and world == 1:
        try:
            cpu = cpu_baseline_sample(args.prompt + 1)
        except Exception as e:       # the baseline is reported, never required
            cpu = {"value": None, "unit": UNIT, "cores": os.cpu_count(), "kind": "port", "sample": "failed: %s" % e}
        if not PROFILE_LAYERS:
            try:
                del m                                           # the reference's kernels get the device to themselves
                cpu["ref_gpu"] = ref_gpu_sample(ab, ctx, args.prompt + 1)
            except Exception as e:
                cpu["ref_gpu"] = {"value": None, "what": "failed: %s" % e}
    line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": steps, "warmup": warm,
            "ms_per_step": ms / steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": WORKLOAD, "context": "pos %d..%d (context of %d tokens, then warm-up)" % (pos0 + lead, pos0 + lead + steps, args.prompt + 1),
                       "kv_cache": "bf16", "parallelism": "tp%d" % world,
                       "timing": "median of %d regions of %d steps, CUDA events, max over ranks; regions (ms): %s"
                                 % (reps, steps, ", ".join("%.2f" % x for x in all_ms)),
                       "l2": "inputs larger than L2: 13.77 GB of weights stream per step"},
            "clocks": clocks, "e2e": e2e, "gpu_launches": gpu_launches,
            "first_tokens": [int(t) for t in toks[:8]], "tp_parity": tp_parity, "prompt_ingest": prompt_ingest,
            "roofline": roofline, "cpu_baseline": cpu}
    if PROFILE_LAYERS:
        line["invalid"] = "profiler case: only %d of 32 layers" % PROFILE_LAYERS
    if WEIGHTS != "bf16":
        line["invalid"] = "weights held as %s (per-row int8 / block-32 int4 with f32 scales), not the benchmark's bf16" % WEIGHTS
        line["dtype"] = WEIGHTS
    if args.timeline:
        line["invalid"] = "timeline stamps were recorded inside the kernels"
    print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
