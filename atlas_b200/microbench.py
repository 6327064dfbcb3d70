"""Per-kernel HBM bandwidth of the decode path (BASELINE configs 2, 3 and 5).

  python -m atlas_b200.microbench gemv      [--formats bf16,int8,int4,int4_f16] [--n 1,4,8,16] [--impl 0|1|2] [--iters 200]
  python -m atlas_b200.microbench attention [--ctx 1024,8192,32768] [--batch 1,8,64] [--iters 50]

One JSON line per case: algorithmic bytes per launch, microseconds per launch (CUDA events
around `iters` back-to-back launches on the launching stream), GB/s and the fraction of the
measured copy bandwidth (MEASURED_PEAKS.json, else 6650 GB/s) and of the nominal 8000 GB/s.
GEMV weights rotate over enough copies to exceed the 126 MB L2 several times; attention cases
smaller than L2 are marked "l2_resident".
"""
import argparse
import ctypes as C
import json
import math
import os

import numpy as np

from . import _ffi
from ._ffi import BF16, F32, INT4, INT8, check
from .tensor import Context, GpuKvCache, GpuMatrix

SHAPES = [(4096, 4096), (11008, 4096), (4096, 11008), (100352, 4096)]
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def peak():
    try:
        return float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def make_matrix(ctx, fmt, M, K, seed):
    """Weights generated on the device; quantised formats by the atlas-quant recipe from f32."""
    L = _ffi.lib()
    if fmt == "bf16":
        p = ctx.malloc(M * K * 2)
        check(L.atlasx_fill_normal_bf16(ctx.handle, p, M * K, seed, 1, 0, 0.02))
        return GpuMatrix.wrap(BF16, p, 0, M, K, ctx=ctx), [p]
    src = ctx.malloc(M * K * 4)
    check(L.atlasx_fill_normal_f32(ctx.handle, src, M * K, seed, 1, 0, 0.02))
    if fmt == "f32":
        return GpuMatrix.wrap(F32, src, 0, M, K, ctx=ctx), [src]
    if fmt == "int8":
        d, s = ctx.malloc(M * K), ctx.malloc(M * 4)
        check(L.atlasx_quantize_int8(ctx.handle, src, M, K, d, s))
        ctx.sync(); ctx.free(src)
        return GpuMatrix.wrap(INT8, d, s, M, K, ctx=ctx), [d, s]
    f16 = fmt == "int4_f16"
    d, s = ctx.malloc(M * K // 2), ctx.malloc(M * K // 32 * 4)
    check(L.atlasx_quantize_int4(ctx.handle, src, M * K, 32, d, s))
    ctx.sync(); ctx.free(src)
    if f16:
        host = ctx.download(s, (M * K // 32,), np.float32).astype(np.float16)
        ctx.free(s)
        s = ctx.to_device(host)
    return GpuMatrix.wrap(INT4, d, s, M, K, block_size=32, scales_f16=f16, ctx=ctx), [d, s]


def run_gemv(args):
    ctx = Context.default()
    ctx.set_gemv_impl(args.impl)
    L = _ffi.lib()
    pk, kind = peak()
    for fmt in args.formats.split(","):
        shapes = [tuple(int(v) for v in t.split("x")) for t in args.shapes.split(",")] if args.shapes else SHAPES
        for (M, K) in shapes:
            m0, bufs = make_matrix(ctx, fmt, M, K, 1)
            wb = m0.weight_bytes
            copies = args.copies if args.copies > 0 else max(2, min(16, int(math.ceil(600e6 / wb))))
            mats, keep = [m0], [bufs]
            for i in range(1, copies):
                mi, bi = make_matrix(ctx, fmt, M, K, 1 + i)
                mats.append(mi); keep.append(bi)
            arr = (C.c_void_p * copies)(*[m._h for m in mats])
            for n in [int(v) for v in args.n.split(",")]:
                x = ctx.malloc(K * n * 4); y = ctx.malloc(M * n * 4)
                check(L.atlasx_fill_normal_f32(ctx.handle, x, K * n, 2, 2, 0, 1.0))
                ms = C.c_float(0)
                iters = max(copies, args.iters if wb < 400e6 else max(args.iters // 8, copies))
                check(L.atlasx_time_gemv(ctx.handle, arr, copies, x, n, y, iters, C.byref(ms)))
                us = ms.value * 1e3 / iters
                by = wb + 4 * K * n + 4 * M * n
                gbs = by / us / 1e3
                print(json.dumps({"kernel": "gemv", "format": fmt, "M": M, "K": K, "n": n, "impl": args.impl,
                                  "bytes": by, "us": round(us, 3), "GBps": round(gbs, 1), "frac": round(gbs / pk, 4),
                                  "peak": pk, "peak_kind": kind, "frac_of_8000": round(gbs / 8000, 4),
                                  "rotating_copies": copies, "iters": iters}), flush=True)
                ctx.free(x); ctx.free(y)
            assert ctx.poll_device_error() == 0
            del mats
            for bi in keep:
                for p in bi:
                    ctx.free(p)


def run_attention(args):
    ctx = Context.default()
    L = _ffi.lib()
    pk, kind = peak()
    nh, nkv, hd = args.heads, args.kv_heads, args.head_dim
    dt = {"bf16": BF16, "f32": F32}[args.kv]
    for c in [int(v) for v in args.ctx.split(",")]:
        for b in [int(v) for v in args.batch.split(",")]:
            esz = 2 if dt == BF16 else 4
            if 2 * b * c * nkv * hd * esz > 60e9:
                continue
            kv = GpuKvCache(c, nkv, hd, dtype=dt, batch=b, ctx=ctx)
            kp, vp, nbytes = kv.ptrs()
            fill = L.atlasx_fill_normal_bf16 if dt == BF16 else L.atlasx_fill_normal_f32
            check(fill(ctx.handle, kp, nbytes // esz, 3, 1, 0, 1.0)); check(fill(ctx.handle, vp, nbytes // esz, 3, 2, 0, 1.0))
            q = ctx.malloc(b * nh * hd * 4); o = ctx.malloc(b * nh * hd * 4)
            check(L.atlasx_fill_normal_f32(ctx.handle, q, b * nh * hd, 3, 3, 0, 1.0))
            pos = np.full(b, c - 1, np.int32)
            for window in [int(v) for v in args.window.split(",")]:
                by = kv.attention_bytes(nh, pos, window)
                ms = C.c_float(0)
                check(L.atlasx_time_attention(ctx.handle, kv._h, q, o, nh, pos.ctypes.data, 1.0 / math.sqrt(hd), window,
                                              args.iters, C.byref(ms)))
                us = ms.value * 1e3 / args.iters
                gbs = by / us / 1e3
                print(json.dumps({"kernel": "attention", "kv": args.kv, "heads": nh, "kv_heads": nkv, "head_dim": hd,
                                  "ctx": c, "batch": b, "window": window, "bytes": by, "us": round(us, 3),
                                  "GBps": round(gbs, 1), "frac": round(gbs / pk, 4), "peak": pk, "peak_kind": kind,
                                  "frac_of_8000": round(gbs / 8000, 4), "l2_resident": by < 126e6}), flush=True)
            ctx.free(q); ctx.free(o)
            del kv


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["gemv", "attention"])
    ap.add_argument("--formats", default="bf16,int8,int4,int4_f16")
    ap.add_argument("--shapes", default="")
    ap.add_argument("--n", default="1")
    ap.add_argument("--impl", type=int, default=0)
    ap.add_argument("--iters", type=int, default=200)
    ap.add_argument("--copies", type=int, default=0, help="rotating weight copies (0 = enough to defeat L2; 1 = L2-resident)")
    ap.add_argument("--ctx", default="1024,8192,32768")
    ap.add_argument("--batch", default="1,8,64")
    ap.add_argument("--window", default="0,4096")
    ap.add_argument("--kv", default="bf16")
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=128)
    args = ap.parse_args()
    (run_gemv if args.what == "gemv" else run_attention)(args)


if __name__ == "__main__":
    main()
