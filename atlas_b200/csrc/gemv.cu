// gemv.cu — weight-streaming GEMV family for decode (y = W·x, W in HBM read exactly once).
//
// Replaces sgemv_bf16_kernel / sgemv_f32_kernel (kernels/matmul.cu:337-377 of the reference:
// one warp per row, 2-byte loads) and adds the int8 / int4 fused-dequant variants that the
// reference's quant formats (crates/atlas-quant/src/lib.rs:32-168) never had a GPU path for.
//
// Kernel ax_gemv_stream_kernel<FMT, TMA>:
//   * each CTA owns a contiguous range of output rows, so no cross-CTA reduction and a
//     load balance within one row pair on 148 SMs;
//   * TMA = true: a producer warp streams 16-row × 2 KB tiles of W into a multi-stage
//     shared-memory ring with cp.async.bulk + mbarrier (full/empty pairs); eight consumer
//     warps (two rows each) read 128-bit fragments conflict-free, dequantise, FMA against
//     the input vector held in shared memory, and finish with warp shuffles;
//   * TMA = false: the same consumers read W with 128-bit streaming global loads;
//   * the input vector is produced by an optional prologue (partial-sum reduction,
//     RMSNorm, residual add, embedding gather) that runs while the first tiles fly;
//   * epilogue: plain store (int8: × row scale) or SwiGLU on interleaved gate/up rows.
// Every wait on an mbarrier is bounded; on expiry the CTA records an error word and leaves.
#include "gemv.cuh"
#include <stdlib.h>

namespace {

constexpr int kConsumerWarps = 8;
constexpr int kRW = 2;                                   // rows per consumer warp
constexpr int kTileRows = kConsumerWarps * kRW;          // 16
constexpr int kSeg = 2048;                               // weight bytes per row per stage
constexpr int kSegChunks = kSeg / 16;                    // 128 sixteen-byte chunks
constexpr int kScaleSegMax = 512;                        // int4 scale bytes per row per stage (f32, block 32)
constexpr int kMaxStages = 6;
constexpr int kConsumerThreads = kConsumerWarps * 32;    // 256
constexpr int kThreadsTma = kConsumerThreads + 32;       // + producer warp
constexpr unsigned long long kWaitLimitNs = 2000000000ull;   // 2 s

template <int FMT> struct Fmt;
template <> struct Fmt<ATLASX_F32>  { static constexpr int EPC = 4;  };   // elements per 16-byte chunk
template <> struct Fmt<ATLASX_BF16> { static constexpr int EPC = 8;  };
template <> struct Fmt<ATLASX_INT8> { static constexpr int EPC = 16; };
template <> struct Fmt<ATLASX_INT4> { static constexpr int EPC = 32; };

struct GemvArgs {
    const uint8_t* W; const uint8_t* scales;
    int M, K;                    // rows, cols (elements)
    int row_bytes;               // bytes of one weight row
    int srow_bytes;              // bytes of one row of int4 scales (0 otherwise)
    int block; int scales_f16;
    int stages; int stage_stride; int seg_pitch;   // ring geometry (TMA)
    int nchunks;                 // 16-byte chunks per row
    int epi;
    float* y;
    AxPrologue pro;
    int* err;
    int dbg;                     // experiments only: bit 0 = consumers skip the arithmetic
};

// ── PTX wrappers ────────────────────────────────────────────────────────────────
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, 1000;\n\t"   // ≤ ~1 µs per try
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ unsigned long long globaltimer_ns() {
    unsigned long long t; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t)); return t;
}
// Bounded wait: false (and the error word set) when the phase has not completed in 2 s.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* err, int code) {
    if (mbar_try_wait(bar, parity)) return true;
    unsigned long long t0 = globaltimer_ns();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 256; i++) if (mbar_try_wait(bar, parity)) return true;
        if (globaltimer_ns() - t0 > kWaitLimitNs) { atomicExch(err, code); return false; }
    }
}
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, 256;" ::: "memory"); }
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void griddep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ── per-format fragment dot: 16 bytes of one weight row against EPC input values ──
// Four independent accumulators per row: with two rows per warp that is eight FMA chains in
// flight, enough to cover the FMA latency with only two or three warps per scheduler.
struct Acc4 {
    float a, b, c, d;
    __device__ __forceinline__ float sum() const { return (a + b) + (c + d); }
};
__device__ __forceinline__ Acc4 acc4_zero() { Acc4 z; z.a = z.b = z.c = z.d = 0.f; return z; }

template <int FMT> __device__ __forceinline__ void dot_chunk(const uint4& w, const float4* xv, Acc4& acc);

template <> __device__ __forceinline__ void dot_chunk<ATLASX_F32>(const uint4& w, const float4* xv, Acc4& acc) {
    acc.a = fmaf(__uint_as_float(w.x), xv[0].x, acc.a); acc.b = fmaf(__uint_as_float(w.y), xv[0].y, acc.b);
    acc.c = fmaf(__uint_as_float(w.z), xv[0].z, acc.c); acc.d = fmaf(__uint_as_float(w.w), xv[0].w, acc.d);
}
template <> __device__ __forceinline__ void dot_chunk<ATLASX_BF16>(const uint4& w, const float4* xv, Acc4& acc) {
    acc.a = fmaf(ax_bf16_lo(w.x), xv[0].x, acc.a); acc.b = fmaf(ax_bf16_hi(w.x), xv[0].y, acc.b);
    acc.c = fmaf(ax_bf16_lo(w.y), xv[0].z, acc.c); acc.d = fmaf(ax_bf16_hi(w.y), xv[0].w, acc.d);
    acc.a = fmaf(ax_bf16_lo(w.z), xv[1].x, acc.a); acc.b = fmaf(ax_bf16_hi(w.z), xv[1].y, acc.b);
    acc.c = fmaf(ax_bf16_lo(w.w), xv[1].z, acc.c); acc.d = fmaf(ax_bf16_hi(w.w), xv[1].w, acc.d);
}
// int8 → f32 without the conversion unit: flip the sign bit, drop the byte into the mantissa
// of 2^23 with one byte-permute, subtract 2^23+128 (exact).
__device__ __forceinline__ void dot_i8_word(uint32_t word, const float4& x, Acc4& acc) {
    const uint32_t u = word ^ 0x80808080u;
    acc.a = fmaf(__uint_as_float(__byte_perm(u, 0x4B000000u, 0x7540)) - 8388736.0f, x.x, acc.a);
    acc.b = fmaf(__uint_as_float(__byte_perm(u, 0x4B000000u, 0x7541)) - 8388736.0f, x.y, acc.b);
    acc.c = fmaf(__uint_as_float(__byte_perm(u, 0x4B000000u, 0x7542)) - 8388736.0f, x.z, acc.c);
    acc.d = fmaf(__uint_as_float(__byte_perm(u, 0x4B000000u, 0x7543)) - 8388736.0f, x.w, acc.d);
}
template <> __device__ __forceinline__ void dot_chunk<ATLASX_INT8>(const uint4& w, const float4* xv, Acc4& acc) {
    dot_i8_word(w.x, xv[0], acc); dot_i8_word(w.y, xv[1], acc);
    dot_i8_word(w.z, xv[2], acc); dot_i8_word(w.w, xv[3], acc);
}
// int4: byte b of a word holds element 2b in its high nibble and 2b+1 in its low nibble
// (atlas-quant/src/lib.rs:137-141).  n ^ 8 = q + 8 goes into the mantissa of 2^23.
__device__ __forceinline__ float i4_val(uint32_t u, int sh) {
    return __uint_as_float(((u >> sh) & 0xFu) | 0x4B000000u) - 8388616.0f;
}
__device__ __forceinline__ void dot_i4_word(uint32_t word, const float4& xa, const float4& xb, Acc4& acc) {
    const uint32_t u = word ^ 0x88888888u;
    acc.a = fmaf(i4_val(u, 4),  xa.x, acc.a); acc.b = fmaf(i4_val(u, 0),  xa.y, acc.b);
    acc.c = fmaf(i4_val(u, 12), xa.z, acc.c); acc.d = fmaf(i4_val(u, 8),  xa.w, acc.d);
    acc.a = fmaf(i4_val(u, 20), xb.x, acc.a); acc.b = fmaf(i4_val(u, 16), xb.y, acc.b);
    acc.c = fmaf(i4_val(u, 28), xb.z, acc.c); acc.d = fmaf(i4_val(u, 24), xb.w, acc.d);
}
template <> __device__ __forceinline__ void dot_chunk<ATLASX_INT4>(const uint4& w, const float4* xv, Acc4& acc) {
    dot_i4_word(w.x, xv[0], xv[1], acc); dot_i4_word(w.y, xv[2], xv[3], acc);
    dot_i4_word(w.z, xv[4], xv[5], acc); dot_i4_word(w.w, xv[6], xv[7], acc);
}

// ── block reduction over the 256 consumer threads ────────────────────────────────
__device__ __forceinline__ float consumer_block_sum(float v, float* red /*[8] + 1*/) {
    v = ax_warp_sum(v);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    consumer_sync();                       // protect `red` from the previous use
    if (lane == 0) red[warp] = v;
    consumer_sync();
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < kConsumerWarps; w++) t += red[w];
    return t;
}

// Input staging.  The vector lives in shared memory as P = EPC/4 planes of float4 so that a
// warp reading one plane for 32 consecutive chunks is conflict-free: element e → plane
// (e % EPC)/4, slot e / EPC.
template <int FMT>
__device__ __forceinline__ void stage_input(const GemvArgs& a, float4* xs, float* red) {
    constexpr int EPC = Fmt<FMT>::EPC;
    const AxPrologue& p = a.pro;
    const int K = a.K, n4 = K >> 2, nch = a.nchunks;
    const int tid = threadIdx.x;
    auto slot = [&](int k4) { const int e = k4 << 2; return ((e % EPC) >> 2) * nch + e / EPC; };

    const float* base = p.base;
    const uint16_t* base16 = nullptr;
    if (p.embed) {
        int pos = *p.pos;
        long long tok = p.seq[pos];
        if (tok < 0) tok = 0;
        if (tok > p.vocab - 1) tok = p.vocab - 1;
        if (p.embed_bf16) base16 = (const uint16_t*)p.embed + (size_t)tok * K;
        else              base = (const float*)p.embed + (size_t)tok * K;
    }
    auto load_base = [&](int k4) -> float4 {
        if (base16) {
            const uint2 r = *reinterpret_cast<const uint2*>(base16 + (k4 << 2));
            return make_float4(ax_bf16_lo(r.x), ax_bf16_hi(r.x), ax_bf16_lo(r.y), ax_bf16_hi(r.y));
        }
        return *reinterpret_cast<const float4*>(base + (k4 << 2));
    };

    if (!p.y && !p.wx) {                                       // plain input
        for (int k4 = tid; k4 < n4; k4 += kConsumerThreads) {
            const float4 v = load_base(k4);
            xs[slot(k4)] = v;
            if (p.resid_out && blockIdx.x == 0) reinterpret_cast<float4*>(p.resid_out)[k4] = v;
        }
        consumer_sync();
        return;
    }
    float inv_y = 1.f;
    if (p.y) {
        float ss = 0.f;
        for (int k4 = tid; k4 < n4; k4 += kConsumerThreads) {
            float4 t = reinterpret_cast<const float4*>(p.y)[k4];
            for (int r = 1; r < p.nparts; r++) {
                const float4 u = reinterpret_cast<const float4*>(p.y + (size_t)r * p.part_stride)[k4];
                t.x += u.x; t.y += u.y; t.z += u.z; t.w += u.w;
            }
            xs[slot(k4)] = t;
            ss += t.x * t.x + t.y * t.y + t.z * t.z + t.w * t.w;
        }
        if (p.wy) {
            ss = consumer_block_sum(ss, red);
            inv_y = 1.0f / sqrtf(ss / (float)K + p.eps);
        }
    }
    float ss2 = 0.f;
    for (int k4 = tid; k4 < n4; k4 += kConsumerThreads) {
        float4 v = load_base(k4);
        if (p.y) {
            float4 t = xs[slot(k4)];
            if (p.wy) {
                const float4 w = reinterpret_cast<const float4*>(p.wy)[k4];
                t.x = t.x * inv_y * w.x; t.y = t.y * inv_y * w.y; t.z = t.z * inv_y * w.z; t.w = t.w * inv_y * w.w;
            }
            v.x += t.x; v.y += t.y; v.z += t.z; v.w += t.w;
        }
        xs[slot(k4)] = v;
        if (p.resid_out && blockIdx.x == 0) reinterpret_cast<float4*>(p.resid_out)[k4] = v;
        ss2 += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    if (p.wx) {
        ss2 = consumer_block_sum(ss2, red);
        const float inv_x = 1.0f / sqrtf(ss2 / (float)K + p.eps);
        for (int k4 = tid; k4 < n4; k4 += kConsumerThreads) {
            float4 v = xs[slot(k4)];
            const float4 w = reinterpret_cast<const float4*>(p.wx)[k4];
            v.x = v.x * inv_x * w.x; v.y = v.y * inv_x * w.y; v.z = v.z * inv_x * w.z; v.w = v.w * inv_x * w.w;
            xs[slot(k4)] = v;
        }
    }
    consumer_sync();
}

__device__ __forceinline__ float load_scale_i4(const void* p, int idx, int f16) {
    return f16 ? __half2float(reinterpret_cast<const __half*>(p)[idx]) : reinterpret_cast<const float*>(p)[idx];
}

template <int FMT>
__device__ __forceinline__ void store_rows(const GemvArgs& a, int row0, bool v0, bool v1, float acc0, float acc1) {
    acc0 = ax_warp_sum(acc0);
    acc1 = ax_warp_sum(acc1);
    if ((threadIdx.x & 31) != 0) return;
    if (FMT == ATLASX_INT8) {
        const float* s = reinterpret_cast<const float*>(a.scales);
        if (v0) acc0 *= s[row0];
        if (v1) acc1 *= s[row0 + 1];
    }
    if (a.epi == AX_EPI_SILU_PAIR) {
        if (v1) a.y[row0 >> 1] = (acc0 / (1.0f + expf(-acc0))) * acc1;     // silu(gate)·up
    } else {
        if (v0) a.y[row0] = acc0;
        if (v1) a.y[row0 + 1] = acc1;
    }
}

// Row range of this CTA, in units of two rows when M is even (keeps gate/up pairs together).
__device__ __forceinline__ void cta_rows(int M, int& lo, int& hi) {
    const int unit = (M & 1) ? 1 : 2;
    const long long units = M / unit;
    lo = (int)(units * blockIdx.x / gridDim.x) * unit;
    hi = (int)(units * (blockIdx.x + 1) / gridDim.x) * unit;
}

// Direct path (no shared-memory ring): every warp streams its two rows with 128-bit loads, four
// chunks per row per batch, software-pipelined — the loads of batch i+1 are issued before the
// arithmetic of batch i, and batch 0 is issued before griddepcontrol.wait, i.e. while the previous
// kernel of the stream is still draining (weights never depend on it).
template <int FMT>
__device__ __forceinline__ void consume_direct(const GemvArgs& a, float4* xs, float* red, int lo, int hi) {
    constexpr int EPC = Fmt<FMT>::EPC;
    constexpr int P = EPC / 4;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nch = a.nchunks;
    const int nbatch = (nch + 127) >> 7;
    const int ntiles = (hi - lo + kTileRows - 1) / kTileRows;
    const int total = ntiles * nbatch;
    uint4 wa[4], wb[4];
    auto load = [&](int i, uint4* A, uint4* B) {
        const int t = i / nbatch, b = i - t * nbatch;
        const int row0 = lo + t * kTileRows + warp * kRW;
        if (row0 < hi) {
            const uint8_t* w0p = a.W + (size_t)row0 * a.row_bytes;
            const uint8_t* w1p = w0p + (row0 + 1 < hi ? a.row_bytes : 0);
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const int c = b * 128 + u * 32 + lane;
                if (c < nch) { A[u] = ax_ldg_stream(w0p + (size_t)c * 16); B[u] = ax_ldg_stream(w1p + (size_t)c * 16); }
            }
        }
    };
    if (total > 0) load(0, wa, wb);
    griddep_wait();                       // activations of the previous kernel are complete
    griddep_launch();
    stage_input<FMT>(a, xs, red);

    Acc4 acc0 = acc4_zero(), acc1 = acc4_zero();
    float sc0 = 0.f, sc1 = 0.f;
    for (int i = 0; i < total; i++) {
        uint4 na[4], nb[4];
        if (i + 1 < total) load(i + 1, na, nb);
        const int t = i / nbatch, b = i - t * nbatch;
        const int row0 = lo + t * kTileRows + warp * kRW;
        const bool v0 = row0 < hi, v1 = row0 + 1 < hi;
        if (v0) {
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const int c = b * 128 + u * 32 + lane;
                if (c < nch) {
                    float4 xv[P];
#pragma unroll
                    for (int p = 0; p < P; p++) xv[p] = xs[p * nch + c];
                    if (FMT == ATLASX_INT4) {
                        const size_t e0 = (size_t)row0 * a.K + (size_t)c * EPC;     // flat element index
                        Acc4 part = acc4_zero(); dot_chunk<FMT>(wa[u], xv, part);
                        sc0 = fmaf(part.sum(), load_scale_i4(a.scales, (int)(e0 / a.block), a.scales_f16), sc0);
                        if (v1) {
                            part = acc4_zero(); dot_chunk<FMT>(wb[u], xv, part);
                            sc1 = fmaf(part.sum(), load_scale_i4(a.scales, (int)((e0 + a.K) / a.block), a.scales_f16), sc1);
                        }
                    } else {
                        dot_chunk<FMT>(wa[u], xv, acc0);
                        if (v1) dot_chunk<FMT>(wb[u], xv, acc1);
                    }
                }
            }
        }
        if (b == nbatch - 1) {
            store_rows<FMT>(a, row0, v0, v1, acc0.sum() + sc0, acc1.sum() + sc1);
            acc0 = acc4_zero(); acc1 = acc4_zero(); sc0 = 0.f; sc1 = 0.f;
        }
#pragma unroll
        for (int u = 0; u < 4; u++) { wa[u] = na[u]; wb[u] = nb[u]; }
    }
}

template <int FMT, bool TMA>
__global__ void __launch_bounds__(TMA ? kThreadsTma : kConsumerThreads)
ax_gemv_stream_kernel(const GemvArgs a) {
    constexpr int EPC = Fmt<FMT>::EPC;
    constexpr int P = EPC / 4;
    extern __shared__ __align__(128) uint8_t smem_raw[];
    // layout: [full[S] | empty[S] | red[16] | pad to 256] [x planes] [ring]
    uint64_t* full = reinterpret_cast<uint64_t*>(smem_raw);
    uint64_t* empty = full + kMaxStages;
    float* red = reinterpret_cast<float*>(empty + kMaxStages);
    float4* xs = reinterpret_cast<float4*>(smem_raw + 256);
    const int x_bytes = ((a.K * 4 + 127) / 128) * 128;
    uint8_t* ring = smem_raw + 256 + x_bytes;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    int lo, hi; cta_rows(a.M, lo, hi);
    const int ntiles = (hi - lo + kTileRows - 1) / kTileRows;
    const int nk = (a.row_bytes + kSeg - 1) / kSeg;

    if (TMA) {
        if (tid == 0) {
            for (int s = 0; s < a.stages; s++) { mbar_init(&full[s], 1); mbar_init(&empty[s], kConsumerWarps); }
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        }
        __syncthreads();
    }

    if (TMA && warp == kConsumerWarps) {
        // ── producer warp: weights do not depend on the previous kernel, so start at once ──
        griddep_launch();
        int fill = 0;
        bool ok = true;
        for (int t = 0; t < ntiles && ok; t++) {
            const int r0 = lo + t * kTileRows;
            const int nrows = min(kTileRows, hi - r0);
            for (int kc = 0; kc < nk && ok; kc++, fill++) {
                const int s = fill % a.stages;
                const uint32_t ph = (uint32_t)(fill / a.stages) & 1u;
                const int seg = min(kSeg, a.row_bytes - kc * kSeg);
                int sseg = 0;
                if (FMT == ATLASX_INT4) sseg = min(a.srow_bytes - kc * (a.seg_pitch - kSeg), a.seg_pitch - kSeg);
                if (lane == 0) {
                    ok = mbar_wait(&empty[s], ph ^ 1u, a.err, 1);
                    if (ok) mbar_arrive_expect_tx(&full[s], (uint32_t)(nrows * (seg + sseg)));
                }
                ok = __shfl_sync(AX_FULL, ok, 0);
                if (ok && lane < nrows) {
                    uint8_t* dst = ring + (size_t)s * a.stage_stride + lane * a.seg_pitch;
                    const size_t row = (size_t)(r0 + lane);
                    bulk_g2s(dst, a.W + row * a.row_bytes + (size_t)kc * kSeg, (uint32_t)seg, &full[s]);
                    if (FMT == ATLASX_INT4)
                        bulk_g2s(dst + kSeg, a.scales + row * a.srow_bytes + (size_t)kc * (a.seg_pitch - kSeg),
                                 (uint32_t)sseg, &full[s]);
                }
            }
        }
        if (!ok) {            // give copies already in flight time to land before the CTA's memory is reused
            for (int i = 0; i < 100; i++) __nanosleep(10000);
        }
        return;
    }

    if (!TMA) { consume_direct<FMT>(a, xs, red, lo, hi); return; }

    // ── consumers ──────────────────────────────────────────────────────────────────
    griddep_wait();                       // activations of the previous kernel are complete
    stage_input<FMT>(a, xs, red);

    int fill = 0;
    bool ok = true;
    for (int t = 0; t < ntiles && ok; t++) {
        const int r0 = lo + t * kTileRows;
        const int row0 = r0 + warp * kRW;
        const bool v0 = row0 < hi, v1 = row0 + 1 < hi;
        Acc4 acc0 = acc4_zero(), acc1 = acc4_zero();
        float sc0 = 0.f, sc1 = 0.f;            // int4: sums already multiplied by their block scales
        if (TMA) {
            for (int kc = 0; kc < nk; kc++, fill++) {
                const int s = fill % a.stages;
                const uint32_t ph = (uint32_t)(fill / a.stages) & 1u;
                ok = mbar_wait(&full[s], ph, a.err, 2);
                if (!ok) break;
                const int seg_chunks = min(kSeg, a.row_bytes - kc * kSeg) >> 4;
                const uint8_t* st = ring + (size_t)s * a.stage_stride + (warp * kRW) * a.seg_pitch;
#pragma unroll
                for (int it = 0; it < kSegChunks / 32; it++) {
                    const int c = it * 32 + lane;
                    if (c < seg_chunks && !(a.dbg & 1)) {
                        const int cg = kc * kSegChunks + c;
                        float4 xv[P];
#pragma unroll
                        for (int p = 0; p < P; p++) xv[p] = xs[p * a.nchunks + cg];
                        if (v0) {
                            const uint4 w = *reinterpret_cast<const uint4*>(st + c * 16);
                            if (FMT == ATLASX_INT4) {
                                Acc4 part = acc4_zero(); dot_chunk<FMT>(w, xv, part);
                                sc0 = fmaf(part.sum(), load_scale_i4(st + kSeg, (c * EPC) / a.block, a.scales_f16), sc0);
                            } else dot_chunk<FMT>(w, xv, acc0);
                        }
                        if (v1) {
                            const uint4 w = *reinterpret_cast<const uint4*>(st + a.seg_pitch + c * 16);
                            if (FMT == ATLASX_INT4) {
                                Acc4 part = acc4_zero(); dot_chunk<FMT>(w, xv, part);
                                sc1 = fmaf(part.sum(), load_scale_i4(st + a.seg_pitch + kSeg, (c * EPC) / a.block, a.scales_f16), sc1);
                            } else dot_chunk<FMT>(w, xv, acc1);
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[s]);
            }
            if (!ok) break;
        }
        store_rows<FMT>(a, row0, v0, v1, acc0.sum() + sc0, acc1.sum() + sc1);
    }
}

// ── scalar kernel: any shape, any alignment, n columns (n ≤ 16); one warp per row ─────────
template <int NMAX>
__global__ void ax_gemv_scalar_kernel(const uint8_t* W, const uint8_t* scales, int dtype, int block, int scales_f16,
                                      int M, int K, int n, const float* x, float* y) {
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= M) return;
    float acc[NMAX];
#pragma unroll
    for (int j = 0; j < NMAX; j++) acc[j] = 0.f;
    for (int k = lane; k < K; k += 32) {
        const size_t e = (size_t)row * K + k;
        float w;
        if (dtype == ATLASX_F32) w = reinterpret_cast<const float*>(W)[e];
        else if (dtype == ATLASX_BF16) w = ax_bf16_to_f32(reinterpret_cast<const uint16_t*>(W)[e]);
        else if (dtype == ATLASX_INT8) w = (float)reinterpret_cast<const int8_t*>(W)[e] * reinterpret_cast<const float*>(scales)[row];
        else {
            const uint8_t b = W[e >> 1];
            const int nib = (e & 1) ? (b & 0xF) : (b >> 4);
            const int q = nib >= 8 ? nib - 16 : nib;
            w = (float)q * load_scale_i4(scales, (int)(e / block), scales_f16);
        }
#pragma unroll
        for (int j = 0; j < NMAX; j++) if (j < n) acc[j] = fmaf(w, x[(size_t)k * n + j], acc[j]);
    }
#pragma unroll
    for (int j = 0; j < NMAX; j++) {
        const float s = ax_warp_sum(acc[j]);
        if (lane == 0 && j < n) y[(size_t)row * n + j] = s;
    }
}

template <int FMT, bool TMA>
int launch_stream(atlasx_ctx* ctx, const GemvArgs& a, int grid, size_t smem, bool pdl) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid); cfg.blockDim = dim3(TMA ? kThreadsTma : kConsumerThreads);
    cfg.dynamicSmemBytes = smem; cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    if (pdl) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr; cfg.numAttrs = 1;
    }
    AX_CUDA(cudaLaunchKernelEx(&cfg, ax_gemv_stream_kernel<FMT, TMA>, a));
    return ATLASX_OK;
}

template <int FMT>
int set_attrs() {
    AX_CUDA(cudaFuncSetAttribute(ax_gemv_stream_kernel<FMT, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448));
    AX_CUDA(cudaFuncSetAttribute(ax_gemv_stream_kernel<FMT, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448));
    return ATLASX_OK;
}

}  // namespace

int ax_gemv_init(atlasx_ctx*) {
    int rc;
    if ((rc = set_attrs<ATLASX_F32>())) return rc;
    if ((rc = set_attrs<ATLASX_BF16>())) return rc;
    if ((rc = set_attrs<ATLASX_INT8>())) return rc;
    if ((rc = set_attrs<ATLASX_INT4>())) return rc;
    return ATLASX_OK;
}

size_t ax_weight_bytes(const AxWeight& w) {
    const size_t n = (size_t)w.rows * w.cols;
    switch (w.dtype) {
        case ATLASX_F32: return n * 4;
        case ATLASX_BF16: return n * 2;
        case ATLASX_INT8: return n + (size_t)w.rows * 4;
        case ATLASX_INT4: return (n + 1) / 2 + ((n + w.block - 1) / w.block) * (w.scales_f16 ? 2 : 4);
    }
    return 0;
}

int ax_gemv_launch(atlasx_ctx* ctx, const AxWeight& w, const AxPrologue& pro, int epi, int n, float* y, bool pdl) {
    AX_ARG(w.data && y, "null pointer");
    AX_ARG(w.rows > 0 && w.cols > 0, "empty matrix");
    AX_ARG(n >= 1 && n <= 16, "n must be in 1..16");
    const int epc = w.dtype == ATLASX_F32 ? 4 : w.dtype == ATLASX_BF16 ? 8 : w.dtype == ATLASX_INT8 ? 16 : 32;
    const int ebits = w.dtype == ATLASX_F32 ? 32 : w.dtype == ATLASX_BF16 ? 16 : w.dtype == ATLASX_INT8 ? 8 : 4;
    const bool has_pro = pro.y || pro.wx || pro.embed || pro.resid_out;
    bool vec_ok = (w.cols % epc == 0) && (((uintptr_t)w.data & 15) == 0) && n == 1;
    if (w.dtype == ATLASX_INT4) vec_ok = vec_ok && w.block >= 32 && (w.block % 32 == 0) && (w.cols % w.block == 0) && w.scales;
    if (w.dtype == ATLASX_INT8) vec_ok = vec_ok && w.scales;
    if (vec_ok && pro.base) vec_ok = (((uintptr_t)pro.base & 15) == 0);

    if (!vec_ok) {
        AX_ARG(!has_pro && epi == AX_EPI_PLAIN && pro.base, "fused prologue/epilogue need 16-byte aligned rows and n == 1");
        const int warps = 8;
        const int grid = (w.rows + warps - 1) / warps;
        ax_gemv_scalar_kernel<16><<<grid, warps * 32, 0, ctx->stream>>>(
            (const uint8_t*)w.data, (const uint8_t*)w.scales, w.dtype, w.block > 0 ? w.block : 1, w.scales_f16,
            w.rows, w.cols, n, pro.base, y);
        AX_CHECK_LAUNCH("ax_gemv_scalar_kernel");
        return ATLASX_OK;
    }
    if (epi == AX_EPI_SILU_PAIR) AX_ARG((w.rows & 1) == 0, "pair epilogue needs an even row count");

    GemvArgs a = {};
    a.W = (const uint8_t*)w.data; a.scales = (const uint8_t*)w.scales;
    a.M = w.rows; a.K = w.cols;
    a.row_bytes = (int)((size_t)w.cols * ebits / 8);
    a.block = w.block > 0 ? w.block : 1; a.scales_f16 = w.scales_f16;
    a.srow_bytes = w.dtype == ATLASX_INT4 ? (w.cols / w.block) * (w.scales_f16 ? 2 : 4) : 0;
    a.nchunks = a.row_bytes / 16;
    a.epi = epi; a.y = y; a.pro = pro; a.err = ctx->dev_error;
    { const char* e = getenv("ATLASX_GEMV_DEBUG"); a.dbg = e ? atoi(e) : 0; }

    const size_t x_bytes = (((size_t)w.cols * 4 + 127) / 128) * 128;
    const size_t smem_max = ctx->smem_optin ? ctx->smem_optin : 232448;
    // bulk-copy ring: needs 16-byte granules everywhere and at least two stages
    int sseg = 0;
    bool tma_ok = true;
    if (w.dtype == ATLASX_INT4) {
        sseg = (kSeg * 2 / w.block) * (w.scales_f16 ? 2 : 4);          // scale bytes matching one 2 KB segment
        tma_ok = (sseg % 16 == 0) && (a.srow_bytes % 16 == 0) && sseg <= kScaleSegMax && (((uintptr_t)w.scales & 15) == 0);
    }
    a.seg_pitch = kSeg + sseg;
    a.stage_stride = kTileRows * a.seg_pitch;
    long long avail = (long long)smem_max - 256 - (long long)x_bytes;
    int stages = (int)(avail / a.stage_stride);
    if (stages > kMaxStages) stages = kMaxStages;
    if (stages < 2) tma_ok = false;
    a.stages = stages;

    int impl = ctx->gemv_impl;
    if (impl == 0) impl = 2;
    if (impl == 2 && !tma_ok) impl = 1;

    const int units = (w.rows & 1) ? w.rows : w.rows / 2;
    int rc;
    if (impl == 2) {
        const int grid = units < ctx->sm_count ? units : ctx->sm_count;
        const size_t smem = 256 + x_bytes + (size_t)stages * a.stage_stride;
        switch (w.dtype) {
            case ATLASX_F32:  rc = launch_stream<ATLASX_F32, true>(ctx, a, grid, smem, pdl); break;
            case ATLASX_BF16: rc = launch_stream<ATLASX_BF16, true>(ctx, a, grid, smem, pdl); break;
            case ATLASX_INT8: rc = launch_stream<ATLASX_INT8, true>(ctx, a, grid, smem, pdl); break;
            default:          rc = launch_stream<ATLASX_INT4, true>(ctx, a, grid, smem, pdl); break;
        }
    } else {
        const size_t smem = 256 + x_bytes;
        AX_ARG(smem <= smem_max, "input vector does not fit in shared memory");
        int per_sm = 1;             // resident CTAs per SM for this format and input size
        switch (w.dtype) {
            case ATLASX_F32:  cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, ax_gemv_stream_kernel<ATLASX_F32, false>, kConsumerThreads, smem); break;
            case ATLASX_BF16: cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, ax_gemv_stream_kernel<ATLASX_BF16, false>, kConsumerThreads, smem); break;
            case ATLASX_INT8: cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, ax_gemv_stream_kernel<ATLASX_INT8, false>, kConsumerThreads, smem); break;
            default:          cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, ax_gemv_stream_kernel<ATLASX_INT4, false>, kConsumerThreads, smem); break;
        }
        if (per_sm < 1) per_sm = 1;
        int grid = ctx->sm_count * per_sm;
        const int tiles = (units * ((w.rows & 1) ? 1 : 2) + kTileRows - 1) / kTileRows;
        if (grid > tiles) grid = tiles;
        if (grid < 1) grid = 1;
        switch (w.dtype) {
            case ATLASX_F32:  rc = launch_stream<ATLASX_F32, false>(ctx, a, grid, smem, pdl); break;
            case ATLASX_BF16: rc = launch_stream<ATLASX_BF16, false>(ctx, a, grid, smem, pdl); break;
            case ATLASX_INT8: rc = launch_stream<ATLASX_INT8, false>(ctx, a, grid, smem, pdl); break;
            default:          rc = launch_stream<ATLASX_INT4, false>(ctx, a, grid, smem, pdl); break;
        }
    }
    return rc;
}
