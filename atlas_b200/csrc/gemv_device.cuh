// gemv_device.cuh — device-side building blocks of the weight-streaming GEMV kernels (gemv.cu):
// ring geometry, mbarrier / bulk-copy wrappers, per-format fragment dot products, input staging
// (prologue).
#pragma once
#include "gemv.cuh"

namespace {

#ifndef AX_SEG
#define AX_SEG 4096
#endif
#ifndef AX_STAGES
#define AX_STAGES 6
#endif
constexpr int kConsumerWarps = 8;
constexpr int kRW = 2;                                   // rows per consumer warp
constexpr int kTileRows = kConsumerWarps * kRW;          // 16 (direct path)
constexpr int kRingRows = kConsumerWarps;                // 8: ring path, one row per consumer warp
constexpr int kSeg = AX_SEG;                             // weight bytes per row per stage
constexpr int kSegChunks = kSeg / 16;                    // 128 sixteen-byte chunks
constexpr int kScaleSegMax = kSeg / 4;                       // int4 scale bytes per row per stage (f32, block 32)
constexpr int kMaxStages = AX_STAGES;
constexpr int kConsumerThreads = kConsumerWarps * 32;    // 256
constexpr int kThreadsTma = kConsumerThreads + 32;       // + producer warp
constexpr unsigned long long kWaitLimitNs = 2000000000ull;   // 2 s

template <int FMT> struct Fmt;
template <> struct Fmt<ATLASX_F32>  { static constexpr int EPC = 4;  };   // elements per 16-byte chunk
template <> struct Fmt<ATLASX_BF16> { static constexpr int EPC = 8;  };
template <> struct Fmt<ATLASX_INT8> { static constexpr int EPC = 16; };
template <> struct Fmt<ATLASX_INT4> { static constexpr int EPC = 32; };


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
template <int NTHR = 256>
__device__ __forceinline__ void consumer_sync() {
    if (NTHR == 512) asm volatile("bar.sync 1, 512;" ::: "memory");
    else asm volatile("bar.sync 1, 256;" ::: "memory");
}
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
// Eight elements of a word: the nibbles are first spread into two words of four bytes each
// (high nibbles = even elements, low nibbles = odd elements: two logic operations per word), then
// every byte is dropped into the mantissa of 2^23 with one byte-permute — three operations per
// element (permute, subtract, FMA) instead of four.
__device__ __forceinline__ float i4_byte(uint32_t t, uint32_t sel) {
    return __uint_as_float(__byte_perm(t, 0x4B000000u, sel)) - 8388616.0f;
}
__device__ __forceinline__ void dot_i4_word(uint32_t word, const float4& xa, const float4& xb, Acc4& acc) {
    const uint32_t u = word ^ 0x88888888u;
    const uint32_t hi = (u >> 4) & 0x0F0F0F0Fu, lo = u & 0x0F0F0F0Fu;
    acc.a = fmaf(i4_byte(hi, 0x7540), xa.x, acc.a); acc.b = fmaf(i4_byte(lo, 0x7540), xa.y, acc.b);
    acc.c = fmaf(i4_byte(hi, 0x7541), xa.z, acc.c); acc.d = fmaf(i4_byte(lo, 0x7541), xa.w, acc.d);
    acc.a = fmaf(i4_byte(hi, 0x7542), xb.x, acc.a); acc.b = fmaf(i4_byte(lo, 0x7542), xb.y, acc.b);
    acc.c = fmaf(i4_byte(hi, 0x7543), xb.z, acc.c); acc.d = fmaf(i4_byte(lo, 0x7543), xb.w, acc.d);
}
template <> __device__ __forceinline__ void dot_chunk<ATLASX_INT4>(const uint4& w, const float4* xv, Acc4& acc) {
    dot_i4_word(w.x, xv[0], xv[1], acc); dot_i4_word(w.y, xv[2], xv[3], acc);
    dot_i4_word(w.z, xv[4], xv[5], acc); dot_i4_word(w.w, xv[6], xv[7], acc);
}

// ── block reduction over the 256 consumer threads ────────────────────────────────
template <int NTHR = 256>
__device__ __forceinline__ float consumer_block_sum(float v, float* red /*[NTHR/32]*/) {
    v = ax_warp_sum(v);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    consumer_sync<NTHR>();                       // protect `red` from the previous use
    if (lane == 0) red[warp] = v;
    consumer_sync<NTHR>();
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < NTHR / 32; w++) t += red[w];
    return t;
}

// Input staging.  The vector lives in shared memory as P = EPC/4 planes of float4 so that a
// warp reading one plane for 32 consecutive chunks is conflict-free: element e → plane
// (e % EPC)/4, slot e / EPC.
// Part of the prologue that does not depend on the previous kernel of the stream: the norm
// weights are pulled into L1, and — when the caller vouches that `base` was written at least
// two kernels back (pro.base_early) — the residual stream is copied into the plane `xb` with
// cp.async (thread-private slots: the same thread reads them back, no barrier needed).
template <int FMT, int NTHR = 256>
__device__ __forceinline__ void stage_input_early(const GemvArgs& a, float4* xb) {
    const AxPrologue& p = a.pro;
    if (!p.y && !p.wx) return;
    const int n4 = a.K >> 2, tid = threadIdx.x;
    for (int line = tid; line * 32 < a.K; line += NTHR) {       // 128-byte lines
        if (p.wy) asm volatile("prefetch.global.L1 [%0];" :: "l"(p.wy + line * 32));
        if (p.wx) asm volatile("prefetch.global.L1 [%0];" :: "l"(p.wx + line * 32));
    }
    if (xb && p.base_early && p.base && !p.embed) {
        for (int k4 = tid; k4 < n4; k4 += NTHR)
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"(smem_u32(xb + k4)), "l"(p.base + (k4 << 2)) : "memory");
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
}

// LINEAR: the staged vector keeps its natural order (callers that do not read it in the
// per-chunk plane layout; no bank conflicts while staging).
template <int FMT, int NTHR = 256, bool LINEAR = false>
__device__ __forceinline__ void stage_input(const GemvArgs& a, float4* xs, float* red, const float4* xb = nullptr) {
    constexpr int EPC = Fmt<FMT>::EPC;
    const AxPrologue& p = a.pro;
    const int K = a.K, n4 = K >> 2, nch = a.nchunks;
    const int tid = threadIdx.x;
    auto slot = [&](int k4) { if (LINEAR) return k4; const int e = k4 << 2; return ((e % EPC) >> 2) * nch + e / EPC; };

    const float* base = p.base;
    const uint16_t* base16 = nullptr;
    if (p.embed) {
        // activations and generation state are read past L1 (__ldcg): other SMs wrote them
        int pos = __ldcg(p.pos);
        long long tok = __ldcg(p.seq + pos);
        if (tok < 0) tok = 0;
        if (tok > p.vocab - 1) tok = p.vocab - 1;
        if (p.embed_bf16) base16 = (const uint16_t*)p.embed + (size_t)tok * K;
        else              base = (const float*)p.embed + (size_t)tok * K;
    }
    const bool early = xb && p.base_early && p.base && !p.embed && (p.y || p.wx);
    auto load_base = [&](int k4) -> float4 {
        if (early) return xb[k4];
        if (base16) {
            const uint2 r = *reinterpret_cast<const uint2*>(base16 + (k4 << 2));
            return make_float4(ax_bf16_lo(r.x), ax_bf16_hi(r.x), ax_bf16_lo(r.y), ax_bf16_hi(r.y));
        }
        return __ldcg(reinterpret_cast<const float4*>(base + (k4 << 2)));
    };

    if (!p.y && !p.wx) {                                       // plain input
        for (int k4 = tid; k4 < n4; k4 += NTHR) {
            const float4 v = load_base(k4);
            xs[slot(k4)] = v;
            if (p.resid_out && blockIdx.x == 0) reinterpret_cast<float4*>(p.resid_out)[k4] = v;
        }
        consumer_sync<NTHR>();
        return;
    }
    float inv_y = 1.f;
    if (p.y) {
        float ss = 0.f;
        const unsigned seq = p.ll_n ? __ldcg(p.ll_epoch) * p.ll_mul + p.ll_add : 0u;
        // four (value, sequence) pairs of one part, polled until all four carry this use's number
        auto load_pairs = [&](const uint2* part, int k4) -> float4 {
            const uint4* q = reinterpret_cast<const uint4*>(part + ((size_t)k4 << 2));
            uint4 a0, a1;
            const unsigned long long t0 = ax_globaltimer();
            for (;;) {
                asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(a0.x), "=r"(a0.y), "=r"(a0.z), "=r"(a0.w) : "l"(q) : "memory");
                asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(a1.x), "=r"(a1.y), "=r"(a1.z), "=r"(a1.w) : "l"(q + 1) : "memory");
                if (a0.y == seq && a0.w == seq && a1.y == seq && a1.w == seq) break;
                // a wait that already expired anywhere on this GPU ends all later ones at once
                if (*reinterpret_cast<volatile int*>(a.err) != 0) break;
                if (ax_globaltimer() - t0 > 2000000000ull) { atomicExch(a.err, 3); break; }
            }
            return make_float4(__uint_as_float(a0.x), __uint_as_float(a0.z), __uint_as_float(a1.x), __uint_as_float(a1.z));
        };
        auto load_ll = [&](int r, int k4) -> float4 { return load_pairs(reinterpret_cast<const uint2*>(p.y) + (size_t)r * p.ll_stride, k4); };
        if (p.ll_n && p.ll_red && (int)blockIdx.x < p.ll_red_ctas) {
            // this CTA's slice of the vector: all parts, in rank order, then the sums with the same sequence number
            const int per = (n4 + p.ll_red_ctas - 1) / p.ll_red_ctas;
            const int k_end = min(n4, ((int)blockIdx.x + 1) * per);
            for (int k4 = (int)blockIdx.x * per + tid; k4 < k_end; k4 += NTHR) {
                float4 t = load_ll(0, k4);
                for (int r = 1; r < p.ll_n; r++) { const float4 u = load_ll(r, k4); t.x += u.x; t.y += u.y; t.z += u.z; t.w += u.w; }
                uint4* dst = reinterpret_cast<uint4*>(p.ll_red + ((size_t)k4 << 2));
                asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" :: "l"(dst), "r"(__float_as_uint(t.x)), "r"(seq),
                             "r"(__float_as_uint(t.y)), "r"(seq) : "memory");
                asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" :: "l"(dst + 1), "r"(__float_as_uint(t.z)), "r"(seq),
                             "r"(__float_as_uint(t.w)), "r"(seq) : "memory");
            }
        }
#pragma unroll 4
        for (int k4 = tid; k4 < n4; k4 += NTHR) {
            float4 t;
            if (p.ll_n && p.ll_red) {
                t = load_pairs(p.ll_red, k4);
            } else if (p.ll_n) {
                t = load_ll(0, k4);
                for (int r = 1; r < p.ll_n; r++) { const float4 u = load_ll(r, k4); t.x += u.x; t.y += u.y; t.z += u.z; t.w += u.w; }
            } else {
                t = __ldcg(reinterpret_cast<const float4*>(p.y) + k4);
                for (int r = 1; r < p.nparts; r++) {
                    const float4 u = __ldcg(reinterpret_cast<const float4*>(p.y + (size_t)r * p.part_stride) + k4);
                    t.x += u.x; t.y += u.y; t.z += u.z; t.w += u.w;
                }
            }
            xs[slot(k4)] = t;
            ss += t.x * t.x + t.y * t.y + t.z * t.z + t.w * t.w;
        }
        if (p.wy) {
            ss = consumer_block_sum<NTHR>(ss, red);
            inv_y = 1.0f / sqrtf(ss / (float)K + p.eps);
        }
    }
    if (early) asm volatile("cp.async.wait_all;" ::: "memory");
    float ss2 = 0.f;
#pragma unroll 4
    for (int k4 = tid; k4 < n4; k4 += NTHR) {
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
        ss2 = consumer_block_sum<NTHR>(ss2, red);
        const float inv_x = 1.0f / sqrtf(ss2 / (float)K + p.eps);
        for (int k4 = tid; k4 < n4; k4 += NTHR) {
            float4 v = xs[slot(k4)];
            const float4 w = reinterpret_cast<const float4*>(p.wx)[k4];
            v.x = v.x * inv_x * w.x; v.y = v.y * inv_x * w.y; v.z = v.z * inv_x * w.z; v.w = v.w * inv_x * w.w;
            xs[slot(k4)] = v;
        }
    }
    consumer_sync<NTHR>();
}

__device__ __forceinline__ float load_scale_i4(const void* p, int idx, int f16) {
    return f16 ? __half2float(reinterpret_cast<const __half*>(p)[idx]) : reinterpret_cast<const float*>(p)[idx];
}


// Row range of this CTA, in units of two rows when M is even (keeps gate/up pairs together).
__device__ __forceinline__ void cta_rows(int M, int& lo, int& hi) {
    const int unit = (M & 1) ? 1 : 2;
    const long long units = M / unit;
    lo = (int)(units * blockIdx.x / gridDim.x) * unit;
    hi = (int)(units * (blockIdx.x + 1) / gridDim.x) * unit;
}

// Shared-memory ring shared by the producer warp and the eight consumer warps.
struct Ring {
    uint64_t* full; uint64_t* empty;
    uint8_t* data;
    int stages, stage_stride, seg_pitch;
};

// Producer warp: stream rows [lo,hi) of one matrix into the ring, 8 rows × one ≤4 KB segment per
// stage, one bulk copy per row (plus the int4 scale segment).  `fill` numbers the stages filled
// so far and carries over from one matrix to the next.
template <int FMT>
__device__ __forceinline__ bool ring_produce(const GemvArgs& a, const Ring& rg, int lo, int hi, int& fill) {
    const int lane = threadIdx.x & 31;
    const int ntiles = (hi - lo + kRingRows - 1) / kRingRows;
    const int nk = (a.row_bytes + kSeg - 1) / kSeg;
    const int sseg_full = rg.seg_pitch - kSeg;                // int4 scale bytes of a full segment
    bool ok = true;
    for (int t = 0; t < ntiles && ok; t++) {
        const int r0 = lo + t * kRingRows;
        const int nrows = min(kRingRows, hi - r0);
        for (int kc = 0; kc < nk && ok; kc++, fill++) {
            const int s = fill % rg.stages;
            const uint32_t ph = (uint32_t)(fill / rg.stages) & 1u;
            const int seg = min(kSeg, a.row_bytes - kc * kSeg);
            int sseg = 0;
            if (FMT == ATLASX_INT4) sseg = min(a.srow_bytes - kc * sseg_full, sseg_full);
            if (lane == 0) {
                ok = mbar_wait(&rg.empty[s], ph ^ 1u, a.err, 1);
                if (ok) mbar_arrive_expect_tx(&rg.full[s], (uint32_t)(nrows * (seg + sseg)));
            }
            ok = __shfl_sync(AX_FULL, ok, 0);
            if (ok && lane < nrows) {
                uint8_t* dst = rg.data + (size_t)s * rg.stage_stride + lane * rg.seg_pitch;
                const size_t row = (size_t)(r0 + lane);
                bulk_g2s(dst, a.W + row * a.row_bytes + (size_t)kc * kSeg, (uint32_t)seg, &rg.full[s]);
                if (FMT == ATLASX_INT4)
                    bulk_g2s(dst + kSeg, a.scales + row * a.srow_bytes + (size_t)kc * sseg_full, (uint32_t)sseg, &rg.full[s]);
            }
        }
    }
    return ok;
}

// Consumer warps: one row per warp per tile; the input vector is already staged in `xs`.
template <int FMT>
__device__ __forceinline__ bool ring_consume(const GemvArgs& a, const Ring& rg, const float4* xs, float* pair,
                                             int lo, int hi, int& fill) {
    constexpr int EPC = Fmt<FMT>::EPC;
    constexpr int P = EPC / 4;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ntiles = (hi - lo + kRingRows - 1) / kRingRows;
    const int nk = (a.row_bytes + kSeg - 1) / kSeg;
    const int nch = a.nchunks;
    bool ok = true;
    for (int t = 0; t < ntiles && ok; t++) {
        const int row = lo + t * kRingRows + warp;
        const bool valid = row < hi;
        Acc4 acc = acc4_zero();
        float sc = 0.f;                   // int4: sums already multiplied by their block scales
        for (int kc = 0; kc < nk; kc++, fill++) {
            const int s = fill % rg.stages;
            const uint32_t ph = (uint32_t)(fill / rg.stages) & 1u;
            ok = mbar_wait(&rg.full[s], ph, a.err, 2);
            if (!ok) break;
            const int seg_chunks = min(kSeg, a.row_bytes - kc * kSeg) >> 4;
            const uint8_t* st = rg.data + (size_t)s * rg.stage_stride + warp * rg.seg_pitch;
            if (valid) {
                const uint4* wp = reinterpret_cast<const uint4*>(st) + lane;
                const float4* xb = xs + kc * kSegChunks + lane;
                if (FMT != ATLASX_INT4 && seg_chunks == kSegChunks) {
                    // full segment: no predicates, addresses are lane base + constants
#pragma unroll
                    for (int it = 0; it < kSegChunks / 32; it++) {
                        float4 xv[P];
#pragma unroll
                        for (int p = 0; p < P; p++) xv[p] = xb[p * nch + it * 32];
                        const uint4 w = wp[it * 32];
                        dot_chunk<FMT>(w, xv, acc);
                    }
                } else {
#pragma unroll 2
                    for (int it = 0; it < kSegChunks / 32; it++) {
                        const int c = it * 32 + lane;
                        if (c < seg_chunks) {
                            float4 xv[P];
#pragma unroll
                            for (int p = 0; p < P; p++) xv[p] = xb[p * nch + it * 32];
                            const uint4 w = wp[it * 32];
                            if (FMT == ATLASX_INT4) {
                                Acc4 part = acc4_zero(); dot_chunk<FMT>(w, xv, part);
                                sc = fmaf(part.sum(), load_scale_i4(st + kSeg, (c * EPC) / a.block, a.scales_f16), sc);
                            } else dot_chunk<FMT>(w, xv, acc);
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&rg.empty[s]);
        }
        if (!ok) break;
        float r = ax_warp_sum(acc.sum() + sc);
        if (FMT == ATLASX_INT8 && valid) r *= reinterpret_cast<const float*>(a.scales)[row];
        if (a.epi == AX_EPI_SILU_PAIR) {
            // gate row (even) and up row (odd) sit in neighbouring warps: exchange through shared
            // memory under a two-warp named barrier; slots alternate with the tile parity
            float* slot = pair + (t & 1) * kConsumerWarps;
            if (lane == 0) slot[warp] = r;
            switch (warp >> 1) {          // immediate ids keep the CTA at six hardware barriers
                case 0: asm volatile("bar.sync 2, 64;" ::: "memory"); break;
                case 1: asm volatile("bar.sync 3, 64;" ::: "memory"); break;
                case 2: asm volatile("bar.sync 4, 64;" ::: "memory"); break;
                default: asm volatile("bar.sync 5, 64;" ::: "memory"); break;
            }
            if (lane == 0 && valid && !(warp & 1)) a.y[row >> 1] = (r / (1.0f + expf(-r))) * slot[warp + 1];
        } else if (lane == 0 && valid) {
            a.y[row] = r;
        }
    }
    return ok;
}

__device__ __forceinline__ void ring_init(const Ring& rg) {
    if (threadIdx.x == 0) {
        for (int s = 0; s < rg.stages; s++) { mbar_init(&rg.full[s], 1); mbar_init(&rg.empty[s], kConsumerWarps); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
}

}  // namespace
