// gemv_device.cuh — device-side building blocks of the weight-streaming GEMV, shared by the
// per-matrix kernels (gemv.cu) and the whole-step persistent kernel (mega.cu): ring geometry,
// mbarrier / bulk-copy wrappers, per-format fragment dot products, input staging (prologue).
#pragma once
#include "gemv.cuh"

namespace {

#ifndef AX_SEG
#define AX_SEG 4096
#endif
#ifndef AX_STAGES
#define AX_STAGES 3
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
        // activations and generation state are read past L1 (__ldcg): inside the persistent
        // whole-step kernel they are rewritten by other SMs while this CTA stays resident
        int pos = __ldcg(p.pos);
        long long tok = __ldcg(p.seq + pos);
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
        return __ldcg(reinterpret_cast<const float4*>(base + (k4 << 2)));
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
            float4 t = __ldcg(reinterpret_cast<const float4*>(p.y) + k4);
            for (int r = 1; r < p.nparts; r++) {
                const float4 u = __ldcg(reinterpret_cast<const float4*>(p.y + (size_t)r * p.part_stride) + k4);
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


}  // namespace
