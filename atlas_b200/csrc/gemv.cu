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
#include "gemv_device.cuh"

namespace {

// Direct path (no shared-memory ring).  The CTA's rows are taken two at a time (a pair shares
// every load of the input vector) and cut into batches of 128 sixteen-byte chunks per row; the
// batches of all pairs form one sequence that is divided evenly among the eight warps, so a
// warp's share may begin and end in the middle of a row.  Each warp streams its batches with
// 128-bit loads, software-pipelined — the loads of batch i+1 are issued before the arithmetic
// of batch i, and the first batch before griddepcontrol.wait, i.e. while the previous kernel of
// the stream is still draining (weights never depend on it).  Per pair every warp leaves one
// partial sum in shared memory (zero if it had no part in it); after a barrier one thread per
// pair adds the eight values in warp order — deterministic — and applies the epilogue.
// ── quantised formats on the integer dot-product unit ─────────────────────────────
// The f32 input is split once per launch into kPlanes int8 digit planes in base 254, with one
// scale per 32 elements:
//   x ≈ s_c·(q1 + q2/254 [+ q3/254²]),  s_c = max|x| over the 32 elements / 127,  digits in [−127, 127].
// Two planes leave |error| ≤ s_c / (2·254) ≈ 1.6e-5·max|x| of the group per element — errors of
// random sign that add up to ≈ 1e-5 of the result, a hundred times inside the 1e-3 parity bar —
// for two thirds of the integer dot products of three planes (which would leave 6e-8·max|x|).
// The weights are then used as they lie in memory in dp4a instructions with integer-exact sums:
// int8 words directly; int4 nibbles as the HIGH halves of signed bytes — (w & 0xF0F0F0F0) is sixteen
// times the even elements in two's complement, ((w << 4) & 0xF0F0F0F0) sixteen times the odd ones,
// so there is no offset to undo and the factor 16 is divided out of the group scale.  That is 0.5
// (int8) or 0.75 (int4) instruction per element instead of 3 for convert-subtract-FMA.
// Scales per 32 elements need no block-wide reduction: eight neighbouring threads own a group.
constexpr float kDigitBase = 254.0f;
constexpr int kPlanes = 2;
__host__ __device__ constexpr int digit_plane_bytes(int K) { return (K + 127) / 128 * 128; }
__host__ __device__ constexpr int digit_groups(int K) { return ((K + 31) / 32 + 31) / 32 * 32; }
// the planes and the group scales
__host__ __device__ constexpr int digit_bytes(int fmt, int K) {
    return (fmt == ATLASX_INT8 || fmt == ATLASX_INT4) ? kPlanes * digit_plane_bytes(K) + digit_groups(K) * 4 : 0;
}
__device__ __forceinline__ int dp4a_ss(uint32_t a, uint32_t b, int c) {
    int d; asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c)); return d;
}

// After stage_input: xs holds the f32 input in natural order.  Writes the digit planes
// (int8: natural element order; int4: inside every group of eight elements the even ones first,
// then the odd ones, matching the nibble masks) and the scale of every 32 elements (for int4 divided by the 16
// the nibbles carry as high halves of their bytes).  Ends with a barrier.
template <int FMT, int NTHR>
__device__ __forceinline__ void digitize_input(const GemvArgs& a, const float4* xs, uint8_t* xq, float* xsc) {
    const int K = a.K, n4 = K >> 2, tid = threadIdx.x;
    const int pb = digit_plane_bytes(K);
    for (int base = 0; base < n4; base += NTHR) {            // every lane of a warp runs the same trips (shuffles below)
        const int k4 = base + tid;
        const bool in = k4 < n4;
        const float4 v = in ? xs[k4] : make_float4(0.f, 0.f, 0.f, 0.f);
        float mx = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
        mx = fmaxf(mx, __shfl_xor_sync(AX_FULL, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(AX_FULL, mx, 2));
        mx = fmaxf(mx, __shfl_xor_sync(AX_FULL, mx, 4));     // eight threads = 32 elements
        // NaN or inf anywhere in the group: the digits below stay finite (the clamp swallows NaN), so the
        // group's scale carries the fault instead — it becomes NaN, and with it every output row, as in
        // the float formats.  0·x is NaN exactly for x = NaN or ±inf; NaN survives the additions.
        float bad = v.x * 0.f + v.y * 0.f + v.z * 0.f + v.w * 0.f;
        bad += __shfl_xor_sync(AX_FULL, bad, 1);
        bad += __shfl_xor_sync(AX_FULL, bad, 2);
        bad += __shfl_xor_sync(AX_FULL, bad, 4);
        if (!(mx < 3.0e38f)) mx = 3.0e38f;
        const float inv = mx > 0.f ? 127.0f / mx : 0.f;
        const float xv[4] = { v.x, v.y, v.z, v.w };
        int d1[4], d2[4], d3[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            // round to nearest by adding 1.5·2^23: the integer then sits in the low mantissa bits, so
            // neither a rounding nor a float-to-int conversion instruction (both quarter-rate) is needed
            constexpr float M = 12582912.0f;
            float t = xv[j] * inv;
            t = fminf(fmaxf(t, -127.f), 127.f);
            const float a1 = t + M, q1 = a1 - M;
            const float r1 = (t - q1) * kDigitBase;
            const float a2 = r1 + M, q2 = a2 - M;
            const float a3 = (r1 - q2) * kDigitBase + M;
            d1[j] = __float_as_int(a1) - 0x4B400000; d2[j] = __float_as_int(a2) - 0x4B400000; d3[j] = __float_as_int(a3) - 0x4B400000;
        }
        if (!in) continue;
        if ((k4 & 7) == 0) xsc[k4 >> 3] = (mx / 127.0f + bad) * (FMT == ATLASX_INT4 ? 0.0625f : 1.0f);
        if (FMT == ATLASX_INT8) {
            auto word = [](const int (&d)[4]) { return (uint32_t)(d[0] & 255) | ((uint32_t)(d[1] & 255) << 8) | ((uint32_t)(d[2] & 255) << 16) | ((uint32_t)(d[3] & 255) << 24); };
            reinterpret_cast<uint32_t*>(xq)[k4] = word(d1);
            reinterpret_cast<uint32_t*>(xq + pb)[k4] = word(d2);
            if (kPlanes > 2) reinterpret_cast<uint32_t*>(xq + 2 * pb)[k4] = word(d3);
        } else {
            // elements 4k4..4k4+3 sit at j0..j0+3 of their group of eight (j0 = 0 or 4): the even ones
            // go to bytes j0/2, j0/2+1 of the group, the odd ones to bytes 4+j0/2, 4+j0/2+1
            const int g8 = (k4 >> 1) * 8, h = (k4 & 1) * 2;
            auto half = [](int lo, int hi) { return (uint16_t)((lo & 255) | ((hi & 255) << 8)); };
            *reinterpret_cast<uint16_t*>(xq + g8 + h) = half(d1[0], d1[2]);           *reinterpret_cast<uint16_t*>(xq + g8 + 4 + h) = half(d1[1], d1[3]);
            *reinterpret_cast<uint16_t*>(xq + pb + g8 + h) = half(d2[0], d2[2]);      *reinterpret_cast<uint16_t*>(xq + pb + g8 + 4 + h) = half(d2[1], d2[3]);
            if (kPlanes > 2) { *reinterpret_cast<uint16_t*>(xq + 2 * pb + g8 + h) = half(d3[0], d3[2]);  *reinterpret_cast<uint16_t*>(xq + 2 * pb + g8 + 4 + h) = half(d3[1], d3[3]); }
        }
    }
    consumer_sync<NTHR>();
}

__host__ __device__ constexpr int scale_land_bytes(int nthr) { return 2 * 8 * nthr * 4; }     // int4 direct path: landing slots of the block scales

template <int FMT, int NTHR>
__device__ __forceinline__ void consume_direct(const GemvArgs& a, float4* xs, float4* xb, float* red, float* part, uint32_t* sland,
                                               uint8_t* xq, float* xsc, int lo, int hi) {
    constexpr int EPC = Fmt<FMT>::EPC;
    constexpr int P = EPC / 4;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nch = a.nchunks;
    const int nbatch = (nch + 127) >> 7;
    const int npairs = (hi - lo + 1) >> 1;
    const int total = npairs * nbatch;
    const int i0 = (int)((long long)total * warp / (NTHR / 32));
    const int i1 = (int)((long long)total * (warp + 1) / (NTHR / 32));
    uint4 wa[4], wb[4];
    // a batch is named by its pair p and its position b inside the pair's row; both are stepped
    // incrementally (no division in the loop)
    auto load = [&](int p, int b, uint4* A, uint4* B) {
        const int row0 = lo + 2 * p;
        const uint8_t* w0p = a.W + (size_t)row0 * a.row_bytes;
        const uint8_t* w1p = w0p + (row0 + 1 < hi ? a.row_bytes : 0);
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const int c = b * 128 + u * 32 + lane;
            if (c < nch) { A[u] = ax_ldg_stream(w0p + (size_t)c * 16); B[u] = ax_ldg_stream(w1p + (size_t)c * 16); }
        }
    };
    // int4: the block scales of a batch travel with its weights — 4-byte cp.async into thread-private
    // slots [buffer][row·4 + chunk][thread], so that the arithmetic never waits for a scale from DRAM
    auto scale_index = [&](int p, int b, int u, int& idx0, int& idx1, bool& ok) {
        const int row0 = lo + 2 * p;
        const int c = b * 128 + u * 32 + lane;
        ok = c < nch;
        const int cb = a.bshift >= 0 ? (c >> a.bshift) : (c * EPC) / a.block;
        idx0 = row0 * a.spr + cb;
        idx1 = row0 + 1 < hi ? idx0 + a.spr : idx0;
    };
    auto load_scales = [&](bool any, int p, int b, int buf) {
        if (FMT == ATLASX_INT4 && any) {
#pragma unroll
            for (int u = 0; u < 4; u++) {
                int idx0, idx1; bool ok;
                scale_index(p, b, u, idx0, idx1, ok);
                if (ok) {
                    const uint8_t* s0 = a.scales + (a.scales_f16 ? ((size_t)idx0 * 2 & ~(size_t)3) : (size_t)idx0 * 4);
                    const uint8_t* s1 = a.scales + (a.scales_f16 ? ((size_t)idx1 * 2 & ~(size_t)3) : (size_t)idx1 * 4);
                    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" :: "r"(smem_u32(sland + ((buf * 8 + u) * NTHR + tid))), "l"(s0) : "memory");
                    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" :: "r"(smem_u32(sland + ((buf * 8 + 4 + u) * NTHR + tid))), "l"(s1) : "memory");
                }
            }
        }
        if (FMT == ATLASX_INT4) asm volatile("cp.async.commit_group;" ::: "memory");
    };
    auto scale_at = [&](int buf, int slot, int idx) -> float {
        const uint32_t w = sland[(buf * 8 + slot) * NTHR + tid];
        if (a.scales_f16) return __half2float(__ushort_as_half((unsigned short)((idx & 1) ? (w >> 16) : (w & 0xFFFFu))));
        return __uint_as_float(w);
    };
    ax_trace_start(a.trace);
    int p = i0 / nbatch, b = i0 - p * nbatch;
    if (i0 < i1) load(p, b, wa, wb);
    load_scales(i0 < i1, p, b, 0);
    stage_input_early<FMT, NTHR>(a, xb);
    for (int j = tid; j < npairs * (NTHR / 32) * 2; j += NTHR) part[j] = 0.f;
    griddep_wait();                       // activations of the previous kernel are complete
    griddep_launch();
    ax_trace_release(a.trace);
    constexpr bool QUANT = FMT == ATLASX_INT8 || FMT == ATLASX_INT4;
    stage_input<FMT, NTHR, QUANT>(a, xs, red, xb);     // ends with a barrier: the zeroed partials are visible too
    if (QUANT) digitize_input<FMT, NTHR>(a, xs, xq, xsc);
    ax_trace_staged(a.trace);
    const int pb = digit_plane_bytes(a.K);
    constexpr float k2 = 1.0f / kDigitBase, k3 = 1.0f / (kDigitBase * kDigitBase);

    Acc4 acc0 = acc4_zero(), acc1 = acc4_zero();
    float sc0 = 0.f, sc1 = 0.f;
    for (int i = i0; i < i1; i++) {
        uint4 na[4], nb[4];
        const int bn = b + 1 == nbatch ? 0 : b + 1, pn = b + 1 == nbatch ? p + 1 : p;
        if (i + 1 < i1) load(pn, bn, na, nb);
        const int sbuf = (i - i0) & 1;
        load_scales(i + 1 < i1, pn, bn, sbuf ^ 1);             // commits a group even when there is nothing left to fetch
        if (FMT == ATLASX_INT4) asm volatile("cp.async.wait_group 1;" ::: "memory");     // the scales of batch i have landed
        const int row0 = lo + 2 * p;
        const bool v1 = row0 + 1 < hi;
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const int c = b * 128 + u * 32 + lane;
            if (c < nch) {
                if (FMT == ATLASX_INT8) {
                    // 16 elements: four weight words against four digit words per plane, then the group's scale
                    float f0 = 0.f, f1 = 0.f;
#pragma unroll
                    for (int pl = 0; pl < kPlanes; pl++) {
                        const uint4 q = *reinterpret_cast<const uint4*>(xq + pl * pb + c * 16);
                        int t0 = dp4a_ss(wa[u].x, q.x, 0); t0 = dp4a_ss(wa[u].y, q.y, t0); t0 = dp4a_ss(wa[u].z, q.z, t0); t0 = dp4a_ss(wa[u].w, q.w, t0);
                        int t1 = 0;
                        if (v1) { t1 = dp4a_ss(wb[u].x, q.x, 0); t1 = dp4a_ss(wb[u].y, q.y, t1); t1 = dp4a_ss(wb[u].z, q.z, t1); t1 = dp4a_ss(wb[u].w, q.w, t1); }
                        const float wgt = pl == 0 ? 1.f : pl == 1 ? k2 : k3;
                        f0 = fmaf((float)t0, wgt, f0); f1 = fmaf((float)t1, wgt, f1);
                    }
                    const float xs_c = xsc[c >> 1];
                    sc0 = fmaf(f0, xs_c, sc0); sc1 = fmaf(f1, xs_c, sc1);
                } else if (FMT == ATLASX_INT4) {
                    // a chunk is 32 elements of one row and lies inside one block (block is a multiple
                    // of 32 and divides the row length): scale index = row · scales_per_row + chunk / (block/32)
                    int idx0, idx1; bool ok;
                    scale_index(p, b, u, idx0, idx1, ok);
                    // a nibble in the high half of a byte IS sixteen times its two's-complement value as a signed byte:
                    // high nibbles = even elements as they lie, low nibbles = odd elements after a shift by four
                    const uint32_t wx[4] = { wa[u].x, wa[u].y, wa[u].z, wa[u].w };
                    const uint32_t wy[4] = { wb[u].x, wb[u].y, wb[u].z, wb[u].w };
                    constexpr uint32_t HI = 0xF0F0F0F0u;
                    float f0 = 0.f, f1 = 0.f;
#pragma unroll
                    for (int pl = 0; pl < kPlanes; pl++) {
                        const uint4 qa = *reinterpret_cast<const uint4*>(xq + pl * pb + c * 32);
                        const uint4 qb = *reinterpret_cast<const uint4*>(xq + pl * pb + c * 32 + 16);
                        const uint32_t qe[4] = { qa.x, qa.z, qb.x, qb.z }, qo[4] = { qa.y, qa.w, qb.y, qb.w };
                        int t0 = 0, t1 = 0;
#pragma unroll
                        for (int g = 0; g < 4; g++) {
                            t0 = dp4a_ss(wx[g] & HI, qe[g], t0); t0 = dp4a_ss((wx[g] << 4) & HI, qo[g], t0);
                            if (v1) { t1 = dp4a_ss(wy[g] & HI, qe[g], t1); t1 = dp4a_ss((wy[g] << 4) & HI, qo[g], t1); }
                        }
                        const float wgt = pl == 0 ? 1.f : pl == 1 ? k2 : k3;
                        f0 = fmaf((float)t0, wgt, f0); f1 = fmaf((float)t1, wgt, f1);
                    }
                    const float xs_c = xsc[c];
                    sc0 = fmaf(f0 * xs_c, scale_at(sbuf, u, idx0), sc0);
                    if (v1) sc1 = fmaf(f1 * xs_c, scale_at(sbuf, 4 + u, idx1), sc1);
                } else {
                float4 xv[P];
#pragma unroll
                for (int q = 0; q < P; q++) xv[q] = xs[q * nch + c];
                    dot_chunk<FMT>(wa[u], xv, acc0);
                    if (v1) dot_chunk<FMT>(wb[u], xv, acc1);
                }
            }
        }
        if (b == nbatch - 1 || i + 1 == i1) {          // the pair, or this warp's share of it, is done
            const float s0 = ax_warp_sum(acc0.sum() + sc0), s1 = ax_warp_sum(acc1.sum() + sc1);
            if (lane == 0) { part[(p * (NTHR / 32) + warp) * 2] = s0; part[(p * (NTHR / 32) + warp) * 2 + 1] = s1; }
            acc0 = acc4_zero(); acc1 = acc4_zero(); sc0 = 0.f; sc1 = 0.f;
        }
#pragma unroll
        for (int u = 0; u < 4; u++) { wa[u] = na[u]; wb[u] = nb[u]; }
        p = pn; b = bn;
    }
    consumer_sync<NTHR>();
    for (int p = tid; p < npairs; p += NTHR) {
        float s0 = 0.f, s1 = 0.f;
#pragma unroll
        for (int w = 0; w < (NTHR / 32); w++) { s0 += part[(p * (NTHR / 32) + w) * 2]; s1 += part[(p * (NTHR / 32) + w) * 2 + 1]; }
        const int row0 = lo + 2 * p;
        const bool v1 = row0 + 1 < hi;
        if (FMT == ATLASX_INT8) {
            const float* sc = reinterpret_cast<const float*>(a.scales);
            s0 *= sc[row0];
            if (v1) s1 *= sc[row0 + 1];
        }
        if (a.peer.n > 0) {                                                    // push to every rank's mailbox
            const unsigned seq = __ldcg(a.peer.epoch) * a.peer.mul + a.peer.add;
            for (int q = 0; q < a.peer.n; q++) {
                uint2* dst = a.peer.y[q] + row0;
                if (v1 && (row0 & 1) == 0) {                                       // both pairs in one 16-byte store
                    asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" :: "l"(dst), "r"(__float_as_uint(s0)), "r"(seq),
                                 "r"(__float_as_uint(s1)), "r"(seq) : "memory");
                } else {
                    asm volatile("st.volatile.global.v2.u32 [%0], {%1,%2};" :: "l"(dst), "r"(__float_as_uint(s0)), "r"(seq) : "memory");
                    if (v1) asm volatile("st.volatile.global.v2.u32 [%0], {%1,%2};" :: "l"(dst + 1), "r"(__float_as_uint(s1)), "r"(seq) : "memory");
                }
            }
        } else if (a.epi == AX_EPI_SILU_PAIR) {
            if (v1) a.y[row0 >> 1] = (s0 / (1.0f + expf(-s0))) * s1;           // silu(gate)·up
        } else {
            a.y[row0] = s0;
            if (v1) a.y[row0 + 1] = s1;
        }
    }
    ax_trace_end(a.trace);
}

template <int FMT, bool TMA, int NTHR = kConsumerThreads>
__global__ void __launch_bounds__(TMA ? kThreadsTma : NTHR)
ax_gemv_stream_kernel(const GemvArgs a) {
    constexpr int EPC = Fmt<FMT>::EPC;
    constexpr int P = EPC / 4;
    extern __shared__ __align__(128) uint8_t smem_raw[];
    // layout: [full[S] | empty[S] | red[16] | pair[16] | pad to 256] [x planes] [ring]
    uint64_t* full = reinterpret_cast<uint64_t*>(smem_raw);
    uint64_t* empty = full + kMaxStages;
    float* red = reinterpret_cast<float*>(empty + kMaxStages);
    float* pair = red + 16;
    float4* xs = reinterpret_cast<float4*>(smem_raw + 256);
    const int x_bytes = ((a.K * 4 + 127) / 128) * 128;
    uint8_t* ring = smem_raw + 256 + x_bytes;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    int lo, hi; cta_rows(a.M, lo, hi);
    if (!TMA) {
        // second plane (raw residual stream, fetched early) only when the launcher reserved it
        float4* xb = a.pro.base_early ? reinterpret_cast<float4*>(ring) : nullptr;
        // after the input planes: [int4 scale slots][digit planes + block sums of the quantised formats][partials]
        uint8_t* after_x = ring + (a.pro.base_early ? x_bytes : 0);
        uint32_t* sland = reinterpret_cast<uint32_t*>(after_x);                              // int4 only: [2][8][threads] scale slots
        uint8_t* xq = after_x + (FMT == ATLASX_INT4 ? scale_land_bytes(NTHR) : 0);
        float* xsc = reinterpret_cast<float*>(xq + kPlanes * digit_plane_bytes(a.K));              // scale per 32 input elements
        float* part = reinterpret_cast<float*>(xq + digit_bytes(FMT, a.K));                  // [pairs][warps][2]
        consume_direct<FMT, NTHR>(a, xs, xb, red, part, sland, xq, xsc, lo, hi);
        return;
    }

    Ring rg;
    rg.full = full; rg.empty = empty; rg.data = ring;
    rg.stages = a.stages; rg.stage_stride = a.stage_stride; rg.seg_pitch = a.seg_pitch;
    ring_init(rg);
    int fill = 0;
    if (warp == kConsumerWarps) {
        // producer warp: weights do not depend on the previous kernel, so it starts at once
        if (!ring_produce<FMT>(a, rg, lo, hi, fill))
            for (int i = 0; i < 100; i++) __nanosleep(10000);   // let copies in flight land before exit
        return;
    }
    griddep_wait();                       // activations of the previous kernel are complete
    griddep_launch();
    stage_input<FMT>(a, xs, red);
    ring_consume<FMT>(a, rg, xs, pair, lo, hi, fill);
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

template <int FMT, bool TMA, int NTHR = kConsumerThreads>
int launch_stream(atlasx_ctx* ctx, const GemvArgs& a, int grid, size_t smem, bool pdl) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid); cfg.blockDim = dim3(TMA ? kThreadsTma : NTHR);
    cfg.dynamicSmemBytes = smem; cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[2];
    int na = 0;
    if (pdl) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        na++;
    }
    if (!TMA && ctx->carveout >= 0) {
        attr[na].id = cudaLaunchAttributePreferredSharedMemoryCarveout;
        attr[na].val.sharedMemCarveout = (unsigned)ctx->carveout;
        na++;
    }
    if (na) { cfg.attrs = attr; cfg.numAttrs = na; }
    AX_CUDA(cudaLaunchKernelEx(&cfg, ax_gemv_stream_kernel<FMT, TMA, NTHR>, a));
    return ATLASX_OK;
}

template <int FMT>
int set_attrs() {
    AX_CUDA(cudaFuncSetAttribute(ax_gemv_stream_kernel<FMT, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448));
    AX_CUDA(cudaFuncSetAttribute(ax_gemv_stream_kernel<FMT, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448));
    AX_CUDA(cudaFuncSetAttribute(ax_gemv_stream_kernel<FMT, false, 512>, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448));
    return ATLASX_OK;
}

}  // namespace

namespace {
__global__ void __launch_bounds__(256) ax_mail_reduce_kernel(const uint2* parts, int n_parts, size_t stride, int d,
                                                             const unsigned* epoch, unsigned mul, unsigned add, float* out, int* err) {
    // The data polled below arrives through the mailbox from all GPUs (this one included), so the
    // wait is not needed for it; it keeps the stream's rule that a kernel runs only after
    // everything before its predecessor is complete, which later launches rely on.
    griddep_wait();
    griddep_launch();
    const unsigned seq = __ldcg(epoch) * mul + add;
    const int k2 = blockIdx.x * blockDim.x + threadIdx.x;          // two elements (16 bytes of pairs) per thread
    if (2 * k2 >= d) return;
    float s0 = 0.f, s1 = 0.f;
    const unsigned long long t0 = ax_globaltimer();
    for (int r = 0; r < n_parts; r++) {
        const uint4* q = reinterpret_cast<const uint4*>(parts + (size_t)r * stride) + k2;
        uint4 v;
        for (;;) {
            asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(q) : "memory");
            if (v.y == seq && v.w == seq) break;
            if (*reinterpret_cast<volatile int*>(err) != 0) break;
            if (ax_globaltimer() - t0 > 2000000000ull) { atomicExch(err, 3); break; }
        }
        s0 += __uint_as_float(v.x); s1 += __uint_as_float(v.z);
    }
    reinterpret_cast<float2*>(out)[k2] = make_float2(s0, s1);
}
}  // namespace

int ax_mail_reduce_launch(atlasx_ctx* ctx, const uint2* parts, int n_parts, size_t stride, int d,
                          const unsigned* epoch, unsigned mul, unsigned add, float* out, bool pdl) {
    AX_ARG(parts && out && epoch && n_parts >= 1 && d > 0 && (d & 1) == 0, "bad argument");
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)((d / 2 + 255) / 256)); cfg.blockDim = dim3(256); cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    if (pdl) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr; cfg.numAttrs = 1;
    }
    AX_CUDA(cudaLaunchKernelEx(&cfg, ax_mail_reduce_kernel, parts, n_parts, stride, d, epoch, mul, add, out, ctx->dev_error));
    return ATLASX_OK;
}

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

int ax_gemv_launch(atlasx_ctx* ctx, const AxWeight& w, const AxPrologue& pro, int epi, int n, float* y, bool pdl, const AxPeerOut* peer) {
    AX_ARG(w.data && y, "null pointer");
    AX_ARG(w.rows > 0 && w.cols > 0, "empty matrix");
    AX_ARG(n >= 1 && n <= 128, "n must be in 1..128");
    const int epc = w.dtype == ATLASX_F32 ? 4 : w.dtype == ATLASX_BF16 ? 8 : w.dtype == ATLASX_INT8 ? 16 : 32;
    const int ebits = w.dtype == ATLASX_F32 ? 32 : w.dtype == ATLASX_BF16 ? 16 : w.dtype == ATLASX_INT8 ? 8 : 4;
    const bool has_pro = pro.y || pro.wx || pro.embed || pro.resid_out;
    bool vec_ok = (w.cols % epc == 0) && (((uintptr_t)w.data & 15) == 0) && n == 1;
    if (w.dtype == ATLASX_INT4) vec_ok = vec_ok && w.block >= 32 && (w.block % 32 == 0) && (w.cols % w.block == 0) && w.scales;
    if (w.dtype == ATLASX_INT8) vec_ok = vec_ok && w.scales;
    if (vec_ok && pro.base) vec_ok = (((uintptr_t)pro.base & 15) == 0);

    if (n > 1 && !has_pro && epi == AX_EPI_PLAIN && ctx->gemv_impl != 3) {   // gemv_impl 3 keeps the scalar kernel (A/B comparison)
        if (ctx->tune.umma && ax_gemv_umma_supported(w, n, pro.base, y)) return ax_gemv_umma_launch(ctx, w, pro.base, n, y, false, pdl);
        if (ax_gemv_mma_supported(w, n, pro.base, y)) return ax_gemv_mma_launch(ctx, w, pro.base, n, y);
        if (ctx->tune.umma && ax_gemv_umma_int4_supported(w, n, pro.base, y)) return ax_gemv_umma_int4_launch(ctx, w, pro.base, n, y, false, pdl);
    }
    AX_ARG(n <= 16, "more than 16 columns need bf16 weights (up to 128) or int8 weights (up to 64) in the tensor-memory kernel's shapes");
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
    a.spr = w.dtype == ATLASX_INT4 ? w.cols / (w.block > 0 ? w.block : 1) : 0;
    a.bshift = -1;
    if (w.dtype == ATLASX_INT4 && w.block >= 32) { const int q = w.block / 32; if ((q & (q - 1)) == 0) { a.bshift = 0; while ((1 << a.bshift) < q) a.bshift++; } }
    a.nchunks = a.row_bytes / 16;
    a.epi = epi; a.y = y; a.pro = pro; a.err = ctx->dev_error;
    a.trace = nullptr;

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
    a.stage_stride = kRingRows * a.seg_pitch;
    // Ring depth: first try to stay within half an SM's shared memory so that two CTAs (this
    // kernel and the next one of the stream, launched programmatically) are resident together;
    // if the input vector leaves no room for two stages that way, take the whole SM.
    const long long half_sm = ((long long)smem_max + 1024) / 2 - 1024 - 512;
    long long avail = half_sm - 256 - (long long)x_bytes;
    int stages = (int)(avail / a.stage_stride);
    if (stages < 2) { avail = (long long)smem_max - 256 - (long long)x_bytes; stages = (int)(avail / a.stage_stride); }
    if (stages > kMaxStages) stages = kMaxStages;
    if (stages < 2) tma_ok = false;
    a.stages = stages;

    int impl = ctx->gemv_impl;
    if (peer && peer->n > 0) {
        AX_ARG(vec_ok && epi == AX_EPI_PLAIN, "peer output needs the vectorised kernel and a plain epilogue");
        a.peer = *peer;
        impl = 1;
    }
    if (impl == 0) impl = 1;              // plain loads: faster than the bulk-copy ring inside a decode step
    if (impl == 2 && !tma_ok) impl = 1;

    const int units = (w.rows & 1) ? w.rows : w.rows / 2;
    int rc;
    if (impl == 2) {
        a.pro.base_early = 0;
        const int grid = units < ctx->sm_count ? units : ctx->sm_count;
        if (a.pro.ll_red_ctas > grid) a.pro.ll_red_ctas = grid;
        const size_t smem = 256 + x_bytes + (size_t)stages * a.stage_stride;
        switch (w.dtype) {
            case ATLASX_F32:  rc = launch_stream<ATLASX_F32, true>(ctx, a, grid, smem, pdl); break;
            case ATLASX_BF16: rc = launch_stream<ATLASX_BF16, true>(ctx, a, grid, smem, pdl); break;
            case ATLASX_INT8: rc = launch_stream<ATLASX_INT8, true>(ctx, a, grid, smem, pdl); break;
            default:          rc = launch_stream<ATLASX_INT4, true>(ctx, a, grid, smem, pdl); break;
        }
    } else {
        // Grid first (it fixes how many row pairs a CTA can own), with the occupancy of the
        // larger of the two shared-memory layouts; the early-fetched residual plane only pays
        // off, and is only reserved, next to a fused norm.
        if (!(a.pro.base_early && (pro.y || pro.wx) && pro.base && !pro.embed)) a.pro.base_early = 0;
        const int tiles = units >= 8 ? units / 4 : (units >= 2 ? units / 2 : 1);     // at least four units of rows per CTA
        // One 512-thread CTA per SM stages the input vector once per SM instead of twice (the same
        // bytes in flight as two 256-thread CTAs): 2.88 against 2.99 ms per token on the 7B shapes.
        // Matrices too small to give every SM a CTA keep the 256-thread form.
        const bool wide = ctx->tune.gemv_threads == 512 && tiles >= ctx->sm_count;
        const int nthr = wide ? 512 : kConsumerThreads;
        const int slots_per_sm = wide ? 1 : 2;
        auto part_bytes = [&](int grid) {
            const int unit = (w.rows & 1) ? 1 : 2;
            const long long rows_max = ((long long)units + grid - 1) / grid * unit + unit;
            return (size_t)((rows_max + 1) / 2 + 1) * (nthr / 32) * 2 * sizeof(float);
        };
        const size_t land = (w.dtype == ATLASX_INT4 ? (size_t)scale_land_bytes(nthr) : 0) + (size_t)digit_bytes(w.dtype, w.cols);
        size_t smem = 0;
        int grid = 1;
        for (int attempt = 0; attempt < 2; attempt++) {
            const size_t fixed = 256 + x_bytes * (a.pro.base_early ? 2 : 1) + land;
            int g = ctx->sm_count * slots_per_sm < tiles ? ctx->sm_count * slots_per_sm : tiles;     // first guess
            if (g < 1) g = 1;
            smem = fixed + part_bytes(g);
            if (smem <= smem_max) break;
            if (a.pro.base_early) a.pro.base_early = 0; else break;
        }
        AX_ARG(smem <= smem_max, "input vector does not fit in shared memory");
        int per_sm = 1;             // resident CTAs per SM for this format and input size
        if (!wide) {
            switch (w.dtype) {
                case ATLASX_F32:  cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, ax_gemv_stream_kernel<ATLASX_F32, false>, kConsumerThreads, smem); break;
                case ATLASX_BF16: cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, ax_gemv_stream_kernel<ATLASX_BF16, false>, kConsumerThreads, smem); break;
                case ATLASX_INT8: cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, ax_gemv_stream_kernel<ATLASX_INT8, false>, kConsumerThreads, smem); break;
                default:          cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, ax_gemv_stream_kernel<ATLASX_INT4, false>, kConsumerThreads, smem); break;
            }
        }
        if (per_sm < 1) per_sm = 1;
        grid = ctx->sm_count * per_sm;
        if (grid > tiles) grid = tiles;
        if (grid < 1) grid = 1;
        if (per_sm != slots_per_sm) {      // partial-sum area for the final grid; re-check the fit
            const size_t s2 = 256 + x_bytes * (a.pro.base_early ? 2 : 1) + land + part_bytes(grid);
            if (s2 > smem) { AX_ARG(s2 <= smem_max, "input vector does not fit in shared memory"); }
            smem = s2 > smem ? s2 : smem;
        }
        if (a.pro.ll_red_ctas > grid) a.pro.ll_red_ctas = grid;     // every slice of the parts needs a CTA that sums it
        if (ctx->trace_next) { a.trace = ctx->trace_next; ctx->trace_next += 6; }
        if (wide) {
            switch (w.dtype) {
                case ATLASX_F32:  rc = launch_stream<ATLASX_F32, false, 512>(ctx, a, grid, smem, pdl); break;
                case ATLASX_BF16: rc = launch_stream<ATLASX_BF16, false, 512>(ctx, a, grid, smem, pdl); break;
                case ATLASX_INT8: rc = launch_stream<ATLASX_INT8, false, 512>(ctx, a, grid, smem, pdl); break;
                default:          rc = launch_stream<ATLASX_INT4, false, 512>(ctx, a, grid, smem, pdl); break;
            }
        } else {
            switch (w.dtype) {
                case ATLASX_F32:  rc = launch_stream<ATLASX_F32, false>(ctx, a, grid, smem, pdl); break;
                case ATLASX_BF16: rc = launch_stream<ATLASX_BF16, false>(ctx, a, grid, smem, pdl); break;
                case ATLASX_INT8: rc = launch_stream<ATLASX_INT8, false>(ctx, a, grid, smem, pdl); break;
                default:          rc = launch_stream<ATLASX_INT4, false>(ctx, a, grid, smem, pdl); break;
            }
        }
    }
    return rc;
}
