// mega_attention.inl — attention and selection phases of the whole-step kernel (included by mega.cu).
//
// Attention phase of one layer, head_dim 128: work item = (kv head, sequence split).  Each item
//   1. rebuilds q (per-head RMSNorm + RoPE) for the group's query heads, the new K row (norm,
//      RoPE, rounded to the cache type) and the new V row from the raw QKV vector — a few hundred
//      flops, cheaper than a kernel and a grid barrier of their own;
//   2. split 0 stores the new K/V row into the cache (crates/atlas-model/src/lib.rs:860-862);
//   3. streams its share of the cached rows [begin, pos) with 128-bit loads, eight rows in flight
//      per lane group, online softmax (the row `pos` itself comes from shared memory);
//   4. writes its partial state (m, l, acc[128]); the o_proj prologue merges the splits.
#include "attention_device.cuh"

namespace {

template <bool BF16, int GT>
__device__ __noinline__ void mega_attention_items(const MegaPhase& P, float* scr) {
    constexpr int HD = 128;
    constexpr int EPL = BF16 ? 8 : 4;
    constexpr int LPR = HD / EPL;                 // lanes per cached row: 16 or 32
    constexpr int RPW = 32 / LPR;
    constexpr int SLOTS = kConsumerWarps * RPW;
    constexpr int ST = HD + 2;
    constexpr int UN = 4;                          // rows per lane group per batch; two batches in flight
    float* q_s = scr;                              // [kMaxGroup][HD]
    float* k_new = scr + kMaxGroup * HD;           // [HD]
    float* v_new = k_new + HD;                     // [HD]
    float* smm = v_new + HD;                       // [warps][kMaxGroup][ST]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int sub = lane % LPR, slot = warp * RPW + lane / LPR;
    const int S = P.splits;
    const int pos = __ldcg(P.pos);
    const int tb = (P.window > 0 && pos - P.window + 1 > 0) ? pos - P.window + 1 : 0;
    const int rows = pos - tb;                     // cached rows; row `pos` is handled from shared memory
    const int per = (rows + S - 1) / S;
    const int q_rows = P.n_heads * HD, kv_rows = P.n_kv * HD;
    const size_t row_bytes = (size_t)P.n_kv * HD * (BF16 ? 2 : 4);
    const size_t esz = BF16 ? 2 : 4;
    const int half = HD / 2;
    const float* cr = P.cos_t ? P.cos_t + (size_t)pos * half : nullptr;
    const float* sr = P.sin_t ? P.sin_t + (size_t)pos * half : nullptr;

    for (int item = blockIdx.x; item < P.n_kv * S; item += gridDim.x) {
        const int kh = item / S, s = item - kh * S;
        consumer_sync();                           // scratch of the previous item is no longer read
        // ── 1. q heads, new K row, new V row ────────────────────────────────────────
        if (warp < GT) {
            const int h = kh * GT + warp;
            const float4 v = mg_norm_rope_128(P.qkv + (size_t)h * HD, P.q_norm ? P.q_norm + (size_t)h * HD : nullptr, cr, sr, P.qk_eps);
            reinterpret_cast<float4*>(q_s + warp * HD)[lane] = v;
        } else if (warp == GT || warp == GT + 1) {
            const bool is_k = warp == GT;
            float4 v;
            if (is_k) v = mg_norm_rope_128(P.qkv + q_rows + (size_t)kh * HD, P.k_norm ? P.k_norm + (size_t)kh * HD : nullptr, cr, sr, P.qk_eps);
            else      v = __ldcg(reinterpret_cast<const float4*>(P.qkv + q_rows + kv_rows + (size_t)kh * HD) + lane);
            const size_t off = ((size_t)pos * P.n_kv + kh) * HD + lane * 4;
            void* cache = is_k ? P.kc : P.vc;
            if (BF16) {
                const uint16_t b0 = ax_f32_to_bf16_rne(v.x), b1 = ax_f32_to_bf16_rne(v.y), b2 = ax_f32_to_bf16_rne(v.z), b3 = ax_f32_to_bf16_rne(v.w);
                if (s == 0) *reinterpret_cast<uint2*>(reinterpret_cast<uint16_t*>(cache) + off) =
                    make_uint2((uint32_t)b0 | ((uint32_t)b1 << 16), (uint32_t)b2 | ((uint32_t)b3 << 16));
                v = make_float4(ax_bf16_to_f32(b0), ax_bf16_to_f32(b1), ax_bf16_to_f32(b2), ax_bf16_to_f32(b3));
            } else if (s == 0) {
                *reinterpret_cast<float4*>(reinterpret_cast<float*>(cache) + off) = v;
            }
            reinterpret_cast<float4*>(is_k ? k_new : v_new)[lane] = v;
        }
        // ── 2. this split's cached rows: first batch is requested before the prep is visible ──
        const int t0 = tb + s * per;
        const int t1 = min(pos, t0 + per);
        const uint8_t* kbase = (const uint8_t*)P.kc + ((size_t)kh * HD + sub * EPL) * esz;
        const uint8_t* vbase = (const uint8_t*)P.vc + ((size_t)kh * HD + sub * EPL) * esz;
        uint4 kr[UN], vr[UN]; bool valid[UN];
        auto load = [&](int base, uint4 (&K)[UN], uint4 (&V)[UN], bool (&ok)[UN]) {
#pragma unroll
            for (int u = 0; u < UN; u++) {
                const int t = base + u * SLOTS + slot;
                ok[u] = t < t1;
                if (ok[u]) { K[u] = ax_ldg_stream(kbase + (size_t)t * row_bytes); V[u] = ax_ldg_stream(vbase + (size_t)t * row_bytes); }
                else { K[u] = make_uint4(0, 0, 0, 0); V[u] = make_uint4(0, 0, 0, 0); }
            }
        };
        load(t0, kr, vr, valid);
        consumer_sync();

        float q[GT][EPL], acc[GT][EPL], m[GT], l[GT];
#pragma unroll
        for (int g = 0; g < GT; g++) {
#pragma unroll
            for (int e = 0; e < EPL; e++) { q[g][e] = q_s[g * HD + sub * EPL + e]; acc[g][e] = 0.f; }
            m[g] = -CUDART_INF_F; l[g] = 0.f;
        }
        for (int base = t0; base + warp * RPW < t1; base += SLOTS * UN) {     // warp-uniform trip count
            uint4 kn[UN], vn[UN]; bool vnok[UN];
            load(base + SLOTS * UN, kn, vn, vnok);                            // next batch in flight
            float sc[UN][GT];
            mg_scores<BF16, UN, EPL, LPR, GT>(q, kr, valid, P.scale, sc);
            mg_update<BF16, UN, EPL, GT>(m, l, acc, sc, valid, vr);
#pragma unroll
            for (int u = 0; u < UN; u++) { kr[u] = kn[u]; vr[u] = vn[u]; valid[u] = vnok[u]; }
        }
        // ── 3. the new row itself (split 0, first lane group of warp 0) ─────────────
        if (s == 0 && warp == 0) {
            uint4 k1[1], v1[1]; bool ok1[1] = { lane / LPR == 0 };
            float sc[1][GT];
            if (BF16) {
                const float* kp = k_new + sub * EPL; const float* vp = v_new + sub * EPL;
                k1[0] = make_uint4(__float_as_uint(kp[0]) >> 16 | (__float_as_uint(kp[1]) & 0xFFFF0000u), __float_as_uint(kp[2]) >> 16 | (__float_as_uint(kp[3]) & 0xFFFF0000u),
                                   __float_as_uint(kp[4]) >> 16 | (__float_as_uint(kp[5]) & 0xFFFF0000u), __float_as_uint(kp[6]) >> 16 | (__float_as_uint(kp[7]) & 0xFFFF0000u));
                v1[0] = make_uint4(__float_as_uint(vp[0]) >> 16 | (__float_as_uint(vp[1]) & 0xFFFF0000u), __float_as_uint(vp[2]) >> 16 | (__float_as_uint(vp[3]) & 0xFFFF0000u),
                                   __float_as_uint(vp[4]) >> 16 | (__float_as_uint(vp[5]) & 0xFFFF0000u), __float_as_uint(vp[6]) >> 16 | (__float_as_uint(vp[7]) & 0xFFFF0000u));
            } else {
                k1[0] = *reinterpret_cast<const uint4*>(k_new + sub * EPL);
                v1[0] = *reinterpret_cast<const uint4*>(v_new + sub * EPL);
            }
            mg_scores<BF16, 1, EPL, LPR, GT>(q, k1, ok1, P.scale, sc);
            mg_update<BF16, 1, EPL, GT>(m, l, acc, sc, ok1, v1);
        }
        // ── 4. merge lane groups → warps → CTA, write the split's state ─────────────
#pragma unroll
        for (int o = LPR; o < 32; o <<= 1) {
#pragma unroll
            for (int g = 0; g < GT; g++) {
                const float mo = __shfl_xor_sync(AX_FULL, m[g], o);
                const float lo = __shfl_xor_sync(AX_FULL, l[g], o);
                const float mn = fmaxf(m[g], mo);
                const float ca = mg_exp_diff(m[g], mn), cb = mg_exp_diff(mo, mn);
                l[g] = l[g] * ca + lo * cb;
#pragma unroll
                for (int e = 0; e < EPL; e++) {
                    const float ao = __shfl_xor_sync(AX_FULL, acc[g][e], o);
                    acc[g][e] = acc[g][e] * ca + ao * cb;
                }
                m[g] = mn;
            }
        }
        if (lane < LPR) {
#pragma unroll
            for (int g = 0; g < GT; g++) {
                float* dst = smm + ((size_t)warp * kMaxGroup + g) * ST;
                if (sub == 0) { dst[0] = m[g]; dst[1] = l[g]; }
#pragma unroll
                for (int e = 0; e < EPL; e++) dst[2 + sub * EPL + e] = acc[g][e];
            }
        }
        consumer_sync();
        for (int idx = threadIdx.x; idx < GT * HD; idx += kConsumerThreads) {
            const int g = idx / HD, d = idx - g * HD;
            float M = -CUDART_INF_F;
            for (int w = 0; w < kConsumerWarps; w++) M = fmaxf(M, smm[((size_t)w * kMaxGroup + g) * ST]);
            float L = 0.f, A = 0.f;
            for (int w = 0; w < kConsumerWarps; w++) {
                const float* st = smm + ((size_t)w * kMaxGroup + g) * ST;
                const float wgt = mg_exp_diff(st[0], M);
                L = fmaf(wgt, st[1], L);
                A = fmaf(wgt, st[2 + d], A);
            }
            float* out = P.partials + (((size_t)(kh * GT + g)) * S + s) * (HD + 4);   // m, l, pad, pad, acc[HD]
            out[4 + d] = A;
            if (d == 0) { out[0] = M; out[1] = L; }
        }
    }
}

template <bool BF16>
__device__ __forceinline__ void mega_attention_phase(const MegaPhase& P, float* scr) {
    const int G = P.n_heads / P.n_kv;
    if (G == 1) mega_attention_items<BF16, 1>(P, scr);
    else if (G == 2) mega_attention_items<BF16, 2>(P, scr);
    else if (G == 4) mega_attention_items<BF16, 4>(P, scr);
}

// Greedy selection, part 1: every CTA reduces its slice of the logits to one (value, index).
__device__ __forceinline__ void mega_select_partial(const MegaPhase& P, float* scr) {
    const long long n = P.vocab;
    const int lo = (int)(n * blockIdx.x / gridDim.x), hi = (int)(n * (blockIdx.x + 1) / gridDim.x);
    float v = 0.f; int idx = -1;
    for (int i = lo + threadIdx.x; i < hi; i += kConsumerThreads) {
        const float xv = __ldcg(P.logits + i);
        if (ax_better(xv, i, v, idx, 1)) { v = xv; idx = i; }
    }
    ax_warp_best(v, idx, 1);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int* si = reinterpret_cast<int*>(scr + 8);
    consumer_sync();
    if (lane == 0) { scr[warp] = v; si[warp] = idx; }
    consumer_sync();
    if (warp == 0) {
        v = lane < kConsumerWarps ? scr[lane] : 0.f; idx = lane < kConsumerWarps ? si[lane] : -1;
        ax_warp_best(v, idx, 1);
        if (lane == 0) { P.sel_vals[blockIdx.x] = v; P.sel_idx[blockIdx.x] = idx; }
    }
}

// Part 2 (CTA 0): last index among equal maxima over all slices, then advance the device state
// exactly as the per-kernel path does: the choice becomes the next input unless that position
// holds a caller-given token.
__device__ __forceinline__ void mega_select_final(const MegaPhase& P, float*) {
    if (blockIdx.x != 0 || threadIdx.x >= 32) return;
    const int lane = threadIdx.x;
    float v = 0.f; int idx = -1;
    for (int j = lane; j < (int)gridDim.x; j += 32) {
        const float bv = __ldcg(P.sel_vals + j); const int bi = __ldcg(P.sel_idx + j);
        if (ax_better(bv, bi, v, idx, 1)) { v = bv; idx = bi; }
    }
    ax_warp_best(v, idx, 1);
    if (lane == 0) {
        if (idx < 0) idx = P.vocab - 1;
        *P.st_last = idx;
        const int p = __ldcg(P.st_pos) + 1;
        if (p >= __ldcg(P.st_nforced) && p < P.seq_cap) P.seq[p] = idx;
        *P.st_pos = p;
    }
}

}  // namespace
