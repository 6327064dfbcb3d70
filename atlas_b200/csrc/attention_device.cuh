// attention_device.cuh — device helpers shared by the fused decode-attention kernel and the
// attention phase of the whole-step kernel (head_dim 128: one warp per head vector, lane l
// holds dims 4l..4l+3; cached rows are read as 16-byte pieces, EPL elements per lane).
#pragma once
#include <math_constants.h>
#include "common.cuh"

namespace {

__device__ __forceinline__ float mg_exp_diff(float m, float m_new) {
    return (m == -CUDART_INF_F) ? 0.f : __expf(m - m_new);
}

template <bool BF16, int EPL>
__device__ __forceinline__ void mg_unpack(const uint4& r, float* f) {
    if (BF16) {
        f[0] = ax_bf16_lo(r.x); f[1] = ax_bf16_hi(r.x); f[2] = ax_bf16_lo(r.y); f[3] = ax_bf16_hi(r.y);
        f[4] = ax_bf16_lo(r.z); f[5] = ax_bf16_hi(r.z); f[6] = ax_bf16_lo(r.w); f[7] = ax_bf16_hi(r.w);
    } else {
        f[0] = __uint_as_float(r.x); f[1] = __uint_as_float(r.y); f[2] = __uint_as_float(r.z); f[3] = __uint_as_float(r.w);
    }
}

// One warp: norm (optional) + rotate-half RoPE of a 128-vector; lane l holds dims 4l..4l+3.
// The norm weights and the table rows do not depend on the token, so a caller can fetch them
// (mg_rope_consts) before the vector itself is ready.
struct MgRopeConsts { float4 w, cc, sn; };
__device__ __forceinline__ MgRopeConsts mg_rope_consts(const float* nw, const float* c, const float* s) {
    const int lane = threadIdx.x & 31;
    MgRopeConsts k;
    k.w = nw ? reinterpret_cast<const float4*>(nw)[lane] : make_float4(1.f, 1.f, 1.f, 1.f);
    k.cc = c ? reinterpret_cast<const float4*>(c)[lane & 15] : make_float4(1.f, 1.f, 1.f, 1.f);
    k.sn = c ? reinterpret_cast<const float4*>(s)[lane & 15] : make_float4(0.f, 0.f, 0.f, 0.f);
    return k;
}
__device__ __forceinline__ float4 mg_norm_rope_apply(const float* src, bool norm, bool rope, const MgRopeConsts& k, float eps) {
    const int lane = threadIdx.x & 31;
    float4 x = __ldcg(reinterpret_cast<const float4*>(src) + lane);
    if (norm) {
        float ss = x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w;
        ss = ax_warp_sum(ss);
        const float inv = 1.0f / sqrtf(ss / 128.0f + eps);
        x.x = x.x * inv * k.w.x; x.y = x.y * inv * k.w.y; x.z = x.z * inv * k.w.z; x.w = x.w * inv * k.w.w;
    }
    // partner half: dims +64 live 16 lanes away
    float4 o;
    o.x = __shfl_xor_sync(AX_FULL, x.x, 16); o.y = __shfl_xor_sync(AX_FULL, x.y, 16);
    o.z = __shfl_xor_sync(AX_FULL, x.z, 16); o.w = __shfl_xor_sync(AX_FULL, x.w, 16);
    if (rope) {
        if (lane < 16) {           // x = x0 (first half), o = x1
            x.x = x.x * k.cc.x - o.x * k.sn.x; x.y = x.y * k.cc.y - o.y * k.sn.y;
            x.z = x.z * k.cc.z - o.z * k.sn.z; x.w = x.w * k.cc.w - o.w * k.sn.w;
        } else {                   // x = x1 (second half), o = x0
            x.x = o.x * k.sn.x + x.x * k.cc.x; x.y = o.y * k.sn.y + x.y * k.cc.y;
            x.z = o.z * k.sn.z + x.z * k.cc.z; x.w = o.w * k.sn.w + x.w * k.cc.w;
        }
    }
    return x;
}
__device__ __forceinline__ float4 mg_norm_rope_128(const float* src, const float* nw, const float* c, const float* s, float eps) {
    const MgRopeConsts k = mg_rope_consts(nw, c, s);
    return mg_norm_rope_apply(src, nw != nullptr, c != nullptr, k, eps);
}

// Online-softmax update of the running state of GT heads with N new rows (V still packed).
template <bool BF16, int N, int EPL, int GT>
__device__ __forceinline__ void mg_update(float (&m)[GT], float (&l)[GT], float (&acc)[GT][EPL],
                                          const float (&sc)[N][GT], const bool (&valid)[N], const uint4 (&vr)[N]) {
    float p[N][GT];
#pragma unroll
    for (int g = 0; g < GT; g++) {
        float mn = m[g];
#pragma unroll
        for (int u = 0; u < N; u++) mn = fmaxf(mn, sc[u][g]);
        const float corr = (mn == -CUDART_INF_F) ? 1.f : mg_exp_diff(m[g], mn);
        l[g] *= corr;
#pragma unroll
        for (int e = 0; e < EPL; e++) acc[g][e] *= corr;
#pragma unroll
        for (int u = 0; u < N; u++) { p[u][g] = valid[u] ? __expf(sc[u][g] - mn) : 0.f; l[g] += p[u][g]; }
        m[g] = mn;
    }
#pragma unroll
    for (int u = 0; u < N; u++) {
        float vf[EPL]; mg_unpack<BF16, EPL>(vr[u], vf);
#pragma unroll
        for (int g = 0; g < GT; g++)
#pragma unroll
            for (int e = 0; e < EPL; e++) acc[g][e] = fmaf(p[u][g], vf[e], acc[g][e]);
    }
}

// scores of N packed K rows against the GT query vectors held in registers
template <bool BF16, int N, int EPL, int LPR, int GT>
__device__ __forceinline__ void mg_scores(const float (&q)[GT][EPL], const uint4 (&kr)[N], const bool (&valid)[N], float scale,
                                          float (&sc)[N][GT]) {
#pragma unroll
    for (int u = 0; u < N; u++) {
        float kf[EPL]; mg_unpack<BF16, EPL>(kr[u], kf);
#pragma unroll
        for (int g = 0; g < GT; g++) {
            float d = 0.f;
#pragma unroll
            for (int e = 0; e < EPL; e++) d = fmaf(q[g][e], kf[e], d);
#pragma unroll
            for (int o = LPR / 2; o > 0; o >>= 1) d += __shfl_xor_sync(AX_FULL, d, o);
            sc[u][g] = valid[u] ? d * scale : -CUDART_INF_F;
        }
    }
}

// Four query heads per KV head, 16 lanes per cached row (bf16): scores and online softmax with the
// work divided instead of repeated.  A segmented butterfly (5 shuffles per row instead of 16)
// leaves each lane with the finished dot product of ONE head — head (sub >> 2), sub = lane % 16 —
// so that lane alone keeps that head's running maximum and sum and computes its exponentials;
// the probabilities and the rescale factor are then handed to the other lanes by shuffles.
// m_own / l_own: state of this lane's head.  acc: all four heads' partial outputs, as elsewhere.
template <int N, int EPL>
__device__ __forceinline__ void mg_step_g4(const float (&q)[4][EPL], const uint4 (&kr)[N], const uint4 (&vr)[N], const bool (&valid)[N],
                                           float scale, float& m_own, float& l_own, float (&acc)[4][EPL]) {
    const int lane = threadIdx.x & 31;
    const bool b3 = (lane & 8) != 0, b2 = (lane & 4) != 0;
    float s[N];
#pragma unroll
    for (int u = 0; u < N; u++) {
        float kf[EPL]; mg_unpack<true, EPL>(kr[u], kf);
        float d[4];
#pragma unroll
        for (int g = 0; g < 4; g++) {
            float t = 0.f;
#pragma unroll
            for (int e = 0; e < EPL; e++) t = fmaf(q[g][e], kf[e], t);
            d[g] = t;
        }
        const float e0 = (b3 ? d[2] : d[0]) + __shfl_xor_sync(AX_FULL, b3 ? d[0] : d[2], 8);
        const float e1 = (b3 ? d[3] : d[1]) + __shfl_xor_sync(AX_FULL, b3 ? d[1] : d[3], 8);
        float f = (b2 ? e1 : e0) + __shfl_xor_sync(AX_FULL, b2 ? e0 : e1, 4);
        f += __shfl_xor_sync(AX_FULL, f, 2);
        f += __shfl_xor_sync(AX_FULL, f, 1);
        s[u] = valid[u] ? f * scale : -CUDART_INF_F;
    }
    float mn = m_own;
#pragma unroll
    for (int u = 0; u < N; u++) mn = fmaxf(mn, s[u]);
    const float corr = (mn == -CUDART_INF_F) ? 1.f : mg_exp_diff(m_own, mn);
    float p[N];
    l_own *= corr;
#pragma unroll
    for (int u = 0; u < N; u++) { p[u] = valid[u] ? __expf(s[u] - mn) : 0.f; l_own += p[u]; }
    m_own = mn;
    const int half = lane & 16;                            // which 16-lane group of the warp
#pragma unroll
    for (int g = 0; g < 4; g++) {
        const float cg = __shfl_sync(AX_FULL, corr, half | (g << 2));
#pragma unroll
        for (int e = 0; e < EPL; e++) acc[g][e] *= cg;
    }
#pragma unroll
    for (int u = 0; u < N; u++) {
        float vf[EPL]; mg_unpack<true, EPL>(vr[u], vf);
#pragma unroll
        for (int g = 0; g < 4; g++) {
            const float pg = __shfl_sync(AX_FULL, p[u], half | (g << 2));
#pragma unroll
            for (int e = 0; e < EPL; e++) acc[g][e] = fmaf(pg, vf[e], acc[g][e]);
        }
    }
}
// hands every lane the state of all four heads (for the merges that follow the row loop)
__device__ __forceinline__ void mg_expand_g4(float m_own, float l_own, float (&m)[4], float (&l)[4]) {
    const int half = threadIdx.x & 16;
#pragma unroll
    for (int g = 0; g < 4; g++) { m[g] = __shfl_sync(AX_FULL, m_own, half | (g << 2)); l[g] = __shfl_sync(AX_FULL, l_own, half | (g << 2)); }
}

}  // namespace
