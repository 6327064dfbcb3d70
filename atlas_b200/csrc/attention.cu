// attention.cu — decode attention for one new token per sequence.
//
// Replaces decode_attention_kernel / kv_cache_write_kernel / qk_norm_inplace_kernel /
// rope_precomputed_kernel of the reference (kernels/matmul.cu:662-766,786-894).  The reference
// runs one CTA per query head, keeps every score in shared memory (which caps the context),
// walks K rows with one thread per row (uncoalesced) and reads V rows even where masked.
// Here the sequence is split across CTAs (grid = splits × kv-head groups × batch), every
// K/V row is read once with 128-bit loads by the lanes that own those dimensions, the
// softmax is computed online, sliding-window layers touch only the rows inside the window,
// and the last CTA of each head group to finish merges the partial results (ticket counter,
// nothing ever waits).  The KV cache may be bf16 (half the traffic) or f32 (reference format).
#include "attention.cuh"

#include <math_constants.h>

namespace {

constexpr int kAttnThreads = 256;
constexpr int kAttnWarps = kAttnThreads / 32;
constexpr int kUnroll = 4;

struct AttnDev {
    AxAttnArgs a;
    float* partials;       // [batch × n_heads × n_splits × (hd + 2)]
    unsigned* tickets;     // [batch × n_groups], zero between launches
    int g_real;            // query heads per kv head
    int chunks;            // head-group chunks per kv head (g_real / G)
};

__device__ __forceinline__ int attn_pos(const AxAttnArgs& a, int b) {
    return a.pos ? a.pos[a.pos_shared ? 0 : b] : a.pos_scalar;
}
__device__ __forceinline__ void attn_range(const AxAttnArgs& a, int pos, int& t_begin, int& t_end) {
    t_begin = (a.window > 0 && pos - a.window + 1 > 0) ? pos - a.window + 1 : 0;   // pos − t < window
    t_end = pos + 1;
}
__device__ __forceinline__ float safe_exp_diff(float m, float m_new) {     // exp(m − m_new), 0 for m = −inf
    return (m == -CUDART_INF_F) ? 0.f : expf(m - m_new);
}

template <bool BF16, int EPL>
__device__ __forceinline__ void unpack_row(const uint4& r, float* f) {
    if (BF16) {
        f[0] = ax_bf16_lo(r.x); f[1] = ax_bf16_hi(r.x); f[2] = ax_bf16_lo(r.y); f[3] = ax_bf16_hi(r.y);
        f[4] = ax_bf16_lo(r.z); f[5] = ax_bf16_hi(r.z); f[6] = ax_bf16_lo(r.w); f[7] = ax_bf16_hi(r.w);
    } else {
        f[0] = __uint_as_float(r.x); f[1] = __uint_as_float(r.y); f[2] = __uint_as_float(r.z); f[3] = __uint_as_float(r.w);
    }
}

// Merge of per-split states written as (m, l, acc[HD]) — used by both the CTA-level and
// the grid-level combine.
template <int HD>
__device__ __forceinline__ void merge_states(const float* states, int n, int stride, int d, float& M, float& L, float& A) {
    M = -CUDART_INF_F;
    for (int i = 0; i < n; i++) M = fmaxf(M, states[(size_t)i * stride]);
    L = 0.f; A = 0.f;
    for (int i = 0; i < n; i++) {
        const float* s = states + (size_t)i * stride;
        const float w = safe_exp_diff(s[0], M);
        L = fmaf(w, s[1], L);
        A = fmaf(w, s[2 + d], A);
    }
}

template <bool BF16, int HD, int G>
__global__ void __launch_bounds__(kAttnThreads) ax_attn_splitk_kernel(const AttnDev dv) {
    constexpr int EPL = BF16 ? 8 : 4;             // elements per lane (16 bytes)
    constexpr int LPR = HD / EPL;                 // lanes per row
    constexpr int RPW = 32 / LPR;                 // rows per warp pass
    constexpr int SLOTS = kAttnWarps * RPW;
    constexpr int ST = HD + 2;
    static_assert(LPR <= 32 && LPR >= 4, "head_dim / lane width out of range");
    __shared__ float sm[kAttnWarps][G][ST];
    __shared__ int s_last;

    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    const AxAttnArgs& a = dv.a;
    const int split = blockIdx.x, grp = blockIdx.y, b = blockIdx.z;
    const int kh = grp / dv.chunks;
    const int h0 = kh * dv.g_real + (grp % dv.chunks) * G;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int sub = lane % LPR, slot = warp * RPW + lane / LPR;

    const int pos = attn_pos(a, b);
    int tb, te; attn_range(a, pos, tb, te);
    const int rows = te - tb;
    const int per = (rows + a.n_splits - 1) / a.n_splits;
    const int t0 = tb + split * per;
    const int t1 = min(te, t0 + per);

    float q[G][EPL], acc[G][EPL], m[G], l[G];
#pragma unroll
    for (int g = 0; g < G; g++) {
        const float* qp = a.q + ((size_t)b * a.n_heads + h0 + g) * HD + sub * EPL;
#pragma unroll
        for (int e = 0; e < EPL; e += 4) {
            const float4 v = *reinterpret_cast<const float4*>(qp + e);
            q[g][e] = v.x; q[g][e + 1] = v.y; q[g][e + 2] = v.z; q[g][e + 3] = v.w;
        }
#pragma unroll
        for (int e = 0; e < EPL; e++) acc[g][e] = 0.f;
        m[g] = -CUDART_INF_F; l[g] = 0.f;
    }

    const size_t row_stride = (size_t)a.n_kv * HD;          // elements
    const size_t esz = BF16 ? 2 : 4;
    const uint8_t* kbase = (const uint8_t*)a.kc + ((size_t)b * a.seq_stride + (size_t)kh * HD + sub * EPL) * esz;
    const uint8_t* vbase = (const uint8_t*)a.vc + ((size_t)b * a.seq_stride + (size_t)kh * HD + sub * EPL) * esz;

    // warp-uniform trip count: the warp's lowest slot decides
    for (int base = t0; base + warp * RPW < t1; base += SLOTS * kUnroll) {
        uint4 kr[kUnroll], vr[kUnroll];
        bool valid[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; u++) {
            const int t = base + u * SLOTS + slot;
            valid[u] = t < t1;
            if (valid[u]) {
                kr[u] = ax_ldg_stream(kbase + (size_t)t * row_stride * esz);
                vr[u] = ax_ldg_stream(vbase + (size_t)t * row_stride * esz);
            } else { kr[u] = make_uint4(0, 0, 0, 0); vr[u] = make_uint4(0, 0, 0, 0); }
        }
        float s[kUnroll][G];
#pragma unroll
        for (int u = 0; u < kUnroll; u++) {
            float kf[EPL]; unpack_row<BF16, EPL>(kr[u], kf);
#pragma unroll
            for (int g = 0; g < G; g++) {
                float d = 0.f;
#pragma unroll
                for (int e = 0; e < EPL; e++) d = fmaf(q[g][e], kf[e], d);
#pragma unroll
                for (int o = LPR / 2; o > 0; o >>= 1) d += __shfl_xor_sync(AX_FULL, d, o);
                s[u][g] = valid[u] ? d * a.scale : -CUDART_INF_F;
            }
        }
#pragma unroll
        for (int g = 0; g < G; g++) {
            float mn = m[g];
#pragma unroll
            for (int u = 0; u < kUnroll; u++) mn = fmaxf(mn, s[u][g]);
            const float corr = (mn == -CUDART_INF_F) ? 1.f : safe_exp_diff(m[g], mn);
            float p[kUnroll], ps = 0.f;
#pragma unroll
            for (int u = 0; u < kUnroll; u++) { p[u] = valid[u] ? expf(s[u][g] - mn) : 0.f; ps += p[u]; }
            l[g] = fmaf(l[g], corr, ps);
#pragma unroll
            for (int e = 0; e < EPL; e++) acc[g][e] *= corr;
            m[g] = mn;
#pragma unroll
            for (int u = 0; u < kUnroll; u++) { s[u][g] = p[u]; }
        }
#pragma unroll
        for (int u = 0; u < kUnroll; u++) {
            float vf[EPL]; unpack_row<BF16, EPL>(vr[u], vf);
#pragma unroll
            for (int g = 0; g < G; g++)
#pragma unroll
                for (int e = 0; e < EPL; e++) acc[g][e] = fmaf(s[u][g], vf[e], acc[g][e]);
        }
    }

    // merge the row groups that share a warp
#pragma unroll
    for (int o = LPR; o < 32; o <<= 1) {
#pragma unroll
        for (int g = 0; g < G; g++) {
            const float mo = __shfl_xor_sync(AX_FULL, m[g], o);
            const float lo = __shfl_xor_sync(AX_FULL, l[g], o);
            const float mn = fmaxf(m[g], mo);
            const float ca = safe_exp_diff(m[g], mn), cb = safe_exp_diff(mo, mn);
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
        for (int g = 0; g < G; g++) {
            if (sub == 0) { sm[warp][g][0] = m[g]; sm[warp][g][1] = l[g]; }
#pragma unroll
            for (int e = 0; e < EPL; e++) sm[warp][g][2 + sub * EPL + e] = acc[g][e];
        }
    }
    __syncthreads();

    const int S = a.n_splits;
    for (int idx = tid; idx < G * HD; idx += kAttnThreads) {
        const int g = idx / HD, d = idx % HD;
        float M, L, A;
        merge_states<HD>(&sm[0][g][0], kAttnWarps, G * ST, d, M, L, A);
        const int h = h0 + g;
        if (S == 1) {
            a.out[((size_t)b * a.n_heads + h) * HD + d] = A / L;
        } else {
            float* P = dv.partials + (((size_t)b * a.n_heads + h) * S + split) * ST;
            P[2 + d] = A;
            if (d == 0) { P[0] = M; P[1] = L; }
        }
    }
    if (S == 1) return;

    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const unsigned tk = atomicAdd(&dv.tickets[(size_t)b * gridDim.y + grp], 1u);
        s_last = (tk == (unsigned)(S - 1));
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    for (int idx = tid; idx < G * HD; idx += kAttnThreads) {
        const int g = idx / HD, d = idx % HD;
        const int h = h0 + g;
        const float* P = dv.partials + ((size_t)b * a.n_heads + h) * S * ST;
        float M, L, A;
        merge_states<HD>(P, S, ST, d, M, L, A);
        a.out[((size_t)b * a.n_heads + h) * HD + d] = A / L;
    }
    if (tid == 0) dv.tickets[(size_t)b * gridDim.y + grp] = 0u;     // ready for the next launch
}

// Any head_dim ≤ 256 and any group size: one CTA per (query head, sequence), warps over rows,
// lanes over dimensions.  Used for shapes the vectorised kernel does not cover.
__global__ void __launch_bounds__(128) ax_attn_generic_kernel(const AxAttnArgs a) {
    constexpr int W = 4, DMAX = 8;
    __shared__ float sm[W][2 + 256];
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int h = blockIdx.x, b = blockIdx.y;
    const int kh = h / (a.n_heads / a.n_kv);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int hd = a.hd;
    const int pos = attn_pos(a, b);
    int tb, te; attn_range(a, pos, tb, te);
    float q[DMAX], acc[DMAX];
#pragma unroll
    for (int j = 0; j < DMAX; j++) {
        const int d = lane + 32 * j;
        q[j] = d < hd ? a.q[((size_t)b * a.n_heads + h) * hd + d] : 0.f;
        acc[j] = 0.f;
    }
    float m = -CUDART_INF_F, l = 0.f;
    const bool bf = a.kv_dtype == ATLASX_BF16;
    for (int t = tb + warp; t < te; t += W) {
        const size_t off = (size_t)b * a.seq_stride + ((size_t)t * a.n_kv + kh) * hd;
        float kf[DMAX], vf[DMAX];
        float d0 = 0.f;
#pragma unroll
        for (int j = 0; j < DMAX; j++) {
            const int d = lane + 32 * j;
            kf[j] = 0.f; vf[j] = 0.f;
            if (d < hd) {
                kf[j] = bf ? ax_bf16_to_f32(((const uint16_t*)a.kc)[off + d]) : ((const float*)a.kc)[off + d];
                vf[j] = bf ? ax_bf16_to_f32(((const uint16_t*)a.vc)[off + d]) : ((const float*)a.vc)[off + d];
            }
            d0 = fmaf(q[j], kf[j], d0);
        }
        const float s = ax_warp_sum(d0) * a.scale;
        const float mn = fmaxf(m, s);
        const float corr = safe_exp_diff(m, mn), p = expf(s - mn);
        l = fmaf(l, corr, p);
#pragma unroll
        for (int j = 0; j < DMAX; j++) acc[j] = fmaf(p, vf[j], acc[j] * corr);
        m = mn;
    }
    if (lane == 0) { sm[warp][0] = m; sm[warp][1] = l; }
#pragma unroll
    for (int j = 0; j < DMAX; j++) { const int d = lane + 32 * j; if (d < hd) sm[warp][2 + d] = acc[j]; }
    __syncthreads();
    for (int d = tid; d < hd; d += 128) {
        float M = -CUDART_INF_F;
        for (int w = 0; w < W; w++) M = fmaxf(M, sm[w][0]);
        float L = 0.f, A = 0.f;
        for (int w = 0; w < W; w++) { const float c = safe_exp_diff(sm[w][0], M); L = fmaf(c, sm[w][1], L); A = fmaf(c, sm[w][2 + d], A); }
        a.out[((size_t)b * a.n_heads + h) * hd + d] = A / L;
    }
}

// ── QK-norm + RoPE + cache write: one warp per head ──────────────────────────────
__global__ void __launch_bounds__(128) ax_qk_prep_kernel(const AxQkPrepArgs a) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int jobs_per = a.n_heads + 2 * a.n_kv;
    const int job = blockIdx.x * 4 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (job >= jobs_per * a.batch) return;
    const int b = job / jobs_per, j = job % jobs_per;
    const int hd = a.hd, half = hd >> 1;
    const int pos = a.pos ? a.pos[a.pos_shared ? 0 : b] : a.pos_scalar;
    const bool bf = a.kv_dtype == ATLASX_BF16;

    if (j >= a.n_heads + a.n_kv) {                                  // V head: plain copy into the cache
        const int h = j - a.n_heads - a.n_kv;
        const float* src = a.v + (size_t)b * a.kv_in_stride + (size_t)h * hd;
        const size_t off = (size_t)b * a.seq_stride + ((size_t)pos * a.n_kv + h) * hd;
        for (int d = lane; d < hd; d += 32) {
            if (bf) ((uint16_t*)a.vc)[off + d] = ax_f32_to_bf16_rne(src[d]);
            else    ((float*)a.vc)[off + d] = src[d];
        }
        return;
    }
    const bool is_q = j < a.n_heads;
    const int h = is_q ? j : j - a.n_heads;
    const float* src = is_q ? a.q + (size_t)b * a.q_stride + (size_t)h * hd
                            : a.k + (size_t)b * a.kv_in_stride + (size_t)h * hd;
    const float* nw = is_q ? a.q_norm : a.k_norm;
    float inv = 1.f;
    if (nw) {
        float ss = 0.f;
        for (int d = lane; d < hd; d += 32) ss = fmaf(src[d], src[d], ss);
        ss = ax_warp_sum(ss);
        inv = 1.0f / sqrtf(ss / (float)hd + a.eps);
        nw += (size_t)h * hd;
    }
    const float* c = a.cos_t ? a.cos_t + (size_t)pos * half : nullptr;
    const float* s = a.sin_t ? a.sin_t + (size_t)pos * half : nullptr;
    const size_t off = (size_t)b * a.seq_stride + ((size_t)pos * a.n_kv + h) * hd;
    float* qdst = a.q + (size_t)b * a.q_stride + (size_t)h * hd;
    __syncwarp();
    for (int i = lane; i < half; i += 32) {
        float x0 = src[i], x1 = src[i + half];
        if (nw) { x0 = x0 * inv * nw[i]; x1 = x1 * inv * nw[i + half]; }
        float o0 = x0, o1 = x1;
        if (c) { o0 = x0 * c[i] - x1 * s[i]; o1 = x0 * s[i] + x1 * c[i]; }
        if (is_q) { qdst[i] = o0; qdst[i + half] = o1; }
        else if (bf) { ((uint16_t*)a.kc)[off + i] = ax_f32_to_bf16_rne(o0); ((uint16_t*)a.kc)[off + i + half] = ax_f32_to_bf16_rne(o1); }
        else { ((float*)a.kc)[off + i] = o0; ((float*)a.kc)[off + i + half] = o1; }
    }
    if ((hd & 1) && lane == 0) {                                    // odd head_dim: last element is not rotated
        float x = src[hd - 1];
        if (nw) x = x * inv * nw[hd - 1];
        if (is_q) qdst[hd - 1] = x;
        else if (bf) ((uint16_t*)a.kc)[off + hd - 1] = ax_f32_to_bf16_rne(x);
        else ((float*)a.kc)[off + hd - 1] = x;
    }
}

template <bool BF16, int HD, int G>
int launch_splitk(atlasx_ctx* ctx, const AttnDev& dv, bool pdl) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)dv.a.n_splits, (unsigned)(dv.a.n_kv * dv.chunks), (unsigned)dv.a.batch);
    cfg.blockDim = dim3(kAttnThreads);
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    if (pdl) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr; cfg.numAttrs = 1;
    }
    AX_CUDA(cudaLaunchKernelEx(&cfg, ax_attn_splitk_kernel<BF16, HD, G>, dv));
    return ATLASX_OK;
}

template <bool BF16, int HD>
int dispatch_g(atlasx_ctx* ctx, AttnDev& dv, bool pdl) {
    const int gr = dv.g_real;
    if (gr % 4 == 0) { dv.chunks = gr / 4; return launch_splitk<BF16, HD, 4>(ctx, dv, pdl); }
    if (gr % 2 == 0) { dv.chunks = gr / 2; return launch_splitk<BF16, HD, 2>(ctx, dv, pdl); }
    dv.chunks = gr; return launch_splitk<BF16, HD, 1>(ctx, dv, pdl);
}

}  // namespace

int ax_attn_pick_splits(const atlasx_ctx* ctx, int n_kv, int batch, int max_rows) {
    const int want = 2 * ctx->sm_count;                 // two CTAs of this kernel fit per SM
    int s = (want + n_kv * batch - 1) / (n_kv * batch);
    const int cap = (max_rows + 63) / 64;               // at least 64 rows per split
    if (s > cap) s = cap;
    if (s > 64) s = 64;
    if (s < 1) s = 1;
    return s;
}

int ax_attn_launch(atlasx_ctx* ctx, const AxAttnArgs& a, bool pdl) {
    AX_ARG(a.q && a.kc && a.vc && a.out, "null pointer");
    AX_ARG(a.n_heads > 0 && a.n_kv > 0 && a.n_heads % a.n_kv == 0, "n_heads must be a multiple of n_kv_heads");
    AX_ARG(a.hd > 0 && a.hd <= 256, "head_dim must be in 1..256");
    AX_ARG(a.batch >= 1, "batch must be positive");
    const bool fast = (a.hd == 64 || a.hd == 128) && (((uintptr_t)a.q | (uintptr_t)a.kc | (uintptr_t)a.vc) & 15) == 0 &&
                      (a.seq_stride * (a.kv_dtype == ATLASX_BF16 ? 2 : 4)) % 16 == 0;
    if (!fast) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)a.n_heads, (unsigned)a.batch); cfg.blockDim = dim3(128); cfg.stream = ctx->stream;
        cudaLaunchAttribute attr[1];
        if (pdl) {
            attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            attr[0].val.programmaticStreamSerializationAllowed = 1;
            cfg.attrs = attr; cfg.numAttrs = 1;
        }
        AX_CUDA(cudaLaunchKernelEx(&cfg, ax_attn_generic_kernel, a));
        return ATLASX_OK;
    }
    AttnDev dv;
    dv.a = a;
    if (dv.a.n_splits < 1) dv.a.n_splits = 1;
    dv.g_real = a.n_heads / a.n_kv;
    dv.chunks = 1;
    const size_t need_p = (size_t)a.batch * a.n_heads * dv.a.n_splits * (a.hd + 2);
    const size_t need_t = (size_t)a.batch * a.n_heads;      // ≥ batch × groups
    int rc = atlasx_ctx_ensure_attn_scratch(ctx, need_p, need_t);
    if (rc) return rc;
    dv.partials = ctx->attn_partials;
    dv.tickets = ctx->attn_tickets;
    const bool bf = a.kv_dtype == ATLASX_BF16;
    if (bf) return a.hd == 128 ? dispatch_g<true, 128>(ctx, dv, pdl) : dispatch_g<true, 64>(ctx, dv, pdl);
    return a.hd == 128 ? dispatch_g<false, 128>(ctx, dv, pdl) : dispatch_g<false, 64>(ctx, dv, pdl);
}

int ax_qk_prep_launch(atlasx_ctx* ctx, const AxQkPrepArgs& a, bool pdl) {
    AX_ARG(a.q && a.k && a.v && a.kc && a.vc, "null pointer");
    const int jobs = a.batch * (a.n_heads + 2 * a.n_kv);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)((jobs + 3) / 4)); cfg.blockDim = dim3(128); cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    if (pdl) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr; cfg.numAttrs = 1;
    }
    AX_CUDA(cudaLaunchKernelEx(&cfg, ax_qk_prep_kernel, a));
    return ATLASX_OK;
}

// ── decode attention for callers that must not allocate ──────────────────────────
// Some hosts of this library may not call cudaMalloc once they are serving: a process whose
// memory pool was handed out in full at start-up, a latency-critical loop where an allocation
// would synchronise the device, a plugin running inside someone else's allocator.  For them
// the split-K scratch (partial results, tickets, positions) lives in this fixed array instead
// of context memory.  Every GPU that loads the library holds these 4.5 MiB until exit.
namespace {
constexpr size_t kStaticPartialFloats = 1u << 20;          // 4 MiB of split partials
constexpr int kStaticTickets = 4096;                       // ≥ batch × n_heads
constexpr int kStaticPos = 4096;                           // ≥ batch
constexpr size_t kStaticTicketOff = kStaticPartialFloats * sizeof(float);
constexpr size_t kStaticPosOff = kStaticTicketOff + kStaticTickets * sizeof(unsigned);
constexpr size_t kStaticBytes = kStaticPosOff + kStaticPos * sizeof(int);
}
static __device__ __align__(256) unsigned char g_attn_static_scratch[kStaticBytes];

namespace {
struct StaticSetup { unsigned char* base = nullptr; int sm_count = 0; };
StaticSetup g_static_setup[64];

// In host code the array's name is only a handle: the device address has to be asked for,
// once per device, with that device current.
int static_scratch_for_current_device(StaticSetup** out) {
    int dev = -1;
    AX_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return atlasx_fail(ATLASX_ERR_ARG, "device index %d not supported", dev);
    StaticSetup& s = g_static_setup[dev];
    if (!s.base) {
        void* p = nullptr;
        AX_CUDA(cudaGetSymbolAddress(&p, g_attn_static_scratch));
        int sms = 0;
        AX_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
        s.sm_count = sms;
        s.base = (unsigned char*)p;
    }
    *out = &s;
    return ATLASX_OK;
}
}  // namespace

extern "C" int atlasx_decode_attention_static(void* stream, int kv_dtype, const void* k_dev, const void* v_dev,
                                              int max_seq, int n_kv_heads, int head_dim, int batch,
                                              const float* q_dev, float* out_dev, int n_heads,
                                              const int* pos_host, float scale, int window) {
    AX_ARG(k_dev && v_dev && q_dev && out_dev && pos_host, "null pointer");
    AX_ARG(kv_dtype == ATLASX_BF16 || kv_dtype == ATLASX_F32, "kv dtype must be bf16 or f32");
    AX_ARG(max_seq > 0 && n_kv_heads > 0 && batch > 0 && n_heads > 0 && n_heads % n_kv_heads == 0, "bad head or batch counts");
    AX_ARG(head_dim > 0 && head_dim <= 256, "head_dim must be in 1..256");
    AX_ARG(window >= 0, "window must be non-negative");
    if (batch > kStaticPos)
        return atlasx_fail(ATLASX_ERR_ARG, "batch %d exceeds the fixed scratch (max %d sequences)", batch, kStaticPos);
    if ((long long)batch * n_heads > kStaticTickets)
        return atlasx_fail(ATLASX_ERR_ARG, "batch × n_heads = %lld exceeds the fixed scratch (max %d)",
                           (long long)batch * n_heads, kStaticTickets);
    int max_rows = 1;
    for (int b = 0; b < batch; b++) {
        if (pos_host[b] < 0 || pos_host[b] >= max_seq)
            return atlasx_fail(ATLASX_ERR_ARG, "pos[%d] = %d is outside the cache (max_seq %d)", b, pos_host[b], max_seq);
        int r = pos_host[b] + 1;
        if (window > 0 && r > window) r = window;
        if (r > max_rows) max_rows = r;
    }
    StaticSetup* ss = nullptr;
    int rc = static_scratch_for_current_device(&ss);
    if (rc) return rc;
    cudaStream_t s = (cudaStream_t)stream;
    float* partials = (float*)ss->base;
    unsigned* tickets = (unsigned*)(ss->base + kStaticTicketOff);
    int* pos_dev = (int*)(ss->base + kStaticPosOff);
    // tickets must start at zero whatever an earlier, possibly failed, call left behind
    AX_CUDA(cudaMemsetAsync(tickets, 0, (size_t)batch * n_heads * sizeof(unsigned), s));
    AX_CUDA(cudaMemcpyAsync(pos_dev, pos_host, (size_t)batch * sizeof(int), cudaMemcpyHostToDevice, s));

    atlasx_ctx tmp;                       // carries the stream and SM count only; owns nothing
    tmp.stream = s; tmp.sm_count = ss->sm_count;
    AxAttnArgs a;
    a.q = q_dev; a.kc = k_dev; a.vc = v_dev; a.out = out_dev;
    a.seq_stride = (size_t)max_seq * n_kv_heads * head_dim;
    a.pos = pos_dev; a.batch = batch; a.n_heads = n_heads; a.n_kv = n_kv_heads; a.hd = head_dim;
    a.window = window; a.kv_dtype = kv_dtype; a.scale = scale;
    a.n_splits = ax_attn_pick_splits(&tmp, n_kv_heads, batch, max_rows);
    while (a.n_splits > 1 && (size_t)batch * n_heads * a.n_splits * (head_dim + 2) > kStaticPartialFloats) a.n_splits--;

    const bool fast = (head_dim == 64 || head_dim == 128) &&
                      (((uintptr_t)q_dev | (uintptr_t)k_dev | (uintptr_t)v_dev) & 15) == 0 &&
                      (a.seq_stride * (kv_dtype == ATLASX_BF16 ? 2 : 4)) % 16 == 0;
    if (!fast) {                          // the generic kernel needs no scratch at all
        ax_attn_generic_kernel<<<dim3((unsigned)n_heads, (unsigned)batch), 128, 0, s>>>(a);
        AX_CHECK_LAUNCH("ax_attn_generic_kernel");
        return ATLASX_OK;
    }
    AttnDev dv;
    dv.a = a; dv.g_real = n_heads / n_kv_heads; dv.chunks = 1;
    dv.partials = partials; dv.tickets = tickets;
    if (kv_dtype == ATLASX_BF16) return head_dim == 128 ? dispatch_g<true, 128>(&tmp, dv, false) : dispatch_g<true, 64>(&tmp, dv, false);
    return head_dim == 128 ? dispatch_g<false, 128>(&tmp, dv, false) : dispatch_g<false, 64>(&tmp, dv, false);
}
