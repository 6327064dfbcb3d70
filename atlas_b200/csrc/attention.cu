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
#include "attention_device.cuh"

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

// ── fused decode attention, head_dim 128 ─────────────────────────────────────────
// grid = (max_splits, kv heads).  Every thread owns a 16-byte piece of UN rows per stage and a
// private landing slot in shared memory for each (stage, row): cp.async fills the slots, the same
// thread consumes them, so the main loop needs no CTA barrier and NST stages (32 KB per CTA, three
// CTAs per SM) stay in flight without costing registers.  The first NST stages are requested
// before griddepcontrol.wait: rows below `pos` are older than the previous kernel.
constexpr int kFusedUnroll = 2;
constexpr int kFusedStagesDefault = 3;
constexpr int kFusedRowsPerSplit = 128;        // cached rows a split takes at least: with few KV heads per GPU (tensor parallel) 64 made
                                               // twice the splits and a slower merge (4 GPUs: 1.476 → 1.420 ms per token)
__host__ __device__ constexpr size_t fused_land_bytes(int nst) { return (size_t)nst * kFusedUnroll * 2 * kAttnThreads * 16; }

struct FusedDev {
    AxFusedAttnArgs a;
    float* partials;       // [n_heads × max_splits × 130]
    unsigned* tickets;     // [batch × n_kv], zero between launches
    unsigned long long* trace;
    int rows_per_split;    // cached rows a split takes at least
    // operator form (q_ready != null): q is already normed and rotated, the cache already holds row
    // `pos`, grid.z runs over sequences; nothing is prepared or written besides the output
    const float* q_ready; size_t seq_stride; const int* pos_b; int pos_shared; int pos_scalar;
};

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" :: "n"(N) : "memory"); }

template <bool BF16, int G, int NST>
__global__ void __launch_bounds__(kAttnThreads) ax_attn_fused_kernel(const FusedDev dv) {
    constexpr int HD = 128;
    constexpr int EPL = BF16 ? 8 : 4;
    constexpr int LPR = HD / EPL;                 // lanes per cached row: 16 or 32
    constexpr int RPW = 32 / LPR;
    constexpr int SLOTS = kAttnWarps * RPW;       // rows per CTA pass: 16 or 8
    constexpr int UN = kFusedUnroll;
    constexpr int ST = HD + 2;
    extern __shared__ __align__(16) uint8_t fsm[];
    uint4* land = reinterpret_cast<uint4*>(fsm);                     // [NST][UN][K,V][thread]
    float* q_s = reinterpret_cast<float*>(fsm + fused_land_bytes(NST));     // [G][HD]
    float* k_new = q_s + G * HD;
    float* v_new = k_new + HD;
    float* smm = reinterpret_cast<float*>(fsm);                       // [warps][G][ST], reuses the landing slots
    __shared__ int s_last;

    const AxFusedAttnArgs& a = dv.a;
    const int split = blockIdx.x, kh = blockIdx.y, b = blockIdx.z;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int sub = lane % LPR, slot = warp * RPW + lane / LPR;
    const bool prep = dv.q_ready == nullptr;

    ax_trace_start(dv.trace);
    const int pos = prep ? __ldcg(a.pos) : (dv.pos_b ? __ldcg(dv.pos_b + (dv.pos_shared ? 0 : b)) : dv.pos_scalar);
    const int tb = (a.window > 0 && pos - a.window + 1 > 0) ? pos - a.window + 1 : 0;
    const int t_end = prep ? pos : pos + 1;       // fused form: row `pos` comes from shared memory
    const int rows = t_end - tb;                  // cached rows to stream
    int S = (rows + dv.rows_per_split - 1) / dv.rows_per_split;
    S = S < 1 ? 1 : (S > (int)gridDim.x ? (int)gridDim.x : S);
    if (split >= S) return;
    const int per = (rows + S - 1) / S;
    const int t0 = tb + split * per;
    const int t1 = min(t_end, t0 + per);
    const int nstages = (t1 - t0 + SLOTS * UN - 1) / (SLOTS * UN);    // CTA-uniform
    const size_t esz = BF16 ? 2 : 4;
    const size_t row_bytes = (size_t)a.n_kv * HD * esz;
    const uint8_t* kbase = (const uint8_t*)a.kc + ((size_t)b * dv.seq_stride + (size_t)kh * HD + sub * EPL) * esz;
    const uint8_t* vbase = (const uint8_t*)a.vc + ((size_t)b * dv.seq_stride + (size_t)kh * HD + sub * EPL) * esz;

    auto issue = [&](int j) {                     // always commits, so that group counts stay aligned
        if (j < nstages) {
            const int base = t0 + j * SLOTS * UN;
            uint4* dst = land + (size_t)(j % NST) * UN * 2 * kAttnThreads + tid;
#pragma unroll
            for (int u = 0; u < UN; u++) {
                const int t = base + u * SLOTS + slot;
                if (t < t1) {
                    cp_async16(dst + (u * 2 + 0) * kAttnThreads, kbase + (size_t)t * row_bytes);
                    cp_async16(dst + (u * 2 + 1) * kAttnThreads, vbase + (size_t)t * row_bytes);
                }
            }
        }
        cp_async_commit();
    };
#pragma unroll
    for (int j = 0; j < NST; j++) issue(j);

    // norm weights and table rows of this CTA's prep warps: independent of the token as well
    const int half = HD / 2;
    const float* cr = a.cos_t ? a.cos_t + (size_t)pos * half : nullptr;
    const float* sr = a.sin_t ? a.sin_t + (size_t)pos * half : nullptr;
    const int q_rows = a.n_heads * HD, kv_rows = a.n_kv * HD;
    const bool prep_q = prep && warp < G, prep_k = prep && split == 0 && warp == G, prep_v = prep && split == 0 && warp == G + 1;
    MgRopeConsts rc = {};
    const float* nw = nullptr;
    if (prep_q) nw = a.q_norm ? a.q_norm + (size_t)(kh * G + warp) * HD : nullptr;
    if (prep_k) nw = a.k_norm ? a.k_norm + (size_t)kh * HD : nullptr;
    if (prep_q || prep_k) rc = mg_rope_consts(nw, cr, sr);

    asm volatile("griddepcontrol.wait;" ::: "memory");                // the raw QKV vector is complete
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    ax_trace_release(dv.trace);

    // q heads of the group; split 0 also makes the new K and V rows and stores them into the cache
    if (prep_q) {
        const float4 v = mg_norm_rope_apply(a.qkv + (size_t)(kh * G + warp) * HD, nw != nullptr, cr != nullptr, rc, a.qk_eps);
        reinterpret_cast<float4*>(q_s + warp * HD)[lane] = v;
    } else if (prep_k || prep_v) {
        float4 v;
        if (prep_k) v = mg_norm_rope_apply(a.qkv + q_rows + (size_t)kh * HD, nw != nullptr, cr != nullptr, rc, a.qk_eps);
        else        v = __ldcg(reinterpret_cast<const float4*>(a.qkv + q_rows + kv_rows + (size_t)kh * HD) + lane);
        const size_t off = ((size_t)pos * a.n_kv + kh) * HD + lane * 4;
        void* cache = prep_k ? a.kc : a.vc;
        if (BF16) {
            const uint16_t b0 = ax_f32_to_bf16_rne(v.x), b1 = ax_f32_to_bf16_rne(v.y), b2 = ax_f32_to_bf16_rne(v.z), b3 = ax_f32_to_bf16_rne(v.w);
            *reinterpret_cast<uint2*>(reinterpret_cast<uint16_t*>(cache) + off) =
                make_uint2((uint32_t)b0 | ((uint32_t)b1 << 16), (uint32_t)b2 | ((uint32_t)b3 << 16));
            v = make_float4(ax_bf16_to_f32(b0), ax_bf16_to_f32(b1), ax_bf16_to_f32(b2), ax_bf16_to_f32(b3));
        } else {
            *reinterpret_cast<float4*>(reinterpret_cast<float*>(cache) + off) = v;
        }
        reinterpret_cast<float4*>(prep_k ? k_new : v_new)[lane] = v;
    } else if (!prep && warp < G) {
        reinterpret_cast<float4*>(q_s + warp * HD)[lane] =
            __ldcg(reinterpret_cast<const float4*>(dv.q_ready + ((size_t)b * a.n_heads + kh * G + warp) * HD) + lane);
    }
    __syncthreads();
    ax_trace_staged(dv.trace);

    float q[G][EPL], acc[G][EPL], m[G], l[G];
#pragma unroll
    for (int g = 0; g < G; g++) {
#pragma unroll
        for (int e = 0; e < EPL; e++) { q[g][e] = q_s[g * HD + sub * EPL + e]; acc[g][e] = 0.f; }
        m[g] = -CUDART_INF_F; l[g] = 0.f;
    }

    for (int j = 0; j < nstages; j++) {
        cp_async_wait<NST - 1>();                 // stage j of this thread has landed
        const int base = t0 + j * SLOTS * UN;
        const uint4* src = land + (size_t)(j % NST) * UN * 2 * kAttnThreads + tid;
        uint4 kr[UN], vr[UN]; bool valid[UN];
#pragma unroll
        for (int u = 0; u < UN; u++) {
            valid[u] = base + u * SLOTS + slot < t1;
            if (valid[u]) { kr[u] = src[(u * 2 + 0) * kAttnThreads]; vr[u] = src[(u * 2 + 1) * kAttnThreads]; }
            else { kr[u] = make_uint4(0, 0, 0, 0); vr[u] = make_uint4(0, 0, 0, 0); }
        }
        issue(j + NST);                           // refill the slots just read
        float sc[UN][G];
        if constexpr (G == 4 && BF16) {
            mg_step_g4<UN, EPL>(q, kr, vr, valid, a.scale, m[0], l[0], acc);          // m[0], l[0]: this lane's own head
        } else {
            mg_scores<BF16, UN, EPL, LPR, G>(q, kr, valid, a.scale, sc);
            mg_update<BF16, UN, EPL, G>(m, l, acc, sc, valid, vr);
        }
    }
    cp_async_wait<0>();

    // the new row itself (split 0, first lane group of warp 0)
    if (prep && split == 0 && warp == 0) {
        uint4 k1[1], v1[1]; bool ok1[1] = { lane / LPR == 0 };
        float sc[1][G];
        const float* kp = k_new + sub * EPL; const float* vp = v_new + sub * EPL;
        if (BF16) {
            k1[0] = make_uint4(__float_as_uint(kp[0]) >> 16 | (__float_as_uint(kp[1]) & 0xFFFF0000u), __float_as_uint(kp[2]) >> 16 | (__float_as_uint(kp[3]) & 0xFFFF0000u),
                               __float_as_uint(kp[4]) >> 16 | (__float_as_uint(kp[5]) & 0xFFFF0000u), __float_as_uint(kp[6]) >> 16 | (__float_as_uint(kp[7]) & 0xFFFF0000u));
            v1[0] = make_uint4(__float_as_uint(vp[0]) >> 16 | (__float_as_uint(vp[1]) & 0xFFFF0000u), __float_as_uint(vp[2]) >> 16 | (__float_as_uint(vp[3]) & 0xFFFF0000u),
                               __float_as_uint(vp[4]) >> 16 | (__float_as_uint(vp[5]) & 0xFFFF0000u), __float_as_uint(vp[6]) >> 16 | (__float_as_uint(vp[7]) & 0xFFFF0000u));
        } else {
            k1[0] = *reinterpret_cast<const uint4*>(kp);
            v1[0] = *reinterpret_cast<const uint4*>(vp);
        }
        if constexpr (G == 4 && BF16) {
            mg_step_g4<1, EPL>(q, k1, v1, ok1, a.scale, m[0], l[0], acc);
        } else {
            mg_scores<BF16, 1, EPL, LPR, G>(q, k1, ok1, a.scale, sc);
            mg_update<BF16, 1, EPL, G>(m, l, acc, sc, ok1, v1);
        }
    }
    if constexpr (G == 4 && BF16) {
        const float mo = m[0], lo = l[0];
        mg_expand_g4(mo, lo, m, l);
    }

    // merge lane groups of a warp, then warps, then (last CTA of the kv head) the splits
#pragma unroll
    for (int o = LPR; o < 32; o <<= 1) {
#pragma unroll
        for (int g = 0; g < G; g++) {
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
    __syncthreads();                              // every thread is done with its landing slots
    if (lane < LPR) {
#pragma unroll
        for (int g = 0; g < G; g++) {
            float* dst = smm + ((size_t)warp * G + g) * ST;
            if (sub == 0) { dst[0] = m[g]; dst[1] = l[g]; }
#pragma unroll
            for (int e = 0; e < EPL; e++) dst[2 + sub * EPL + e] = acc[g][e];
        }
    }
    __syncthreads();
    const int SP = (int)gridDim.x;                // partial slots per head
    for (int idx = tid; idx < G * HD; idx += kAttnThreads) {
        const int g = idx / HD, d = idx % HD;
        float M, L, A;
        merge_states<HD>(smm + (size_t)g * ST, kAttnWarps, G * ST, d, M, L, A);
        const size_t h = (size_t)b * a.n_heads + kh * G + g;
        if (S == 1) {
            a.out[h * HD + d] = A / L;
        } else {
            float* P = dv.partials + (h * SP + split) * ST;
            P[2 + d] = A;
            if (d == 0) { P[0] = M; P[1] = L; }
        }
    }
    ax_trace_end(dv.trace);
    if (S == 1) return;
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const unsigned tk = atomicAdd(&dv.tickets[b * gridDim.y + kh], 1u);
        s_last = (tk == (unsigned)(S - 1));
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    for (int idx = tid; idx < G * HD; idx += kAttnThreads) {
        const int g = idx / HD, d = idx % HD;
        const size_t h = (size_t)b * a.n_heads + kh * G + g;
        float M, L, A;
        merge_states<HD>(dv.partials + h * SP * ST, S, ST, d, M, L, A);
        a.out[h * HD + d] = A / L;
    }
    if (tid == 0) dv.tickets[b * gridDim.y + kh] = 0u;            // ready for the next launch
    ax_trace_end(dv.trace);
}

template <bool BF16, int G, int NST>
int launch_fused_n(atlasx_ctx* ctx, const FusedDev& dv, bool pdl, int batch) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)dv.a.max_splits, (unsigned)dv.a.n_kv, (unsigned)batch);
    cfg.blockDim = dim3(kAttnThreads);
    cfg.dynamicSmemBytes = fused_land_bytes(NST) + (size_t)(G + 2) * 128 * 4;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[2];
    int na = 0;
    if (pdl) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        na++;
    }
    if (ctx->carveout >= 0) {
        attr[na].id = cudaLaunchAttributePreferredSharedMemoryCarveout;
        attr[na].val.sharedMemCarveout = (unsigned)ctx->carveout;
        na++;
    }
    if (na) { cfg.attrs = attr; cfg.numAttrs = na; }
    AX_CUDA(cudaLaunchKernelEx(&cfg, ax_attn_fused_kernel<BF16, G, NST>, dv));
    return ATLASX_OK;
}
int g_fused_stages = kFusedStagesDefault;       // 2..4; ATLASX_ATTN_STAGES overrides (experiments)

// Inside a decode step three stages are best (the kernel shares the SM with its GEMV neighbours);
// the stand-alone operator streams with four.
template <bool BF16, int G>
int launch_fused(atlasx_ctx* ctx, const FusedDev& dv, bool pdl, int batch = 1) {
    switch (dv.q_ready ? 4 : g_fused_stages) {
        case 4:  return launch_fused_n<BF16, G, 4>(ctx, dv, pdl, batch);
        case 2:  return launch_fused_n<BF16, G, 2>(ctx, dv, pdl, batch);
        default: return launch_fused_n<BF16, G, 3>(ctx, dv, pdl, batch);
    }
}

template <bool BF16, int G>
int fused_attr() {
    AX_CUDA(cudaFuncSetAttribute(ax_attn_fused_kernel<BF16, G, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(fused_land_bytes(2) + (size_t)(G + 2) * 128 * 4)));
    AX_CUDA(cudaFuncSetAttribute(ax_attn_fused_kernel<BF16, G, 3>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(fused_land_bytes(3) + (size_t)(G + 2) * 128 * 4)));
    AX_CUDA(cudaFuncSetAttribute(ax_attn_fused_kernel<BF16, G, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(fused_land_bytes(4) + (size_t)(G + 2) * 128 * 4)));
    return ATLASX_OK;
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
    const int want = 3 * ctx->sm_count;                 // about three CTAs of these kernels fit per SM
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
    const int g_real = a.n_heads / a.n_kv;
    if (a.hd == 128 && (g_real == 1 || g_real == 2 || g_real == 4) && (((uintptr_t)a.out) & 15) == 0) {
        // head_dim 128: the landing-slot kernel in its operator form
        FusedDev fd;
        fd.a.kc = const_cast<void*>(a.kc); fd.a.vc = const_cast<void*>(a.vc); fd.a.out = a.out;
        fd.a.n_heads = a.n_heads; fd.a.n_kv = a.n_kv; fd.a.window = a.window; fd.a.kv_dtype = a.kv_dtype; fd.a.scale = a.scale;
        int sp = a.n_splits < 1 ? 1 : (a.n_splits > 64 ? 64 : a.n_splits);
        fd.a.max_splits = sp;
        if (a.scratch_partials && a.scratch_tickets) { fd.partials = a.scratch_partials; fd.tickets = a.scratch_tickets; }
        else {
            int rc2 = atlasx_ctx_ensure_attn_scratch(ctx, (size_t)a.batch * a.n_heads * sp * (128 + 2), (size_t)a.batch * a.n_heads);
            if (rc2) return rc2;
            fd.partials = ctx->attn_partials; fd.tickets = ctx->attn_tickets;
        }
        fd.trace = nullptr;
        fd.rows_per_split = kFusedRowsPerSplit;
        fd.q_ready = a.q; fd.seq_stride = a.seq_stride; fd.pos_b = a.pos; fd.pos_shared = a.pos_shared; fd.pos_scalar = a.pos_scalar;
        if (a.kv_dtype == ATLASX_BF16)
            return g_real == 1 ? launch_fused<true, 1>(ctx, fd, pdl, a.batch) : g_real == 2 ? launch_fused<true, 2>(ctx, fd, pdl, a.batch)
                                                                                          : launch_fused<true, 4>(ctx, fd, pdl, a.batch);
        return g_real == 1 ? launch_fused<false, 1>(ctx, fd, pdl, a.batch) : g_real == 2 ? launch_fused<false, 2>(ctx, fd, pdl, a.batch)
                                                                                       : launch_fused<false, 4>(ctx, fd, pdl, a.batch);
    }
    AttnDev dv;
    dv.a = a;
    if (dv.a.n_splits < 1) dv.a.n_splits = 1;
    dv.g_real = a.n_heads / a.n_kv;
    dv.chunks = 1;
    const size_t need_p = (size_t)a.batch * a.n_heads * dv.a.n_splits * (a.hd + 2);
    const size_t need_t = (size_t)a.batch * a.n_heads;      // ≥ batch × groups
    if (a.scratch_partials && a.scratch_tickets) { dv.partials = a.scratch_partials; dv.tickets = a.scratch_tickets; }
    else {
        int rc = atlasx_ctx_ensure_attn_scratch(ctx, need_p, need_t);
        if (rc) return rc;
        dv.partials = ctx->attn_partials;
        dv.tickets = ctx->attn_tickets;
    }
    const bool bf = a.kv_dtype == ATLASX_BF16;
    if (bf) return a.hd == 128 ? dispatch_g<true, 128>(ctx, dv, pdl) : dispatch_g<true, 64>(ctx, dv, pdl);
    return a.hd == 128 ? dispatch_g<false, 128>(ctx, dv, pdl) : dispatch_g<false, 64>(ctx, dv, pdl);
}

bool ax_attn_fused_supported(int hd, int n_heads, int n_kv) {
    if (hd != 128 || n_kv <= 0 || n_heads % n_kv) return false;
    const int g = n_heads / n_kv;
    return g == 1 || g == 2 || g == 4;
}
int ax_attn_fused_max_splits(const atlasx_ctx* ctx, int n_kv, int max_rows) {
    // one wave of CTAs
    const int rps = ctx->tune.attn_rows > 0 ? ctx->tune.attn_rows : kFusedRowsPerSplit;
    int s = (max_rows + rps - 1) / rps;
    const int per_sm = ctx->tune.attn_wave;      // 2 measured best with three landing stages (48 KB per CTA)
    const int wave = (per_sm * ctx->sm_count) / (n_kv > 0 ? n_kv : 1);
    if (s > wave) s = wave;
    return s < 1 ? 1 : (s > 64 ? 64 : s);
}
int ax_attn_init(atlasx_ctx* ctx) {
    int rc;
    g_fused_stages = ctx->tune.attn_stages;
    if ((rc = fused_attr<true, 1>()) || (rc = fused_attr<true, 2>()) || (rc = fused_attr<true, 4>())) return rc;
    if ((rc = fused_attr<false, 1>()) || (rc = fused_attr<false, 2>()) || (rc = fused_attr<false, 4>())) return rc;
    return ATLASX_OK;
}
int ax_attn_fused_launch(atlasx_ctx* ctx, const AxFusedAttnArgs& a, bool pdl) {
    AX_ARG(a.qkv && a.kc && a.vc && a.out && a.pos, "null pointer");
    AX_ARG(ax_attn_fused_supported(128, a.n_heads, a.n_kv), "fused attention needs 1, 2 or 4 query heads per KV head");
    AX_ARG(a.max_splits >= 1 && a.max_splits <= 64, "max_splits must be in 1..64");
    AX_ARG((((uintptr_t)a.qkv | (uintptr_t)a.kc | (uintptr_t)a.vc | (uintptr_t)a.out) & 15) == 0, "buffers must be 16-byte aligned");
    FusedDev dv;
    dv.a = a;
    if (a.scratch_partials && a.scratch_tickets) { dv.partials = a.scratch_partials; dv.tickets = a.scratch_tickets; }
    else {
        int rc = atlasx_ctx_ensure_attn_scratch(ctx, (size_t)a.n_heads * a.max_splits * (128 + 2), (size_t)a.n_heads);
        if (rc) return rc;
        dv.partials = ctx->attn_partials;
        dv.tickets = ctx->attn_tickets;
    }
    dv.trace = nullptr;
    dv.rows_per_split = ctx->tune.attn_rows > 0 ? ctx->tune.attn_rows : kFusedRowsPerSplit;
    dv.q_ready = nullptr; dv.seq_stride = 0; dv.pos_b = nullptr; dv.pos_shared = 1; dv.pos_scalar = 0;
    if (ctx->trace_next) { dv.trace = ctx->trace_next; ctx->trace_next += 6; }
    const int g = a.n_heads / a.n_kv;
    if (a.kv_dtype == ATLASX_BF16)
        return g == 1 ? launch_fused<true, 1>(ctx, dv, pdl) : g == 2 ? launch_fused<true, 2>(ctx, dv, pdl) : launch_fused<true, 4>(ctx, dv, pdl);
    return g == 1 ? launch_fused<false, 1>(ctx, dv, pdl) : g == 2 ? launch_fused<false, 2>(ctx, dv, pdl) : launch_fused<false, 4>(ctx, dv, pdl);
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
