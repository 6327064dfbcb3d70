// attention_mma.cu — GQA decode attention on the tensor cores (bf16 cache, head_dim 128, 3..8
// query heads per KV head).
//
// With several query heads per KV head the scalar kernels of attention.cu are bound by
// instruction issue, not by HBM: every cached row costs 128·G multiply-adds twice.  Here the
// cached rows are the 16-row A operand of mma.sync m16n8k16 and the query heads of a KV head the 8
// columns of B, so a 32-row tile of K and V costs a warp 32 tensor instructions (up to four heads;
// 64 for five to eight) instead of ~8000 scalar ones.  Semantics are those of decode_attention_kernel of the reference
// (kernels/matmul.cu:786-894): kv head = head / group, rows pos − t ≥ window masked, softmax over
// the rest — computed flash-decoding style (online softmax, sequence split across CTAs and merged
// by the last CTA of a head group).
//   * Each of the four warps of a CTA streams its own 32-row tiles: cp.async into warp-private
//     shared memory (three stages, rows padded to 272 bytes so that ldmatrix is conflict-free),
//     no CTA barrier in the loop.
//   * Accuracy: K and V are bf16 already, so products with them are exact in the f32 accumulator;
//     the f32 queries and probabilities enter as hi + lo bf16 pairs (two MMAs each), which leaves
//     an error of 2⁻¹⁷ relative — far inside the 1e-3 parity bound.
#include <math_constants.h>

#include "attention.cuh"
#include "attention_mma.cuh"

namespace {

constexpr int kWarps = 6;                      // chunk kernel; the operator kernel takes its shape as template arguments
constexpr int kThreads = kWarps * 32;
constexpr int kTileRows = 32;                  // cached rows per warp tile
constexpr int kPitch = 272;                    // bytes per staged row: 256 + 16, shifts rows across the banks
constexpr int kStages = 2;
constexpr int kTileBytes = kTileRows * kPitch; // one of K or V
constexpr int kStageBytes = 2 * kTileBytes;
constexpr int kWarpBytes = kStages * kStageBytes;
constexpr int kST = 130;                       // partial state: m, l, 128 outputs
constexpr int kChunkMaxSplits = 16;

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16_zfill(uint32_t dst, const void* src, bool valid) {
    const int n = valid ? 16 : 0;              // 0 source bytes: the 16 destination bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" :: "r"(dst), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
// D += A·B, A 16×16 bf16 (rows 8..15 of A are zero here: a1 = a3 = 0), B 16×8 bf16, f32 accumulate
__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_bf16_full(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// two floats → (hi pair, lo pair) of bf16, x = hi + lo to 2⁻¹⁷; first argument in the low half
__device__ __forceinline__ void split2(float x, float y, uint32_t& hi, uint32_t& lo) {
    const uint16_t hx = ax_f32_to_bf16_rne(x), hy = ax_f32_to_bf16_rne(y);
    const uint16_t lx = ax_f32_to_bf16_rne(x - ax_bf16_to_f32(hx)), ly = ax_f32_to_bf16_rne(y - ax_bf16_to_f32(hy));
    hi = (uint32_t)hx | ((uint32_t)hy << 16);
    lo = (uint32_t)lx | ((uint32_t)ly << 16);
}
__device__ __forceinline__ float fast_exp2(float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }

struct MmaDev {
    const float* q; const uint16_t* kc; const uint16_t* vc; float* out;
    size_t seq_stride;              // elements between sequences of the cache
    const int* pos; int pos_shared; int pos_scalar;
    int n_heads, n_kv, g, window, n_splits;
    float scale;
    float* partials; unsigned* tickets;
};

__device__ __forceinline__ float merge_exp(float m, float M) { return (m == -CUDART_INF_F) ? 0.f : expf(m - M); }

// movmatrix: transposes an 8×8 matrix of 16-bit elements held one 32-bit register per lane
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
    return d;
}
__device__ __forceinline__ void mma_bf16_4(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Operand roles.  The MMAs of a tile depend on one another (scores, softmax, output) and a warp gets each
// back after tens of clocks, so the kernel is built to issue as few of them per byte as possible: the
// cached rows are the 16-row A operand and the query heads the 8 columns of B.
//   Sᵀ[16 keys × 8 cols] = K[16 keys × 16 dims]·Qᵀ[16 dims × 8 cols]      (A by ldmatrix from the staged K rows)
//   Oᵀ[16 dims × 8 cols] = Vᵀ[16 dims × 16 keys]·Pᵀ[16 keys × 8 cols]     (A by ldmatrix.trans from the staged V rows,
//                                                                           B from the Sᵀ fragments by movmatrix)
// PACK (≤ 4 heads per KV head): columns 0..3 carry the bf16 hi parts of the heads' queries (and
// probabilities), columns 4..7 the lo parts, so ONE MMA yields both products — 32 MMAs per 32-row
// tile where the heads-as-rows form needs 128.  Otherwise (5..8 heads) columns are heads and the hi
// and lo products are two MMAs into the same accumulator.
template <bool PACK, int WARPS, int STAGES, int TR>
__global__ void __launch_bounds__(WARPS * 32) ax_attn_mma_kernel(const MmaDev dv) {
    constexpr int kWarps = WARPS, kThreads = WARPS * 32, kStages = STAGES, kTileRows = TR;      // TR: 16 or 32 cached rows per warp tile
    constexpr int kTileBytes = TR * kPitch, kStageBytes = 2 * kTileBytes, kWarpBytes = STAGES * kStageBytes;
    constexpr int kMT = TR / 16;
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ int s_last;
    const int split = blockIdx.x, kh = blockIdx.y, b = blockIdx.z;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = dv.g;
    const int quad = lane >> 2, qi = lane & 3;
    // this thread's two columns 2·qi, 2·qi + 1 belong to heads hA, hA + 1; with PACK lanes qi ≥ 2 hold the lo parts
    const int hA = PACK ? 2 * (qi & 1) : 2 * qi;
    const bool lo_part = PACK && qi >= 2;

    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    const int pos = dv.pos ? dv.pos[dv.pos_shared ? 0 : b] : dv.pos_scalar;
    const int tb = (dv.window > 0 && pos - dv.window + 1 > 0) ? pos - dv.window + 1 : 0;      // pos − t < window
    const int te = pos + 1;
    const int rows = te - tb;
    const int tiles_all = (rows + kTileRows - 1) / kTileRows;
    int S = dv.n_splits; if (S > tiles_all) S = tiles_all; if (S < 1) S = 1;
    if (split >= S) return;
    const int tile0 = (int)((long long)tiles_all * split / S), tile1 = (int)((long long)tiles_all * (split + 1) / S);
    const int t0 = tb + tile0 * kTileRows, t1 = min(te, tb + tile1 * kTileRows);
    const int n_tiles = tile1 - tile0;                        // of this CTA; warp w takes tiles w, w + 4, …
    const int my_tiles = n_tiles > warp ? (n_tiles - warp + kWarps - 1) / kWarps : 0;

    // ── B fragments of Qᵀ: column `quad`, dims 16·ks + 2·qi + {0,1} and + 8; scaled by scale·log2 e, hi / lo ──
    uint32_t qb[8][2], qb2[PACK ? 1 : 8][2];                  // qb2: the lo parts when columns are heads
    {
        const float sc = dv.scale * 1.4426950408889634f;
        const int head = PACK ? (quad & 3) : quad;
        const bool want_lo = PACK && quad >= 4;
        const bool ok = head < G;
        const float* qp = dv.q + ((size_t)b * dv.n_heads + (size_t)kh * G + (ok ? head : 0)) * 128;
#pragma unroll
        for (int ks = 0; ks < 8; ks++) {
            float2 v0 = make_float2(0.f, 0.f), v1 = make_float2(0.f, 0.f);
            if (ok) {
                v0 = *reinterpret_cast<const float2*>(qp + ks * 16 + qi * 2);
                v1 = *reinterpret_cast<const float2*>(qp + ks * 16 + 8 + qi * 2);
            }
            uint32_t h0, l0, h1, l1;
            split2(v0.x * sc, v0.y * sc, h0, l0);
            split2(v1.x * sc, v1.y * sc, h1, l1);
            if (PACK) { qb[ks][0] = want_lo ? l0 : h0; qb[ks][1] = want_lo ? l1 : h1; }
            else { qb[ks][0] = h0; qb[ks][1] = h1; qb2[ks][0] = l0; qb2[ks][1] = l1; }
        }
    }

    uint8_t* wbase = smem + (size_t)warp * kWarpBytes;
    const size_t row_elems = (size_t)dv.n_kv * 128;
    const uint16_t* kg = dv.kc + (size_t)b * dv.seq_stride + (size_t)kh * 128;
    const uint16_t* vg = dv.vc + (size_t)b * dv.seq_stride + (size_t)kh * 128;
    // tile j of this warp → stage j % kStages; each lane copies TR/2 pieces of K and as many of V (row = 2i + lane/16, piece = lane % 16)
    auto issue = [&](int j) {
        if (j < my_tiles) {
            const int tt = t0 + (warp + j * kWarps) * kTileRows;
            uint8_t* st = wbase + (size_t)(j % kStages) * kStageBytes;
            const int piece = lane & 15;
#pragma unroll
            for (int i = 0; i < TR / 2; i++) {
                const int r = i * 2 + (lane >> 4);
                const int t = tt + r;
                const bool ok = t < t1;
                const size_t go = (size_t)(ok ? t : t0) * row_elems + piece * 8;
                cp_async16_zfill(smem_addr(st + r * kPitch + piece * 16), kg + go, ok);
                cp_async16_zfill(smem_addr(st + kTileBytes + r * kPitch + piece * 16), vg + go, ok);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
#pragma unroll
    for (int j = 0; j < kStages - 1; j++) issue(j);

    float ot[8][4];                                           // Oᵀ: 8 blocks of 16 dims × this thread's two columns
#pragma unroll
    for (int md = 0; md < 8; md++) { ot[md][0] = ot[md][1] = ot[md][2] = ot[md][3] = 0.f; }
    float m_run[2] = { -CUDART_INF_F, -CUDART_INF_F }, l_run[2] = { 0.f, 0.f };     // heads hA, hA + 1 (log2 domain); l: this lane's keys

    for (int j = 0; j < my_tiles; j++) {
        asm volatile("cp.async.wait_group %0;" :: "n"(kStages - 2) : "memory");
        __syncwarp();                                         // tile j has landed for every lane; tile j − 1 is consumed
        issue(j + kStages - 1);                               // into the stage tile j − 1 occupied
        const int tt = t0 + (warp + j * kWarps) * kTileRows;
        const uint8_t* st = wbase + (size_t)(j % kStages) * kStageBytes;
        const uint32_t ks_addr = smem_addr(st), vs_addr = smem_addr(st + kTileBytes);

        // ── Sᵀ: two blocks of 16 keys, 8 steps of 16 dims ──
        float sT[kMT][4];
#pragma unroll
        for (int mt = 0; mt < kMT; mt++) { sT[mt][0] = sT[mt][1] = sT[mt][2] = sT[mt][3] = 0.f; }
#pragma unroll
        for (int ks = 0; ks < 8; ks++) {
#pragma unroll
            for (int mt = 0; mt < kMT; mt++) {
                // matrices: (keys 0-7, dims 0-7) (keys 8-15, dims 0-7) (keys 0-7, dims 8-15) (keys 8-15, dims 8-15) of the block
                uint32_t a0, a1, a2, a3;
                ldsm_x4(ks_addr + (mt * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * kPitch + ks * 32 + (lane >> 4) * 16, a0, a1, a2, a3);
                mma_bf16_4(sT[mt], a0, a1, a2, a3, qb[ks][0], qb[ks][1]);
                if (!PACK) mma_bf16_4(sT[mt], a0, a1, a2, a3, qb2[ks][0], qb2[ks][1]);
            }
        }
        if (PACK) {                                            // hi columns + lo columns: lanes qi and qi ^ 2
#pragma unroll
            for (int mt = 0; mt < kMT; mt++)
#pragma unroll
                for (int e = 0; e < 4; e++) sT[mt][e] += __shfl_xor_sync(AX_FULL, sT[mt][e], 2);
        }
        // ── online softmax of heads hA (elements 0, 2) and hA + 1 (elements 1, 3); keys tt + 16·mt + quad (+ 8) ──
        float mx[2] = { -CUDART_INF_F, -CUDART_INF_F };
#pragma unroll
        for (int mt = 0; mt < kMT; mt++) {
            const int k0 = tt + mt * 16 + quad;
            if (k0 >= t1) { sT[mt][0] = -CUDART_INF_F; sT[mt][1] = -CUDART_INF_F; }
            if (k0 + 8 >= t1) { sT[mt][2] = -CUDART_INF_F; sT[mt][3] = -CUDART_INF_F; }
            mx[0] = fmaxf(mx[0], fmaxf(sT[mt][0], sT[mt][2]));
            mx[1] = fmaxf(mx[1], fmaxf(sT[mt][1], sT[mt][3]));
        }
        float corr[2], m_use[2];
#pragma unroll
        for (int h = 0; h < 2; h++) {
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(AX_FULL, mx[h], 4));
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(AX_FULL, mx[h], 8));
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(AX_FULL, mx[h], 16));
            const float m_new = fmaxf(m_run[h], mx[h]);
            m_use[h] = (m_new == -CUDART_INF_F) ? 0.f : m_new;
            corr[h] = fast_exp2(m_run[h] - m_use[h]);         // 0 for the first tile (m_run = −inf)
            m_run[h] = m_new;
            l_run[h] *= corr[h];
        }
        // probabilities → B fragments of Pᵀ (k = keys, n = columns) through movmatrix
        uint32_t pb[kMT][2], pb2[PACK ? 1 : kMT][2];              // [16-key block][keys 0-7 | keys 8-15]; pb2: lo parts when columns are heads
#pragma unroll
        for (int mt = 0; mt < kMT; mt++) {
            const float p0 = fast_exp2(sT[mt][0] - m_use[0]), p1 = fast_exp2(sT[mt][1] - m_use[1]);
            const float p2 = fast_exp2(sT[mt][2] - m_use[0]), p3 = fast_exp2(sT[mt][3] - m_use[1]);
            l_run[0] += p0 + p2; l_run[1] += p1 + p3;
            uint32_t h01, l01, h23, l23;
            split2(p0, p1, h01, l01);
            split2(p2, p3, h23, l23);
            if (PACK) {
                pb[mt][0] = movmatrix_trans(lo_part ? l01 : h01);
                pb[mt][1] = movmatrix_trans(lo_part ? l23 : h23);
            } else {
                pb[mt][0] = movmatrix_trans(h01); pb[mt][1] = movmatrix_trans(h23);
                pb2[mt][0] = movmatrix_trans(l01); pb2[mt][1] = movmatrix_trans(l23);
            }
        }
#pragma unroll
        for (int md = 0; md < 8; md++) { ot[md][0] *= corr[0]; ot[md][1] *= corr[1]; ot[md][2] *= corr[0]; ot[md][3] *= corr[1]; }
        // ── Oᵀ += Vᵀ·Pᵀ: 8 blocks of 16 dims, 2 steps of 16 keys ──
#pragma unroll
        for (int kk = 0; kk < kMT; kk++) {
#pragma unroll
            for (int md = 0; md < 8; md++) {
                // stored matrices (rows = keys): (keys 0-7, dims 0-7) (keys 0-7, dims 8-15) (keys 8-15, dims 0-7) (keys 8-15, dims 8-15);
                // transposed on load they are a0..a3 of Vᵀ
                uint32_t a0, a1, a2, a3;
                ldsm_x4_trans(vs_addr + (kk * 16 + (lane >> 4) * 8 + (lane & 7)) * kPitch + md * 32 + ((lane >> 3) & 1) * 16, a0, a1, a2, a3);
                mma_bf16_4(ot[md], a0, a1, a2, a3, pb[kk][0], pb[kk][1]);
                if (!PACK) mma_bf16_4(ot[md], a0, a1, a2, a3, pb2[kk][0], pb2[kk][1]);
            }
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");

    // ── merge the warps, then (last CTA of the head group) the splits ──
#pragma unroll
    for (int h = 0; h < 2; h++) {
        l_run[h] += __shfl_xor_sync(AX_FULL, l_run[h], 4);
        l_run[h] += __shfl_xor_sync(AX_FULL, l_run[h], 8);
        l_run[h] += __shfl_xor_sync(AX_FULL, l_run[h], 16);
    }
    if (PACK) {                                                // hi columns + lo columns of the output
#pragma unroll
        for (int md = 0; md < 8; md++)
#pragma unroll
            for (int e = 0; e < 4; e++) ot[md][e] += __shfl_xor_sync(AX_FULL, ot[md][e], 2);
    }
    __syncthreads();                                          // all warps are done with their staging memory
    float* smm = reinterpret_cast<float*>(smem);              // [warp][G][kST]
    if (!lo_part) {
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int head = hA + h;
            if (head < G) {
                float* dst = smm + ((size_t)warp * G + head) * kST;
                if (quad == 0) { dst[0] = m_run[h] * 0.6931471805599453f; dst[1] = l_run[h]; }     // back to natural-log units
#pragma unroll
                for (int md = 0; md < 8; md++) { dst[2 + md * 16 + quad] = ot[md][h]; dst[2 + md * 16 + quad + 8] = ot[md][2 + h]; }
            }
        }
    }
    __syncthreads();
    const int SP = dv.n_splits;                               // partial slots per head
    for (int idx = tid; idx < G * 128; idx += kThreads) {
        const int g = idx >> 7, d = idx & 127;
        float M = -CUDART_INF_F;
        for (int w = 0; w < kWarps; w++) M = fmaxf(M, smm[((size_t)w * G + g) * kST]);
        float L = 0.f, A = 0.f;
        for (int w = 0; w < kWarps; w++) {
            const float* sp = smm + ((size_t)w * G + g) * kST;
            const float c = merge_exp(sp[0], M);
            L = fmaf(c, sp[1], L); A = fmaf(c, sp[2 + d], A);
        }
        const size_t h = (size_t)b * dv.n_heads + (size_t)kh * G + g;
        if (S == 1) dv.out[h * 128 + d] = A / L;
        else {
            float* P = dv.partials + (h * SP + split) * kST;
            P[2 + d] = A;
            if (d == 0) { P[0] = M; P[1] = L; }
        }
    }
    if (S == 1) return;
    __threadfence();
    __syncthreads();
    if (tid == 0) s_last = atomicAdd(&dv.tickets[(size_t)b * gridDim.y + kh], 1u) == (unsigned)(S - 1);
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    for (int idx = tid; idx < G * 128; idx += kThreads) {
        const int g = idx >> 7, d = idx & 127;
        const size_t h = (size_t)b * dv.n_heads + (size_t)kh * G + g;
        const float* P = dv.partials + h * SP * kST;
        float M = -CUDART_INF_F;
        for (int i = 0; i < S; i++) M = fmaxf(M, P[(size_t)i * kST]);
        float L = 0.f, A = 0.f;
        for (int i = 0; i < S; i++) {
            const float c = merge_exp(P[(size_t)i * kST], M);
            L = fmaf(c, P[(size_t)i * kST + 1], L); A = fmaf(c, P[(size_t)i * kST + 2 + d], A);
        }
        dv.out[h * 128 + d] = A / L;
    }
    if (tid == 0) dv.tickets[(size_t)b * gridDim.y + kh] = 0u;       // ready for the next launch
}

constexpr size_t kSmemBytes = (size_t)kWarps * kWarpBytes;

// ── causal attention of a chunk of prompt tokens ──────────────────────────────────────
// The n tokens of a chunk (positions pos0 .. pos0 + n − 1, their K/V rows already in the cache) in ONE
// launch per layer instead of one decode-attention launch per token
// (crates/atlas-model/src/lib.rs:1611-1618 feeds the prompt token by token).  The 16 rows of the A
// operand are (token, head of the group) pairs — 16 tokens for one head per KV head, 4 tokens × 4
// heads, … — and each row carries its own causal and window mask: row of token i sees keys
// t ≤ pos0 + i with pos0 + i − t < window.  Otherwise the kernel is ax_attn_mma_kernel with both
// halves of the fragments in use.
struct ChunkDev {
    const float* q; size_t q_stride;            // token i, head h: q + i·q_stride + h·128 (normed and rotated)
    const uint16_t* kc; const uint16_t* vc;
    float* out; size_t out_stride;
    uint16_t* out_plane; int plane_rows;               // set: the result goes to a bf16 hi|lo token plane instead of out
    const int* pos0;                            // device: position of the chunk's first token
    int n_tok, n_heads, n_kv, g, window, n_splits;
    float scale;
    float* partials; unsigned* tickets;         // [n_tok·n_heads][n_splits][130]; [n_kv · row groups]
};

__device__ __forceinline__ void chunk_store(const ChunkDev& dv, int tok, int head, int d, float v) {
    if (dv.out_plane) {
        const size_t cols = (size_t)dv.n_heads * 128, k = (size_t)head * 128 + d;
        const uint16_t h = ax_f32_to_bf16_rne(v);
        dv.out_plane[(size_t)tok * cols + k] = h;
        dv.out_plane[(size_t)(dv.plane_rows + tok) * cols + k] = ax_f32_to_bf16_rne(v - ax_bf16_to_f32(h));
    } else dv.out[(size_t)tok * dv.out_stride + (size_t)head * 128 + d] = v;
}

__global__ void __launch_bounds__(kThreads) ax_attn_mma_chunk_kernel(const ChunkDev dv) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ int s_last;
    asm volatile("griddepcontrol.wait;" ::: "memory");        // queries and the chunk's K/V rows come from the kernels before
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int split = blockIdx.x, kh = blockIdx.y, rg = blockIdx.z;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = dv.g, TPG = 16 / G;                          // tokens per row group
    const int quad = lane >> 2, qi = lane & 3;

    const int pos0 = *dv.pos0;
    const int tok_lo = rg * TPG, tok_hi = min(dv.n_tok, tok_lo + TPG);       // tokens of this row group
    // rows `quad` and `quad + 8` of the fragments
    int r_tok[2], r_head[2], r_pos[2], r_lo[2];
    bool r_ok[2];
#pragma unroll
    for (int hf = 0; hf < 2; hf++) {
        const int r = quad + 8 * hf;
        r_tok[hf] = tok_lo + r / G; r_head[hf] = kh * G + r % G;
        r_ok[hf] = r < TPG * G && r_tok[hf] < dv.n_tok;
        r_pos[hf] = pos0 + r_tok[hf];
        r_lo[hf] = (dv.window > 0 && r_pos[hf] - dv.window + 1 > 0) ? r_pos[hf] - dv.window + 1 : 0;
    }
    const int p_first = pos0 + tok_lo, p_last = pos0 + tok_hi - 1;
    const int tb = (dv.window > 0 && p_first - dv.window + 1 > 0) ? p_first - dv.window + 1 : 0;
    const int te = p_last + 1;
    const int rows = te - tb;
    const int tiles_all = (rows + kTileRows - 1) / kTileRows;
    int S = dv.n_splits; if (S > tiles_all) S = tiles_all; if (S < 1) S = 1;
    if (split >= S) return;
    const int tile0 = (int)((long long)tiles_all * split / S), tile1 = (int)((long long)tiles_all * (split + 1) / S);
    const int t0 = tb + tile0 * kTileRows, t1 = min(te, tb + tile1 * kTileRows);
    const int n_tiles = tile1 - tile0;
    const int my_tiles = n_tiles > warp ? (n_tiles - warp + kWarps - 1) / kWarps : 0;

    uint32_t qh[8][4], ql[8][4];                               // a0..a3 per 16-dim step
    {
        const float sc = dv.scale * 1.4426950408889634f;
#pragma unroll
        for (int hf = 0; hf < 2; hf++) {
            const float* qp = dv.q + (size_t)(r_ok[hf] ? r_tok[hf] : 0) * dv.q_stride + (size_t)r_head[hf] * 128;
#pragma unroll
            for (int ks = 0; ks < 8; ks++) {
                float2 v0 = make_float2(0.f, 0.f), v1 = make_float2(0.f, 0.f);
                if (r_ok[hf]) {
                    v0 = *reinterpret_cast<const float2*>(qp + ks * 16 + qi * 2);
                    v1 = *reinterpret_cast<const float2*>(qp + ks * 16 + 8 + qi * 2);
                }
                split2(v0.x * sc, v0.y * sc, qh[ks][hf], ql[ks][hf]);              // a0 (row quad) / a1 (row quad + 8)
                split2(v1.x * sc, v1.y * sc, qh[ks][2 + hf], ql[ks][2 + hf]);      // a2 / a3
            }
        }
    }

    uint8_t* wbase = smem + (size_t)warp * kWarpBytes;
    const size_t row_elems = (size_t)dv.n_kv * 128;
    const uint16_t* kg = dv.kc + (size_t)kh * 128;
    const uint16_t* vg = dv.vc + (size_t)kh * 128;
    auto issue = [&](int j) {
        if (j < my_tiles) {
            const int tt = t0 + (warp + j * kWarps) * kTileRows;
            uint8_t* st = wbase + (size_t)(j % kStages) * kStageBytes;
            const int piece = lane & 15;
#pragma unroll
            for (int i = 0; i < 16; i++) {
                const int r = i * 2 + (lane >> 4);
                const int t = tt + r;
                const bool ok = t < t1;
                const size_t go = (size_t)(ok ? t : t0) * row_elems + piece * 8;
                cp_async16_zfill(smem_addr(st + r * kPitch + piece * 16), kg + go, ok);
                cp_async16_zfill(smem_addr(st + kTileBytes + r * kPitch + piece * 16), vg + go, ok);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
#pragma unroll
    for (int j = 0; j < kStages - 1; j++) issue(j);

    float o[16][4];
#pragma unroll
    for (int nt = 0; nt < 16; nt++) { o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.f; }
    float m_run[2] = { -CUDART_INF_F, -CUDART_INF_F }, l_run[2] = { 0.f, 0.f };

    for (int j = 0; j < my_tiles; j++) {
        asm volatile("cp.async.wait_group %0;" :: "n"(kStages - 2) : "memory");
        __syncwarp();
        issue(j + kStages - 1);
        const int tt = t0 + (warp + j * kWarps) * kTileRows;
        const uint8_t* st = wbase + (size_t)(j % kStages) * kStageBytes;
        const uint32_t ks_addr = smem_addr(st), vs_addr = smem_addr(st + kTileBytes);
        float s[4][4];
#pragma unroll
        for (int nt = 0; nt < 4; nt++) {
            s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
            for (int k2 = 0; k2 < 4; k2++) {
                uint32_t b0, b1, b2, b3;
                ldsm_x4(ks_addr + (nt * 8 + (lane & 7)) * kPitch + k2 * 64 + (lane >> 3) * 16, b0, b1, b2, b3);
                mma_bf16_full(s[nt], qh[2 * k2], b0, b1);
                mma_bf16_full(s[nt], ql[2 * k2], b0, b1);
                mma_bf16_full(s[nt], qh[2 * k2 + 1], b2, b3);
                mma_bf16_full(s[nt], ql[2 * k2 + 1], b2, b3);
            }
        }
        // per-row causal / window mask and online softmax, rows quad (c0, c1) and quad + 8 (c2, c3)
        float corr[2], m_use[2];
#pragma unroll
        for (int hf = 0; hf < 2; hf++) {
            float mx = -CUDART_INF_F;
#pragma unroll
            for (int nt = 0; nt < 4; nt++) {
#pragma unroll
                for (int e = 0; e < 2; e++) {
                    const int c = tt + nt * 8 + qi * 2 + e;
                    const bool ok = r_ok[hf] && c <= r_pos[hf] && c >= r_lo[hf] && c < t1;
                    if (!ok) s[nt][2 * hf + e] = -CUDART_INF_F;
                    mx = fmaxf(mx, s[nt][2 * hf + e]);
                }
            }
            mx = fmaxf(mx, __shfl_xor_sync(AX_FULL, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(AX_FULL, mx, 2));
            const float m_new = fmaxf(m_run[hf], mx);
            m_use[hf] = (m_new == -CUDART_INF_F) ? 0.f : m_new;
            corr[hf] = fast_exp2(m_run[hf] - m_use[hf]);
            m_run[hf] = m_new;
            l_run[hf] *= corr[hf];
        }
        uint32_t ph[2][4], pl[2][4];                          // [16-row step][a0..a3]
#pragma unroll
        for (int nt = 0; nt < 4; nt++) {
#pragma unroll
            for (int hf = 0; hf < 2; hf++) {
                const float p0 = fast_exp2(s[nt][2 * hf] - m_use[hf]), p1 = fast_exp2(s[nt][2 * hf + 1] - m_use[hf]);
                l_run[hf] += p0 + p1;
                split2(p0, p1, ph[nt >> 1][(nt & 1) * 2 + hf], pl[nt >> 1][(nt & 1) * 2 + hf]);
            }
        }
#pragma unroll
        for (int nt = 0; nt < 16; nt++) { o[nt][0] *= corr[0]; o[nt][1] *= corr[0]; o[nt][2] *= corr[1]; o[nt][3] *= corr[1]; }
#pragma unroll
        for (int kk = 0; kk < 2; kk++) {
#pragma unroll
            for (int n2 = 0; n2 < 8; n2++) {
                uint32_t b0, b1, b2, b3;
                ldsm_x4_trans(vs_addr + (kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * kPitch + n2 * 32 + (lane >> 4) * 16, b0, b1, b2, b3);
                mma_bf16_full(o[2 * n2], ph[kk], b0, b1);
                mma_bf16_full(o[2 * n2], pl[kk], b0, b1);
                mma_bf16_full(o[2 * n2 + 1], ph[kk], b2, b3);
                mma_bf16_full(o[2 * n2 + 1], pl[kk], b2, b3);
            }
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");

#pragma unroll
    for (int hf = 0; hf < 2; hf++) {
        l_run[hf] += __shfl_xor_sync(AX_FULL, l_run[hf], 1);
        l_run[hf] += __shfl_xor_sync(AX_FULL, l_run[hf], 2);
    }
    __syncthreads();
    float* smm = reinterpret_cast<float*>(smem);              // [warp][16 rows][kST]
#pragma unroll
    for (int hf = 0; hf < 2; hf++) {
        float* dst = smm + ((size_t)warp * 16 + quad + 8 * hf) * kST;
        if (qi == 0) { dst[0] = m_run[hf] * 0.6931471805599453f; dst[1] = l_run[hf]; }
#pragma unroll
        for (int nt = 0; nt < 16; nt++) { dst[2 + nt * 8 + qi * 2] = o[nt][2 * hf]; dst[2 + nt * 8 + qi * 2 + 1] = o[nt][2 * hf + 1]; }
    }
    __syncthreads();
    const int SP = dv.n_splits;
    const int n_rows = (tok_hi - tok_lo) * G;                  // real rows of this group
    for (int idx = tid; idx < n_rows * 128; idx += kThreads) {
        const int r = idx >> 7, d = idx & 127;
        float M = -CUDART_INF_F;
        for (int w = 0; w < kWarps; w++) M = fmaxf(M, smm[((size_t)w * 16 + r) * kST]);
        float L = 0.f, A = 0.f;
        for (int w = 0; w < kWarps; w++) {
            const float* sp = smm + ((size_t)w * 16 + r) * kST;
            const float c = merge_exp(sp[0], M);
            L = fmaf(c, sp[1], L); A = fmaf(c, sp[2 + d], A);
        }
        const int tok = tok_lo + r / G, head = kh * G + r % G;
        if (S == 1) chunk_store(dv, tok, head, d, A / L);
        else {
            float* P = dv.partials + (((size_t)tok * dv.n_heads + head) * SP + split) * kST;
            P[2 + d] = A;
            if (d == 0) { P[0] = M; P[1] = L; }
        }
    }
    if (S == 1) return;
    __threadfence();
    __syncthreads();
    unsigned* ticket = dv.tickets + (size_t)rg * gridDim.y + kh;
    if (tid == 0) s_last = atomicAdd(ticket, 1u) == (unsigned)(S - 1);
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    for (int idx = tid; idx < n_rows * 128; idx += kThreads) {
        const int r = idx >> 7, d = idx & 127;
        const int tok = tok_lo + r / G, head = kh * G + r % G;
        const float* P = dv.partials + ((size_t)tok * dv.n_heads + head) * SP * kST;
        float M = -CUDART_INF_F;
        for (int i = 0; i < S; i++) M = fmaxf(M, P[(size_t)i * kST]);
        float L = 0.f, A = 0.f;
        for (int i = 0; i < S; i++) {
            const float c = merge_exp(P[(size_t)i * kST], M);
            L = fmaf(c, P[(size_t)i * kST + 1], L); A = fmaf(c, P[(size_t)i * kST + 2 + d], A);
        }
        chunk_store(dv, tok, head, d, A / L);
    }
    if (tid == 0) *ticket = 0u;
}

}  // namespace

bool ax_attn_mma_supported(const AxAttnArgs& a) {
    if (a.hd != 128 || a.kv_dtype != ATLASX_BF16 || a.n_kv <= 0 || a.n_heads % a.n_kv) return false;
    const int g = a.n_heads / a.n_kv;
    if (g < 3 || g > 8) return false;
    return ((((uintptr_t)a.q | (uintptr_t)a.kc | (uintptr_t)a.vc | (uintptr_t)a.out) & 15) == 0) && (a.seq_stride % 8 == 0);
}

// Split count by a small cost model: the launch takes ⌈CTAs / SMs⌉ waves (one CTA per SM), and a CTA costs
// its share of a head group's tiles spread over its four warps plus a fixed part (query split, merges,
// partial results) worth about two tiles per warp.
namespace {
// shapes of the operator kernel: warps, stages, cached rows per warp tile, CTAs that fit one SM's shared memory
struct MmaShape { int warps, stages, rows, per_sm; };
constexpr MmaShape kShapes[] = { {6, 2, 32, 1}, {4, 3, 32, 1}, {8, 2, 16, 1}, {6, 2, 16, 2}, {4, 2, 16, 3} };
constexpr int kNumShapes = (int)(sizeof(kShapes) / sizeof(kShapes[0]));
// Many (sequence, KV head) groups: two smaller CTAs per SM, so that one CTA's pipeline fill and merge run
// under the other's steady state.  Few groups: one CTA per SM with eight warps, fewer and longer splits.
inline int shape_index(const atlasx_ctx* ctx, int groups) {
    const int i = ctx->tune.attn_cfg;
    if (i >= 0 && i < kNumShapes) return i;
    return groups >= 2 * ctx->sm_count ? 3 : 2;
}
}  // namespace

// Splits per (sequence, KV head): the cost of a launch is modelled as waves of CTAs × (tiles one warp
// walks + a fixed two tiles for the pipeline fill and the merge); the cheapest split count wins.
int ax_attn_mma_pick_splits(const atlasx_ctx* ctx, int n_kv, int batch, int max_rows) {
    const int groups = n_kv * batch;
    const MmaShape& sh = kShapes[shape_index(ctx, groups)];
    const int tiles = (max_rows + sh.rows - 1) / sh.rows;
    int cap = tiles / sh.warps; if (cap < 1) cap = 1; if (cap > 128) cap = 128;     // at least one tile per warp
    const long long slots = (long long)ctx->sm_count * sh.per_sm;
    const double fixed = 2.0 * 32 / sh.rows / sh.per_sm;        // co-resident CTAs hide each other's fill
    int best = 1; double best_cost = 1e300;
    for (int s = 1; s <= cap; s++) {
        const long long ctas = (long long)groups * s;
        const double waves = (double)((ctas + slots - 1) / slots);
        const double per_warp = (double)((tiles + s - 1) / s + sh.warps - 1) / sh.warps;
        const double cost = waves * (per_warp + fixed);
        if (cost < best_cost - 1e-9) { best_cost = cost; best = s; }
    }
    return best;
}

namespace {
template <bool PACK, int WARPS, int STAGES, int TR>
int launch_mma_cfg(atlasx_ctx* ctx, const MmaDev& dv, int batch, bool pdl) {
    constexpr size_t smem = (size_t)WARPS * STAGES * 2 * TR * kPitch;
    static_assert(smem >= (size_t)WARPS * 8 * kST * sizeof(float), "the warps' merge area reuses the staging memory");
    static bool attr_done[64] = {};                          // per device: the attribute belongs to the device's copy of the function
    const int dev = ctx->device & 63;
    if (!attr_done[dev]) {
        AX_CUDA(cudaFuncSetAttribute(ax_attn_mma_kernel<PACK, WARPS, STAGES, TR>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attr_done[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)dv.n_splits, (unsigned)dv.n_kv, (unsigned)batch);
    cfg.blockDim = dim3(WARPS * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    if (pdl) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr; cfg.numAttrs = 1;
    }
    AX_CUDA(cudaLaunchKernelEx(&cfg, ax_attn_mma_kernel<PACK, WARPS, STAGES, TR>, dv));
    return ATLASX_OK;
}
}  // namespace

int ax_attn_mma_launch(atlasx_ctx* ctx, const AxAttnArgs& a, bool pdl) {
    AX_ARG(ax_attn_mma_supported(a), "shape not covered by the tensor-core attention kernel");
    MmaDev dv;
    dv.q = a.q; dv.kc = (const uint16_t*)a.kc; dv.vc = (const uint16_t*)a.vc; dv.out = a.out; dv.seq_stride = a.seq_stride;
    dv.pos = a.pos; dv.pos_shared = a.pos_shared; dv.pos_scalar = a.pos_scalar;
    dv.n_heads = a.n_heads; dv.n_kv = a.n_kv; dv.g = a.n_heads / a.n_kv; dv.window = a.window; dv.scale = a.scale;
    dv.n_splits = a.n_splits < 1 ? 1 : a.n_splits;
    if (a.scratch_partials && a.scratch_tickets) { dv.partials = a.scratch_partials; dv.tickets = a.scratch_tickets; }
    else {
        int rc = atlasx_ctx_ensure_attn_scratch(ctx, (size_t)a.batch * a.n_heads * dv.n_splits * kST, (size_t)a.batch * a.n_heads);
        if (rc) return rc;
        dv.partials = ctx->attn_partials; dv.tickets = ctx->attn_tickets;
    }
    const bool pack = dv.g <= 4 && ctx->tune.attn_pack != 0;
    switch (shape_index(ctx, a.n_kv * a.batch)) {           // rows of kShapes
#define AX_CFG(n, W, S, T) case n: return pack ? launch_mma_cfg<true, W, S, T>(ctx, dv, a.batch, pdl) : launch_mma_cfg<false, W, S, T>(ctx, dv, a.batch, pdl)
        AX_CFG(1, 4, 3, 32);
        AX_CFG(2, 8, 2, 16);
        AX_CFG(3, 6, 2, 16);
        AX_CFG(4, 4, 2, 16);
        default: AX_CFG(0, 6, 2, 32);
#undef AX_CFG
    }
}

bool ax_attn_mma_chunk_supported(int hd, int n_heads, int n_kv, int kv_dtype) {
    if (hd != 128 || kv_dtype != ATLASX_BF16 || n_kv <= 0 || n_heads % n_kv) return false;
    const int g = n_heads / n_kv;
    return g == 1 || g == 2 || g == 4 || g == 8 || g == 16;
}
// Splits over the context for a chunk launch that sees `rows` cached rows: waves of CTAs (one CTA per SM) ×
// (tiles a warp walks + four tile times for building the query fragments, the merge of the warps and the partial
// states), the cheapest count up to kChunkMaxSplits.  Short contexts run unsplit: a split that leaves a warp two
// tiles spends most of its time on the fixed part.
int ax_attn_mma_chunk_splits(const atlasx_ctx* ctx, int n_heads, int n_kv, int n_tok, int rows) {
    const int g = n_heads / n_kv, tpg = 16 / g;
    const int groups = n_kv * ((n_tok + tpg - 1) / tpg);
    const int tiles = (rows + kTileRows - 1) / kTileRows;
    int best = 1; double best_cost = 1e300;
    for (int s = 1; s <= kChunkMaxSplits && s <= (tiles > 1 ? tiles : 1); s++) {
        const long long ctas = (long long)groups * s;
        const double waves = (double)((ctas + ctx->sm_count - 1) / ctx->sm_count);
        const double per_warp = (double)((tiles + s - 1) / s + kWarps - 1) / kWarps;
        const double cost = waves * (per_warp + 4.0);
        if (cost < best_cost - 1e-9) { best_cost = cost; best = s; }
    }
    return best;
}
int ax_attn_mma_chunk_max_splits() { return kChunkMaxSplits; }
size_t ax_attn_mma_chunk_partial_floats(int n_tok, int n_heads, int n_splits) { return (size_t)n_tok * n_heads * n_splits * kST; }

int ax_attn_mma_chunk_launch(atlasx_ctx* ctx, const AxAttnChunkArgs& a, bool pdl) {
    AX_ARG(ax_attn_mma_chunk_supported(128, a.n_heads, a.n_kv, ATLASX_BF16), "shape not covered by the chunk attention kernel");
    AX_ARG(a.q && a.kc && a.vc && a.out && a.pos0 && a.partials && a.tickets && a.n_tok >= 1 && a.n_tok <= 128, "bad argument");
    static bool attr_done[64] = {};
    if (!attr_done[ctx->device & 63]) {
        AX_CUDA(cudaFuncSetAttribute(ax_attn_mma_chunk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes));
        attr_done[ctx->device & 63] = true;
    }
    ChunkDev dv;
    dv.q = a.q; dv.q_stride = a.q_stride; dv.kc = (const uint16_t*)a.kc; dv.vc = (const uint16_t*)a.vc;
    dv.out = a.out; dv.out_stride = a.out_stride; dv.pos0 = a.pos0;
    dv.out_plane = a.out_plane; dv.plane_rows = a.plane_rows;
    AX_ARG(!a.out_plane || a.plane_rows >= a.n_tok, "token plane with fewer rows than tokens");
    dv.n_tok = a.n_tok; dv.n_heads = a.n_heads; dv.n_kv = a.n_kv; dv.g = a.n_heads / a.n_kv; dv.window = a.window;
    dv.n_splits = a.n_splits < 1 ? 1 : a.n_splits; dv.scale = a.scale;
    dv.partials = a.partials; dv.tickets = a.tickets;
    const int tpg = 16 / dv.g;
    dim3 grid((unsigned)dv.n_splits, (unsigned)a.n_kv, (unsigned)((a.n_tok + tpg - 1) / tpg));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = dim3(kThreads); cfg.dynamicSmemBytes = kSmemBytes; cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    if (pdl) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr; cfg.numAttrs = 1;
    }
    AX_CUDA(cudaLaunchKernelEx(&cfg, ax_attn_mma_chunk_kernel, dv));
    return ATLASX_OK;
}
