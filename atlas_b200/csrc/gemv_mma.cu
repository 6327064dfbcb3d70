// gemv_mma.cu — multi-column weight-streaming product Y[M×N] = W[M×K]·X[K×N], N = 2..16, on the
// tensor cores (warp-level mma m16n8k16, bf16 inputs, f32 accumulation).
//
// Replaces sgemm_bf16_kernel of the reference (kernels/matmul.cu:384-420, one thread per output
// element, every weight re-read N times through L1) for the "few columns" case of speculative
// verification and k-token prompt ingestion, and adds the int8 / int4 weight formats of
// crates/atlas-quant/src/lib.rs:32-168.  W is read exactly once; the work is HBM-bound
// (2·N flop per weight element), so the tensor cores are only the way to keep the instruction
// count per byte low — CUDA-core FMAs would cap N = 16 at about half the HBM rate.
//
//   * X (f32) is split into bf16 hi + lo parts (x = hi + lo to 2^-17 relative) and kept in shared
//     memory as [column][k]; the product runs twice, once per part, into the same accumulators.
//   * A 16-row tile of W is the A operand, fetched straight from global memory with 128-bit
//     loads into the fragment registers.  The k index inside a 32-element step is permuted
//     (thread t of a quad owns k = 8t..8t+7) — legal because A and B use the same permutation
//     and a dot product does not care about the order of its terms.  The matching B fragment is
//     one 16-byte shared-memory load.
//   * The eight warps of a CTA split K; their partial tiles meet in shared memory at the end.
//   * int8 / int4 weights are converted to bf16 exactly (|q| ≤ 128); the int8 row scale is applied
//     to the finished sum, the int4 block scale (one 32-element step lies inside one block) to the
//     step's partial product.
#include "gemv.cuh"
#include "gemv_device.cuh"

namespace {

constexpr int kMmaThreads = 256;
constexpr int kMmaWarps = 8;
constexpr int kMaxTiles = 4;          // 16-row tiles per row group
constexpr int kMmaUnroll = 4;         // k-steps whose loads are issued together
constexpr size_t kScratchHead = 16384; // the first bytes of the context scratch belong to the tcgen05 product (its item counter)

struct MmaArgs {
    const uint8_t* W; const uint8_t* scales;
    int M, K, N;
    int row_bytes, block, scales_f16;
    const float* X; float* Y;
    const uint16_t* xh; const uint16_t* xl;   // split input in global memory: [N+1][kpad] bf16 each
    int kpad;
    int kc;                           // k elements staged per chunk (multiple of 64 · 8 warps)
    int pitch;                        // bf16 elements between columns of the staged X
    int tiles;                        // 16-row tiles per row group (1, 2 or 4)
    int token_major;                  // X is [N][K] and Y is [N][M] (one contiguous vector per column) instead of [K][N] / [M][N]
};

__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {          // both exactly representable
    return (__float_as_uint(lo) >> 16) | (__float_as_uint(hi) & 0xFFFF0000u);
}
// four int8 of a word → two bf16 pairs (elements 0,1 and 2,3)
__device__ __forceinline__ void i8_to_bf16x4(uint32_t word, uint32_t& p01, uint32_t& p23) {
    const uint32_t u = word ^ 0x80808080u;
    const float f0 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7540)) - 8388736.0f;
    const float f1 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7541)) - 8388736.0f;
    const float f2 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7542)) - 8388736.0f;
    const float f3 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7543)) - 8388736.0f;
    p01 = pack_bf16(f0, f1); p23 = pack_bf16(f2, f3);
}
// eight int4 of a word (byte b: element 2b in the high nibble, 2b+1 in the low one) → four bf16 pairs
__device__ __forceinline__ void i4_to_bf16x8(uint32_t word, uint32_t (&p)[4]) {
    const uint32_t u = word ^ 0x88888888u;
#pragma unroll
    for (int b = 0; b < 4; b++) p[b] = pack_bf16(i4_val(u, 8 * b + 4), i4_val(u, 8 * b));
}

template <int FMT> struct MmaFmt;
template <> struct MmaFmt<ATLASX_BF16> { static constexpr int KS = 32; static constexpr int TK = 8;  using Frag = uint4; };
template <> struct MmaFmt<ATLASX_INT8> { static constexpr int KS = 64; static constexpr int TK = 16; using Frag = uint4; };
template <> struct MmaFmt<ATLASX_INT4> { static constexpr int KS = 32; static constexpr int TK = 8;  using Frag = uint32_t; };

template <int FMT>
__device__ __forceinline__ typename MmaFmt<FMT>::Frag load_frag(const uint8_t* p) {
    if constexpr (FMT == ATLASX_INT4) {
        uint32_t v;
        asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
        return v;
    } else {
        return ax_ldg_stream(p);
    }
}

// One k-step of one 16-row tile: rows g and g+8 of the tile in ra / rb, B from shared memory.
template <int FMT, int NT>
__device__ __forceinline__ void step_mma(float (&acc)[NT][4], const typename MmaFmt<FMT>::Frag& ra, const typename MmaFmt<FMT>::Frag& rb,
                                         const uint16_t* xh, const uint16_t* xl, int pitch, int g, int n_cols, float sa, float sb) {
    constexpr int TK = MmaFmt<FMT>::TK;
    uint32_t A[TK / 2], B[TK / 2];                       // bf16 pairs of row g and of row g+8
    if constexpr (FMT == ATLASX_BF16) {
        A[0] = ra.x; A[1] = ra.y; A[2] = ra.z; A[3] = ra.w;
        B[0] = rb.x; B[1] = rb.y; B[2] = rb.z; B[3] = rb.w;
    } else if constexpr (FMT == ATLASX_INT8) {
        i8_to_bf16x4(ra.x, A[0], A[1]); i8_to_bf16x4(ra.y, A[2], A[3]); i8_to_bf16x4(ra.z, A[4], A[5]); i8_to_bf16x4(ra.w, A[6], A[7]);
        i8_to_bf16x4(rb.x, B[0], B[1]); i8_to_bf16x4(rb.y, B[2], B[3]); i8_to_bf16x4(rb.z, B[4], B[5]); i8_to_bf16x4(rb.w, B[6], B[7]);
    } else {
        uint32_t pa[4], pb[4];
        i4_to_bf16x8(ra, pa); i4_to_bf16x8(rb, pb);
#pragma unroll
        for (int i = 0; i < 4; i++) { A[i] = pa[i]; B[i] = pb[i]; }
    }
#pragma unroll
    for (int nt = 0; nt < NT; nt++) {
        const int col = (nt * 8 + g) < n_cols ? nt * 8 + g : n_cols;      // columns past N read the zero column
        float c[4];
        if constexpr (FMT == ATLASX_INT4) { c[0] = c[1] = c[2] = c[3] = 0.f; }
        else { c[0] = acc[nt][0]; c[1] = acc[nt][1]; c[2] = acc[nt][2]; c[3] = acc[nt][3]; }
        {
#pragma unroll
            for (int j = 0; j < TK / 8; j++) {           // 16 bytes of X per part and per 8 k
                const uint4 bh = *reinterpret_cast<const uint4*>(xh + (size_t)col * pitch + j * 8);
                const uint4 bl = *reinterpret_cast<const uint4*>(xl + (size_t)col * pitch + j * 8);
                mma_bf16(c, A[4 * j + 0], B[4 * j + 0], A[4 * j + 1], B[4 * j + 1], bh.x, bh.y);
                mma_bf16(c, A[4 * j + 2], B[4 * j + 2], A[4 * j + 3], B[4 * j + 3], bh.z, bh.w);
                mma_bf16(c, A[4 * j + 0], B[4 * j + 0], A[4 * j + 1], B[4 * j + 1], bl.x, bl.y);
                mma_bf16(c, A[4 * j + 2], B[4 * j + 2], A[4 * j + 3], B[4 * j + 3], bl.z, bl.w);
            }
        }
        if constexpr (FMT == ATLASX_INT4) {
            acc[nt][0] = fmaf(c[0], sa, acc[nt][0]); acc[nt][1] = fmaf(c[1], sa, acc[nt][1]);
            acc[nt][2] = fmaf(c[2], sb, acc[nt][2]); acc[nt][3] = fmaf(c[3], sb, acc[nt][3]);
        } else {
            acc[nt][0] = c[0]; acc[nt][1] = c[1]; acc[nt][2] = c[2]; acc[nt][3] = c[3];
        }
    }
}

// X [K×N] f32 → two bf16 planes [N+1][kpad] in global memory (hi, lo), column-major, the extra
// column and the tail past K all zero: what the main kernel copies into shared memory verbatim.
__global__ void ax_gemv_mma_split_x(const float* X, int K, int N, int kpad, int token_major, uint16_t* xh, uint16_t* xl) {
    const int k = blockIdx.x * blockDim.x + threadIdx.x;
    if (k >= kpad) return;
    for (int n = 0; n <= N; n++) {
        uint16_t h = 0, l = 0;
        if (n < N && k < K) {
            const float x = token_major ? X[(size_t)n * K + k] : X[(size_t)k * N + n];
            h = ax_f32_to_bf16_rne(x);
            l = ax_f32_to_bf16_rne(x - ax_bf16_to_f32(h));
        }
        xh[(size_t)n * kpad + k] = h;
        xl[(size_t)n * kpad + k] = l;
    }
}

template <int FMT, int NT>
__global__ void __launch_bounds__(kMmaThreads, 2) ax_gemv_mma_kernel(const MmaArgs a) {
    constexpr int KS = MmaFmt<FMT>::KS;                  // k elements per step
    constexpr int TK = MmaFmt<FMT>::TK;                  // k elements per thread and step
    constexpr int NC = 8 * NT;                           // padded column count
    using Frag = typename MmaFmt<FMT>::Frag;
    extern __shared__ __align__(16) uint8_t msm[];
    const int cols = a.N + 1;                            // staged columns; the last one is all zero
    uint16_t* xh = reinterpret_cast<uint16_t*>(msm);                         // [cols][pitch] bf16 hi
    uint16_t* xl = xh + (size_t)cols * a.pitch;                              // [cols][pitch] bf16 lo
    float* red = reinterpret_cast<float*>(xl + (size_t)cols * a.pitch);      // [warps][16][NC]

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int rows_per_group = 16 * a.tiles;
    const int n_groups = (a.M + rows_per_group - 1) / rows_per_group;

    for (int kc0 = 0; kc0 < a.K; kc0 += a.kc) {
        const int klen = min(a.kc, a.K - kc0);
        // stage this chunk of the split input: 16-byte copies, column by column
        __syncthreads();                                                     // earlier readers of the staged chunk are done
        {
            const int vec_per_col = a.kc / 8;                                // kc is a multiple of 512
            for (int i = tid; i < 2 * cols * vec_per_col; i += kMmaThreads) {
                const int plane = i / (cols * vec_per_col), r = i - plane * cols * vec_per_col;
                const int c = r / vec_per_col, v = r - c * vec_per_col;
                const uint16_t* src = (plane ? a.xl : a.xh) + (size_t)c * a.kpad + kc0 + v * 8;
                uint16_t* dst = (plane ? xl : xh) + (size_t)c * a.pitch + v * 8;
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"(smem_u32(dst)), "l"(src) : "memory");
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        const int steps = klen / KS;
        const int s0 = steps * warp / kMmaWarps, s1 = steps * (warp + 1) / kMmaWarps;

        for (int grp = blockIdx.x; grp < n_groups; grp += gridDim.x) {
            const int r0 = grp * rows_per_group;
#pragma unroll
            for (int ti = 0; ti < kMaxTiles; ti++) {
                if (ti >= a.tiles || r0 + 16 * ti >= a.M) continue;
                float acc[NT][4];
#pragma unroll
                for (int nt = 0; nt < NT; nt++) { acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f; }
                const int rowa = min(r0 + 16 * ti + g, a.M - 1), rowb = min(r0 + 16 * ti + g + 8, a.M - 1);
                const size_t tbytes = (FMT == ATLASX_INT4) ? (size_t)t * 4 : (size_t)t * 16;
                const uint8_t* pa = a.W + (size_t)rowa * a.row_bytes + tbytes;
                const uint8_t* pb = a.W + (size_t)rowb * a.row_bytes + tbytes;
                auto kbytes = [&](int s) -> size_t {                         // byte offset of step s inside a row
                    const size_t k = (size_t)kc0 + (size_t)s * KS;
                    return FMT == ATLASX_BF16 ? k * 2 : FMT == ATLASX_INT8 ? k : k / 2;
                };
                auto scale_of = [&](int row, int s) -> float {
                    if (FMT != ATLASX_INT4) return 1.f;
                    const size_t e = (size_t)row * a.K + (size_t)kc0 + (size_t)s * KS;
                    return load_scale_i4(a.scales, (int)(e / a.block), a.scales_f16);
                };
                Frag fa[kMmaUnroll], fb[kMmaUnroll]; float sa[kMmaUnroll], sb[kMmaUnroll];
                auto fetch = [&](int s, Frag (&A)[kMmaUnroll], Frag (&B)[kMmaUnroll], float (&SA)[kMmaUnroll], float (&SB)[kMmaUnroll]) {
#pragma unroll
                    for (int u = 0; u < kMmaUnroll; u++) {
                        if (s + u < s1) {
                            A[u] = load_frag<FMT>(pa + kbytes(s + u)); B[u] = load_frag<FMT>(pb + kbytes(s + u));
                            SA[u] = scale_of(rowa, s + u); SB[u] = scale_of(rowb, s + u);
                        }
                    }
                };
                if (s0 < s1) fetch(s0, fa, fb, sa, sb);
                for (int s = s0; s < s1; s += kMmaUnroll) {
                    Frag na[kMmaUnroll], nb[kMmaUnroll]; float nsa[kMmaUnroll], nsb[kMmaUnroll];
                    if (s + kMmaUnroll < s1) fetch(s + kMmaUnroll, na, nb, nsa, nsb);
#pragma unroll
                    for (int u = 0; u < kMmaUnroll; u++) {
                        if (s + u < s1) {
                            const int kloc = (s + u) * KS + t * TK;          // this thread's k inside the staged chunk
                            step_mma<FMT, NT>(acc, fa[u], fb[u], xh + kloc, xl + kloc, a.pitch, g, a.N, sa[u], sb[u]);
                        }
                    }
#pragma unroll
                    for (int u = 0; u < kMmaUnroll; u++) { fa[u] = na[u]; fb[u] = nb[u]; sa[u] = nsa[u]; sb[u] = nsb[u]; }
                }
                // the eight k-slices of the tile meet in shared memory; one thread per output element adds
                // them and stores (first chunk) or accumulates (later chunks: same thread, same element)
                __syncthreads();
                float* mine = red + (size_t)warp * 16 * NC;
#pragma unroll
                for (int nt = 0; nt < NT; nt++) {
                    mine[g * NC + nt * 8 + 2 * t] = acc[nt][0];       mine[g * NC + nt * 8 + 2 * t + 1] = acc[nt][1];
                    mine[(g + 8) * NC + nt * 8 + 2 * t] = acc[nt][2]; mine[(g + 8) * NC + nt * 8 + 2 * t + 1] = acc[nt][3];
                }
                __syncthreads();
                for (int e = tid; e < 16 * NC; e += kMmaThreads) {
                    const int r = e / NC, n = e - r * NC;
                    const int row = r0 + 16 * ti + r;
                    if (row < a.M && n < a.N) {
                        float s = 0.f;
#pragma unroll
                        for (int w = 0; w < kMmaWarps; w++) s += red[(size_t)w * 16 * NC + e];
                        if (FMT == ATLASX_INT8) s *= reinterpret_cast<const float*>(a.scales)[row];
                        float* dst = a.token_major ? a.Y + (size_t)n * a.M + row : a.Y + (size_t)row * a.N + n;
                        *dst = kc0 == 0 ? s : *dst + s;
                    }
                }
            }
        }
    }
}

template <int FMT, int NT>
int launch_mma(atlasx_ctx* ctx, const MmaArgs& a, int grid, size_t smem) {
    static bool attr_set = false;
    if (!attr_set) {
        AX_CUDA(cudaFuncSetAttribute(ax_gemv_mma_kernel<FMT, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448 - 1024));
        attr_set = true;
    }
    ax_gemv_mma_kernel<FMT, NT><<<grid, kMmaThreads, smem, ctx->stream>>>(a);
    AX_CHECK_LAUNCH("ax_gemv_mma_kernel");
    return ATLASX_OK;
}

}  // namespace

bool ax_gemv_mma_supported(const AxWeight& w, int n, const float* x, const float* y) {
    if (n < 2 || n > 16 || !x || !y) return false;
    if (((uintptr_t)w.data & 15) != 0) return false;
    switch (w.dtype) {
        case ATLASX_BF16: return w.cols % 32 == 0;
        case ATLASX_INT8: return w.cols % 64 == 0 && w.scales;
        case ATLASX_INT4: return w.cols % 32 == 0 && w.block >= 32 && w.block % 32 == 0 && w.scales;
        default: return false;
    }
}

// Context scratch one such product needs: the two split planes [n + 1][K rounded up to whole chunks] bf16.
size_t ax_gemv_mma_scratch_bytes(int rows, int cols) {
    (void)rows;
    return kScratchHead + (size_t)2 * 17 * ((size_t)cols + 8192) * sizeof(uint16_t);
}

int ax_gemv_mma_launch(atlasx_ctx* ctx, const AxWeight& w, const float* x, int n, float* y, bool token_major) {
    AX_ARG(ax_gemv_mma_supported(w, n, x, y), "shape or format not covered by the tensor-core multi-column kernel");
    const int nt = n <= 8 ? 1 : 2;
    const int nc = 8 * nt;
    const int gran = 64 * kMmaWarps;                       // every warp gets whole steps of any format
    MmaArgs a = {};
    a.W = (const uint8_t*)w.data; a.scales = (const uint8_t*)w.scales;
    a.M = w.rows; a.K = w.cols; a.N = n;
    a.row_bytes = w.dtype == ATLASX_BF16 ? w.cols * 2 : w.dtype == ATLASX_INT8 ? w.cols : w.cols / 2;
    a.block = w.block > 0 ? w.block : 32; a.scales_f16 = w.scales_f16;
    a.X = x; a.Y = y; a.token_major = token_major ? 1 : 0;
    // chunk of K staged at a time: about 100 KB of shared memory, so that two CTAs share an SM
    const size_t red_bytes = (size_t)kMmaWarps * 16 * nc * sizeof(float);
    const long long k_pad = ((long long)w.cols + gran - 1) / gran * gran;
    long long kc = ((long long)(100 * 1024 - (long long)red_bytes) / (4 * (n + 1)) - 32) / gran * gran;
    if (kc < gran) kc = gran;
    if (kc > k_pad) kc = k_pad;
    a.kc = (int)kc; a.pitch = (int)kc + 32;
    a.kpad = (int)(((long long)w.cols + kc - 1) / kc * kc);                 // whole chunks: the copies never run past the planes
    const size_t smem = (size_t)4 * (n + 1) * a.pitch + red_bytes;
    // split planes in context scratch (grown on demand, never inside a stream capture)
    const size_t plane = (size_t)(n + 1) * a.kpad;
    int rc = atlasx_ctx_ensure_split_scratch(ctx, kScratchHead + 2 * plane * sizeof(uint16_t));
    if (rc) return rc;
    uint16_t* xh = reinterpret_cast<uint16_t*>(reinterpret_cast<uint8_t*>(ctx->split_scratch) + kScratchHead);
    a.xh = xh; a.xl = xh + plane;
    ax_gemv_mma_split_x<<<(a.kpad + 255) / 256, 256, 0, ctx->stream>>>(x, w.cols, n, a.kpad, a.token_major, xh, xh + plane);
    AX_CHECK_LAUNCH("ax_gemv_mma_split_x");
    // rows per CTA pass: as many 16-row tiles (1, 2 or 4) as still give every CTA slot a group
    const int slots = 2 * ctx->sm_count;
    int tiles = 4;
    while (tiles > 1 && (w.rows + 16 * tiles - 1) / (16 * tiles) < slots) tiles >>= 1;
    a.tiles = tiles;
    const int n_groups = (w.rows + 16 * tiles - 1) / (16 * tiles);
    const int grid = n_groups < slots ? n_groups : slots;
    switch (w.dtype) {
        case ATLASX_BF16: return nt == 1 ? launch_mma<ATLASX_BF16, 1>(ctx, a, grid, smem) : launch_mma<ATLASX_BF16, 2>(ctx, a, grid, smem);
        case ATLASX_INT8: return nt == 1 ? launch_mma<ATLASX_INT8, 1>(ctx, a, grid, smem) : launch_mma<ATLASX_INT8, 2>(ctx, a, grid, smem);
        default:          return nt == 1 ? launch_mma<ATLASX_INT4, 1>(ctx, a, grid, smem) : launch_mma<ATLASX_INT4, 2>(ctx, a, grid, smem);
    }
}
