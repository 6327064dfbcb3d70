// gemv_cols.cu — multi-column weight-streaming product Y[M×N] = W[M×K]·X[K×N], N = 2..16, on the
// tensor cores: the N activation columns ("tokens") are the 16-row A operand of mma.sync m16n8k16,
// eight weight rows are the B operand, so W — read exactly once, straight from global memory into
// the fragment registers — is never re-laid-out.
//
// Replaces sgemm_bf16_kernel of the reference (kernels/matmul.cu:384-420: one thread per output
// element, W re-read N times) for speculative verification and k-token prompt ingestion, and
// covers the int8 / int4 formats of crates/atlas-quant/src/lib.rs:32-168.
//
// Work is cut two ways: K into chunks of up to 1024 elements, rows into tiles of eight.  A CTA
// works on a contiguous range of (chunk, tile) items, so it stages only the chunk of X it needs —
// 16 tokens × 1024 k as bf16 hi + lo planes, 66 KB — instead of all of X; each of its eight warps
// owns whole items (a tile's 8 rows × the chunk's k), streams them with 128-bit loads eight steps
// ahead, and leaves 8 × N partial sums.  There is no barrier and no cross-warp reduction inside a
// chunk.  With more than one chunk the partial sums go to a scratch [chunks][M][16] and a small
// second kernel adds them in chunk order (deterministic), applies the int8 row scale and writes Y in
// the caller's layout.
//   * Accuracy: x = hi + lo (bf16 pair, 2⁻¹⁷ relative), W exact in bf16 (int8/int4 values convert
//     exactly), f32 accumulation: inside the 1e-3 parity bound by four orders of magnitude.
//   * The k index inside a 32-element step is permuted (thread t of a quad owns k = 8t..8t+7) in A
//     and B alike — a dot product does not care — so one 16-byte global load is the B fragment of
//     two MMAs and one 16-byte shared-memory load the matching A fragment.
#include "gemv.cuh"
#include "gemv_device.cuh"

namespace {

constexpr int kColsThreads = 256;
constexpr int kColsWarps = 8;
constexpr int kChunk = 1024;                  // k elements of X staged per chunk
// bf16 elements added to a staged token row so that the eight lanes of a quarter-warp (two tokens × four
// k pieces) hit distinct banks: the pieces of a token are 16 bytes apart for 8 k per thread (shift the next
// token by 64 bytes), 32 bytes apart for 16 k per thread (shift it by 16 bytes)
__host__ __device__ constexpr int cols_pad(int tk) { return tk == 16 ? 8 : 32; }
constexpr int kAhead = 8;                     // steps whose weight loads are in flight per warp

struct ColsArgs {
    const uint8_t* W; const uint8_t* scales;
    int M, K, N;
    int row_bytes, block, scales_f16;
    const uint16_t* xh; const uint16_t* xl;   // split input in global memory: [16][kpad] bf16 each, tokens ≥ N and k ≥ K zero
    int kpad;
    int n_chunks, n_tiles;                    // ⌈K / kChunk⌉, ⌈M / 8⌉
    int rows16;                               // 1: tokens 8..15 exist (N > 8)
    float* partial;                           // [n_chunks][M][16], or null when n_chunks == 1 …
    float* Y; int token_major;                // … then the kernel writes Y itself
};

__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack2_bf16(float lo, float hi) {           // both exactly representable in bf16
    return (__float_as_uint(lo) >> 16) | (__float_as_uint(hi) & 0xFFFF0000u);
}
// four int8 of a word → two bf16 pairs (elements 0,1 and 2,3), exact
__device__ __forceinline__ void i8x4_to_bf16(uint32_t word, uint32_t& p01, uint32_t& p23) {
    const uint32_t u = word ^ 0x80808080u;
    const float f0 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7540)) - 8388736.0f;
    const float f1 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7541)) - 8388736.0f;
    const float f2 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7542)) - 8388736.0f;
    const float f3 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7543)) - 8388736.0f;
    p01 = pack2_bf16(f0, f1); p23 = pack2_bf16(f2, f3);
}

// Per format: k elements of one step (KS), of one thread per step (TK), and the load that fetches them.
template <int FMT> struct ColsFmt;
template <> struct ColsFmt<ATLASX_BF16> { static constexpr int KS = 32; static constexpr int TK = 8;  using Frag = uint4; };
template <> struct ColsFmt<ATLASX_INT8> { static constexpr int KS = 64; static constexpr int TK = 16; using Frag = uint4; };
template <> struct ColsFmt<ATLASX_INT4> { static constexpr int KS = 32; static constexpr int TK = 8;  using Frag = uint32_t; };

template <int FMT>
__device__ __forceinline__ typename ColsFmt<FMT>::Frag cols_load(const uint8_t* p) {
    if constexpr (FMT == ATLASX_INT4) {
        uint32_t v;
        asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
        return v;
    } else {
        return ax_ldg_stream(p);
    }
}

// One step of one item: this thread's TK weights of row `quad` of the tile against the staged tokens.
// xrow points at this thread's k inside the staged chunk for token `quad` (hi plane); lo plane and
// token quad + 8 lie at fixed offsets.
template <int FMT, bool ROWS16>
__device__ __forceinline__ void cols_step(float (&acc)[4], const typename ColsFmt<FMT>::Frag& w, const uint16_t* xrow,
                                          int plane_off, int row8_off, float scale0, float scale1) {
    constexpr int TK = ColsFmt<FMT>::TK;
    uint32_t B[TK / 2];                                   // bf16 pairs of the weights, in k order
    if constexpr (FMT == ATLASX_BF16) { B[0] = w.x; B[1] = w.y; B[2] = w.z; B[3] = w.w; }
    else if constexpr (FMT == ATLASX_INT8) {
        i8x4_to_bf16(w.x, B[0], B[1]); i8x4_to_bf16(w.y, B[2], B[3]); i8x4_to_bf16(w.z, B[4], B[5]); i8x4_to_bf16(w.w, B[6], B[7]);
    } else {
        const uint32_t u = w ^ 0x88888888u;               // byte b: element 2b in the high nibble, 2b+1 in the low one
#pragma unroll
        for (int b = 0; b < 4; b++) B[b] = pack2_bf16(i4_val(u, 8 * b + 4), i4_val(u, 8 * b));
    }
    float c[4];
    if constexpr (FMT == ATLASX_INT4) { c[0] = c[1] = c[2] = c[3] = 0.f; }
    else { c[0] = acc[0]; c[1] = acc[1]; c[2] = acc[2]; c[3] = acc[3]; }
#pragma unroll
    for (int j = 0; j < TK / 8; j++) {                    // 8 k = 16 bytes of X per token and plane: two MMAs
        const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
        const uint4 h0 = *reinterpret_cast<const uint4*>(xrow + j * 8);
        const uint4 l0 = *reinterpret_cast<const uint4*>(xrow + plane_off + j * 8);
        const uint4 h8 = ROWS16 ? *reinterpret_cast<const uint4*>(xrow + row8_off + j * 8) : zero;
        const uint4 l8 = ROWS16 ? *reinterpret_cast<const uint4*>(xrow + row8_off + plane_off + j * 8) : zero;
        mma_16816(c, h0.x, h8.x, h0.y, h8.y, B[4 * j + 0], B[4 * j + 1]);
        mma_16816(c, h0.z, h8.z, h0.w, h8.w, B[4 * j + 2], B[4 * j + 3]);
        mma_16816(c, l0.x, l8.x, l0.y, l8.y, B[4 * j + 0], B[4 * j + 1]);
        mma_16816(c, l0.z, l8.z, l0.w, l8.w, B[4 * j + 2], B[4 * j + 3]);
    }
    if constexpr (FMT == ATLASX_INT4) {                   // the step lies inside one block of each row: the block scales of
        acc[0] = fmaf(c[0], scale0, acc[0]); acc[1] = fmaf(c[1], scale1, acc[1]);     // rows 2·qi and 2·qi + 1 (the rows of
        acc[2] = fmaf(c[2], scale0, acc[2]); acc[3] = fmaf(c[3], scale1, acc[3]);     // this thread's sums) on the partial products
    } else { acc[0] = c[0]; acc[1] = c[1]; acc[2] = c[2]; acc[3] = c[3]; }
}

// X [K×N] (or token-major [N][K]) f32 → bf16 planes [16][kpad] (hi, lo); tokens ≥ N and k ≥ K zero.
__global__ void ax_gemv_cols_split_x(const float* X, int K, int N, int kpad, int token_major, uint16_t* xh, uint16_t* xl) {
    const int k = blockIdx.x * blockDim.x + threadIdx.x;
    if (k >= kpad) return;
    for (int n = 0; n < 16; n++) {
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

template <int FMT, bool ROWS16>
__global__ void __launch_bounds__(kColsThreads, 2) ax_gemv_cols_kernel(const ColsArgs a) {
    constexpr int KS = ColsFmt<FMT>::KS, TK = ColsFmt<FMT>::TK;
    using Frag = typename ColsFmt<FMT>::Frag;
    constexpr int TOK = ROWS16 ? 16 : 8;
    constexpr int PITCH = kChunk + cols_pad(TK);          // bf16 elements per staged token row
    extern __shared__ __align__(16) uint8_t csm[];
    uint16_t* xs = reinterpret_cast<uint16_t*>(csm);      // [2 planes][TOK][PITCH]
    constexpr int PLANE = TOK * PITCH;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int quad = lane >> 2, qi = lane & 3;
    const long long items = (long long)a.n_chunks * a.n_tiles;            // chunk-major: item = chunk · n_tiles + tile
    const long long it0 = items * blockIdx.x / gridDim.x, it1 = items * (blockIdx.x + 1) / gridDim.x;

    for (long long seg0 = it0; seg0 < it1;) {
        const int chunk = (int)(seg0 / a.n_tiles);
        const long long seg1 = min(it1, (long long)(chunk + 1) * a.n_tiles);   // items of this CTA inside the chunk
        const int k0 = chunk * kChunk, klen = min(kChunk, a.K - k0);
        // ── stage the chunk of both planes: 16-byte copies, token by token ──
        __syncthreads();                                                    // readers of the previous chunk are done
        {
            const int vec = (klen + 7) / 8;
            for (int i = tid; i < 2 * TOK * vec; i += kColsThreads) {
                const int plane = i / (TOK * vec), r = i - plane * TOK * vec;
                const int tok = r / vec, v = r - tok * vec;
                const uint16_t* src = (plane ? a.xl : a.xh) + (size_t)tok * a.kpad + k0 + v * 8;
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"(smem_u32(xs + plane * PLANE + tok * PITCH + v * 8)), "l"(src) : "memory");
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        const int steps = klen / KS;                                        // K is a multiple of KS
        const size_t step_bytes = FMT == ATLASX_BF16 ? KS * 2 : FMT == ATLASX_INT8 ? KS : KS / 2;
        const size_t k0_bytes = FMT == ATLASX_BF16 ? (size_t)k0 * 2 : FMT == ATLASX_INT8 ? (size_t)k0 : (size_t)k0 / 2;
        const size_t t_bytes = FMT == ATLASX_INT4 ? (size_t)qi * 4 : (size_t)qi * 16;
        const uint16_t* xrow = xs + quad * PITCH + qi * TK;                 // token `quad`, this thread's k of step 0

        for (long long it = seg0 + warp; it < seg1; it += kColsWarps) {
            const int tile = (int)(it - (long long)chunk * a.n_tiles);
            const int row = min(tile * 8 + quad, a.M - 1);                  // rows past M repeat the last one and are not stored
            const uint8_t* wp = a.W + (size_t)row * a.row_bytes + k0_bytes + t_bytes;
            // int4: block scales of the two rows this thread's sums belong to (2·qi, 2·qi + 1 of the tile)
            const int sr0 = min(tile * 8 + 2 * qi, a.M - 1), sr1 = min(tile * 8 + 2 * qi + 1, a.M - 1);
            auto scale_of = [&](int r, int s) -> float {
                if (FMT != ATLASX_INT4) return 1.f;
                const size_t e = (size_t)r * a.K + (size_t)k0 + (size_t)s * KS;
                return load_scale_i4(a.scales, (int)(e / a.block), a.scales_f16);
            };
            float acc[4] = { 0.f, 0.f, 0.f, 0.f };
            Frag w[kAhead]; float sc0[kAhead], sc1[kAhead];
#pragma unroll
            for (int u = 0; u < kAhead; u++)
                if (u < steps) { w[u] = cols_load<FMT>(wp + (size_t)u * step_bytes); sc0[u] = scale_of(sr0, u); sc1[u] = scale_of(sr1, u); }
            for (int s = 0; s < steps; s += kAhead) {
#pragma unroll
                for (int u = 0; u < kAhead; u++) {
                    if (s + u < steps) {
                        const Frag cur = w[u]; const float c0 = sc0[u], c1 = sc1[u];
                        if (s + u + kAhead < steps) {
                            w[u] = cols_load<FMT>(wp + (size_t)(s + u + kAhead) * step_bytes);
                            sc0[u] = scale_of(sr0, s + u + kAhead); sc1[u] = scale_of(sr1, s + u + kAhead);
                        }
                        cols_step<FMT, ROWS16>(acc, cur, xrow + (s + u) * KS, PLANE, 8 * PITCH, c0, c1);
                    }
                }
            }
            // c0, c1: token `quad`, rows 2·qi and 2·qi + 1 of the tile; c2, c3: token quad + 8
            const int r0 = tile * 8 + 2 * qi;
            if (a.partial) {
                float* P = a.partial + ((size_t)chunk * a.M) * 16;
                if (r0 < a.M) { P[(size_t)r0 * 16 + quad] = acc[0]; if (ROWS16) P[(size_t)r0 * 16 + quad + 8] = acc[2]; }
                if (r0 + 1 < a.M) { P[(size_t)(r0 + 1) * 16 + quad] = acc[1]; if (ROWS16) P[(size_t)(r0 + 1) * 16 + quad + 8] = acc[3]; }
            } else {
                const float* rs = FMT == ATLASX_INT8 ? reinterpret_cast<const float*>(a.scales) : nullptr;
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const int r = r0 + (e & 1), tok = quad + (e >> 1) * 8;
                    if (r < a.M && tok < a.N) {
                        const float v = rs ? acc[e] * rs[r] : acc[e];
                        if (a.token_major) a.Y[(size_t)tok * a.M + r] = v; else a.Y[(size_t)r * a.N + tok] = v;
                    }
                }
            }
        }
        seg0 = seg1;
    }
}

// Sum of the per-chunk partials in chunk order; int8 row scale; Y in the caller's layout.
__global__ void ax_gemv_cols_reduce(const float* partial, int n_chunks, int M, int N, const float* row_scale, int token_major, float* Y) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;                    // (row, token slot)
    if (i >= M * 16) return;
    const int r = i >> 4, tok = i & 15;
    if (tok >= N) return;
    float s = 0.f;
    for (int c = 0; c < n_chunks; c++) s += partial[((size_t)c * M) * 16 + i];
    if (row_scale) s *= row_scale[r];
    if (token_major) Y[(size_t)tok * M + r] = s; else Y[(size_t)r * N + tok] = s;
}

template <int FMT, bool ROWS16>
int launch_cols(atlasx_ctx* ctx, const ColsArgs& a, int grid) {
    const size_t smem = (size_t)2 * (ROWS16 ? 16 : 8) * (kChunk + cols_pad(ColsFmt<FMT>::TK)) * sizeof(uint16_t);
    static bool attr_set = false;
    if (!attr_set) {
        AX_CUDA(cudaFuncSetAttribute(ax_gemv_cols_kernel<FMT, ROWS16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attr_set = true;
    }
    ax_gemv_cols_kernel<FMT, ROWS16><<<grid, kColsThreads, smem, ctx->stream>>>(a);
    AX_CHECK_LAUNCH("ax_gemv_cols_kernel");
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

// Scratch of one call: the two split planes [16][kpad] bf16 and, with several chunks, the partials.
size_t ax_gemv_mma_scratch_bytes(int rows, int cols) {
    const size_t kpad = ((size_t)cols + kChunk - 1) / kChunk * kChunk;
    const size_t n_chunks = kpad / kChunk;
    return 2 * 16 * kpad * sizeof(uint16_t) + (n_chunks > 1 ? n_chunks * (size_t)rows * 16 * sizeof(float) : 0) + 256;
}

int ax_gemv_mma_launch(atlasx_ctx* ctx, const AxWeight& w, const float* x, int n, float* y, bool token_major) {
    AX_ARG(ax_gemv_mma_supported(w, n, x, y), "shape or format not covered by the tensor-core multi-column kernel");
    ColsArgs a = {};
    a.W = (const uint8_t*)w.data; a.scales = (const uint8_t*)w.scales;
    a.M = w.rows; a.K = w.cols; a.N = n;
    a.row_bytes = w.dtype == ATLASX_BF16 ? w.cols * 2 : w.dtype == ATLASX_INT8 ? w.cols : w.cols / 2;
    a.block = w.block > 0 ? w.block : 32; a.scales_f16 = w.scales_f16;
    a.kpad = (w.cols + kChunk - 1) / kChunk * kChunk;
    a.n_chunks = a.kpad / kChunk; a.n_tiles = (w.rows + 7) / 8;
    a.rows16 = n > 8;
    a.Y = y; a.token_major = token_major ? 1 : 0;
    int rc = atlasx_ctx_ensure_split_scratch(ctx, ax_gemv_mma_scratch_bytes(w.rows, w.cols));
    if (rc) return rc;
    uint16_t* xh = reinterpret_cast<uint16_t*>(ctx->split_scratch);
    const size_t plane = (size_t)16 * a.kpad;
    a.xh = xh; a.xl = xh + plane;
    a.partial = a.n_chunks > 1 ? reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(xh + 2 * plane) + 128) : nullptr;
    if (a.partial) a.partial = reinterpret_cast<float*>(((uintptr_t)a.partial + 127) & ~(uintptr_t)127);
    ax_gemv_cols_split_x<<<(a.kpad + 255) / 256, 256, 0, ctx->stream>>>(x, w.cols, n, a.kpad, a.token_major, xh, xh + plane);
    AX_CHECK_LAUNCH("ax_gemv_cols_split_x");
    const long long items = (long long)a.n_chunks * a.n_tiles;
    long long grid = 2LL * ctx->sm_count;                                   // two CTAs per SM
    if (grid * kColsWarps > items) grid = (items + kColsWarps - 1) / kColsWarps;
    if (grid < 1) grid = 1;
    const bool r16 = a.rows16 != 0;
    switch (w.dtype) {
        case ATLASX_BF16: rc = r16 ? launch_cols<ATLASX_BF16, true>(ctx, a, (int)grid) : launch_cols<ATLASX_BF16, false>(ctx, a, (int)grid); break;
        case ATLASX_INT8: rc = r16 ? launch_cols<ATLASX_INT8, true>(ctx, a, (int)grid) : launch_cols<ATLASX_INT8, false>(ctx, a, (int)grid); break;
        default:          rc = r16 ? launch_cols<ATLASX_INT4, true>(ctx, a, (int)grid) : launch_cols<ATLASX_INT4, false>(ctx, a, (int)grid); break;
    }
    if (rc || !a.partial) return rc;
    ax_gemv_cols_reduce<<<(w.rows * 16 + 255) / 256, 256, 0, ctx->stream>>>(
        a.partial, a.n_chunks, w.rows, n, w.dtype == ATLASX_INT8 ? reinterpret_cast<const float*>(w.scales) : nullptr, a.token_major, y);
    AX_CHECK_LAUNCH("ax_gemv_cols_reduce");
    return ATLASX_OK;
}
