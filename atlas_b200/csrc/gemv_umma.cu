// gemv_umma.cu — many-column weight-streaming product Y[n][M] = X[n][K]·W[M][K]ᵀ, n = 2..128 tokens (64 with int8 weights), on the
// fifth-generation tensor cores: tcgen05.mma with the accumulator in tensor memory, operands brought into
// shared memory by tiled bulk copies (cp.async.bulk.tensor) and handed over through mbarriers.
//
// It serves the same callers as the warp-level kernel of gemv_mma.cu — the token batches of prompt ingestion
// and speculative verification, which the reference runs as one sgemm_bf16_kernel thread per output element
// (kernels/matmul.cu:384-420) or token by token (crates/atlas-model/src/lib.rs:1611-1618) — and exists because
// the warp-level kernel falls to half the HBM rate at 16 columns and cannot take more.
//
//   * Work item = (128-row tile of W, range of K blocks of 128 bytes per row), two CTAs per SM.  K is split so that
//     short matrices still give every SM work; the partial tiles of a row tile meet in global scratch and a small
//     kernel behind the product (ax_umma_merge_kernel, the whole GPU) adds them in split order, so the result does
//     not depend on timing.  (Merged by the CTA of a tile that arrived last it was a tail of 16 µs at 64 tokens.)  Items
//     are handed out dynamically — SMs do not stream at equal rates: one item per CTA by the hardware's CTA
//     scheduler, or, for matrices with many long items, resident CTAs that take item numbers from a global counter and
//     keep two accumulators in tensor memory, so that the epilogue of an item runs under the MMAs of the next.
//   * A operand: the W tile, 128 rows × 64 bf16 per stage (16 KB), 128-byte swizzle.  Rows beyond M are filled
//     with zeros by the copy engine.
//   * B operand: the tokens.  The f32 activations are split into bf16 hi + lo parts (x = hi + lo to 2⁻¹⁷
//     relative) stored as 2·n8 rows of one plane (n8 = n rounded up to 8): rows 0..n8−1 hi, n8..2·n8−1 lo.
//     One MMA of width N = 2·n8 yields both partial products; the epilogue adds column j and column n8 + j.
//     Products with bf16 W are exact in the f32 accumulator, so the result matches an f32 dot product to the
//     accumulation order.
//   * Roles: warp 0 issues the copies, warp 1 owns tensor memory and issues the MMAs (one lane), warps 2..5
//     read the accumulator (tcgen05.ld, one lane quarter each) and write Y or the partial tile.
//   * Every wait on an mbarrier is bounded (two seconds of %globaltimer): on expiry the CTA raises the
//     context's device error word, all roles leave their loops, copies in flight are waited for (bounded again)
//     and tensor memory is released before the CTA returns.
//   * int8 weights (crates/atlas-quant/src/lib.rs:41-75: one f32 scale per row) run as kind::i8 with the raw
//     weight bytes as A (128 int8 per K block) and the tokens as three int8 digit planes in base 254 with one
//     scale per token (x ≈ s·(q1 + q2/254 + q3/254²), |error| ≤ 1.2e-7·max|x| of the token): the s32 sums in
//     tensor memory are exact, the epilogue combines the planes and applies token and row scale.
//   * int4 weights (more than 16 tokens) are first expanded into two bf16 planes side by side, [M][hi | lo] of q · scale,
//     and multiplied as a bf16 matrix of 2K columns whose K block kb meets block kb mod (K / 64) of the token plane.
//   * The tensor maps cover this GPU's own memory only and no copy is multicast.
#include <cuda.h>

#include "gemv.cuh"

namespace {

constexpr int kTileM = 128;
constexpr int kBlockBytes = 128;                  // bytes of a row per K block: one swizzle row (64 bf16 or 128 int8)
constexpr int kABytes = kTileM * kBlockBytes;     // 16 KB
constexpr float kDigitBase = 254.0f;
constexpr int kThreads = 192;
constexpr int kMaxStages = 8;
constexpr int kMaxTokens = 128;                  // bf16 weights: hi and lo plane fill the 256 columns one MMA can have
constexpr int kMaxTokensI8 = 64;                 // int8 weights: three digit planes
constexpr int kMaxSplits = 8;
constexpr int kItemRing = 8;
constexpr size_t kHeadBytes = 16384;            // area at the start of the context scratch that holds the item counter
constexpr unsigned long long kWaitNs = 2000000000ull;

struct UmmaArgs {
    float* Y;
    int M, n, nc;                 // rows of W, tokens, columns per plane (tokens rounded up to 8; to 16 for int8)
    int i8, planes;               // int8 weights with three digit planes, or bf16 with hi and lo planes
    int kblk;                     // elements per K block (64 bf16, 128 int8)
    const float* wscale;          // int8: scale per row of W
    const float* xscale;          // int8: scale per token
    int KB, KS, T;                // K blocks, K splits, row tiles
    int KBx;                      // K blocks of the token plane: block kb of W meets block kb mod KBx of the tokens (KBx = KB unless W is
                                  // two bf16 planes side by side — int4 weights expanded to hi | lo)
    int stages, b_bytes;          // pipeline depth, bytes of one B stage (planes·nc rows × 128)
    int acc_cols, tmem_cols;      // columns of one accumulator (power of two ≥ 32 holding planes·nc) and of the allocation
    int persist;                  // 1: CTAs stay and take items from the counter; 0: one item per CTA
    unsigned* counter;            // [0] next item (resident form), [1] CTAs that are through; both zero between launches
    int token_major;              // Y[j·M + row] (one contiguous vector per token) or Y[row·n + j]
    float* parts;                 // [T·KS][n][128] partial tiles (KS > 1), added up by ax_umma_merge_kernel
    int* err;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ unsigned long long global_ns() { unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait.  false: gave up (this thread's deadline passed, or another role raised the abort flag).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* err, int code) {
    unsigned spins = 0;
    unsigned long long t0 = 0;
    while (!mbar_try(bar, parity)) {
        if (*abort_flag) return false;
        if ((++spins & 255u) == 0) {
            const unsigned long long t = global_ns();
            if (t0 == 0) t0 = t;
            else if (t - t0 > kWaitNs) { *abort_flag = 1; atomicExch(err, code); return false; }
        }
    }
    return true;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 :: "r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}
// Shared-memory matrix descriptor of a K-major tile with 128-byte swizzle: rows of 128 bytes, groups of eight
// rows 1024 bytes apart (stride offset), descriptor version 1, layout code 2.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 :: "r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_i8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
                 :: "r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {       // the barrier gets one arrival when every MMA issued so far is done
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, float (&v)[8]) {
    uint32_t r[8];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]) : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 8; i++) v[i] = __uint_as_float(r[i]);
}

// f32 tokens → one bf16 plane [2·n8][K]: rows 0..n8−1 hi parts, rows n8..2·n8−1 lo parts, rows of absent tokens zero.
// Also resets the item counter of the product that follows.
__global__ void ax_umma_split_kernel(const float* __restrict__ X, int K, int n, int n8, int token_major,
                                     uint16_t* __restrict__ plane, unsigned* counter) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx < 2) counter[idx] = 0u;
    const int k8 = K / 8;
    if (idx >= (size_t)2 * n8 * k8) return;
    const int row = (int)(idx / k8), kg = (int)(idx % k8);
    const int j = row < n8 ? row : row - n8;
    const bool lo = row >= n8;
    uint32_t out[4] = { 0u, 0u, 0u, 0u };
    if (j < n) {
        float x[8];
        if (token_major) {
            const float4 a = *reinterpret_cast<const float4*>(X + (size_t)j * K + kg * 8);
            const float4 b = *reinterpret_cast<const float4*>(X + (size_t)j * K + kg * 8 + 4);
            x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w; x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
        } else {
#pragma unroll
            for (int i = 0; i < 8; i++) x[i] = X[(size_t)(kg * 8 + i) * n + j];
        }
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const uint16_t h = ax_f32_to_bf16_rne(x[i]);
            const uint16_t v = lo ? ax_f32_to_bf16_rne(x[i] - ax_bf16_to_f32(h)) : h;
            out[i >> 1] |= (uint32_t)v << ((i & 1) * 16);
        }
    }
    *reinterpret_cast<uint4*>(plane + (size_t)row * K + kg * 8) = make_uint4(out[0], out[1], out[2], out[3]);
}

// f32 tokens → three int8 digit planes [3·n16][K] in base 254 with one scale per token: rows p·n16 + j hold
// digit p of token j, rows of absent tokens are zero.  One CTA per row index j < n16.  A NaN or inf in a token
// makes its scale NaN, and with it every output of that token.  Also resets the item counter.
__global__ void __launch_bounds__(256) ax_umma_digits_kernel(const float* __restrict__ X, int K, int n, int n16, int token_major,
                                                             int8_t* __restrict__ plane, float* __restrict__ xscale,
                                                             unsigned* counter) {
    __shared__ float red[8];
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int j = blockIdx.x, tid = threadIdx.x;
    if (j == 0 && tid < 2) counter[tid] = 0u;
    const size_t plane_stride = (size_t)n16 * K;
    int8_t* r0 = plane + (size_t)j * K;
    if (j >= n) {
        for (int k = tid * 16; k < K; k += 256 * 16)
            for (int pl = 0; pl < 3; pl++) *reinterpret_cast<uint4*>(r0 + pl * plane_stride + k) = make_uint4(0u, 0u, 0u, 0u);
        return;
    }
    auto xat = [&](int k) { return token_major ? X[(size_t)j * K + k] : X[(size_t)k * n + j]; };
    float mx = 0.f, bad = 0.f;
    for (int k = tid; k < K; k += 256) { const float v = xat(k); mx = fmaxf(mx, fabsf(v)); bad += v * 0.f; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) { mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o)); bad += __shfl_xor_sync(0xFFFFFFFFu, bad, o); }
    if ((tid & 31) == 0) red[tid >> 5] = mx;
    __syncthreads();
    mx = red[0];
#pragma unroll
    for (int w = 1; w < 8; w++) mx = fmaxf(mx, red[w]);
    __syncthreads();
    if ((tid & 31) == 0) red[tid >> 5] = bad;
    __syncthreads();
    bad = 0.f;
#pragma unroll
    for (int w = 0; w < 8; w++) bad += red[w];
    if (!(mx < 3.0e38f)) mx = 3.0e38f;
    const float inv = mx > 0.f ? 127.0f / mx : 0.f;
    if (tid == 0) xscale[j] = mx / 127.0f + bad;                 // bad is 0, or NaN when the token holds a NaN or an inf
    for (int k4 = tid; k4 * 4 < K; k4 += 256) {
        uint32_t w1 = 0, w2 = 0, w3 = 0;
#pragma unroll
        for (int e = 0; e < 4; e++) {
            // round to nearest by adding 1.5·2^23: the integer then sits in the low mantissa bits
            constexpr float Mg = 12582912.0f;
            float t = xat(k4 * 4 + e) * inv;
            t = fminf(fmaxf(t, -127.f), 127.f);
            const float a1 = t + Mg, q1 = a1 - Mg;
            const float rr = (t - q1) * kDigitBase;
            const float a2 = rr + Mg, q2 = a2 - Mg;
            const float a3 = (rr - q2) * kDigitBase + Mg;
            w1 |= (uint32_t)((__float_as_int(a1) - 0x4B400000) & 255) << (8 * e);
            w2 |= (uint32_t)((__float_as_int(a2) - 0x4B400000) & 255) << (8 * e);
            w3 |= (uint32_t)((__float_as_int(a3) - 0x4B400000) & 255) << (8 * e);
        }
        *reinterpret_cast<uint32_t*>(r0 + k4 * 4) = w1;
        *reinterpret_cast<uint32_t*>(r0 + plane_stride + k4 * 4) = w2;
        *reinterpret_cast<uint32_t*>(r0 + 2 * plane_stride + k4 * 4) = w3;
    }
}

__global__ void __launch_bounds__(kThreads) ax_gemv_umma_kernel(const __grid_constant__ CUtensorMap map_w,
                                                                const __grid_constant__ CUtensorMap map_x, const UmmaArgs a) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[kMaxStages], empty_bar[kMaxStages], acc_full[2], acc_empty[2], item_bar[kItemRing];
    __shared__ uint32_t s_tmem;
    __shared__ int s_abort, s_issued, s_go, s_item[kItemRing];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int ST = a.stages;
    const int NP = a.planes * a.nc;
    const int n_items = a.T * a.KS;
    const uint32_t stage_bytes = (uint32_t)kABytes + (uint32_t)a.b_bytes;
    const uint32_t smem0 = (smem_u32(smem_raw) + 1023u) & ~1023u;           // swizzled tiles want 1024-byte alignment
    volatile int* abort_flag = &s_abort;
    auto item_range = [&](int item, int& tile, int& kb0, int& nkb) {
        tile = item / a.KS;
        const int ks = item - tile * a.KS;
        kb0 = (int)((long long)a.KB * ks / a.KS);
        nkb = (int)((long long)a.KB * (ks + 1) / a.KS) - kb0;
    };

    if (tid == 0) {
        for (int s = 0; s < ST; s++) { mbar_init(smem_u32(&full_bar[s]), 1); mbar_init(smem_u32(&empty_bar[s]), 1); }
        for (int u = 0; u < 2; u++) { mbar_init(smem_u32(&acc_full[u]), 1); mbar_init(smem_u32(&acc_empty[u]), 1); }
        for (int u = 0; u < kItemRing; u++) mbar_init(smem_u32(&item_bar[u]), 1);
        s_abort = 0; s_issued = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {                                                         // tensor memory: allocated and released by this warp
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(smem_u32(&s_tmem)), "r"((uint32_t)a.tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = s_tmem;

    // Items reach the three roles through a small ring: the copy warp takes the next item (its own block index, or —
    // persistent form — the next number of a global counter, so faster SMs take more items), writes it into the ring
    // and arrives on the slot's mbarrier; the MMA warp and the epilogue read it from there.  −1 ends the walk.
    if (warp == 0) {
        if (lane == 0) {
            int f = 0;                                                       // stages filled so far, over all items
            bool ok = true;
            // One item per CTA: the item is known from the block index and W does not depend on the launch before, so the
            // W tiles of the first stages are requested before the dependency wait; their token tiles follow after it
            // (same barrier: a stage is full when both have landed).
            int pre = 0, next = (int)blockIdx.x;
            if (!a.persist) {
                int tile, kb0, nkb; item_range(next, tile, kb0, nkb);
                pre = nkb < ST ? nkb : ST;
                for (int i = 0; i < pre; i++) {
                    const uint32_t bar = smem_u32(&full_bar[i]);
                    mbar_expect_tx(bar, stage_bytes);
                    tma_load_2d(smem0 + (uint32_t)i * stage_bytes, &map_w, (kb0 + i) * a.kblk, tile * kTileM, bar);
                }
                s_issued = pre;
            }
            asm volatile("griddepcontrol.wait;" ::: "memory");              // the token plane and the counter are written by the launch before
            if (a.persist) next = (int)atomicAdd(a.counter, 1u);
            for (int li = 0; ok; li++) {
                const int item = next < n_items ? next : -1;
                s_item[li % kItemRing] = item;
                asm volatile("mbarrier.arrive.release.cta.shared::cta.b64 _, [%0];" :: "r"(smem_u32(&item_bar[li % kItemRing])) : "memory");
                if (item < 0) break;
                // the number of the item after this one is asked for before this item's copies are issued: the atomic's
                // round trip runs under them instead of leaving the stages idle between two items
                next = a.persist ? (int)atomicAdd(a.counter, 1u) : n_items;
                int tile, kb0, nkb; item_range(item, tile, kb0, nkb);
                for (int i = 0; i < nkb; i++, f++) {
                    const int s = f % ST;
                    const uint32_t bar = smem_u32(&full_bar[s]);
                    const uint32_t dst = smem0 + (uint32_t)s * stage_bytes;
                    if (f >= pre) {                                          // the first stages already expect their bytes and have their W tile on the way
                        if (f >= ST && !mbar_wait(smem_u32(&empty_bar[s]), (uint32_t)((f / ST) - 1) & 1u, abort_flag, a.err, 701)) { ok = false; break; }
                        mbar_expect_tx(bar, stage_bytes);
                        tma_load_2d(dst, &map_w, (kb0 + i) * a.kblk, tile * kTileM, bar);
                    }
                    tma_load_2d(dst + kABytes, &map_x, ((kb0 + i) >= a.KBx ? (kb0 + i) - a.KBx : (kb0 + i)) * a.kblk, 0, bar);
                    s_issued = f + 1;
                }
            }
            // Resident form: a CTA that has taken its last number (one beyond the items) says so; the CTA that says it
            // last knows that nobody will ask again and sets both counters back to zero for the next launch.
            if (a.persist && ok && atomicAdd(a.counter + 1, 1u) == gridDim.x - 1) { a.counter[1] = 0u; a.counter[0] = 0u; }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // instruction descriptor: accumulator f32 (1) or s32 (2), A and B bf16 (1) or signed int8 (1), both K-major,
            // N = planes·nc, M = 128
            const uint32_t idesc = ((a.i8 ? 2u : 1u) << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(NP >> 3) << 17) | ((uint32_t)(kTileM >> 4) << 24);
            const bool i8 = a.i8 != 0;
            bool ok = true;
            int f = 0;
            for (int li = 0; ok; li++) {
                if (!mbar_wait(smem_u32(&item_bar[li % kItemRing]), (uint32_t)(li / kItemRing) & 1u, abort_flag, a.err, 705)) break;
                const int item = *reinterpret_cast<volatile int*>(&s_item[li % kItemRing]);
                if (item < 0) break;
                int tile, kb0, nkb; item_range(item, tile, kb0, nkb);
                const int buf = li & 1;                                      // two accumulators: the epilogue of one item runs under the next
                if (li >= 2 && !mbar_wait(smem_u32(&acc_empty[buf]), (uint32_t)((li >> 1) - 1) & 1u, abort_flag, a.err, 704)) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t acc = tmem + (uint32_t)(buf * a.acc_cols);
                for (int i = 0; i < nkb; i++, f++) {
                    const int s = f % ST;
                    if (!mbar_wait(smem_u32(&full_bar[s]), (uint32_t)(f / ST) & 1u, abort_flag, a.err, 702)) { ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t sa = smem0 + (uint32_t)s * stage_bytes, sb = sa + kABytes;
                    if (i8) {                                                // 16 bf16 or 32 int8 = 32 bytes along the swizzled row per MMA
#pragma unroll
                        for (int k = 0; k < kBlockBytes / 32; k++)
                            umma_i8(acc, smem_desc_sw128(sa + k * 32), smem_desc_sw128(sb + k * 32), idesc, (uint32_t)((i | k) != 0));
                    } else {
#pragma unroll
                        for (int k = 0; k < kBlockBytes / 32; k++)
                            umma_bf16(acc, smem_desc_sw128(sa + k * 32), smem_desc_sw128(sb + k * 32), idesc, (uint32_t)((i | k) != 0));
                    }
                    umma_commit(smem_u32(&empty_bar[s]));                    // the stage is free once these MMAs have read it
                }
                umma_commit(smem_u32(&acc_full[buf]));                       // also on the way out of a failed wait
            }
        }
    } else {
        const int q = warp & 3;                                              // lane quarter of tensor memory this warp may read
        const int r_in = q * 32 + lane;
        for (int li = 0;; li++) {
            // one thread waits (for the item, then for its accumulator) and tells the other 127: a deadline that only
            // some of them saw pass must not split the group
            if (tid == 64) {
                int item = -1;
                if (mbar_wait(smem_u32(&item_bar[li % kItemRing]), (uint32_t)(li / kItemRing) & 1u, abort_flag, a.err, 706)) {
                    item = *reinterpret_cast<volatile int*>(&s_item[li % kItemRing]);
                    if (item >= 0 && !mbar_wait(smem_u32(&acc_full[li & 1]), (uint32_t)(li >> 1) & 1u, abort_flag, a.err, 703)) item = -1;
                }
                s_go = item;
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            const int item = s_go;
            asm volatile("bar.sync 1, 128;" ::: "memory");                   // s_go is rewritten for the next item
            if (item < 0) break;
            int tile, kb0, nkb; item_range(item, tile, kb0, nkb);
            const int buf = li & 1;
            const int row = tile * kTileM + r_in;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t t_row = tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * a.acc_cols);
            float* part = a.parts + (size_t)item * a.n * kTileM;
            const float ws = (a.i8 && row < a.M) ? a.wscale[row] : 1.f;
            for (int c = 0; c < a.nc && c < a.n; c += 8) {
                float hi[8], lo[8], d3[8];
                tmem_ld8(t_row + (uint32_t)c, hi);
                tmem_ld8(t_row + (uint32_t)(a.nc + c), lo);
                if (a.i8) tmem_ld8(t_row + (uint32_t)(2 * a.nc + c), d3);
#pragma unroll
                for (int e = 0; e < 8; e++) {
                    const int j = c + e;
                    if (j < a.n) {
                        float v;
                        if (a.i8) {                                          // exact s32 sums of the three digit planes
                            constexpr float k2 = 1.0f / kDigitBase, k3 = 1.0f / (kDigitBase * kDigitBase);
                            v = (float)__float_as_int(hi[e]) + (float)__float_as_int(lo[e]) * k2 + (float)__float_as_int(d3[e]) * k3;
                            v *= a.xscale[j] * ws;
                        } else v = hi[e] + lo[e];
                        if (a.KS > 1) part[(size_t)j * kTileM + r_in] = v;
                        else if (row < a.M) a.Y[a.token_major ? (size_t)j * a.M + row : (size_t)row * a.n + j] = v;
                    }
                }
            }
            // the accumulator is read (every tcgen05.ld above has been waited for): hand it back to the MMA warp
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            asm volatile("bar.sync 1, 128;" ::: "memory");                   // the four epilogue warps
            if (tid == 64) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(smem_u32(&acc_empty[buf])) : "memory");
        }
    }
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    // ── tail: nothing of this CTA may still be in flight when its shared and tensor memory go away ──
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (s_abort) {
        if (tid == 0) {                                                      // copies issued into stages nobody consumed any more
            const int issued = s_issued;
            for (int i = issued > ST ? issued - ST : 0; i < issued; i++) {
                unsigned long long t0 = global_ns();
                while (!mbar_try(smem_u32(&full_bar[i % ST]), (uint32_t)(i / ST) & 1u) && global_ns() - t0 < kWaitNs) { }
            }
        }
        if (tid == 32) {                                                     // MMAs issued before the failure: time to drain
            unsigned long long t0 = global_ns();
            while (global_ns() - t0 < 2000000ull) { }
        }
        __syncthreads();
    }
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem), "r"((uint32_t)a.tmem_cols) : "memory");
    }
}

// int4 weights (crates/atlas-quant/src/lib.rs:111-168: two values per byte, even index in the high nibble, one scale per
// block of the flat index) → two bf16 planes side by side, out[r][0..K) the hi parts and out[r][K..2K) the lo parts of
// w = q · scale (dequant_nibble, :150-157): w = hi + lo to 2⁻¹⁷ relative.  A product over the 2K columns against the
// tokens repeated (block kb of W meets block kb mod KBx of the token plane) is Σ w·x.  Thread = eight weights.
__global__ void __launch_bounds__(256) ax_int4_planes_kernel(const uint32_t* __restrict__ q, const void* __restrict__ scales, int scales_f16,
                                                             int block, int M, int K, uint16_t* __restrict__ out) {
    const size_t idx = (size_t)blockIdx.x * 256 + threadIdx.x;
    const int k8 = K / 8;
    if (idx >= (size_t)M * k8) return;
    const size_t r = idx / k8; const int wi = (int)(idx % k8);
    const uint32_t word = __ldg(q + idx);
    const size_t bi = (r * (size_t)K + (size_t)wi * 8) / (size_t)block;
    const float sc = scales_f16 ? __half2float(reinterpret_cast<const __half*>(scales)[bi]) : reinterpret_cast<const float*>(scales)[bi];
    uint32_t hi[4] = { 0u, 0u, 0u, 0u }, lo[4] = { 0u, 0u, 0u, 0u };
#pragma unroll
    for (int e = 0; e < 8; e++) {
        const uint32_t byte = (word >> (8 * (e >> 1))) & 0xFFu;
        const int nib = (e & 1) ? (int)(byte & 0xFu) : (int)(byte >> 4);
        const float w = (float)(nib >= 8 ? nib - 16 : nib) * sc;
        const uint16_t h = ax_f32_to_bf16_rne(w);
        const uint16_t l = ax_f32_to_bf16_rne(w - ax_bf16_to_f32(h));
        hi[e >> 1] |= (uint32_t)h << ((e & 1) * 16);
        lo[e >> 1] |= (uint32_t)l << ((e & 1) * 16);
    }
    uint16_t* o = out + r * 2 * (size_t)K + (size_t)wi * 8;
    *reinterpret_cast<uint4*>(o) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
    *reinterpret_cast<uint4*>(o + K) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
}

// ── int4 weights dequantised inside the product ─────────────────────────────────────────────────────────────────────
// Same product for int4 weights (crates/atlas-quant/src/lib.rs:111-168) without a detour through HBM: the four warps that
// read the accumulator at the end of an item spend its main loop as PRODUCERS of the A operand.  Thread r of them owns
// row r of the 128-row tile: per K block it loads the 32 bytes of its row (64 weights) and the two block scales,
// forms w = q · scale as dequant_nibble does (:150-157), splits w into bf16 hi + lo (w = hi + lo to 2⁻¹⁷ relative) and
// stores the two 128-byte rows into the stage's hi and lo tiles in the 128-byte swizzle the MMA descriptors expect
// (16-byte chunk c of row r at r·128 + ((c xor (r mod 8))·16)), then makes the stores visible to the tensor core
// (fence.proxy.async) and arrives on the stage's barrier beside the token tile's bulk copy.  The MMA warp issues the
// four K steps against the hi tile and the four against the lo tile into the same accumulator.  One CTA per SM, one item
// per CTA; HBM sees half a byte per weight.
struct Umma4Args {
    float* Y;
    int M, n, nc;
    const uint8_t* Wq; int row_bytes;       // int4 bytes, K / 2 per row
    const void* scales; int scales_f16, spr, block;   // scales per row = K / block, block a multiple of 32
    int KB, KS, T, stages, b_bytes, acc_cols, token_major;
    float* parts;
    int* err;
};

__device__ __forceinline__ uint32_t pack_bf16x2(float lo_elem, float hi_elem) {       // element with the lower index in the low half
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi_elem), "f"(lo_elem));      // round to nearest even, like ax_f32_to_bf16_rne
    return r;
}

__global__ void __launch_bounds__(kThreads) ax_gemv_umma_int4_kernel(const __grid_constant__ CUtensorMap map_x, const Umma4Args a) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[kMaxStages], empty_bar[kMaxStages], acc_full;
    __shared__ uint32_t s_tmem;
    __shared__ int s_abort, s_issued, s_go;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int ST = a.stages;
    const int NP = 2 * a.nc;
    const uint32_t stage_bytes = 2u * (uint32_t)kABytes + (uint32_t)a.b_bytes;
    const uint32_t smem0 = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* const smem_gen = smem_raw + (smem0 - smem_u32(smem_raw));          // the same place as a generic pointer
    volatile int* abort_flag = &s_abort;
    const int item = (int)blockIdx.x;
    const int tile = item / a.KS, ks = item - tile * a.KS;
    const int kb0 = (int)((long long)a.KB * ks / a.KS);
    const int nkb = (int)((long long)a.KB * (ks + 1) / a.KS) - kb0;

    if (tid == 0) {
        for (int s = 0; s < ST; s++) { mbar_init(smem_u32(&full_bar[s]), 1 + 128); mbar_init(smem_u32(&empty_bar[s]), 1); }
        mbar_init(smem_u32(&acc_full), 1);
        s_abort = 0; s_issued = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(smem_u32(&s_tmem)), "r"((uint32_t)a.acc_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = s_tmem;

    if (warp == 0) {
        if (lane == 0) {                                                     // token tiles
            asm volatile("griddepcontrol.wait;" ::: "memory");
            for (int i = 0; i < nkb; i++) {
                const int s = i % ST;
                if (i >= ST && !mbar_wait(smem_u32(&empty_bar[s]), (uint32_t)((i / ST) - 1) & 1u, abort_flag, a.err, 711)) break;
                const uint32_t bar = smem_u32(&full_bar[s]);
                mbar_expect_tx(bar, (uint32_t)a.b_bytes);
                tma_load_2d(smem0 + (uint32_t)s * stage_bytes + 2u * kABytes, &map_x, (kb0 + i) * 64, 0, bar);
                s_issued = i + 1;
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(NP >> 3) << 17) | ((uint32_t)(kTileM >> 4) << 24);
            for (int i = 0; i < nkb; i++) {
                const int s = i % ST;
                if (!mbar_wait(smem_u32(&full_bar[s]), (uint32_t)(i / ST) & 1u, abort_flag, a.err, 712)) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t sh = smem0 + (uint32_t)s * stage_bytes, sl = sh + kABytes, sb = sl + kABytes;
#pragma unroll
                for (int k = 0; k < kBlockBytes / 32; k++)
                    umma_bf16(tmem, smem_desc_sw128(sh + k * 32), smem_desc_sw128(sb + k * 32), idesc, (uint32_t)((i | k) != 0));
#pragma unroll
                for (int k = 0; k < kBlockBytes / 32; k++)
                    umma_bf16(tmem, smem_desc_sw128(sl + k * 32), smem_desc_sw128(sb + k * 32), idesc, 1u);
                umma_commit(smem_u32(&empty_bar[s]));
            }
            umma_commit(smem_u32(&acc_full));                                // also on the way out of a failed wait
        }
    } else {
        const int q = warp & 3;
        const int r_in = q * 32 + lane;
        const int row = tile * kTileM + r_in;
        const bool live = row < a.M;
        // ── producer of the A operand ──
        const uint8_t* wrow = a.Wq + (size_t)(live ? row : 0) * a.row_bytes;
        const size_t srow = (size_t)(live ? row : 0) * a.spr;
        // the weights of three K blocks are on their way while one is dequantised
        uint4 w0 = make_uint4(0u, 0u, 0u, 0u), w1 = w0, x0 = w0, x1 = w0, y0 = w0, y1 = w0;
        if (live) {
            w0 = ax_ldg_stream(wrow + (size_t)kb0 * 32); w1 = ax_ldg_stream(wrow + (size_t)kb0 * 32 + 16);
            if (nkb > 1) { x0 = ax_ldg_stream(wrow + (size_t)(kb0 + 1) * 32); x1 = ax_ldg_stream(wrow + (size_t)(kb0 + 1) * 32 + 16); }
            if (nkb > 2) { y0 = ax_ldg_stream(wrow + (size_t)(kb0 + 2) * 32); y1 = ax_ldg_stream(wrow + (size_t)(kb0 + 2) * 32 + 16); }
        }
        // the two block scales of a K block (its 64 weights lie in one or two blocks), fetched as far ahead as the weights
        auto scales_of = [&](int kb) {
            float2 r;
            const size_t b0 = srow + (size_t)((kb * 64) / a.block), b1 = srow + (size_t)((kb * 64 + 32) / a.block);
            if (a.scales_f16) { r.x = __half2float(reinterpret_cast<const __half*>(a.scales)[b0]); r.y = __half2float(reinterpret_cast<const __half*>(a.scales)[b1]); }
            else { r.x = reinterpret_cast<const float*>(a.scales)[b0]; r.y = reinterpret_cast<const float*>(a.scales)[b1]; }
            return r;
        };
        float2 sw = make_float2(0.f, 0.f), sx = sw, sy = sw;
        if (live) { sw = scales_of(kb0); if (nkb > 1) sx = scales_of(kb0 + 1); if (nkb > 2) sy = scales_of(kb0 + 2); }
        bool ok = true;
        for (int i = 0; i < nkb; i++) {
            const int s = i % ST, kb = kb0 + i;
            uint4 n0 = make_uint4(0u, 0u, 0u, 0u), n1 = n0;
            if (live && i + 3 < nkb) { n0 = ax_ldg_stream(wrow + (size_t)(kb + 3) * 32); n1 = ax_ldg_stream(wrow + (size_t)(kb + 3) * 32 + 16); }
            const float sc[2] = { sw.x, sw.y };
            float2 sn = make_float2(0.f, 0.f);
            if (live && i + 3 < nkb) sn = scales_of(kb + 3);
            if (i >= ST) {                                                   // one thread waits for the stage and tells the others
                if (tid == 64) s_go = mbar_wait(smem_u32(&empty_bar[s]), (uint32_t)((i / ST) - 1) & 1u, abort_flag, a.err, 713) ? 1 : 0;
                asm volatile("bar.sync 1, 128;" ::: "memory");
                const int go = s_go;
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (!go) { ok = false; break; }
            }
            uint8_t* hi_row = smem_gen + (size_t)s * stage_bytes + (size_t)r_in * 128;
            uint8_t* lo_row = hi_row + kABytes;
            const uint32_t words[8] = { w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w };
#pragma unroll
            for (int c = 0; c < 8; c++) {                                    // word c: elements 8c .. 8c+7, two per byte, even index in the high nibble
                const float scale = sc[c >> 2];
                float v[8];
#pragma unroll
                for (int e = 0; e < 8; e++) {                                // signed bit-field extract: one instruction per nibble
                    int nib;
                    asm("bfe.s32 %0, %1, %2, 4;" : "=r"(nib) : "r"(words[c]), "r"(8 * (e >> 1) + ((e & 1) ? 0 : 4)));
                    v[e] = (float)nib * scale;
                }
                uint32_t h[4], l[4];
#pragma unroll
                for (int p2 = 0; p2 < 4; p2++) {
                    h[p2] = pack_bf16x2(v[2 * p2], v[2 * p2 + 1]);
                    l[p2] = pack_bf16x2(v[2 * p2] - __uint_as_float(h[p2] << 16), v[2 * p2 + 1] - __uint_as_float(h[p2] & 0xFFFF0000u));
                }
                const int off = (c ^ (r_in & 7)) << 4;
                *reinterpret_cast<uint4*>(hi_row + off) = make_uint4(h[0], h[1], h[2], h[3]);
                *reinterpret_cast<uint4*>(lo_row + off) = make_uint4(l[0], l[1], l[2], l[3]);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // generic-proxy stores → visible to the tensor core's reads
            asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(smem_u32(&full_bar[s])) : "memory");
            w0 = x0; w1 = x1; x0 = y0; x1 = y1; y0 = n0; y1 = n1;
            sw = sx; sx = sy; sy = sn;
        }
        // ── epilogue ──
        if (tid == 64) s_go = (ok && mbar_wait(smem_u32(&acc_full), 0u, abort_flag, a.err, 714)) ? 1 : 0;
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (s_go) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t t_row = tmem + ((uint32_t)(q * 32) << 16);
            float* part = a.parts + (size_t)item * a.n * kTileM;
            for (int c = 0; c < a.nc && c < a.n; c += 8) {
                float hi[8], lo[8];
                tmem_ld8(t_row + (uint32_t)c, hi);
                tmem_ld8(t_row + (uint32_t)(a.nc + c), lo);
#pragma unroll
                for (int e = 0; e < 8; e++) {
                    const int j = c + e;
                    if (j < a.n) {
                        const float v = hi[e] + lo[e];
                        if (a.KS > 1) part[(size_t)j * kTileM + r_in] = v;
                        else if (live) a.Y[a.token_major ? (size_t)j * a.M + row : (size_t)row * a.n + j] = v;
                    }
                }
            }
        }
    }
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (s_abort) {
        if (tid == 32) { unsigned long long t0 = global_ns(); while (global_ns() - t0 < 2000000ull) { } }     // MMAs and copies issued before the failure: time to drain
        __syncthreads();
    }
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem), "r"((uint32_t)a.acc_cols) : "memory");
    }
}

// Partial tiles of a K-split product → Y: thread = four rows of one token of one row tile, splits added in order (the
// result does not depend on timing).  The whole GPU takes part: the sums are a few MB that lie in L2.
__global__ void __launch_bounds__(256) ax_umma_merge_kernel(const float* __restrict__ parts, float* __restrict__ Y, int M, int n, int KS, int T,
                                                            int token_major) {
    asm volatile("griddepcontrol.wait;" ::: "memory");                      // every partial tile of the product is written
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const size_t idx = (size_t)blockIdx.x * 256 + threadIdx.x;
    if (idx >= (size_t)T * n * (kTileM / 4)) return;
    const int r4 = (int)(idx & (kTileM / 4 - 1)) * 4;
    const size_t tj = idx / (kTileM / 4);
    const int j = (int)(tj % (size_t)n), tile = (int)(tj / (size_t)n);
    const size_t split_stride = (size_t)n * kTileM;
    const float* p = parts + (size_t)tile * KS * split_stride + (size_t)j * kTileM + r4;
    float4 v[kMaxSplits];
#pragma unroll
    for (int s = 0; s < kMaxSplits; s++)
        if (s < KS) v[s] = __ldcg(reinterpret_cast<const float4*>(p + s * split_stride));
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int s = 0; s < kMaxSplits; s++)
        if (s < KS) { acc.x += v[s].x; acc.y += v[s].y; acc.z += v[s].z; acc.w += v[s].w; }
    const int row = tile * kTileM + r4;
    if (token_major) {
        // one 16-byte store where the four rows exist and the address allows it (row is a multiple of 4, so M must be one too)
        if (row + 3 < M && (M & 3) == 0) *reinterpret_cast<float4*>(Y + (size_t)j * M + row) = acc;
        else { const float o[4] = { acc.x, acc.y, acc.z, acc.w }; for (int e = 0; e < 4; e++) if (row + e < M) Y[(size_t)j * M + row + e] = o[e]; }
    } else {
        const float o[4] = { acc.x, acc.y, acc.z, acc.w };
        for (int e = 0; e < 4; e++) if (row + e < M) Y[(size_t)(row + e) * n + j] = o[e];
    }
}

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// bf16 or int8 matrix [rows][cols] (cols contiguous), boxes of 128 bytes × box_rows rows, 128-byte swizzle, zeros outside
int make_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows, bool i8) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return atlasx_fail(ATLASX_ERR_CUDA, "the driver does not export cuTensorMapEncodeTiled");
    const cuuint64_t esz = i8 ? 1 : 2;
    const cuuint64_t dims[2] = { cols, rows };
    const cuuint64_t strides[1] = { cols * esz };
    const cuuint32_t box[2] = { (cuuint32_t)(kBlockBytes / esz), box_rows };
    const cuuint32_t elem[2] = { 1, 1 };
    const CUresult r = fn(map, i8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return atlasx_fail(ATLASX_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
    return ATLASX_OK;
}

struct UmmaPlan { int nc, planes, kblk, T, KB, KS, stages, b_bytes, acc_cols, tmem_cols, persist, grid; size_t plane_bytes, xscale_bytes, parts_bytes, head_bytes, smem; };

// cols: columns of W as the product walks them; x_cols: columns of the tokens (= cols, or cols / 2 for expanded int4 weights)
UmmaPlan make_plan(const atlasx_ctx* ctx, int rows, int cols, int n, bool i8, int x_cols = 0) {
    if (x_cols <= 0) x_cols = cols;
    UmmaPlan p;
    p.planes = i8 ? 3 : 2;
    p.nc = i8 ? (n + 15) / 16 * 16 : (n + 7) / 8 * 8;         // planes·nc must be a multiple of 16
    p.kblk = i8 ? 128 : 64;
    p.T = (rows + kTileM - 1) / kTileM;
    p.KB = (cols + p.kblk - 1) / p.kblk;                       // the copy engine zero-fills a last, partial block
    // K splits: the launch is modelled as waves of CTAs (two per SM), each wave lasting as long as one item — its K blocks,
    // stretched by the partial tile it writes and the merge reads (relative to the weight bytes of the item), plus a
    // fixed cost per item (start-up, latency of the first copies, epilogue) of six blocks' streaming time.  Fitted on
    // 4096², 12288×4096, 22016×4096 and 4096×11008 at 16 and 64 tokens: within 2 % of the best count on average
    // (plain wave filling chose five splits for 22016×4096, 15 % slower than three).  At least four K blocks per item.
    // Resident CTAs (see below) pay less per item — no start-up, the epilogue runs under the next item: two blocks.
    constexpr double kItemBlocks = 6.0, kItemBlocksResident = 2.0;
    int c = 32; while (c < p.planes * p.nc) c <<= 1;           // columns of one accumulator
    const int per_sm = 2 * c <= 256 ? 2 : 1;                   // resident form: two accumulators per CTA inside 512 columns
    const long long slots_p = (long long)per_sm * ctx->sm_count;
    auto resident = [&](int ks) {
        const long long items = (long long)p.T * ks;
        return ctx->tune.umma_persist && p.KB / ks >= 4 && items > slots_p &&
               (ctx->tune.umma_persist == 2 || p.KB / ks >= 16 || items >= 4 * slots_p);
    };
    const int slots = 2 * ctx->sm_count;
    int best = 1; double best_cost = 1e300;
    for (int ks = 1; ks <= kMaxSplits && ks * 4 <= (p.KB > 4 ? p.KB : 4); ks++) {
        const long long items = (long long)p.T * ks;
        const long long waves = (items + slots - 1) / slots;
        const double extra = ks > 1 ? 2.0 * n * kTileM * sizeof(float) * ks / ((double)p.KB * kABytes) : 0.0;
        const double cost = (double)waves * ((double)p.KB / ks * (1.0 + extra) + (resident(ks) ? kItemBlocksResident : kItemBlocks));
        if (cost < best_cost - 1e-9) { best_cost = cost; best = ks; }
    }
    if (ctx->tune.umma_ks > 0 && ctx->tune.umma_ks <= kMaxSplits && ctx->tune.umma_ks * 4 <= (p.KB > 4 ? p.KB : 4)) best = ctx->tune.umma_ks;
    p.KS = best;
    p.b_bytes = p.planes * p.nc * kBlockBytes;
    int st = (100 * 1024) / (kABytes + p.b_bytes);
    if (st > kMaxStages) st = kMaxStages;
    if (st < 2) st = 2;
    p.stages = st;
    p.acc_cols = c;
    // Persistent form (the rule is `resident` above): CTAs stay and take items from a counter, with two accumulators so
    // that the epilogue of an item runs under the MMAs of the next.  Used when there are more items than CTA slots and
    // either the items are long (at least 16 K blocks) or there are many per CTA (at least four): lm_head-like matrices
    // and the wide layer matrices, where it measured 10–25 % faster; a few SHORT items per CTA cost more in handshakes
    // than fresh CTAs do.  Two CTAs per SM need their two allocations inside the 512 columns of tensor memory (with
    // 256-column accumulators one CTA per SM stays, with twice the stages); the item ring needs items of at least four blocks.
    p.persist = resident(p.KS) ? 1 : 0;
    p.tmem_cols = p.persist ? 2 * c : c;
    p.grid = p.persist ? per_sm * ctx->sm_count : p.T * p.KS;
    if (p.persist && per_sm == 1) {                                          // one CTA per SM: it may use twice the stages
        st = (200 * 1024) / (kABytes + p.b_bytes);
        if (st > kMaxStages) st = kMaxStages;
        p.stages = st;
    }
    p.plane_bytes = ((size_t)p.planes * p.nc * x_cols * (i8 ? 1 : 2) + 1023) / 1024 * 1024;
    p.xscale_bytes = i8 ? 256 : 0;
    p.parts_bytes = p.KS > 1 ? (size_t)p.T * p.KS * n * kTileM * sizeof(float) : 0;
    p.head_bytes = kHeadBytes;                                           // the item counter
    p.smem = (size_t)st * (kABytes + p.b_bytes) + 1024;
    return p;
}

}  // namespace

bool ax_gemv_umma_supported(const AxWeight& w, int n, const float* x, const float* y) {
    if (n < 2 || n > kMaxTokens || !x || !y) return false;
    if ((((uintptr_t)w.data | (uintptr_t)x) & 15) != 0) return false;
    if (w.dtype == ATLASX_BF16) return w.cols % 8 == 0 && w.cols >= 64;          // row pitch a multiple of 16 bytes
    if (w.dtype == ATLASX_INT8) return n <= kMaxTokensI8 && w.cols % 16 == 0 && w.cols >= 128 && w.scales != nullptr;
    return false;
}

size_t ax_gemv_umma_scratch_bytes(const atlasx_ctx* ctx, const AxWeight& w, int n) {
    const UmmaPlan p = make_plan(ctx, w.rows, w.cols, n, w.dtype == ATLASX_INT8);
    return p.plane_bytes + p.xscale_bytes + p.parts_bytes + p.head_bytes;
}

// Where a producer kernel may leave the bf16 hi|lo plane of n tokens for a product with w (bf16 weights): rows 0..n8−1
// hi parts, n8..2·n8−1 lo parts, row pitch w.cols, rows of absent tokens zero.  *plane stays null where the product
// takes its tokens as f32 only (int8 weights, a scratch that was not sized for it).
int ax_gemv_umma_plane(atlasx_ctx* ctx, const AxWeight& w, int n, uint16_t** plane, int* n8) {
    AX_ARG(plane && n8, "null argument");
    *plane = nullptr; *n8 = 0;                                               // no plane: the caller hands x over as usual
    alignas(16) static float dummy[4];
    if (w.dtype != ATLASX_BF16 || !ax_gemv_umma_supported(w, n, dummy, dummy)) return ATLASX_OK;
    const UmmaPlan p = make_plan(ctx, w.rows, w.cols, n, false);
    if (p.head_bytes + p.plane_bytes + p.parts_bytes > ctx->split_scratch_cap) return ATLASX_OK;
    *plane = reinterpret_cast<uint16_t*>(reinterpret_cast<uint8_t*>(ctx->split_scratch) + p.head_bytes);
    *n8 = p.nc;
    return ATLASX_OK;
}

// x == nullptr: the token plane was left at ax_gemv_umma_plane's address by the kernels before (bf16 weights; the
// item counter of the resident form sets itself back).
size_t ax_gemv_umma_parts_bytes(const atlasx_ctx* ctx, const AxWeight& w, int n) {
    return make_plan(ctx, w.rows, w.cols, n, w.dtype == ATLASX_INT8).parts_bytes;
}

namespace {
// x_cols: columns of the tokens; w.cols = 2 · x_cols for int4 weights expanded into two planes side by side
int umma_launch(atlasx_ctx* ctx, const AxWeight& w, const float* x, int n, float* y, bool token_major, bool pdl,
                float* ext_parts, AxUmmaParts* pend, int x_cols) {
    const bool prepared = x == nullptr;
    if (prepared) x = y;                                                     // for the argument checks only
    AX_ARG(ax_gemv_umma_supported(w, n, x, y), "shape or format not covered by the tcgen05 multi-column kernel");
    const bool i8 = w.dtype == ATLASX_INT8;
    const UmmaPlan p = make_plan(ctx, w.rows, w.cols, n, i8, x_cols);
    int rc = atlasx_ctx_ensure_split_scratch(ctx, p.plane_bytes + p.xscale_bytes + p.parts_bytes + p.head_bytes);
    if (rc) return rc;
    // scratch: [item counter, in an area of its own at the start][token planes][token scales][partial tiles]
    unsigned* counter = reinterpret_cast<unsigned*>(ctx->split_scratch);
    uint8_t* base = reinterpret_cast<uint8_t*>(ctx->split_scratch) + p.head_bytes;
    float* xscale = reinterpret_cast<float*>(base + p.plane_bytes);
    float* parts = reinterpret_cast<float*>(base + p.plane_bytes + p.xscale_bytes);

    CUtensorMap map_w, map_x;
    const uint32_t np = (uint32_t)(p.planes * p.nc);
    if ((rc = make_map(&map_w, w.data, (uint64_t)w.rows, (uint64_t)w.cols, kTileM, i8))) return rc;
    if ((rc = make_map(&map_x, base, (uint64_t)np, (uint64_t)x_cols, np, i8))) return rc;

    static bool attr_done[64] = {};
    const int dev = ctx->device & 63;
    if (!attr_done[dev]) {
        AX_CUDA(cudaFuncSetAttribute(ax_gemv_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 210 * 1024));
        attr_done[dev] = true;
    }
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    AX_ARG(!prepared || !i8, "a prepared token plane needs bf16 weights");
    AX_ARG((ext_parts == nullptr) == (pend == nullptr), "a buffer for the partial tiles and their description go together");
    const bool defer = ext_parts != nullptr;
    if (defer) { pend->parts = p.KS > 1 ? ext_parts : nullptr; pend->KS = p.KS; pend->n = n; }
    if (!prepared) {
        cudaLaunchConfig_t cfg = {};
        cfg.blockDim = dim3(256); cfg.stream = ctx->stream;
        if (pdl) { cfg.attrs = attr; cfg.numAttrs = 1; }
        if (i8) {
            cfg.gridDim = dim3((unsigned)p.nc);
            AX_CUDA(cudaLaunchKernelEx(&cfg, ax_umma_digits_kernel, x, x_cols, n, p.nc, token_major ? 1 : 0,
                                       reinterpret_cast<int8_t*>(base), xscale, counter));
        } else {
            const size_t work = (size_t)2 * p.nc * (x_cols / 8);
            cfg.gridDim = dim3((unsigned)((work + 255) / 256));
            AX_CUDA(cudaLaunchKernelEx(&cfg, ax_umma_split_kernel, x, x_cols, n, p.nc, token_major ? 1 : 0,
                                       reinterpret_cast<uint16_t*>(base), counter));
        }
    }
    UmmaArgs a;
    a.Y = y; a.M = w.rows; a.n = n; a.nc = p.nc; a.i8 = i8 ? 1 : 0; a.planes = p.planes; a.kblk = p.kblk;
    a.wscale = reinterpret_cast<const float*>(w.scales); a.xscale = xscale;
    a.KB = p.KB; a.KS = p.KS; a.T = p.T; a.KBx = (x_cols + p.kblk - 1) / p.kblk;
    a.stages = p.stages; a.b_bytes = p.b_bytes; a.acc_cols = p.acc_cols; a.tmem_cols = p.tmem_cols; a.persist = p.persist; a.counter = counter; a.token_major = token_major ? 1 : 0;
    a.parts = defer ? ext_parts : parts; a.err = ctx->dev_error;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)p.grid); cfg.blockDim = dim3(kThreads); cfg.dynamicSmemBytes = p.smem; cfg.stream = ctx->stream;
    if (!prepared || pdl) { cfg.attrs = attr; cfg.numAttrs = 1; }            // its producer warp waits for the kernel before itself
    AX_CUDA(cudaLaunchKernelEx(&cfg, ax_gemv_umma_kernel, map_w, map_x, a));
    if (p.KS > 1 && !defer) {
        cudaLaunchConfig_t mc = {};
        mc.gridDim = dim3((unsigned)(((size_t)p.T * n * (kTileM / 4) + 255) / 256)); mc.blockDim = dim3(256); mc.stream = ctx->stream;
        mc.attrs = attr; mc.numAttrs = 1;                                    // it waits for the product itself
        AX_CUDA(cudaLaunchKernelEx(&mc, ax_umma_merge_kernel, (const float*)parts, y, w.rows, n, p.KS, p.T, token_major ? 1 : 0));
    }
    return ATLASX_OK;
}
}  // namespace

int ax_gemv_umma_launch(atlasx_ctx* ctx, const AxWeight& w, const float* x, int n, float* y, bool token_major, bool pdl,
                        float* ext_parts, AxUmmaParts* pend) {
    return umma_launch(ctx, w, x, n, y, token_major, pdl, ext_parts, pend, w.cols);
}

// int4 weights, 17..128 tokens: the matrix is expanded into two bf16 planes side by side in context scratch (eight
// bytes per weight written and read back — still several times faster than 16 tokens at a time on the warp-level
// kernel, whose block scales stand between the MMAs of a row) and multiplied like a bf16 matrix of twice the columns.
bool ax_gemv_umma_int4_supported(const AxWeight& w, int n, const float* x, const float* y) {
    if (w.dtype != ATLASX_INT4 || n < 2 || n > kMaxTokens || !x || !y || !w.scales) return false;
    if ((((uintptr_t)w.data | (uintptr_t)x) & 15) != 0) return false;
    return w.block >= 8 && w.block % 8 == 0 && w.cols % w.block == 0 && w.cols % 64 == 0;     // whole K blocks: the token tile index wraps at K
}

namespace {
// int4 weights dequantised inside the product (ax_gemv_umma_int4_kernel): block scales over multiples of 32 elements
int umma_int4_fused_launch(atlasx_ctx* ctx, const AxWeight& w, const float* x, int n, float* y, bool token_major) {
    const int K = w.cols, nc = (n + 7) / 8 * 8, NP = 2 * nc;
    const int b_bytes = NP * kBlockBytes;
    const int stage = 2 * kABytes + b_bytes;
    int st = (200 * 1024) / stage;
    if (st > kMaxStages) st = kMaxStages;
    if (st < 2) st = 2;
    const int T = (w.rows + kTileM - 1) / kTileM, KB = K / 64;
    // K splits as in make_plan, with one CTA per SM
    int best = 1; double best_cost = 1e300;
    for (int ks = 1; ks <= kMaxSplits && ks * 4 <= (KB > 4 ? KB : 4); ks++) {
        const long long items = (long long)T * ks;
        const long long waves = (items + ctx->sm_count - 1) / ctx->sm_count;
        const double extra = ks > 1 ? 2.0 * n * kTileM * sizeof(float) * ks / ((double)KB * kABytes) : 0.0;
        const double cost = (double)waves * ((double)KB / ks * (1.0 + extra) + 6.0);
        if (cost < best_cost - 1e-9) { best_cost = cost; best = ks; }
    }
    const int KS = best;
    int c = 32; while (c < NP) c <<= 1;
    const size_t plane_bytes = ((size_t)NP * K * 2 + 1023) / 1024 * 1024;
    const size_t parts_bytes = KS > 1 ? (size_t)T * KS * n * kTileM * sizeof(float) : 0;
    int rc = atlasx_ctx_ensure_split_scratch(ctx, kHeadBytes + plane_bytes + parts_bytes);
    if (rc) return rc;
    unsigned* counter = reinterpret_cast<unsigned*>(ctx->split_scratch);
    uint8_t* base = reinterpret_cast<uint8_t*>(ctx->split_scratch) + kHeadBytes;
    float* parts = reinterpret_cast<float*>(base + plane_bytes);
    CUtensorMap map_x;
    if ((rc = make_map(&map_x, base, (uint64_t)NP, (uint64_t)K, (uint32_t)NP, false))) return rc;
    static bool attr_done[64] = {};
    const int dev = ctx->device & 63;
    if (!attr_done[dev]) {
        AX_CUDA(cudaFuncSetAttribute(ax_gemv_umma_int4_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 210 * 1024));
        attr_done[dev] = true;
    }
    {
        const size_t work = (size_t)2 * nc * (K / 8);
        ax_umma_split_kernel<<<(unsigned)((work + 255) / 256), 256, 0, ctx->stream>>>(x, K, n, nc, token_major ? 1 : 0, reinterpret_cast<uint16_t*>(base), counter);
        AX_CHECK_LAUNCH("ax_umma_split_kernel");
    }
    Umma4Args a;
    a.Y = y; a.M = w.rows; a.n = n; a.nc = nc;
    a.Wq = reinterpret_cast<const uint8_t*>(w.data); a.row_bytes = K / 2;
    a.scales = w.scales; a.scales_f16 = w.scales_f16; a.spr = K / w.block; a.block = w.block;
    a.KB = KB; a.KS = KS; a.T = T; a.stages = st; a.b_bytes = b_bytes; a.acc_cols = c; a.token_major = token_major ? 1 : 0;
    a.parts = parts; a.err = ctx->dev_error;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(T * KS)); cfg.blockDim = dim3(kThreads); cfg.dynamicSmemBytes = (size_t)st * stage + 1024; cfg.stream = ctx->stream;
    cfg.attrs = attr; cfg.numAttrs = 1;                                      // the weights are dequantised while the split kernel still runs
    AX_CUDA(cudaLaunchKernelEx(&cfg, ax_gemv_umma_int4_kernel, map_x, a));
    if (KS > 1) {
        cudaLaunchConfig_t mc = {};
        mc.gridDim = dim3((unsigned)(((size_t)T * n * (kTileM / 4) + 255) / 256)); mc.blockDim = dim3(256); mc.stream = ctx->stream;
        mc.attrs = attr; mc.numAttrs = 1;
        AX_CUDA(cudaLaunchKernelEx(&mc, ax_umma_merge_kernel, (const float*)parts, y, w.rows, n, KS, T, token_major ? 1 : 0));
    }
    return ATLASX_OK;
}
}  // namespace

int ax_gemv_umma_int4_launch(atlasx_ctx* ctx, const AxWeight& w, const float* x, int n, float* y, bool token_major, bool pdl) {
    AX_ARG(ax_gemv_umma_int4_supported(w, n, x, y), "shape or format not covered by the expanded int4 product");
    if (ctx->tune.int4_fused && w.block % 32 == 0) return umma_int4_fused_launch(ctx, w, x, n, y, token_major);
    const size_t need = (size_t)w.rows * 2 * (size_t)w.cols * sizeof(uint16_t);
    if (need > ctx->w_planes_cap) {
        cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
        cudaStreamIsCapturing(ctx->stream, &st);
        if (st != cudaStreamCaptureStatusNone) return atlasx_fail(ATLASX_ERR_STATE, "the int4 plane scratch must be sized before stream capture");
        AX_CUDA(cudaStreamSynchronize(ctx->stream));
        cudaFree(ctx->w_planes); ctx->w_planes = nullptr; ctx->w_planes_cap = 0;
        AX_CUDA(cudaMalloc(&ctx->w_planes, need));
        ctx->w_planes_cap = need;
    }
    const size_t words = (size_t)w.rows * (w.cols / 8);
    ax_int4_planes_kernel<<<(unsigned)((words + 255) / 256), 256, 0, ctx->stream>>>(
        reinterpret_cast<const uint32_t*>(w.data), w.scales, w.scales_f16, w.block, w.rows, w.cols, reinterpret_cast<uint16_t*>(ctx->w_planes));
    AX_CHECK_LAUNCH("ax_int4_planes_kernel");
    AxWeight wp;
    wp.data = ctx->w_planes; wp.rows = w.rows; wp.cols = 2 * w.cols; wp.dtype = ATLASX_BF16;
    (void)pdl;                                                // the expansion kernel in front is an ordinary launch
    return umma_launch(ctx, wp, x, n, y, token_major, false, nullptr, nullptr, w.cols);
}
