// gemv.cuh — launch interface of the weight-streaming GEMV family.
#pragma once
#include "common.cuh"

// One weight matrix in HBM, row-major [rows × cols].
//   F32  : float
//   BF16 : bf16 bit patterns
//   INT8 : int8 + f32 scale per row                      (Int8Tensor, atlas-quant/src/lib.rs:32-39)
//   INT4 : two nibbles per byte, even index in the high nibble, one scale per `block`
//          elements of the flat index, f32 or f16          (Int4Tensor, :101-109)
struct AxWeight {
    const void* data = nullptr;
    const void* scales = nullptr;
    int rows = 0, cols = 0;
    int dtype = ATLASX_F32;
    int block = 0;
    int scales_f16 = 0;
};

// Optional input transform run by every CTA while the first weight tiles are in flight:
//   t   = Σ_{p<nparts} y[p·part_stride + i]                     (row-parallel partial sums)
//   t   = wy ? rmsnorm(t, wy, eps) : t
//   v   = base + t            (base = residual stream, or an embedding row)  [if y]
//   resid_out = v             (CTA 0 only)
//   x   = wx ? rmsnorm(v, wx, eps) : v
// With y == nullptr and wx == nullptr the GEMV input is just `base`.
struct AxPrologue {
    const float* base = nullptr;        // f32 vector [K] …
    const void*  embed = nullptr;       // … or an embedding table (row = seq[*pos], clamped to vocab−1)
    int embed_bf16 = 0; int vocab = 0;
    const int* seq = nullptr; const int* pos = nullptr;
    const float* y = nullptr; int nparts = 0; size_t part_stride = 0;
    const float* wy = nullptr; const float* wx = nullptr;
    float eps = 0.f;
    float* resid_out = nullptr;
    // Tensor parallel with peer mailboxes: `y` points at ll_n parts of (value, sequence) pairs,
    // 8 bytes per element, written by the GPUs of the group with single 8-byte stores.  An element
    // is valid once its sequence word equals *ll_epoch·ll_mul + ll_add; the prologue polls each
    // element it needs (bounded) — no fence and no separate flag on either side.
    int ll_n = 0; size_t ll_stride = 0;              // parts, and elements between parts
    const unsigned* ll_epoch = nullptr; unsigned ll_mul = 0, ll_add = 0;
    // With ll_red set the parts are summed once per GPU instead of by every CTA: the first
    // ll_red_ctas CTAs of the grid each poll a slice of all parts, add them in rank order and leave
    // the sums in ll_red as (value, sequence) pairs again; every CTA then polls that one local
    // vector.  Same result as summing the parts itself, one L2 round trip later, without the
    // n × 8·K bytes of polling per CTA and without a reduction kernel of its own in the stream.
    uint2* ll_red = nullptr; int ll_red_ctas = 0;
    int base_early = 0;                 // `base` was written at least two kernels back in the stream: may be read before the dependency wait
};

// Row-parallel output under tensor parallelism: instead of a local vector the result (this rank's
// partial sums) goes into slot `rank` of every rank's mailbox over NVLink as (value, sequence)
// pairs — one 8-byte store per element, so value and sequence number arrive together and the
// reader needs neither a fence nor a flag (the scheme NCCL calls LL).
struct AxPeerOut {
    int n = 0;                           // ranks (0: plain local store into y)
    uint2* y[AX_MAX_PEERS] = {};         // destination of this rank's part in rank p's mailbox
    const unsigned* epoch = nullptr; unsigned mul = 0, add = 0;   // sequence word: *epoch·mul + add
};

// Sum of the n_parts mailbox parts (value, sequence pairs) of one use into a plain f32 vector, in
// rank order; every pair is polled (bounded) until its sequence word equals *epoch·mul + add.
// One small kernel between producer and consumer: with many ranks it replaces the polling of all
// parts by every CTA of the consumer (n_parts × 8·d bytes per CTA) by one pass per GPU.
int ax_mail_reduce_launch(atlasx_ctx* ctx, const uint2* parts, int n_parts, size_t stride, int d,
                          const unsigned* epoch, unsigned mul, unsigned add, float* out, bool pdl);

enum { AX_EPI_PLAIN = 0, AX_EPI_SILU_PAIR = 1 };   // pair: out[r/2] = silu(acc[r])·acc[r+1], r even

// Kernel-side view of one GEMV (built by ax_gemv_launch).
struct GemvArgs {
    const uint8_t* W; const uint8_t* scales;
    int M, K;                    // rows, cols (elements)
    int row_bytes;               // bytes of one weight row
    int srow_bytes;              // bytes of one row of int4 scales (0 otherwise)
    int block; int scales_f16;
    int spr;                     // int4: scales per row (cols / block)
    int bshift;                  // int4: log2(block / 32), or −1 when block / 32 is no power of two
    int stages; int stage_stride; int seg_pitch;   // ring geometry (TMA)
    int nchunks;                 // 16-byte chunks per row
    int epi;
    float* y;
    AxPrologue pro;
    AxPeerOut peer;
    int* err;
    unsigned long long* trace;   // diagnostics: timeline stamps of this launch, or null
};

// y[rows×n] = W·x.  n == 1: pro/epi honoured.  n in 2..16: plain only, x is [cols×n] row-major.
int ax_gemv_launch(atlasx_ctx* ctx, const AxWeight& w, const AxPrologue& pro, int epi, int n, float* y,
                   bool pdl = false, const AxPeerOut* peer = nullptr);
// Tensor-core path for n = 2..16 columns (bf16 / int8 / int4 weights); X [cols×n], Y [rows×n] row-major f32.
bool ax_gemv_mma_supported(const AxWeight& w, int n, const float* x, const float* y);
size_t ax_gemv_mma_scratch_bytes(int rows, int cols);   // context scratch one such product needs
// token_major: X is [n][cols] and Y is [n][rows] (one contiguous vector per column).
int ax_gemv_mma_launch(atlasx_ctx* ctx, const AxWeight& w, const float* x, int n, float* y, bool token_major = false);
// tcgen05 path for n = 2..64 tokens (bf16 weights with cols a multiple of 8, int8 weights with cols a multiple of 16);
// same operand layouts as above.
bool ax_gemv_umma_supported(const AxWeight& w, int n, const float* x, const float* y);
size_t ax_gemv_umma_scratch_bytes(const atlasx_ctx* ctx, const AxWeight& w, int n);
// Partial tiles of a K-split product that its caller adds up itself: element (token j, row r) is the sum over
// s = 0..KS−1, in this order and starting from 0.0f, of parts[((r / 128 · KS + s) · n + j) · 128 + r % 128].
// KS ≤ 1: nothing is pending, Y holds the result.
struct AxUmmaParts {
    const float* parts = nullptr; int KS = 0, n = 0;
    __host__ __device__ bool pending() const { return KS > 1; }
    __device__ __forceinline__ float at(int j, int r) const {
        const float* p = parts + ((size_t)(r >> 7) * KS * n + j) * 128 + (r & 127);
        float v[8];                                       // every split's load is issued before the first addition
#pragma unroll
        for (int s = 0; s < 8; s++) if (s < KS) v[s] = __ldcg(p + (size_t)s * n * 128);
        float acc = 0.f;
#pragma unroll
        for (int s = 0; s < 8; s++) if (s < KS) acc += v[s];
        return acc;
    }
};
// ext_parts + pend: the partial tiles of a K-split product go to the caller's buffer (ax_gemv_umma_parts_bytes) and
// are NOT added up — Y is then not written; *pend tells the consumer how to read them.
int ax_gemv_umma_launch(atlasx_ctx* ctx, const AxWeight& w, const float* x, int n, float* y, bool token_major = false, bool pdl = false,
                        float* ext_parts = nullptr, AxUmmaParts* pend = nullptr);
size_t ax_gemv_umma_parts_bytes(const atlasx_ctx* ctx, const AxWeight& w, int n);
// int4 weights, up to 128 tokens: expanded to two bf16 planes in context scratch, then the bf16 product
bool ax_gemv_umma_int4_supported(const AxWeight& w, int n, const float* x, const float* y);
int ax_gemv_umma_int4_launch(atlasx_ctx* ctx, const AxWeight& w, const float* x, int n, float* y, bool token_major = false, bool pdl = false);
// bf16 weights: address at which producer kernels may leave the hi|lo token plane themselves (then x = nullptr above)
int ax_gemv_umma_plane(atlasx_ctx* ctx, const AxWeight& w, int n, uint16_t** plane, int* n8);
int ax_gemv_init(atlasx_ctx* ctx);      // one-time function attributes
size_t ax_weight_bytes(const AxWeight& w);
