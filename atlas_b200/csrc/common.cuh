// common.cuh — shared device helpers and host-side error plumbing (sm_100a only).
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stddef.h>
#include <stdio.h>
#include <string>

#include "../../include/atlas_kernels.h"

// ── host error plumbing ─────────────────────────────────────────────────────────
void atlasx_set_error(const char* fmt, ...);
int  atlasx_fail(int code, const char* fmt, ...);

#define AX_CUDA(expr)                                                                     \
    do {                                                                                  \
        cudaError_t _e = (expr);                                                          \
        if (_e != cudaSuccess)                                                            \
            return atlasx_fail(ATLASX_ERR_CUDA, "%s failed: %s (%s:%d)", #expr,           \
                               cudaGetErrorString(_e), __FILE__, __LINE__);               \
    } while (0)

#define AX_CHECK_LAUNCH(what)                                                             \
    do {                                                                                  \
        cudaError_t _e = cudaGetLastError();                                              \
        if (_e != cudaSuccess)                                                            \
            return atlasx_fail(ATLASX_ERR_CUDA, "launch of %s failed: %s", what,          \
                               cudaGetErrorString(_e));                                   \
    } while (0)

#define AX_ARG(cond, msg)                                                                 \
    do { if (!(cond)) return atlasx_fail(ATLASX_ERR_ARG, "%s: %s", __func__, msg); } while (0)

#define AX_MAX_PEERS 8

// ── context ─────────────────────────────────────────────────────────────────────
struct atlasx_comm;   // comm.cpp

// scratch of the device sampling pipeline (sampling.cu), sized for the largest vocabulary seen
struct AxSampleScratch {
    int cap = 0;
    float* work = nullptr; float* cval = nullptr; int* cidx = nullptr; float* skey = nullptr; int* sval = nullptr;
    int* cnt_all = nullptr; int* cnt_win = nullptr;
    unsigned long long* rng = nullptr; int* token = nullptr;
    unsigned* list = nullptr; int list_cap = 0;        // suppress list + history of the operator form
};

struct atlasx_ctx {
    int device = 0;
    int sm_count = 148;
    size_t smem_optin = 0;
    cudaStream_t stream = nullptr;
    int gemv_impl = 0;                 // 0 auto, 1 plain loads, 2 bulk-copy pipeline
    int carveout = 50;                 // shared-memory share of the L1 array requested per launch (percent), −1: driver's choice.
                                       // One value for every kernel of a step: neighbours in the stream then fit on an SM together
    // Experiment switches, read from the environment once when the context is created (never on a launch path)
    struct Tuning {
        int gemv_threads = 512;        // ATLASX_GEMV_THREADS=256: two 256-thread CTAs per SM instead of one 512-thread CTA
        int pdl_mask = 0x7FFFFFFF;     // ATLASX_PDL_MASK: bit per launch class of the decode step
        int attn_fused = 1;            // ATLASX_ATTN_FUSED=0: QK-norm/RoPE/cache write and attention as two launches
        int attn_stages = 3;           // ATLASX_ATTN_STAGES: landing stages of the one-launch attention inside a step (2..4)
        int attn_rows = 0;             // ATLASX_ATTN_ROWS: cached rows per split of the one-launch attention (0: 64)
        int attn_wave = 2;             // ATLASX_ATTN_WAVE: attention CTAs per SM that one wave of splits may fill
        int attn_mma = 1;              // ATLASX_ATTN_MMA=0: operator-form GQA attention on the scalar kernels instead of the tensor cores
        int umma = 1;                  // ATLASX_UMMA=0: token batches on the warp-level MMA kernel instead of tcgen05
        int umma_fused = 1;            // ATLASX_UMMA_FUSED=0: prompt chunks always split their tokens in a kernel of its own
        int int4_fused = 1;            // ATLASX_INT4_FUSED=0: int4 token batches through bf16 planes in scratch instead of dequantising inside the product
        int umma_ks = 0;               // ATLASX_UMMA_KS=k: K splits of the tcgen05 product fixed instead of chosen by its cost model
        int umma_persist = 1;          // ATLASX_UMMA_PERSIST=0: one item per CTA instead of resident CTAs fed by a counter
        int attn_pack = 1;             // ATLASX_ATTN_PACK=0: ≤ 4 heads per KV head as columns with separate hi / lo MMAs
        int attn_cfg = -1;             // ATLASX_ATTN_CFG: shape 0..4 (warps × stages × rows per tile) of the tensor-core attention; -1 = by problem size
        int peer_allreduce = 1;        // ATLASX_PEER_ALLREDUCE=0: ncclAllReduce instead of the peer mailboxes
        int mail_reduce = -1;          // ATLASX_MAIL_REDUCE: mailbox parts summed 0 = by every consumer CTA, 1 = by a kernel of their own,
                                       // 2 = by the first CTAs of the consumer (default, −1)
        int tp_select = 1;             // ATLASX_TP_SELECT=0: greedy selection always over all-gathered logits
        int step_trace = 0;            // ATLASX_STEP_TRACE=1: timeline stamps in the captured step
        int comm_timeout_ms = 30000;   // ATLASX_COMM_TIMEOUT_MS: host deadline for a tensor-parallel step to complete
    } tune;
    // attention scratch (split-K partials + tickets), grown on demand
    float* attn_partials = nullptr;  size_t attn_partials_cap = 0;   // floats
    unsigned* attn_tickets = nullptr; size_t attn_tickets_cap = 0;   // uints, always zero between launches
    int* pos_dev = nullptr; size_t pos_cap = 0;
    void* split_scratch = nullptr; size_t split_scratch_cap = 0;   // bf16 hi/lo planes of the multi-column input
    void* w_planes = nullptr; size_t w_planes_cap = 0;             // int4 weights of one matrix expanded to bf16 hi | lo planes (token batches)
    // argmax scratch
    float* amax_vals = nullptr; int* amax_idx = nullptr; unsigned* amax_ticket = nullptr; int* amax_out = nullptr;
    // device error word written by bounded waits
    int* dev_error = nullptr;          // device
    int* host_pin = nullptr;           // pinned scratch (ints)
    atlasx_comm* comm = nullptr;
    AxSampleScratch sample;
    // timeline recording (diagnostics): when non-null, the next traced launch stamps six u64
    // at this address — first/last CTA start, first dependency release, last CTA end, first CTA end, last input staged —
    // and the launcher advances the pointer
    unsigned long long* trace_next = nullptr;
};

// Timeline stamps of one launch; t is read from %globaltimer (ns).
struct AxTraceSlot { unsigned long long first_start, last_start, first_release, last_end, first_end, last_staged; };
__device__ __forceinline__ unsigned long long ax_globaltimer() {
    unsigned long long t; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t)); return t;
}
__device__ __forceinline__ void ax_trace_start(unsigned long long* tr) {
    if (tr && threadIdx.x == 0) { const unsigned long long t = ax_globaltimer(); atomicMin(tr + 0, t); atomicMax(tr + 1, t); }
}
__device__ __forceinline__ void ax_trace_release(unsigned long long* tr) {
    if (tr && threadIdx.x == 0) atomicMin(tr + 2, ax_globaltimer());
}
__device__ __forceinline__ void ax_trace_end(unsigned long long* tr) {
    if (tr && threadIdx.x == 0) { const unsigned long long t = ax_globaltimer(); atomicMax(tr + 3, t); atomicMin(tr + 4, t); }
}
__device__ __forceinline__ void ax_trace_staged(unsigned long long* tr) {
    if (tr && threadIdx.x == 0) atomicMax(tr + 5, ax_globaltimer());
}

int atlasx_ctx_ensure_attn_scratch(atlasx_ctx* ctx, size_t partial_floats, size_t tickets);
int atlasx_ctx_ensure_split_scratch(atlasx_ctx* ctx, size_t bytes);

// ── device helpers ──────────────────────────────────────────────────────────────
#define AX_FULL 0xFFFFFFFFu

__device__ __forceinline__ float ax_warp_sum(float v) {
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(AX_FULL, v, d);
    return v;
}
__device__ __forceinline__ float ax_warp_max(float v) {
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) v = fmaxf(v, __shfl_xor_sync(AX_FULL, v, d));
    return v;
}
__device__ __forceinline__ float ax_bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float ax_bf16_hi(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }
__device__ __forceinline__ float ax_bf16_to_f32(uint16_t h) { return __uint_as_float(((uint32_t)h) << 16); }
__device__ __host__ __forceinline__ uint16_t ax_f32_to_bf16_rne_bits(uint32_t u) {
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((u >> 16) | 0x40);
    u += 0x7FFFu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}
__device__ __forceinline__ uint16_t ax_f32_to_bf16_rne(float f) { return ax_f32_to_bf16_rne_bits(__float_as_uint(f)); }

// 128-bit streaming load that does not pollute L1 (weights are read exactly once)
__device__ __forceinline__ uint4 ax_ldg_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// argmax candidates: index −1 means "none yet"; NaN never beats a candidate; `last` selects the
// CPU rule of generate() (last index among equal maxima) instead of the first.
__device__ __forceinline__ bool ax_better(float va, int ia, float vb, int ib, int last) {
    if (ia < 0) return false;
    if (ib < 0) return true;
    if (va > vb) return true;
    if (va == vb) return last ? ia > ib : ia < ib;
    return false;
}
__device__ __forceinline__ void ax_warp_best(float& v, int& i, int last) {
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
        const float ov = __shfl_xor_sync(AX_FULL, v, d);
        const int oi = __shfl_xor_sync(AX_FULL, i, d);
        if (ax_better(ov, oi, v, i, last)) { v = ov; i = oi; }
    }
}

// ── seeded synthetic data: integer-exact hash → approximately N(0,1) ────────────
// base = mix64(seed ^ mix64(stream)); h1 = mix64(base+2i); h2 = mix64(base+2i+1);
// z = ((bytesum(h1)+bytesum(h2 & 0xffffffff) − 1530)·65536 + ((h2>>32)&0xffff) − 32768) / 2^24
__host__ __device__ __forceinline__ uint64_t ax_mix64(uint64_t z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
__host__ __device__ __forceinline__ uint32_t ax_bytesum64(uint64_t v) {
    v = (v & 0x00FF00FF00FF00FFull) + ((v >> 8) & 0x00FF00FF00FF00FFull);
    v = (v & 0x0000FFFF0000FFFFull) + ((v >> 16) & 0x0000FFFF0000FFFFull);
    return (uint32_t)(v & 0xFFFFFFFFull) + (uint32_t)(v >> 32);
}
__host__ __device__ __forceinline__ float ax_synth_normal(uint64_t base, uint64_t i) {
    uint64_t h1 = ax_mix64(base + 2 * i);
    uint64_t h2 = ax_mix64(base + 2 * i + 1);
    int32_t s = (int32_t)(ax_bytesum64(h1) + ax_bytesum64(h2 & 0xFFFFFFFFull));
    int32_t u = (int32_t)((h2 >> 32) & 0xFFFF);
    int32_t zi = (s - 1530) * 65536 + (u - 32768);
    return (float)zi * (1.0f / 16777216.0f);
}
