// attention.cuh — KV-cache write, QK-norm + RoPE, and split-K GQA decode attention.
#pragma once
#include "common.cuh"

struct AxAttnArgs {
    const float* q = nullptr;        // [batch × n_heads × hd], already normed and rotated
    const void* kc = nullptr;        // [batch][max_seq × n_kv × hd], bf16 bits or f32
    const void* vc = nullptr;
    size_t seq_stride = 0;           // elements between batch entries of the cache
    float* out = nullptr;            // [batch × n_heads × hd]
    const int* pos = nullptr;        // device [batch] (or one shared value if pos_shared) …
    int pos_shared = 0;              // … 1: every batch entry uses pos[0]
    int pos_scalar = 0;              // … used when pos == nullptr
    int batch = 1, n_heads = 0, n_kv = 0, hd = 0, window = 0;
    int kv_dtype = ATLASX_BF16;
    float scale = 1.f;
    int n_splits = 1;
    // split partials [batch × n_heads × n_splits × (hd + 2)] floats and tickets [batch × n_heads] (zero
    // between launches) owned by the caller; null: context scratch, grown on demand (never inside a graph)
    float* scratch_partials = nullptr; unsigned* scratch_tickets = nullptr;
};

// Chooses the split count for a launch that must fill the GPU whatever the position is.
int ax_attn_pick_splits(const atlasx_ctx* ctx, int n_kv, int batch, int max_rows);
int ax_attn_launch(atlasx_ctx* ctx, const AxAttnArgs& a, bool pdl = false);

// Per-head RMSNorm of q and k (eps given by the caller), rotate-half RoPE from tables at row
// pos, then k and v stored into the cache at pos (bf16 nearest-even or f32).  q is rewritten
// in place.  Restates the sequence of crates/atlas-model/src/lib.rs:848-862.
struct AxQkPrepArgs {
    float* q = nullptr;              // [batch × n_heads × hd]
    const float* k = nullptr;        // [batch × n_kv × hd]
    const float* v = nullptr;
    const float* q_norm = nullptr;   // [n_heads × hd] or null
    const float* k_norm = nullptr;   // [n_kv × hd] or null
    const float* cos_t = nullptr;    // [max_seq × hd/2] or null (no rotation)
    const float* sin_t = nullptr;
    void* kc = nullptr; void* vc = nullptr; size_t seq_stride = 0;
    const int* pos = nullptr; int pos_shared = 0; int pos_scalar = 0;
    int batch = 1, n_heads = 0, n_kv = 0, hd = 0, kv_dtype = ATLASX_BF16;
    float eps = 1e-6f;
    size_t q_stride = 0, kv_in_stride = 0;   // elements between batch entries of q and of k/v
};
int ax_qk_prep_launch(atlasx_ctx* ctx, const AxQkPrepArgs& a, bool pdl = false);

// Decode attention of one layer for one sequence, head_dim 128, as ONE launch: per-head RMSNorm
// of q and k, rotate-half RoPE, the cache write at `pos`, and split attention over the cached
// rows (restates crates/atlas-model/src/lib.rs:848-870).  Cached rows are requested before the
// kernel waits for its predecessor in the stream — they were written by earlier steps.
struct AxFusedAttnArgs {
    const float* qkv = nullptr;      // raw [q (n_heads·128) | k (n_kv·128) | v (n_kv·128)] of this token
    const float* q_norm = nullptr;   // [n_heads × 128] or null
    const float* k_norm = nullptr;   // [n_kv × 128] or null
    const float* cos_t = nullptr;    // [max_seq × 64] or null
    const float* sin_t = nullptr;
    void* kc = nullptr; void* vc = nullptr;      // [max_seq × n_kv × 128], bf16 bits or f32
    float* out = nullptr;            // [n_heads × 128]
    const int* pos = nullptr;        // device scalar, written at least two kernels earlier in the stream
    int n_heads = 0, n_kv = 0, window = 0, kv_dtype = ATLASX_BF16;
    int max_splits = 1;              // grid.x; the kernel uses ⌈rows/64⌉ of them, the rest exit at once
    float scale = 1.f, qk_eps = 1e-6f;
    // split partials [n_heads × max_splits × 130] floats and tickets [n_heads] (zero between launches)
    // owned by the caller — a captured graph must not depend on context scratch that a later call may
    // re-allocate; null: context scratch
    float* scratch_partials = nullptr; unsigned* scratch_tickets = nullptr;
};
bool ax_attn_fused_supported(int hd, int n_heads, int n_kv);
int ax_attn_fused_max_splits(const atlasx_ctx* ctx, int n_kv, int max_rows);
int ax_attn_fused_launch(atlasx_ctx* ctx, const AxFusedAttnArgs& a, bool pdl = false);
int ax_attn_init(atlasx_ctx* ctx);      // one-time function attributes
