// mega.cuh — the whole decode step as ONE persistent kernel (one CTA per SM).
//
// Why: at batch 1 a token is ~190 dependent kernels of 5–30 µs each.  Even with programmatic
// dependent launch every kernel boundary leaves HBM idle for a few microseconds (drain, launch,
// input staging, first DRAM round trip).  Here the producer warp of every CTA walks the list of
// weight matrices of the whole token and keeps its shared-memory ring full without ever waiting
// for activations, so the weight stream does not stop at operation boundaries; the consumer warps
// run the operations in order and meet at a grid-wide barrier between them (a monotonic counter
// in global memory, bounded waits).  Attention, QK-norm, RoPE, the KV write and the greedy
// selection are phases of the same kernel.
#pragma once
#include "gemv_device.cuh"

enum { MEGA_GEMV = 0, MEGA_ATTN = 1, MEGA_SELECT_PART = 2, MEGA_SELECT_FINAL = 3 };

struct MegaPhase {
    int type;
    // MEGA_GEMV
    GemvArgs g;
    // prologue source "merged attention output": x[h·hd + d] = Σ_s w_s·acc_s[d] / Σ_s w_s·l_s
    const float* merge_partials;     // [n_heads × splits × (hd + 2)] or null
    int merge_heads, merge_hd, merge_splits;
    // MEGA_ATTN: QK-norm + RoPE + KV write + split attention for one layer
    const float* qkv;                // raw [q | k | v] of this token
    const float* q_norm; const float* k_norm; const float* cos_t; const float* sin_t;
    void* kc; void* vc;
    float* partials;
    const int* pos;
    int n_heads, n_kv, hd, window, kv_bf16, splits;
    float scale, qk_eps;
    // MEGA_SELECT_*
    const float* logits; int vocab;
    float* sel_vals; int* sel_idx;
    int* st_pos; int* st_nforced; int* st_last; int* seq; int seq_cap;
};

struct MegaSync {
    unsigned long long count;        // arrivals, monotonic over the life of the model
    unsigned long long base;         // value of `count` when the current launch began
};

struct MegaArgs {
    const MegaPhase* phases;
    int n_phases;
    MegaSync* sync;
    int* err;
    int stages, stage_stride, seg_pitch;
    int x_bytes;                     // shared memory reserved for the staged input / attention scratch
    unsigned long long* trace;       // optional [n_phases × 4] timestamps of CTA 0 (ns): wait begin/end, staged, done
};

// fmt: weight format of every matrix of the step; kv_bf16: cache element type
int ax_mega_launch(atlasx_ctx* ctx, int fmt, int kv_bf16, const MegaArgs& args, size_t smem_bytes);
int ax_mega_init(atlasx_ctx* ctx);
