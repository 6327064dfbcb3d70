// attention_mma.cuh — tensor-core GQA decode attention (attention_mma.cu).
#pragma once
#include "attention.cuh"

// bf16 cache, head_dim 128, 3..8 query heads per KV head, 16-byte aligned buffers
bool ax_attn_mma_supported(const AxAttnArgs& a);
int ax_attn_mma_pick_splits(const atlasx_ctx* ctx, int n_kv, int batch, int max_rows);
// a.q already normed and rotated, the cache already holds row pos; partial results of split s of head h
// at (h·n_splits + s)·130 floats of the scratch
int ax_attn_mma_launch(atlasx_ctx* ctx, const AxAttnArgs& a, bool pdl = false);

// Causal attention of a chunk of n_tok ≤ 16 prompt tokens at positions *pos0 .. *pos0 + n_tok − 1, whose K/V
// rows are already in the (bf16, head_dim 128) cache: one launch per layer.
struct AxAttnChunkArgs {
    const float* q = nullptr; size_t q_stride = 0;     // token i, head h: q + i·q_stride + h·128, normed and rotated
    const void* kc = nullptr; const void* vc = nullptr;
    float* out = nullptr; size_t out_stride = 0;       // token i, head h: out + i·out_stride + h·128
    uint16_t* out_plane = nullptr; int plane_rows = 0; // instead of out: bf16 hi|lo plane [2·plane_rows][n_heads·128] (row i hi parts of
                                                       // token i, row plane_rows + i lo parts), as the tcgen05 product reads its tokens
    const int* pos0 = nullptr;                         // device
    int n_tok = 0, n_heads = 0, n_kv = 0, window = 0, n_splits = 1;
    float scale = 1.f;
    float* partials = nullptr; unsigned* tickets = nullptr;   // ax_attn_mma_chunk_partial_floats(); n_kv · row groups, zero between launches
};
bool ax_attn_mma_chunk_supported(int hd, int n_heads, int n_kv, int kv_dtype);
int ax_attn_mma_chunk_splits(const atlasx_ctx* ctx, int n_heads, int n_kv, int n_tok, int max_rows);
size_t ax_attn_mma_chunk_partial_floats(int n_tok, int n_heads, int n_splits);
int ax_attn_mma_chunk_max_splits();                  // scratch is sized for this many
int ax_attn_mma_chunk_launch(atlasx_ctx* ctx, const AxAttnChunkArgs& a, bool pdl = false);
