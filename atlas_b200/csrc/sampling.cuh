// sampling.cuh — launch interface of the device sampling pipeline (sampling.cu).
#pragma once
#include "common.cuh"

struct AxSamplingParams {
    float temperature = 1.f, repetition_penalty = 1.f; int repetition_window = 64;
    float frequency_penalty = 0.f, presence_penalty = 0.f, top_p = 1.f; int top_k = 0; float min_p = 0.f;
};
AxSamplingParams ax_sampling_params(const atlasx_sampling_config& c);

struct AxSampleArgs {
    const float* logits; int n;
    AxSamplingParams cfg;
    int step;                                  // 0: the suppress list applies
    const unsigned* suppress; int n_suppress;  // device list
    // history counts: either rebuilt from a device token list (counts must be zero on entry) …
    const unsigned* hist; int n_hist; int win_len;
    // … or advanced by one token: tok_in joins the history (and the repetition window), tok_out leaves the window (−1: none)
    int tok_in, tok_out;
    float* work; float* cval; int* cidx; float* skey; int* sval; int* cnt_all; int* cnt_win;
    unsigned long long* rng;                   // XorShift64 state, advanced by one draw
    int* token_out;
    float* probs_out;                          // optional [n]: the final distribution
    // generation state of a model (optional): the token becomes the input of the position about to be processed
    int* last_token; int* seq; const int* pos; int seq_cap;
};
int ax_sample_ensure_scratch(atlasx_ctx* ctx, int n);
void ax_sample_free_scratch(atlasx_ctx* ctx);
int ax_sample_reset_counts(atlasx_ctx* ctx, int n);
int ax_sample_launch(atlasx_ctx* ctx, const AxSampleArgs& a);
