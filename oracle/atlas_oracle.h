/*
 * atlas_oracle.h — CPU restatement of ATLAS's single-token decode path.
 *
 * TEST INFRASTRUCTURE ONLY.  This is the checker that the CUDA path is compared
 * against (tests, the smoke check and the CPU-baseline leg of the benchmark).
 * Nothing in the shipped library links, loads or calls it.
 *
 * Every function follows one function of the reference, cited as
 * crate/file:line of web3guru888/ATLAS.  Arithmetic is f32 with the reference's
 * operation order (sequential left-to-right sums, no fused multiply-add), so the
 * build must use -ffp-contract=off and must not use -ffast-math.
 *
 * Pinning: the reference holds no byte-level golden vectors for this path, only
 * scalar known answers and tolerance tests (atlas-tensor/src/lib.rs:1097-1220,
 * atlas-quant/src/lib.rs:258-297, atlas-model/src/lib.rs:3108-3123,3393-3517).
 * Those are reproduced in tests/test_oracle_pins.py.  Token/logit parity of the
 * whole model is additionally checked on the GPU against the reference's own
 * CUDA kernels compiled from kernels/matmul.cu (oracle/_ref).
 */
#ifndef ATLAS_ORACLE_H
#define ATLAS_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ── seeded synthetic data (integer-exact, identical on host and device) ───── */
uint64_t orc_mix64(uint64_t z);
/* element i of stream (seed, stream): approximately N(0,1); construction described in the .c file */
float    orc_synth_normal(uint64_t seed, uint64_t stream, uint64_t i);
void     orc_fill_normal_f32(float* dst, size_t n, uint64_t seed, uint64_t stream, float std);
/* bf16 by round-to-nearest-even of the f32 value */
void     orc_fill_normal_bf16(uint16_t* dst, size_t n, uint64_t seed, uint64_t stream, float std);
void     orc_fill_uniform_u32(uint32_t* dst, size_t n, uint64_t seed, uint64_t stream, uint32_t modulo);
uint16_t orc_f32_to_bf16_rne(float f);
uint16_t orc_f32_to_bf16_trunc(float f);      /* atlas-model/src/lib.rs:2274 */
float    orc_bf16_to_f32(uint16_t h);         /* atlas-model/src/lib.rs:2217-2225 */

/* reference's own LCG initialiser, atlas-model/src/lib.rs:2725-2732 */
void     orc_pseudo_randn(float* dst, size_t n, uint64_t seed);

/* ── atlas-quant formats ───────────────────────────────────────────────────── */
/* Int8Tensor::quantize / dequantize, atlas-quant/src/lib.rs:41-75 */
void orc_int8_quantize(const float* src, size_t rows, size_t cols, int8_t* data, float* scales);
void orc_int8_dequantize(const int8_t* data, const float* scales, size_t rows, size_t cols, float* out);
/* Int4Tensor::quantize / dequantize, atlas-quant/src/lib.rs:111-168.
 * data must hold (n+1)/2 bytes and be zero-initialised by the caller (the reference
 * starts from vec![0u8]); scales holds ceil(n/block) floats. */
void orc_int4_quantize(const float* src, size_t n, size_t block, uint8_t* data, float* scales);
void orc_int4_dequantize(const uint8_t* data, const float* scales, size_t n, size_t block, float* out);

/* ── math helpers ──────────────────────────────────────────────────────────── */
void  orc_rmsnorm_inplace(float* x, const float* w, size_t n, float eps); /* atlas-model/src/lib.rs:335-342 */
float orc_silu(float x);                                                  /* :346-348 */
void  orc_softmax_inplace(float* x, size_t n);                            /* :351-357 */
size_t orc_argmax(const float* x, size_t n);                              /* :2701-2706 (last of equal maxima) */

/* RopeCache::new, atlas-model/src/lib.rs:380-423.  scaling: 0 none, 1 YaRN. */
void orc_rope_tables(int head_dim, int max_seq, float theta, int scaling,
                     float factor, int orig_max_pos, float beta_fast, float beta_slow,
                     float* cos_out, float* sin_out);
/* RopeCache::apply, :427-437 */
void orc_rope_apply(float* x, int head_dim, const float* cos_row, const float* sin_row);

/* Linear::forward CPU branch, :494-498.  Rows run in parallel (bit-identical). */
void orc_linear_f32 (const float*    W, const float* x, float* y, size_t out_dim, size_t in_dim);
void orc_linear_bf16(const uint16_t* W, const float* x, float* y, size_t out_dim, size_t in_dim);
/* multi-column: Y[out×n] = W[out×in] · X[in×n], X and Y row-major (layout of
 * kernels/matmul.cu:384-420), each output a sequential f32 sum over k. */
void orc_gemm_f32 (const float*    W, const float* X, float* Y, size_t out_dim, size_t n, size_t in_dim);
void orc_gemm_bf16(const uint16_t* W, const float* X, float* Y, size_t out_dim, size_t n, size_t in_dim);

/* one-token GQA attention over an f32 cache laid out [max_seq × n_kv × hd];
 * restates the loop of Attention::forward_token, atlas-model/src/lib.rs:689-721.
 * window 0 = full. */
void orc_decode_attention(const float* q, const float* kc, const float* vc, float* out,
                          int n_heads, int n_kv, int hd, int pos, float scale, int window);

/* ── model ─────────────────────────────────────────────────────────────────── */
typedef struct {
    int   vocab_size, d_model, n_layers, n_heads, n_kv_heads, ffn_hidden, max_seq_len;
    float rope_theta, rms_norm_eps;
    int   sliding_window;        /* 0 = none */
    int   rope_scaling;          /* 0 none, 1 YaRN */
    float yarn_factor; int yarn_orig_max_pos;
    float yarn_attn_factor, yarn_beta_fast, yarn_beta_slow;
    int   post_norm;             /* OLMo-2/3 post-norm branch */
    int   eos_token_id;          /* -1 = none */
} orc_config;

enum {
    ORC_T_EMBED = 0, ORC_T_FINAL_NORM = 1, ORC_T_LM_HEAD = 2,
    ORC_T_WQ = 10, ORC_T_WK, ORC_T_WV, ORC_T_WO, ORC_T_GATE, ORC_T_UP, ORC_T_DOWN,
    ORC_T_ATTN_NORM, ORC_T_FFN_NORM, ORC_T_Q_NORM, ORC_T_K_NORM
};

typedef struct orc_model orc_model;

/* layer_sliding: n_layers ints (1 = sliding) or NULL for all-full. */
orc_model* orc_model_new(const orc_config* cfg, const int* layer_sliding);
void       orc_model_free(orc_model* m);
/* Borrow a tensor (not copied).  dtype 0 = f32, 1 = bf16 bits.  Norm vectors must be f32. */
int        orc_model_set_tensor(orc_model* m, int layer, int which, const void* data, int dtype);
/* OlmoModel::new random init, atlas-model/src/lib.rs:1322-1353 (LCG weights, tied lm_head,
 * unit norms, pre-norm, no QK-norm).  Allocates and owns the weights. */
void       orc_model_init_reference_random(orc_model* m);
/* round K (after RoPE) and V to bf16 (nearest-even) when written to the cache */
void       orc_model_set_kv_round_bf16(orc_model* m, int on);
void       orc_model_reset(orc_model* m);                         /* :1389-1392 */
int        orc_model_pos(const orc_model* m);
/* Measurement aid (no reference counterpart): pretend `pos` tokens were already processed — the
 * cache rows [0,pos) of every layer are filled with seeded N(0,1) values and the position is set,
 * so that a timed forward_one reads as much context as a run that really ingested a prompt. */
void       orc_model_seed_context(orc_model* m, int pos, uint64_t seed);
/* forward_one_hooked, :1425-1445.  hidden_out (optional) receives the residual
 * stream after every layer, n_layers × d_model. */
void       orc_forward_one(orc_model* m, uint32_t token, float* logits, float* hidden_out);
/* generate_with_sampling greedy branch, :1605-1646,1713-1730.
 * logits_trace (optional): max_new × vocab logits that each emitted token was chosen from.
 * margin_trace (optional): per step top1−top2 of the (modified) logits.
 * Returns the number of tokens written to out_tokens. */
int        orc_generate_greedy(orc_model* m, const uint32_t* prompt, int n_prompt, int max_new,
                               const uint32_t* suppress, int n_suppress,
                               float rep_penalty, int rep_window,
                               const uint32_t* stops, int n_stops,
                               uint32_t* out_tokens, float* logits_trace, float* margin_trace);

/* ── sampling (atlas-model/src/lib.rs: Rng :1190-1216, SamplingConfig :1223-1294, primitives
 *    :2581-2717, generate_with_sampling :1599-1732) ─────────────────────────────────────────── */
typedef struct {
    float temperature;          /* ≤ 0 or < 1e-6: greedy */
    float repetition_penalty;   /* 1.0 = off */
    int   repetition_window;
    float frequency_penalty, presence_penalty;
    float top_p;                /* 1.0 = off */
    int   top_k;                /* 0 = off */
    float min_p;                /* 0.0 = off */
} orc_sampling;
uint64_t orc_rng_from_seed(uint64_t seed);                       /* Rng::from_seed :1205-1207: seed | 1 */
float    orc_rng_next_f32(uint64_t* state);                      /* xorshift 13/7/17, top 31 bits / 2^31 :1210-1215 */
void   orc_apply_repetition_penalty(float* logits, size_t n, const uint32_t* toks, int nt, float theta);   /* :2581-2592 */
void   orc_apply_frequency_penalty(float* logits, size_t n, const uint32_t* history, int nh, float penalty); /* counts as built at :1662-1670, then :2598-2605 */
void   orc_apply_presence_penalty(float* logits, size_t n, const uint32_t* history, int nh, float penalty);  /* :1675-1680, :2610-2617 */
void   orc_apply_top_k(float* logits, size_t n, size_t k);       /* :2657-2686 */
/* :2625-2655.  The reference orders equal probabilities with an unstable sort (unspecified);
 * here ties keep index order. */
void   orc_apply_top_p(float* logits, size_t n, float p);
void   orc_apply_min_p(float* logits, size_t n, float min_p);    /* :2692-2699 */
size_t orc_sample_from_probs(const float* probs, size_t n, float r);   /* :2710-2717 */
/* One selection as generate_with_sampling makes it (:1625-1710) from the logits of the last forward:
 * step-0 suppression, penalties over `history` (the tokens generated so far), temperature, top-k,
 * top-p, min-p, softmax, sample with one draw from *rng — or the greedy branch.  probs_out
 * (optional, n floats) receives the final distribution (sampling branch only). */
size_t orc_sample_token(const float* last_logits, size_t n, const orc_sampling* cfg, int step,
                        const uint32_t* suppress, int n_suppress, const uint32_t* history, int n_hist,
                        uint64_t* rng, float* probs_out);
/* generate_with_sampling with a fixed seed instead of the system time.  Returns the token count. */
int    orc_generate_sampling(orc_model* m, const uint32_t* prompt, int n_prompt, int max_new, const orc_sampling* cfg,
                             const uint32_t* suppress, int n_suppress, const uint32_t* stops, int n_stops,
                             uint64_t seed, uint32_t* out_tokens);

void orc_set_threads(int n);
int  orc_get_threads(void);

#ifdef __cplusplus
}
#endif
#endif
