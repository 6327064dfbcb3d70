/*
 * atlas_kernels.h — C ABI of the B200 (sm_100a) decode-path library, libatlas_kernels.
 *
 * Two groups of entry points:
 *
 *  1. atlas_*  — the reference's existing kernel ABI, symbol for symbol, so that
 *     crates/atlas-tensor (mod ffi, src/lib.rs:17-92) links against this library
 *     instead of the archive built from kernels/matmul.cu.  Same argument order,
 *     same layouts, legacy default stream, void returns.
 *
 *  2. atlasx_* — the surface the B200 path adds behind the same Rust types
 *     (GpuMatrix, GpuVec, GpuRopeTables, GpuKvCache, OlmoModel, Int8Tensor,
 *     Int4Tensor): weight formats bf16/f32/int8/int4, fused decode step, BF16 KV
 *     cache, split-K attention, tensor-parallel sharding.  Every atlasx_* call
 *     returns 0 on success or a negative code; atlasx_last_error() gives the text.
 *
 * All pointers named *_dev are device pointers, *_host are host pointers.
 * There is no CPU fallback: without a CUDA device every atlasx_* call fails.
 */
#ifndef ATLAS_KERNELS_H
#define ATLAS_KERNELS_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ════════════════════════════════════════════════════════════════════════════
 * 1. Reference ABI (declared in crates/atlas-tensor/src/lib.rs:20-91, defined in
 *    kernels/matmul.cu at the lines given).  Device pointers, stream 0.
 * ════════════════════════════════════════════════════════════════════════════ */
void atlas_sync(void);                                                              /* matmul.cu:464 */
/* C[M×N] = A[M×K]·B[K×N], all row-major f32; N==1 is the GEMV path.                   matmul.cu:470 */
void atlas_matmul_f32(const float* A, const float* B, float* C, int M, int N, int K);
/* same with A as bf16 bit patterns (W16A32).                                          matmul.cu:636 */
void atlas_sgemm_bf16_f32(const uint16_t* A_bf16, const float* B, float* C, int M, int N, int K);
void atlas_vec_add_f32(const float* a, const float* b, float* out, int n);          /* matmul.cu:522 */
void atlas_scale_f32(const float* x, float s, float* out, int n);                   /* matmul.cu:528 */
void atlas_relu_f32(const float* x, float* out, int n);                             /* matmul.cu:534 */
void atlas_softmax_f32(const float* x, float* out, int rows, int cols);             /* matmul.cu:540 */
void atlas_rmsnorm_f32(const float* x, const float* w, float* out, int n, float eps); /* matmul.cu:597 */
void atlas_rope_apply_f32(float* x, int pos, int head_dim, float theta_base);       /* matmul.cu:607 */
void atlas_silu_mul_f32(const float* gate, const float* up, float* out, int n);     /* matmul.cu:614 */
void atlas_vram_copy_f32(const float* src, float* dst, int n);                      /* matmul.cu:620 */
void atlas_adamw_step(float* param, float* m, float* v, const float* grad,          /* matmul.cu:546 */
                      float lr, float beta1, float beta2, float eps, float wd,
                      float bc1, float bc2, int n);
void atlas_qk_norm_inplace(float* x, const float* w, int n_heads, int head_dim, float eps); /* matmul.cu:703 */
void atlas_rope_precomputed(float* x, const float* cos_tab, const float* sin_tab,   /* matmul.cu:898 */
                            int n_heads, int head_dim, int pos, int max_seq);
void atlas_kv_cache_write(float* k_cache, float* v_cache, const float* new_k,       /* matmul.cu:909 */
                          const float* new_v, int pos, int n_kv_heads, int head_dim);
/* f32 cache [max_seq × n_kv × hd]; window 0 = full.  Any context length (the reference
 * kernel is limited by its shared-memory score array).                                matmul.cu:921 */
void atlas_decode_attention(const float* q, const float* k_cache, const float* v_cache,
                            float* out, int n_heads, int n_kv_heads, int head_dim,
                            int pos, float scale, int window_size);
/* index of the FIRST maximum, written as a float, as the reference kernel does.       matmul.cu:997 */
void atlas_gpu_argmax(const float* x, float* out_f32, int n);
int  atlas_cuda_available(void);                                                    /* matmul.cu:589 */
int  atlas_cuda_device_count(void);                                                 /* matmul.cu:582 */
/* exported by the reference but not declared in its Rust FFI block.  NOTE: these keep the
 * reference KERNEL semantics (ties-to-even, zero scale for an all-zero row, per-tensor
 * int4 scale), which differ from the atlas-quant formats; use atlasx_quantize_* for those. */
void atlas_quantize_int8(const float* input, int8_t* output, float* scale, int n_rows, int n_cols); /* matmul.cu:559 */
void atlas_dequantize_int8(const int8_t* input, const float* scale, float* output, int n_rows, int n_cols); /* matmul.cu:567 */
void atlas_quantize_int4(const float* input, uint8_t* output, float* scale, int n);  /* matmul.cu:575 */

/* ════════════════════════════════════════════════════════════════════════════
 * 2. B200 surface
 * ════════════════════════════════════════════════════════════════════════════ */
#define ATLASX_OK            0
#define ATLASX_ERR_ARG      (-1)
#define ATLASX_ERR_CUDA     (-2)
#define ATLASX_ERR_NOGPU    (-3)
#define ATLASX_ERR_COMM     (-4)
#define ATLASX_ERR_TIMEOUT  (-5)   /* a bounded device-side wait ran out */
#define ATLASX_ERR_STATE    (-6)

enum atlasx_dtype { ATLASX_F32 = 0, ATLASX_BF16 = 1, ATLASX_INT8 = 2, ATLASX_INT4 = 3,
                    ATLASX_F16 = 4 /* a file dtype only: converted to f32 while loading */ };
#define ATLASX_AUTO (-1)      /* weight_format for the loaders: bf16 when the file's linear weights are BF16, else f32 */

/* message of the last failing atlasx_* call on this thread ("" if none) */
const char* atlasx_last_error(void);

/* ── context: one GPU, one stream; replaces the implicit stream-0 world of
 *    crates/atlas-tensor/src/lib.rs:147-292 for the new path ───────────────────── */
typedef struct atlasx_ctx atlasx_ctx;
int   atlasx_ctx_create(int device, atlasx_ctx** out);
int   atlasx_ctx_destroy(atlasx_ctx* ctx);
int   atlasx_ctx_sync(atlasx_ctx* ctx);
void* atlasx_ctx_stream(atlasx_ctx* ctx);                 /* cudaStream_t */
int   atlasx_ctx_sm_count(atlasx_ctx* ctx);
/* GEMV kernel choice: 0 = automatic (plain loads), 1 = plain 128-bit loads, 2 = bulk-copy (TMA) ring,
 * 3 = as 1 but multi-column products keep the scalar kernel instead of the tensor-core one (A/B comparison) */
int   atlasx_ctx_set_gemv_impl(atlasx_ctx* ctx, int impl);
/* nonzero when a device-side bounded wait gave up since the last call (clears it) */
int   atlasx_ctx_poll_device_error(atlasx_ctx* ctx, int* code_out);

/* GpuBuf / GpuBufBf16 (crates/atlas-tensor/src/lib.rs:178-280): raw device memory */
int atlasx_malloc(atlasx_ctx* ctx, size_t bytes, void** out_dev);
int atlasx_free(atlasx_ctx* ctx, void* dev);
int atlasx_memset(atlasx_ctx* ctx, void* dev, int value, size_t bytes);
int atlasx_upload(atlasx_ctx* ctx, void* dst_dev, const void* src_host, size_t bytes);     /* GpuBuf::upload   :208 */
int atlasx_download(atlasx_ctx* ctx, void* dst_host, const void* src_dev, size_t bytes);   /* GpuBuf::download :217 */
int atlasx_copy_dev(atlasx_ctx* ctx, void* dst_dev, const void* src_dev, size_t bytes);

/* seeded synthetic data, integer-exact (same bits as a host implementation of the same hash):
 * element i = z(seed, stream, first + i)·std with z ≈ N(0,1) */
int atlasx_fill_normal_f32(atlasx_ctx* ctx, float* dst_dev, size_t n, uint64_t seed, uint64_t stream, uint64_t first, float std);
int atlasx_fill_normal_bf16(atlasx_ctx* ctx, uint16_t* dst_dev, size_t n, uint64_t seed, uint64_t stream, uint64_t first, float std);
int atlasx_convert_bf16_to_f32(atlasx_ctx* ctx, const uint16_t* src_dev, float* dst_dev, size_t n);
int atlasx_convert_f32_to_bf16(atlasx_ctx* ctx, const float* src_dev, uint16_t* dst_dev, size_t n, int truncate);

/* ── atlas-quant formats on the device, bit-exact with
 *    Int8Tensor::quantize (crates/atlas-quant/src/lib.rs:43-63) and
 *    Int4Tensor::quantize (:113-145): round half away from zero, multiply by the
 *    reciprocal scale, scale 1.0 for an all-zero row/block, even index → high nibble ── */
int atlasx_quantize_int8(atlasx_ctx* ctx, const float* src_dev, int rows, int cols, int8_t* data_dev, float* scales_dev);
int atlasx_dequantize_int8(atlasx_ctx* ctx, const int8_t* data_dev, const float* scales_dev, int rows, int cols, float* out_dev); /* :66-75 */
int atlasx_quantize_int4(atlasx_ctx* ctx, const float* src_dev, size_t n, int block_size, uint8_t* data_dev, float* scales_dev);
int atlasx_dequantize_int4(atlasx_ctx* ctx, const uint8_t* data_dev, const float* scales_dev, size_t n, int block_size, float* out_dev); /* :157-168 */

/* ── GpuMatrix (crates/atlas-tensor/src/lib.rs:309-436): a weight [rows=out × cols=in],
 *    row-major, resident in HBM ───────────────────────────────────────────────── */
typedef struct atlasx_matrix atlasx_matrix;
int atlasx_matrix_upload_f32(atlasx_ctx* ctx, const float* host, int rows, int cols, atlasx_matrix** out);      /* GpuMatrix::upload      :319 */
int atlasx_matrix_upload_bf16(atlasx_ctx* ctx, const uint16_t* host, int rows, int cols, atlasx_matrix** out);  /* GpuMatrix::upload_bf16 :336 */
/* exactly the arrays of Int8Tensor {data, scales} */
int atlasx_matrix_upload_int8(atlasx_ctx* ctx, const int8_t* data_host, const float* scales_host, int rows, int cols, atlasx_matrix** out);
/* exactly the arrays of Int4Tensor {data, scales, block_size}; scales_f16 != 0 stores the
 * scales as IEEE half in HBM (bandwidth format; not a reference format) */
int atlasx_matrix_upload_int4(atlasx_ctx* ctx, const uint8_t* data_host, const float* scales_host, int rows, int cols,
                              int block_size, int scales_f16, atlasx_matrix** out);
/* take over existing device arrays (not copied, not freed by atlasx_matrix_free) */
int atlasx_matrix_wrap(atlasx_ctx* ctx, int dtype, const void* data_dev, const void* scales_dev, int rows, int cols,
                       int block_size, int scales_f16, atlasx_matrix** out);
int atlasx_matrix_free(atlasx_matrix* m);
int atlasx_matrix_info(const atlasx_matrix* m, int* rows, int* cols, int* dtype);   /* is_on_gpu / is_bf16 :349-362 */
size_t atlasx_matrix_bytes(const atlasx_matrix* m);     /* weight bytes one product streams from HBM */
/* GpuMatrix::sgemm_vec (:409-435): y[rows×n] = W·x[cols×n], x and y row-major in HBM, f32.
 * n == 1 is the decode GEMV; 2..16 (2..128 for bf16 weights with at least 64 columns, a multiple of 8, and for int4
 * weights whose column count is a multiple of 64 and of the block; 2..64 for int8 weights with at least 128 columns, a
 * multiple of 16) is the skinny batched/verify case. */
int atlasx_gemv(atlasx_ctx* ctx, const atlasx_matrix* m, const float* x_dev, int n, float* y_dev);
/* GpuMatrix::sgemm (:371-400): same with host rhs/out (uploads x, downloads y) */
int atlasx_matrix_sgemm(atlasx_ctx* ctx, const atlasx_matrix* m, const float* rhs_host, int k, int n, float* out_host);

/* ── GpuVec ops used by the decode path (crates/atlas-tensor/src/lib.rs:506-654) ── */
int atlasx_vec_add(atlasx_ctx* ctx, const float* a_dev, const float* b_dev, float* out_dev, int n);            /* add_inplace     :506 */
int atlasx_rmsnorm(atlasx_ctx* ctx, const float* x_dev, const float* w_dev, float* out_dev, int n, float eps); /* rmsnorm_inplace :522 */
int atlasx_silu_mul(atlasx_ctx* ctx, const float* gate_dev, const float* up_dev, float* out_dev, int n);       /* silu_mul_gpu    :590 */
int atlasx_qk_norm_inplace(atlasx_ctx* ctx, float* x_dev, const float* w_dev, int n_heads, int head_dim, float eps); /* :633 */
/* last index among equal maxima, the rule of the CPU argmax that generate() uses
 * (crates/atlas-model/src/lib.rs:2701-2706) */
int atlasx_argmax(atlasx_ctx* ctx, const float* x_dev, int n, int* out_index_host);

/* ── GpuRopeTables (crates/atlas-tensor/src/lib.rs:662-693) ────────────────────── */
/* RopeCache::new (crates/atlas-model/src/lib.rs:380-423) on the host: cos/sin [max_seq × hd/2].
 * rope_scaling 0 = none, 1 = YaRN. */
int atlasx_rope_tables_host(int head_dim, int max_seq, float theta, int rope_scaling, float factor,
                            int orig_max_pos, float beta_fast, float beta_slow, float* cos_host, float* sin_host);
int atlasx_rope_apply(atlasx_ctx* ctx, float* x_dev, const float* cos_dev, const float* sin_dev,
                      int n_heads, int head_dim, int pos, int max_seq);                                   /* apply_to :681 */

/* ── GpuKvCache (crates/atlas-tensor/src/lib.rs:701-785) with a batch dimension and a
 *    choice of element type: [batch][max_seq × n_kv × hd], bf16 (rounded to nearest even
 *    on write) or f32 (the reference's format) ─────────────────────────────────── */
typedef struct atlasx_kvcache atlasx_kvcache;
int atlasx_kvcache_create(atlasx_ctx* ctx, int max_seq, int n_kv_heads, int head_dim, int dtype, int batch, atlasx_kvcache** out); /* new :713 */
int atlasx_kvcache_free(atlasx_kvcache* kv);
int atlasx_kvcache_ptrs(atlasx_kvcache* kv, void** k_dev, void** v_dev, size_t* bytes_each);
/* write k,v [batch × n_kv × hd] f32 at pos[b] (host array of batch ints)             write :722 */
int atlasx_kvcache_write(atlasx_ctx* ctx, atlasx_kvcache* kv, const float* k_dev, const float* v_dev, const int* pos_host);
/* q,out [batch × n_heads × hd] f32; attends t ∈ [0,pos[b]] (window>0: pos−t < window).
 * Split over the sequence; partial results live in context scratch.      decode_attention :743 */
int atlasx_decode_attention(atlasx_ctx* ctx, const atlasx_kvcache* kv, const float* q_dev, float* out_dev,
                            int n_heads, const int* pos_host, float scale, int window);
/* algorithmic HBM bytes of one such call (K and V rows read + q + out) */
size_t atlasx_decode_attention_bytes(const atlasx_kvcache* kv, int n_heads, const int* pos_host, int window);
/* Same attention for callers that must not allocate (no counterpart in the reference, whose
 * wrappers never allocate but also never split the sequence).  It takes no context and no cache
 * object: the caller passes its own stream (cudaStream_t, may be 0) and raw cache pointers
 * laid out [batch][max_seq × n_kv × hd].  Split partials, tickets and the device copy of pos
 * live in a fixed 4.5 MiB device array inside the library, so no cudaMalloc / cudaFree (or
 * any allocating routine) runs.  Limits, rejected with ATLASX_ERR_ARG: batch ≤ 4096 and
 * batch × n_heads ≤ 4096; the split count is lowered to fit 1 Mi floats of partials.
 * The first call on a device looks up the array's device address (make that call before any
 * stream capture).  All calls share the array: two calls whose kernels overlap on the GPU
 * (different streams, or different host threads) race; serialise them on one stream. */
int atlasx_decode_attention_static(void* stream, int kv_dtype, const void* k_dev, const void* v_dev,
                                   int max_seq, int n_kv_heads, int head_dim, int batch,
                                   const float* q_dev, float* out_dev, int n_heads,
                                   const int* pos_host, float scale, int window);

/* ── SamplingConfig and the sampling pipeline (crates/atlas-model/src/lib.rs:1223-1294, 2581-2717) ── */
typedef struct {
    float temperature;          /* <= 0 (or < 1e-6): greedy                      */
    float repetition_penalty;   /* 1.0 = off                                     */
    int   repetition_window;
    float frequency_penalty;    /* 0.0 = off                                     */
    float presence_penalty;     /* 0.0 = off                                     */
    float top_p;                /* 1.0 = off                                     */
    int   top_k;                /* 0 = off                                       */
    float min_p;                /* 0.0 = off                                     */
} atlasx_sampling_config;
/* One selection of generate_with_sampling's sampling branch (:1650-1710) from `n` logits on the device:
 * first-token suppression (step == 0), repetition / frequency / presence penalties over `history` (the
 * tokens generated so far; the last repetition_window of them for the repetition penalty), temperature,
 * top-k, top-p, min-p, softmax, and one draw of the XorShift64 generator whose state *rng_state holds
 * (Rng :1190-1216; advanced by the call).  Only the token comes back; probs_dev_out (optional, n floats
 * on the device) receives the final distribution.  The RNG stream, the top-k set and all tie rules are
 * bit-exact with the reference; probabilities agree to the last bits of expf.  Equal probabilities in
 * top-p — ordered by an unstable sort in the reference, so unspecified there — keep index order. */
int atlasx_sample_token(atlasx_ctx* ctx, const float* logits_dev, int n, const atlasx_sampling_config* cfg, int step,
                        const uint32_t* suppress_host, int n_suppress, const uint32_t* history_host, int n_hist,
                        uint64_t* rng_state, int* token_out, float* probs_dev_out);

/* ── OlmoModel (crates/atlas-model/src/lib.rs:1298-1732) ───────────────────────── */
typedef struct {
    int   vocab_size, d_model, n_layers, n_heads, n_kv_heads, ffn_hidden, max_seq_len;
    float rope_theta, rms_norm_eps;
    int   sliding_window;          /* 0 = none */
    int   rope_scaling;            /* 0 none, 1 YaRN */
    float yarn_factor; int yarn_orig_max_pos;
    float yarn_attn_factor, yarn_beta_fast, yarn_beta_slow;
    int   post_norm;               /* 1 = OLMo-2/3 post-norm, 0 = Llama pre-norm */
    int   eos_token_id;            /* -1 = none */
    int   kv_dtype;                /* ATLASX_BF16 or ATLASX_F32 */
    int   weight_format;           /* storage of the linear weights: F32, BF16, INT8 or INT4 (quantised on load) */
    int   int4_block;              /* block size when weight_format == INT4 (32 or 64) */
    int   tp_rank, tp_world;       /* tensor-parallel position of this process (0,1 = single GPU) */
} atlasx_model_config;

/* tensor ids for atlasx_model_set_tensor (names as loaded at crates/atlas-model/src/lib.rs:2328-2346) */
enum {
    ATLASX_T_EMBED = 0, ATLASX_T_FINAL_NORM = 1, ATLASX_T_LM_HEAD = 2,
    ATLASX_T_WQ = 10, ATLASX_T_WK, ATLASX_T_WV, ATLASX_T_WO, ATLASX_T_GATE, ATLASX_T_UP, ATLASX_T_DOWN,
    ATLASX_T_ATTN_NORM, ATLASX_T_FFN_NORM, ATLASX_T_Q_NORM, ATLASX_T_K_NORM
};

typedef struct atlasx_model atlasx_model;
/* layer_sliding: n_layers ints (1 = sliding-window layer) or NULL */
int atlasx_model_create(atlasx_ctx* ctx, const atlasx_model_config* cfg, const int* layer_sliding, atlasx_model** out);
int atlasx_model_free(atlasx_model* m);
/* Give the FULL (unsharded) tensor, f32 or bf16 bits, from host (on_device 0) or device
 * memory (1); the model keeps its tensor-parallel slice in its own layout. */
int atlasx_model_set_tensor(atlasx_model* m, int layer, int which, const void* data, int dtype, int on_device);
/* Tensor-parallel loading without the detour through the full tensor: atlasx_model_tensor_slice
 * names the rows [r0,r1) × columns [c0,c1) of the full [full_rows × full_cols] tensor `which` that
 * this rank keeps; atlasx_model_set_tensor_slice takes exactly that part (row-major).  whole = 1
 * means the rank needs the full tensor (replicated tensors; int8 weights split by columns, whose
 * per-row scale is defined over the full row): hand it to atlasx_model_set_tensor.  With one rank
 * every tensor is whole. */
int atlasx_model_tensor_slice(const atlasx_model* m, int which, size_t* full_rows, size_t* full_cols,
                              size_t* r0, size_t* r1, size_t* c0, size_t* c1, int* whole);
int atlasx_model_set_tensor_slice(atlasx_model* m, int layer, int which, const void* data, int dtype, int on_device);
/* init_gpu_resources (:1360-1386): RoPE tables, KV caches, step graph.  Call once after the tensors. */
int atlasx_model_finalize(atlasx_model* m);
int atlasx_model_reset(atlasx_model* m);                                            /* reset :1389 */
int atlasx_model_pos(const atlasx_model* m);
/* forward_one_gpu (:1463-1505): logits_host may be NULL (no download).  Tensor parallel: every rank of the
 * group must make the same choice — with NULL the ranks exchange only their local maxima, otherwise they
 * all-gather the logits. */
int atlasx_model_forward_one(atlasx_model* m, uint32_t token, float* logits_host);
/* generate_with_sampling, greedy branch (:1599-1646,1713-1730): EOS/stop tokens end the
 * run before being emitted; suppress applies to the first generated token only;
 * rep_penalty 1.0 = off.  out_tokens holds max_new entries. */
int atlasx_model_generate_greedy(atlasx_model* m, const uint32_t* prompt, int n_prompt, int max_new,
                                 const uint32_t* suppress, int n_suppress, float rep_penalty, int rep_window,
                                 const uint32_t* stops, int n_stops, uint32_t* out_tokens, int* n_out);
/* generate_with_sampling, sampling branch (:1599-1732): as atlasx_model_generate_greedy, with the next token
 * picked on the device by the pipeline of atlasx_sample_token — only the 4-byte token id crosses to the
 * host per step.  The generator is seeded as Rng::from_seed(seed) (seed | 1), or from the clock as
 * Rng::from_entropy does when seed_from_time != 0 (the reference's behaviour for every call).
 * temperature <= 0 runs the greedy call (repetition penalty and suppression still apply, :1625-1646). */
int atlasx_model_generate_sampling(atlasx_model* m, const uint32_t* prompt, int n_prompt, int max_new,
                                   const atlasx_sampling_config* cfg, const uint32_t* suppress, int n_suppress,
                                   const uint32_t* stops, int n_stops, uint64_t seed, int seed_from_time,
                                   uint32_t* out_tokens, int* n_out);
/* device-resident decode for timing: runs `lead` + `steps` greedy steps from the current state
 * with no host round trip per token; returns the device time of the last `steps` of them (CUDA
 * events; the lead-in steps line the ranks of a tensor-parallel group up before the first
 * event).  tokens_host receives lead + steps tokens. */
int atlasx_model_decode_timed(atlasx_model* m, int steps, int lead, float* elapsed_ms, uint32_t* tokens_host);
/* one step outside the graph with an event pair around every kernel: per kernel class
 * (see atlasx_model_class_name) launches, milliseconds and algorithmic HBM bytes */
int atlasx_model_profile_step(atlasx_model* m, int n_classes_max, int* launches, float* ms, double* bytes, int* n_classes);
/* Device time of the launches of the classes in `mask` (bit = class index as in
 * atlasx_model_profile_step) in step order, inside one CUDA graph with the step's programmatic
 * dependent launch attributes, replayed `iters` times between two CUDA events: the family's time
 * under the launch conditions of the decode loop, without the other families.  Single GPU. */
int atlasx_model_time_classes(atlasx_model* m, unsigned mask, int iters, float* ms_per_pass, double* bytes_per_pass, int* launches);
const char* atlasx_model_class_name(int cls);
/* algorithmic HBM bytes of one decode step at position pos (weights + KV read/write) */
double atlasx_model_step_bytes(const atlasx_model* m, int pos);
int atlasx_model_kernel_launches_per_step(const atlasx_model* m);
int atlasx_model_set_options(atlasx_model* m, int use_graph, int use_pdl);
/* Prompt ingestion in chunks: atlasx_model_generate_greedy feeds the prompt `chunk` tokens at a
 * time (2..128 with bf16 and int4 weights, at most 64 with int8 weights) through the multi-column kernels, so the weights stream once per chunk instead of
 * once per token (the reference feeds one token per forward, crates/atlas-model/src/lib.rs:1611-1618).
 * 0 or 1 restores token-by-token ingestion (the default).  *effective receives the chunk in use:
 * 1 when a weight format or shape is outside what the multi-column kernel covers (f32 weights,
 * K not a multiple of 32, or of 64 for int8).  Call after atlasx_model_finalize. */
int atlasx_model_set_prefill(atlasx_model* m, int chunk, int* effective);
/* residual stream after the last forward (d_model floats), for layer-level parity checks */
int atlasx_model_hidden(atlasx_model* m, float* hidden_host);
/* the same after layer `layer` of the last forward (every layer's output survives the step) */
int atlasx_model_layer_hidden(atlasx_model* m, int layer, float* hidden_host);
/* StigmergicHook on the GPU path (crates/atlas-infer/src/hook.rs:31-33: on_layer(layer_idx, hidden) -> Option<f32>).
 * The reference runs hooked generation on its CPU model (crates/atlas-infer/src/engine.rs:144-162); here the
 * layer outputs of a forward are copied to pinned host memory behind the step (n_layers × d_model floats) and
 * the hook runs on the host while the next forward executes.  The hook returns nonzero for Some(delta) and
 * stores the delta.  With a hook attached atlasx_model_forward_one calls it for every layer before returning
 * (forward_one_gpu_hooked, crates/atlas-model/src/lib.rs:1524-1557); atlasx_model_generate_greedy / _sampling call
 * it for every layer of every forward, prompt included, and collect one deposit per generated token
 * (generate_with_sampling_hooked, :1745-1846: negative deltas count as zero), read with atlasx_model_deposits
 * after the call.  Prompt tokens are then ingested one by one.  fn = NULL detaches the hook. */
typedef int (*atlasx_layer_hook)(void* user, int layer, const float* hidden_host, int d_model, float* delta_out);
/* generate_streaming (crates/atlas-model/src/lib.rs:1855-1965, crates/atlas-infer/src/engine.rs:171-190): with a callback set,
 * atlasx_model_generate_greedy / _sampling call it with every token right after it is emitted (EOS and stop tokens end
 * the run before and are not seen); a zero return ends the generation there, without a forward for that token.
 * fn = NULL detaches it. */
typedef int (*atlasx_token_callback)(void* user, uint32_t token);
int atlasx_model_set_token_callback(atlasx_model* m, atlasx_token_callback fn, void* user);
int atlasx_model_set_layer_hook(atlasx_model* m, atlasx_layer_hook fn, void* user);
/* deposits of the last generate call: per generated token its id, the sum of the deltas and the number of
 * layers that returned one; *n receives the count (all of them, even if cap is smaller) */
int atlasx_model_deposits(atlasx_model* m, uint32_t* token_ids, float* total_delta, uint32_t* layers_fired, int cap, int* n);

/* ── safetensors (crates/atlas-model/src/lib.rs: SafetensorsFile :2046-2240, loaders :2283-2570) ──
 * A file is mapped, not read: opening costs the header only. */
typedef struct atlasx_safetensors atlasx_safetensors;
int atlasx_safetensors_open(const char* path, atlasx_safetensors** out);            /* open / from_bytes :2071-2125 */
int atlasx_safetensors_close(atlasx_safetensors* st);
int atlasx_safetensors_count(const atlasx_safetensors* st);                         /* len :2133 */
int atlasx_safetensors_find(const atlasx_safetensors* st, const char* name);        /* index or -1; contains / get_desc :2143-2150 */
/* descriptor of tensor `index` (header order): name, dtype (ATLASX_F32 / _BF16 / _F16, -1 = a dtype the
 * path cannot read), number of dimensions, the first four extents (1-padded), bytes in the file */
int atlasx_safetensors_tensor(const atlasx_safetensors* st, int index, const char** name, int* dtype,
                              int* n_dims, size_t* dims4, size_t* nbytes);
/* rows [r0,r1) × columns [c0,c1) of the tensor seen as [product of leading extents × last extent], into host
 * memory as f32 (get_f32 :2205-2240: F32 as is, BF16 as the upper half of an f32, F16 converted) or as raw
 * bf16 bits (get_bf16 :2187-2202, BF16 tensors only) */
int atlasx_safetensors_read(const atlasx_safetensors* st, int index, size_t r0, size_t r1, size_t c0, size_t c1,
                            int out_dtype, void* dst_host);
/* the synthetic writer of the reference's tests (build_f32 :2154-2185; same header text), F32 and BF16 tensors;
 * dims4 holds four extents per tensor */
int atlasx_safetensors_write(const char* path, int n, const char* const* names, const int* dtypes,
                             const int* n_dims, const size_t* dims4, const void* const* data_host);

typedef struct {
    double seconds;               /* open → model finalised */
    size_t file_bytes_read;       /* bytes of the files this rank touched */
    size_t bytes_uploaded;        /* host → device */
    size_t peak_host_rss_bytes;   /* getrusage maximum resident set of the process */
    int    n_tensors_used;
    int    post_norm;             /* detected from the tensor names (:2508-2515) */
    int    tied_lm_head;          /* no lm_head.weight in the files: lm_head = embedding (:2493-2497) */
    int    weight_format;         /* the format in effect (ATLASX_AUTO resolved) */
} atlasx_load_stats;
/* load_model_from_safetensors (:2283-2360) over one or several files: creates the model, places every
 * known tensor (names :2300-2346; unknown ones ignored; post-norm and a separate lm_head detected from the
 * names first), finalises it.  BF16 tensors go to the device as stored, F32 as stored, F16 as f32; each
 * tensor-parallel rank reads only its part; cfg->weight_format INT8 / INT4 quantises on the device while
 * loading, ATLASX_AUTO follows the file.  cfg->post_norm is overridden by the detection.  stats may be NULL. */
int atlasx_model_load_safetensors(atlasx_ctx* ctx, const char* const* paths, int n_paths, const atlasx_model_config* cfg,
                                  const int* layer_sliding, atlasx_model** out, atlasx_load_stats* stats);
/* patch_config_from_hf_json (:2367-2432): layer_types, sliding_window, rope_scaling (yarn), rope_theta,
 * rms_norm_eps, eos_token_id — only fields present in the file change; max_seq_len never.
 * sliding_out (n_layers ints, may be NULL) is filled and *have_layer_types set to the array length when the
 * file has layer_types. */
int atlasx_config_patch_from_json(const char* config_json_path, atlasx_model_config* cfg, int* sliding_out, int* have_layer_types);
/* load_model_from_dir (:2437-2570): config.json overlay when present, the shards named in
 * model.safetensors.index.json (sorted), else model.safetensors */
int atlasx_model_load_dir(atlasx_ctx* ctx, const char* dir, const atlasx_model_config* cfg, const int* layer_sliding,
                          atlasx_model** out, atlasx_load_stats* stats);

/* ── measurement helpers: `iters` launches back to back between two CUDA events on the context
 *    stream; elapsed device time in milliseconds.  GEMV launches rotate over n_mats matrices so
 *    that the weights come from HBM, not from L2. ─────────────────────────────────────────── */
int atlasx_time_gemv(atlasx_ctx* ctx, const atlasx_matrix* const* mats, int n_mats, const float* x_dev, int n,
                     float* y_dev, int iters, float* ms_out);
int atlasx_time_attention(atlasx_ctx* ctx, const atlasx_kvcache* kv, const float* q_dev, float* out_dev, int n_heads,
                          const int* pos_host, float scale, int window, int iters, float* ms_out);

/* ── tensor parallel plumbing (no counterpart in the reference, which is single-GPU) ── */
/* 128-byte NCCL unique id: rank 0 creates it, every rank passes it to atlasx_comm_init */
int atlasx_comm_unique_id(void* id128_out);
int atlasx_comm_init(atlasx_ctx* ctx, const void* id128, int rank, int world);
int atlasx_comm_world(const atlasx_ctx* ctx);
/* Diagnostics: launches a mailbox reduction whose data never arrives and reports the device error
 * word after the kernel gave up (code 3 after its 2 s limit).  Shows that an absent peer ends in
 * an error status, not in a hang; the context stays usable.  keep = 0 clears the word again;
 * keep != 0 leaves it set, as a real expiry does: atlasx_model_forward_one / _generate_greedy /
 * _decode_timed then fail with ATLASX_ERR_TIMEOUT until atlasx_ctx_poll_device_error clears it.
 * No reference counterpart. */
int atlasx_comm_selftest_wait_expiry(atlasx_ctx* ctx, int* code, int keep);
/* sum-allreduce of n floats in place on the context stream */
int atlasx_comm_allreduce(atlasx_ctx* ctx, float* buf_dev, int n);

#ifdef __cplusplus
}
#endif
#endif /* ATLAS_KERNELS_H */
