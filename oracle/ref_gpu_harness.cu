/*
 * ref_gpu_harness.cu — drives the reference's OWN CUDA kernels (kernels/matmul.cu,
 * compiled unchanged from the reference checkout and linked into the same shared
 * object) through the call sequence of the reference's GPU decode path.
 *
 * TEST INFRASTRUCTURE ONLY: it is the GPU-side checker for whole-model parity
 * and the kernel-level baseline the benchmark reports beside the new kernels.
 *
 * Sequence restated from web3guru888/ATLAS:
 *   OlmoModel::forward_one_gpu            crates/atlas-model/src/lib.rs:1463-1505
 *   TransformerBlock::forward_token_gpu_v2 :1015-1091 (post-norm and pre-norm branches)
 *   Attention::forward_token_gpu_full      :837-870   (QK-norm eps is the literal 1e-6)
 *   FeedForward::forward_gpu               :902-908
 * Each reference op allocates a fresh output buffer; here the buffers are
 * preallocated, which does not change any arithmetic.
 */
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <math.h>

extern "C" {
/* prototypes of the reference's C ABI, crates/atlas-tensor/src/lib.rs:20-91 */
void atlas_matmul_f32(const float*, const float*, float*, int, int, int);
void atlas_sgemm_bf16_f32(const uint16_t*, const float*, float*, int, int, int);
void atlas_vec_add_f32(const float*, const float*, float*, int);
void atlas_rmsnorm_f32(const float*, const float*, float*, int, float);
void atlas_silu_mul_f32(const float*, const float*, float*, int);
void atlas_qk_norm_inplace(float*, const float*, int, int, float);
void atlas_rope_precomputed(float*, const float*, const float*, int, int, int, int);
void atlas_kv_cache_write(float*, float*, const float*, const float*, int, int, int);
void atlas_decode_attention(const float*, const float*, const float*, float*, int, int, int, int, float, int);
}

struct ref_w { const void* p; int dtype; };
struct ref_layer {
    ref_w wq, wk, wv, wo, gate, up, down;
    const float *attn_norm, *ffn_norm, *q_norm, *k_norm;
    float *kc, *vc;
    int window;
};
struct ref_model {
    int vocab, d, n_layers, n_heads, n_kv, ffn, max_seq, hd, post_norm;
    float eps, scale;
    ref_w embed, lm_head;
    const float* final_norm;
    ref_layer* layers;
    float *cos_t, *sin_t;
    float *x, *x2, *q, *k, *v, *attn, *o, *normed, *gate, *up, *h, *logits;
    int pos;
};

static __global__ void embed_row_kernel(const void* table, int dtype, size_t row, int d, float* x) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= d) return;
    if (dtype) x[i] = __uint_as_float(((uint32_t)((const uint16_t*)table)[row * d + i]) << 16);
    else       x[i] = ((const float*)table)[row * d + i];
}

static float* dalloc(size_t n) { float* p = nullptr; cudaMalloc((void**)&p, n * sizeof(float)); return p; }

extern "C" {

ref_model* refgpu_model_new(int vocab, int d, int n_layers, int n_heads, int n_kv, int ffn,
                            int max_seq, float eps, float scale, int post_norm,
                            const int* layer_window /* n_layers, 0 = full */) {
    ref_model* m = (ref_model*)calloc(1, sizeof(ref_model));
    m->vocab = vocab; m->d = d; m->n_layers = n_layers; m->n_heads = n_heads; m->n_kv = n_kv;
    m->ffn = ffn; m->max_seq = max_seq; m->hd = d / n_heads; m->post_norm = post_norm;
    m->eps = eps; m->scale = scale;
    m->layers = (ref_layer*)calloc((size_t)n_layers, sizeof(ref_layer));
    size_t cap = (size_t)max_seq * n_kv * m->hd;
    for (int l = 0; l < n_layers; l++) {
        m->layers[l].kc = dalloc(cap); m->layers[l].vc = dalloc(cap);
        cudaMemset(m->layers[l].kc, 0, cap * 4); cudaMemset(m->layers[l].vc, 0, cap * 4);
        m->layers[l].window = layer_window ? layer_window[l] : 0;
    }
    size_t kvd = (size_t)n_kv * m->hd;
    m->x = dalloc(d); m->x2 = dalloc(d); m->q = dalloc(d); m->k = dalloc(kvd); m->v = dalloc(kvd);
    m->attn = dalloc(d); m->o = dalloc(d); m->normed = dalloc(d);
    m->gate = dalloc(ffn); m->up = dalloc(ffn); m->h = dalloc(ffn); m->logits = dalloc(vocab);
    return m;
}

void refgpu_model_free(ref_model* m) {
    if (!m) return;
    for (int l = 0; l < m->n_layers; l++) { cudaFree(m->layers[l].kc); cudaFree(m->layers[l].vc); }
    float* bufs[] = { m->x, m->x2, m->q, m->k, m->v, m->attn, m->o, m->normed, m->gate, m->up, m->h, m->logits, m->cos_t, m->sin_t };
    for (size_t i = 0; i < sizeof(bufs) / sizeof(bufs[0]); i++) if (bufs[i]) cudaFree(bufs[i]);
    free(m->layers); free(m);
}

/* device pointers are borrowed; `which` uses the numbering of atlas_oracle.h */
int refgpu_set_tensor(ref_model* m, int layer, int which, const void* dev, int dtype) {
    ref_w w = { dev, dtype };
    if (which == 0) { m->embed = w; return 0; }
    if (which == 1) { m->final_norm = (const float*)dev; return 0; }
    if (which == 2) { m->lm_head = w; return 0; }
    if (layer < 0 || layer >= m->n_layers) return -1;
    ref_layer* L = &m->layers[layer];
    switch (which) {
        case 10: L->wq = w; break; case 11: L->wk = w; break; case 12: L->wv = w; break;
        case 13: L->wo = w; break; case 14: L->gate = w; break; case 15: L->up = w; break;
        case 16: L->down = w; break;
        case 17: L->attn_norm = (const float*)dev; break; case 18: L->ffn_norm = (const float*)dev; break;
        case 19: L->q_norm = (const float*)dev; break;    case 20: L->k_norm = (const float*)dev; break;
        default: return -1;
    }
    return 0;
}

/* GpuRopeTables::upload, crates/atlas-tensor/src/lib.rs:673-678 (host tables, max_seq × hd/2) */
void refgpu_upload_rope(ref_model* m, const float* cos_h, const float* sin_h) {
    size_t n = (size_t)m->max_seq * (m->hd / 2);
    m->cos_t = dalloc(n); m->sin_t = dalloc(n);
    cudaMemcpy(m->cos_t, cos_h, n * 4, cudaMemcpyHostToDevice);
    cudaMemcpy(m->sin_t, sin_h, n * 4, cudaMemcpyHostToDevice);
}

void refgpu_reset(ref_model* m) { m->pos = 0; }
/* measurement aid: continue at position `pos` as if a prompt of that length had been processed (the cache
 * rows below keep whatever they hold — zeros after creation —, which costs the kernels the same traffic) */
void refgpu_set_pos(ref_model* m, int pos) { m->pos = pos < 0 ? 0 : (pos >= m->max_seq ? m->max_seq - 1 : pos); }

static void gemv(ref_w w, const float* x, float* y, int out_dim, int in_dim) {
    if (w.dtype) atlas_sgemm_bf16_f32((const uint16_t*)w.p, x, y, out_dim, 1, in_dim);
    else         atlas_matmul_f32((const float*)w.p, x, y, out_dim, 1, in_dim);
}

static void attention_full(ref_model* m, ref_layer* L, const float* x, int pos, float* out) {
    int kvd = m->n_kv * m->hd;
    gemv(L->wq, x, m->q, m->d, m->d);
    gemv(L->wk, x, m->k, kvd, m->d);
    gemv(L->wv, x, m->v, kvd, m->d);
    if (L->q_norm) atlas_qk_norm_inplace(m->q, L->q_norm, m->n_heads, m->hd, 1e-6f);
    if (L->k_norm) atlas_qk_norm_inplace(m->k, L->k_norm, m->n_kv, m->hd, 1e-6f);
    atlas_rope_precomputed(m->q, m->cos_t, m->sin_t, m->n_heads, m->hd, pos, m->max_seq);
    atlas_rope_precomputed(m->k, m->cos_t, m->sin_t, m->n_kv, m->hd, pos, m->max_seq);
    atlas_kv_cache_write(L->kc, L->vc, m->k, m->v, pos, m->n_kv, m->hd);
    atlas_decode_attention(m->q, L->kc, L->vc, m->attn, m->n_heads, m->n_kv, m->hd, pos, m->scale, L->window);
    gemv(L->wo, m->attn, out, m->d, m->d);
}

static void ffn_gpu(ref_model* m, ref_layer* L, const float* x, float* out) {
    gemv(L->gate, x, m->gate, m->ffn, m->d);
    gemv(L->up, x, m->up, m->ffn, m->d);
    atlas_silu_mul_f32(m->gate, m->up, m->h, m->ffn);
    gemv(L->down, m->h, out, m->d, m->ffn);
}

/* returns 0, or the CUDA error code seen after the token's launches */
int refgpu_forward_one(ref_model* m, uint32_t token, float* logits_host) {
    int pos = m->pos; m->pos += 1;
    size_t id = token; if (id > (size_t)m->vocab - 1) id = (size_t)m->vocab - 1;
    embed_row_kernel<<<(m->d + 255) / 256, 256>>>(m->embed.p, m->embed.dtype, id, m->d, m->x);
    float* x = m->x; float* xn = m->x2;
    for (int l = 0; l < m->n_layers; l++) {
        ref_layer* L = &m->layers[l];
        if (m->post_norm) {
            attention_full(m, L, x, pos, m->o);
            atlas_rmsnorm_f32(m->o, L->attn_norm, m->normed, m->d, m->eps);
            atlas_vec_add_f32(x, m->normed, xn, m->d);
            { float* t = x; x = xn; xn = t; }
            ffn_gpu(m, L, x, m->o);
            atlas_rmsnorm_f32(m->o, L->ffn_norm, m->normed, m->d, m->eps);
            atlas_vec_add_f32(x, m->normed, xn, m->d);
            { float* t = x; x = xn; xn = t; }
        } else {
            atlas_rmsnorm_f32(x, L->attn_norm, m->normed, m->d, m->eps);
            attention_full(m, L, m->normed, pos, m->o);
            atlas_vec_add_f32(x, m->o, xn, m->d);
            { float* t = x; x = xn; xn = t; }
            atlas_rmsnorm_f32(x, L->ffn_norm, m->normed, m->d, m->eps);
            ffn_gpu(m, L, m->normed, m->o);
            atlas_vec_add_f32(x, m->o, xn, m->d);
            { float* t = x; x = xn; xn = t; }
        }
    }
    m->x = x; m->x2 = xn;
    atlas_rmsnorm_f32(x, m->final_norm, m->normed, m->d, m->eps);
    gemv(m->lm_head, m->normed, m->logits, m->vocab, m->d);
    if (logits_host) cudaMemcpy(logits_host, m->logits, (size_t)m->vocab * 4, cudaMemcpyDeviceToHost);
    cudaError_t e = cudaGetLastError();
    return (int)e;
}

/* device pointer to the last logits (valid after a forward; no sync implied) */
const float* refgpu_logits_dev(ref_model* m) { return m->logits; }

} /* extern "C" */
