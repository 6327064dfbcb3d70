/*
 * atlas_oracle.c — CPU restatement of ATLAS's single-token decode path.
 * TEST INFRASTRUCTURE ONLY (see atlas_oracle.h).  Build: see Makefile
 * (-O2 -ffp-contract=off, no -ffast-math: the reference is plain scalar Rust).
 */
#include "atlas_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* ── threads ───────────────────────────────────────────────────────────────── */
static int g_threads = 1;
void orc_set_threads(int n) {
    g_threads = n < 1 ? 1 : n;
#ifdef _OPENMP
    omp_set_num_threads(g_threads);
#endif
}
int orc_get_threads(void) { return g_threads; }

/* ── seeded synthetic data ─────────────────────────────────────────────────────
 * Counter-based and integer-exact so that host and device produce the same bits.
 *   base = mix64(seed ^ mix64(stream));  h1 = mix64(base + 2i);  h2 = mix64(base + 2i + 1)
 *   s    = sum of the 8 bytes of h1 and the low 4 bytes of h2   (Irwin–Hall, 12 terms:
 *          mean 1530, variance 65535 ≈ 256²)
 *   u    = bits 32..47 of h2 (16-bit dither that removes the 1/256 grid)
 *   z    = ((s − 1530)·65536 + u − 32768) / 2²⁴            ≈ N(0,1), |z| < 6
 * The only float operations are one int→float conversion and one multiply by a
 * power of two, then one multiply by std. */
uint64_t orc_mix64(uint64_t z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
static inline uint32_t bytesum64(uint64_t v) {
    v = (v & 0x00FF00FF00FF00FFull) + ((v >> 8) & 0x00FF00FF00FF00FFull);
    v = (v & 0x0000FFFF0000FFFFull) + ((v >> 16) & 0x0000FFFF0000FFFFull);
    return (uint32_t)(v & 0xFFFFFFFFull) + (uint32_t)(v >> 32);
}
static inline uint64_t stream_base(uint64_t seed, uint64_t stream) {
    return orc_mix64(seed ^ orc_mix64(stream));
}
static inline float normal_from_base(uint64_t base, uint64_t i) {
    uint64_t h1 = orc_mix64(base + 2 * i);
    uint64_t h2 = orc_mix64(base + 2 * i + 1);
    int32_t s = (int32_t)(bytesum64(h1) + bytesum64(h2 & 0xFFFFFFFFull));
    int32_t u = (int32_t)((h2 >> 32) & 0xFFFF);
    int32_t zi = (s - 1530) * 65536 + (u - 32768);
    return (float)zi * (1.0f / 16777216.0f);
}
float orc_synth_normal(uint64_t seed, uint64_t stream, uint64_t i) {
    return normal_from_base(stream_base(seed, stream), i);
}
void orc_fill_normal_f32(float* dst, size_t n, uint64_t seed, uint64_t stream, float std) {
    uint64_t base = stream_base(seed, stream);
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; i++) dst[i] = normal_from_base(base, i) * std;
}
uint16_t orc_f32_to_bf16_rne(float f) {
    uint32_t u; memcpy(&u, &f, 4);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((u >> 16) | 0x40); /* NaN */
    u += 0x7FFFu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}
uint16_t orc_f32_to_bf16_trunc(float f) { uint32_t u; memcpy(&u, &f, 4); return (uint16_t)(u >> 16); }
float orc_bf16_to_f32(uint16_t h) { uint32_t u = (uint32_t)h << 16; float f; memcpy(&f, &u, 4); return f; }
void orc_fill_normal_bf16(uint16_t* dst, size_t n, uint64_t seed, uint64_t stream, float std) {
    uint64_t base = stream_base(seed, stream);
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; i++) dst[i] = orc_f32_to_bf16_rne(normal_from_base(base, i) * std);
}
void orc_fill_uniform_u32(uint32_t* dst, size_t n, uint64_t seed, uint64_t stream, uint32_t modulo) {
    uint64_t base = stream_base(seed, stream);
    for (size_t i = 0; i < n; i++) dst[i] = (uint32_t)(orc_mix64(base + i) % modulo);
}

/* atlas-model/src/lib.rs:2725-2732 — LCG uniform in [-1,1) */
void orc_pseudo_randn(float* dst, size_t n, uint64_t seed) {
    uint64_t state = seed + 12345ull;
    for (size_t i = 0; i < n; i++) {
        state = state * 6364136223846793005ull + 1442695040888963407ull;
        float u = (float)(state >> 33) / (float)(1ull << 31);
        dst[i] = u * 2.0f - 1.0f;
    }
}

/* ── atlas-quant ───────────────────────────────────────────────────────────── */
static inline int8_t sat_i8(float r) { /* Rust `as i8`: saturating, NaN → 0 */
    if (r != r) return 0;
    if (r >= 127.0f) return 127;
    if (r <= -128.0f) return -128;
    return (int8_t)r;
}
static inline float clampf(float v, float lo, float hi) { /* f32::clamp */
    if (v < lo) return lo;
    if (v > hi) return hi;
    return v;
}

/* atlas-quant/src/lib.rs:52-61 */
void orc_int8_quantize(const float* src, size_t rows, size_t cols, int8_t* data, float* scales) {
#pragma omp parallel for schedule(static)
    for (size_t r = 0; r < rows; r++) {
        const float* row = src + r * cols;
        float mx = 0.0f;
        for (size_t j = 0; j < cols; j++) mx = fmaxf(mx, fabsf(row[j]));
        float s = mx > 0.0f ? mx / 127.0f : 1.0f;
        scales[r] = s;
        float inv = 1.0f / s;
        for (size_t j = 0; j < cols; j++)
            data[r * cols + j] = sat_i8(roundf(clampf(row[j] * inv, -127.0f, 127.0f)));
    }
}
/* atlas-quant/src/lib.rs:66-75 */
void orc_int8_dequantize(const int8_t* data, const float* scales, size_t rows, size_t cols, float* out) {
    for (size_t r = 0; r < rows; r++) {
        float s = scales[r];
        for (size_t j = 0; j < cols; j++) out[r * cols + j] = (float)data[r * cols + j] * s;
    }
}
/* atlas-quant/src/lib.rs:118-144.  Blocks run over the flat row-major index. */
void orc_int4_quantize(const float* src, size_t n, size_t block, uint8_t* data, float* scales) {
    size_t n_blocks = (n + block - 1) / block;
    /* parallel over blocks is safe when block is even (no byte shared by two blocks) */
#pragma omp parallel for schedule(static) if ((block & 1) == 0)
    for (size_t b = 0; b < n_blocks; b++) {
        size_t start = b * block;
        size_t end = start + block < n ? start + block : n;
        float mx = 0.0f;
        for (size_t i = start; i < end; i++) mx = fmaxf(mx, fabsf(src[i]));
        float s = mx > 0.0f ? mx / 7.0f : 1.0f;
        scales[b] = s;
        float inv = 1.0f / s;
        for (size_t idx = start; idx < end; idx++) {
            int8_t q = sat_i8(roundf(clampf(src[idx] * inv, -7.0f, 7.0f)));
            uint8_t nib = (uint8_t)(q & 0x0F);
            if ((idx & 1) == 0) data[idx / 2] = (uint8_t)((data[idx / 2] & 0x0F) | (nib << 4));
            else                data[idx / 2] = (uint8_t)((data[idx / 2] & 0xF0) | nib);
        }
    }
}
/* atlas-quant/src/lib.rs:149-168 */
void orc_int4_dequantize(const uint8_t* data, const float* scales, size_t n, size_t block, float* out) {
    for (size_t i = 0; i < n; i++) {
        float s = scales[i / block];
        uint8_t byte = data[i / 2];
        uint8_t nib = (i & 1) == 0 ? (uint8_t)(byte >> 4) : (uint8_t)(byte & 0x0F);
        int sgn = nib >= 8 ? (int)nib - 16 : (int)nib;
        out[i] = (float)sgn * s;
    }
}

/* ── math helpers ──────────────────────────────────────────────────────────── */
void orc_rmsnorm_inplace(float* x, const float* w, size_t n, float eps) {
    float ss = 0.0f;
    for (size_t i = 0; i < n; i++) ss += x[i] * x[i];
    ss = ss / (float)n;
    float inv = 1.0f / sqrtf(ss + eps);
    for (size_t i = 0; i < n; i++) x[i] = x[i] * inv * w[i];
}
float orc_silu(float x) { return x / (1.0f + expf(-x)); }
void orc_softmax_inplace(float* x, size_t n) {
    float mx = -INFINITY;
    for (size_t i = 0; i < n; i++) mx = fmaxf(mx, x[i]);
    float sum = 0.0f;
    for (size_t i = 0; i < n; i++) { x[i] = expf(x[i] - mx); sum += x[i]; }
    float inv = 1.0f / sum;
    for (size_t i = 0; i < n; i++) x[i] *= inv;
}
/* Iterator::max_by with partial_cmp().unwrap_or(Equal): the running best is kept only
 * when it compares Greater; Equal (ties and NaN) moves to the later element. */
size_t orc_argmax(const float* x, size_t n) {
    if (n == 0) return 0;
    size_t idx = 0; float best = x[0];
    for (size_t i = 1; i < n; i++) {
        if (!(best > x[i])) { best = x[i]; idx = i; }
    }
    return idx;
}

void orc_rope_tables(int head_dim, int max_seq, float theta, int scaling,
                     float factor, int orig_max_pos, float beta_fast, float beta_slow,
                     float* cos_out, float* sin_out) {
    int half = head_dim / 2;
    float two_pi = 2.0f * (float)M_PI;   /* 2.0 * std::f32::consts::PI */
    float* freqs = (float*)malloc(sizeof(float) * (size_t)(half > 0 ? half : 1));
    for (int i = 0; i < half; i++) {
        float base_freq = 1.0f / powf(theta, 2.0f * (float)i / (float)head_dim);
        float f = base_freq;
        if (scaling == 1) {
            float wavelength = two_pi / base_freq;
            float low  = (float)orig_max_pos / (two_pi * beta_slow);
            float high = (float)orig_max_pos / (two_pi * beta_fast);
            if (wavelength < high)      f = base_freq;
            else if (wavelength > low)  f = base_freq / factor;
            else {
                float alpha = (wavelength - high) / (low - high);
                f = base_freq / (alpha * factor + (1.0f - alpha));
            }
        }
        freqs[i] = f;
    }
    for (int pos = 0; pos < max_seq; pos++)
        for (int i = 0; i < half; i++) {
            cos_out[(size_t)pos * half + i] = cosf((float)pos * freqs[i]);
            sin_out[(size_t)pos * half + i] = sinf((float)pos * freqs[i]);
        }
    free(freqs);
}
void orc_rope_apply(float* x, int head_dim, const float* c, const float* s) {
    int half = head_dim / 2;
    for (int i = 0; i < half; i++) {
        float x0 = x[i], x1 = x[i + half];
        x[i]        = x0 * c[i] - x1 * s[i];
        x[i + half] = x0 * s[i] + x1 * c[i];
    }
}

void orc_linear_f32(const float* W, const float* x, float* y, size_t out_dim, size_t in_dim) {
#pragma omp parallel for schedule(static)
    for (size_t o = 0; o < out_dim; o++) {
        const float* row = W + o * in_dim;
        float acc = 0.0f;
        for (size_t k = 0; k < in_dim; k++) acc += row[k] * x[k];
        y[o] = acc;
    }
}
void orc_linear_bf16(const uint16_t* W, const float* x, float* y, size_t out_dim, size_t in_dim) {
#pragma omp parallel for schedule(static)
    for (size_t o = 0; o < out_dim; o++) {
        const uint16_t* row = W + o * in_dim;
        float acc = 0.0f;
        for (size_t k = 0; k < in_dim; k++) acc += orc_bf16_to_f32(row[k]) * x[k];
        y[o] = acc;
    }
}
void orc_gemm_f32(const float* W, const float* X, float* Y, size_t out_dim, size_t n, size_t in_dim) {
#pragma omp parallel for schedule(static)
    for (size_t o = 0; o < out_dim; o++)
        for (size_t c = 0; c < n; c++) {
            float acc = 0.0f;
            for (size_t k = 0; k < in_dim; k++) acc += W[o * in_dim + k] * X[k * n + c];
            Y[o * n + c] = acc;
        }
}
void orc_gemm_bf16(const uint16_t* W, const float* X, float* Y, size_t out_dim, size_t n, size_t in_dim) {
#pragma omp parallel for schedule(static)
    for (size_t o = 0; o < out_dim; o++)
        for (size_t c = 0; c < n; c++) {
            float acc = 0.0f;
            for (size_t k = 0; k < in_dim; k++) acc += orc_bf16_to_f32(W[o * in_dim + k]) * X[k * n + c];
            Y[o * n + c] = acc;
        }
}

void orc_decode_attention(const float* q, const float* kc, const float* vc, float* out,
                          int n_heads, int n_kv, int hd, int pos, float scale, int window) {
    int group = n_heads / n_kv;
    size_t stride = (size_t)n_kv * hd;
#pragma omp parallel for schedule(static)
    for (int h = 0; h < n_heads; h++) {
        int kv_h = h / group;
        const float* q_h = q + (size_t)h * hd;
        float* sc = (float*)malloc(sizeof(float) * (size_t)(pos + 1));
        for (int t = 0; t <= pos; t++) {
            int masked = window > 0 && (pos - t) >= window;
            if (masked) sc[t] = -INFINITY;
            else {
                const float* k_t = kc + (size_t)t * stride + (size_t)kv_h * hd;
                float s = 0.0f;
                for (int d = 0; d < hd; d++) s += q_h[d] * k_t[d];
                sc[t] = s * scale;
            }
        }
        orc_softmax_inplace(sc, (size_t)pos + 1);
        float* o_h = out + (size_t)h * hd;
        for (int d = 0; d < hd; d++) o_h[d] = 0.0f;
        for (int t = 0; t <= pos; t++) {
            const float* v_t = vc + (size_t)t * stride + (size_t)kv_h * hd;
            float a = sc[t];
            for (int d = 0; d < hd; d++) o_h[d] += a * v_t[d];
        }
        free(sc);
    }
}

/* ── model ─────────────────────────────────────────────────────────────────── */
typedef struct { const void* p; int dtype; } orc_w;

typedef struct {
    orc_w wq, wk, wv, wo, gate, up, down;
    const float *attn_norm, *ffn_norm, *q_norm, *k_norm;
    float *kc, *vc;           /* [max_seq × n_kv × hd] */
    int window;               /* 0 = full */
} orc_layer;

struct orc_model {
    orc_config cfg;
    int head_dim;
    float scale;
    orc_w embed, lm_head;
    const float* final_norm;
    orc_layer* layers;
    float *rope_cos, *rope_sin;
    int pos;
    int kv_round_bf16;
    /* owned storage (reference-random init, default unit norms) */
    float* ones;
    void** owned; int n_owned;
};

static void* own(orc_model* m, void* p) {
    m->owned = (void**)realloc(m->owned, sizeof(void*) * (size_t)(m->n_owned + 1));
    m->owned[m->n_owned++] = p;
    return p;
}

/* OlmoModel::new, atlas-model/src/lib.rs:1322-1353: RoPE tables, scale × attn_factor
 * when it differs from 1 by more than 1e-6, sliding window wired per layer type. */
orc_model* orc_model_new(const orc_config* cfg, const int* layer_sliding) {
    orc_model* m = (orc_model*)calloc(1, sizeof(orc_model));
    m->cfg = *cfg;
    m->head_dim = cfg->d_model / cfg->n_heads;
    int hd = m->head_dim, half = hd / 2;
    m->rope_cos = (float*)malloc(sizeof(float) * (size_t)cfg->max_seq_len * (size_t)(half > 0 ? half : 1));
    m->rope_sin = (float*)malloc(sizeof(float) * (size_t)cfg->max_seq_len * (size_t)(half > 0 ? half : 1));
    orc_rope_tables(hd, cfg->max_seq_len, cfg->rope_theta, cfg->rope_scaling, cfg->yarn_factor,
                    cfg->yarn_orig_max_pos, cfg->yarn_beta_fast, cfg->yarn_beta_slow,
                    m->rope_cos, m->rope_sin);
    m->scale = 1.0f / sqrtf((float)hd);
    float af = cfg->rope_scaling == 1 ? cfg->yarn_attn_factor : 1.0f;
    if (fabsf(af - 1.0f) > 1e-6f) m->scale *= af;
    m->ones = (float*)malloc(sizeof(float) * (size_t)cfg->d_model);
    for (int i = 0; i < cfg->d_model; i++) m->ones[i] = 1.0f;
    m->final_norm = m->ones;
    m->layers = (orc_layer*)calloc((size_t)cfg->n_layers, sizeof(orc_layer));
    size_t cap = (size_t)cfg->max_seq_len * cfg->n_kv_heads * hd;
    for (int l = 0; l < cfg->n_layers; l++) {
        orc_layer* L = &m->layers[l];
        L->kc = (float*)calloc(cap, sizeof(float));
        L->vc = (float*)calloc(cap, sizeof(float));
        L->attn_norm = m->ones; L->ffn_norm = m->ones;
        L->window = (layer_sliding && layer_sliding[l]) ? cfg->sliding_window : 0;
    }
    return m;
}
void orc_model_free(orc_model* m) {
    if (!m) return;
    for (int l = 0; l < m->cfg.n_layers; l++) { free(m->layers[l].kc); free(m->layers[l].vc); }
    for (int i = 0; i < m->n_owned; i++) free(m->owned[i]);
    free(m->owned); free(m->layers); free(m->rope_cos); free(m->rope_sin); free(m->ones); free(m);
}
int orc_model_set_tensor(orc_model* m, int layer, int which, const void* data, int dtype) {
    orc_w w = { data, dtype };
    if (which == ORC_T_EMBED) { m->embed = w; return 0; }
    if (which == ORC_T_LM_HEAD) { m->lm_head = w; return 0; }
    if (which == ORC_T_FINAL_NORM) { if (dtype) return -1; m->final_norm = (const float*)data; return 0; }
    if (layer < 0 || layer >= m->cfg.n_layers) return -1;
    orc_layer* L = &m->layers[layer];
    switch (which) {
        case ORC_T_WQ: L->wq = w; break;   case ORC_T_WK: L->wk = w; break;
        case ORC_T_WV: L->wv = w; break;   case ORC_T_WO: L->wo = w; break;
        case ORC_T_GATE: L->gate = w; break; case ORC_T_UP: L->up = w; break;
        case ORC_T_DOWN: L->down = w; break;
        case ORC_T_ATTN_NORM: if (dtype) return -1; L->attn_norm = (const float*)data; break;
        case ORC_T_FFN_NORM:  if (dtype) return -1; L->ffn_norm  = (const float*)data; break;
        case ORC_T_Q_NORM:    if (dtype) return -1; L->q_norm    = (const float*)data; break;
        case ORC_T_K_NORM:    if (dtype) return -1; L->k_norm    = (const float*)data; break;
        default: return -1;
    }
    return 0;
}

/* Linear::new, atlas-model/src/lib.rs:452-458: pseudo_randn × sqrt(2/(in+out)) */
static orc_w ref_linear(orc_model* m, size_t in_dim, size_t out_dim, uint64_t seed) {
    float* w = (float*)own(m, malloc(sizeof(float) * in_dim * out_dim));
    orc_pseudo_randn(w, in_dim * out_dim, seed);
    float scale = sqrtf(2.0f / (float)(in_dim + out_dim));
    for (size_t i = 0; i < in_dim * out_dim; i++) w[i] = w[i] * scale;
    orc_w r = { w, 0 };
    return r;
}
void orc_model_init_reference_random(orc_model* m) {
    const orc_config* c = &m->cfg;
    size_t d = (size_t)c->d_model, kv = (size_t)m->head_dim * c->n_kv_heads, f = (size_t)c->ffn_hidden;
    /* Embedding::new, :528-532: seed 0, × 0.02; lm_head is a copy (:1346-1350) */
    float* e = (float*)own(m, malloc(sizeof(float) * (size_t)c->vocab_size * d));
    orc_pseudo_randn(e, (size_t)c->vocab_size * d, 0);
    for (size_t i = 0; i < (size_t)c->vocab_size * d; i++) e[i] = e[i] * 0.02f;
    m->embed.p = e; m->embed.dtype = 0; m->lm_head = m->embed;
    for (int l = 0; l < c->n_layers; l++) {
        orc_layer* L = &m->layers[l];
        uint64_t sa = 1000 + (uint64_t)l * 10, sf = 2000 + (uint64_t)l * 10;   /* :627, :893 */
        L->wq = ref_linear(m, d, d, sa);      L->wk = ref_linear(m, d, kv, sa + 1);
        L->wv = ref_linear(m, d, kv, sa + 2); L->wo = ref_linear(m, d, d, sa + 3);
        L->gate = ref_linear(m, d, f, sf);    L->up = ref_linear(m, d, f, sf + 1);
        L->down = ref_linear(m, f, d, sf + 2);
    }
}
void orc_model_set_kv_round_bf16(orc_model* m, int on) { m->kv_round_bf16 = on; }
void orc_model_reset(orc_model* m) { m->pos = 0; }   /* caches are not cleared, :872-880 */
int  orc_model_pos(const orc_model* m) { return m->pos; }
void orc_model_seed_context(orc_model* m, int pos, uint64_t seed) {
    if (pos < 0) pos = 0;
    if (pos > m->cfg.max_seq_len) pos = m->cfg.max_seq_len;
    size_t n = (size_t)pos * m->cfg.n_kv_heads * m->head_dim;
    for (int l = 0; l < m->cfg.n_layers; l++) {
        orc_fill_normal_f32(m->layers[l].kc, n, seed, (uint64_t)(2 * l), 1.0f);
        orc_fill_normal_f32(m->layers[l].vc, n, seed, (uint64_t)(2 * l + 1), 1.0f);
    }
    m->pos = pos;
}

static void linear(orc_w w, const float* x, float* y, size_t out_dim, size_t in_dim) {
    if (w.dtype) orc_linear_bf16((const uint16_t*)w.p, x, y, out_dim, in_dim);
    else         orc_linear_f32((const float*)w.p, x, y, out_dim, in_dim);
}

/* Attention::forward_token, atlas-model/src/lib.rs:648-727 */
static void attention_forward_token(orc_model* m, orc_layer* L, const float* x, int pos, float* result) {
    const orc_config* c = &m->cfg;
    int hd = m->head_dim, nh = c->n_heads, nkv = c->n_kv_heads, half = hd / 2;
    size_t d = (size_t)nh * hd, kv = (size_t)nkv * hd;
    float* q = (float*)malloc(sizeof(float) * d);
    float* k = (float*)malloc(sizeof(float) * kv);
    float* v = (float*)malloc(sizeof(float) * kv);
    float* out = (float*)malloc(sizeof(float) * d);
    linear(L->wq, x, q, d, (size_t)c->d_model);
    linear(L->wk, x, k, kv, (size_t)c->d_model);
    linear(L->wv, x, v, kv, (size_t)c->d_model);
    if (L->q_norm) for (int h = 0; h < nh; h++)  orc_rmsnorm_inplace(q + (size_t)h * hd, L->q_norm + (size_t)h * hd, (size_t)hd, 1e-6f);
    if (L->k_norm) for (int h = 0; h < nkv; h++) orc_rmsnorm_inplace(k + (size_t)h * hd, L->k_norm + (size_t)h * hd, (size_t)hd, 1e-6f);
    const float* cr = m->rope_cos + (size_t)pos * half;
    const float* sr = m->rope_sin + (size_t)pos * half;
    for (int h = 0; h < nh; h++)  orc_rope_apply(q + (size_t)h * hd, hd, cr, sr);
    for (int h = 0; h < nkv; h++) orc_rope_apply(k + (size_t)h * hd, hd, cr, sr);
    if (m->kv_round_bf16) {
        for (size_t i = 0; i < kv; i++) { k[i] = orc_bf16_to_f32(orc_f32_to_bf16_rne(k[i])); v[i] = orc_bf16_to_f32(orc_f32_to_bf16_rne(v[i])); }
    }
    memcpy(L->kc + (size_t)pos * kv, k, sizeof(float) * kv);
    memcpy(L->vc + (size_t)pos * kv, v, sizeof(float) * kv);
    orc_decode_attention(q, L->kc, L->vc, out, nh, nkv, hd, pos, m->scale, L->window);
    linear(L->wo, out, result, d, d);
    free(q); free(k); free(v); free(out);
}

/* FeedForward::forward, :911-924 */
static void ffn_forward(orc_model* m, orc_layer* L, const float* x, float* out) {
    size_t f = (size_t)m->cfg.ffn_hidden, d = (size_t)m->cfg.d_model;
    float* gate = (float*)malloc(sizeof(float) * f);
    float* up = (float*)malloc(sizeof(float) * f);
    linear(L->gate, x, gate, f, d);
    linear(L->up, x, up, f, d);
    for (size_t i = 0; i < f; i++) gate[i] = orc_silu(gate[i]) * up[i];
    linear(L->down, gate, out, d, f);
    free(gate); free(up);
}

/* TransformerBlock::forward_token_cpu, :982-1006 */
static void block_forward_token(orc_model* m, orc_layer* L, float* x, int pos) {
    size_t d = (size_t)m->cfg.d_model;
    float eps = m->cfg.rms_norm_eps;
    float* t = (float*)malloc(sizeof(float) * d);
    float* xn = (float*)malloc(sizeof(float) * d);
    if (m->cfg.post_norm) {
        attention_forward_token(m, L, x, pos, t);
        orc_rmsnorm_inplace(t, L->attn_norm, d, eps);
        for (size_t i = 0; i < d; i++) x[i] += t[i];
        ffn_forward(m, L, x, t);
        orc_rmsnorm_inplace(t, L->ffn_norm, d, eps);
        for (size_t i = 0; i < d; i++) x[i] += t[i];
    } else {
        memcpy(xn, x, sizeof(float) * d);
        orc_rmsnorm_inplace(xn, L->attn_norm, d, eps);
        attention_forward_token(m, L, xn, pos, t);
        for (size_t i = 0; i < d; i++) x[i] += t[i];
        memcpy(xn, x, sizeof(float) * d);
        orc_rmsnorm_inplace(xn, L->ffn_norm, d, eps);
        ffn_forward(m, L, xn, t);
        for (size_t i = 0; i < d; i++) x[i] += t[i];
    }
    free(t); free(xn);
}

void orc_forward_one(orc_model* m, uint32_t token, float* logits, float* hidden_out) {
    const orc_config* c = &m->cfg;
    size_t d = (size_t)c->d_model;
    int pos = m->pos; m->pos += 1;
    /* Embedding::embed_token, :539-542 — id clamped to vocab−1 */
    size_t id = token; if (id > (size_t)c->vocab_size - 1) id = (size_t)c->vocab_size - 1;
    float* x = (float*)malloc(sizeof(float) * d);
    if (m->embed.dtype) for (size_t i = 0; i < d; i++) x[i] = orc_bf16_to_f32(((const uint16_t*)m->embed.p)[id * d + i]);
    else memcpy(x, (const float*)m->embed.p + id * d, sizeof(float) * d);
    for (int l = 0; l < c->n_layers; l++) {
        block_forward_token(m, &m->layers[l], x, pos);
        if (hidden_out) memcpy(hidden_out + (size_t)l * d, x, sizeof(float) * d);
    }
    orc_rmsnorm_inplace(x, m->final_norm, d, c->rms_norm_eps);
    linear(m->lm_head, x, logits, (size_t)c->vocab_size, d);
    free(x);
}

/* apply_repetition_penalty, :2581-2592 */
static void repetition_penalty(float* logits, size_t n, const uint32_t* toks, int nt, float theta) {
    for (int i = 0; i < nt; i++) {
        size_t idx = toks[i];
        if (idx < n) { if (logits[idx] > 0.0f) logits[idx] /= theta; else logits[idx] *= theta; }
    }
}

int orc_generate_greedy(orc_model* m, const uint32_t* prompt, int n_prompt, int max_new,
                        const uint32_t* suppress, int n_suppress, float rep_penalty, int rep_window,
                        const uint32_t* stops, int n_stops,
                        uint32_t* out_tokens, float* logits_trace, float* margin_trace) {
    size_t V = (size_t)m->cfg.vocab_size;
    orc_model_reset(m);
    float* last = (float*)calloc(V, sizeof(float));   /* vec![0.0; vocab] */
    float* work = (float*)malloc(sizeof(float) * V);
    for (int i = 0; i < n_prompt; i++) orc_forward_one(m, prompt[i], last, NULL);
    int n_out = 0;
    for (int step = 0; step < max_new; step++) {
        memcpy(work, last, sizeof(float) * V);
        if (step == 0) for (int i = 0; i < n_suppress; i++) if ((size_t)suppress[i] < V) work[suppress[i]] = -INFINITY;
        if (rep_penalty != 1.0f && n_out > 0) {
            int start = n_out > rep_window ? n_out - rep_window : 0;
            repetition_penalty(work, V, out_tokens + start, n_out - start, rep_penalty);
        }
        size_t next = orc_argmax(work, V);
        if (margin_trace) {
            float second = -INFINITY;
            for (size_t i = 0; i < V; i++) if (i != next && work[i] > second) second = work[i];
            margin_trace[step] = work[next] - second;
        }
        uint32_t tok = (uint32_t)next;
        if (m->cfg.eos_token_id >= 0 && tok == (uint32_t)m->cfg.eos_token_id) break;
        int stop = 0;
        for (int i = 0; i < n_stops; i++) if (stops[i] == tok) stop = 1;
        if (stop) break;
        if (logits_trace) memcpy(logits_trace + (size_t)n_out * V, work, sizeof(float) * V);
        out_tokens[n_out++] = tok;
        orc_forward_one(m, tok, last, NULL);
    }
    free(last); free(work);
    return n_out;
}

/* ── sampling ──────────────────────────────────────────────────────────────── */
uint64_t orc_rng_from_seed(uint64_t seed) { return seed | 1u; }
float orc_rng_next_f32(uint64_t* st) {
    uint64_t x = *st;
    x ^= x << 13; x ^= x >> 7; x ^= x << 17;
    *st = x;
    return (float)(x >> 33) / (float)(1ull << 31);
}
void orc_apply_repetition_penalty(float* logits, size_t n, const uint32_t* toks, int nt, float theta) {
    repetition_penalty(logits, n, toks, nt, theta);
}
void orc_apply_frequency_penalty(float* logits, size_t n, const uint32_t* history, int nh, float penalty) {
    /* (token, count) pairs in order of first occurrence, one subtraction per distinct token */
    for (int i = 0; i < nh; i++) {
        int first = 1;
        for (int j = 0; j < i; j++) if (history[j] == history[i]) { first = 0; break; }
        if (!first) continue;
        size_t count = 0;
        for (int j = i; j < nh; j++) if (history[j] == history[i]) count++;
        size_t idx = history[i];
        if (idx < n) logits[idx] -= penalty * (float)count;
    }
}
void orc_apply_presence_penalty(float* logits, size_t n, const uint32_t* history, int nh, float penalty) {
    for (int i = 0; i < nh; i++) {
        int first = 1;
        for (int j = 0; j < i; j++) if (history[j] == history[i]) { first = 0; break; }
        size_t idx = history[i];
        if (first && idx < n) logits[idx] -= penalty;
    }
}
static int cmp_desc_f32(const void* a, const void* b) {
    float x = *(const float*)a, y = *(const float*)b;
    return (y > x) - (y < x);
}
void orc_apply_top_k(float* logits, size_t n, size_t k) {
    if (k == 0 || k >= n) return;
    float* sorted = (float*)malloc(sizeof(float) * n);
    memcpy(sorted, logits, sizeof(float) * n);
    qsort(sorted, n, sizeof(float), cmp_desc_f32);
    float threshold = sorted[k - 1];
    free(sorted);
    size_t at_or_above = 0, above = 0;
    for (size_t i = 0; i < n; i++) { if (logits[i] >= threshold) at_or_above++; if (logits[i] > threshold) above++; }
    if (at_or_above <= k) {
        for (size_t i = 0; i < n; i++) if (logits[i] < threshold) logits[i] = -INFINITY;
    } else {                                   /* ties at the threshold: the first ones in index order are kept */
        size_t need = k - above, kept = 0;
        for (size_t i = 0; i < n; i++) {
            if (logits[i] > threshold) continue;
            if (logits[i] == threshold && kept < need) { kept++; continue; }
            logits[i] = -INFINITY;
        }
    }
}
typedef struct { size_t idx; float p; } orc_ip;
static int cmp_ip_desc(const void* a, const void* b) {
    const orc_ip* x = (const orc_ip*)a; const orc_ip* y = (const orc_ip*)b;
    if (y->p > x->p) return 1;
    if (y->p < x->p) return -1;
    return (x->idx > y->idx) - (x->idx < y->idx);
}
void orc_apply_top_p(float* logits, size_t n, float p) {
    if (n == 0) return;
    float max_l = -INFINITY;
    for (size_t i = 0; i < n; i++) max_l = fmaxf(max_l, logits[i]);
    orc_ip* pr = (orc_ip*)malloc(sizeof(orc_ip) * n);
    float sum = 0.0f;
    for (size_t i = 0; i < n; i++) { pr[i].idx = i; pr[i].p = expf(logits[i] - max_l); }
    for (size_t i = 0; i < n; i++) sum += pr[i].p;
    if (sum <= 0.0f) { free(pr); return; }
    for (size_t i = 0; i < n; i++) pr[i].p /= sum;
    qsort(pr, n, sizeof(orc_ip), cmp_ip_desc);
    float cum = 0.0f; size_t cutoff = n;
    for (size_t i = 0; i < n; i++) { cum += pr[i].p; if (cum >= p) { cutoff = i + 1; break; } }
    for (size_t i = cutoff; i < n; i++) logits[pr[i].idx] = -INFINITY;
    free(pr);
}
void orc_apply_min_p(float* logits, size_t n, float min_p) {
    if (min_p <= 0.0f) return;
    float max_l = -INFINITY;
    for (size_t i = 0; i < n; i++) max_l = fmaxf(max_l, logits[i]);
    float threshold = max_l + logf(min_p);
    for (size_t i = 0; i < n; i++) if (logits[i] < threshold) logits[i] = -INFINITY;
}
size_t orc_sample_from_probs(const float* probs, size_t n, float r) {
    float cum = 0.0f;
    for (size_t i = 0; i < n; i++) { cum += probs[i]; if (r < cum) return i; }
    return n - 1;
}
size_t orc_sample_token(const float* last_logits, size_t n, const orc_sampling* cfg, int step,
                        const uint32_t* suppress, int n_suppress, const uint32_t* history, int n_hist,
                        uint64_t* rng, float* probs_out) {
    float* l = (float*)malloc(sizeof(float) * n);
    memcpy(l, last_logits, sizeof(float) * n);
    if (step == 0) for (int i = 0; i < n_suppress; i++) if ((size_t)suppress[i] < n) l[suppress[i]] = -INFINITY;
    if (cfg->repetition_penalty != 1.0f && n_hist > 0) {
        int start = n_hist > cfg->repetition_window ? n_hist - cfg->repetition_window : 0;
        repetition_penalty(l, n, history + start, n_hist - start, cfg->repetition_penalty);
    }
    size_t next;
    if (cfg->temperature <= 0.0f || cfg->temperature < 1e-6f) {
        next = orc_argmax(l, n);
    } else {
        if (cfg->frequency_penalty != 0.0f && n_hist > 0) orc_apply_frequency_penalty(l, n, history, n_hist, cfg->frequency_penalty);
        if (cfg->presence_penalty != 0.0f && n_hist > 0) orc_apply_presence_penalty(l, n, history, n_hist, cfg->presence_penalty);
        for (size_t i = 0; i < n; i++) l[i] /= cfg->temperature;
        if (cfg->top_k > 0) orc_apply_top_k(l, n, (size_t)cfg->top_k);
        if (cfg->top_p < 1.0f) orc_apply_top_p(l, n, cfg->top_p);
        if (cfg->min_p > 0.0f) orc_apply_min_p(l, n, cfg->min_p);
        orc_softmax_inplace(l, n);
        if (probs_out) memcpy(probs_out, l, sizeof(float) * n);
        next = orc_sample_from_probs(l, n, orc_rng_next_f32(rng));
    }
    free(l);
    return next;
}
int orc_generate_sampling(orc_model* m, const uint32_t* prompt, int n_prompt, int max_new, const orc_sampling* cfg,
                          const uint32_t* suppress, int n_suppress, const uint32_t* stops, int n_stops,
                          uint64_t seed, uint32_t* out_tokens) {
    size_t V = (size_t)m->cfg.vocab_size;
    orc_model_reset(m);
    uint64_t rng = orc_rng_from_seed(seed);
    float* last = (float*)calloc(V, sizeof(float));
    for (int i = 0; i < n_prompt; i++) orc_forward_one(m, prompt[i], last, NULL);
    int n_out = 0;
    for (int step = 0; step < max_new; step++) {
        uint32_t tok = (uint32_t)orc_sample_token(last, V, cfg, step, suppress, n_suppress, out_tokens, n_out, &rng, NULL);
        if (m->cfg.eos_token_id >= 0 && tok == (uint32_t)m->cfg.eos_token_id) break;
        int stop = 0;
        for (int i = 0; i < n_stops; i++) if (stops[i] == tok) stop = 1;
        if (stop) break;
        out_tokens[n_out++] = tok;
        orc_forward_one(m, tok, last, NULL);
    }
    free(last);
    return n_out;
}
