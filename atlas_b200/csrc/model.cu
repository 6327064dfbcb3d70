// model.cu — the decode step of OlmoModel on one GPU (or one tensor-parallel rank).
//
// Restates, for the device, crates/atlas-model/src/lib.rs of the reference:
//   OlmoModel::forward_one_gpu :1463-1505, TransformerBlock::forward_token_gpu_v2 :1015-1091,
//   Attention::forward_token_gpu_full :837-870, FeedForward::forward_gpu :902-908,
//   generate_with_sampling (greedy branch) :1599-1646,1713-1730, init_gpu_resources :1360-1386.
// The reference issues 18 launches and 18 allocations per layer; here a layer is five launches
//   QKV GEMV (prologue: residual + RMSNorm of the previous sub-layer, or embedding gather)
//   QK-norm + RoPE + KV write
//   split-K attention
//   o_proj GEMV
//   gate/up GEMV (prologue: post-attention norm + residual; epilogue: SwiGLU)
//   down GEMV
// and the whole token (plus lm_head, argmax and position advance) is one CUDA graph whose
// token id and position live in device memory, so replaying it needs no host data.
#include <limits.h>
#include <stdlib.h>
#include <math.h>
#include <string.h>
#include <vector>

#include "attention.cuh"
#include "attention_mma.cuh"
#include "comm.h"
#include "common.cuh"
#include "elementwise.cuh"
#include "gemv.cuh"
#include "objects.h"
#include "sampling.cuh"
#include <time.h>

namespace {

enum { CLS_QKV = 0, CLS_QKPREP, CLS_ATTN, CLS_OPROJ, CLS_GATEUP, CLS_DOWN, CLS_LMHEAD, CLS_SELECT, CLS_COMM, CLS_COUNT };
const char* kClassNames[CLS_COUNT] = { "gemv_qkv", "qk_norm_rope_kvwrite", "attention_splitk", "gemv_o_proj",
                                       "gemv_gate_up_swiglu", "gemv_down", "gemv_lm_head", "argmax_advance", "collective" };

struct StepState {           // device-resident generation state
    int pos;                 // next position to be processed
    int n_forced;            // positions below this hold caller-given tokens
    int last_token;          // argmax of the most recent logits
};

struct Layer {
    AxWeight qkv, wo, gateup, down;
    float *attn_norm = nullptr, *ffn_norm = nullptr, *q_norm = nullptr, *k_norm = nullptr;
    atlasx_kvcache* kv = nullptr;
    int window = 0;
    bool have[11] = {};      // which - ATLASX_T_WQ
};

struct Profile {
    std::vector<cudaEvent_t> ev;
    std::vector<int> cls;
    std::vector<double> bytes;
    int n = 0;
};

}  // namespace

struct atlasx_model {
    atlasx_ctx* ctx = nullptr;
    atlasx_model_config cfg;
    int hd = 0, nh_loc = 0, nkv_loc = 0, ffn_loc = 0, vocab_loc = 0, world = 1, rank = 0;
    int q_rows = 0, kv_rows = 0;                 // nh_loc·hd, nkv_loc·hd
    float scale = 1.f;
    std::vector<Layer> layers;
    void* embed = nullptr; int embed_bf16 = 0; bool have_embed = false;
    float* final_norm = nullptr;
    AxWeight lm_head; bool have_lm_head = false;
    float *cos_t = nullptr, *sin_t = nullptr;
    // activations
    float *resid[2] = { nullptr, nullptr }, *qkv = nullptr, *attn = nullptr, *o = nullptr, *h = nullptr, *dn = nullptr;
    float *logits_loc = nullptr, *logits = nullptr;
    int* seq = nullptr; StepState* st = nullptr;
    // Residual stream: resid[0] holds the embedding of the token, resid[1] the stream after each
    // attention sub-layer, taps[l] the stream after layer l — one buffer per layer instead of a
    // ping-pong pair, so that every layer's output survives the step and can be handed to a hook.
    float* taps = nullptr;                       // [n_layers][d_model]
    // per-layer hook (StigmergicHook, crates/atlas-infer/src/hook.rs): the taps of a forward are copied to
    // pinned host memory behind it and the hook runs on the host while the next forward executes
    atlasx_layer_hook hook_fn = nullptr; void* hook_user = nullptr;
    atlasx_token_callback tok_fn = nullptr; void* tok_user = nullptr;     // generate_streaming: called per emitted token, 0 stops
    float* tap_host[2] = { nullptr, nullptr }; cudaEvent_t tap_ev[2] = { nullptr, nullptr };
    int tap_k = 0; bool tap_pending = false; long long tap_tok[2] = { -1, -1 };
    std::vector<uint32_t> dep_tok, dep_fired; std::vector<float> dep_delta;
    int host_pos = 0;
    bool finalized = false;
    int use_graph = 1, use_pdl = 1;
    cudaGraphExec_t graph = nullptr;
    int attn_splits = 1;
    bool fused_attn = false; int fused_splits = 1;   // one-launch attention (head_dim 128)
    float* attn_partials = nullptr; unsigned* attn_tickets = nullptr;   // split-attention scratch of this model's step graph
    const AxPeerMail* mail = nullptr;            // tensor parallel: all-reduce fused into o_proj/down over peer memory
    int class_mask = (1 << CLS_COUNT) - 1;       // launch classes issued by run_step (all, except while one family is timed)
    int mail_mode = 0;                           // who sums the mailbox parts: 0 every consumer CTA, 1 a kernel of its own, 2 the consumer's first CTAs
    uint2* mail_red[2] = { nullptr, nullptr };   // mode 2: the summed vector as (value, sequence) pairs, per mailbox buffer
    bool tp_select = false;                      // greedy selection over the ranks' local maxima instead of all-gathered logits
    cudaGraphExec_t graph_tok = nullptr;         // the step without the logits all-gather (tensor parallel, token-only callers)
    std::vector<void*> owned;                    // device allocations to free
    int* pin = nullptr;                          // pinned host ints
    float* pin_logits = nullptr;                 // pinned staging for logits handed to the host (allocated on first use)
    int launches_per_step = 0;
    // prompt ingestion in chunks of up to kPrefillMax tokens through the multi-column kernels
    int prefill_chunk = 1;                       // 1: token by token (the reference's way)
    float *pf_r = nullptr, *pf_a = nullptr, *pf_qkv = nullptr, *pf_att = nullptr, *pf_o = nullptr,
          *pf_gu = nullptr, *pf_h = nullptr, *pf_dn = nullptr;
    int* pf_pos = nullptr;
    float* pf_parts = nullptr;                          // partial tiles of K-split layer products that the next kernel adds up
    float* pf_attn_partials = nullptr; unsigned* pf_attn_tickets = nullptr; int pf_attn_splits = 0;   // causal chunk attention (bf16 cache, head_dim 128)
    // timeline diagnostics of the captured step (ATLASX_STEP_TRACE)
    unsigned long long* step_trace = nullptr; int step_trace_slots = 0;
};

namespace {

int dmalloc(atlasx_model* m, void** p, size_t bytes) {
    AX_CUDA(cudaMalloc(p, bytes ? bytes : 16));
    m->owned.push_back(*p);
    return ATLASX_OK;
}
int format_ebits(int fmt) { return fmt == ATLASX_F32 ? 32 : fmt == ATLASX_BF16 ? 16 : fmt == ATLASX_INT8 ? 8 : 4; }

// Allocate the device arrays of a weight [rows × cols] in the model's storage format.
int alloc_weight(atlasx_model* m, AxWeight& w, int rows, int cols) {
    const int fmt = m->cfg.weight_format;
    w.rows = rows; w.cols = cols; w.dtype = fmt;
    w.block = fmt == ATLASX_INT4 ? m->cfg.int4_block : 0;
    w.scales_f16 = 0;
    void* d = nullptr;
    int rc = dmalloc(m, &d, (size_t)rows * cols * format_ebits(fmt) / 8);
    if (rc) return rc;
    AX_CUDA(cudaMemsetAsync(d, 0, (size_t)rows * cols * format_ebits(fmt) / 8, m->ctx->stream));
    w.data = d;
    if (fmt == ATLASX_INT8) { rc = dmalloc(m, &d, (size_t)rows * 4); if (rc) return rc; w.scales = d; AX_CUDA(cudaMemsetAsync(d, 0, (size_t)rows * 4, m->ctx->stream)); }
    if (fmt == ATLASX_INT4) {
        const size_t nb = (size_t)rows * (cols / w.block);
        rc = dmalloc(m, &d, nb * 4); if (rc) return rc; w.scales = d;
        AX_CUDA(cudaMemsetAsync(d, 0, nb * 4, m->ctx->stream));
    }
    return ATLASX_OK;
}

// Convert the FULL tensor (device, f32 or bf16) to the storage format, then copy the slice
// rows [r0,r0+nr) × cols [c0,c0+nc) into dest rows dest_r0 + i·step (+ phase is folded into dest_r0).
int place_slice(atlasx_model* m, const void* src, int src_dtype, int rows, int cols,
                int r0, int nr, int c0, int nc, AxWeight& dest, int dest_r0, int step) {
    atlasx_ctx* c = m->ctx;
    cudaStream_t s = c->stream;
    const int fmt = dest.dtype;
    const size_t n = (size_t)rows * cols;
    void *t_f32 = nullptr, *t_data = nullptr, *t_scales = nullptr;
    const void* data = src;            // full tensor in storage format
    const void* scales = nullptr;
    int rc = ATLASX_OK;
    auto cleanup = [&]() { cudaStreamSynchronize(s); cudaFree(t_f32); cudaFree(t_data); cudaFree(t_scales); };
    if (fmt == ATLASX_F32) {
        if (src_dtype == ATLASX_BF16) {
            AX_CUDA(cudaMalloc(&t_data, n * 4));
            ax_bf16_to_f32(s, (const uint16_t*)src, (float*)t_data, n); data = t_data;
        }
    } else if (fmt == ATLASX_BF16) {
        if (src_dtype == ATLASX_F32) {       // f32 → bf16 by truncation, as make_linear_bf16_aware (:2271-2279)
            AX_CUDA(cudaMalloc(&t_data, n * 2));
            ax_f32_to_bf16(s, (const float*)src, (uint16_t*)t_data, n, 1); data = t_data;
        }
    } else {
        const float* f = (const float*)src;
        if (src_dtype == ATLASX_BF16) {
            AX_CUDA(cudaMalloc(&t_f32, n * 4));
            ax_bf16_to_f32(s, (const uint16_t*)src, (float*)t_f32, n); f = (const float*)t_f32;
        }
        if (fmt == ATLASX_INT8) {
            if (cudaMalloc(&t_data, n) != cudaSuccess || cudaMalloc(&t_scales, (size_t)rows * 4) != cudaSuccess) {
                cleanup(); return atlasx_fail(ATLASX_ERR_CUDA, "out of device memory while quantising");
            }
            ax_quant_int8(s, f, rows, cols, (int8_t*)t_data, (float*)t_scales);
        } else {
            const size_t nb = (n + dest.block - 1) / dest.block;
            if (cudaMalloc(&t_data, (n + 1) / 2) != cudaSuccess || cudaMalloc(&t_scales, nb * 4) != cudaSuccess) {
                cleanup(); return atlasx_fail(ATLASX_ERR_CUDA, "out of device memory while quantising");
            }
            ax_quant_int4(s, f, n, dest.block, (uint8_t*)t_data, (float*)t_scales);
        }
        data = t_data; scales = t_scales;
    }
    // data slice
    const int eb = format_ebits(fmt);
    if (fmt == ATLASX_INT4) {          // copy in bytes (two elements each)
        ax_copy2d(s, (uint8_t*)dest.data + (size_t)dest_r0 * (dest.cols / 2), (size_t)step * (dest.cols / 2),
                  (const uint8_t*)data + ((size_t)r0 * cols + c0) / 2, (size_t)cols / 2, nr, nc / 2, 1);
        const int bs = dest.block;
        ax_copy2d(s, (float*)dest.scales + (size_t)dest_r0 * (dest.cols / bs), (size_t)step * (dest.cols / bs),
                  (const float*)scales + (size_t)r0 * (cols / bs) + c0 / bs, (size_t)cols / bs, nr, nc / bs, 4);
    } else {
        const int es = eb / 8;
        ax_copy2d(s, (uint8_t*)dest.data + (size_t)dest_r0 * dest.cols * es, (size_t)step * dest.cols,
                  (const uint8_t*)data + ((size_t)r0 * cols + c0) * es, (size_t)cols, nr, nc, es);
        if (fmt == ATLASX_INT8)
            ax_copy2d(s, (float*)dest.scales + dest_r0, (size_t)step, (const float*)scales + r0, 1, nr, 1, 4);
    }
    cudaError_t e = cudaGetLastError();
    cleanup();
    if (e != cudaSuccess) rc = atlasx_fail(ATLASX_ERR_CUDA, "weight placement failed: %s", cudaGetErrorString(e));
    return rc;
}

// ── argmax of the logits + advance of the device-resident state ─────────────────
// Last CTA: last_token = argmax; if the next position is not a caller-given one, the token is
// stored as the next input; pos += 1.
// Vocabulary-parallel selection: every rank holds the logits of its own rows only.  The last CTA
// leaves the local best in entry `rank` of every rank's selection slots (one 16-byte store: value,
// vocabulary index, sequence number twice) and then picks the best of all ranks' entries — the same
// (value, last index) rule, so every rank arrives at the same token without the logits leaving their GPU.
struct SelPeers {
    int n = 0, rank = 0, index_base = 0, vocab = 0;
    uint4* dst[AX_MAX_PEERS] = {};        // this rank's entry in rank p's slots
    const uint4* mine = nullptr;          // this rank's slots [n]
    int* err = nullptr;
};

// useq (may be null): the mailbox use counter of the tensor-parallel group, advanced by `bump` per step.
__global__ void __launch_bounds__(256) select_advance_k(const float* x, int n, AxArgmaxScratch sc, StepState* st, int* seq, int seq_cap, int advance,
                                                        unsigned* useq, unsigned bump, SelPeers peers) {
    __shared__ float sv[8];
    __shared__ int si[8];
    __shared__ int s_last;
    asm volatile("griddepcontrol.wait;" ::: "memory");
    float v = 0.f; int idx = -1;
    const int base = blockIdx.x * 1024;
#pragma unroll
    for (int u = 0; u < 4; u++) {
        const int i = base + u * 256 + threadIdx.x;
        if (i < n) { const float xv = x[i]; if (ax_better(xv, i, v, idx, 1)) { v = xv; idx = i; } }
    }
    ax_warp_best(v, idx, 1);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) { sv[warp] = v; si[warp] = idx; }
    __syncthreads();
    if (warp == 0) {
        v = lane < 8 ? sv[lane] : 0.f; idx = lane < 8 ? si[lane] : -1;
        ax_warp_best(v, idx, 1);
        if (lane == 0) {
            sc.vals[blockIdx.x] = v; sc.idx[blockIdx.x] = idx;
            __threadfence();
            s_last = atomicAdd(sc.ticket, 1u) == gridDim.x - 1;
        }
    }
    __syncthreads();
    if (!s_last || warp != 0) return;
    __threadfence();
    v = 0.f; idx = -1;
    for (int j = lane; j < (int)gridDim.x; j += 32) {
        const float bv = sc.vals[j]; const int bi = sc.idx[j];
        if (ax_better(bv, bi, v, idx, 1)) { v = bv; idx = bi; }
    }
    ax_warp_best(v, idx, 1);
    if (peers.n > 0) {
        const unsigned stamp = *useq + bump;                      // the counter's value after this step: unique per step, never 0
        if (idx >= 0) idx += peers.index_base;
        if (lane < peers.n)
            asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" :: "l"(peers.dst[lane]), "r"(__float_as_uint(v)), "r"((unsigned)idx),
                         "r"(stamp), "r"(stamp) : "memory");
        float pv = 0.f; int pi = -1;
        if (lane < peers.n) {
            uint4 e;
            const unsigned long long t0 = ax_globaltimer();
            for (;;) {
                asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(e.x), "=r"(e.y), "=r"(e.z), "=r"(e.w) : "l"(peers.mine + lane) : "memory");
                if (e.z == stamp && e.w == stamp) break;
                if (*reinterpret_cast<volatile int*>(peers.err) != 0) break;
                if (ax_globaltimer() - t0 > 2000000000ull) { atomicExch(peers.err, 4); break; }
            }
            pv = __uint_as_float(e.x); pi = (int)e.y;
        }
        v = pv; idx = pi;
        ax_warp_best(v, idx, 1);
        n = peers.vocab;                                          // idx is a vocabulary index now
    }
    if (lane == 0) {
        if (idx < 0) idx = n - 1;
        *sc.ticket = 0u;
        st->last_token = idx;
        if (useq) *useq += bump;
        if (advance) {
            const int p = st->pos + 1;
            if (p >= st->n_forced && p < seq_cap) seq[p] = idx;
            st->pos = p;
        } else {
            const int p = st->pos;                 // re-selection for the position about to be processed
            if (p < seq_cap) seq[p] = idx;
        }
    }
}

// Greedy-path logit edits of generate_with_sampling (:1631-1644), applied in order by one thread:
// first-token suppression, then the repetition penalty once per occurrence in the window.
__global__ void logit_fixups_k(float* logits, int n, const int* suppress, int n_suppress,
                               const int* history, int n_hist, float theta) {
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    for (int i = 0; i < n_suppress; i++) { const int t = suppress[i]; if (t >= 0 && t < n) logits[t] = -INFINITY; }
    if (theta != 1.0f)
        for (int i = 0; i < n_hist; i++) {
            const int t = history[i];
            if (t >= 0 && t < n) { if (logits[t] > 0.0f) logits[t] /= theta; else logits[t] *= theta; }
        }
}

// seq_fix != null: the token at `pos` is the most recent greedy choice (it may not have been
// stored yet when the previous steps ran with caller-given tokens)
__global__ void set_state_k(StepState* st, int pos, int n_forced, int* seq_fix = nullptr) {
    st->pos = pos; st->n_forced = n_forced;
    if (seq_fix) seq_fix[pos] = st->last_token;
}

double gemv_bytes(const AxWeight& w) { return (double)ax_weight_bytes(w) + 4.0 * w.cols + 4.0 * w.rows; }

#define STEP_LAUNCH(CLS, BYTES, CALL)                                                        \
    do {                                                                                     \
        if (!((m->class_mask >> (CLS)) & 1)) break;                                          \
        if (prof) cudaEventRecord(prof->ev[2 * prof->n], s);                                 \
        rc = (CALL);                                                                         \
        if (rc) return rc;                                                                   \
        if (prof) { cudaEventRecord(prof->ev[2 * prof->n + 1], s); prof->cls[prof->n] = (CLS); prof->bytes[prof->n] = (BYTES); prof->n++; } \
        n_launch++;                                                                          \
    } while (0)

// One token: every launch of the step, in order, on the context stream.
// gather: under tensor parallelism, all-gather the logits and select over the full vector (callers
// that read logits); otherwise the ranks exchange only their local maxima.
int run_step(atlasx_model* m, Profile* prof, bool advance, bool gather = true) {
    atlasx_ctx* c = m->ctx;
    cudaStream_t s = c->stream;
    const atlasx_model_config& cf = m->cfg;
    const bool pdl = m->use_pdl && !prof;
    auto P = [&](int cls) { return pdl && ((c->tune.pdl_mask >> cls) & 1); };
    const int d = cf.d_model, L = cf.n_layers;
    const bool post = cf.post_norm != 0;
    int rc = ATLASX_OK, n_launch = 0;
    const int nparts = 1;                                  // partial sums are reduced by the collective …
    // … unless the ranks push them into each other's mailboxes: then the consumer's prologue
    // waits for the sequence number of (step, layer) and adds the parts itself, in rank order
    const AxPeerMail* mail = m->mail;
    auto peer_out = [&](int buf, int l) {
        AxPeerOut po;
        po.n = mail->world;
        for (int q = 0; q < mail->world; q++) po.y[q] = mail->part(q, buf, mail->rank);
        po.epoch = mail->useq; po.mul = 1u; po.add = (unsigned)l + 1u;                // use number = uses so far + layer + 1
        return po;
    };
    auto peer_in = [&](AxPrologue& p, int buf, int l) {
        if (m->mail_mode == 1) return;                     // p.y already names the reduced vector
        p.y = reinterpret_cast<const float*>(mail->part(mail->rank, buf, 0));
        p.nparts = mail->world; p.part_stride = (size_t)mail->d;
        p.ll_n = mail->world; p.ll_stride = (size_t)mail->d;
        p.ll_epoch = mail->useq; p.ll_mul = 1u; p.ll_add = (unsigned)l + 1u;
        if (m->mail_mode == 2) { p.ll_red = m->mail_red[buf]; p.ll_red_ctas = 8; }
    };

    for (int l = 0; l < L; l++) {
        Layer& ly = m->layers[l];
        // ── QKV projection ──────────────────────────────────────────────────────
        AxPrologue p;
        p.eps = cf.rms_norm_eps;
        if (l == 0) {
            p.embed = m->embed; p.embed_bf16 = m->embed_bf16; p.vocab = cf.vocab_size;
            p.seq = m->seq; p.pos = &m->st->pos;
            p.resid_out = m->resid[0];
            if (!post) p.wx = ly.attn_norm;
        } else {
            p.base = m->resid[1]; p.y = m->dn; p.nparts = nparts; p.part_stride = d;
            if (mail) peer_in(p, 1, l - 1);
            p.base_early = 1;                              // written by the gate/up launch, two kernels back
            if (post) p.wy = m->layers[l - 1].ffn_norm; else p.wx = ly.attn_norm;
            p.resid_out = m->taps + (size_t)(l - 1) * d;                         // output of layer l−1
        }
        STEP_LAUNCH(CLS_QKV, gemv_bytes(ly.qkv), ax_gemv_launch(c, ly.qkv, p, AX_EPI_PLAIN, 1, m->qkv, P(CLS_QKV)));

        double abytes = 0;
        if (prof) {
            int rows = m->host_pos + 1;
            if (ly.window > 0 && rows > ly.window) rows = ly.window;
            abytes = (double)rows * 2 * m->kv_rows * (cf.kv_dtype == ATLASX_BF16 ? 2 : 4) + 8.0 * m->q_rows;
        }
        if (m->fused_attn) {
            // ── QK-norm, RoPE, cache write and attention in one launch ─────────────
            AxFusedAttnArgs fa;
            fa.qkv = m->qkv; fa.q_norm = ly.q_norm; fa.k_norm = ly.k_norm; fa.cos_t = m->cos_t; fa.sin_t = m->sin_t;
            fa.kc = ly.kv->k; fa.vc = ly.kv->v; fa.out = m->attn; fa.pos = &m->st->pos;
            fa.n_heads = m->nh_loc; fa.n_kv = m->nkv_loc; fa.window = ly.window; fa.kv_dtype = cf.kv_dtype;
            fa.max_splits = m->fused_splits; fa.scale = m->scale;
            fa.qk_eps = 1e-6f;                             // the reference hard-codes 1e-6 here (:850,853)
            fa.scratch_partials = m->attn_partials; fa.scratch_tickets = m->attn_tickets;
            STEP_LAUNCH(CLS_ATTN, abytes + 4.0 * (m->q_rows + 2 * m->kv_rows), ax_attn_fused_launch(c, fa, P(CLS_ATTN)));
        } else {
        // ── QK-norm, RoPE, cache write ──────────────────────────────────────────
        AxQkPrepArgs qa;
        qa.q = m->qkv; qa.k = m->qkv + m->q_rows; qa.v = m->qkv + m->q_rows + m->kv_rows;
        qa.q_norm = ly.q_norm; qa.k_norm = ly.k_norm; qa.cos_t = m->cos_t; qa.sin_t = m->sin_t;
        qa.kc = ly.kv->k; qa.vc = ly.kv->v; qa.pos = &m->st->pos; qa.pos_shared = 1;
        qa.batch = 1; qa.n_heads = m->nh_loc; qa.n_kv = m->nkv_loc; qa.hd = m->hd; qa.kv_dtype = cf.kv_dtype;
        qa.eps = 1e-6f;                                    // the reference hard-codes 1e-6 here (:850,853)
        STEP_LAUNCH(CLS_QKPREP, 4.0 * (2 * m->q_rows + 2 * m->kv_rows) + (double)2 * m->kv_rows * (cf.kv_dtype == ATLASX_BF16 ? 2 : 4),
                    ax_qk_prep_launch(c, qa, P(CLS_QKPREP)));

        // ── attention over the cache ────────────────────────────────────────────
        AxAttnArgs aa;
        aa.q = m->qkv; aa.kc = ly.kv->k; aa.vc = ly.kv->v; aa.out = m->attn;
        aa.pos = &m->st->pos; aa.pos_shared = 1; aa.batch = 1;
        aa.n_heads = m->nh_loc; aa.n_kv = m->nkv_loc; aa.hd = m->hd; aa.window = ly.window;
        aa.kv_dtype = cf.kv_dtype; aa.scale = m->scale; aa.n_splits = m->attn_splits;
        aa.scratch_partials = m->attn_partials; aa.scratch_tickets = m->attn_tickets;
        STEP_LAUNCH(CLS_ATTN, abytes, ax_attn_launch(c, aa, P(CLS_ATTN)));
        }

        // ── output projection (row-parallel under TP) ───────────────────────────
        AxPrologue po; po.base = m->attn;
        if (mail) {
            const AxPeerOut px = peer_out(0, l);
            STEP_LAUNCH(CLS_OPROJ, gemv_bytes(ly.wo), ax_gemv_launch(c, ly.wo, po, AX_EPI_PLAIN, 1, m->o, P(CLS_OPROJ), &px));
            if (m->mail_mode == 1)
                STEP_LAUNCH(CLS_COMM, 8.0 * d * mail->world, ax_mail_reduce_launch(c, mail->part(mail->rank, 0, 0), mail->world, (size_t)mail->d, d,
                                                                                   mail->useq, 1u, (unsigned)l + 1u, m->o, P(CLS_COMM)));
        } else {
            STEP_LAUNCH(CLS_OPROJ, gemv_bytes(ly.wo), ax_gemv_launch(c, ly.wo, po, AX_EPI_PLAIN, 1, m->o, P(CLS_OPROJ)));
            if (m->world > 1) STEP_LAUNCH(CLS_COMM, 4.0 * d, ax_comm_allreduce_sum(c, m->o, (size_t)d));
        }

        // ── gate/up with SwiGLU epilogue ────────────────────────────────────────
        AxPrologue pg;
        pg.eps = cf.rms_norm_eps;
        pg.base = l == 0 ? m->resid[0] : m->taps + (size_t)(l - 1) * d; pg.y = m->o; pg.nparts = nparts; pg.part_stride = d;
        if (mail) peer_in(pg, 0, l);
        pg.base_early = 1;                                 // written by the QKV launch, at least two kernels back
        if (post) pg.wy = ly.attn_norm; else pg.wx = ly.ffn_norm;
        pg.resid_out = m->resid[1];
        STEP_LAUNCH(CLS_GATEUP, gemv_bytes(ly.gateup), ax_gemv_launch(c, ly.gateup, pg, AX_EPI_SILU_PAIR, 1, m->h, P(CLS_GATEUP)));

        // ── down projection (row-parallel under TP) ─────────────────────────────
        AxPrologue pd; pd.base = m->h;
        if (mail) {
            const AxPeerOut px = peer_out(1, l);
            STEP_LAUNCH(CLS_DOWN, gemv_bytes(ly.down), ax_gemv_launch(c, ly.down, pd, AX_EPI_PLAIN, 1, m->dn, P(CLS_DOWN), &px));
            if (m->mail_mode == 1)
                STEP_LAUNCH(CLS_COMM, 8.0 * d * mail->world, ax_mail_reduce_launch(c, mail->part(mail->rank, 1, 0), mail->world, (size_t)mail->d, d,
                                                                                   mail->useq, 1u, (unsigned)l + 1u, m->dn, P(CLS_COMM)));
        } else {
            STEP_LAUNCH(CLS_DOWN, gemv_bytes(ly.down), ax_gemv_launch(c, ly.down, pd, AX_EPI_PLAIN, 1, m->dn, P(CLS_DOWN)));
            if (m->world > 1) STEP_LAUNCH(CLS_COMM, 4.0 * d, ax_comm_allreduce_sum(c, m->dn, (size_t)d));
        }
    }
    // ── final norm + lm_head ────────────────────────────────────────────────────
    AxPrologue pl;
    pl.eps = cf.rms_norm_eps;
    pl.base = m->resid[1]; pl.y = m->dn; pl.nparts = nparts; pl.part_stride = d;
    if (mail) peer_in(pl, 1, L - 1);
    pl.base_early = 1;
    if (post) pl.wy = m->layers[L - 1].ffn_norm;
    pl.wx = m->final_norm;
    pl.resid_out = m->taps + (size_t)(L - 1) * d;
    STEP_LAUNCH(CLS_LMHEAD, gemv_bytes(m->lm_head), ax_gemv_launch(c, m->lm_head, pl, AX_EPI_PLAIN, 1, m->logits_loc, P(CLS_LMHEAD)));
    const bool local_select = m->world > 1 && m->tp_select && mail && !gather;
    if (m->world > 1 && !local_select)
        STEP_LAUNCH(CLS_COMM, 4.0 * m->vocab_loc * m->world, ax_comm_allgather(c, m->logits_loc, m->logits, (size_t)m->vocab_loc));

    // ── greedy selection + state advance ────────────────────────────────────────
    if ((m->class_mask >> CLS_SELECT) & 1) {
        AxArgmaxScratch sc = { c->amax_vals, c->amax_idx, c->amax_ticket };
        int n = cf.vocab_size;
        const float* sel_from = m->logits;
        SelPeers sp;
        if (local_select) {
            sp.n = mail->world; sp.rank = mail->rank; sp.index_base = m->rank * m->vocab_loc; sp.vocab = cf.vocab_size; sp.err = c->dev_error;
            for (int q = 0; q < mail->world; q++) sp.dst[q] = mail->sel(q, mail->rank);
            sp.mine = mail->sel(mail->rank, 0);
            sel_from = m->logits_loc;
            n = cf.vocab_size - sp.index_base; n = n > m->vocab_loc ? m->vocab_loc : (n < 0 ? 0 : n);   // this rank's rows (none past the vocabulary)
        }
        if (prof) cudaEventRecord(prof->ev[2 * prof->n], s);
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)((n + 1023) / 1024 > 0 ? (n + 1023) / 1024 : 1)); cfg.blockDim = dim3(256); cfg.stream = s;
        cudaLaunchAttribute attr[1];
        if (pdl) { attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization; attr[0].val.programmaticStreamSerializationAllowed = 1; cfg.attrs = attr; cfg.numAttrs = 1; }
        AX_CUDA(cudaLaunchKernelEx(&cfg, select_advance_k, sel_from, n, sc, m->st, m->seq, cf.max_seq_len + 1, advance ? 1 : 0,
                                   mail ? mail->useq : (unsigned*)nullptr, (unsigned)L, sp));
        if (prof) { cudaEventRecord(prof->ev[2 * prof->n + 1], s); prof->cls[prof->n] = CLS_SELECT; prof->bytes[prof->n] = 4.0 * n; prof->n++; }
        n_launch++;
    }
    m->launches_per_step = n_launch;
    return ATLASX_OK;
}

constexpr int kPrefillMax = 128;               // tokens per chunk with the tcgen05 kernel and bf16 weights; 64 with int8 weights;
constexpr int kPrefillMaxMma = 16;             // 16 with the warp-level kernel
constexpr int kAttnChunk = 128;                // tokens per launch of the chunk attention (one launch per chunk: 16520 tok/s against 16430 with two of 64)

// ── prompt ingestion: row-wise helpers, one CTA per token ───────────────────────────
// Every kernel of a chunk starts with griddepcontrol.wait, so each may be launched with programmatic stream
// serialization: it becomes resident while its predecessor drains and touches memory only after that one is complete.
__global__ void pf_positions_k(const StepState* st, int* pos_arr, int n) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if ((int)threadIdx.x < n) pos_arr[threadIdx.x] = st->pos + threadIdx.x;
}
__global__ void pf_embed_rows_k(const void* embed, int bf16, int vocab, const int* seq, const int* pos_arr, int d, float* out) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int i = blockIdx.x;
    long long tok = seq[pos_arr[i]];
    if (tok < 0) tok = 0;
    if (tok > vocab - 1) tok = vocab - 1;
    for (int k = threadIdx.x; k < d; k += blockDim.x)
        out[(size_t)i * d + k] = bf16 ? ax_bf16_to_f32(((const uint16_t*)embed)[(size_t)tok * d + k]) : ((const float*)embed)[(size_t)tok * d + k];
}
__device__ __forceinline__ float pf_block_sum(float v, float* red) {
    v = ax_warp_sum(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = 0.f;
    for (int w = 0; w < (int)(blockDim.x >> 5); w++) t += red[w];
    return t;
}
// The fused prologue of the GEMVs, row by row:  v = base + (wy ? rmsnorm(y, wy) : y);  resid = v;
// x = wx ? rmsnorm(v, wx) : v.   y may be null (v = base).  resid may alias base, x may alias resid.
// plane (may be null): the bf16 hi|lo plane the tcgen05 product of the NEXT projection reads — row i the hi parts of
// token i's x, row n8 + i the lo parts; CTAs n..n8−1 only clear their two rows.  With a plane x is not written.
__device__ __forceinline__ void pf_plane_store(uint16_t* plane, int n8, int d, int row, int k, float v) {
    const uint16_t h = ax_f32_to_bf16_rne(v);
    plane[(size_t)row * d + k] = h;
    plane[(size_t)(n8 + row) * d + k] = ax_f32_to_bf16_rne(v - ax_bf16_to_f32(h));
}
// yp pending: y is not read; its elements are the sums of the partial tiles of the product before (same order as its merge kernel).
__global__ void __launch_bounds__(1024) pf_rows_norm_add_k(const float* y, const float* base, const float* wy, const float* wx, float eps,
                                                           int d, float* resid, float* x, uint16_t* plane, int n8, int n, AxUmmaParts yp) {
    __shared__ float red[32];
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int nt = blockDim.x;
    if ((int)blockIdx.x >= n) {                                  // padding rows of the plane
        for (int k = threadIdx.x; k < d; k += nt) { plane[(size_t)blockIdx.x * d + k] = 0; plane[(size_t)(n8 + blockIdx.x) * d + k] = 0; }
        return;
    }
    const size_t o = (size_t)blockIdx.x * d;
    const bool parts = yp.pending();
    auto y_at = [&](int k) { return parts ? yp.at((int)blockIdx.x, k) : y[o + k]; };
    // the first kKeep elements a thread reads of y stay in registers between the two passes (all of them up to d = 8192)
    constexpr int kKeep = 8;
    float yk[kKeep];
    float inv_y = 1.f;
    if (y && wy) {
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < kKeep; i++) { const int k = threadIdx.x + i * nt; if (k < d) { yk[i] = y_at(k); ss = fmaf(yk[i], yk[i], ss); } }
        for (int k = threadIdx.x + kKeep * nt; k < d; k += nt) { const float t = y_at(k); ss = fmaf(t, t, ss); }
        inv_y = 1.0f / sqrtf(pf_block_sum(ss, red) / (float)d + eps);
    } else if (y) {
#pragma unroll
        for (int i = 0; i < kKeep; i++) { const int k = threadIdx.x + i * nt; if (k < d) yk[i] = y_at(k); }
    }
    float ss2 = 0.f;
#pragma unroll
    for (int i = 0; i < kKeep; i++) {
        const int k = threadIdx.x + i * nt;
        if (k < d) {
            float v = base[o + k];
            if (y) { float t = yk[i]; if (wy) t = t * inv_y * wy[k]; v += t; }
            resid[o + k] = v;
            ss2 = fmaf(v, v, ss2);
        }
    }
    for (int k = threadIdx.x + kKeep * nt; k < d; k += nt) {
        float v = base[o + k];
        if (y) { float t = y_at(k); if (wy) t = t * inv_y * wy[k]; v += t; }
        resid[o + k] = v;
        ss2 = fmaf(v, v, ss2);
    }
    if (wx) {
        const float inv_x = 1.0f / sqrtf(pf_block_sum(ss2, red) / (float)d + eps);
        for (int k = threadIdx.x; k < d; k += nt) {
            const float v = resid[o + k] * inv_x * wx[k];
            if (plane) pf_plane_store(plane, n8, d, (int)blockIdx.x, k, v); else x[o + k] = v;
        }
    } else if (plane) {
        for (int k = threadIdx.x; k < d; k += nt) pf_plane_store(plane, n8, d, (int)blockIdx.x, k, resid[o + k]);
    } else if (x != resid) {
        for (int k = threadIdx.x; k < d; k += nt) x[o + k] = resid[o + k];
    }
}
// gate/up rows are interleaved (even: gate, odd: up): out[i][j] = silu(gu[i][2j]) · gu[i][2j+1]
__global__ void pf_silu_pair_rows_k(const float* gu, int f, float* out, uint16_t* plane, int n8, int n, AxUmmaParts gp) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const size_t i = blockIdx.y;
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= f) return;
    if ((int)i >= n) { plane[i * (size_t)f + j] = 0; plane[(n8 + i) * (size_t)f + j] = 0; return; }       // padding rows of the plane
    const float2 v = gp.pending() ? make_float2(gp.at((int)i, 2 * j), gp.at((int)i, 2 * j + 1))
                                  : reinterpret_cast<const float2*>(gu + i * 2 * (size_t)f)[j];
    const float r = (v.x / (1.0f + expf(-v.x))) * v.y;
    if (plane) pf_plane_store(plane, n8, f, (int)i, j, r); else out[i * (size_t)f + j] = r;
}
__global__ void pf_advance_k(StepState* st, int by) { st->pos += by; }

// Largest chunk the layer products of this model can take: kPrefillMax when every matrix goes through the
// tcgen05 kernel, kPrefillMaxMma when some need the warp-level one, 1 when neither covers a matrix.
int prefill_limit(const atlasx_model* m) {
    if (m->cfg.weight_format == ATLASX_F32) return 1;
    alignas(16) static float dummy[4];
    int limit = kPrefillMax;
    for (const Layer& ly : m->layers) {
        const AxWeight* ws[4] = { &ly.qkv, &ly.wo, &ly.gateup, &ly.down };
        for (const AxWeight* w : ws) {
            if (m->ctx->tune.umma && ax_gemv_umma_supported(*w, 2, dummy, dummy)) {
                while (limit > 2 && !ax_gemv_umma_supported(*w, limit, dummy, dummy)) limit /= 2;      // 128 → 64 with int8 weights
                continue;
            }
            if (!ax_gemv_mma_supported(*w, 2, dummy, dummy)) return 1;
            if (m->ctx->tune.umma && ax_gemv_umma_int4_supported(*w, limit, dummy, dummy)) continue;      // int4: expanded, then the bf16 product
            if (limit > kPrefillMaxMma) limit = kPrefillMaxMma;
        }
    }
    return limit;
}
// One layer product of a chunk: X [n][cols] → Y [n][rows]
// x == nullptr: the kernel before left the token plane of this product in place (ax_gemv_umma_plane)
// ext_parts + pend: where the product splits K, its partial tiles stay in ext_parts for the next kernel to add up
int pf_product(atlasx_ctx* c, const AxWeight& w, const float* x, int n, float* y, bool pdl, float* ext_parts = nullptr, AxUmmaParts* pend = nullptr) {
    if (pend) *pend = AxUmmaParts();
    if (!ext_parts) pend = nullptr;
    if (!x) return ax_gemv_umma_launch(c, w, nullptr, n, y, true, pdl, ext_parts, pend);
    if (c->tune.umma && ax_gemv_umma_supported(w, n, x, y)) return ax_gemv_umma_launch(c, w, x, n, y, true, pdl, ext_parts, pend);
    if (ax_gemv_mma_supported(w, n, x, y)) return ax_gemv_mma_launch(c, w, x, n, y, true);
    return ax_gemv_umma_int4_launch(c, w, x, n, y, true, pdl);
}

// Launch with programmatic stream serialization (the kernel waits for its predecessor itself).
template <typename... KArgs, typename... Args>
int pf_launch(cudaStream_t s, bool pdl, void (*kernel)(KArgs...), dim3 grid, dim3 block, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.stream = s;
    cudaLaunchAttribute attr[1];
    if (pdl) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr; cfg.numAttrs = 1;
    }
    AX_CUDA(cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...));
    return ATLASX_OK;
}

// n prompt tokens (2..kPrefillMax) at once: seq[pos .. pos+n) → caches, logits of the last one,
// selection, pos += n.  Same arithmetic as n single steps (crates/atlas-model/src/lib.rs:1611-1618
// feeds the prompt token by token); the weights stream once per chunk instead of once per token.
int run_prefill_chunk(atlasx_model* m, int n) {
    atlasx_ctx* c = m->ctx;
    cudaStream_t s = c->stream;
    const atlasx_model_config& cf = m->cfg;
    const int d = cf.d_model, L = cf.n_layers;
    const bool post = cf.post_norm != 0;
    const int qkv_rows = m->q_rows + 2 * m->kv_rows;
    int rc;
    const bool pdl = m->use_pdl != 0;
    if ((rc = pf_launch(s, false, pf_positions_k, dim3(1), dim3(kPrefillMax), (const StepState*)m->st, m->pf_pos, n))) return rc;
    if ((rc = pf_launch(s, pdl, pf_embed_rows_k, dim3((unsigned)n), dim3(256), (const void*)m->embed, (int)m->embed_bf16, cf.vocab_size,
                        (const int*)m->seq, (const int*)m->pf_pos, d, m->pf_r))) return rc;
    // Where the next product runs on the tcgen05 kernel with bf16 weights, the kernel that makes its input writes the
    // bf16 hi|lo token plane itself (no split launch): the plane's address and row count, or null.
    auto plane_for = [&](const AxWeight& w, uint16_t** pl, int* n8) {
        *pl = nullptr; *n8 = 0;
        return (c->tune.umma && c->tune.umma_fused) ? ax_gemv_umma_plane(c, w, n, pl, n8) : ATLASX_OK;
    };
    uint16_t* tpl = nullptr; int n8 = 0;
    const float* a_in = m->pf_r;
    if (!post) {
        if ((rc = plane_for(m->layers[0].qkv, &tpl, &n8))) return rc;
        if ((rc = pf_launch(s, pdl, pf_rows_norm_add_k, dim3((unsigned)(tpl ? n8 : n)), dim3(1024), (const float*)nullptr, (const float*)m->pf_r, (const float*)nullptr,
                            (const float*)m->layers[0].attn_norm, cf.rms_norm_eps, d, m->pf_r, m->pf_a, tpl, n8, n, AxUmmaParts()))) return rc;
        a_in = tpl ? nullptr : m->pf_a;
    }
    for (int l = 0; l < L; l++) {
        Layer& ly = m->layers[l];
        uint16_t* att_pl = nullptr;
        if ((rc = pf_product(c, ly.qkv, a_in, n, m->pf_qkv, pdl))) return rc;
        if (m->pf_attn_splits > 0) {
            // QK-norm, RoPE and cache write of all n tokens at once, then ONE causal attention launch
            AxQkPrepArgs qa;
            qa.q = m->pf_qkv; qa.k = m->pf_qkv + m->q_rows; qa.v = m->pf_qkv + m->q_rows + m->kv_rows;
            qa.q_norm = ly.q_norm; qa.k_norm = ly.k_norm; qa.cos_t = m->cos_t; qa.sin_t = m->sin_t;
            qa.kc = ly.kv->k; qa.vc = ly.kv->v; qa.seq_stride = 0;
            qa.pos = m->pf_pos; qa.pos_shared = 0; qa.batch = n;
            qa.n_heads = m->nh_loc; qa.n_kv = m->nkv_loc; qa.hd = m->hd; qa.kv_dtype = cf.kv_dtype; qa.eps = 1e-6f;
            qa.q_stride = (size_t)qkv_rows; qa.kv_in_stride = (size_t)qkv_rows;
            if ((rc = ax_qk_prep_launch(c, qa, pdl))) return rc;
            // causal attention of the chunk: one launch per kAttnChunk tokens (all K/V rows of the chunk are in the cache;
            // a token sees the rows up to its own position).  It writes o_proj's token plane itself where the chunk
            // fills the plane's rows (no padding rows to clear).
            if (n % 8 == 0 && (rc = plane_for(ly.wo, &att_pl, &n8))) return rc;
            for (int t0 = 0; t0 < n; t0 += kAttnChunk) {
                const int nt = n - t0 < kAttnChunk ? n - t0 : kAttnChunk;
                AxAttnChunkArgs ca;
                ca.q = m->pf_qkv + (size_t)t0 * qkv_rows; ca.q_stride = (size_t)qkv_rows; ca.kc = ly.kv->k; ca.vc = ly.kv->v;
                ca.out = m->pf_att + (size_t)t0 * m->q_rows; ca.out_stride = (size_t)m->q_rows; ca.pos0 = m->pf_pos + t0;
                ca.n_tok = nt; ca.n_heads = m->nh_loc; ca.n_kv = m->nkv_loc; ca.window = ly.window;
                {   // splits for the rows these tokens really see in this layer (the position is known on the host)
                    int rows_seen = m->host_pos + t0 + nt;
                    if (ly.window > 0 && rows_seen > ly.window + nt) rows_seen = ly.window + nt;
                    ca.n_splits = ax_attn_mma_chunk_splits(c, m->nh_loc, m->nkv_loc, nt, rows_seen);
                    if (ca.n_splits > m->pf_attn_splits) ca.n_splits = m->pf_attn_splits;
                }
                ca.scale = m->scale; ca.partials = m->pf_attn_partials; ca.tickets = m->pf_attn_tickets;
                ca.out_plane = att_pl ? att_pl + (size_t)t0 * m->q_rows : nullptr; ca.plane_rows = n8;
                if ((rc = ax_attn_mma_chunk_launch(c, ca, pdl))) return rc;
            }
        } else
        for (int i = 0; i < n; i++) {
            float* qkv = m->pf_qkv + (size_t)i * qkv_rows;
            float* out = m->pf_att + (size_t)i * m->q_rows;
            if (m->fused_attn) {
                AxFusedAttnArgs fa;
                fa.qkv = qkv; fa.q_norm = ly.q_norm; fa.k_norm = ly.k_norm; fa.cos_t = m->cos_t; fa.sin_t = m->sin_t;
                fa.kc = ly.kv->k; fa.vc = ly.kv->v; fa.out = out; fa.pos = m->pf_pos + i;
                fa.n_heads = m->nh_loc; fa.n_kv = m->nkv_loc; fa.window = ly.window; fa.kv_dtype = cf.kv_dtype;
                fa.max_splits = m->fused_splits; fa.scale = m->scale; fa.qk_eps = 1e-6f;
                fa.scratch_partials = m->attn_partials; fa.scratch_tickets = m->attn_tickets;
                if ((rc = ax_attn_fused_launch(c, fa, false))) return rc;
            } else {
                AxQkPrepArgs qa;
                qa.q = qkv; qa.k = qkv + m->q_rows; qa.v = qkv + m->q_rows + m->kv_rows;
                qa.q_norm = ly.q_norm; qa.k_norm = ly.k_norm; qa.cos_t = m->cos_t; qa.sin_t = m->sin_t;
                qa.kc = ly.kv->k; qa.vc = ly.kv->v; qa.pos = m->pf_pos + i; qa.pos_shared = 1;
                qa.batch = 1; qa.n_heads = m->nh_loc; qa.n_kv = m->nkv_loc; qa.hd = m->hd; qa.kv_dtype = cf.kv_dtype; qa.eps = 1e-6f;
                if ((rc = ax_qk_prep_launch(c, qa, false))) return rc;
                AxAttnArgs aa;
                aa.q = qkv; aa.kc = ly.kv->k; aa.vc = ly.kv->v; aa.out = out;
                aa.pos = m->pf_pos + i; aa.pos_shared = 1; aa.batch = 1;
                aa.n_heads = m->nh_loc; aa.n_kv = m->nkv_loc; aa.hd = m->hd; aa.window = ly.window;
                aa.kv_dtype = cf.kv_dtype; aa.scale = m->scale; aa.n_splits = m->attn_splits;
                aa.scratch_partials = m->attn_partials; aa.scratch_tickets = m->attn_tickets;
                if ((rc = ax_attn_launch(c, aa, false))) return rc;
            }
        }
        const bool after_nccl = m->world > 1;             // an NCCL kernel in front: plain stream order
        float* own_parts = after_nccl ? nullptr : m->pf_parts;         // the all-reduce wants the finished vector
        AxUmmaParts yp;
        if ((rc = pf_product(c, ly.wo, att_pl ? nullptr : m->pf_att, n, m->pf_o, pdl, own_parts, &yp))) return rc;
        if (m->world > 1 && (rc = ax_comm_allreduce_sum(c, m->pf_o, (size_t)n * d))) return rc;
        if ((rc = plane_for(ly.gateup, &tpl, &n8))) return rc;
        if ((rc = pf_launch(s, pdl && !after_nccl, pf_rows_norm_add_k, dim3((unsigned)(tpl ? n8 : n)), dim3(1024), (const float*)m->pf_o, (const float*)m->pf_r,
                            (const float*)(post ? ly.attn_norm : nullptr), (const float*)(post ? nullptr : ly.ffn_norm),
                            cf.rms_norm_eps, d, m->pf_r, m->pf_a, tpl, n8, n, yp))) return rc;
        AxUmmaParts gp;
        if ((rc = pf_product(c, ly.gateup, tpl ? nullptr : m->pf_a, n, m->pf_gu, pdl, m->pf_parts, &gp))) return rc;
        if ((rc = plane_for(ly.down, &tpl, &n8))) return rc;
        if ((rc = pf_launch(s, pdl, pf_silu_pair_rows_k, dim3((unsigned)((m->ffn_loc + 255) / 256), (unsigned)(tpl ? n8 : n)), dim3(256),
                            (const float*)m->pf_gu, m->ffn_loc, m->pf_h, tpl, n8, n, gp))) return rc;
        if ((rc = pf_product(c, ly.down, tpl ? nullptr : m->pf_h, n, m->pf_dn, pdl, own_parts, &yp))) return rc;
        if (m->world > 1 && (rc = ax_comm_allreduce_sum(c, m->pf_dn, (size_t)n * d))) return rc;
        const float* next_wx = (post || l == L - 1) ? nullptr : m->layers[l + 1].attn_norm;
        tpl = nullptr; n8 = 0;
        if (l + 1 < L && (rc = plane_for(m->layers[l + 1].qkv, &tpl, &n8))) return rc;
        if ((rc = pf_launch(s, pdl && !after_nccl, pf_rows_norm_add_k, dim3((unsigned)(tpl ? n8 : n)), dim3(1024), (const float*)m->pf_dn, (const float*)m->pf_r,
                            (const float*)(post ? ly.ffn_norm : nullptr), next_wx, cf.rms_norm_eps, d, m->pf_r, m->pf_a, tpl, n8, n, yp))) return rc;
        a_in = tpl ? nullptr : m->pf_a;
    }
    AX_CHECK_LAUNCH("prefill chunk");
    // logits of the chunk's last token through the single-column path, then selection
    AxPrologue pl;
    pl.eps = cf.rms_norm_eps;
    pl.base = m->pf_r + (size_t)(n - 1) * d;
    pl.wx = m->final_norm;
    pl.resid_out = m->taps + (size_t)(L - 1) * d;
    if ((rc = ax_gemv_launch(c, m->lm_head, pl, AX_EPI_PLAIN, 1, m->logits_loc, false))) return rc;
    if (m->world > 1 && (rc = ax_comm_allgather(c, m->logits_loc, m->logits, (size_t)m->vocab_loc))) return rc;
    pf_advance_k<<<1, 1, 0, s>>>(m->st, n - 1);
    AxArgmaxScratch sc = { c->amax_vals, c->amax_idx, c->amax_ticket };
    // the chunk used NCCL, not the mailboxes: the use counter stays where it is
    select_advance_k<<<(cf.vocab_size + 1023) / 1024, 256, 0, s>>>(m->logits, cf.vocab_size, sc, m->st, m->seq, cf.max_seq_len + 1, 1, nullptr, 0u, SelPeers());
    AX_CHECK_LAUNCH("prefill selection");
    m->host_pos += n;
    return ATLASX_OK;
}

int capture_one(atlasx_model* m, bool gather, cudaGraphExec_t* out);
int capture_graph(atlasx_model* m) {
    if (m->graph) { cudaGraphExecDestroy(m->graph); m->graph = nullptr; }
    if (m->graph_tok) { cudaGraphExecDestroy(m->graph_tok); m->graph_tok = nullptr; }
    int rc = capture_one(m, true, &m->graph);
    if (!rc && m->world > 1 && m->tp_select && m->mail) rc = capture_one(m, false, &m->graph_tok);
    return rc;
}
int capture_one(atlasx_model* m, bool gather, cudaGraphExec_t* out) {
    atlasx_ctx* c = m->ctx;
    cudaGraph_t g = nullptr;
    if (c->tune.step_trace && !m->step_trace) {
        int r0 = dmalloc(m, (void**)&m->step_trace, 1024 * sizeof(AxTraceSlot));
        if (r0) return r0;
    }
    AX_CUDA(cudaStreamBeginCapture(c->stream, cudaStreamCaptureModeThreadLocal));
    c->trace_next = m->step_trace;
    int rc = run_step(m, nullptr, true, gather);
    if (m->step_trace) { m->step_trace_slots = (int)((c->trace_next - m->step_trace) / 6); c->trace_next = nullptr; }
    cudaError_t e = cudaStreamEndCapture(c->stream, &g);
    if (rc) { if (g) cudaGraphDestroy(g); return rc; }
    if (e != cudaSuccess) return atlasx_fail(ATLASX_ERR_CUDA, "stream capture failed: %s", cudaGetErrorString(e));
    e = cudaGraphInstantiate(out, g, 0);
    cudaGraphDestroy(g);
    if (e != cudaSuccess) { *out = nullptr; return atlasx_fail(ATLASX_ERR_CUDA, "graph instantiation failed: %s", cudaGetErrorString(e)); }
    return ATLASX_OK;
}

// need_logits = false: the caller only wants the token (tensor parallel: no logits all-gather)
int step(atlasx_model* m, bool need_logits = true) {
    if (m->host_pos >= m->cfg.max_seq_len)
        return atlasx_fail(ATLASX_ERR_STATE, "position %d is past max_seq_len %d", m->host_pos, m->cfg.max_seq_len);
    int rc;
    const bool tok_only = !need_logits && m->world > 1 && m->tp_select && m->mail;
    if (m->use_graph && m->graph) { AX_CUDA(cudaGraphLaunch(tok_only && m->graph_tok ? m->graph_tok : m->graph, m->ctx->stream)); rc = ATLASX_OK; }
    else rc = run_step(m, nullptr, true, !tok_only);
    if (!rc) m->host_pos++;
    return rc;
}

// ── per-layer hook ───────────────────────────────────────────────────────────────────
// Runs the hook over the layer outputs of the forward whose taps were copied into host buffer k
// (the reference's accumulate, crates/atlas-infer/src/hook.rs:60-67: negative deltas count as 0).
int run_hooks(atlasx_model* m, int k) {
    AX_CUDA(cudaEventSynchronize(m->tap_ev[k]));
    const int L = m->cfg.n_layers, d = m->cfg.d_model;
    float acc = 0.f; uint32_t fired = 0;
    for (int l = 0; l < L; l++) {
        float delta = 0.f;
        if (m->hook_fn(m->hook_user, l, m->tap_host[k] + (size_t)l * d, d, &delta)) { acc += delta > 0.f ? delta : 0.f; fired++; }
    }
    if (m->tap_tok[k] >= 0) { m->dep_tok.push_back((uint32_t)m->tap_tok[k]); m->dep_delta.push_back(acc); m->dep_fired.push_back(fired); }
    return ATLASX_OK;
}
// One forward inside generate: the step, then — with a hook attached — the copy of its layer outputs
// to the host, and the hook calls of the PREVIOUS forward while this one runs on the GPU.
// tok: the generated token this forward processes (−1 for a prompt token: hook results are dropped).
int gen_step(atlasx_model* m, long long tok, bool need_logits = true) {
    int rc = step(m, need_logits);
    if (rc || !m->hook_fn) return rc;
    const int k = m->tap_k;
    AX_CUDA(cudaMemcpyAsync(m->tap_host[k], m->taps, (size_t)m->cfg.n_layers * m->cfg.d_model * 4, cudaMemcpyDeviceToHost, m->ctx->stream));
    AX_CUDA(cudaEventRecord(m->tap_ev[k], m->ctx->stream));
    m->tap_tok[k] = tok;
    if (m->tap_pending && (rc = run_hooks(m, k ^ 1))) return rc;
    m->tap_pending = true; m->tap_k = k ^ 1;
    return ATLASX_OK;
}
int flush_hooks(atlasx_model* m) {
    if (!m->hook_fn || !m->tap_pending) return ATLASX_OK;
    m->tap_pending = false;
    return run_hooks(m, m->tap_k ^ 1);
}

}  // namespace

// StigmergicHook on the GPU path (crates/atlas-infer/src/hook.rs:31-33; the reference runs hooked
// generation on its CPU model, engine.rs:144-162).  fn = NULL detaches.
// generate_streaming (crates/atlas-model/src/lib.rs:1855-1965): fn is called with every token right after it is
// emitted (EOS and stop tokens end the run before, unseen); a zero return ends the generation there.
extern "C" int atlasx_model_set_token_callback(atlasx_model* m, atlasx_token_callback fn, void* user) {
    AX_ARG(m, "model is null");
    m->tok_fn = fn; m->tok_user = user;
    return ATLASX_OK;
}
extern "C" int atlasx_model_set_layer_hook(atlasx_model* m, atlasx_layer_hook fn, void* user) {
    AX_ARG(m && m->finalized, "model is not finalised");
    AX_CUDA(cudaStreamSynchronize(m->ctx->stream));
    m->hook_fn = fn; m->hook_user = user; m->tap_pending = false; m->tap_k = 0;
    if (fn && !m->tap_host[0]) {
        const size_t bytes = (size_t)m->cfg.n_layers * m->cfg.d_model * 4;
        for (int k = 0; k < 2; k++) {
            AX_CUDA(cudaMallocHost((void**)&m->tap_host[k], bytes));
            AX_CUDA(cudaEventCreateWithFlags(&m->tap_ev[k], cudaEventDisableTiming));
        }
    }
    return ATLASX_OK;
}
extern "C" int atlasx_model_deposits(atlasx_model* m, uint32_t* token_ids, float* total_delta, uint32_t* layers_fired, int cap, int* n) {
    AX_ARG(m && n, "null argument");
    const int have = (int)m->dep_tok.size();
    *n = have;
    for (int i = 0; i < have && i < cap; i++) {
        if (token_ids) token_ids[i] = m->dep_tok[(size_t)i];
        if (total_delta) total_delta[i] = m->dep_delta[(size_t)i];
        if (layers_fired) layers_fired[i] = m->dep_fired[(size_t)i];
    }
    return ATLASX_OK;
}
extern "C" int atlasx_model_layer_hidden(atlasx_model* m, int layer, float* hidden_host) {
    AX_ARG(m && m->finalized && hidden_host && layer >= 0 && layer < m->cfg.n_layers, "bad argument");
    AX_CUDA(cudaMemcpyAsync(hidden_host, m->taps + (size_t)layer * m->cfg.d_model, (size_t)m->cfg.d_model * 4, cudaMemcpyDeviceToHost, m->ctx->stream));
    AX_CUDA(cudaStreamSynchronize(m->ctx->stream));
    return ATLASX_OK;
}

extern "C" const char* atlasx_model_class_name(int cls) { return (cls >= 0 && cls < CLS_COUNT) ? kClassNames[cls] : ""; }

extern "C" int atlasx_model_create(atlasx_ctx* ctx, const atlasx_model_config* cfg, const int* layer_sliding, atlasx_model** out) {
    AX_ARG(ctx && cfg && out, "null argument");
    AX_ARG(cfg->n_layers > 0 && cfg->d_model > 0 && cfg->n_heads > 0 && cfg->n_kv_heads > 0 && cfg->ffn_hidden > 0 &&
           cfg->vocab_size > 0 && cfg->max_seq_len > 0, "dimensions must be positive");
    AX_ARG(cfg->d_model % cfg->n_heads == 0 && cfg->n_heads % cfg->n_kv_heads == 0, "head counts do not divide");
    AX_ARG(cfg->kv_dtype == ATLASX_BF16 || cfg->kv_dtype == ATLASX_F32, "kv_dtype must be bf16 or f32");
    AX_ARG(cfg->weight_format >= ATLASX_F32 && cfg->weight_format <= ATLASX_INT4, "unknown weight_format (ATLASX_AUTO is for the loaders)");
    const int world = cfg->tp_world > 0 ? cfg->tp_world : 1;
    AX_ARG(cfg->tp_rank >= 0 && cfg->tp_rank < world, "tp_rank out of range");
    AX_ARG(cfg->n_heads % world == 0 && cfg->n_kv_heads % world == 0 && cfg->ffn_hidden % world == 0,
           "heads, kv heads and ffn_hidden must divide by the tensor-parallel degree");
    AX_ARG(world == ax_comm_world(ctx), "tp_world does not match the context's communicator");
    const int hd = cfg->d_model / cfg->n_heads;
    const int epc = cfg->weight_format == ATLASX_F32 ? 4 : cfg->weight_format == ATLASX_BF16 ? 8 : cfg->weight_format == ATLASX_INT8 ? 16 : 32;
    AX_ARG(cfg->d_model % 32 == 0 && (cfg->ffn_hidden / world) % epc == 0 && ((cfg->n_heads / world) * hd) % epc == 0,
           "d_model must be a multiple of 32 and the sharded inner dimensions multiples of the 16-byte weight granule");
    if (cfg->weight_format == ATLASX_INT4) {
        AX_ARG(cfg->int4_block >= 32 && cfg->int4_block % 32 == 0, "int4_block must be a multiple of 32");
        AX_ARG(cfg->d_model % cfg->int4_block == 0 && (cfg->ffn_hidden / world) % cfg->int4_block == 0 &&
               ((cfg->n_heads / world) * hd) % cfg->int4_block == 0, "int4 blocks must not straddle rows or shards");
    }
    atlasx_model* m = new atlasx_model();
    m->ctx = ctx; m->cfg = *cfg; m->cfg.tp_world = world;
    m->world = world; m->rank = cfg->tp_rank;
    m->hd = hd; m->nh_loc = cfg->n_heads / world; m->nkv_loc = cfg->n_kv_heads / world; m->ffn_loc = cfg->ffn_hidden / world;
    m->vocab_loc = (cfg->vocab_size + world - 1) / world;
    m->q_rows = m->nh_loc * hd; m->kv_rows = m->nkv_loc * hd;
    // OlmoModel::new (:1331-1335): scale × attn_factor when it differs from 1 by more than 1e-6
    m->scale = 1.0f / sqrtf((float)hd);
    const float af = cfg->rope_scaling == 1 ? cfg->yarn_attn_factor : 1.0f;
    if (fabsf(af - 1.0f) > 1e-6f) m->scale *= af;
    m->layers.resize(cfg->n_layers);
    int rc = ATLASX_OK;
    const int d = cfg->d_model;
    for (int l = 0; l < cfg->n_layers && !rc; l++) {
        Layer& ly = m->layers[l];
        ly.window = (layer_sliding && layer_sliding[l]) ? cfg->sliding_window : 0;
        rc = alloc_weight(m, ly.qkv, m->q_rows + 2 * m->kv_rows, d);
        if (!rc) rc = alloc_weight(m, ly.wo, d, m->q_rows);
        if (!rc) rc = alloc_weight(m, ly.gateup, 2 * m->ffn_loc, d);
        if (!rc) rc = alloc_weight(m, ly.down, d, m->ffn_loc);
    }
    if (!rc) rc = alloc_weight(m, m->lm_head, m->vocab_loc, d);
    if (rc) { atlasx_model_free(m); return rc; }
    *out = m;
    return ATLASX_OK;
}

extern "C" int atlasx_model_free(atlasx_model* m) {
    if (!m) return ATLASX_OK;
    cudaStreamSynchronize(m->ctx->stream);
    if (m->graph) cudaGraphExecDestroy(m->graph);
    if (m->graph_tok) cudaGraphExecDestroy(m->graph_tok);
    for (Layer& ly : m->layers) if (ly.kv) atlasx_kvcache_free(ly.kv);
    for (void* p : m->owned) cudaFree(p);
    for (int k = 0; k < 2; k++) { if (m->tap_host[k]) cudaFreeHost(m->tap_host[k]); if (m->tap_ev[k]) cudaEventDestroy(m->tap_ev[k]); }
    if (m->pin) cudaFreeHost(m->pin);
    if (m->pin_logits) cudaFreeHost(m->pin_logits);
    delete m;
    return ATLASX_OK;
}

static int set_vector(atlasx_model* m, float** dst, const void* src_dev, int dtype, int first, int n) {
    if (!*dst) { int rc = dmalloc(m, (void**)dst, (size_t)n * 4); if (rc) return rc; }
    if (dtype == ATLASX_BF16) ax_bf16_to_f32(m->ctx->stream, (const uint16_t*)src_dev + first, *dst, (size_t)n);
    else AX_CUDA(cudaMemcpyAsync(*dst, (const float*)src_dev + first, (size_t)n * 4, cudaMemcpyDeviceToDevice, m->ctx->stream));
    return ATLASX_OK;
}

namespace {
// Shape of the full tensor `which` and the part [r0,r0+nr) × [c0,c0+nc) of it this tensor-parallel
// rank keeps.  whole = 1 when the rank must be handed the full tensor all the same: replicated
// tensors, and int8 weights that are split by columns (their per-row scale is the maximum over the
// FULL row, so the row has to be quantised before it is cut).
struct TensorPart { int rows = 0, cols = 0, r0 = 0, nr = 0, c0 = 0, nc = 0, whole = 1; };
int tensor_part(const atlasx_model* m, int which, TensorPart* tp) {
    const atlasx_model_config& cf = m->cfg;
    const int d = cf.d_model, hd = m->hd, r = m->rank;
    TensorPart t;
    auto rows_of = [&](int rows, int cols, int r0, int nr) { t.rows = rows; t.cols = cols; t.r0 = r0; t.nr = nr; t.c0 = 0; t.nc = cols; t.whole = m->world == 1; };
    auto cols_of = [&](int rows, int cols, int c0, int nc) {
        t.rows = rows; t.cols = cols; t.r0 = 0; t.nr = rows; t.c0 = c0; t.nc = nc;
        t.whole = m->world == 1 || cf.weight_format == ATLASX_INT8;
    };
    auto all_of = [&](int rows, int cols) { t.rows = rows; t.cols = cols; t.r0 = 0; t.nr = rows; t.c0 = 0; t.nc = cols; t.whole = 1; };
    switch (which) {
        case ATLASX_T_EMBED: all_of(cf.vocab_size, d); break;
        case ATLASX_T_LM_HEAD: {
            const int r0 = r * m->vocab_loc < cf.vocab_size ? r * m->vocab_loc : cf.vocab_size;
            int nr = cf.vocab_size - r0; if (nr > m->vocab_loc) nr = m->vocab_loc;
            rows_of(cf.vocab_size, d, r0, nr); break;
        }
        case ATLASX_T_FINAL_NORM: case ATLASX_T_ATTN_NORM: case ATLASX_T_FFN_NORM: all_of(1, d); break;
        case ATLASX_T_WQ: rows_of(cf.n_heads * hd, d, r * m->q_rows, m->q_rows); break;
        case ATLASX_T_WK: case ATLASX_T_WV: rows_of(cf.n_kv_heads * hd, d, r * m->kv_rows, m->kv_rows); break;
        case ATLASX_T_WO: cols_of(d, cf.n_heads * hd, r * m->q_rows, m->q_rows); break;
        case ATLASX_T_GATE: case ATLASX_T_UP: rows_of(cf.ffn_hidden, d, r * m->ffn_loc, m->ffn_loc); break;
        case ATLASX_T_DOWN: cols_of(d, cf.ffn_hidden, r * m->ffn_loc, m->ffn_loc); break;
        case ATLASX_T_Q_NORM: all_of(1, cf.n_heads * hd); break;                    // small: given whole, the slice is cut on the device
        case ATLASX_T_K_NORM: all_of(1, cf.n_kv_heads * hd); break;
        default: return atlasx_fail(ATLASX_ERR_ARG, "unknown tensor id %d", which);
    }
    *tp = t;
    return ATLASX_OK;
}

// is_part: `data` holds exactly the part tensor_part() names (row-major nr × nc) instead of the full tensor.
int set_tensor_impl(atlasx_model* m, int layer, int which, const void* data, int dtype, int on_device, bool is_part) {
    AX_ARG(m && data, "null argument");
    AX_ARG(dtype == ATLASX_F32 || dtype == ATLASX_BF16, "tensors are given as f32 or bf16");
    AX_ARG(!m->finalized, "model already finalised");
    const atlasx_model_config& cf = m->cfg;
    const int d = cf.d_model;
    TensorPart tp;
    int rc = tensor_part(m, which, &tp);
    if (rc) return rc;
    if (which >= ATLASX_T_WQ) AX_ARG(layer >= 0 && layer < cf.n_layers, "layer out of range");
    if (tp.whole) is_part = false;
    // the tensor as handed over: the full one, or the rank's part standing in for it
    const int rows = is_part ? tp.nr : tp.rows, cols = is_part ? tp.nc : tp.cols;
    const int r0 = is_part ? 0 : tp.r0, c0 = is_part ? 0 : tp.c0;
    const size_t n = (size_t)rows * cols, esz = dtype == ATLASX_BF16 ? 2 : 4;
    cudaStream_t s = m->ctx->stream;
    void* staged = nullptr;
    const void* src = data;
    if (!on_device) {
        AX_CUDA(cudaMalloc(&staged, n * esz ? n * esz : 16));
        cudaError_t e = cudaMemcpyAsync(staged, data, n * esz, cudaMemcpyHostToDevice, s);
        if (e == cudaSuccess) e = cudaStreamSynchronize(s);
        if (e != cudaSuccess) { cudaFree(staged); return atlasx_fail(ATLASX_ERR_CUDA, "upload failed: %s", cudaGetErrorString(e)); }
        src = staged;
    }
    const int r = m->rank;
    Layer* ly = which >= ATLASX_T_WQ ? &m->layers[layer] : nullptr;
    switch (which) {
        case ATLASX_T_EMBED: {
            // replicated; kept in the precision it was given in (bf16 rows are exact in f32)
            if (!m->embed || m->embed_bf16 != (dtype == ATLASX_BF16)) { rc = dmalloc(m, &m->embed, n * esz); }
            if (!rc) { m->embed_bf16 = dtype == ATLASX_BF16; cudaMemcpyAsync(m->embed, src, n * esz, cudaMemcpyDeviceToDevice, s); m->have_embed = true; }
            break;
        }
        case ATLASX_T_LM_HEAD:
            if (tp.nr > 0) rc = place_slice(m, src, dtype, rows, cols, r0, tp.nr, 0, d, m->lm_head, 0, 1);
            m->have_lm_head = true;
            break;
        case ATLASX_T_FINAL_NORM: rc = set_vector(m, &m->final_norm, src, dtype, 0, d); break;
        case ATLASX_T_ATTN_NORM: rc = set_vector(m, &ly->attn_norm, src, dtype, 0, d); break;
        case ATLASX_T_FFN_NORM: rc = set_vector(m, &ly->ffn_norm, src, dtype, 0, d); break;
        case ATLASX_T_Q_NORM: rc = set_vector(m, &ly->q_norm, src, dtype, r * m->q_rows, m->q_rows); break;
        case ATLASX_T_K_NORM: rc = set_vector(m, &ly->k_norm, src, dtype, r * m->kv_rows, m->kv_rows); break;
        case ATLASX_T_WQ: rc = place_slice(m, src, dtype, rows, cols, r0, tp.nr, 0, d, ly->qkv, 0, 1); break;
        case ATLASX_T_WK: rc = place_slice(m, src, dtype, rows, cols, r0, tp.nr, 0, d, ly->qkv, m->q_rows, 1); break;
        case ATLASX_T_WV: rc = place_slice(m, src, dtype, rows, cols, r0, tp.nr, 0, d, ly->qkv, m->q_rows + m->kv_rows, 1); break;
        case ATLASX_T_WO: rc = place_slice(m, src, dtype, rows, cols, 0, d, c0, tp.nc, ly->wo, 0, 1); break;
        case ATLASX_T_GATE: rc = place_slice(m, src, dtype, rows, cols, r0, tp.nr, 0, d, ly->gateup, 0, 2); break;
        case ATLASX_T_UP: rc = place_slice(m, src, dtype, rows, cols, r0, tp.nr, 0, d, ly->gateup, 1, 2); break;
        case ATLASX_T_DOWN: rc = place_slice(m, src, dtype, rows, cols, 0, d, c0, tp.nc, ly->down, 0, 1); break;
    }
    if (ly && !rc) ly->have[which - ATLASX_T_WQ] = true;
    cudaStreamSynchronize(s);
    cudaFree(staged);
    return rc;
}
}  // namespace

extern "C" int atlasx_model_set_tensor(atlasx_model* m, int layer, int which, const void* data, int dtype, int on_device) {
    return set_tensor_impl(m, layer, which, data, dtype, on_device, false);
}
extern "C" int atlasx_model_set_tensor_slice(atlasx_model* m, int layer, int which, const void* data, int dtype, int on_device) {
    return set_tensor_impl(m, layer, which, data, dtype, on_device, true);
}
extern "C" int atlasx_model_tensor_slice(const atlasx_model* m, int which, size_t* full_rows, size_t* full_cols,
                                         size_t* r0, size_t* r1, size_t* c0, size_t* c1, int* whole) {
    AX_ARG(m, "model is null");
    TensorPart tp;
    int rc = tensor_part(m, which, &tp);
    if (rc) return rc;
    if (full_rows) *full_rows = (size_t)tp.rows;
    if (full_cols) *full_cols = (size_t)tp.cols;
    // what the caller has to hand over: the kept part, or everything
    if (r0) *r0 = tp.whole ? 0 : (size_t)tp.r0;
    if (r1) *r1 = tp.whole ? (size_t)tp.rows : (size_t)(tp.r0 + tp.nr);
    if (c0) *c0 = tp.whole ? 0 : (size_t)tp.c0;
    if (c1) *c1 = tp.whole ? (size_t)tp.cols : (size_t)(tp.c0 + tp.nc);
    if (whole) *whole = tp.whole;
    return ATLASX_OK;
}

extern "C" int atlasx_model_finalize(atlasx_model* m) {
    AX_ARG(m, "model is null");
    AX_ARG(!m->finalized, "model already finalised");
    const atlasx_model_config& cf = m->cfg;
    atlasx_ctx* c = m->ctx;
    cudaStream_t s = c->stream;
    const int d = cf.d_model;
    AX_ARG(m->have_embed, "embedding table was not set");
    for (int l = 0; l < cf.n_layers; l++)
        for (int t = ATLASX_T_WQ; t <= ATLASX_T_DOWN; t++)
            if (!m->layers[l].have[t - ATLASX_T_WQ]) return atlasx_fail(ATLASX_ERR_STATE, "layer %d: tensor %d was not set", l, t);
    int rc = ATLASX_OK;
    // unit norm weights where none were loaded (TransformerBlock::new, :950-951; OlmoModel::new :1344)
    std::vector<float> ones((size_t)d, 1.0f);
    float* ones_dev = nullptr;
    if ((rc = dmalloc(m, (void**)&ones_dev, (size_t)d * 4))) return rc;
    AX_CUDA(cudaMemcpyAsync(ones_dev, ones.data(), (size_t)d * 4, cudaMemcpyHostToDevice, s));
    AX_CUDA(cudaStreamSynchronize(s));
    if (!m->final_norm) m->final_norm = ones_dev;
    for (Layer& ly : m->layers) { if (!ly.attn_norm) ly.attn_norm = ones_dev; if (!ly.ffn_norm) ly.ffn_norm = ones_dev; }
    // weight tying: lm_head is a copy of the embedding when none was given (:1345-1350)
    if (!m->have_lm_head) {
        const int r0 = m->rank * m->vocab_loc;
        int nr = cf.vocab_size - r0; if (nr > m->vocab_loc) nr = m->vocab_loc;
        if (nr > 0) rc = place_slice(m, m->embed, m->embed_bf16 ? ATLASX_BF16 : ATLASX_F32, cf.vocab_size, d, r0, nr, 0, d, m->lm_head, 0, 1);
        if (rc) return rc;
        m->have_lm_head = true;
    }
    // RoPE tables (init_gpu_resources, :1363-1376)
    const int half = m->hd / 2;
    std::vector<float> ch((size_t)cf.max_seq_len * (half > 0 ? half : 1)), sh(ch.size());
    rc = atlasx_rope_tables_host(m->hd, cf.max_seq_len, cf.rope_theta, cf.rope_scaling, cf.yarn_factor, cf.yarn_orig_max_pos,
                                 cf.yarn_beta_fast, cf.yarn_beta_slow, ch.data(), sh.data());
    if (rc) return rc;
    if ((rc = dmalloc(m, (void**)&m->cos_t, ch.size() * 4))) return rc;
    if ((rc = dmalloc(m, (void**)&m->sin_t, ch.size() * 4))) return rc;
    AX_CUDA(cudaMemcpyAsync(m->cos_t, ch.data(), ch.size() * 4, cudaMemcpyHostToDevice, s));
    AX_CUDA(cudaMemcpyAsync(m->sin_t, sh.data(), sh.size() * 4, cudaMemcpyHostToDevice, s));
    AX_CUDA(cudaStreamSynchronize(s));
    // KV caches (:1381-1385)
    for (Layer& ly : m->layers)
        if ((rc = atlasx_kvcache_create(c, cf.max_seq_len, m->nkv_loc, m->hd, cf.kv_dtype, 1, &ly.kv))) return rc;
    // activations
    const size_t vocab_pad = (size_t)m->vocab_loc * m->world;
    if ((rc = dmalloc(m, (void**)&m->resid[0], (size_t)d * 4))) return rc;
    if ((rc = dmalloc(m, (void**)&m->resid[1], (size_t)d * 4))) return rc;
    if ((rc = dmalloc(m, (void**)&m->taps, (size_t)cf.n_layers * d * 4))) return rc;
    if ((rc = dmalloc(m, (void**)&m->qkv, (size_t)(m->q_rows + 2 * m->kv_rows) * 4))) return rc;
    if ((rc = dmalloc(m, (void**)&m->attn, (size_t)m->q_rows * 4))) return rc;
    if ((rc = dmalloc(m, (void**)&m->o, (size_t)d * 4))) return rc;
    if ((rc = dmalloc(m, (void**)&m->h, (size_t)m->ffn_loc * 4))) return rc;
    if ((rc = dmalloc(m, (void**)&m->dn, (size_t)d * 4))) return rc;
    if ((rc = dmalloc(m, (void**)&m->logits, vocab_pad * 4))) return rc;
    if (m->world > 1) { if ((rc = dmalloc(m, (void**)&m->logits_loc, (size_t)m->vocab_loc * 4))) return rc; }
    else m->logits_loc = m->logits;
    if ((rc = dmalloc(m, (void**)&m->seq, (size_t)(cf.max_seq_len + 1) * 4))) return rc;
    if ((rc = dmalloc(m, (void**)&m->st, sizeof(StepState)))) return rc;
    AX_CUDA(cudaMemsetAsync(m->seq, 0, (size_t)(cf.max_seq_len + 1) * 4, s));
    AX_CUDA(cudaMemsetAsync(m->st, 0, sizeof(StepState), s));
    AX_CUDA(cudaMemsetAsync(m->logits, 0, vocab_pad * 4, s));
    AX_CUDA(cudaMallocHost((void**)&m->pin, 64 * sizeof(int)));
    // attention split count fixed for the graph; scratch sized once
    int max_rows = cf.max_seq_len;
    m->attn_splits = ax_attn_pick_splits(c, m->nkv_loc, 1, max_rows);
    m->fused_attn = ax_attn_fused_supported(m->hd, m->nh_loc, m->nkv_loc) && c->tune.attn_fused != 0;
    m->fused_splits = ax_attn_fused_max_splits(c, m->nkv_loc, max_rows);
    const int scratch_splits = m->fused_attn && m->fused_splits > m->attn_splits ? m->fused_splits : m->attn_splits;
    // the model's own scratch: its captured graph holds these pointers, so they must not move when
    // another model or an operator call on the same context needs more
    if ((rc = dmalloc(m, (void**)&m->attn_partials, (size_t)m->nh_loc * scratch_splits * (m->hd + 2) * 4))) return rc;
    if ((rc = dmalloc(m, (void**)&m->attn_tickets, (size_t)m->nh_loc * sizeof(unsigned)))) return rc;
    AX_CUDA(cudaMemsetAsync(m->attn_tickets, 0, (size_t)m->nh_loc * sizeof(unsigned), s));
    AX_ARG(cf.vocab_size <= 4096 * 1024, "vocabulary too large for the selection scratch");
    m->finalized = true;
    m->host_pos = 0;
    set_state_k<<<1, 1, 0, s>>>(m->st, 0, INT_MAX);
    AX_CUDA(cudaStreamSynchronize(s));
    if (m->world > 1) {
        // collective: every rank finalises its model at the same point of the program.  The small
        // all-reduce afterwards lines the ranks up, so that the bounded waits of the first step
        // measure the step and not the difference in set-up time.
        rc = ax_comm_peer_setup(c, d, &m->mail); if (rc) return rc;
        // every consumer CTA polling every part costs world × 8·d bytes of L2 reads per CTA; one more
        // small launch per use is cheaper already with two ranks (466 against 462 tok/s)
        if (m->mail) {
            m->mail_mode = (c->tune.mail_reduce >= 0 && c->tune.mail_reduce <= 2) ? c->tune.mail_reduce : 2;
            for (int b = 0; b < 2; b++) {
                if ((rc = dmalloc(m, (void**)&m->mail_red[b], (size_t)d * sizeof(uint2)))) return rc;
                AX_CUDA(cudaMemsetAsync(m->mail_red[b], 0, (size_t)d * sizeof(uint2), s));
            }
            m->tp_select = c->tune.tp_select != 0;
        }
        AX_CUDA(cudaMemsetAsync(m->o, 0, (size_t)d * 4, s));
        rc = ax_comm_allreduce_sum(c, m->o, (size_t)d); if (rc) return rc;
        AX_CUDA(cudaStreamSynchronize(s));
    }
    // one eager step loads every kernel before capture; it only touches cache row 0, which the
    // first real token rewrites
    rc = run_step(m, nullptr, true); if (rc) return rc;
    set_state_k<<<1, 1, 0, s>>>(m->st, 0, INT_MAX);
    {
        cudaError_t e = cudaStreamSynchronize(s);
        if (e != cudaSuccess) return atlasx_fail(ATLASX_ERR_CUDA, "first decode step failed: %s", cudaGetErrorString(e));
        int code = 0;
        rc = atlasx_ctx_poll_device_error(c, &code); if (rc) return rc;
    }
    if (m->use_graph) { rc = capture_graph(m); if (rc) return rc; }
    return ATLASX_OK;
}

// Prompt tokens are ingested `chunk` at a time (2..128) through the multi-column kernels; 0 or 1
// restores the token-by-token path.  Returns the chunk size in effect through *effective: at most 16
// when a matrix needs the warp-level kernel (int8 / int4 weights), 1 when the weight format or a
// matrix shape is outside what the multi-column kernels cover.
extern "C" int atlasx_model_set_prefill(atlasx_model* m, int chunk, int* effective) {
    AX_ARG(m && m->finalized, "model is not finalised");
    AX_ARG(chunk >= 0 && chunk <= kPrefillMax, "chunk must be in 0..128");
    int eff = chunk < 2 ? 1 : chunk;
    if (eff > 1) { const int lim = prefill_limit(m); if (eff > lim) eff = lim; }
    if (eff > 1 && !m->pf_r) {
        const size_t P = kPrefillMax;
        const int d = m->cfg.d_model, qkv_rows = m->q_rows + 2 * m->kv_rows;
        int rc;
        if ((rc = dmalloc(m, (void**)&m->pf_r, P * d * 4)) || (rc = dmalloc(m, (void**)&m->pf_a, P * d * 4)) ||
            (rc = dmalloc(m, (void**)&m->pf_qkv, P * qkv_rows * 4)) || (rc = dmalloc(m, (void**)&m->pf_att, P * m->q_rows * 4)) ||
            (rc = dmalloc(m, (void**)&m->pf_o, P * d * 4)) || (rc = dmalloc(m, (void**)&m->pf_gu, P * 2 * (size_t)m->ffn_loc * 4)) ||
            (rc = dmalloc(m, (void**)&m->pf_h, P * (size_t)m->ffn_loc * 4)) || (rc = dmalloc(m, (void**)&m->pf_dn, P * d * 4)) ||
            (rc = dmalloc(m, (void**)&m->pf_pos, P * sizeof(int)))) return rc;
        // scratch of the multi-column kernel for the largest of the layer's products
        size_t need = 0;
        for (const Layer& ly : m->layers) {
            const AxWeight* ws[4] = { &ly.qkv, &ly.wo, &ly.gateup, &ly.down };
            for (const AxWeight* w : ws) {
                size_t b = ax_gemv_mma_scratch_bytes(w->rows, w->cols); if (b > need) need = b;
                if (w->dtype == ATLASX_BF16 || w->dtype == ATLASX_INT8)
                    for (int n = 2; n <= kPrefillMax; n++) { b = ax_gemv_umma_scratch_bytes(m->ctx, *w, n); if (b > need) need = b; }
            }
        }
        rc = atlasx_ctx_ensure_split_scratch(m->ctx, need);
        if (rc) return rc;
        // o_proj, gate/up and down leave the partial tiles of a K split to the row-wise kernel behind them
        if (m->ctx->tune.umma && m->ctx->tune.umma_fused == 1) {
            alignas(16) static float dummy[4];
            size_t pb = 0;
            for (const Layer& ly : m->layers) {
                const AxWeight* ws[3] = { &ly.wo, &ly.gateup, &ly.down };
                for (const AxWeight* w : ws)
                    for (int n = 2; n <= kPrefillMax; n++)
                        if (ax_gemv_umma_supported(*w, n, dummy, dummy)) { const size_t b = ax_gemv_umma_parts_bytes(m->ctx, *w, n); if (b > pb) pb = b; }
            }
            if (pb && (rc = dmalloc(m, (void**)&m->pf_parts, pb))) return rc;
        }
        if (m->cfg.kv_dtype == ATLASX_BF16 && ax_attn_mma_chunk_supported(m->hd, m->nh_loc, m->nkv_loc, m->cfg.kv_dtype)) {
            const int A = kPrefillMax;
            m->pf_attn_splits = ax_attn_mma_chunk_max_splits();      // scratch for the largest split count; each chunk picks its own
            if ((rc = dmalloc(m, (void**)&m->pf_attn_partials, ax_attn_mma_chunk_partial_floats(A, m->nh_loc, m->pf_attn_splits) * 4)) ||
                (rc = dmalloc(m, (void**)&m->pf_attn_tickets, (size_t)m->nkv_loc * A * sizeof(unsigned)))) return rc;
            AX_CUDA(cudaMemsetAsync(m->pf_attn_tickets, 0, (size_t)m->nkv_loc * A * sizeof(unsigned), m->ctx->stream));
        }
    }
    m->prefill_chunk = eff;
    if (effective) *effective = eff;
    return ATLASX_OK;
}

// Debug aid: runs one captured step and returns, per traced launch, six %globaltimer stamps (ns):
// first/last CTA start, first dependency release, last CTA end, first CTA end, last input staged.  Needs ATLASX_STEP_TRACE
// set when the graph was captured.
extern "C" int atlasx_model_step_trace(atlasx_model* m, unsigned long long* out, int cap, int* n_slots) {
    AX_ARG(m && out && n_slots, "null argument");
    AX_ARG(m->step_trace && m->graph && m->step_trace_slots > 0, "no traced graph");
    const int n = m->step_trace_slots < cap ? m->step_trace_slots : cap;
    std::vector<unsigned long long> init((size_t)m->step_trace_slots * 6);
    for (int i = 0; i < m->step_trace_slots; i++) {
        unsigned long long* q = &init[(size_t)i * 6];
        q[0] = ~0ull; q[1] = 0; q[2] = ~0ull; q[3] = 0; q[4] = ~0ull; q[5] = 0;
    }
    AX_CUDA(cudaMemcpyAsync(m->step_trace, init.data(), init.size() * 8, cudaMemcpyHostToDevice, m->ctx->stream));
    AX_CUDA(cudaStreamSynchronize(m->ctx->stream));
    int rc = step(m);
    if (rc) return rc;
    AX_CUDA(cudaStreamSynchronize(m->ctx->stream));
    AX_CUDA(cudaMemcpy(out, m->step_trace, (size_t)n * 6 * 8, cudaMemcpyDeviceToHost));
    *n_slots = n;
    return ATLASX_OK;
}

extern "C" int atlasx_model_set_options(atlasx_model* m, int use_graph, int use_pdl) {
    AX_ARG(m, "model is null");
    const bool changed = m->use_pdl != (use_pdl ? 1 : 0) || m->use_graph != (use_graph ? 1 : 0);
    m->use_graph = use_graph ? 1 : 0; m->use_pdl = use_pdl ? 1 : 0;
    if (m->finalized && changed) {
        AX_CUDA(cudaStreamSynchronize(m->ctx->stream));
        if (m->graph) { cudaGraphExecDestroy(m->graph); m->graph = nullptr; }
        if (m->graph_tok) { cudaGraphExecDestroy(m->graph_tok); m->graph_tok = nullptr; }
        if (m->use_graph) return capture_graph(m);
    }
    return ATLASX_OK;
}

// reset (:1389-1392): position back to zero, caches are not cleared
extern "C" int atlasx_model_reset(atlasx_model* m) {
    AX_ARG(m && m->finalized, "model is not finalised");
    m->host_pos = 0;
    set_state_k<<<1, 1, 0, m->ctx->stream>>>(m->st, 0, INT_MAX);
    AX_CHECK_LAUNCH("set_state");
    // arrival counters are zero between launches; a launch that gave up on a bounded wait may have left some counted
    if (m->attn_tickets) AX_CUDA(cudaMemsetAsync(m->attn_tickets, 0, (size_t)m->nh_loc * sizeof(unsigned), m->ctx->stream));
    if (m->pf_attn_tickets)
        AX_CUDA(cudaMemsetAsync(m->pf_attn_tickets, 0, (size_t)m->nkv_loc * kPrefillMax * sizeof(unsigned), m->ctx->stream));
    return ATLASX_OK;
}
extern "C" int atlasx_model_pos(const atlasx_model* m) { return m ? m->host_pos : -1; }

// Bounded device-side waits (peer mailbox polls, bulk-copy barriers) that gave up set the context's
// error word and let the step run on with whatever was in memory.  The entry points that hand
// results to the host fetch the word beside their own read-back (queue_wait_status before the
// host synchronisation, wait_status after it) and fail with ATLASX_ERR_TIMEOUT instead of returning
// such results.  The word stays set — every later call fails too — until the caller clears it with
// atlasx_ctx_poll_device_error.
static int queue_wait_status(atlasx_model* m) {
    AX_CUDA(cudaMemcpyAsync(m->pin + 1, m->ctx->dev_error, sizeof(int), cudaMemcpyDeviceToHost, m->ctx->stream));
    return ATLASX_OK;
}
static int wait_status(const atlasx_model* m) {
    const int code = m->pin[1];
    return code ? atlasx_fail(ATLASX_ERR_TIMEOUT, "a bounded device-side wait expired during the step (code %d): results are not valid; "
                                                  "clear with atlasx_ctx_poll_device_error", code) : ATLASX_OK;
}

extern "C" int atlasx_model_forward_one(atlasx_model* m, uint32_t token, float* logits_host) {
    AX_ARG(m && m->finalized, "model is not finalised");
    cudaStream_t s = m->ctx->stream;
    AX_ARG(m->host_pos < m->cfg.max_seq_len, "position is past max_seq_len");
    m->pin[0] = (int)token;
    AX_CUDA(cudaMemcpyAsync(m->seq + m->host_pos, m->pin, 4, cudaMemcpyHostToDevice, s));
    set_state_k<<<1, 1, 0, s>>>(m->st, m->host_pos, INT_MAX);
    int rc = step(m, logits_host != nullptr); if (rc) return rc;
    if (m->hook_fn) {                     // forward_one_gpu_hooked (:1524-1557): the hook sees every layer's output of this token
        m->tap_pending = false;
        AX_CUDA(cudaMemcpyAsync(m->tap_host[0], m->taps, (size_t)m->cfg.n_layers * m->cfg.d_model * 4, cudaMemcpyDeviceToHost, s));
        AX_CUDA(cudaEventRecord(m->tap_ev[0], s));
        m->tap_tok[0] = -1;
        if ((rc = run_hooks(m, 0))) return rc;
    }
    if ((rc = queue_wait_status(m))) return rc;
    if (logits_host) {
        // through pinned memory: a copy into pageable memory is staged by the driver in small pieces
        const size_t bytes = (size_t)m->cfg.vocab_size * 4;
        if (!m->pin_logits) AX_CUDA(cudaMallocHost((void**)&m->pin_logits, bytes));
        AX_CUDA(cudaMemcpyAsync(m->pin_logits, m->logits, bytes, cudaMemcpyDeviceToHost, s));
        if ((rc = ax_comm_stream_sync(m->ctx))) return rc;
        if ((rc = wait_status(m))) return rc;
        memcpy(logits_host, m->pin_logits, bytes);
        return ATLASX_OK;
    }
    if ((rc = ax_comm_stream_sync(m->ctx))) return rc;
    return wait_status(m);
}

extern "C" int atlasx_model_hidden(atlasx_model* m, float* hidden_host) {
    AX_ARG(m && m->finalized && hidden_host, "bad argument");
    AX_CUDA(cudaMemcpyAsync(hidden_host, m->taps + (size_t)(m->cfg.n_layers - 1) * m->cfg.d_model, (size_t)m->cfg.d_model * 4,
                            cudaMemcpyDeviceToHost, m->ctx->stream));
    AX_CUDA(cudaStreamSynchronize(m->ctx->stream));
    return ATLASX_OK;
}

extern "C" int atlasx_model_generate_greedy(atlasx_model* m, const uint32_t* prompt, int n_prompt, int max_new,
                                            const uint32_t* suppress, int n_suppress, float rep_penalty, int rep_window,
                                            const uint32_t* stops, int n_stops, uint32_t* out_tokens, int* n_out) {
    AX_ARG(m && m->finalized && n_out, "bad argument");
    AX_ARG(n_prompt >= 0 && max_new >= 0 && (n_prompt == 0 || prompt) && (max_new == 0 || out_tokens), "bad argument");
    AX_ARG(n_prompt + max_new <= m->cfg.max_seq_len, "prompt + max_new exceeds max_seq_len");
    atlasx_ctx* c = m->ctx;
    cudaStream_t s = c->stream;
    const int V = m->cfg.vocab_size;
    *n_out = 0;
    int rc = atlasx_model_reset(m); if (rc) return rc;
    m->dep_tok.clear(); m->dep_delta.clear(); m->dep_fired.clear(); m->tap_pending = false;
    if (n_prompt > 0) AX_CUDA(cudaMemcpyAsync(m->seq, prompt, (size_t)n_prompt * 4, cudaMemcpyHostToDevice, s));
    set_state_k<<<1, 1, 0, s>>>(m->st, 0, n_prompt);
    struct DevInts {                    // freed on every way out, after the stream has drained
        int* p = nullptr; cudaStream_t s;
        ~DevInts() { if (p) { cudaStreamSynchronize(s); cudaFree(p); } }
    } sup_guard;
    sup_guard.s = s;
    const bool fix = n_suppress > 0 || rep_penalty != 1.0f;
    const bool need_logits = fix || n_prompt == 0;     // logit edits work on the full vector: every step all-gathers it under tensor parallelism
    if (n_suppress > 0) {
        AX_CUDA(cudaMalloc((void**)&sup_guard.p, (size_t)n_suppress * 4));
        AX_CUDA(cudaMemcpyAsync(sup_guard.p, suppress, (size_t)n_suppress * 4, cudaMemcpyHostToDevice, s));
    }
    int* const sup_dev = sup_guard.p;
    auto done = [&](int r) { cudaStreamSynchronize(s); const int rh = flush_hooks(m); return r ? r : rh; };
    if (n_prompt == 0) {
        // last_logits starts as zeros (:1609): the first choice is made among equal logits
        AX_CUDA(cudaMemsetAsync(m->logits, 0, (size_t)V * 4, s));
    }
    for (int i = 0; i < n_prompt;) {
        const int left = n_prompt - i;
        // with a hook every prompt token is a forward of its own: the hook sees each token's layers
        const int n = (m->prefill_chunk > 1 && left >= 2 && !m->hook_fn) ? (left < m->prefill_chunk ? left : m->prefill_chunk) : 1;
        rc = n > 1 ? run_prefill_chunk(m, n) : gen_step(m, -1, need_logits);
        if (rc) return done(rc);
        i += n;
    }
    AxArgmaxScratch sc = { c->amax_vals, c->amax_idx, c->amax_ticket };
    for (int stepi = 0; stepi < max_new; stepi++) {
        const bool need_fix = fix && ((stepi == 0 && n_suppress > 0) || (rep_penalty != 1.0f && stepi > 0));
        if (need_fix || (n_prompt == 0 && stepi == 0)) {
            // re-select on edited logits: history = generated tokens seq[n_prompt .. n_prompt+stepi)
            int start = stepi > rep_window ? stepi - rep_window : 0;
            if (need_fix)
                logit_fixups_k<<<1, 32, 0, s>>>(m->logits, V, sup_dev, stepi == 0 ? n_suppress : 0,
                                                m->seq + n_prompt + start, rep_penalty != 1.0f ? stepi - start : 0, rep_penalty);
            select_advance_k<<<(V + 1023) / 1024, 256, 0, s>>>(m->logits, V, sc, m->st, m->seq, m->cfg.max_seq_len + 1, 0, nullptr, 0u, SelPeers());
            cudaError_t e = cudaGetLastError();
            if (e != cudaSuccess) return done(atlasx_fail(ATLASX_ERR_CUDA, "selection launch failed: %s", cudaGetErrorString(e)));
        }
        AX_CUDA(cudaMemcpyAsync(m->pin, &m->st->last_token, 4, cudaMemcpyDeviceToHost, s));
        if ((rc = queue_wait_status(m))) return rc;
        if ((rc = ax_comm_stream_sync(c))) return rc;
        if ((rc = wait_status(m))) return rc;
        const uint32_t tok = (uint32_t)m->pin[0];
        if (m->cfg.eos_token_id >= 0 && tok == (uint32_t)m->cfg.eos_token_id) break;
        bool stop = false;
        for (int i = 0; i < n_stops; i++) if (stops[i] == tok) stop = true;
        if (stop) break;
        out_tokens[(*n_out)++] = tok;
        if (m->tok_fn && !m->tok_fn(m->tok_user, tok)) break;            // the caller has enough (:1958-1960): no forward for this token
        rc = gen_step(m, (long long)tok, need_logits); if (rc) return done(rc);
    }
    return done(ATLASX_OK);
}

// generate_with_sampling, sampling branch (:1599-1732): the prompt and every step run exactly as in
// the greedy call; between steps one launch of the sampling kernel picks the next token from the
// logits on the device (penalties, temperature, top-k, top-p, min-p, one XorShift64 draw) and makes
// it the input of the next position.  Per token only the 4-byte id crosses to the host (for the
// EOS / stop test).  temperature ≤ 0 takes the greedy call.
extern "C" int atlasx_model_generate_sampling(atlasx_model* m, const uint32_t* prompt, int n_prompt, int max_new,
                                              const atlasx_sampling_config* cfg, const uint32_t* suppress, int n_suppress,
                                              const uint32_t* stops, int n_stops, uint64_t seed, int seed_from_time,
                                              uint32_t* out_tokens, int* n_out) {
    AX_ARG(m && m->finalized && n_out && cfg, "bad argument");
    if (cfg->temperature <= 0.0f || cfg->temperature < 1e-6f)
        return atlasx_model_generate_greedy(m, prompt, n_prompt, max_new, suppress, n_suppress, cfg->repetition_penalty,
                                            cfg->repetition_window, stops, n_stops, out_tokens, n_out);
    AX_ARG(n_prompt >= 0 && max_new >= 0 && (n_prompt == 0 || prompt) && (max_new == 0 || out_tokens) && n_suppress >= 0, "bad argument");
    AX_ARG(n_prompt + max_new <= m->cfg.max_seq_len, "prompt + max_new exceeds max_seq_len");
    AX_ARG(cfg->repetition_window >= 0 && cfg->top_k >= 0, "repetition_window and top_k must not be negative");
    atlasx_ctx* c = m->ctx;
    cudaStream_t s = c->stream;
    const int V = m->cfg.vocab_size;
    *n_out = 0;
    int rc = atlasx_model_reset(m); if (rc) return rc;
    m->dep_tok.clear(); m->dep_delta.clear(); m->dep_fired.clear(); m->tap_pending = false;
    if ((rc = ax_sample_ensure_scratch(c, V))) return rc;
    AxSampleScratch& sc = c->sample;
    AX_ARG(n_suppress <= sc.list_cap, "suppress list too long");
    if ((rc = ax_sample_reset_counts(c, V))) return rc;
    if (n_suppress) AX_CUDA(cudaMemcpyAsync(sc.list, suppress, (size_t)n_suppress * 4, cudaMemcpyHostToDevice, s));
    // Rng::from_entropy (:1196-1203) or a fixed seed as Rng::from_seed (:1205-1207)
    unsigned long long state = seed | 1ull;
    if (seed_from_time) {
        struct timespec ts; clock_gettime(CLOCK_REALTIME, &ts);
        state = ((unsigned long long)ts.tv_sec * 1000000000ull + (unsigned long long)ts.tv_nsec) ^ 0x517cc1b727220a95ull;
    }
    AX_CUDA(cudaMemcpyAsync(sc.rng, &state, 8, cudaMemcpyHostToDevice, s));
    if (n_prompt > 0) AX_CUDA(cudaMemcpyAsync(m->seq, prompt, (size_t)n_prompt * 4, cudaMemcpyHostToDevice, s));
    set_state_k<<<1, 1, 0, s>>>(m->st, 0, n_prompt);
    AX_CUDA(cudaStreamSynchronize(s));                        // `state` and the caller's lists may go out of scope
    if (n_prompt == 0) AX_CUDA(cudaMemsetAsync(m->logits, 0, (size_t)V * 4, s));      // last_logits starts as zeros (:1609)
    for (int i = 0; i < n_prompt;) {
        const int left = n_prompt - i;
        const int n = (m->prefill_chunk > 1 && left >= 2 && !m->hook_fn) ? (left < m->prefill_chunk ? left : m->prefill_chunk) : 1;
        rc = n > 1 ? run_prefill_chunk(m, n) : gen_step(m, -1);
        if (rc) { cudaStreamSynchronize(s); return rc; }
        i += n;
    }
    AxSampleArgs a = {};
    a.logits = m->logits; a.n = V; a.cfg = ax_sampling_params(*cfg);
    a.suppress = sc.list; a.n_suppress = n_suppress;
    a.hist = nullptr; a.n_hist = 0; a.win_len = 0;
    a.work = sc.work; a.cval = sc.cval; a.cidx = sc.cidx; a.skey = sc.skey; a.sval = sc.sval;
    a.cnt_all = sc.cnt_all; a.cnt_win = sc.cnt_win; a.rng = sc.rng; a.token_out = sc.token; a.probs_out = nullptr;
    a.last_token = &m->st->last_token; a.seq = m->seq; a.pos = &m->st->pos; a.seq_cap = m->cfg.max_seq_len + 1;
    const int W = cfg->repetition_window;
    for (int stepi = 0; stepi < max_new; stepi++) {
        a.step = stepi;
        a.tok_in = stepi > 0 ? (int)out_tokens[stepi - 1] : -1;               // joins the history and the window …
        a.tok_out = stepi - 1 - W >= 0 ? (int)out_tokens[stepi - 1 - W] : -1;   // … whose oldest member leaves
        if ((rc = ax_sample_launch(c, a))) break;
        AX_CUDA(cudaMemcpyAsync(m->pin, sc.token, 4, cudaMemcpyDeviceToHost, s));
        if ((rc = queue_wait_status(m))) break;
        if ((rc = ax_comm_stream_sync(c))) break;
        if ((rc = wait_status(m))) break;
        const uint32_t tok = (uint32_t)m->pin[0];
        if (m->cfg.eos_token_id >= 0 && tok == (uint32_t)m->cfg.eos_token_id) break;
        bool stop = false;
        for (int i = 0; i < n_stops; i++) if (stops[i] == tok) stop = true;
        if (stop) break;
        out_tokens[(*n_out)++] = tok;
        if (m->tok_fn && !m->tok_fn(m->tok_user, tok)) break;
        if ((rc = gen_step(m, (long long)tok))) break;
    }
    cudaStreamSynchronize(s);
    const int rh = flush_hooks(m);
    return rc ? rc : rh;
}

extern "C" int atlasx_model_decode_timed(atlasx_model* m, int steps, int lead, float* elapsed_ms, uint32_t* tokens_host) {
    AX_ARG(m && m->finalized && steps > 0 && lead >= 0, "bad argument");
    AX_ARG(m->host_pos + lead + steps <= m->cfg.max_seq_len, "steps run past max_seq_len");
    cudaStream_t s = m->ctx->stream;
    const int p0 = m->host_pos;
    set_state_k<<<1, 1, 0, s>>>(m->st, p0, p0, m->seq);      // every token from here on is generated
    cudaEvent_t e0, e1;
    AX_CUDA(cudaEventCreate(&e0)); AX_CUDA(cudaEventCreate(&e1));
    AX_CUDA(cudaStreamSynchronize(s));
    int rc = ATLASX_OK;
    // untimed lead-in steps, queued without a host synchronisation before the first event: the ranks
    // of a tensor-parallel group leave them coupled through their mailboxes, so the timed region
    // starts at the same moment on every GPU however far apart the hosts got here
    for (int i = 0; i < lead && !rc; i++) rc = step(m, false);
    if (!rc) AX_CUDA(cudaEventRecord(e0, s));
    for (int i = 0; i < steps && !rc; i++) rc = step(m, false);
    cudaEventRecord(e1, s);
    const int rq = queue_wait_status(m);
    const int rs = ax_comm_stream_sync(m->ctx);
    cudaError_t e = rs ? cudaSuccess : cudaStreamSynchronize(s);
    float ms = 0.f;
    if (!rs) cudaEventElapsedTime(&ms, e0, e1);
    cudaEventDestroy(e0); cudaEventDestroy(e1);
    if (rs) return rs;
    if (rc) return rc;
    if (e != cudaSuccess) return atlasx_fail(ATLASX_ERR_CUDA, "decode failed: %s", cudaGetErrorString(e));
    if (rq) return rq;
    if ((rc = wait_status(m))) return rc;
    if (elapsed_ms) *elapsed_ms = ms;
    if (tokens_host) AX_CUDA(cudaMemcpy(tokens_host, m->seq + p0 + 1, (size_t)(lead + steps) * 4, cudaMemcpyDeviceToHost));
    return ATLASX_OK;
}

// Device time of one launch family inside the step's launch conditions: a graph holding only the
// launches of the classes in `mask` (bit = class index), in step order, with the same programmatic
// dependent launch attributes, replayed `iters` times between two CUDA events.  Nothing is selected
// and the position does not advance; activations are left meaningless until the next real step,
// which starts from the embedding again.  Single GPU only (peer mailboxes would wait for data).
extern "C" int atlasx_model_time_classes(atlasx_model* m, unsigned mask, int iters, float* ms_per_pass, double* bytes_per_pass, int* launches) {
    AX_ARG(m && m->finalized && iters > 0 && ms_per_pass, "bad argument");
    AX_ARG(m->world == 1, "single GPU only");
    atlasx_ctx* c = m->ctx;
    cudaStream_t s = c->stream;
    AX_CUDA(cudaStreamSynchronize(s));
    const int saved = m->class_mask, saved_launches = m->launches_per_step;
    m->class_mask = (int)(mask & ((1u << CLS_COUNT) - 1u)) & ~(1 << CLS_SELECT);
    // bytes and launch count of the family from one eager, profiled pass
    {
        const int cap = m->cfg.n_layers * 8 + 8;
        Profile pr;
        pr.ev.resize((size_t)cap * 2); pr.cls.resize(cap); pr.bytes.resize(cap);
        for (auto& e : pr.ev) cudaEventCreate(&e);
        int rc0 = run_step(m, &pr, true);
        cudaStreamSynchronize(s);
        double b = 0; for (int i = 0; i < pr.n; i++) b += pr.bytes[i];
        if (bytes_per_pass) *bytes_per_pass = b;
        if (launches) *launches = pr.n;
        for (auto& e : pr.ev) cudaEventDestroy(e);
        if (rc0) { m->class_mask = saved; m->launches_per_step = saved_launches; return rc0; }
    }
    cudaGraph_t g = nullptr; cudaGraphExec_t ge = nullptr;
    int rc = ATLASX_OK;
    cudaError_t e = cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal);
    if (e == cudaSuccess) {
        rc = run_step(m, nullptr, true);
        e = cudaStreamEndCapture(s, &g);
    }
    m->class_mask = saved; m->launches_per_step = saved_launches;
    if (rc) { if (g) cudaGraphDestroy(g); return rc; }
    if (e != cudaSuccess) return atlasx_fail(ATLASX_ERR_CUDA, "capture failed: %s", cudaGetErrorString(e));
    e = cudaGraphInstantiate(&ge, g, 0);
    cudaGraphDestroy(g);
    if (e != cudaSuccess) return atlasx_fail(ATLASX_ERR_CUDA, "graph instantiation failed: %s", cudaGetErrorString(e));
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0); cudaEventCreate(&e1);
    for (int i = 0; i < 3; i++) cudaGraphLaunch(ge, s);             // warm-up
    cudaEventRecord(e0, s);
    for (int i = 0; i < iters; i++) cudaGraphLaunch(ge, s);
    cudaEventRecord(e1, s);
    e = cudaStreamSynchronize(s);
    float ms = 0.f;
    cudaEventElapsedTime(&ms, e0, e1);
    cudaEventDestroy(e0); cudaEventDestroy(e1);
    cudaGraphExecDestroy(ge);
    if (e != cudaSuccess) return atlasx_fail(ATLASX_ERR_CUDA, "timed replay failed: %s", cudaGetErrorString(e));
    *ms_per_pass = ms / iters;
    return ATLASX_OK;
}

extern "C" int atlasx_model_profile_step(atlasx_model* m, int n_max, int* launches, float* ms, double* bytes, int* n_classes) {
    AX_ARG(m && m->finalized && launches && ms && bytes && n_classes && n_max >= CLS_COUNT, "bad argument");
    AX_ARG(m->host_pos < m->cfg.max_seq_len, "position is past max_seq_len");
    cudaStream_t s = m->ctx->stream;
    const int cap = m->cfg.n_layers * 8 + 8;
    Profile pr;
    pr.ev.resize((size_t)cap * 2); pr.cls.resize(cap); pr.bytes.resize(cap);
    for (auto& e : pr.ev) AX_CUDA(cudaEventCreate(&e));
    set_state_k<<<1, 1, 0, s>>>(m->st, m->host_pos, m->host_pos, m->seq);
    int rc = run_step(m, &pr, true);
    cudaError_t e = cudaStreamSynchronize(s);
    if (!rc && e != cudaSuccess) rc = atlasx_fail(ATLASX_ERR_CUDA, "profiled step failed: %s", cudaGetErrorString(e));
    if (!rc) {
        m->host_pos++;
        for (int i = 0; i < CLS_COUNT; i++) { launches[i] = 0; ms[i] = 0.f; bytes[i] = 0.0; }
        for (int i = 0; i < pr.n; i++) {
            float t = 0.f; cudaEventElapsedTime(&t, pr.ev[2 * i], pr.ev[2 * i + 1]);
            launches[pr.cls[i]]++; ms[pr.cls[i]] += t; bytes[pr.cls[i]] += pr.bytes[i];
        }
        *n_classes = CLS_COUNT;
    }
    for (auto& ev : pr.ev) cudaEventDestroy(ev);
    return rc;
}

extern "C" double atlasx_model_step_bytes(const atlasx_model* m, int pos) {
    if (!m) return 0;
    double b = 0;
    const double esz = m->cfg.kv_dtype == ATLASX_BF16 ? 2 : 4;
    for (const Layer& ly : m->layers) {
        b += (double)ax_weight_bytes(ly.qkv) + (double)ax_weight_bytes(ly.wo) + (double)ax_weight_bytes(ly.gateup) + (double)ax_weight_bytes(ly.down);
        int rows = pos + 1;
        if (ly.window > 0 && rows > ly.window) rows = ly.window;
        b += (double)rows * 2 * m->kv_rows * esz + 2.0 * m->kv_rows * esz;
    }
    b += (double)ax_weight_bytes(m->lm_head);
    return b;
}
extern "C" int atlasx_model_kernel_launches_per_step(const atlasx_model* m) { return m ? m->launches_per_step : 0; }
