// sampling.cu — the sampling pipeline of generate_with_sampling on the device.
//
// The reference downloads 400 KB of logits per token and runs this on the CPU
// (crates/atlas-model/src/lib.rs: pipeline :1650-1710, primitives :2581-2717, Rng :1190-1216):
//   suppress (first token) → repetition penalty → frequency penalty → presence penalty →
//   ÷ temperature → top-k → top-p → min-p → softmax → sample with one XorShift64 draw.
// Here one 1024-thread CTA does all of it on the logits where they lie, and only the 4-byte token
// leaves the device.  The arithmetic follows the reference operation by operation: IEEE division
// where it divides, multiplication by the reciprocal where it multiplies, and every sum that the
// reference takes sequentially over the vocabulary is taken sequentially here too, in index order
// (masked entries contribute an exact 0, so only the survivors are visited) — the RNG stream, the
// top-k set and the tie rules are bit-exact, probabilities differ only by the last bit of expf.
// Where the reference leaves an order open (its unstable sort of equal probabilities in top-p),
// ties keep index order.
#include <math_constants.h>

#include "common.cuh"
#include "sampling.cuh"

namespace {

constexpr int kT = 1024;

__device__ __forceinline__ unsigned f32_key(float f) {          // order-preserving map to unsigned
    unsigned u = __float_as_uint(f);
    if (u == 0x80000000u) u = 0u;                                // −0 and +0 compare equal
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// exclusive prefix sum of one int per thread over the CTA; *total (shared memory) receives the sum
__device__ __forceinline__ int block_exscan(int v, int* warp_tot /*[32]*/, int* total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) { const int t = __shfl_up_sync(AX_FULL, inc, o); if (lane >= o) inc += t; }
    __syncthreads();
    if (lane == 31) warp_tot[warp] = inc;
    __syncthreads();
    if (warp == 0) {
        int w = warp_tot[lane];
        int winc = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) { const int t = __shfl_up_sync(AX_FULL, winc, o); if (lane >= o) winc += t; }
        warp_tot[lane] = winc - w;                               // exclusive offsets of the warps
        if (lane == 31) *total = winc;
    }
    __syncthreads();
    return warp_tot[warp] + inc - v;
}

__device__ __forceinline__ float block_max(float v, float* red /*[32]*/) {
    v = ax_warp_max(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float m = red[0];
#pragma unroll
    for (int w = 1; w < kT / 32; w++) m = fmaxf(m, red[w]);
    return m;
}

// "a sorts before b": larger probability first, equal probabilities in candidate (= index) order
__device__ __forceinline__ bool sorts_before(float pa, int ia, float pb, int ib) {
    return pa > pb || (pa == pb && ia < ib);
}

__global__ void __launch_bounds__(kT) ax_sample_kernel(const AxSampleArgs a) {
    __shared__ int s_hist[256];
    __shared__ int s_scan[32];
    __shared__ float s_red[32];
    __shared__ int s_i[4];
    __shared__ unsigned s_u[2];
    __shared__ float s_f[2];
    const int tid = threadIdx.x, n = a.n;
    const AxSamplingParams& c = a.cfg;

    // ── history counts: rebuilt from a token list (operator form) or advanced by one token ──────
    if (a.hist) {
        for (int i = tid; i < a.n_hist; i += kT) {
            const unsigned t = a.hist[i];
            if (t < (unsigned)n) { atomicAdd(&a.cnt_all[t], 1); if (i >= a.n_hist - a.win_len) atomicAdd(&a.cnt_win[t], 1); }
        }
    } else if (tid == 0) {
        if (a.tok_in >= 0 && a.tok_in < n) { a.cnt_all[a.tok_in] += 1; a.cnt_win[a.tok_in] += 1; }
        if (a.tok_out >= 0 && a.tok_out < n) a.cnt_win[a.tok_out] -= 1;
    }
    __syncthreads();

    // ── suppress, penalties, temperature (elementwise; :1652-1690) ───────────────────────────────
    const bool rep = c.repetition_penalty != 1.0f, freq = c.frequency_penalty != 0.0f, pres = c.presence_penalty != 0.0f;
    for (int i = tid; i < n; i += kT) {
        float l = a.logits[i];
        if (a.step == 0)
            for (int j = 0; j < a.n_suppress; j++) if (a.suppress[j] == (unsigned)i) l = -CUDART_INF_F;
        if (rep) for (int r = a.cnt_win[i]; r > 0; r--) l = l > 0.0f ? l / c.repetition_penalty : l * c.repetition_penalty;
        const int ca = a.cnt_all[i];
        if (freq && ca > 0) l -= c.frequency_penalty * (float)ca;
        if (pres && ca > 0) l -= c.presence_penalty;
        a.work[i] = l / c.temperature;
    }
    __syncthreads();

    // ── top-k (:2657-2686): the k-th largest value by radix select, then the survivors in index order ──
    const int chunk = (n + kT - 1) / kT;
    const int i0 = min(n, tid * chunk), i1 = min(n, i0 + chunk);
    unsigned thr_key = 0u;                       // keep everything above −inf …
    int need = 0;
    const bool use_k = c.top_k > 0 && c.top_k < n;
    if (use_k) {
        unsigned prefix = 0u; int k_left = c.top_k;
        for (int shift = 24; shift >= 0; shift -= 8) {
            for (int b = tid; b < 256; b += kT) s_hist[b] = 0;
            __syncthreads();
            const unsigned mask = shift == 24 ? 0u : (0xFFFFFFFFu << (shift + 8));
            for (int i = tid; i < n; i += kT) {
                const unsigned k = f32_key(a.work[i]);
                if ((k & mask) == prefix) atomicAdd(&s_hist[(k >> shift) & 255u], 1);
            }
            __syncthreads();
            if (tid == 0) {
                int b = 255, left = k_left;
                for (; b > 0; b--) { if (s_hist[b] >= left) break; left -= s_hist[b]; }
                s_u[0] = prefix | ((unsigned)b << shift); s_i[0] = left;
            }
            __syncthreads();
            prefix = s_u[0]; k_left = s_i[0];
            __syncthreads();
        }
        thr_key = prefix; need = k_left;         // k_left: how many of the values equal to the threshold are kept
    }
    // A −inf threshold (fewer than k finite logits) keeps every finite entry: the reference's tie
    // branch leaves the −inf ones as they are (:2670-2684) — the same as no top-k at all.
    const unsigned ninf_key = f32_key(-CUDART_INF_F);
    const bool by_thr = use_k && thr_key != ninf_key;
    int n_eq = 0, n_gt = 0;
    for (int i = i0; i < i1; i++) {
        const unsigned k = f32_key(a.work[i]);
        if (by_thr) { if (k > thr_key) n_gt++; else if (k == thr_key) n_eq++; }
        else if (k > ninf_key) n_gt++;
    }
    int eq_kept = 0;
    if (by_thr) {                                 // of the ties, the first `need` in index order survive
        const int eq_before = block_exscan(n_eq, s_scan, &s_i[3]);
        eq_kept = need - eq_before;
        eq_kept = eq_kept < 0 ? 0 : (eq_kept > n_eq ? n_eq : eq_kept);
    }
    int o = block_exscan(n_gt + eq_kept, s_scan, &s_i[1]);      // s_i[1]: number of candidates
    {
        int eq_seen = 0;
        for (int i = i0; i < i1; i++) {
            const float v = a.work[i];
            const unsigned k = f32_key(v);
            const bool keep = by_thr ? (k > thr_key || (k == thr_key && eq_seen++ < eq_kept)) : k > ninf_key;
            if (keep) { a.cval[o] = v; a.cidx[o] = i; o++; }
        }
    }
    __syncthreads();
    const int M = s_i[1];                         // candidates, in index order

    // the maximum survives every filter below, so it is taken once
    float mx = -CUDART_INF_F;
    for (int j = tid; j < M; j += kT) mx = fmaxf(mx, a.cval[j]);
    mx = block_max(mx, s_red);

    // ── top-p (:2625-2655) ───────────────────────────────────────────────────────────────────────
    if (c.top_p < 1.0f && M > 0) {
        int P2 = 1; while (P2 < M) P2 <<= 1;
        for (int j = tid; j < P2; j += kT) { a.skey[j] = j < M ? expf(a.cval[j] - mx) : -1.0f; a.sval[j] = j; }
        __syncthreads();
        if (tid == 0) { float s = 0.0f; for (int j = 0; j < M; j++) s += a.skey[j]; s_f[0] = s; }
        __syncthreads();
        const float sum = s_f[0];
        if (sum > 0.0f) {
            for (int j = tid; j < M; j += kT) a.skey[j] = a.skey[j] / sum;
            __syncthreads();
            for (int k = 2; k <= P2; k <<= 1)
                for (int j = k >> 1; j > 0; j >>= 1) {
                    for (int i = tid; i < P2; i += kT) {
                        const int x = i ^ j;
                        if (x > i) {
                            const float pa = a.skey[i], pb = a.skey[x]; const int ia = a.sval[i], ib = a.sval[x];
                            const bool up = (i & k) == 0;              // this pair ends in sorted order
                            const bool swap = up ? sorts_before(pb, ib, pa, ia) : sorts_before(pa, ia, pb, ib);
                            if (swap) { a.skey[i] = pb; a.skey[x] = pa; a.sval[i] = ib; a.sval[x] = ia; }
                        }
                    }
                    __syncthreads();
                }
            if (tid == 0) {
                float cum = 0.0f; int cut = M;
                for (int j = 0; j < M; j++) { cum += a.skey[j]; if (cum >= c.top_p) { cut = j + 1; break; } }
                s_i[2] = cut;
            }
            __syncthreads();
            const int cut = s_i[2];
            for (int j = cut + tid; j < M; j += kT) a.cval[a.sval[j]] = -CUDART_INF_F;
            __syncthreads();
        }
    }
    // ── min-p (:2692-2699) ───────────────────────────────────────────────────────────────────────
    if (c.min_p > 0.0f) {
        const float thr = mx + logf(c.min_p);
        for (int j = tid; j < M; j += kT) if (a.cval[j] < thr) a.cval[j] = -CUDART_INF_F;
        __syncthreads();
    }
    // ── softmax (:351-357) and the draw (:2710-2717) ─────────────────────────────────────────────
    for (int j = tid; j < M; j += kT) a.skey[j] = expf(a.cval[j] - mx);
    if (a.probs_out) for (int i = tid; i < n; i += kT) a.probs_out[i] = 0.0f;
    __syncthreads();
    if (tid == 0) {
        float s = 0.0f;
        for (int j = 0; j < M; j++) s += a.skey[j];
        s_f[1] = 1.0f / s;
        unsigned long long x = *a.rng;                                   // Rng::next_f32 (:1210-1215)
        x ^= x << 13; x ^= x >> 7; x ^= x << 17;
        *a.rng = x;
        s_f[0] = (float)(unsigned)(x >> 33) / 2147483648.0f;
    }
    __syncthreads();
    const float inv = s_f[1], r = s_f[0];
    for (int j = tid; j < M; j += kT) {
        const float p = a.skey[j] * inv;
        a.skey[j] = p;
        if (a.probs_out) a.probs_out[a.cidx[j]] = p;
    }
    __syncthreads();
    if (tid == 0) {
        float cum = 0.0f; int tok = n - 1;
        for (int j = 0; j < M; j++) { cum += a.skey[j]; if (r < cum) { tok = a.cidx[j]; break; } }
        *a.token_out = tok;
        if (a.last_token) *a.last_token = tok;
        if (a.seq && a.pos) { const int p = *a.pos; if (p >= 0 && p < a.seq_cap) a.seq[p] = tok; }
    }
}

}  // namespace

int ax_sample_ensure_scratch(atlasx_ctx* ctx, int n) {
    if (ctx->sample.cap >= n) return ATLASX_OK;
    AX_CUDA(cudaStreamSynchronize(ctx->stream));
    AxSampleScratch& s = ctx->sample;
    cudaFree(s.work); cudaFree(s.cval); cudaFree(s.cidx); cudaFree(s.skey); cudaFree(s.sval);
    cudaFree(s.cnt_all); cudaFree(s.cnt_win); cudaFree(s.rng); cudaFree(s.token); cudaFree(s.list);
    s = AxSampleScratch();
    int p2 = 1; while (p2 < n) p2 <<= 1;
    AX_CUDA(cudaMalloc((void**)&s.work, (size_t)n * 4));
    AX_CUDA(cudaMalloc((void**)&s.cval, (size_t)n * 4));
    AX_CUDA(cudaMalloc((void**)&s.cidx, (size_t)n * 4));
    AX_CUDA(cudaMalloc((void**)&s.skey, (size_t)p2 * 4));
    AX_CUDA(cudaMalloc((void**)&s.sval, (size_t)p2 * 4));
    AX_CUDA(cudaMalloc((void**)&s.cnt_all, (size_t)n * 4));
    AX_CUDA(cudaMalloc((void**)&s.cnt_win, (size_t)n * 4));
    AX_CUDA(cudaMalloc((void**)&s.rng, 8));
    AX_CUDA(cudaMalloc((void**)&s.token, 4));
    s.list_cap = 1 << 16;
    AX_CUDA(cudaMalloc((void**)&s.list, (size_t)s.list_cap * 4));
    s.cap = n;
    return ATLASX_OK;
}

void ax_sample_free_scratch(atlasx_ctx* ctx) {
    AxSampleScratch& s = ctx->sample;
    cudaFree(s.work); cudaFree(s.cval); cudaFree(s.cidx); cudaFree(s.skey); cudaFree(s.sval);
    cudaFree(s.cnt_all); cudaFree(s.cnt_win); cudaFree(s.rng); cudaFree(s.token); cudaFree(s.list);
    s = AxSampleScratch();
}

int ax_sample_reset_counts(atlasx_ctx* ctx, int n) {
    AX_CUDA(cudaMemsetAsync(ctx->sample.cnt_all, 0, (size_t)n * 4, ctx->stream));
    AX_CUDA(cudaMemsetAsync(ctx->sample.cnt_win, 0, (size_t)n * 4, ctx->stream));
    return ATLASX_OK;
}

int ax_sample_launch(atlasx_ctx* ctx, const AxSampleArgs& a) {
    ax_sample_kernel<<<1, kT, 0, ctx->stream>>>(a);
    AX_CHECK_LAUNCH("ax_sample_kernel");
    return ATLASX_OK;
}

static int check_config(const atlasx_sampling_config* c) {
    AX_ARG(c, "sampling configuration is null");
    AX_ARG(c->temperature > 0.0f && c->temperature >= 1e-6f, "the sampling kernel needs temperature > 0 (greedy decoding has its own path)");
    AX_ARG(c->repetition_window >= 0 && c->top_k >= 0, "repetition_window and top_k must not be negative");
    return ATLASX_OK;
}

AxSamplingParams ax_sampling_params(const atlasx_sampling_config& c) {
    AxSamplingParams p;
    p.temperature = c.temperature; p.repetition_penalty = c.repetition_penalty; p.repetition_window = c.repetition_window;
    p.frequency_penalty = c.frequency_penalty; p.presence_penalty = c.presence_penalty;
    p.top_p = c.top_p; p.top_k = c.top_k; p.min_p = c.min_p;
    return p;
}

// One selection from logits already on the device (operator form of the pipeline, for callers
// that drive the decode loop themselves and for parity tests).
extern "C" int atlasx_sample_token(atlasx_ctx* ctx, const float* logits_dev, int n, const atlasx_sampling_config* cfg, int step,
                                   const uint32_t* suppress_host, int n_suppress, const uint32_t* history_host, int n_hist,
                                   uint64_t* rng_state, int* token_out, float* probs_dev_out) {
    AX_ARG(ctx && logits_dev && n > 0 && rng_state && token_out, "bad argument");
    AX_ARG(n_suppress >= 0 && n_hist >= 0 && (n_suppress == 0 || suppress_host) && (n_hist == 0 || history_host), "bad list");
    int rc = check_config(cfg); if (rc) return rc;
    rc = ax_sample_ensure_scratch(ctx, n); if (rc) return rc;
    AxSampleScratch& s = ctx->sample;
    AX_ARG(n_suppress + n_hist <= s.list_cap, "suppress list + history too long for the operator form");
    cudaStream_t st = ctx->stream;
    rc = ax_sample_reset_counts(ctx, n); if (rc) return rc;
    if (n_suppress) AX_CUDA(cudaMemcpyAsync(s.list, suppress_host, (size_t)n_suppress * 4, cudaMemcpyHostToDevice, st));
    if (n_hist) AX_CUDA(cudaMemcpyAsync(s.list + n_suppress, history_host, (size_t)n_hist * 4, cudaMemcpyHostToDevice, st));
    AX_CUDA(cudaMemcpyAsync(s.rng, rng_state, 8, cudaMemcpyHostToDevice, st));
    AxSampleArgs a = {};
    a.logits = logits_dev; a.n = n; a.cfg = ax_sampling_params(*cfg); a.step = step;
    a.suppress = s.list; a.n_suppress = n_suppress;
    a.hist = n_hist ? s.list + n_suppress : nullptr; a.n_hist = n_hist;
    a.win_len = n_hist < cfg->repetition_window ? n_hist : cfg->repetition_window;
    a.tok_in = -1; a.tok_out = -1;
    a.work = s.work; a.cval = s.cval; a.cidx = s.cidx; a.skey = s.skey; a.sval = s.sval;
    a.cnt_all = s.cnt_all; a.cnt_win = s.cnt_win; a.rng = s.rng; a.token_out = s.token; a.probs_out = probs_dev_out;
    rc = ax_sample_launch(ctx, a); if (rc) return rc;
    AX_CUDA(cudaMemcpyAsync(token_out, s.token, 4, cudaMemcpyDeviceToHost, st));
    AX_CUDA(cudaMemcpyAsync(rng_state, s.rng, 8, cudaMemcpyDeviceToHost, st));
    AX_CUDA(cudaStreamSynchronize(st));
    return ATLASX_OK;
}
