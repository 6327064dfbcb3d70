// mega.cu — one persistent kernel for the whole decode step (see mega.cuh for the rationale).
//
// Grid = one CTA per SM, launched cooperatively so that every CTA is resident (the grid barrier
// needs that).  Per CTA: warp 8 is the weight producer, warps 0–7 are consumers.
//   producer : for every GEMV phase of the program, in order, stream this CTA's rows into the
//              shared-memory ring (cp.async.bulk + mbarrier).  Never looks at activations.
//   consumers: for every phase, in order: wait for the grid barrier of the previous phase, run the
//              phase (GEMV with fused prologue/epilogue, attention, selection), arrive.
// All waits are bounded; on expiry an error word is set and every later wait returns at once.
#include "mega.cuh"

#include <math_constants.h>

namespace {

constexpr int kAttnUnroll = 8;          // K/V rows in flight per lane group
constexpr int kMaxGroup = 4;            // query heads per KV head handled in registers

__device__ __forceinline__ unsigned long long ld_acquire_u64(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}

// Grid barrier over the consumer warps of all CTAs.  arrive: release + one atomic per CTA;
// wait: one thread polls the counter (bounded), then the 256 consumers of the CTA meet.
__device__ __forceinline__ void grid_arrive(MegaSync* sync) {
    consumer_sync();                                   // every consumer's stores are issued
    if (threadIdx.x == 0)                              // release: everything the CTA stored is visible first
        asm volatile("red.release.gpu.global.add.u64 [%0], 1;" ::"l"(&sync->count) : "memory");
}
__device__ __forceinline__ bool grid_wait(MegaSync* sync, unsigned long long target, int* err, int* s_flag) {
    if (threadIdx.x == 0) {
        int okv = 1;
        if (ld_acquire_u64(&sync->count) < target) {
            const unsigned long long t0 = globaltimer_ns();
            for (;;) {
                if (ld_acquire_u64(&sync->count) >= target) break;
                if (__ldcg(err) != 0) { okv = 0; break; }
                if (globaltimer_ns() - t0 > kWaitLimitNs) { atomicExch(err, 3); okv = 0; break; }
            }
        }
        *s_flag = okv;
    }
    consumer_sync();
    const bool ok = *s_flag != 0;
    consumer_sync();                                   // s_flag may be rewritten by the next wait
    return ok;
}

// x = merged attention output, written straight into the staged-input planes.  Partial states are
// laid out [head][split][hd + 4] (m, l, pad, pad, acc[hd]) so that acc is 16-byte aligned; all loads
// of a thread are issued before any is used (one L2 round trip).
constexpr int kMaxSplits = 8;
template <int FMT>
__device__ __noinline__ void stage_attention_merge(const MegaPhase& p, float4* xs) {
    constexpr int EPC = Fmt<FMT>::EPC;
    const int hd = p.merge_hd, S = p.merge_splits, ST = hd + 4;
    const int n4 = p.merge_heads * hd / 4, nch = p.g.nchunks;
    for (int e4 = threadIdx.x; e4 < n4; e4 += kConsumerThreads) {
        const int e = e4 * 4;
        const int h = e / hd, d = e - h * hd;
        const float* P = p.merge_partials + (size_t)h * S * ST;
        float2 ml[kMaxSplits]; float4 ac[kMaxSplits];
#pragma unroll
        for (int s = 0; s < kMaxSplits; s++) {
            if (s < S) {
                ml[s] = __ldcg(reinterpret_cast<const float2*>(P + (size_t)s * ST));
                ac[s] = __ldcg(reinterpret_cast<const float4*>(P + (size_t)s * ST + 4 + d));
            }
        }
        float M = -CUDART_INF_F;
#pragma unroll
        for (int s = 0; s < kMaxSplits; s++) if (s < S) M = fmaxf(M, ml[s].x);
        float L = 0.f; float4 A = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int s = 0; s < kMaxSplits; s++) {
            if (s < S) {
                const float w = (ml[s].x == -CUDART_INF_F) ? 0.f : expf(ml[s].x - M);
                L = fmaf(w, ml[s].y, L);
                A.x = fmaf(w, ac[s].x, A.x); A.y = fmaf(w, ac[s].y, A.y); A.z = fmaf(w, ac[s].z, A.z); A.w = fmaf(w, ac[s].w, A.w);
            }
        }
        const float inv = 1.0f / L;
        xs[((e % EPC) >> 2) * nch + e / EPC] = make_float4(A.x * inv, A.y * inv, A.z * inv, A.w * inv);
    }
    consumer_sync();
}

// Input staging split around the grid barrier.  When the GEMV input is  base + norm(y)  the
// residual stream `base` and the norm weights were final one barrier earlier, so they are loaded
// BEFORE the wait; only y (the previous phase's output) is loaded after it.
constexpr int kPreV = 4;                               // float4 per thread: K ≤ 4·4·256 = 4096
struct StagePre { float4 b[kPreV], wy[kPreV], wx[kPreV]; bool active; };

__device__ __forceinline__ void stage_prefetch(const GemvArgs& a, StagePre& pre) {
    const AxPrologue& p = a.pro;
    const int n4 = a.K >> 2;
    pre.active = p.y != nullptr && p.base != nullptr && !p.embed && n4 <= kPreV * kConsumerThreads;
    if (!pre.active) return;
#pragma unroll
    for (int j = 0; j < kPreV; j++) {
        const int k4 = threadIdx.x + j * kConsumerThreads;
        if (k4 < n4) {
            pre.b[j] = __ldcg(reinterpret_cast<const float4*>(p.base) + k4);
            if (p.wy) pre.wy[j] = reinterpret_cast<const float4*>(p.wy)[k4];
            if (p.wx) pre.wx[j] = reinterpret_cast<const float4*>(p.wx)[k4];
        }
    }
}

template <int FMT>
__device__ __forceinline__ void stage_finish(const GemvArgs& a, const StagePre& pre, float4* xs, float* red) {
    constexpr int EPC = Fmt<FMT>::EPC;
    const AxPrologue& p = a.pro;
    const int n4 = a.K >> 2, nch = a.nchunks, K = a.K;
    float4 t[kPreV];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < kPreV; j++) {
        const int k4 = threadIdx.x + j * kConsumerThreads;
        if (k4 < n4) {
            t[j] = __ldcg(reinterpret_cast<const float4*>(p.y) + k4);
            for (int r = 1; r < p.nparts; r++) {
                const float4 u = __ldcg(reinterpret_cast<const float4*>(p.y + (size_t)r * p.part_stride) + k4);
                t[j].x += u.x; t[j].y += u.y; t[j].z += u.z; t[j].w += u.w;
            }
            ss += t[j].x * t[j].x + t[j].y * t[j].y + t[j].z * t[j].z + t[j].w * t[j].w;
        }
    }
    float inv_y = 1.f;
    if (p.wy) {
        ss = consumer_block_sum(ss, red);
        inv_y = 1.0f / sqrtf(ss / (float)K + p.eps);
    }
    float ss2 = 0.f;
#pragma unroll
    for (int j = 0; j < kPreV; j++) {
        const int k4 = threadIdx.x + j * kConsumerThreads;
        if (k4 < n4) {
            float4 v = pre.b[j];
            if (p.wy) {
                v.x += t[j].x * inv_y * pre.wy[j].x; v.y += t[j].y * inv_y * pre.wy[j].y;
                v.z += t[j].z * inv_y * pre.wy[j].z; v.w += t[j].w * inv_y * pre.wy[j].w;
            } else { v.x += t[j].x; v.y += t[j].y; v.z += t[j].z; v.w += t[j].w; }
            t[j] = v;
            if (p.resid_out && blockIdx.x == 0) reinterpret_cast<float4*>(p.resid_out)[k4] = v;
            ss2 += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
    }
    float inv_x = 1.f;
    if (p.wx) {
        ss2 = consumer_block_sum(ss2, red);
        inv_x = 1.0f / sqrtf(ss2 / (float)K + p.eps);
    }
#pragma unroll
    for (int j = 0; j < kPreV; j++) {
        const int k4 = threadIdx.x + j * kConsumerThreads;
        if (k4 < n4) {
            float4 v = t[j];
            if (p.wx) { v.x = v.x * inv_x * pre.wx[j].x; v.y = v.y * inv_x * pre.wx[j].y; v.z = v.z * inv_x * pre.wx[j].z; v.w = v.w * inv_x * pre.wx[j].w; }
            const int e = k4 << 2;
            xs[((e % EPC) >> 2) * nch + e / EPC] = v;
        }
    }
    consumer_sync();
}

}  // namespace

#include "mega_attention.inl"

namespace {

template <int FMT, bool KVBF16>
__global__ void __launch_bounds__(kThreadsTma, 1) ax_decode_mega_kernel(const MegaArgs ma) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    // layout: [full | empty | red[16] | pair[16] | flag | pad to 256] [two phase records, 2 KB] [x / attention scratch] [ring]
    uint64_t* full = reinterpret_cast<uint64_t*>(smem_raw);
    uint64_t* empty = full + kMaxStages;
    float* red = reinterpret_cast<float*>(empty + kMaxStages);
    float* pair = red + 16;
    int* s_flag = reinterpret_cast<int*>(pair + 16);
    MegaPhase* sp = reinterpret_cast<MegaPhase*>(smem_raw + 256);          // two slots
    static_assert(sizeof(MegaPhase) <= 1024, "phase record must fit its shared-memory slot");
    float4* xs = reinterpret_cast<float4*>(smem_raw + 256 + 2048);
    Ring rg;
    rg.full = full; rg.empty = empty; rg.data = smem_raw + 256 + 2048 + ma.x_bytes;
    rg.stages = ma.stages; rg.stage_stride = ma.stage_stride; rg.seg_pitch = ma.seg_pitch;
    ring_init(rg);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int fill = 0;

    if (warp == kConsumerWarps) {
        // ── producer: the weight stream of the whole token ──────────────────────────
        bool ok = true;
        for (int ph = 0; ph < ma.n_phases && ok; ph++) {
            const MegaPhase* P = ma.phases + ph;
            if (P->type != MEGA_GEMV) continue;
            GemvArgs g;                               // only the fields the producer needs
            g.W = P->g.W; g.scales = P->g.scales; g.M = P->g.M; g.row_bytes = P->g.row_bytes;
            g.srow_bytes = P->g.srow_bytes; g.err = ma.err;
            int lo, hi; cta_rows(g.M, lo, hi);
            ok = ring_produce<FMT>(g, rg, lo, hi, fill);
        }
        if (!ok) for (int i = 0; i < 100; i++) __nanosleep(10000);
        return;
    }

    // ── consumers ──────────────────────────────────────────────────────────────────
    const unsigned long long base = ld_acquire_u64(&ma.sync->base);
    const unsigned long long G = gridDim.x;
    auto fetch_record = [&](int ph) {                  // phase record → shared memory (two slots)
        const uint32_t* src = reinterpret_cast<const uint32_t*>(ma.phases + ph);
        uint32_t* dst = reinterpret_cast<uint32_t*>(sp + (ph & 1));
        for (int i = threadIdx.x; i < (int)(sizeof(MegaPhase) / 4); i += kConsumerThreads) dst[i] = src[i];
    };
    fetch_record(0);
    consumer_sync();
    bool ok = true;
    for (int ph = 0; ph < ma.n_phases && ok; ph++) {
        const bool tr = ma.trace && blockIdx.x == 0 && threadIdx.x == 0;
        const MegaPhase& P = sp[ph & 1];
        // work that does not depend on the previous phase goes in front of the barrier wait
        if (ph + 1 < ma.n_phases) fetch_record(ph + 1);
        StagePre pre; pre.active = false;
        if (P.type == MEGA_GEMV && !P.merge_partials) stage_prefetch(P.g, pre);
        if (tr) ma.trace[ph * 4 + 0] = globaltimer_ns();
        if (ph > 0) ok = grid_wait(ma.sync, base + (unsigned long long)ph * G, ma.err, s_flag);
        else consumer_sync();
        if (!ok) break;
        if (tr) ma.trace[ph * 4 + 1] = globaltimer_ns();
        if (P.type == MEGA_GEMV) {
            GemvArgs g = P.g;
            g.err = ma.err;
            if (P.merge_partials) stage_attention_merge<FMT>(P, xs);
            else if (pre.active) stage_finish<FMT>(g, pre, xs, red);
            else stage_input<FMT>(g, xs, red);
            if (tr) ma.trace[ph * 4 + 2] = globaltimer_ns();
            int lo, hi; cta_rows(g.M, lo, hi);
            ok = ring_consume<FMT>(g, rg, xs, pair, lo, hi, fill);
        } else if (P.type == MEGA_ATTN) {
            mega_attention_phase<KVBF16>(P, reinterpret_cast<float*>(xs));
        } else if (P.type == MEGA_SELECT_PART) {
            mega_select_partial(P, reinterpret_cast<float*>(xs));
        } else {
            mega_select_final(P, reinterpret_cast<float*>(xs));
        }
        if (tr) ma.trace[ph * 4 + 3] = globaltimer_ns();
        if (ph + 1 < ma.n_phases) grid_arrive(ma.sync);
        else consumer_sync();
    }
    // the next launch starts counting where this one stopped
    if (blockIdx.x == 0 && threadIdx.x == 0)
        ma.sync->base = base + (unsigned long long)(ma.n_phases - 1) * G;
}

template <int FMT, bool KVBF16>
int launch_one(atlasx_ctx* ctx, const MegaArgs& args, size_t smem) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)ctx->sm_count); cfg.blockDim = dim3(kThreadsTma);
    cfg.dynamicSmemBytes = smem; cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    AX_CUDA(cudaLaunchKernelEx(&cfg, ax_decode_mega_kernel<FMT, KVBF16>, args));
    return ATLASX_OK;
}
template <int FMT>
int set_attr() {
    AX_CUDA(cudaFuncSetAttribute(ax_decode_mega_kernel<FMT, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448));
    AX_CUDA(cudaFuncSetAttribute(ax_decode_mega_kernel<FMT, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448));
    return ATLASX_OK;
}

}  // namespace

int ax_mega_init(atlasx_ctx*) {
    int rc;
    if ((rc = set_attr<ATLASX_F32>())) return rc;
    if ((rc = set_attr<ATLASX_BF16>())) return rc;
    if ((rc = set_attr<ATLASX_INT8>())) return rc;
    if ((rc = set_attr<ATLASX_INT4>())) return rc;
    return ATLASX_OK;
}

int ax_mega_launch(atlasx_ctx* ctx, int fmt, int kv_bf16, const MegaArgs& args, size_t smem) {
    if (kv_bf16) {
        switch (fmt) {
            case ATLASX_F32:  return launch_one<ATLASX_F32, true>(ctx, args, smem);
            case ATLASX_BF16: return launch_one<ATLASX_BF16, true>(ctx, args, smem);
            case ATLASX_INT8: return launch_one<ATLASX_INT8, true>(ctx, args, smem);
            default:          return launch_one<ATLASX_INT4, true>(ctx, args, smem);
        }
    }
    switch (fmt) {
        case ATLASX_F32:  return launch_one<ATLASX_F32, false>(ctx, args, smem);
        case ATLASX_BF16: return launch_one<ATLASX_BF16, false>(ctx, args, smem);
        case ATLASX_INT8: return launch_one<ATLASX_INT8, false>(ctx, args, smem);
        default:          return launch_one<ATLASX_INT4, false>(ctx, args, smem);
    }
}
