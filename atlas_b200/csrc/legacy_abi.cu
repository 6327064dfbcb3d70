// legacy_abi.cu — the reference's own kernel ABI (kernels/matmul.cu:461-1008, declared to Rust at
// crates/atlas-tensor/src/lib.rs:20-91) served by the sm_100a kernels.  Same symbols, argument
// order, layouts and stream semantics (legacy default stream, asynchronous, void returns), so
// atlas-tensor links against this library without source changes.
#include <mutex>

#include "attention.cuh"
#include "common.cuh"
#include "elementwise.cuh"
#include "gemv.cuh"

namespace {

// One implicit context per device on the legacy default stream.
atlasx_ctx* g_legacy[16] = {};
std::mutex g_mu;

atlasx_ctx* legacy_ctx() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 16) return nullptr;
    std::lock_guard<std::mutex> lk(g_mu);
    if (g_legacy[dev]) return g_legacy[dev];
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, dev) != cudaSuccess) return nullptr;
    atlasx_ctx* c = new atlasx_ctx();
    c->device = dev;
    c->sm_count = prop.multiProcessorCount;
    c->smem_optin = prop.sharedMemPerBlockOptin;
    c->stream = cudaStreamLegacy;
    bool ok = cudaMalloc((void**)&c->dev_error, sizeof(int)) == cudaSuccess &&
              cudaMemset(c->dev_error, 0, sizeof(int)) == cudaSuccess &&
              cudaMalloc((void**)&c->amax_vals, 4096 * sizeof(float)) == cudaSuccess &&
              cudaMalloc((void**)&c->amax_idx, 4096 * sizeof(int)) == cudaSuccess &&
              cudaMalloc((void**)&c->amax_ticket, sizeof(unsigned)) == cudaSuccess &&
              cudaMemset(c->amax_ticket, 0, sizeof(unsigned)) == cudaSuccess &&
              ax_gemv_init(c) == ATLASX_OK && ax_attn_init(c) == ATLASX_OK;
    if (!ok) {
        fprintf(stderr, "[atlas_kernels] cannot initialise device %d: %s\n", dev, atlasx_last_error());
        delete c;
        return nullptr;
    }
    g_legacy[dev] = c;
    return c;
}

void report(const char* what, int rc) {
    if (rc) fprintf(stderr, "[atlas_kernels] %s failed: %s\n", what, atlasx_last_error());
}

// C[M×N] = A[M×K]·B[K×N] for N > 16 (prefill-shaped calls; not on the decode path)
template <bool BF16>
__global__ void gemm_tiled_k(const void* A, const float* B, float* C, int M, int N, int K) {
    __shared__ float sa[32][33], sb[32][33];
    const int row = blockIdx.y * 32 + threadIdx.y, col = blockIdx.x * 32 + threadIdx.x;
    float acc = 0.f;
    for (int t = 0; t < (K + 31) / 32; t++) {
        const int ac = t * 32 + threadIdx.x, br = t * 32 + threadIdx.y;
        float av = 0.f;
        if (row < M && ac < K)
            av = BF16 ? ax_bf16_to_f32(((const uint16_t*)A)[(size_t)row * K + ac]) : ((const float*)A)[(size_t)row * K + ac];
        sa[threadIdx.y][threadIdx.x] = av;
        sb[threadIdx.y][threadIdx.x] = (br < K && col < N) ? B[(size_t)br * N + col] : 0.f;
        __syncthreads();
#pragma unroll
        for (int k = 0; k < 32; k++) acc = fmaf(sa[threadIdx.y][k], sb[k][threadIdx.x], acc);
        __syncthreads();
    }
    if (row < M && col < N) C[(size_t)row * N + col] = acc;
}

void matmul_any(int dtype, const void* A, const float* B, float* C, int M, int N, int K) {
    if (M <= 0 || N <= 0 || K <= 0) return;
    atlasx_ctx* c = legacy_ctx();
    if (!c) return;
    if (N <= 16) {
        AxWeight w; w.data = A; w.rows = M; w.cols = K; w.dtype = dtype;
        AxPrologue pro; pro.base = B;
        report("gemv", ax_gemv_launch(c, w, pro, AX_EPI_PLAIN, N, C, false));
        return;
    }
    dim3 block(32, 32), grid((N + 31) / 32, (M + 31) / 32);
    if (dtype == ATLASX_BF16) gemm_tiled_k<true><<<grid, block, 0, cudaStreamLegacy>>>(A, B, C, M, N, K);
    else gemm_tiled_k<false><<<grid, block, 0, cudaStreamLegacy>>>(A, B, C, M, N, K);
}

}  // namespace

extern "C" {

void atlas_sync(void) { cudaDeviceSynchronize(); }

void atlas_matmul_f32(const float* A, const float* B, float* C, int M, int N, int K) { matmul_any(ATLASX_F32, A, B, C, M, N, K); }
void atlas_sgemm_bf16_f32(const uint16_t* A, const float* B, float* C, int M, int N, int K) { matmul_any(ATLASX_BF16, A, B, C, M, N, K); }

void atlas_vec_add_f32(const float* a, const float* b, float* out, int n) { ax_vec_add(cudaStreamLegacy, a, b, out, n); }
void atlas_scale_f32(const float* x, float s, float* out, int n) { ax_scale(cudaStreamLegacy, x, s, out, n); }
void atlas_relu_f32(const float* x, float* out, int n) { ax_relu(cudaStreamLegacy, x, out, n); }
void atlas_softmax_f32(const float* x, float* out, int rows, int cols) { ax_softmax_rows(cudaStreamLegacy, x, out, rows, cols); }
void atlas_rmsnorm_f32(const float* x, const float* w, float* out, int n, float eps) { ax_rmsnorm(cudaStreamLegacy, x, w, out, n, eps); }
void atlas_rope_apply_f32(float* x, int pos, int head_dim, float theta) { ax_rope_onthefly(cudaStreamLegacy, x, pos, head_dim, theta); }
void atlas_silu_mul_f32(const float* g, const float* u, float* out, int n) { ax_silu_mul(cudaStreamLegacy, g, u, out, n); }
void atlas_vram_copy_f32(const float* src, float* dst, int n) { ax_copy(cudaStreamLegacy, src, dst, n); }

void atlas_adamw_step(float* p, float* m, float* v, const float* g, float lr, float b1, float b2, float eps, float wd,
                      float bc1, float bc2, int n) {
    ax_adamw(cudaStreamLegacy, p, m, v, g, lr, b1, b2, eps, wd, bc1, bc2, n);
    cudaDeviceSynchronize();          // the reference wrapper synchronises (matmul.cu:556)
}

void atlas_qk_norm_inplace(float* x, const float* w, int n_heads, int head_dim, float eps) {
    atlasx_ctx* c = legacy_ctx();
    if (!c || n_heads <= 0 || head_dim <= 0) return;
    AxQkPrepArgs a;
    a.q = x; a.k = x; a.v = x; a.kc = x; a.vc = x;
    a.q_norm = w; a.batch = 1; a.n_heads = n_heads; a.n_kv = 0; a.hd = head_dim; a.eps = eps;
    report("qk_norm", ax_qk_prep_launch(c, a, false));
}
void atlas_rope_precomputed(float* x, const float* cos_tab, const float* sin_tab, int n_heads, int head_dim, int pos, int max_seq) {
    atlasx_ctx* c = legacy_ctx();
    (void)max_seq;
    if (!c || n_heads <= 0 || head_dim <= 0) return;
    AxQkPrepArgs a;
    a.q = x; a.k = x; a.v = x; a.kc = x; a.vc = x;
    a.cos_t = cos_tab; a.sin_t = sin_tab; a.pos_scalar = pos;
    a.batch = 1; a.n_heads = n_heads; a.n_kv = 0; a.hd = head_dim;
    report("rope", ax_qk_prep_launch(c, a, false));
}
void atlas_kv_cache_write(float* kc, float* vc, const float* nk, const float* nv, int pos, int n_kv, int hd) {
    atlasx_ctx* c = legacy_ctx();
    if (!c || n_kv <= 0 || hd <= 0) return;
    AxQkPrepArgs a;
    a.q = kc; a.k = nk; a.v = nv; a.kc = kc; a.vc = vc;
    a.pos_scalar = pos; a.batch = 1; a.n_heads = 0; a.n_kv = n_kv; a.hd = hd; a.kv_dtype = ATLASX_F32;
    report("kv_cache_write", ax_qk_prep_launch(c, a, false));
}
void atlas_decode_attention(const float* q, const float* kc, const float* vc, float* out, int n_heads, int n_kv, int hd,
                            int pos, float scale, int window) {
    atlasx_ctx* c = legacy_ctx();
    if (!c) return;
    AxAttnArgs a;
    a.q = q; a.kc = kc; a.vc = vc; a.out = out;
    a.pos_scalar = pos; a.batch = 1; a.n_heads = n_heads; a.n_kv = n_kv; a.hd = hd;
    a.window = window; a.kv_dtype = ATLASX_F32; a.scale = scale;
    int rows = pos + 1;
    if (window > 0 && rows > window) rows = window;
    a.n_splits = ax_attn_pick_splits(c, n_kv, 1, rows);
    report("decode_attention", ax_attn_launch(c, a, false));
}
void atlas_gpu_argmax(const float* x, float* out_f32, int n) {
    atlasx_ctx* c = legacy_ctx();
    if (!c || n <= 0 || n > 4096 * 1024) return;
    AxArgmaxScratch sc = { c->amax_vals, c->amax_idx, c->amax_ticket };
    ax_argmax(cudaStreamLegacy, x, n, /*last_of_equal=*/0, sc, nullptr, out_f32);
}

int atlas_cuda_device_count(void) { int n = 0; cudaGetDeviceCount(&n); return n; }
int atlas_cuda_available(void) { int n = 0; return (cudaGetDeviceCount(&n) == cudaSuccess && n > 0) ? 1 : 0; }

void atlas_quantize_int8(const float* in, int8_t* out, float* scale, int rows, int cols) {
    ax_refkernel_quant_int8(cudaStreamLegacy, in, out, scale, rows, cols);
    cudaDeviceSynchronize();
}
void atlas_dequantize_int8(const int8_t* in, const float* scale, float* out, int rows, int cols) {
    ax_dequant_int8(cudaStreamLegacy, in, scale, rows, cols, out);
    cudaDeviceSynchronize();
}
void atlas_quantize_int4(const float* in, uint8_t* out, float* scale, int n) {
    ax_refkernel_quant_int4(cudaStreamLegacy, in, out, scale, n);
    cudaDeviceSynchronize();
}

}  // extern "C"
