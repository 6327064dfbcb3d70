// ctx.cu — context, device buffers, GpuMatrix / GpuKvCache objects and the op-level atlasx_* ABI.
#include <stdarg.h>
#include <stdlib.h>
#include <string.h>
#include <math.h>
#include <vector>

#include "attention.cuh"
#include "attention_mma.cuh"
#include "common.cuh"
#include "elementwise.cuh"
#include "gemv.cuh"
#include "objects.h"
#include "sampling.cuh"

// ── error text ───────────────────────────────────────────────────────────────────
static thread_local char g_err[512] = "";
void atlasx_set_error(const char* fmt, ...) {
    va_list ap; va_start(ap, fmt); vsnprintf(g_err, sizeof(g_err), fmt, ap); va_end(ap);
}
int atlasx_fail(int code, const char* fmt, ...) {
    va_list ap; va_start(ap, fmt); vsnprintf(g_err, sizeof(g_err), fmt, ap); va_end(ap);
    return code;
}
extern "C" const char* atlasx_last_error(void) { return g_err; }

// ── context ──────────────────────────────────────────────────────────────────────
extern "C" int atlasx_ctx_create(int device, atlasx_ctx** out) {
    AX_ARG(out, "out is null");
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count <= 0)
        return atlasx_fail(ATLASX_ERR_NOGPU, "no CUDA device: this library has no CPU fallback");
    AX_ARG(device >= 0 && device < count, "device index out of range");
    AX_CUDA(cudaSetDevice(device));
    cudaDeviceProp prop;
    AX_CUDA(cudaGetDeviceProperties(&prop, device));
    if (prop.major < 10)
        return atlasx_fail(ATLASX_ERR_NOGPU, "device %s is sm_%d%d; this library is built for sm_100a only",
                           prop.name, prop.major, prop.minor);
    atlasx_ctx* c = new atlasx_ctx();
    c->device = device;
    c->sm_count = prop.multiProcessorCount;
    c->smem_optin = prop.sharedMemPerBlockOptin;
    AX_CUDA(cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking));
    AX_CUDA(cudaMalloc((void**)&c->dev_error, sizeof(int)));
    AX_CUDA(cudaMemset(c->dev_error, 0, sizeof(int)));
    AX_CUDA(cudaMallocHost((void**)&c->host_pin, 64 * sizeof(int)));
    const int amax_blocks = 4096;
    AX_CUDA(cudaMalloc((void**)&c->amax_vals, amax_blocks * sizeof(float)));
    AX_CUDA(cudaMalloc((void**)&c->amax_idx, amax_blocks * sizeof(int)));
    AX_CUDA(cudaMalloc((void**)&c->amax_ticket, sizeof(unsigned)));
    AX_CUDA(cudaMemset(c->amax_ticket, 0, sizeof(unsigned)));
    AX_CUDA(cudaMalloc((void**)&c->amax_out, sizeof(int)));
    {   // experiment switches: the only place the library reads its environment (besides ATLAS_NCCL_LIB at NCCL load)
        auto env_int = [](const char* name, int* dst) { const char* e = getenv(name); if (e && *e) *dst = atoi(e); };
        env_int("ATLASX_CARVEOUT", &c->carveout);
        env_int("ATLASX_GEMV_THREADS", &c->tune.gemv_threads);
        env_int("ATLASX_PDL_MASK", &c->tune.pdl_mask);
        env_int("ATLASX_ATTN_FUSED", &c->tune.attn_fused);
        env_int("ATLASX_ATTN_STAGES", &c->tune.attn_stages);
        env_int("ATLASX_ATTN_WAVE", &c->tune.attn_wave);
        env_int("ATLASX_ATTN_ROWS", &c->tune.attn_rows);
        env_int("ATLASX_ATTN_MMA", &c->tune.attn_mma);
        env_int("ATLASX_UMMA", &c->tune.umma);
        env_int("ATLASX_UMMA_PERSIST", &c->tune.umma_persist);
        env_int("ATLASX_UMMA_KS", &c->tune.umma_ks);
        env_int("ATLASX_INT4_FUSED", &c->tune.int4_fused);
        env_int("ATLASX_UMMA_FUSED", &c->tune.umma_fused);
        env_int("ATLASX_ATTN_PACK", &c->tune.attn_pack);
        env_int("ATLASX_ATTN_CFG", &c->tune.attn_cfg);
        env_int("ATLASX_PEER_ALLREDUCE", &c->tune.peer_allreduce);
        env_int("ATLASX_MAIL_REDUCE", &c->tune.mail_reduce);
        env_int("ATLASX_TP_SELECT", &c->tune.tp_select);
        env_int("ATLASX_STEP_TRACE", &c->tune.step_trace);
        env_int("ATLASX_COMM_TIMEOUT_MS", &c->tune.comm_timeout_ms);
        if (c->tune.attn_stages < 2 || c->tune.attn_stages > 4) c->tune.attn_stages = 3;
        if (c->tune.attn_wave < 1 || c->tune.attn_wave > 8) c->tune.attn_wave = 2;
    }
    int rc = ax_gemv_init(c);
    if (!rc) rc = ax_attn_init(c);
    if (rc) { delete c; return rc; }
    *out = c;
    return ATLASX_OK;
}

void atlasx_comm_destroy(atlasx_ctx* ctx);   // comm.cpp

extern "C" int atlasx_ctx_destroy(atlasx_ctx* c) {
    if (!c) return ATLASX_OK;
    cudaSetDevice(c->device);
    cudaStreamSynchronize(c->stream);
    atlasx_comm_destroy(c);
    ax_sample_free_scratch(c);
    cudaFree(c->attn_partials); cudaFree(c->attn_tickets); cudaFree(c->pos_dev); cudaFree(c->split_scratch); cudaFree(c->w_planes);
    cudaFree(c->amax_vals); cudaFree(c->amax_idx); cudaFree(c->amax_ticket); cudaFree(c->amax_out);
    cudaFree(c->dev_error); cudaFreeHost(c->host_pin);
    cudaStreamDestroy(c->stream);
    delete c;
    return ATLASX_OK;
}
extern "C" int atlasx_ctx_sync(atlasx_ctx* c) {
    AX_ARG(c, "ctx is null");
    AX_CUDA(cudaStreamSynchronize(c->stream));
    return ATLASX_OK;
}
extern "C" void* atlasx_ctx_stream(atlasx_ctx* c) { return c ? (void*)c->stream : nullptr; }
extern "C" int atlasx_ctx_sm_count(atlasx_ctx* c) { return c ? c->sm_count : 0; }
extern "C" int atlasx_ctx_set_gemv_impl(atlasx_ctx* c, int impl) {
    AX_ARG(c && impl >= 0 && impl <= 3, "impl must be 0 (automatic), 1 (plain loads), 2 (bulk-copy ring) or 3 (as 1, scalar multi-column kernel)");
    c->gemv_impl = impl;
    return ATLASX_OK;
}
extern "C" int atlasx_ctx_poll_device_error(atlasx_ctx* c, int* code_out) {
    AX_ARG(c, "ctx is null");
    AX_CUDA(cudaMemcpyAsync(c->host_pin, c->dev_error, sizeof(int), cudaMemcpyDeviceToHost, c->stream));
    AX_CUDA(cudaStreamSynchronize(c->stream));
    const int code = c->host_pin[0];
    if (code) {
        AX_CUDA(cudaMemsetAsync(c->dev_error, 0, sizeof(int), c->stream));
        // kernels that gave up may have left their arrival counters half counted; they are zero between launches otherwise
        if (c->split_scratch) AX_CUDA(cudaMemsetAsync(c->split_scratch, 0, 16384, c->stream));
        if (c->attn_tickets) AX_CUDA(cudaMemsetAsync(c->attn_tickets, 0, c->attn_tickets_cap * sizeof(unsigned), c->stream));
    }
    if (code_out) *code_out = code;
    return code ? atlasx_fail(ATLASX_ERR_TIMEOUT, "a bounded device-side wait expired (code %d)", code) : ATLASX_OK;
}

int atlasx_ctx_ensure_split_scratch(atlasx_ctx* c, size_t bytes) {
    if (bytes <= c->split_scratch_cap) return ATLASX_OK;
    cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
    cudaStreamIsCapturing(c->stream, &st);
    if (st != cudaStreamCaptureStatusNone)
        return atlasx_fail(ATLASX_ERR_STATE, "multi-column scratch must be sized before stream capture");
    AX_CUDA(cudaStreamSynchronize(c->stream));
    cudaFree(c->split_scratch);
    c->split_scratch = nullptr; c->split_scratch_cap = 0;
    if (bytes < (1u << 21)) bytes = 1u << 21;
    AX_CUDA(cudaMalloc(&c->split_scratch, bytes));
    AX_CUDA(cudaMemsetAsync(c->split_scratch, 0, 16384, c->stream));      // the item counter of the tcgen05 product starts out zero
    c->split_scratch_cap = bytes;
    return ATLASX_OK;
}

int atlasx_ctx_ensure_attn_scratch(atlasx_ctx* c, size_t partial_floats, size_t tickets) {
    if (partial_floats > c->attn_partials_cap) {
        cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
        cudaStreamIsCapturing(c->stream, &st);
        if (st != cudaStreamCaptureStatusNone)
            return atlasx_fail(ATLASX_ERR_STATE, "attention scratch must be sized before stream capture");
        AX_CUDA(cudaStreamSynchronize(c->stream));
        cudaFree(c->attn_partials);
        c->attn_partials = nullptr; c->attn_partials_cap = 0;
        AX_CUDA(cudaMalloc((void**)&c->attn_partials, partial_floats * sizeof(float)));
        c->attn_partials_cap = partial_floats;
    }
    if (tickets > c->attn_tickets_cap) {
        AX_CUDA(cudaStreamSynchronize(c->stream));
        cudaFree(c->attn_tickets);
        c->attn_tickets = nullptr; c->attn_tickets_cap = 0;
        AX_CUDA(cudaMalloc((void**)&c->attn_tickets, tickets * sizeof(unsigned)));
        AX_CUDA(cudaMemset(c->attn_tickets, 0, tickets * sizeof(unsigned)));
        c->attn_tickets_cap = tickets;
    }
    return ATLASX_OK;
}

static int ensure_pos(atlasx_ctx* c, const int* pos_host, int batch) {
    if ((size_t)batch > c->pos_cap) {
        AX_CUDA(cudaStreamSynchronize(c->stream));
        cudaFree(c->pos_dev); c->pos_dev = nullptr; c->pos_cap = 0;
        AX_CUDA(cudaMalloc((void**)&c->pos_dev, (size_t)batch * sizeof(int)));
        c->pos_cap = batch;
    }
    AX_CUDA(cudaMemcpyAsync(c->pos_dev, pos_host, (size_t)batch * sizeof(int), cudaMemcpyHostToDevice, c->stream));
    return ATLASX_OK;
}

// ── raw buffers ──────────────────────────────────────────────────────────────────
extern "C" int atlasx_malloc(atlasx_ctx* c, size_t bytes, void** out) {
    AX_ARG(c && out, "null argument");
    *out = nullptr;
    if (bytes == 0) return ATLASX_OK;
    AX_CUDA(cudaMalloc(out, bytes));
    return ATLASX_OK;
}
extern "C" int atlasx_free(atlasx_ctx* c, void* dev) {
    AX_ARG(c, "ctx is null");
    if (dev) { AX_CUDA(cudaStreamSynchronize(c->stream)); AX_CUDA(cudaFree(dev)); }
    return ATLASX_OK;
}
extern "C" int atlasx_memset(atlasx_ctx* c, void* dev, int value, size_t bytes) {
    AX_ARG(c, "ctx is null");
    if (bytes) AX_CUDA(cudaMemsetAsync(dev, value, bytes, c->stream));
    return ATLASX_OK;
}
extern "C" int atlasx_upload(atlasx_ctx* c, void* dst, const void* src, size_t bytes) {
    AX_ARG(c, "ctx is null");
    if (!bytes) return ATLASX_OK;
    AX_ARG(dst && src, "null pointer");
    AX_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, c->stream));
    AX_CUDA(cudaStreamSynchronize(c->stream));
    return ATLASX_OK;
}
extern "C" int atlasx_download(atlasx_ctx* c, void* dst, const void* src, size_t bytes) {
    AX_ARG(c, "ctx is null");
    if (!bytes) return ATLASX_OK;
    AX_ARG(dst && src, "null pointer");
    AX_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, c->stream));
    AX_CUDA(cudaStreamSynchronize(c->stream));
    return ATLASX_OK;
}
extern "C" int atlasx_copy_dev(atlasx_ctx* c, void* dst, const void* src, size_t bytes) {
    AX_ARG(c, "ctx is null");
    if (bytes) AX_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, c->stream));
    return ATLASX_OK;
}

// ── synthetic data / conversions ─────────────────────────────────────────────────
extern "C" int atlasx_fill_normal_f32(atlasx_ctx* c, float* dst, size_t n, uint64_t seed, uint64_t stream, uint64_t first, float std) {
    AX_ARG(c && (dst || !n), "null argument");
    ax_fill_normal_f32(c->stream, dst, n, seed, stream, first, std); AX_CHECK_LAUNCH("fill_normal_f32");
    return ATLASX_OK;
}
extern "C" int atlasx_fill_normal_bf16(atlasx_ctx* c, uint16_t* dst, size_t n, uint64_t seed, uint64_t stream, uint64_t first, float std) {
    AX_ARG(c && (dst || !n), "null argument");
    ax_fill_normal_bf16(c->stream, dst, n, seed, stream, first, std); AX_CHECK_LAUNCH("fill_normal_bf16");
    return ATLASX_OK;
}
extern "C" int atlasx_convert_bf16_to_f32(atlasx_ctx* c, const uint16_t* src, float* dst, size_t n) {
    AX_ARG(c, "ctx is null");
    ax_bf16_to_f32(c->stream, src, dst, n); AX_CHECK_LAUNCH("bf16_to_f32");
    return ATLASX_OK;
}
extern "C" int atlasx_convert_f32_to_bf16(atlasx_ctx* c, const float* src, uint16_t* dst, size_t n, int truncate) {
    AX_ARG(c, "ctx is null");
    ax_f32_to_bf16(c->stream, src, dst, n, truncate); AX_CHECK_LAUNCH("f32_to_bf16");
    return ATLASX_OK;
}

// ── atlas-quant on the device ────────────────────────────────────────────────────
extern "C" int atlasx_quantize_int8(atlasx_ctx* c, const float* src, int rows, int cols, int8_t* data, float* scales) {
    AX_ARG(c && rows >= 0 && cols >= 0, "bad shape");
    ax_quant_int8(c->stream, src, rows, cols, data, scales); AX_CHECK_LAUNCH("quant_int8");
    return ATLASX_OK;
}
extern "C" int atlasx_dequantize_int8(atlasx_ctx* c, const int8_t* data, const float* scales, int rows, int cols, float* out) {
    AX_ARG(c && rows >= 0 && cols >= 0, "bad shape");
    ax_dequant_int8(c->stream, data, scales, rows, cols, out); AX_CHECK_LAUNCH("dequant_int8");
    return ATLASX_OK;
}
extern "C" int atlasx_quantize_int4(atlasx_ctx* c, const float* src, size_t n, int block, uint8_t* data, float* scales) {
    AX_ARG(c && block > 0, "block_size must be positive");
    ax_quant_int4(c->stream, src, n, block, data, scales); AX_CHECK_LAUNCH("quant_int4");
    return ATLASX_OK;
}
extern "C" int atlasx_dequantize_int4(atlasx_ctx* c, const uint8_t* data, const float* scales, size_t n, int block, float* out) {
    AX_ARG(c && block > 0, "block_size must be positive");
    ax_dequant_int4(c->stream, data, scales, n, block, out); AX_CHECK_LAUNCH("dequant_int4");
    return ATLASX_OK;
}

// ── GpuMatrix ────────────────────────────────────────────────────────────────────
static int matrix_new(atlasx_ctx* c, int dtype, int rows, int cols, int block, int scales_f16, atlasx_matrix** out) {
    AX_ARG(c && out, "null argument");
    AX_ARG(rows > 0 && cols > 0, "rows and cols must be positive");
    atlasx_matrix* m = new atlasx_matrix();
    m->ctx = c;
    m->w.rows = rows; m->w.cols = cols; m->w.dtype = dtype; m->w.block = block; m->w.scales_f16 = scales_f16;
    *out = m;
    return ATLASX_OK;
}
static int upload_owned(atlasx_ctx* c, const void* host, size_t bytes, void** dev) {
    AX_CUDA(cudaMalloc(dev, bytes ? bytes : 16));
    if (bytes) {
        AX_CUDA(cudaMemcpyAsync(*dev, host, bytes, cudaMemcpyHostToDevice, c->stream));
        AX_CUDA(cudaStreamSynchronize(c->stream));
    }
    return ATLASX_OK;
}
extern "C" int atlasx_matrix_upload_f32(atlasx_ctx* c, const float* host, int rows, int cols, atlasx_matrix** out) {
    AX_ARG(host, "host pointer is null");
    int rc = matrix_new(c, ATLASX_F32, rows, cols, 0, 0, out); if (rc) return rc;
    (*out)->owned = true;
    rc = upload_owned(c, host, (size_t)rows * cols * 4, &(*out)->data_own);
    (*out)->w.data = (*out)->data_own;
    if (rc) { atlasx_matrix_free(*out); *out = nullptr; }
    return rc;
}
extern "C" int atlasx_matrix_upload_bf16(atlasx_ctx* c, const uint16_t* host, int rows, int cols, atlasx_matrix** out) {
    AX_ARG(host, "host pointer is null");
    int rc = matrix_new(c, ATLASX_BF16, rows, cols, 0, 0, out); if (rc) return rc;
    (*out)->owned = true;
    rc = upload_owned(c, host, (size_t)rows * cols * 2, &(*out)->data_own);
    (*out)->w.data = (*out)->data_own;
    if (rc) { atlasx_matrix_free(*out); *out = nullptr; }
    return rc;
}
extern "C" int atlasx_matrix_upload_int8(atlasx_ctx* c, const int8_t* data, const float* scales, int rows, int cols, atlasx_matrix** out) {
    AX_ARG(data && scales, "host pointer is null");
    int rc = matrix_new(c, ATLASX_INT8, rows, cols, 0, 0, out); if (rc) return rc;
    atlasx_matrix* m = *out; m->owned = true;
    rc = upload_owned(c, data, (size_t)rows * cols, &m->data_own);
    if (!rc) rc = upload_owned(c, scales, (size_t)rows * 4, &m->scales_own);
    m->w.data = m->data_own; m->w.scales = m->scales_own;
    if (rc) { atlasx_matrix_free(m); *out = nullptr; }
    return rc;
}
extern "C" int atlasx_matrix_upload_int4(atlasx_ctx* c, const uint8_t* data, const float* scales, int rows, int cols,
                                         int block, int scales_f16, atlasx_matrix** out) {
    AX_ARG(data && scales, "host pointer is null");
    AX_ARG(block > 0, "block_size must be positive");
    int rc = matrix_new(c, ATLASX_INT4, rows, cols, block, scales_f16 ? 1 : 0, out); if (rc) return rc;
    atlasx_matrix* m = *out; m->owned = true;
    const size_t n = (size_t)rows * cols, nb = (n + block - 1) / block;
    rc = upload_owned(c, data, (n + 1) / 2, &m->data_own);
    if (!rc) rc = upload_owned(c, scales, nb * 4, &m->scales_own);
    if (!rc && scales_f16) {
        void* h = nullptr;
        cudaError_t e = cudaMalloc(&h, nb * 2 + 16);
        if (e != cudaSuccess) rc = atlasx_fail(ATLASX_ERR_CUDA, "cudaMalloc failed: %s", cudaGetErrorString(e));
        else {
            ax_f32_to_f16(c->stream, (const float*)m->scales_own, (uint16_t*)h, nb);
            cudaStreamSynchronize(c->stream);
            cudaFree(m->scales_own); m->scales_own = h;
        }
    }
    m->w.data = m->data_own; m->w.scales = m->scales_own;
    if (rc) { atlasx_matrix_free(m); *out = nullptr; }
    return rc;
}
extern "C" int atlasx_matrix_wrap(atlasx_ctx* c, int dtype, const void* data, const void* scales, int rows, int cols,
                                  int block, int scales_f16, atlasx_matrix** out) {
    AX_ARG(data, "data pointer is null");
    AX_ARG(dtype >= ATLASX_F32 && dtype <= ATLASX_INT4, "unknown dtype");
    AX_ARG(dtype < ATLASX_INT8 || scales, "quantised formats need scales");
    AX_ARG(dtype != ATLASX_INT4 || block > 0, "block_size must be positive");
    int rc = matrix_new(c, dtype, rows, cols, block, scales_f16 ? 1 : 0, out); if (rc) return rc;
    (*out)->w.data = data; (*out)->w.scales = scales;
    return ATLASX_OK;
}
extern "C" int atlasx_matrix_free(atlasx_matrix* m) {
    if (!m) return ATLASX_OK;
    if (m->owned) {
        cudaStreamSynchronize(m->ctx->stream);
        cudaFree(m->data_own); cudaFree(m->scales_own);
    }
    delete m;
    return ATLASX_OK;
}
extern "C" int atlasx_matrix_info(const atlasx_matrix* m, int* rows, int* cols, int* dtype) {
    AX_ARG(m, "matrix is null");
    if (rows) *rows = m->w.rows;
    if (cols) *cols = m->w.cols;
    if (dtype) *dtype = m->w.dtype;
    return ATLASX_OK;
}
extern "C" size_t atlasx_matrix_bytes(const atlasx_matrix* m) { return m ? ax_weight_bytes(m->w) : 0; }

extern "C" int atlasx_gemv(atlasx_ctx* c, const atlasx_matrix* m, const float* x, int n, float* y) {
    AX_ARG(c && m && x && y, "null argument");
    AxPrologue pro; pro.base = x;
    return ax_gemv_launch(c, m->w, pro, AX_EPI_PLAIN, n, y, false);
}
extern "C" int atlasx_matrix_sgemm(atlasx_ctx* c, const atlasx_matrix* m, const float* rhs, int k, int n, float* out) {
    AX_ARG(c && m && rhs && out, "null argument");
    AX_ARG(k == m->w.cols, "k must equal the matrix column count");
    float *xd = nullptr, *yd = nullptr;
    AX_CUDA(cudaMalloc((void**)&xd, (size_t)k * n * 4));
    cudaError_t e = cudaMalloc((void**)&yd, (size_t)m->w.rows * n * 4);
    if (e != cudaSuccess) { cudaFree(xd); return atlasx_fail(ATLASX_ERR_CUDA, "cudaMalloc failed: %s", cudaGetErrorString(e)); }
    int rc = atlasx_upload(c, xd, rhs, (size_t)k * n * 4);
    if (!rc) rc = atlasx_gemv(c, m, xd, n, yd);
    if (!rc) rc = atlasx_download(c, out, yd, (size_t)m->w.rows * n * 4);
    cudaStreamSynchronize(c->stream);
    cudaFree(xd); cudaFree(yd);
    return rc;
}

// ── GpuVec ops ───────────────────────────────────────────────────────────────────
extern "C" int atlasx_vec_add(atlasx_ctx* c, const float* a, const float* b, float* out, int n) {
    AX_ARG(c && n >= 0, "bad argument");
    ax_vec_add(c->stream, a, b, out, n); AX_CHECK_LAUNCH("vec_add");
    return ATLASX_OK;
}
extern "C" int atlasx_rmsnorm(atlasx_ctx* c, const float* x, const float* w, float* out, int n, float eps) {
    AX_ARG(c && n >= 0, "bad argument");
    ax_rmsnorm(c->stream, x, w, out, n, eps); AX_CHECK_LAUNCH("rmsnorm");
    return ATLASX_OK;
}
extern "C" int atlasx_silu_mul(atlasx_ctx* c, const float* g, const float* u, float* out, int n) {
    AX_ARG(c && n >= 0, "bad argument");
    ax_silu_mul(c->stream, g, u, out, n); AX_CHECK_LAUNCH("silu_mul");
    return ATLASX_OK;
}
extern "C" int atlasx_argmax(atlasx_ctx* c, const float* x, int n, int* out_index) {
    AX_ARG(c && x && out_index && n > 0, "bad argument");
    AX_ARG(n <= 4096 * 1024, "n too large");
    AxArgmaxScratch sc = { c->amax_vals, c->amax_idx, c->amax_ticket };
    ax_argmax(c->stream, x, n, 1, sc, c->amax_out, nullptr); AX_CHECK_LAUNCH("argmax");
    AX_CUDA(cudaMemcpyAsync(c->host_pin, c->amax_out, sizeof(int), cudaMemcpyDeviceToHost, c->stream));
    AX_CUDA(cudaStreamSynchronize(c->stream));
    *out_index = c->host_pin[0];
    return ATLASX_OK;
}

// ── RoPE tables ──────────────────────────────────────────────────────────────────
// Host computation in f32 with the C library's powf/cosf/sinf, the same functions the Rust
// reference reaches through f32::powf/cos/sin (crates/atlas-model/src/lib.rs:380-423).
extern "C" int atlasx_rope_tables_host(int head_dim, int max_seq, float theta, int scaling, float factor,
                                       int orig_max_pos, float beta_fast, float beta_slow, float* cos_h, float* sin_h) {
    AX_ARG(head_dim > 0 && max_seq >= 0 && cos_h && sin_h, "bad argument");
    const int half = head_dim / 2;
    const float two_pi = 2.0f * 3.14159265358979323846f;
    std::vector<float> freqs((size_t)(half > 0 ? half : 1));
    for (int i = 0; i < half; i++) {
        const float base = 1.0f / powf(theta, 2.0f * (float)i / (float)head_dim);
        float f = base;
        if (scaling == 1) {
            const float wavelength = two_pi / base;
            const float low = (float)orig_max_pos / (two_pi * beta_slow);
            const float high = (float)orig_max_pos / (two_pi * beta_fast);
            if (wavelength < high) f = base;
            else if (wavelength > low) f = base / factor;
            else { const float alpha = (wavelength - high) / (low - high); f = base / (alpha * factor + (1.0f - alpha)); }
        }
        freqs[i] = f;
    }
    for (int p = 0; p < max_seq; p++)
        for (int i = 0; i < half; i++) {
            cos_h[(size_t)p * half + i] = cosf((float)p * freqs[i]);
            sin_h[(size_t)p * half + i] = sinf((float)p * freqs[i]);
        }
    return ATLASX_OK;
}

static int qk_prep_simple(atlasx_ctx* c, float* x, const float* w, const float* cos_t, const float* sin_t,
                          int n_heads, int hd, int pos, float eps) {
    // q-only form of the prep kernel (no cache write): used by the op-level entry points
    AxQkPrepArgs a;
    a.q = x; a.k = x; a.v = x; a.kc = x; a.vc = x;       // k/v unused: n_kv = 0
    a.q_norm = w; a.cos_t = cos_t; a.sin_t = sin_t;
    a.pos_scalar = pos; a.batch = 1; a.n_heads = n_heads; a.n_kv = 0; a.hd = hd; a.eps = eps;
    return ax_qk_prep_launch(c, a, false);
}
extern "C" int atlasx_qk_norm_inplace(atlasx_ctx* c, float* x, const float* w, int n_heads, int hd, float eps) {
    AX_ARG(c && x && w && n_heads > 0 && hd > 0, "bad argument");
    return qk_prep_simple(c, x, w, nullptr, nullptr, n_heads, hd, 0, eps);
}
extern "C" int atlasx_rope_apply(atlasx_ctx* c, float* x, const float* cos_t, const float* sin_t, int n_heads, int hd, int pos, int max_seq) {
    AX_ARG(c && x && cos_t && sin_t && n_heads > 0 && hd > 0, "bad argument");
    AX_ARG(pos >= 0 && pos < max_seq, "pos outside the tables");
    return qk_prep_simple(c, x, nullptr, cos_t, sin_t, n_heads, hd, pos, 0.f);
}

// ── GpuKvCache ───────────────────────────────────────────────────────────────────
extern "C" int atlasx_kvcache_create(atlasx_ctx* c, int max_seq, int n_kv, int hd, int dtype, int batch, atlasx_kvcache** out) {
    AX_ARG(c && out, "null argument");
    AX_ARG(max_seq > 0 && n_kv > 0 && hd > 0 && batch > 0, "dimensions must be positive");
    AX_ARG(dtype == ATLASX_BF16 || dtype == ATLASX_F32, "kv dtype must be bf16 or f32");
    atlasx_kvcache* kv = new atlasx_kvcache();
    kv->ctx = c; kv->max_seq = max_seq; kv->n_kv = n_kv; kv->hd = hd; kv->dtype = dtype; kv->batch = batch;
    kv->bytes = (size_t)batch * max_seq * n_kv * hd * (dtype == ATLASX_BF16 ? 2 : 4);
    cudaError_t e = cudaMalloc(&kv->k, kv->bytes);
    if (e == cudaSuccess) e = cudaMalloc(&kv->v, kv->bytes);
    if (e != cudaSuccess) {
        cudaFree(kv->k); delete kv;
        return atlasx_fail(ATLASX_ERR_CUDA, "KV cache allocation of 2×%zu bytes failed: %s", kv->bytes, cudaGetErrorString(e));
    }
    cudaMemsetAsync(kv->k, 0, kv->bytes, c->stream);      // GpuKvCache::new allocates zeroed vectors
    cudaMemsetAsync(kv->v, 0, kv->bytes, c->stream);
    *out = kv;
    return ATLASX_OK;
}
extern "C" int atlasx_kvcache_free(atlasx_kvcache* kv) {
    if (!kv) return ATLASX_OK;
    cudaStreamSynchronize(kv->ctx->stream);
    cudaFree(kv->k); cudaFree(kv->v);
    delete kv;
    return ATLASX_OK;
}
extern "C" int atlasx_kvcache_ptrs(atlasx_kvcache* kv, void** k, void** v, size_t* bytes_each) {
    AX_ARG(kv, "kv is null");
    if (k) *k = kv->k;
    if (v) *v = kv->v;
    if (bytes_each) *bytes_each = kv->bytes;
    return ATLASX_OK;
}
static int check_pos(const atlasx_kvcache* kv, const int* pos_host) {
    for (int b = 0; b < kv->batch; b++)
        if (pos_host[b] < 0 || pos_host[b] >= kv->max_seq)
            return atlasx_fail(ATLASX_ERR_ARG, "pos[%d] = %d is outside the cache (max_seq %d)", b, pos_host[b], kv->max_seq);
    return ATLASX_OK;
}
extern "C" int atlasx_kvcache_write(atlasx_ctx* c, atlasx_kvcache* kv, const float* k, const float* v, const int* pos_host) {
    AX_ARG(c && kv && k && v && pos_host, "null argument");
    int rc = check_pos(kv, pos_host); if (rc) return rc;
    rc = ensure_pos(c, pos_host, kv->batch); if (rc) return rc;
    AxQkPrepArgs a;
    a.q = const_cast<float*>(k);            // no query heads: n_heads = 0
    a.k = k; a.v = v; a.kc = kv->k; a.vc = kv->v;
    a.seq_stride = (size_t)kv->max_seq * kv->n_kv * kv->hd;
    a.pos = c->pos_dev; a.batch = kv->batch; a.n_heads = 0; a.n_kv = kv->n_kv; a.hd = kv->hd; a.kv_dtype = kv->dtype;
    a.kv_in_stride = (size_t)kv->n_kv * kv->hd;
    return ax_qk_prep_launch(c, a, false);
}
extern "C" int atlasx_decode_attention(atlasx_ctx* c, const atlasx_kvcache* kv, const float* q, float* out,
                                       int n_heads, const int* pos_host, float scale, int window) {
    AX_ARG(c && kv && q && out && pos_host, "null argument");
    AX_ARG(window >= 0, "window must be non-negative");
    int rc = check_pos(kv, pos_host); if (rc) return rc;
    int max_rows = 1;
    bool uniform = true;                  // every sequence at the same position (always so at batch 1): the position
    for (int b = 0; b < kv->batch; b++) { // travels as a kernel argument and no copy is queued
        int r = pos_host[b] + 1;
        if (window > 0 && r > window) r = window;
        if (r > max_rows) max_rows = r;
        uniform = uniform && pos_host[b] == pos_host[0];
    }
    if (!uniform) { rc = ensure_pos(c, pos_host, kv->batch); if (rc) return rc; }
    AxAttnArgs a;
    a.q = q; a.kc = kv->k; a.vc = kv->v; a.out = out;
    a.seq_stride = (size_t)kv->max_seq * kv->n_kv * kv->hd;
    a.pos = uniform ? nullptr : c->pos_dev; a.pos_scalar = pos_host[0]; a.batch = kv->batch; a.n_heads = n_heads; a.n_kv = kv->n_kv; a.hd = kv->hd;
    a.window = window; a.kv_dtype = kv->dtype; a.scale = scale;
    if (c->tune.attn_mma && ax_attn_mma_supported(a)) {       // several query heads per KV head: tensor-core kernel
        a.n_splits = ax_attn_mma_pick_splits(c, kv->n_kv, kv->batch, max_rows);
        return ax_attn_mma_launch(c, a, false);
    }
    a.n_splits = ax_attn_pick_splits(c, kv->n_kv, kv->batch, max_rows);
    return ax_attn_launch(c, a, false);
}
extern "C" size_t atlasx_decode_attention_bytes(const atlasx_kvcache* kv, int n_heads, const int* pos_host, int window) {
    if (!kv || !pos_host) return 0;
    size_t total = 0;
    const size_t esz = kv->dtype == ATLASX_BF16 ? 2 : 4;
    for (int b = 0; b < kv->batch; b++) {
        size_t rows = (size_t)pos_host[b] + 1;
        if (window > 0 && rows > (size_t)window) rows = window;
        total += rows * 2 * kv->n_kv * kv->hd * esz + (size_t)2 * n_heads * kv->hd * 4;
    }
    return total;
}

// ── measurement helpers ──────────────────────────────────────────────────────────
extern "C" int atlasx_time_gemv(atlasx_ctx* c, const atlasx_matrix* const* mats, int n_mats, const float* x, int n,
                                float* y, int iters, float* ms_out) {
    AX_ARG(c && mats && n_mats > 0 && x && y && iters > 0 && ms_out, "bad argument");
    cudaEvent_t e0, e1;
    AX_CUDA(cudaEventCreate(&e0)); AX_CUDA(cudaEventCreate(&e1));
    int rc = ATLASX_OK;
    for (int i = 0; i < n_mats && !rc; i++) rc = atlasx_gemv(c, mats[i], x, n, y);       // warm-up pass
    cudaStreamSynchronize(c->stream);
    cudaEventRecord(e0, c->stream);
    for (int i = 0; i < iters && !rc; i++) rc = atlasx_gemv(c, mats[i % n_mats], x, n, y);
    cudaEventRecord(e1, c->stream);
    cudaError_t e = cudaStreamSynchronize(c->stream);
    float ms = 0.f;
    cudaEventElapsedTime(&ms, e0, e1);
    cudaEventDestroy(e0); cudaEventDestroy(e1);
    if (rc) return rc;
    if (e != cudaSuccess) return atlasx_fail(ATLASX_ERR_CUDA, "timed GEMV failed: %s", cudaGetErrorString(e));
    *ms_out = ms;
    return ATLASX_OK;
}
extern "C" int atlasx_time_attention(atlasx_ctx* c, const atlasx_kvcache* kv, const float* q, float* out, int n_heads,
                                     const int* pos_host, float scale, int window, int iters, float* ms_out) {
    AX_ARG(c && kv && q && out && pos_host && iters > 0 && ms_out, "bad argument");
    cudaEvent_t e0, e1;
    AX_CUDA(cudaEventCreate(&e0)); AX_CUDA(cudaEventCreate(&e1));
    int rc = atlasx_decode_attention(c, kv, q, out, n_heads, pos_host, scale, window);   // warm-up, sizes the scratch
    cudaStreamSynchronize(c->stream);
    cudaEventRecord(e0, c->stream);
    for (int i = 0; i < iters && !rc; i++) rc = atlasx_decode_attention(c, kv, q, out, n_heads, pos_host, scale, window);
    cudaEventRecord(e1, c->stream);
    cudaError_t e = cudaStreamSynchronize(c->stream);
    float ms = 0.f;
    cudaEventElapsedTime(&ms, e0, e1);
    cudaEventDestroy(e0); cudaEventDestroy(e1);
    if (rc) return rc;
    if (e != cudaSuccess) return atlasx_fail(ATLASX_ERR_CUDA, "timed attention failed: %s", cudaGetErrorString(e));
    *ms_out = ms;
    return ATLASX_OK;
}
