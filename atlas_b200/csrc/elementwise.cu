// elementwise.cu — small kernels: the element-wise part of the reference ABI
// (kernels/matmul.cu:91-161,241-314,424-427,942-995), the atlas-quant formats on the device
// (crates/atlas-quant/src/lib.rs:41-168) and seeded synthetic data.
#include "elementwise.cuh"

#include <math_constants.h>

namespace {

constexpr int kT = 256;
inline int blocks_for(size_t n, int per = kT) { return (int)((n + per - 1) / per); }

__global__ void vec_add_k(const float* a, const float* b, float* out, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = a[i] + b[i];
}
__global__ void scale_k(const float* x, float k, float* out, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = x[i] * k;
}
__global__ void relu_k(const float* x, float* out, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = x[i] > 0.f ? x[i] : 0.f;
}
__global__ void copy_k(const float* s, float* d, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) d[i] = s[i];
}
__global__ void silu_mul_k(const float* g, const float* u, float* out, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) { const float x = g[i]; out[i] = (x / (1.0f + expf(-x))) * u[i]; }
}
// one warp per row, three passes (max, sum of exp, normalise) as matmul.cu:107-134
__global__ void softmax_rows_k(const float* x, float* out, int rows, int cols) {
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= rows) return;
    const float* xr = x + (size_t)row * cols;
    float* o = out + (size_t)row * cols;
    float mx = -1e30f;
    for (int j = lane; j < cols; j += 32) mx = fmaxf(mx, xr[j]);
    mx = ax_warp_max(mx);
    float s = 0.f;
    for (int j = lane; j < cols; j += 32) s += expf(xr[j] - mx);
    s = ax_warp_sum(s);
    for (int j = lane; j < cols; j += 32) o[j] = expf(xr[j] - mx) / s;
}
__device__ __forceinline__ float block_sum_256(float v, float* red) {
    v = ax_warp_sum(v);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = 0.f;
    for (int w = 0; w < (int)(blockDim.x >> 5); w++) t += red[w];
    __syncthreads();
    return t;
}
__device__ __forceinline__ float block_max_256(float v, float* red) {
    v = ax_warp_max(v);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = red[0];
    for (int w = 1; w < (int)(blockDim.x >> 5); w++) t = fmaxf(t, red[w]);
    __syncthreads();
    return t;
}
// single CTA, any n (including n < 32)
__global__ void rmsnorm_k(const float* x, const float* w, float* out, int n, float eps) {
    __shared__ float red[8];
    float ss = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) ss = fmaf(x[i], x[i], ss);
    ss = block_sum_256(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)n + eps);
    for (int i = threadIdx.x; i < n; i += blockDim.x) out[i] = x[i] * inv * w[i];
}
__global__ void rope_onthefly_k(float* x, int pos, int head_dim, float theta) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    const int half = head_dim / 2;
    if (i >= half) return;
    const float freq = 1.0f / powf(theta, (float)(2 * i) / (float)head_dim);
    const float ang = (float)pos * freq;
    const float c = cosf(ang), s = sinf(ang);
    const float x0 = x[i], x1 = x[i + half];
    x[i] = x0 * c - x1 * s;
    x[i + half] = x0 * s + x1 * c;
}
__global__ void adamw_k(float* p, float* m, float* v, const float* g, float lr, float b1, float b2, float eps,
                        float wd, float bc1, float bc2, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float gi = g[i];
    const float mi = b1 * m[i] + (1.0f - b1) * gi;
    const float vi = b2 * v[i] + (1.0f - b2) * gi * gi;
    m[i] = mi; v[i] = vi;
    p[i] = p[i] * (1.0f - lr * wd) - lr * (mi * bc1) / (sqrtf(vi * bc2) + eps);
}

// ── argmax ───────────────────────────────────────────────────────────────────────
// Each CTA reduces 1024 values to one (value, index); the last CTA to finish (ticket) reduces
// those.  Nothing waits.
__global__ void __launch_bounds__(256) argmax_k(const float* x, int n, int last, AxArgmaxScratch sc, int* out_i, float* out_f) {
    __shared__ float sv[8];
    __shared__ int si[8];
    __shared__ int s_last;
    asm volatile("griddepcontrol.wait;" ::: "memory");
    float v = 0.f; int idx = -1;
    const int base = blockIdx.x * 1024;
#pragma unroll
    for (int u = 0; u < 4; u++) {
        const int i = base + u * 256 + threadIdx.x;
        if (i < n) { const float xv = x[i]; if (ax_better(xv, i, v, idx, last)) { v = xv; idx = i; } }
    }
    ax_warp_best(v, idx, last);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) { sv[warp] = v; si[warp] = idx; }
    __syncthreads();
    if (warp == 0) {
        v = lane < 8 ? sv[lane] : 0.f; idx = lane < 8 ? si[lane] : -1;
        ax_warp_best(v, idx, last);
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
        if (ax_better(bv, bi, v, idx, last)) { v = bv; idx = bi; }
    }
    ax_warp_best(v, idx, last);
    if (lane == 0) {
        if (idx < 0) idx = last ? n - 1 : 0;          // every value was NaN
        if (out_i) *out_i = idx;
        if (out_f) *out_f = (float)idx;
        *sc.ticket = 0u;
    }
}

// ── atlas-quant: Int8Tensor::quantize, one CTA per row ───────────────────────────
__device__ __forceinline__ float round_half_away_clamped(float v, float lim) {
    if (v != v) return 0.f;                         // Rust: NaN as i8 → 0
    v = v < -lim ? -lim : (v > lim ? lim : v);      // f32::clamp
    return roundf(v);                               // f32::round: half away from zero
}
__global__ void __launch_bounds__(256) quant_int8_k(const float* src, int rows, int cols, int8_t* data, float* scales) {
    __shared__ float red[8];
    const int r = blockIdx.x;
    const float* row = src + (size_t)r * cols;
    float mx = 0.f;
    for (int j = threadIdx.x; j < cols; j += blockDim.x) mx = fmaxf(mx, fabsf(row[j]));
    mx = block_max_256(mx, red);
    const float s = mx > 0.f ? __fdiv_rn(mx, 127.0f) : 1.0f;
    if (threadIdx.x == 0) scales[r] = s;
    const float inv = __fdiv_rn(1.0f, s);
    for (int j = threadIdx.x; j < cols; j += blockDim.x)
        data[(size_t)r * cols + j] = (int8_t)(int)round_half_away_clamped(__fmul_rn(row[j], inv), 127.0f);
}
__global__ void dequant_int8_k(const int8_t* data, const float* scales, int rows, int cols, float* out) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)rows * cols) return;
    out[i] = __fmul_rn((float)data[i], scales[i / cols]);
}
// Int4Tensor::quantize: blocks over the flat index.  Pass 1: one warp per block → scale.
__global__ void quant_int4_scales_k(const float* src, size_t n, int block, float* scales, size_t n_blocks) {
    const size_t b = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (b >= n_blocks) return;
    const size_t start = b * block;
    const size_t end = start + block < n ? start + block : n;
    float mx = 0.f;
    for (size_t i = start + lane; i < end; i += 32) mx = fmaxf(mx, fabsf(src[i]));
    mx = ax_warp_max(mx);
    if (lane == 0) scales[b] = mx > 0.f ? __fdiv_rn(mx, 7.0f) : 1.0f;
}
// Pass 2: one thread per output byte (two elements that may belong to different blocks).
__global__ void quant_int4_pack_k(const float* src, size_t n, int block, const float* scales, uint8_t* data) {
    const size_t byte = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (byte >= (n + 1) / 2) return;
    uint8_t out = 0;
#pragma unroll
    for (int h = 0; h < 2; h++) {
        const size_t idx = byte * 2 + h;
        if (idx < n) {
            const float inv = __fdiv_rn(1.0f, scales[idx / block]);
            const int q = (int)round_half_away_clamped(__fmul_rn(src[idx], inv), 7.0f);
            const uint8_t nib = (uint8_t)(q & 0x0F);
            out |= h == 0 ? (uint8_t)(nib << 4) : nib;
        }
    }
    data[byte] = out;
}
__global__ void dequant_int4_k(const uint8_t* data, const float* scales, size_t n, int block, float* out) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const uint8_t b = data[i >> 1];
    const int nib = (i & 1) ? (b & 0x0F) : (b >> 4);
    const int q = nib >= 8 ? nib - 16 : nib;
    out[i] = __fmul_rn((float)q, scales[i / block]);
}

// ── the reference KERNEL's quantisers (matmul.cu:166-237): ties-to-even, zero reciprocal
//    for an all-zero input, int4 with one scale for the whole tensor and pairs only ──────
__global__ void __launch_bounds__(256) refk_quant_int8_k(const float* in, int8_t* out, float* scale, int rows, int cols) {
    __shared__ float red[8];
    const int r = blockIdx.x;
    float mx = 0.f;
    for (int j = threadIdx.x; j < cols; j += blockDim.x) mx = fmaxf(mx, fabsf(in[(size_t)r * cols + j]));
    mx = block_max_256(mx, red);
    const float s = __fdiv_rn(mx, 127.0f);
    if (threadIdx.x == 0) scale[r] = s;
    const float inv = s > 0.f ? __fdiv_rn(1.0f, s) : 0.f;
    for (int j = threadIdx.x; j < cols; j += blockDim.x) {
        const float v = fminf(fmaxf(__fmul_rn(in[(size_t)r * cols + j], inv), -127.f), 127.f);
        out[(size_t)r * cols + j] = (int8_t)__float2int_rn(v);
    }
}
__global__ void __launch_bounds__(256) refk_quant_int4_k(const float* in, uint8_t* out, float* scale, int n) {
    __shared__ float red[8];
    float mx = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) mx = fmaxf(mx, fabsf(in[i]));
    mx = block_max_256(mx, red);
    const float s = __fdiv_rn(mx, 7.0f);
    if (threadIdx.x == 0) *scale = s;
    const float inv = s > 0.f ? __fdiv_rn(1.0f, s) : 0.f;
    for (int i = threadIdx.x * 2; i < n - 1; i += blockDim.x * 2) {
        const int q0 = __float2int_rn(fminf(fmaxf(__fmul_rn(in[i], inv), -7.f), 7.f));
        const int q1 = __float2int_rn(fminf(fmaxf(__fmul_rn(in[i + 1], inv), -7.f), 7.f));
        out[i / 2] = (uint8_t)(((q0 & 0xF) << 4) | (q1 & 0xF));
    }
}

// ── synthetic data and conversions ───────────────────────────────────────────────
__global__ void fill_normal_f32_k(float* dst, size_t n, uint64_t base, uint64_t first, float std) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        dst[i] = __fmul_rn(ax_synth_normal(base, first + i), std);
}
__global__ void fill_normal_bf16_k(uint16_t* dst, size_t n, uint64_t base, uint64_t first, float std) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        dst[i] = ax_f32_to_bf16_rne(__fmul_rn(ax_synth_normal(base, first + i), std));
}
__global__ void bf16_to_f32_k(const uint16_t* s, float* d, size_t n) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        d[i] = ax_bf16_to_f32(s[i]);
}
__global__ void f32_to_bf16_k(const float* s, uint16_t* d, size_t n, int trunc) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        d[i] = trunc ? (uint16_t)(__float_as_uint(s[i]) >> 16) : ax_f32_to_bf16_rne(s[i]);
}
__global__ void f32_to_f16_k(const float* s, uint16_t* d, size_t n) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        d[i] = __half_as_ushort(__float2half_rn(s[i]));
}
template <typename T>
__global__ void copy2d_k(T* dst, size_t dst_ld, const T* src, size_t src_ld, size_t rows, size_t cols) {
    const size_t total = rows * cols;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / cols, c = i % cols;
        dst[r * dst_ld + c] = src[r * src_ld + c];
    }
}
inline int grid_stride_blocks(size_t n) {
    size_t b = (n + kT - 1) / kT;
    if (b > 148 * 16) b = 148 * 16;
    if (b < 1) b = 1;
    return (int)b;
}

}  // namespace

void ax_vec_add(cudaStream_t s, const float* a, const float* b, float* out, int n) { if (n > 0) vec_add_k<<<blocks_for(n), kT, 0, s>>>(a, b, out, n); }
void ax_scale(cudaStream_t s, const float* x, float k, float* out, int n) { if (n > 0) scale_k<<<blocks_for(n), kT, 0, s>>>(x, k, out, n); }
void ax_relu(cudaStream_t s, const float* x, float* out, int n) { if (n > 0) relu_k<<<blocks_for(n), kT, 0, s>>>(x, out, n); }
void ax_copy(cudaStream_t s, const float* src, float* dst, int n) { if (n > 0) copy_k<<<blocks_for(n), kT, 0, s>>>(src, dst, n); }
void ax_silu_mul(cudaStream_t s, const float* g, const float* u, float* out, int n) { if (n > 0) silu_mul_k<<<blocks_for(n), kT, 0, s>>>(g, u, out, n); }
void ax_softmax_rows(cudaStream_t s, const float* x, float* out, int rows, int cols) {
    if (rows > 0 && cols > 0) softmax_rows_k<<<(rows + 7) / 8, kT, 0, s>>>(x, out, rows, cols);
}
void ax_rmsnorm(cudaStream_t s, const float* x, const float* w, float* out, int n, float eps) { if (n > 0) rmsnorm_k<<<1, kT, 0, s>>>(x, w, out, n, eps); }
void ax_rope_onthefly(cudaStream_t s, float* x, int pos, int head_dim, float theta) {
    const int half = head_dim / 2;
    if (half > 0) rope_onthefly_k<<<blocks_for(half), kT, 0, s>>>(x, pos, head_dim, theta);
}
void ax_adamw(cudaStream_t s, float* p, float* m, float* v, const float* g, float lr, float b1, float b2, float eps,
              float wd, float bc1, float bc2, int n) {
    if (n > 0) adamw_k<<<blocks_for(n), kT, 0, s>>>(p, m, v, g, lr, b1, b2, eps, wd, bc1, bc2, n);
}
void ax_argmax(cudaStream_t s, const float* x, int n, int last, AxArgmaxScratch sc, int* out_i, float* out_f) {
    if (n > 0) argmax_k<<<(n + 1023) / 1024, 256, 0, s>>>(x, n, last, sc, out_i, out_f);
}
void ax_quant_int8(cudaStream_t s, const float* src, int rows, int cols, int8_t* data, float* scales) {
    if (rows > 0 && cols > 0) quant_int8_k<<<rows, 256, 0, s>>>(src, rows, cols, data, scales);
}
void ax_dequant_int8(cudaStream_t s, const int8_t* data, const float* scales, int rows, int cols, float* out) {
    const size_t n = (size_t)rows * cols;
    if (n) dequant_int8_k<<<blocks_for(n), kT, 0, s>>>(data, scales, rows, cols, out);
}
void ax_quant_int4(cudaStream_t s, const float* src, size_t n, int block, uint8_t* data, float* scales) {
    if (!n) return;
    const size_t nb = (n + block - 1) / block;
    quant_int4_scales_k<<<blocks_for(nb, 8), kT, 0, s>>>(src, n, block, scales, nb);
    quant_int4_pack_k<<<blocks_for((n + 1) / 2), kT, 0, s>>>(src, n, block, scales, data);
}
void ax_dequant_int4(cudaStream_t s, const uint8_t* data, const float* scales, size_t n, int block, float* out) {
    if (n) dequant_int4_k<<<blocks_for(n), kT, 0, s>>>(data, scales, n, block, out);
}
void ax_refkernel_quant_int8(cudaStream_t s, const float* in, int8_t* out, float* scale, int rows, int cols) {
    if (rows > 0 && cols > 0) refk_quant_int8_k<<<rows, 256, 0, s>>>(in, out, scale, rows, cols);
}
void ax_refkernel_quant_int4(cudaStream_t s, const float* in, uint8_t* out, float* scale, int n) {
    if (n > 0) refk_quant_int4_k<<<1, 256, 0, s>>>(in, out, scale, n);
}
void ax_fill_normal_f32(cudaStream_t s, float* dst, size_t n, uint64_t seed, uint64_t stream, uint64_t first, float std) {
    if (n) fill_normal_f32_k<<<grid_stride_blocks(n), kT, 0, s>>>(dst, n, ax_mix64(seed ^ ax_mix64(stream)), first, std);
}
void ax_fill_normal_bf16(cudaStream_t s, uint16_t* dst, size_t n, uint64_t seed, uint64_t stream, uint64_t first, float std) {
    if (n) fill_normal_bf16_k<<<grid_stride_blocks(n), kT, 0, s>>>(dst, n, ax_mix64(seed ^ ax_mix64(stream)), first, std);
}
void ax_bf16_to_f32(cudaStream_t s, const uint16_t* src, float* dst, size_t n) { if (n) bf16_to_f32_k<<<grid_stride_blocks(n), kT, 0, s>>>(src, dst, n); }
void ax_f32_to_bf16(cudaStream_t s, const float* src, uint16_t* dst, size_t n, int t) { if (n) f32_to_bf16_k<<<grid_stride_blocks(n), kT, 0, s>>>(src, dst, n, t); }
void ax_f32_to_f16(cudaStream_t s, const float* src, uint16_t* dst, size_t n) { if (n) f32_to_f16_k<<<grid_stride_blocks(n), kT, 0, s>>>(src, dst, n); }
void ax_copy2d(cudaStream_t s, void* dst, size_t dst_ld, const void* src, size_t src_ld, size_t rows, size_t cols, int esize) {
    const size_t n = rows * cols;
    if (!n) return;
    if (esize == 1) copy2d_k<uint8_t><<<grid_stride_blocks(n), kT, 0, s>>>((uint8_t*)dst, dst_ld, (const uint8_t*)src, src_ld, rows, cols);
    else if (esize == 2) copy2d_k<uint16_t><<<grid_stride_blocks(n), kT, 0, s>>>((uint16_t*)dst, dst_ld, (const uint16_t*)src, src_ld, rows, cols);
    else copy2d_k<uint32_t><<<grid_stride_blocks(n), kT, 0, s>>>((uint32_t*)dst, dst_ld, (const uint32_t*)src, src_ld, rows, cols);
}
