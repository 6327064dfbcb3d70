// elementwise.cuh — small kernels of the decode path and of the reference's wider ABI.
#pragma once
#include "common.cuh"

// launchers take an explicit stream so the reference ABI can use the legacy default stream
void ax_vec_add(cudaStream_t s, const float* a, const float* b, float* out, int n);
void ax_scale(cudaStream_t s, const float* x, float k, float* out, int n);
void ax_relu(cudaStream_t s, const float* x, float* out, int n);
void ax_copy(cudaStream_t s, const float* src, float* dst, int n);
void ax_softmax_rows(cudaStream_t s, const float* x, float* out, int rows, int cols);
void ax_rmsnorm(cudaStream_t s, const float* x, const float* w, float* out, int n, float eps);
void ax_silu_mul(cudaStream_t s, const float* gate, const float* up, float* out, int n);
void ax_rope_onthefly(cudaStream_t s, float* x, int pos, int head_dim, float theta);
void ax_adamw(cudaStream_t s, float* p, float* m, float* v, const float* g, float lr, float b1, float b2,
              float eps, float wd, float bc1, float bc2, int n);

// argmax of x[0..n): last_of_equal selects the CPU rule of generate() (last index among equal
// maxima) or the reference kernel's rule (first).  Result as int and/or float; scratch must
// hold ceil(n/1024) (value,index) pairs plus one ticket that is zero between launches.
struct AxArgmaxScratch { float* vals; int* idx; unsigned* ticket; };
void ax_argmax(cudaStream_t s, const float* x, int n, int last_of_equal, AxArgmaxScratch sc,
               int* out_i, float* out_f);

// atlas-quant formats (bit-exact) and the reference-kernel quantisers (reference semantics)
void ax_quant_int8(cudaStream_t s, const float* src, int rows, int cols, int8_t* data, float* scales);
void ax_dequant_int8(cudaStream_t s, const int8_t* data, const float* scales, int rows, int cols, float* out);
void ax_quant_int4(cudaStream_t s, const float* src, size_t n, int block, uint8_t* data, float* scales);
void ax_dequant_int4(cudaStream_t s, const uint8_t* data, const float* scales, size_t n, int block, float* out);
void ax_refkernel_quant_int8(cudaStream_t s, const float* in, int8_t* out, float* scale, int rows, int cols);
void ax_refkernel_quant_int4(cudaStream_t s, const float* in, uint8_t* out, float* scale, int n);

void ax_fill_normal_f32(cudaStream_t s, float* dst, size_t n, uint64_t seed, uint64_t stream, uint64_t first, float std);
void ax_fill_normal_bf16(cudaStream_t s, uint16_t* dst, size_t n, uint64_t seed, uint64_t stream, uint64_t first, float std);
void ax_bf16_to_f32(cudaStream_t s, const uint16_t* src, float* dst, size_t n);
void ax_f32_to_bf16(cudaStream_t s, const float* src, uint16_t* dst, size_t n, int truncate);
void ax_f32_to_f16(cudaStream_t s, const float* src, uint16_t* dst, size_t n);

// strided 2-D copy of 1-, 2- or 4-byte elements: dst[r·dst_ld + c] = src[r·src_ld + c]
void ax_copy2d(cudaStream_t s, void* dst, size_t dst_ld, const void* src, size_t src_ld, size_t rows, size_t cols, int esize);
