// comm.h — collectives used by the tensor-parallel decode step.
#pragma once
#include "common.cuh"

int ax_comm_world(const atlasx_ctx* ctx);
int ax_comm_rank(const atlasx_ctx* ctx);
int ax_comm_allreduce_sum(atlasx_ctx* ctx, float* buf_dev, size_t n);                         // in place, on ctx->stream
int ax_comm_allgather(atlasx_ctx* ctx, const float* send_dev, float* recv_dev, size_t n_each);
void atlasx_comm_destroy(atlasx_ctx* ctx);
