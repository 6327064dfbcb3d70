// objects.h — host-side objects behind the opaque handles of the C ABI.
#pragma once
#include "gemv.cuh"

// GpuMatrix (crates/atlas-tensor/src/lib.rs:309-315)
struct atlasx_matrix {
    atlasx_ctx* ctx = nullptr;
    AxWeight w;
    bool owned = false;
    void* data_own = nullptr;
    void* scales_own = nullptr;
};

// GpuKvCache (crates/atlas-tensor/src/lib.rs:701-709) with batch and element type
struct atlasx_kvcache {
    atlasx_ctx* ctx = nullptr;
    int max_seq = 0, n_kv = 0, hd = 0, dtype = ATLASX_BF16, batch = 1;
    size_t bytes = 0;          // of k (and of v)
    void* k = nullptr;
    void* v = nullptr;
};
