// comm.h — collectives used by the tensor-parallel decode step.
#pragma once
#include "common.cuh"

constexpr int kMaxPeers = AX_MAX_PEERS;

// Mailboxes in peer memory for the all-reduce that is fused into the row-parallel GEMVs.
// Every rank owns one allocation, mapped into every other rank of the node (CUDA IPC):
//   parts : [2 buffers][world][d] pairs (value bits, sequence number), 8 bytes each — rank r's
//           partial output lands in slot r of EVERY rank.
// Buffer 0 carries the o_proj partials, buffer 1 the down-projection partials; two buffers are
// enough because a rank can only reach its next write into a buffer after it has consumed a
// part that every peer produced after reading the previous content of that buffer.
struct AxPeerMail {
    int world = 1, rank = 0, d = 0;
    // Device word beside this rank's mailbox: number of mailbox uses so far.  It belongs to the
    // mailbox, not to a model — every model of the context stamps its partial sums with
    // *useq + layer + 1 and advances the word by its layer count per step, so sequence numbers
    // never repeat while the mailbox lives, whatever models come and go on the context.
    unsigned* useq = nullptr;
    // Selection slots: rank r leaves its local best (value bits, vocabulary index, sequence, sequence) in
    // entry r of every rank's `sel` array with one 16-byte store (vocabulary-parallel argmax).
    uint4* sel_base[kMaxPeers] = {};
    uint4* sel(int owner, int from) const { return sel_base[owner] + from; }
    uint2* base[kMaxPeers] = {};        // mailbox of rank p as mapped in this process (own allocation for p == rank)
    uint2* part(int owner, int buf, int from) const { return base[owner] + ((size_t)buf * world + from) * d; }
};

int ax_comm_world(const atlasx_ctx* ctx);
int ax_comm_rank(const atlasx_ctx* ctx);
int ax_comm_allreduce_sum(atlasx_ctx* ctx, float* buf_dev, size_t n);                         // in place, on ctx->stream
int ax_comm_allgather(atlasx_ctx* ctx, const float* send_dev, float* recv_dev, size_t n_each);
// Host wait for the context stream.  Single GPU: cudaStreamSynchronize.  With a communicator the
// host polls instead — stream completion, ncclCommGetAsyncError, and a deadline
// (ATLASX_COMM_TIMEOUT_MS, default 30 s) — so that a peer that never joins a collective ends in
// ATLASX_ERR_COMM / ATLASX_ERR_TIMEOUT on the host instead of an endless wait.
int ax_comm_stream_sync(atlasx_ctx* ctx);
// Collective over all ranks: allocates and exchanges the mailboxes for vectors of d floats.
// Returns ATLASX_OK with *out == nullptr when peer mapping is not possible (the caller keeps NCCL).
int ax_comm_peer_setup(atlasx_ctx* ctx, int d, const AxPeerMail** out);
void atlasx_comm_destroy(atlasx_ctx* ctx);
