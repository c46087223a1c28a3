// Peer-mapped exchange windows shared by the sharded GEMV entry point and the sharded decoder.
//
// One process per GPU.  Each rank allocates one window: kSlots full-size slots followed by an array of
// `world` arrival counters per slot and eight more words (the tickets and the use counts of the GEMV's three
// slots).  Windows are exported as CUDA IPC handles, exchanged by the host framework, and opened by every
// peer.  Data moves with plain peer stores issued by the producing GPU into the consumer's own HBM (all
// later reads are local).  The row-sharded GEMV signals completion with system-scope release increments
// of the consumer's arrival counters; the sharded decoder's exchanges carry their sequence number inside
// every word.  Either way the consumer's wait is a bounded spin.  No TMA, no multicast.
#pragma once
#include "gemv_q8.cuh"

namespace rcu_window {
constexpr int kSlots = 6;       // x (two, alternating), qkv, head outputs, MLP activations, logits: one per vector of a decode layer

struct Window {
    char* base = nullptr;
    size_t slot_bytes = 0;
    char* slot(int s) const { return base + (size_t)s * slot_bytes; }
    unsigned int* flags(int s, int world) const { return reinterpret_cast<unsigned int*>(base + kSlots * slot_bytes) + (size_t)s * world; }
    unsigned int* ticket(int world, int which = 0) const { return flags(kSlots, world) + which; }
    static size_t bytes(size_t slot_bytes, int world) { return kSlots * slot_bytes + (size_t)(kSlots * world + 8) * sizeof(unsigned int); }
};
}  // namespace rcu_window

struct rcu_comm {
    rcu_device* dev = nullptr;
    int rank = 0, world = 1;
    rcu_window::Window local;
    rcu_window::Window peers[gemvq8::kMaxPeers];   // peers[rank] == local
    bool opened[gemvq8::kMaxPeers] = {};           // imported through CUDA IPC (closed at destruction)
    bool linked[gemvq8::kMaxPeers] = {};           // another window of this process (rcu_comm_import_local)
    unsigned int seq = 0;          // host-side sequence of rcu_gemv_q8_allgather
    bool bound = false;            // a sharded decoder owns the flags of this window
};
