// Row-sharded Linear across the GPUs of one node: peer-mapped output buffers and a GEMV whose warps
// push their finished rows to every peer as they go (gemvq8::GatherEpilogueH), so the all-gather that
// follows a column-parallel Linear costs no extra collective launch.
//
// The reference has no multi-device path (gpu/device.rs:15-16 pins the ordinal to 0); this is the
// sharding its Linear (ratchet-nn/src/linear.rs:17-24) admits: the rows of W[N,K] are independent,
// Q8_0 blocks run along K inside a row, so rank r owns rows [r N/g, (r+1) N/g) as its own ratchet
// buffer and the only exchange is the gather of the output slices.
//
// One process per GPU.  Each rank allocates one "window" (comm.cuh): full-size output slots (this
// entry point rotates through the first three) followed by an array of `world` arrival counters per
// slot and the ticket / use-count words.  Windows are exported as CUDA IPC handles, exchanged by the
// host framework, and opened by every peer.  Data moves with plain peer stores issued by the producing
// GPU into the consumer's own HBM (all later reads are local); completion is a system-scope release
// increment of the consumer's arrival counter, one per producing CTA, which the consumer acquires with a
// bounded spin.  No TMA, no multicast.
#include "comm.cuh"
#include "ring.cuh"

namespace {
using rcu_window::Window;
using rcu_window::kSlots;
}  // namespace

extern "C" {

rcu_status rcu_comm_create(rcu_device* dev, int rank, int world, uint64_t slot_bytes, rcu_comm** out) {
    if (!dev || !out) return RCU_ERR_INVALID_ARG;
    RCU_REQUIRE(dev, world >= 1 && world <= gemvq8::kMaxPeers && rank >= 0 && rank < world, "comm: rank %d of %d", rank, world);
    RCU_REQUIRE(dev, slot_bytes % 16 == 0 && slot_bytes > 0, "comm: slot size must be a positive multiple of 16 bytes");
    DevGuard g(dev->ordinal);
    rcu_comm* c = new rcu_comm();
    c->dev = dev;
    c->rank = rank;
    c->world = world;
    c->local.slot_bytes = slot_bytes;
    const size_t total = Window::bytes(slot_bytes, world);
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, total);   // a dedicated allocation: IPC handles export whole allocations
    if (e != cudaSuccess) { delete c; return rcu_fail(dev, RCU_ERR_OOM, "comm: cudaMalloc(%zu): %s", total, cudaGetErrorString(e)); }
    c->local.base = (char*)p;
    cudaMemsetAsync(p, 0, total, dev->stream);
    cudaStreamSynchronize(dev->stream);
    c->peers[rank] = c->local;
    c->opened[rank] = false;
    *out = c;
    return RCU_OK;
}

rcu_status rcu_comm_export(rcu_comm* c, void* handle64) {
    if (!c || !handle64) return RCU_ERR_INVALID_ARG;
    DevGuard g(c->dev->ordinal);
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    RCU_CUDA(c->dev, cudaIpcGetMemHandle((cudaIpcMemHandle_t*)handle64, c->local.base));
    return RCU_OK;
}

rcu_status rcu_comm_import(rcu_comm* c, int peer, const void* handle64) {
    if (!c || !handle64) return RCU_ERR_INVALID_ARG;
    RCU_REQUIRE(c->dev, peer >= 0 && peer < c->world && peer != c->rank, "comm: bad peer %d", peer);
    DevGuard g(c->dev->ordinal);
    void* p = nullptr;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, sizeof(h));
    RCU_CUDA(c->dev, cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    c->peers[peer].base = (char*)p;
    c->peers[peer].slot_bytes = c->local.slot_bytes;
    c->opened[peer] = true;
    return RCU_OK;
}

rcu_status rcu_comm_import_local(rcu_comm* c, int peer, rcu_comm* other) {
    if (!c || !other) return RCU_ERR_INVALID_ARG;
    RCU_REQUIRE(c->dev, peer >= 0 && peer < c->world && peer != c->rank, "comm: bad peer %d", peer);
    RCU_REQUIRE(c->dev, other->rank == peer && other->world == c->world && other->local.slot_bytes == c->local.slot_bytes,
                "comm: the other window is not rank %d of the same exchange", peer);
    RCU_REQUIRE(c->dev, other->dev->ordinal == c->dev->ordinal, "comm: windows of one process are linked directly only on one device");
    c->peers[peer] = other->local;
    c->opened[peer] = false;             // nothing to close: the memory belongs to `other`
    c->linked[peer] = true;
    return RCU_OK;
}

void rcu_comm_destroy(rcu_comm* c) {
    if (!c) return;
    DevGuard g(c->dev->ordinal);
    cudaStreamSynchronize(c->dev->stream);
    for (int p = 0; p < c->world; ++p)
        if (c->opened[p]) cudaIpcCloseMemHandle(c->peers[p].base);
    cudaFree(c->local.base);
    delete c;
}

int rcu_comm_rank(const rcu_comm* c) { return c ? c->rank : -1; }
int rcu_comm_world(const rcu_comm* c) { return c ? c->world : 0; }

rcu_status rcu_gemv_q8_allgather(rcu_comm* c, const rcu_tensor* w_shard, const rcu_tensor* x, const rcu_tensor* bias_shard,
                                 void** y_full) {
    if (!c || !y_full) return RCU_ERR_INVALID_ARG;
    rcu_device* dev = c->dev;
    RCU_REQUIRE(dev, t_valid(w_shard) && t_valid(x), "gemv_allgather: invalid tensor descriptor");
    RCU_REQUIRE(dev, w_shard->rank == 2 && dt_is_q8(w_shard->dt) && x->dt == RCU_F16, "gemv_allgather: needs a Q8_0 [N/g, K] shard and f16 activations");
    const uint64_t n_local = w_shard->shape[0], K = w_shard->shape[1];
    RCU_REQUIRE(dev, t_numel(x) == K && K % 32 == 0, "gemv_allgather: x must hold K = %llu elements", (unsigned long long)K);
    RCU_REQUIRE(dev, n_local % 8 == 0, "gemv_allgather: shard rows must be a multiple of 8");
    RCU_REQUIRE(dev, n_local * c->world * 2 <= c->local.slot_bytes, "gemv_allgather: output (%llu B) exceeds the window slot", (unsigned long long)(n_local * c->world * 2));
    RCU_REQUIRE(dev, !bias_shard || (bias_shard->dt == RCU_F16 && t_numel(bias_shard) == n_local), "gemv_allgather: bias shard mismatch");
    for (int p = 0; p < c->world; ++p)
        RCU_REQUIRE(dev, p == c->rank || c->opened[p] || c->linked[p], "gemv_allgather: peer %d has not been imported", p);
    DevGuard g(dev->ordinal);
    RCU_REQUIRE(dev, !c->bound, "gemv_allgather: this window belongs to a sharded decoder");
    // Three output slots in rotation: a result stays valid until the call after next, and a peer that is one
    // call ahead writes a slot nobody reads any more.
    const int slot = (int)(c->seq++ % 3u);
    gemvq8::GatherEpilogueH epi;
    epi.bias = bias_shard ? (const __half*)bias_shard->data : nullptr;
    epi.y_local = reinterpret_cast<__half*>(c->local.slot(slot)) + (size_t)c->rank * n_local;
    epi.ticket = c->local.ticket(c->world, slot);           // per slot: the next call's CTAs may start (and count) while this call's last CTA still waits
    epi.uses = c->local.ticket(c->world, 3 + slot);
    epi.n_peers = 0;
    for (int p = 0; p < c->world; ++p) {
        if (p == c->rank) continue;
        epi.peer_dst[epi.n_peers] = reinterpret_cast<__half*>(c->peers[p].slot(slot)) + (size_t)c->rank * n_local;
        epi.peer_count[epi.n_peers] = c->peers[p].flags(slot, c->world) + c->rank;
        epi.n_peers++;
    }
    epi.my_counts = c->local.flags(slot, c->world);
    epi.world = c->world;
    epi.self = c->rank;
    epi.status = dev->d_status;
    const int8_t* qs = (const int8_t*)w_shard->data;
    const void* sc = (const char*)w_shard->data + align256(n_local * K);
    // Every rank must launch the same grid (a CTA counts once on every peer): the choice of kernel and its grid
    // depend on the shard's shape and the device alone.
    rcu_status st = RCU_ERR_UNSUPPORTED;
    if (K >= 2048) {
        ringq8::PlainPlanes<ringq8::VecSource> rpro{{(const __half*)x->data}};
        // Programmatic dependent launch: until griddepcontrol.wait the kernel only requests weights into its rings, so
        // its start overlaps the previous call's wait for the peers.
        st = w_shard->dt == RCU_Q8_0H ? ringq8::launch<__half>(dev, qs, sc, rpro, epi, (int)n_local, (int)K, true)
                                      : ringq8::launch<float>(dev, qs, sc, rpro, epi, (int)n_local, (int)K, true);
    }
    if (st == RCU_ERR_UNSUPPORTED) {
        gemvq8::PlainPrologue<__half> pro{(const __half*)x->data};
        st = w_shard->dt == RCU_Q8_0H ? gemvq8::launch<__half, __half, 2>(dev, qs, sc, pro, epi, (int)n_local, (int)K, false, 3, true)
                                      : gemvq8::launch<float, __half, 2>(dev, qs, sc, pro, epi, (int)n_local, (int)K, false, 3, true);
    }
    if (st != RCU_OK) return st;
    *y_full = c->local.slot(slot);
    return RCU_OK;
}

}  // extern "C"
