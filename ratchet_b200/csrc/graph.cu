// Lazy tensor graph and its resolver: the host-side half of the device.
//
// Restates, in C++, what ratchet-core does in Rust between a model's `schedule()` and the GPU:
//   * `Tensor` = Arc<Inner{id, op, device, view, storage}> and the builder methods that validate
//     and compute the output view (tensor.rs:45-47,131-151,294-510; op.rs:12-31);
//   * `Tensor::execution_order`: iterative post-order DFS that visits a node's sources with
//     dependencies before its leaf sources (tensor.rs:696-740);
//   * `BufferAllocator::allocate_cfg`: liveness intervals over that order, largest-first greedy
//     sharing of buffers whose intervals do not overlap, in-place chains leasing the buffer of
//     their root (gpu/buffer_allocator/allocator.rs:141-340);
//   * `Tensor::resolve_gpu`: per node attach the buffer, decide in-place
//     (`supports_inplace() && srcs()[0].strong_count() == 1`, tensor.rs:823-824), run the op.
// Where the reference builds a compute pass of WGSL dispatches and submits it once, this resolver
// issues one CUDA kernel per node on the device's stream through the eager entry points.
//
// Two deliberate differences from the reference's planner:
//   * a `view` aliases its source's storage (as in tensor.rs:454-461), and here the source's buffer
//     also stays live until the last consumer of any of its views has run;
//   * a node that is still referenced from outside the graph being resolved (a handle the caller
//     keeps) gets a buffer of its own, so it stays readable after the resolve.
#include <algorithm>
#include <atomic>
#include <memory>
#include <unordered_set>

#include <cstdio>

#include "common.cuh"

namespace {

enum LazyKind {
    K_CONST = 0, K_VIEW, K_BINARY, K_UNARY, K_CAST, K_MATMUL, K_NORM, K_SOFTMAX, K_ROPE, K_CONCAT, K_SELECT,
    K_PERMUTE, K_SLICE, K_BROADCAST, K_CACHE, K_INDEX_WRITE, K_CONV
};

struct Storage {
    rcu_device* dev;
    void* ptr;
    uint64_t nbytes;
    bool owned;
    Storage(rcu_device* d, void* p, uint64_t n, bool o) : dev(d), ptr(p), nbytes(n), owned(o) {}
    Storage(const Storage&) = delete;              // exactly one owner returns the block to the pool
    Storage& operator=(const Storage&) = delete;
    ~Storage() {
        if (owned && ptr) rcu_free(dev, ptr);
    }
};

std::atomic<uint64_t> g_next_id{1};

}  // namespace

struct rcu_lazy {
    std::atomic<uint32_t> refs{1};
    uint64_t id = g_next_id++;
    int kind = K_CONST;
    rcu_device* dev = nullptr;
    int32_t dt = RCU_F32;
    uint32_t rank = 1;
    uint64_t shape[RCU_MAX_RANK] = {1, 1, 1, 1};
    std::vector<rcu_lazy*> srcs;   // each entry holds one reference
    // op parameters
    int op = 0;                    // binary / unary op, norm kind
    int flags[3] = {0, 0, 0};      // matmul transposes
    uint32_t u[4] = {0, 0, 0, 0};  // dim / offset / stride / padding / groups / perm
    uint64_t a[RCU_MAX_RANK] = {0, 0, 0, 0}, b[RCU_MAX_RANK] = {0, 0, 0, 0};   // slice start/stop, index_write start
    float f[2] = {0.f, 0.f};       // eps, rope base
    std::shared_ptr<Storage> storage;
    bool resident_const = false;   // uploaded from the host and waited for: nothing in flight writes it

    bool resolved() const { return storage != nullptr; }
    uint64_t numel() const {
        uint64_t n = 1;
        for (uint32_t i = 0; i < rank; ++i) n *= shape[i];
        return n;
    }
    uint64_t nbytes() const { return rcu_dtype_nbytes(dt, numel()); }
    rcu_tensor desc() const {
        rcu_tensor t;
        t.dt = dt;
        t.rank = rank;
        for (uint32_t i = 0; i < RCU_MAX_RANK; ++i) t.shape[i] = i < rank ? shape[i] : 1;
        t.data = storage ? storage->ptr : nullptr;
        return t;
    }
};

namespace {

void retain(rcu_lazy* t) { t->refs.fetch_add(1, std::memory_order_relaxed); }

void release(rcu_lazy* t) {
    // iterative: a long chain of nodes must not recurse through destructors
    std::vector<rcu_lazy*> work{t};
    while (!work.empty()) {
        rcu_lazy* n = work.back();
        work.pop_back();
        if (n->refs.fetch_sub(1, std::memory_order_acq_rel) == 1) {
            for (rcu_lazy* s : n->srcs) work.push_back(s);
            delete n;
        }
    }
}

rcu_lazy* new_node(rcu_device* dev, int kind, int32_t dt, uint32_t rank, const uint64_t* shape, std::initializer_list<rcu_lazy*> srcs) {
    rcu_lazy* n = new rcu_lazy();
    n->dev = dev;
    n->kind = kind;
    n->dt = dt;
    n->rank = rank;
    for (uint32_t i = 0; i < rank; ++i) n->shape[i] = shape[i];
    for (rcu_lazy* s : srcs)
        if (s) {
            retain(s);
            n->srcs.push_back(s);
        }
    return n;
}

bool supports_inplace(int kind) {
    // ops/binary.rs:179, ops/unary.rs:268, ops/softmax.rs:196, ops/rope.rs:80, ops/index_write.rs:49
    return kind == K_BINARY || kind == K_UNARY || kind == K_SOFTMAX || kind == K_ROPE || kind == K_INDEX_WRITE;
}

// The op about to overwrite `s`'s buffer must be the only thing that can still read it: `s` has one
// owner (tensor.rs:823-824) and, where `s` is a view, so has every tensor whose storage it aliases.
bool sole_owner(const rcu_lazy* s) {
    while (s->kind == K_VIEW) {
        if (s->refs.load() != 1) return false;
        s = s->srcs[0];
    }
    return s->refs.load() == 1;
}

#define LAZY_REQUIRE(dev, cond, ...)                                        \
    do {                                                                     \
        if (!(cond)) return rcu_fail((dev), RCU_ERR_INVALID_ARG, __VA_ARGS__); \
    } while (0)

// Shape::multi_broadcast (shape.rs:118-136)
bool multi_broadcast(const rcu_lazy* x, const rcu_lazy* y, uint32_t* rank, uint64_t* out) {
    const uint32_t r = std::max(x->rank, y->rank);
    for (uint32_t i = 0; i < r; ++i) {
        const uint64_t dx = i < x->rank ? x->shape[x->rank - 1 - i] : 1;
        const uint64_t dy = i < y->rank ? y->shape[y->rank - 1 - i] : 1;
        if (dx != 1 && dy != 1 && dx != dy) return false;
        out[r - 1 - i] = dx != 1 ? dx : dy;
    }
    *rank = r;
    return true;
}

// ------------------------------------------------------------------------------------------------
// execution order (tensor.rs:696-740): post-order walk without recursion.  A node's sources are visited
// leaves first, then the sources that have sources of their own — what the reference's
// `partition(|s| s.op().srcs().is_empty())` followed by `chain` does (its variable names say the
// opposite) — each group in the order the op lists them.  Meeting a node that is still open means the
// graph has a cycle.
// ------------------------------------------------------------------------------------------------
rcu_status execution_order(rcu_lazy* root, std::vector<rcu_lazy*>* order) {
    enum Mark : char { kOpen = 1, kDone = 2 };
    struct Frame {
        rcu_lazy* node;
        std::vector<rcu_lazy*> srcs;   // in visiting order
        size_t next;
    };
    auto open_frame = [](rcu_lazy* n) {
        Frame f{n, {}, 0};
        f.srcs.reserve(n->srcs.size());
        for (rcu_lazy* s : n->srcs)
            if (s->srcs.empty()) f.srcs.push_back(s);
        for (rcu_lazy* s : n->srcs)
            if (!s->srcs.empty()) f.srcs.push_back(s);
        return f;
    };
    std::unordered_map<uint64_t, Mark> mark;
    std::vector<Frame> stack;
    stack.push_back(open_frame(root));
    mark[root->id] = kOpen;
    while (!stack.empty()) {
        Frame& f = stack.back();
        if (f.next == f.srcs.size()) {
            mark[f.node->id] = kDone;
            order->push_back(f.node);
            stack.pop_back();
            continue;
        }
        rcu_lazy* pre = f.srcs[f.next++];
        auto it = mark.find(pre->id);
        if (it == mark.end()) {
            mark[pre->id] = kOpen;
            stack.push_back(open_frame(pre));      // invalidates `f`; nothing below uses it
        } else if (it->second == kOpen) {
            return rcu_fail(root->dev, RCU_ERR_INVALID_ARG, "Cycle detected whilst computing topological order: %llu", (unsigned long long)pre->id);
        }
    }
    return RCU_OK;
}

// Kernel key of a node for the per-op timing table (the reference keys its table by kernel name, gpu/profiler.rs:150-158).
const char* kind_name(int kind) {
    switch (kind) {
        case K_BINARY: return "binary";
        case K_UNARY: return "unary";
        case K_CAST: return "cast";
        case K_MATMUL: return "matmul";
        case K_NORM: return "norm";
        case K_SOFTMAX: return "softmax";
        case K_ROPE: return "rope";
        case K_CONCAT: return "concat";
        case K_SELECT: return "index_select";
        case K_PERMUTE: return "permute";
        case K_SLICE: return "slice";
        case K_BROADCAST: return "broadcast";
        case K_CACHE: return "cache";
        case K_INDEX_WRITE: return "index_write";
        case K_CONV: return "conv";
        default: return "other";
    }
}
const char* dt_name(int dt) {
    static const char* names[] = {"f32", "f16", "bf16", "i32", "u32", "q8_0f", "q8_0h", "q4_kf", "q4_kh"};
    return dt >= 0 && dt <= RCU_Q4_KH ? names[dt] : "?";
}

// ------------------------------------------------------------------------------------------------
// op dispatch
// ------------------------------------------------------------------------------------------------
rcu_status run_node(rcu_lazy* n) {
    rcu_device* dev = n->dev;
    rcu_tensor dst = n->desc();
    auto S = [&](size_t i) { return n->srcs[i]->desc(); };
    switch (n->kind) {
        case K_BINARY: { rcu_tensor x = S(0), y = S(1); return rcu_binary(dev, n->op, &x, &y, &dst); }
        case K_UNARY: { rcu_tensor x = S(0); return rcu_unary(dev, n->op, &x, &dst); }
        case K_CAST: { rcu_tensor x = S(0); return rcu_cast(dev, &x, &dst); }
        case K_MATMUL: {
            rcu_tensor l = S(0), r = S(1), bias;
            if (n->srcs.size() > 2) bias = S(2);
            // weights that were uploaded and waited for cannot be written by anything in flight: the GEMV may start early
            const bool before = dev->const_weights;
            if (n->srcs[0]->resident_const) dev->const_weights = true;
            const rcu_status st = rcu_matmul(dev, &l, &r, n->srcs.size() > 2 ? &bias : nullptr, n->flags[0], n->flags[1], n->flags[2], &dst);
            dev->const_weights = before;
            return st;
        }
        case K_NORM: {
            rcu_tensor x = S(0), sc = S(1), bias;
            if (n->srcs.size() > 2) bias = S(2);
            return rcu_norm(dev, n->op, &x, &sc, n->srcs.size() > 2 ? &bias : nullptr, n->f[0], n->u[0], &dst);
        }
        case K_SOFTMAX: { rcu_tensor x = S(0); return rcu_softmax(dev, &x, n->u[0], &dst); }
        case K_ROPE: { rcu_tensor x = S(0); return rcu_rope(dev, &x, n->u[0], n->f[1], n->u[1], &dst); }
        case K_CONCAT: {
            rcu_tensor descs[RCU_MAX_CONCAT];
            const rcu_tensor* ptrs[RCU_MAX_CONCAT];
            for (size_t i = 0; i < n->srcs.size(); ++i) { descs[i] = S(i); ptrs[i] = &descs[i]; }
            return rcu_concat(dev, ptrs, (uint32_t)n->srcs.size(), n->u[0], &dst);
        }
        case K_SELECT: { rcu_tensor s = S(0), ids = S(1); return rcu_index_select(dev, &s, &ids, n->u[0], &dst); }
        case K_PERMUTE: { rcu_tensor x = S(0); return rcu_permute(dev, &x, n->u, &dst); }
        case K_SLICE: { rcu_tensor x = S(0); return rcu_slice(dev, &x, n->a, n->b, &dst); }
        case K_BROADCAST: { rcu_tensor x = S(0); return rcu_broadcast(dev, &x, &dst); }
        case K_CACHE: { rcu_tensor c = S(0), s = S(1); return rcu_cache(dev, &c, &s, n->u[0], n->u[1], &dst); }
        case K_INDEX_WRITE: {
            // dst storage is srcs[0]'s when in place; otherwise copy srcs[0] first
            rcu_tensor d0 = S(0), s = S(1);
            if (dst.data != d0.data) {
                rcu_status st = rcu_d2d(dev, dst.data, d0.data, n->numel() * dt_esize(n->dt));
                if (st != RCU_OK) return st;
            }
            return rcu_index_write(dev, &dst, &s, n->a);
        }
        case K_CONV: {
            rcu_tensor x = S(0), w = S(1), bias;
            if (n->srcs.size() > 2) bias = S(2);
            return rcu_conv1d(dev, &x, &w, n->srcs.size() > 2 ? &bias : nullptr, n->u[0], n->u[1], &dst);
        }
        default: return rcu_fail(dev, RCU_ERR_UNSUPPORTED, "resolve: node kind %d has no kernel", n->kind);
    }
}

// ------------------------------------------------------------------------------------------------
// resolve (tensor.rs:795-859 + allocator.rs:209-340)
// ------------------------------------------------------------------------------------------------
struct Plan {
    rcu_lazy* root;           // node whose buffer this is
    size_t first, last;       // producer index, last consumer index in the execution order
    uint64_t size;
    bool exclusive;           // output / externally referenced: never shared
    int object = -1;
};

rcu_status resolve(rcu_lazy* out) {
    rcu_device* dev = out->dev;
    if (out->resolved()) return RCU_OK;
    std::vector<rcu_lazy*> order;
    rcu_status st = execution_order(out, &order);
    if (st != RCU_OK) return st;
    const size_t n = order.size();
    std::unordered_map<uint64_t, size_t> index;
    for (size_t i = 0; i < n; ++i) index[order[i]->id] = i;
    // Debug aid (the reference's RATCHET_DEBUG, gpu/buffer_allocator/allocator.rs:121): every tensor gets a buffer
    // of its own and nothing runs in place, so a wrong result that goes away points at the planner.
    const bool no_reuse = (dev->debug_flags & RCU_DEBUG_NO_REUSE) != 0;
    const bool profile = (dev->debug_flags & RCU_DEBUG_PROFILE) != 0;
    const bool log = (dev->debug_flags & RCU_DEBUG_LOG) != 0;

    // how many references to each node come from inside this graph
    std::unordered_map<uint64_t, uint32_t> internal_refs;
    for (rcu_lazy* t : order)
        for (rcu_lazy* s : t->srcs) internal_refs[s->id]++;

    // which node's buffer does each unresolved node write to?  view -> its source's; an op that runs
    // in place -> its first source's (the lease of allocator.rs:141-162); otherwise its own.
    std::vector<size_t> owner(n);
    std::vector<char> inplace(n, 0);
    for (size_t i = 0; i < n; ++i) {
        rcu_lazy* t = order[i];
        owner[i] = i;
        if (t->resolved() || t->srcs.empty()) continue;
        rcu_lazy* s0 = t->srcs[0];
        if (t->kind == K_VIEW) {
            owner[i] = owner[index[s0->id]];
        } else if (!no_reuse && supports_inplace(t->kind) && sole_owner(s0) && s0->dt == t->dt && s0->numel() == t->numel() &&
                   !(s0->resolved() && !s0->storage->owned)) {
            // the op is the sole owner of its first source (tensor.rs:823-824); a borrowed buffer
            // (rcu_lazy_wrap) is never written in place
            owner[i] = owner[index[s0->id]];
            inplace[i] = 1;
        }
    }
    // liveness per owning buffer
    std::vector<Plan> plans;
    std::unordered_map<size_t, size_t> plan_of;   // owner index -> plans index
    uint64_t naive = 0;
    for (size_t i = 0; i < n; ++i) {
        rcu_lazy* t = order[i];
        if (t->resolved()) continue;
        if (t->kind != K_VIEW) naive += t->nbytes();
        const size_t o = owner[i];
        if (order[o]->resolved()) continue;   // in place on (or view of) an already resolved tensor
        auto it = plan_of.find(o);
        if (it == plan_of.end()) {
            plan_of[o] = plans.size();
            plans.push_back(Plan{order[o], o, o, order[o]->nbytes(), false});
            it = plan_of.find(o);
        }
        Plan& p = plans[it->second];
        p.last = std::max(p.last, i);
        // externally held (or the output itself): keep the buffer out of the sharing pool
        if (no_reuse || t == out || t->refs.load() > internal_refs[t->id]) p.exclusive = true;
    }
    for (size_t i = 0; i < n; ++i) {
        rcu_lazy* t = order[i];
        if (t->resolved()) continue;
        for (rcu_lazy* s : t->srcs) {
            const size_t si = index[s->id];
            if (order[si]->resolved() && owner[si] == si) continue;
            auto it = plan_of.find(owner[si]);
            if (it != plan_of.end()) plans[it->second].last = std::max(plans[it->second].last, i);
        }
    }
    // greedy by size (arXiv 2001.03288, allocator.rs:209-271): largest first, reuse an object whose
    // assigned intervals do not overlap this one
    std::vector<size_t> by_size(plans.size());
    for (size_t i = 0; i < plans.size(); ++i) by_size[i] = i;
    std::stable_sort(by_size.begin(), by_size.end(), [&](size_t x, size_t y) { return plans[x].size > plans[y].size; });
    struct Object { uint64_t size; std::shared_ptr<Storage> storage; std::vector<size_t> users; bool exclusive; };
    std::vector<Object> objects;
    uint64_t planned = 0;
    for (size_t pi : by_size) {
        Plan& p = plans[pi];
        int best = -1;
        if (!p.exclusive) {
            for (size_t oi = 0; oi < objects.size(); ++oi) {
                if (objects[oi].exclusive || objects[oi].size < p.size) continue;
                bool ok = true;
                for (size_t u : objects[oi].users)
                    if (std::max(plans[u].first, p.first) <= std::min(plans[u].last, p.last)) { ok = false; break; }
                if (ok) best = (int)oi;
            }
        }
        if (best < 0) {
            void* ptr = nullptr;
            st = rcu_alloc(dev, p.size, &ptr);
            if (st != RCU_OK) return st;
            objects.push_back(Object{p.size, std::make_shared<Storage>(dev, ptr, p.size, true), {}, p.exclusive});
            planned += p.size;
            best = (int)objects.size() - 1;
        }
        objects[best].users.push_back(pi);
        p.object = best;
    }

    // run
    struct TimedNode { std::string key; uint64_t bytes; cudaEvent_t e0, e1; };
    std::vector<TimedNode> timed;
    uint32_t launched = 0, n_inplace = 0;
    const uint64_t launches0 = dev->launches;
    for (size_t i = 0; i < n; ++i) {
        rcu_lazy* t = order[i];
        if (t->resolved()) continue;
        const size_t o = owner[i];
        if (o == i) t->storage = objects[plans[plan_of[o]].object].storage;
        else t->storage = order[o]->storage;
        if (!t->storage) return rcu_fail(dev, RCU_ERR_INVALID_ARG, "resolve: tensor %llu has no storage", (unsigned long long)t->id);   // TensorError::NoStorage
        if (t->kind == K_VIEW || t->kind == K_CONST) continue;
        if (inplace[i]) ++n_inplace;
        if (log) {
            std::fprintf(stderr, "[rcu] node %llu %s %s [", (unsigned long long)t->id, kind_name(t->kind), dt_name(t->dt));
            for (uint32_t a = 0; a < t->rank; ++a) std::fprintf(stderr, a ? ", %llu" : "%llu", (unsigned long long)t->shape[a]);
            std::fprintf(stderr, "]%s\n", inplace[i] ? " in place" : "");
        }
        cudaEvent_t e0 = nullptr, e1 = nullptr;
        if (profile) {
            // one event pair per node, as the reference's timestamp-query pairs (gpu/profiler.rs:95-133)
            if (cudaEventCreate(&e0) != cudaSuccess || cudaEventCreate(&e1) != cudaSuccess) return rcu_fail(dev, RCU_ERR_CUDA, "resolve: cudaEventCreate");
            cudaEventRecord(e0, dev->stream);
        }
        st = run_node(t);
        if (st != RCU_OK) return st;
        if (profile) {
            cudaEventRecord(e1, dev->stream);
            uint64_t bytes = t->nbytes();
            for (rcu_lazy* s : t->srcs) bytes += s->nbytes();
            std::string key = std::string(kind_name(t->kind)) + " " + dt_name(t->srcs.empty() ? t->dt : t->srcs[0]->dt);
            timed.push_back(TimedNode{std::move(key), bytes, e0, e1});
        }
        ++launched;
    }
    if (profile) {
        cudaStreamSynchronize(dev->stream);
        for (TimedNode& tn : timed) {
            float ms = 0.f;
            cudaEventElapsedTime(&ms, tn.e0, tn.e1);
            rcu_device::OpTime& ot = dev->op_times[tn.key];
            ot.count += 1;
            ot.us += (double)ms * 1e3;
            ot.bytes += tn.bytes;
            cudaEventDestroy(tn.e0);
            cudaEventDestroy(tn.e1);
        }
    }
    dev->last_resolve.nodes = (uint32_t)n;
    dev->last_resolve.launched = (uint32_t)(dev->launches - launches0);
    dev->last_resolve.inplace = n_inplace;
    dev->last_resolve.buffers = (uint32_t)objects.size();
    dev->last_resolve.planned_bytes = planned;
    dev->last_resolve.naive_bytes = naive;
    (void)launched;
    if (log)
        std::fprintf(stderr, "[rcu] resolve: %zu nodes, %u launches, %u in place, %zu buffers, %llu bytes planned (%llu unshared)\n", n,
                     dev->last_resolve.launched, n_inplace, objects.size(), (unsigned long long)planned, (unsigned long long)naive);
    return RCU_OK;
}

rcu_status check_same_device(rcu_lazy* a, rcu_lazy* b) {
    if (a && b && a->dev != b->dev) return rcu_fail(a->dev, RCU_ERR_INVALID_ARG, "Mixed devices");
    return RCU_OK;
}

}  // namespace

extern "C" {

rcu_status rcu_lazy_from_host(rcu_device* dev, int32_t dt, uint32_t rank, const uint64_t* shape, const void* host, uint64_t nbytes, rcu_lazy** out) {
    if (!dev || !out || !shape || rank < 1 || rank > RCU_MAX_RANK) return RCU_ERR_INVALID_ARG;
    rcu_lazy* n = new_node(dev, K_CONST, dt, rank, shape, {});
    const uint64_t need = n->nbytes();
    void* ptr = nullptr;
    rcu_status st = rcu_alloc(dev, need, &ptr);
    if (st != RCU_OK) { delete n; return st; }
    n->storage = std::make_shared<Storage>(dev, ptr, need, true);
    if (host) {
        if (nbytes > need) nbytes = need;
        st = rcu_h2d(dev, ptr, host, nbytes);
        // the host buffer is borrowed for the call only: wait for the copy before returning
        if (st == RCU_OK) st = rcu_sync(dev);
        if (st != RCU_OK) { release(n); return st; }
        n->resident_const = true;
    }
    *out = n;
    return RCU_OK;
}

rcu_status rcu_lazy_zeros(rcu_device* dev, int32_t dt, uint32_t rank, const uint64_t* shape, rcu_lazy** out) {
    rcu_status st = rcu_lazy_from_host(dev, dt, rank, shape, nullptr, 0, out);
    if (st != RCU_OK) return st;
    return rcu_memset(dev, (*out)->storage->ptr, 0, (*out)->storage->nbytes);
}

rcu_status rcu_lazy_wrap(rcu_device* dev, const rcu_tensor* t, rcu_lazy** out) {
    if (!out || !t_valid(t)) return RCU_ERR_INVALID_ARG;      // dev may be NULL: a graph that is built and inspected, never resolved
    rcu_lazy* n = new_node(dev, K_CONST, t->dt, t->rank, t->shape, {});
    n->storage = std::make_shared<Storage>(dev, t->data, n->nbytes(), false);
    *out = n;
    return RCU_OK;
}

void rcu_lazy_retain(rcu_lazy* t) { if (t) retain(t); }
void rcu_lazy_release(rcu_lazy* t) { if (t) release(t); }

int rcu_lazy_info(const rcu_lazy* t, rcu_tensor* out) {
    if (!t || !out) return 0;
    *out = t->desc();
    return t->resolved() ? 1 : 0;
}

uint32_t rcu_lazy_strong_count(const rcu_lazy* t) { return t ? t->refs.load() : 0; }

rcu_status rcu_lazy_binary(int op, rcu_lazy* x, rcu_lazy* y, rcu_lazy** out) {
    if (!x || !y || !out) return RCU_ERR_INVALID_ARG;
    rcu_status st = check_same_device(x, y);
    if (st != RCU_OK) return st;
    LAZY_REQUIRE(x->dev, op >= RCU_ADD && op <= RCU_DIV, "binary: unknown op %d", op);
    LAZY_REQUIRE(x->dev, x->dt == y->dt, "binary: dtype mismatch %d vs %d", x->dt, y->dt);   // ops/binary.rs check_dtypes
    uint32_t rank;
    uint64_t shape[RCU_MAX_RANK];
    if (!multi_broadcast(x, y, &rank, shape)) return rcu_fail(x->dev, RCU_ERR_INVALID_ARG, "BroadcastingFailed");   // tensor.rs:258-261
    rcu_lazy* n = new_node(x->dev, K_BINARY, x->dt, rank, shape, {x, y});
    n->op = op;
    *out = n;
    return RCU_OK;
}

rcu_status rcu_lazy_unary(int op, rcu_lazy* x, rcu_lazy** out) {
    if (!x || !out) return RCU_ERR_INVALID_ARG;
    LAZY_REQUIRE(x->dev, op >= RCU_GELU && op <= RCU_SIGMOID, "unary: unknown op %d", op);
    LAZY_REQUIRE(x->dev, dt_is_float(x->dt), "unary: input must be a float tensor");
    rcu_lazy* n = new_node(x->dev, K_UNARY, x->dt, x->rank, x->shape, {x});
    n->op = op;
    *out = n;
    return RCU_OK;
}

rcu_status rcu_lazy_cast(rcu_lazy* x, int32_t dt, rcu_lazy** out) {
    if (!x || !out) return RCU_ERR_INVALID_ARG;
    if (x->dt == dt) {   // tensor.rs:315-318: casting to the same dtype returns the tensor itself
        retain(x);
        *out = x;
        return RCU_OK;
    }
    LAZY_REQUIRE(x->dev, !dt_is_quant(dt) && !dt_is_quant(x->dt), "cast: quantised dtypes cannot be cast");
    rcu_lazy* n = new_node(x->dev, K_CAST, dt, x->rank, x->shape, {x});
    *out = n;
    return RCU_OK;
}

rcu_status rcu_lazy_norm(int kind, rcu_lazy* x, rcu_lazy* scale, rcu_lazy* bias, float eps, uint32_t groups, rcu_lazy** out) {
    if (!x || !scale || !out) return RCU_ERR_INVALID_ARG;
    LAZY_REQUIRE(x->dev, kind >= RCU_LAYER_NORM && kind <= RCU_GROUP_NORM, "norm: unknown kind %d", kind);
    LAZY_REQUIRE(x->dev, x->rank >= 2, "norm: input rank must be at least 2");   // ops/norm/mod.rs check_shapes
    LAZY_REQUIRE(x->dev, kind == RCU_GROUP_NORM || scale->numel() == x->shape[x->rank - 1], "norm: scale length must equal the last dimension");
    rcu_lazy* n = new_node(x->dev, K_NORM, x->dt, x->rank, x->shape, {x, scale, bias});
    n->op = kind;
    n->f[0] = eps;
    n->u[0] = groups;
    *out = n;
    return RCU_OK;
}

rcu_status rcu_lazy_softmax(rcu_lazy* x, uint32_t dim, rcu_lazy** out) {
    if (!x || !out) return RCU_ERR_INVALID_ARG;
    LAZY_REQUIRE(x->dev, dim < x->rank, "softmax: dim %u out of range", dim);   // ops/softmax.rs check_custom
    rcu_lazy* n = new_node(x->dev, K_SOFTMAX, x->dt, x->rank, x->shape, {x});
    n->u[0] = dim;
    *out = n;
    return RCU_OK;
}

rcu_status rcu_lazy_rope(rcu_lazy* x, uint32_t dim, float base, uint32_t offset, rcu_lazy** out) {
    if (!x || !out) return RCU_ERR_INVALID_ARG;
    LAZY_REQUIRE(x->dev, x->rank == 4, "rope: input must be rank 4");   // ops/rope.rs check_shapes
    rcu_lazy* n = new_node(x->dev, K_ROPE, x->dt, x->rank, x->shape, {x});
    n->u[0] = dim;
    n->u[1] = offset;
    n->f[1] = base;
    *out = n;
    return RCU_OK;
}

rcu_status rcu_lazy_matmul(rcu_lazy* lhs, rcu_lazy* rhs, rcu_lazy* bias, int tl, int tr, int td, rcu_lazy** out) {
    if (!lhs || !rhs || !out) return RCU_ERR_INVALID_ARG;
    rcu_status st = check_same_device(lhs, rhs);
    if (st != RCU_OK) return st;
    rcu_tensor l = lhs->desc(), r = rhs->desc(), d;
    // descriptors of unresolved tensors have no data pointer; the shape rule does not need one
    st = rcu_matmul_dst_shape(&l, &r, tl, tr, td, &d);
    if (st != RCU_OK) return rcu_fail(lhs->dev, st, "Matmul broadcasting failed");
    rcu_lazy* n = new_node(lhs->dev, K_MATMUL, d.dt, d.rank, d.shape, {lhs, rhs, bias});
    n->flags[0] = tl; n->flags[1] = tr; n->flags[2] = td;
    *out = n;
    return RCU_OK;
}

rcu_status rcu_lazy_conv1d(rcu_lazy* x, rcu_lazy* w, rcu_lazy* bias, uint32_t stride, uint32_t padding, rcu_lazy** out) {
    if (!x || !w || !out) return RCU_ERR_INVALID_ARG;
    LAZY_REQUIRE(x->dev, x->rank == 3 && w->rank == 3, "conv1d: input and weight must be rank 3");
    LAZY_REQUIRE(x->dev, w->shape[2] == 3, "conv1d: only kernel size 3 is supported");   // ops/conv.rs:139-144
    LAZY_REQUIRE(x->dev, stride >= 1 && x->shape[2] + 2 * padding >= 3, "conv1d: bad stride/padding");
    // ops/conv.rs compute_view: [N, Cout, (Lin + 2p - (K-1) - 1)/s + 1]
    uint64_t shape[3] = {x->shape[0], w->shape[0], (x->shape[2] + 2 * padding - 3) / stride + 1};
    rcu_lazy* n = new_node(x->dev, K_CONV, x->dt, 3, shape, {x, w, bias});
    n->u[0] = stride;
    n->u[1] = padding;
    *out = n;
    return RCU_OK;
}

rcu_status rcu_lazy_view(rcu_lazy* x, uint32_t rank, const uint64_t* shape, rcu_lazy** out) {
    if (!x || !out || !shape || rank < 1 || rank > RCU_MAX_RANK) return RCU_ERR_INVALID_ARG;
    uint64_t nn = 1;
    for (uint32_t i = 0; i < rank; ++i) nn *= shape[i];
    LAZY_REQUIRE(x->dev, nn == x->numel(), "view: element count changes (%llu -> %llu)", (unsigned long long)x->numel(), (unsigned long long)nn);   // ops/view.rs
    LAZY_REQUIRE(x->dev, !dt_is_quant(x->dt), "view: quantised tensors cannot be reshaped");
    rcu_lazy* n = new_node(x->dev, K_VIEW, x->dt, rank, shape, {x});
    n->storage = x->storage;   // shares storage when the source is already resolved (tensor.rs:456)
    *out = n;
    return RCU_OK;
}

rcu_status rcu_lazy_slice(rcu_lazy* x, const uint64_t* start, const uint64_t* stop, rcu_lazy** out) {
    if (!x || !out || !start || !stop) return RCU_ERR_INVALID_ARG;
    uint64_t shape[RCU_MAX_RANK];
    for (uint32_t i = 0; i < x->rank; ++i) {
        LAZY_REQUIRE(x->dev, start[i] < stop[i] && stop[i] <= x->shape[i], "slice: bad range on axis %u", i);
        shape[i] = stop[i] - start[i];
    }
    rcu_lazy* n = new_node(x->dev, K_SLICE, x->dt, x->rank, shape, {x});
    for (uint32_t i = 0; i < x->rank; ++i) { n->a[i] = start[i]; n->b[i] = stop[i]; }
    *out = n;
    return RCU_OK;
}

rcu_status rcu_lazy_permute(rcu_lazy* x, const uint32_t* perm, rcu_lazy** out) {
    if (!x || !out || !perm) return RCU_ERR_INVALID_ARG;
    uint64_t shape[RCU_MAX_RANK];
    uint32_t seen = 0;
    for (uint32_t i = 0; i < x->rank; ++i) {
        LAZY_REQUIRE(x->dev, perm[i] < x->rank, "permute: axis out of range");
        seen |= 1u << perm[i];
        shape[i] = x->shape[perm[i]];
    }
    LAZY_REQUIRE(x->dev, seen == (1u << x->rank) - 1, "permute: dims must be unique");   // ops/reindex/permute.rs check_shapes
    rcu_lazy* n = new_node(x->dev, K_PERMUTE, x->dt, x->rank, shape, {x});
    for (uint32_t i = 0; i < x->rank; ++i) n->u[i] = perm[i];
    *out = n;
    return RCU_OK;
}

rcu_status rcu_lazy_broadcast(rcu_lazy* x, uint32_t rank, const uint64_t* shape, rcu_lazy** out) {
    if (!x || !out || !shape || rank < x->rank || rank > RCU_MAX_RANK) return RCU_ERR_INVALID_ARG;
    for (uint32_t i = 0; i < x->rank; ++i) {
        const uint64_t s = x->shape[x->rank - 1 - i], d = shape[rank - 1 - i];
        LAZY_REQUIRE(x->dev, s == d || s == 1, "broadcast: %llu does not broadcast to %llu", (unsigned long long)s, (unsigned long long)d);
    }
    rcu_lazy* n = new_node(x->dev, K_BROADCAST, x->dt, rank, shape, {x});
    *out = n;
    return RCU_OK;
}

rcu_status rcu_lazy_concat(rcu_lazy* const* inputs, uint32_t cnt, uint32_t dim, rcu_lazy** out) {
    if (!inputs || !out || cnt < 1) return RCU_ERR_INVALID_ARG;
    rcu_lazy* first = inputs[0];
    LAZY_REQUIRE(first->dev, cnt <= RCU_MAX_CONCAT, "concat: at most 8 inputs");   // ops/concat.rs:120-124
    LAZY_REQUIRE(first->dev, dim < first->rank, "concat: dim out of range");
    uint64_t shape[RCU_MAX_RANK];
    for (uint32_t i = 0; i < first->rank; ++i) shape[i] = first->shape[i];
    shape[dim] = 0;
    for (uint32_t k = 0; k < cnt; ++k) {
        LAZY_REQUIRE(first->dev, inputs[k] && inputs[k]->dev == first->dev, "Mixed devices");
        LAZY_REQUIRE(first->dev, inputs[k]->rank == first->rank && inputs[k]->dt == first->dt, "concat: rank/dtype mismatch");
        for (uint32_t i = 0; i < first->rank; ++i)
            LAZY_REQUIRE(first->dev, i == dim || inputs[k]->shape[i] == first->shape[i], "concat: shapes differ off the concat axis");
        shape[dim] += inputs[k]->shape[dim];
    }
    rcu_lazy* n = new_node(first->dev, K_CONCAT, first->dt, first->rank, shape, {});
    for (uint32_t k = 0; k < cnt; ++k) { retain(inputs[k]); n->srcs.push_back(inputs[k]); }
    n->u[0] = dim;
    *out = n;
    return RCU_OK;
}

rcu_status rcu_lazy_index_select(rcu_lazy* src, rcu_lazy* ids, uint32_t dim, rcu_lazy** out) {
    if (!src || !ids || !out) return RCU_ERR_INVALID_ARG;
    LAZY_REQUIRE(src->dev, src->rank == 2 && ids->rank == 1, "index_select: src must be rank 2 and indices rank 1");
    LAZY_REQUIRE(src->dev, ids->dt == RCU_I32, "index_select: indices must be I32");
    LAZY_REQUIRE(src->dev, dim < 2, "index_select: dim out of range");
    uint64_t shape[2] = {src->shape[0], src->shape[1]};
    shape[dim] = ids->shape[0];
    rcu_lazy* n = new_node(src->dev, K_SELECT, rcu_activation_dtype(src->dt), 2, shape, {src, ids});
    n->u[0] = dim;
    *out = n;
    return RCU_OK;
}

rcu_status rcu_lazy_cache(rcu_lazy* cache, rcu_lazy* src, uint32_t dim, uint32_t offset, rcu_lazy** out) {
    if (!cache || !src || !out) return RCU_ERR_INVALID_ARG;
    LAZY_REQUIRE(cache->dev, cache->rank == src->rank && cache->dt == src->dt && dim < cache->rank, "cache: rank/dtype mismatch");
    LAZY_REQUIRE(cache->dev, offset + src->shape[dim] <= cache->shape[dim], "cache: offset + length exceeds the cache");
    uint64_t shape[RCU_MAX_RANK];
    for (uint32_t i = 0; i < cache->rank; ++i) shape[i] = cache->shape[i];
    shape[dim] = offset + src->shape[dim];
    rcu_lazy* n = new_node(cache->dev, K_CACHE, cache->dt, cache->rank, shape, {cache, src});
    n->u[0] = dim;
    n->u[1] = offset;
    *out = n;
    return RCU_OK;
}

rcu_status rcu_lazy_index_write(rcu_lazy* dst, rcu_lazy* src, const uint64_t* start, rcu_lazy** out) {
    if (!dst || !src || !start || !out) return RCU_ERR_INVALID_ARG;
    LAZY_REQUIRE(dst->dev, dst->rank == src->rank && dst->dt == src->dt, "index_write: rank/dtype mismatch");
    for (uint32_t i = 0; i < dst->rank; ++i)
        LAZY_REQUIRE(dst->dev, start[i] + src->shape[i] <= dst->shape[i], "index_write: block exceeds dst on axis %u", i);
    rcu_lazy* n = new_node(dst->dev, K_INDEX_WRITE, dst->dt, dst->rank, dst->shape, {dst, src});
    for (uint32_t i = 0; i < dst->rank; ++i) n->a[i] = start[i];
    *out = n;
    return RCU_OK;
}

rcu_status rcu_lazy_resolve(rcu_lazy* t) {
    if (!t) return RCU_ERR_INVALID_ARG;
    if (!t->dev) return RCU_ERR_INVALID_ARG;                  // built without a device
    return resolve(t);
}

uint64_t rcu_lazy_id(const rcu_lazy* t) { return t ? t->id : 0; }

rcu_status rcu_lazy_execution_order(rcu_lazy* t, uint64_t* ids, uint32_t capacity, uint32_t* n_nodes) {
    if (!t || !n_nodes || (capacity && !ids)) return RCU_ERR_INVALID_ARG;
    std::vector<rcu_lazy*> order;
    const rcu_status st = execution_order(t, &order);
    if (st != RCU_OK) return st;
    *n_nodes = (uint32_t)order.size();
    for (size_t i = 0; i < order.size() && i < capacity; ++i) ids[i] = order[i]->id;
    return RCU_OK;
}

rcu_status rcu_set_debug(rcu_device* dev, uint32_t flags) {
    if (!dev) return RCU_ERR_INVALID_ARG;
    dev->debug_flags = flags;
    return RCU_OK;
}

uint64_t rcu_profile_report(rcu_device* dev, char* buf, uint64_t capacity, int reset) {
    if (!dev) return 0;
    double total = 0.0;
    for (auto& kv : dev->op_times) total += kv.second.us;
    std::vector<std::pair<std::string, rcu_device::OpTime>> rows(dev->op_times.begin(), dev->op_times.end());
    std::sort(rows.begin(), rows.end(), [](const auto& a, const auto& b) { return a.second.us > b.second.us; });
    std::string text = "kernel                    count     total us      %     GB/s\n";
    char line[160];
    for (auto& r : rows) {
        snprintf(line, sizeof(line), "%-24s %6llu %12.1f %6.1f %8.1f\n", r.first.c_str(), (unsigned long long)r.second.count, r.second.us,
                 total > 0 ? 100.0 * r.second.us / total : 0.0, r.second.us > 0 ? (double)r.second.bytes / r.second.us * 1e-3 : 0.0);
        text += line;
    }
    if (reset) dev->op_times.clear();
    if (buf && capacity) {
        const uint64_t n = std::min<uint64_t>(capacity - 1, text.size());
        memcpy(buf, text.data(), n);
        buf[n] = 0;
    }
    return text.size() + 1;
}

rcu_status rcu_lazy_to_host(rcu_lazy* t, void* host, uint64_t nbytes) {
    if (!t || !host) return RCU_ERR_INVALID_ARG;
    rcu_status st = resolve(t);
    if (st != RCU_OK) return st;
    const uint64_t have = dt_is_quant(t->dt) ? t->nbytes() : t->numel() * dt_esize(t->dt);
    if (nbytes > have) nbytes = have;
    return rcu_d2h(t->dev, host, t->storage->ptr, nbytes);
}

void rcu_last_resolve_stats(rcu_device* dev, rcu_resolve_stats* out) {
    if (dev && out) *out = dev->last_resolve;
}

}  // extern "C"
