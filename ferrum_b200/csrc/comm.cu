// All-gather of row-sharded projection outputs over NVLink peer memory (one process per GPU).
//
// The reference is single-GPU; this is the exchange step of this build's tensor-parallel sharding.  The
// payloads are tiny (M = 1: a few KB per rank and projection), so the cost is latency, and a library
// collective per projection would cost more than the projection.  Each rank owns one "symmetric" buffer
// (same size and layout on every rank, mapped into every peer through CUDA IPC).  A projection writes its
// shard straight into its own slice of the gathered region; `fq_comm_all_gather` is then ONE small kernel:
// block p stores the local shard into peer p's copy of the region (plain peer stores), publishes a sequence
// number in peer p's flag word (release, system scope), and waits -- bounded -- until peer p's sequence number
// for the same call site has arrived locally.  When the kernel ends every shard is in local memory, and stream
// order makes it visible to whatever runs next.  Nothing here uses multicast or TMA; the kernel can be
// captured into a graph because sequence numbers live in device memory.
#include <algorithm>
#include <cstdlib>
#include <cstring>

#include "internal.h"

constexpr int FQ_COMM_MAX_WORLD = 8;
constexpr uint32_t FQ_COMM_SLOTS = 2048;      // distinct call sites before flag words are reused

struct fq_comm {
    fq_device *dev = nullptr;
    int rank = 0, world = 1;
    size_t bytes = 0;       // payload bytes of the symmetric buffer
    uint8_t *local = nullptr; // payload, then flags[FQ_COMM_SLOTS][FQ_COMM_MAX_WORLD]
    uint32_t *seq = nullptr;  // local only: last sequence number used per (slot, peer)
    uint8_t *peer[FQ_COMM_MAX_WORLD] = {};
    bool opened = false;
    uint32_t next_slot = 0;
    uint64_t wait_ns = 2000000000ull; // wall-time limit of every device-side wait for a peer
    uint8_t *fake_peer = nullptr;     // fq_comm_open_local: a second local buffer standing in for the peers
    // The region of the exchange enqueued last (eagerly or by the last graph replayed): the next exchange must
    // not touch it, because a rank that runs ahead would overwrite what a slower peer is still reading.
    size_t last_off = 0, last_bytes = 0;
};

namespace {

struct Peers {
    uint8_t *base[FQ_COMM_MAX_WORLD];
};

// After the blocks of grid column `other` have stored their share into that peer's buffer: the stores are made
// visible, the chunks are counted in, and the last chunk's first thread raises this rank's flag in the peer's
// flag words and waits -- bounded by wall time -- for the peer's flag for the same call site.
__device__ __forceinline__ void finish_push(const Peers &peers, int rank, int other, size_t payload_bytes, uint32_t slot, uint32_t *seq,
                                            uint64_t wait_ns, int *status) {
    __threadfence_system();
    __syncthreads();
    __shared__ bool last;
    uint32_t *done = seq + (size_t)FQ_COMM_SLOTS * FQ_COMM_MAX_WORLD * 2 + (size_t)slot * FQ_COMM_MAX_WORLD + other;
    if (threadIdx.x == 0) last = atomicAdd(done, 1u) + 1u == gridDim.y;
    __syncthreads();
    if (!last || threadIdx.x != 0) return;
    *done = 0;
    uint32_t *my_seq = seq + (size_t)slot * FQ_COMM_MAX_WORLD + other;
    const uint32_t expect = *my_seq + 1u;
    *my_seq = expect;
    __threadfence_system();
    // flags[slot][sender] on the receiving rank
    uint32_t *remote_flag = reinterpret_cast<uint32_t *>(peers.base[other] + payload_bytes) + (size_t)slot * FQ_COMM_MAX_WORLD + rank;
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(remote_flag), "r"(expect) : "memory");
    const uint32_t *local_flag = reinterpret_cast<const uint32_t *>(peers.base[rank] + payload_bytes) + (size_t)slot * FQ_COMM_MAX_WORLD + other;
    uint64_t t0 = 0;
    for (uint32_t i = 0;; i++) {
        uint32_t v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(local_flag) : "memory");
        if ((int32_t)(v - expect) >= 0) return;
        __nanosleep(20);
        if ((i & 63u) == 63u) { // wall-time limit
            uint64_t now;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
            if (t0 == 0) t0 = now;
            else if (now - t0 > wait_ns) break;
        }
    }
    *(volatile int *)status = (int)FQ_ERR_TIMEOUT; // the peer never arrived: report, do not hang
}

// grid (world - 1, chunks): block (p, c) copies chunk c of the shard to the p-th other rank; the last chunk's
// block also does the handshake with that rank.
// With `bounds` (device memory, written by an earlier kernel of the stream) the shards are runs of rows of
// unequal length: rank r owns rows bounds[r * stride] .. bounds[(r + 1) * stride] of `shard_bytes` bytes each,
// laid out from region_off in row order (the expert-sorted rows of an expert-parallel MoE block).
__global__ void __launch_bounds__(256)
k_all_gather_push(const __grid_constant__ Peers peers, int rank, int world, size_t payload_bytes, size_t region_off,
                  size_t shard_bytes, const uint32_t *__restrict__ bounds, uint32_t stride, uint32_t slot, uint32_t *seq, uint64_t wait_ns,
                  int *status) {
    // Launched with programmatic stream serialization: let the next kernel stage itself, then wait for the
    // projection that produced the local shard.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int other = (int)blockIdx.x < rank ? (int)blockIdx.x : (int)blockIdx.x + 1;
    size_t mine = region_off + (size_t)rank * shard_bytes;
    if (bounds) {
        const uint32_t lo = bounds[(size_t)rank * stride], hi = bounds[(size_t)(rank + 1) * stride];
        mine = region_off + (size_t)lo * shard_bytes;
        shard_bytes *= hi - lo;
    }
    const uint4 *src = reinterpret_cast<const uint4 *>(peers.base[rank] + mine);
    uint4 *dst = reinterpret_cast<uint4 *>(peers.base[other] + mine);
    const size_t n16 = shard_bytes / 16;
    for (size_t i = (size_t)blockIdx.y * blockDim.x + threadIdx.x; i < n16; i += (size_t)gridDim.y * blockDim.x) dst[i] = src[i];
    finish_push(peers, rank, other, payload_bytes, slot, seq, wait_ns, status);
}

// The dispatch half of an all-to-all over expert-sorted rows: of this rank's run of rows
// [bounds[rank * stride], bounds[(rank + 1) * stride]) -- the rows its experts produced -- row p goes ONLY to the
// rank that owns its token, sorted[p] / used / tokens_per_rank, at the same place in that rank's buffer.  Same
// grid and handshake as the gather: block (p, c) serves the p-th other rank.
__global__ void __launch_bounds__(256)
k_dispatch_rows(const __grid_constant__ Peers peers, int rank, int world, size_t payload_bytes, size_t region_off, size_t row_bytes,
                const uint32_t *__restrict__ bounds, uint32_t stride, const uint32_t *__restrict__ sorted, uint32_t used, uint32_t tokens_per_rank,
                uint32_t slot, uint32_t *seq, uint64_t wait_ns, int *status) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int other = (int)blockIdx.x < rank ? (int)blockIdx.x : (int)blockIdx.x + 1;
    const uint32_t lo = bounds[(size_t)rank * stride], hi = bounds[(size_t)(rank + 1) * stride];
    const size_t n16 = row_bytes / 16;
    for (uint32_t row = lo + blockIdx.y; row < hi; row += gridDim.y) {
        const uint32_t owner = min(sorted[row] / used / tokens_per_rank, (uint32_t)world - 1u);
        if ((int)owner != other) continue;
        const size_t at = region_off + (size_t)row * row_bytes;
        const uint4 *src = reinterpret_cast<const uint4 *>(peers.base[rank] + at);
        uint4 *dst = reinterpret_cast<uint4 *>(peers.base[other] + at);
        for (size_t i = threadIdx.x; i < n16; i += blockDim.x) dst[i] = src[i];
    }
    finish_push(peers, rank, other, payload_bytes, slot, seq, wait_ns, status);
}

size_t flag_bytes() { return (size_t)FQ_COMM_SLOTS * FQ_COMM_MAX_WORLD * sizeof(uint32_t); }

} // namespace

extern "C" int fq_comm_create(fq_device *dev, int rank, int world, size_t bytes, fq_comm **out) {
    if (!dev || !out) return FQ_ERR_PARAM;
    *out = nullptr;
    if (world < 1 || world > FQ_COMM_MAX_WORLD || rank < 0 || rank >= world || bytes == 0 || bytes % 256)
        return fq_fail(dev, FQ_ERR_PARAM, "communicator of rank %d / %d with %zu bytes (a multiple of 256, at most %d ranks)", rank, world, bytes, FQ_COMM_MAX_WORLD);
    if (int rc = fq_check_cuda(dev, cudaSetDevice(dev->ordinal), "cudaSetDevice")) return rc;
    fq_comm *c = new fq_comm();
    c->dev = dev;
    c->rank = rank;
    c->world = world;
    c->bytes = bytes;
    // payload | flag words | mirror of {value, sequence number} slots for the fused exchange (8 bytes per float)
    cudaError_t e = cudaMalloc((void **)&c->local, bytes + flag_bytes() + 2 * bytes);
    if (e == cudaSuccess) e = cudaMemset(c->local, 0, bytes + flag_bytes() + 2 * bytes);
    if (e == cudaSuccess) e = cudaMalloc((void **)&c->seq, flag_bytes() * 3);
    if (e == cudaSuccess) e = cudaMemset(c->seq, 0, flag_bytes() * 3);
    if (e != cudaSuccess) {
        if (c->local) cudaFree(c->local);
        if (c->seq) cudaFree(c->seq);
        delete c;
        return fq_check_cuda(dev, e, "symmetric buffer");
    }
    c->peer[rank] = c->local;
    c->opened = world == 1;
    *out = c;
    return FQ_OK;
}

extern "C" int fq_comm_handle(fq_comm *c, void *out64) {
    if (!c || !out64) return FQ_ERR_PARAM;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    cudaIpcMemHandle_t h;
    if (int rc = fq_check_cuda(c->dev, cudaIpcGetMemHandle(&h, c->local), "cudaIpcGetMemHandle")) return rc;
    memcpy(out64, &h, 64);
    return FQ_OK;
}

extern "C" int fq_comm_open(fq_comm *c, const void *handles) {
    if (!c || !handles) return FQ_ERR_PARAM;
    cudaSetDevice(c->dev->ordinal);
    for (int r = 0; r < c->world; r++) {
        if (r == c->rank) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, (const uint8_t *)handles + 64 * r, 64);
        void *p = nullptr;
        if (int rc = fq_check_cuda(c->dev, cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle")) return rc;
        c->peer[r] = (uint8_t *)p;
    }
    c->opened = true;
    return FQ_OK;
}

// Test-only: a communicator of world 2 whose "peer" is a second local buffer that nothing ever writes, so that
// every wait for the peer runs out (on one GPU, without a second process).
extern "C" int fq_comm_open_local(fq_comm *c) {
    if (!c) return FQ_ERR_PARAM;
    if (c->world != 2 || c->opened) return fq_fail(c->dev, FQ_ERR_PARAM, "a local stand-in peer needs an unopened communicator of two ranks");
    cudaSetDevice(c->dev->ordinal);
    const size_t total = c->bytes + flag_bytes() + 2 * c->bytes;
    cudaError_t e = cudaMalloc((void **)&c->fake_peer, total);
    if (e == cudaSuccess) e = cudaMemset(c->fake_peer, 0, total);
    if (int rc = fq_check_cuda(c->dev, e, "stand-in peer buffer")) return rc;
    c->peer[1 - c->rank] = c->fake_peer;
    c->opened = true;
    return FQ_OK;
}

// Wall-time limit of the device-side waits of this communicator's exchanges (default 2 s).
extern "C" int fq_comm_set_wait_ns(fq_comm *c, uint64_t ns) {
    if (!c || ns == 0) return FQ_ERR_PARAM;
    c->wait_ns = ns;
    return FQ_OK;
}

extern "C" void *fq_comm_buffer(fq_comm *c) { return c ? c->local : nullptr; }

// Every exchange passes here before it is enqueued: consecutive exchanges of a communicator must use disjoint
// regions.  While the handle records a graph, the graph remembers its first and last region instead, and
// `fq_graph_launch` repeats the check against what ran before it.
int fq_comm_note_region(fq_device *dev, fq_comm *c, size_t off, size_t bytes) {
    if (c->world == 1) return FQ_OK;
    if (dev->capturing) {
        if (dev->cap_comm && dev->cap_comm != c) return fq_fail(dev, FQ_ERR_PARAM, "one communicator per recorded graph");
        if (dev->cap_comm && off < dev->cap_last_off + dev->cap_last_bytes && dev->cap_last_off < off + bytes)
            return fq_fail(dev, FQ_ERR_PARAM, "exchange region [%zu, +%zu) was also the region of the exchange before it; alternate regions", off, bytes);
        if (!dev->cap_comm) {
            dev->cap_comm = c;
            dev->cap_first_off = off;
            dev->cap_first_bytes = bytes;
        }
        dev->cap_last_off = off;
        dev->cap_last_bytes = bytes;
        return FQ_OK;
    }
    if (c->last_bytes && off < c->last_off + c->last_bytes && c->last_off < off + bytes)
        return fq_fail(dev, FQ_ERR_PARAM, "exchange region [%zu, +%zu) was also the region of the exchange before it; alternate regions", off, bytes);
    c->last_off = off;
    c->last_bytes = bytes;
    return FQ_OK;
}
int fq_comm_note_graph(fq_device *dev, const fq_graph *g) {
    fq_comm *c = g->comm;
    if (!c) return FQ_OK;
    if (c->last_bytes && g->first_off < c->last_off + c->last_bytes && c->last_off < g->first_off + g->first_bytes)
        return fq_fail(dev, FQ_ERR_PARAM, "the graph's first exchange uses the region of the exchange before it; alternate regions");
    c->last_off = g->last_off;
    c->last_bytes = g->last_bytes;
    return FQ_OK;
}
int fq_comm_begin_push(fq_comm *c, const void *y, size_t bytes, TpPush *out) {
    const uint8_t *p = (const uint8_t *)y;
    if (!c->opened || p < c->local || p + bytes > c->local + c->bytes) return FQ_ERR_RANGE;
    for (int r = 0; r < FQ_COMM_MAX_WORLD; r++) out->peer[r] = r < c->world ? c->peer[r] : nullptr;
    out->world = (uint32_t)c->world;
    out->rank = (uint32_t)c->rank;
    out->pad = 0;
    out->slot = c->next_slot;
    c->next_slot = (c->next_slot + 1) % FQ_COMM_SLOTS;
    out->epoch = c->seq + (size_t)FQ_COMM_SLOTS * FQ_COMM_MAX_WORLD; // a word of the local bookkeeping array nothing else uses
    out->counter = c->seq + (size_t)FQ_COMM_SLOTS * FQ_COMM_MAX_WORLD * 2 + (size_t)out->slot * FQ_COMM_MAX_WORLD; // the slot's chunk counters
    out->mirror_off = c->bytes + flag_bytes();
    out->slice_off = (size_t)(p - c->local);
    out->slice_bytes = bytes;
    out->covered_bytes = bytes; // the caller lowers it when its outputs do not fill the slice
    out->wait_ns = c->wait_ns;
    out->status = c->dev->status_dev;
    return FQ_OK;
}
uint8_t *fq_comm_local(fq_comm *c) { return c->local; }
fq_device *fq_comm_device(const fq_comm *c) { return c->dev; }
size_t fq_comm_bytes(const fq_comm *c) { return c->bytes; }
int fq_comm_rank(const fq_comm *c) { return c->rank; }
int fq_comm_world(const fq_comm *c) { return c->world; }

static int launch_gather(fq_device *dev, fq_comm *c, size_t region_offset, size_t shard_bytes, const uint32_t *bounds, uint32_t stride,
                         size_t most_bytes) {
    Peers peers{};
    for (int r = 0; r < c->world; r++) peers.base[r] = c->peer[r];
    const uint32_t slot = c->next_slot;
    c->next_slot = (c->next_slot + 1) % FQ_COMM_SLOTS;
    const unsigned chunks = (unsigned)std::min<size_t>(32, std::max<size_t>(1, most_bytes / (256 * 16 * 4)));
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(c->world - 1, chunks);
    cfg.blockDim = dim3(256);
    cfg.stream = dev->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (int rc = fq_check_cuda(dev, cudaLaunchKernelEx(&cfg, k_all_gather_push, peers, c->rank, c->world, c->bytes, region_offset,
                                                       shard_bytes, bounds, stride, slot, c->seq, c->wait_ns, dev->status_dev), "all-gather launch"))
        return rc;
    return fq_end_enqueue(dev, "all_gather", 1);
}

extern "C" int fq_comm_all_gather(fq_device *dev, fq_comm *c, size_t region_offset, size_t shard_bytes) {
    if (int rc = fq_begin_enqueue(dev)) return rc;
    if (!c || c->dev != dev) return fq_fail(dev, FQ_ERR_DEVICE, "communicator belongs to another device handle");
    if (!c->opened) return fq_fail(dev, FQ_ERR_PARAM, "communicator peers are not opened");
    if (shard_bytes == 0 || shard_bytes % 16 || region_offset % 16 || region_offset + shard_bytes * c->world > c->bytes)
        return fq_fail(dev, FQ_ERR_RANGE, "gather of %zu bytes per rank at offset %zu does not fit %zu bytes", shard_bytes, region_offset, c->bytes);
    if (c->world == 1) return FQ_OK;
    if (int rc = fq_comm_note_region(dev, c, region_offset, shard_bytes * c->world)) return rc;
    return launch_gather(dev, c, region_offset, shard_bytes, nullptr, 0, shard_bytes);
}

// The gather of a region whose use has been noted already (the fallback of fq_project_many_gather).
int fq_comm_all_gather_unchecked(fq_device *dev, fq_comm *c, size_t region_offset, size_t shard_bytes) {
    if (int rc = fq_begin_enqueue(dev)) return rc;
    return launch_gather(dev, c, region_offset, shard_bytes, nullptr, 0, shard_bytes);
}

extern "C" int fq_comm_all_gather_rows(fq_device *dev, fq_comm *c, size_t region_offset, size_t row_bytes, const uint32_t *bounds,
                                       uint32_t stride, size_t total_rows) {
    if (int rc = fq_begin_enqueue(dev)) return rc;
    if (!c || c->dev != dev) return fq_fail(dev, FQ_ERR_DEVICE, "communicator belongs to another device handle");
    if (!c->opened) return fq_fail(dev, FQ_ERR_PARAM, "communicator peers are not opened");
    if (row_bytes == 0 || row_bytes % 16 || region_offset % 16 || stride == 0 || total_rows == 0 || region_offset + row_bytes * total_rows > c->bytes)
        return fq_fail(dev, FQ_ERR_RANGE, "gather of %zu rows of %zu bytes at offset %zu does not fit %zu bytes", total_rows, row_bytes, region_offset, c->bytes);
    if (int rc = fq_check_binding(dev, bounds, ((size_t)c->world * stride + 1) * 4, "bounds")) return rc;
    if (c->world == 1) return FQ_OK;
    if (int rc = fq_comm_note_region(dev, c, region_offset, row_bytes * total_rows)) return rc;
    return launch_gather(dev, c, region_offset, row_bytes, bounds, stride, row_bytes * total_rows / c->world);
}

// Rows of this rank's run to the ranks that own their tokens (see k_dispatch_rows); every rank makes the call.
int fq_comm_dispatch_rows(fq_device *dev, fq_comm *c, size_t region_offset, size_t row_bytes, const uint32_t *bounds, uint32_t stride,
                          const uint32_t *sorted, uint32_t used, uint32_t tokens_per_rank, size_t total_rows) {
    if (int rc = fq_begin_enqueue(dev)) return rc;
    if (!c || c->dev != dev) return fq_fail(dev, FQ_ERR_DEVICE, "communicator belongs to another device handle");
    if (!c->opened) return fq_fail(dev, FQ_ERR_PARAM, "communicator peers are not opened");
    if (row_bytes == 0 || row_bytes % 16 || region_offset % 16 || stride == 0 || used == 0 || tokens_per_rank == 0 ||
        region_offset + row_bytes * total_rows > c->bytes)
        return fq_fail(dev, FQ_ERR_RANGE, "dispatch of %zu rows of %zu bytes at offset %zu does not fit %zu bytes", total_rows, row_bytes, region_offset, c->bytes);
    if (c->world == 1) return FQ_OK;
    if (int rc = fq_comm_note_region(dev, c, region_offset, row_bytes * total_rows)) return rc;
    Peers peers{};
    for (int r = 0; r < c->world; r++) peers.base[r] = c->peer[r];
    const uint32_t slot = c->next_slot;
    c->next_slot = (c->next_slot + 1) % FQ_COMM_SLOTS;
    const unsigned chunks = (unsigned)std::min<size_t>(64, std::max<size_t>(1, total_rows / c->world / 8));
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(c->world - 1, chunks);
    cfg.blockDim = dim3(256);
    cfg.stream = dev->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (int rc = fq_check_cuda(dev, cudaLaunchKernelEx(&cfg, k_dispatch_rows, peers, c->rank, c->world, c->bytes, region_offset, row_bytes, bounds,
                                                       stride, sorted, used, tokens_per_rank, slot, c->seq, c->wait_ns, dev->status_dev),
                               "row dispatch launch"))
        return rc;
    return fq_end_enqueue(dev, "dispatch_rows", 1);
}

extern "C" int fq_comm_destroy(fq_comm *c) {
    if (!c) return FQ_ERR_PARAM;
    cudaSetDevice(c->dev->ordinal);
    cudaStreamSynchronize(c->dev->stream);
    for (int r = 0; r < c->world; r++)
        if (r != c->rank && c->peer[r] && c->peer[r] != c->fake_peer) cudaIpcCloseMemHandle(c->peer[r]);
    if (c->fake_peer) cudaFree(c->fake_peer);
    cudaFree(c->local);
    cudaFree(c->seq);
    delete c;
    return FQ_OK;
}
