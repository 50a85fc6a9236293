// Mixture-of-experts glue: routing, expert-major map, gather, combine and the gated unit.
// Contracts follow the reference kernels h_moe_route / h_moe_map / h_moe_gather / h_moe_combine /
// h_swiglu (src/metal/shaders/hybrid.metal:2252-2388, 1606-1613).
#include <cooperative_groups.h>
#include <cuda_bf16.h>

#include "gemv_common.cuh"
#include "internal.h"

namespace {

constexpr int ROUTE_WARPS = 4;    // tokens per block of the routing kernel: one warp each
constexpr int MAX_EXPERTS = 1024; // the reference's map kernel holds counts[1024]

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
}

// One warp per token (no block-wide barrier anywhere: a decode step's single token is one warp's latency).
// Scores: softmax over the logits (max, exp, sum, divide) or a logistic per logit; `used` rounds of arg-max
// with ties to the lower index; weights divided by the picked sum when `norm`; shared-expert gate =
// logistic(dot(x, shared_w)) or 1.  Lane l owns experts l, l + 32, ...
__device__ __forceinline__ void route_token(float *route_smem, const float *__restrict__ logits, const float *__restrict__ x,
                                            const float *__restrict__ shared_w, uint32_t experts, uint32_t used, uint32_t hidden, uint32_t tokens,
                                            int sigmoid, int norm, int shared_gate, uint32_t *__restrict__ ids, float *__restrict__ weights,
                                            float *__restrict__ gate, int *status) {
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t t = blockIdx.x * ROUTE_WARPS + warp;
    if (t >= tokens) return;
    float *prob = route_smem + (size_t)warp * experts;
    const float *row = logits + (size_t)t * experts;
    // A NaN or an infinity among the logits has no ranking (the reference's router refuses such a row:
    // "router produced invalid logits", src/nn/moe.rs:392-397): report it through the status word, give the token
    // the first `used` experts with weight zero so that everything downstream stays in range, and stop.
    int bad = 0;
    float mx = -INFINITY;
    for (uint32_t e = lane; e < experts; e += 32) {
        const float v = row[e];
        prob[e] = v;
        bad |= !(fabsf(v) < INFINITY);
        mx = fmaxf(mx, v);
    }
    if (__any_sync(0xffffffffu, bad)) {
        if (lane == 0) {
            *(volatile int *)status = (int)FQ_ERR_WEIGHT;
            gate[t] = 0.f;
        }
        for (uint32_t k = lane; k < used; k += 32) {
            ids[(size_t)t * used + k] = k;
            weights[(size_t)t * used + k] = 0.f;
        }
        return;
    }
    if (sigmoid) {
        for (uint32_t e = lane; e < experts; e += 32) prob[e] = 1.f / (1.f + expf(-prob[e]));
    } else {
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
        float part = 0.f;
        for (uint32_t e = lane; e < experts; e += 32) {
            const float v = expf(prob[e] - mx);
            prob[e] = v;
            part += v;
        }
        const float total = warp_sum(part);
        for (uint32_t e = lane; e < experts; e += 32) prob[e] = prob[e] / total;
    }
    // The lane's best remaining score; recomputed only by the lane whose expert was taken.
    float bv = -INFINITY;
    uint32_t bi = 0xffffffffu;
    auto rescan = [&]() {
        bv = -INFINITY;
        bi = 0xffffffffu;
        for (uint32_t e = lane; e < experts; e += 32) {
            const float v = prob[e];
            if (v > bv) { bv = v; bi = e; } // ascending e: ties keep the lower index
        }
    };
    rescan();
    float picked_sum = 0.f, mine = 0.f; // lane k % 32 keeps the k-th picked score (k < 32; later ones go through `weights`)
    for (uint32_t k = 0; k < used; k++) {
        float wv = bv;
        uint32_t wi = bi;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, wv, off);
            const uint32_t oi = __shfl_xor_sync(0xffffffffu, wi, off);
            if (ov > wv || (ov == wv && oi < wi)) { wv = ov; wi = oi; }
        }
        picked_sum += wv;
        if (k < 32) {
            if (lane == k) mine = wv;
        } else if (lane == 0) {
            weights[(size_t)t * used + k] = wv;
        }
        if (lane == 0) ids[(size_t)t * used + k] = wi;
        if ((wi & 31u) == lane) {
            prob[wi] = -1.f; // scores are non-negative, so a taken expert never wins again
            rescan();
        }
    }
    __syncwarp();
    for (uint32_t k = lane; k < used; k += 32) {
        const float v = k < 32 ? mine : weights[(size_t)t * used + k];
        weights[(size_t)t * used + k] = norm ? v / picked_sum : v;
    }
    if (shared_gate) {
        float dot = 0.f;
        for (uint32_t i = lane; i < hidden; i += 32) dot = fmaf(x[(size_t)t * hidden + i], shared_w[i], dot);
        dot = warp_sum(dot);
        if (lane == 0) gate[t] = 1.f / (1.f + expf(-dot));
    } else if (lane == 0) {
        gate[t] = 1.f;
    }
}

// The map of at most 32 routes by one warp: lane r ranks its route among the others.
__device__ __forceinline__ void map_small(const uint32_t *ids, uint32_t experts, uint32_t routes, uint32_t *__restrict__ offsets,
                                          uint32_t *__restrict__ sorted, uint32_t *__restrict__ position) {
    const uint32_t lane = threadIdx.x & 31;
    const bool live = lane < routes;
    const uint32_t e = live ? ids[lane] : 0xffffffffu;
    const bool valid = live && e < experts;
    uint32_t before = 0; // valid routes that sort before this one: a smaller expert, or the same expert and a lower index
    for (uint32_t l = 0; l < routes; l++) {
        const uint32_t oe = __shfl_sync(0xffffffffu, e, l);
        before += (oe < experts) && (oe < e || (oe == e && l < lane));
    }
    if (valid) {
        sorted[before] = lane;
        position[lane] = before;
    } else if (live) {
        position[lane] = 0; // an id that names no expert: the route belongs to no row
    }
    const uint32_t placed = __popc(__ballot_sync(0xffffffffu, valid));
    if (lane >= placed && lane < routes) sorted[lane] = 0; // rows past the last expert's point at route 0
    // offsets[x] = valid routes whose expert is below x
    for (uint32_t x0 = 0; x0 <= experts; x0 += 32) { // every lane takes every turn: the shuffles need the whole warp
        const uint32_t x = x0 + lane;
        uint32_t n = 0;
        for (uint32_t l = 0; l < routes; l++) n += __shfl_sync(0xffffffffu, e, l) < x;
        if (x <= experts) offsets[x] = n;
    }
}

// `offsets` (may be null; with it the grid is one block and tokens * used <= 32): the expert-major map of the
// routes just written, by the block's first warp -- a decode step's routing and map are then one launch.
__global__ void __launch_bounds__(ROUTE_WARPS * 32)
k_moe_route(const float *__restrict__ logits, const float *__restrict__ x, const float *__restrict__ shared_w,
            uint32_t experts, uint32_t used, uint32_t hidden, uint32_t tokens, int sigmoid, int norm, int shared_gate,
            uint32_t *__restrict__ ids, float *__restrict__ weights, float *__restrict__ gate, int *status,
            uint32_t *__restrict__ offsets, uint32_t *__restrict__ sorted, uint32_t *__restrict__ position) {
    extern __shared__ float route_smem[]; // [ROUTE_WARPS][experts]
    fqk::pdl_trigger(); // the next kernel may be scheduled now; it waits for this one's results itself
    fqk::pdl_wait();    // the logits come from the kernel before
    route_token(route_smem, logits, x, shared_w, experts, used, hidden, tokens, sigmoid, norm, shared_gate, ids, weights, gate, status);
    if (offsets) {
        __syncthreads(); // the block's ids are written
        if (threadIdx.x < 32) map_small(ids, experts, tokens * used, offsets, sorted, position);
    }
}

// Stable counting sort of routes by expert, one block of 32 warps.  Warp w owns the contiguous
// slice [w*S, (w+1)*S) of routes; `cnt[w][e]` first holds the slice's count of expert e, then the
// row where the slice's next route of expert e goes.  Up to 16384 routes a lane keeps its ids in registers
// (all loads in flight at once, one pass over global memory); beyond, both passes read them again.
constexpr int MAP_CACHED = 16; // ids per lane held in registers
__global__ void __launch_bounds__(1024)
k_moe_map(const uint32_t *__restrict__ ids, uint32_t experts, uint32_t routes, uint32_t *__restrict__ offsets,
          uint32_t *__restrict__ sorted, uint32_t *__restrict__ position) {
    extern __shared__ uint32_t cnt[]; // [32][experts] + [experts + 1]
    uint32_t *total = cnt + 32 * experts;
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t slice = ((routes + 31) / 32 + 31) / 32 * 32; // multiple of 32 routes per warp
    const uint32_t begin = warp * slice, end = min(routes, begin + slice);
    const bool cached = slice <= 32u * MAP_CACHED;
    uint32_t ev[MAP_CACHED];
    if (cached) {
#pragma unroll
        for (int i = 0; i < MAP_CACHED; i++) {
            const uint32_t r = begin + 32u * i + lane;
            ev[i] = r < end ? ids[r] : 0xffffffffu;
        }
    }
    for (uint32_t i = tid; i < 32 * experts + experts + 1; i += 1024) cnt[i] = 0;
    __syncthreads();
    // Lanes of the warp that hold the same (valid) expert id: one ballot per bit of the id.  (The hardware match
    // instruction measured several times slower on this kernel's single SM.)
    const int id_bits = 32 - __clz((int)experts - 1);
    auto same_as = [&](uint32_t e, bool valid) {
        uint32_t peers = __ballot_sync(0xffffffffu, valid);
        for (int b = 0; b < id_bits; b++) {
            const bool bit = (e >> b) & 1u;
            const uint32_t bal = __ballot_sync(0xffffffffu, bit);
            peers &= bit ? bal : ~bal;
        }
        return peers;
    };
    auto count_one = [&](uint32_t e, bool live) {
        const bool valid = live && e < experts;
        const uint32_t peers = same_as(e, valid);
        if (valid && lane == (uint32_t)(__ffs(peers) - 1)) cnt[warp * experts + e] += __popc(peers);
        __syncwarp();
    };
    if (cached) {
#pragma unroll
        for (int i = 0; i < MAP_CACHED; i++)
            if (begin + 32u * i < end) count_one(ev[i], begin + 32u * i + lane < end);
    } else {
        for (uint32_t base = begin; base < end; base += 32) {
            const bool live = base + lane < end;
            count_one(live ? ids[base + lane] : 0xffffffffu, live);
        }
    }
    __syncthreads();
    // Per expert: totals, then an exclusive scan over experts, then per-warp bases.
    for (uint32_t e = tid; e < experts; e += 1024) {
        uint32_t n = 0;
        for (int w = 0; w < 32; w++) n += cnt[w * experts + e];
        total[e] = n;
    }
    __syncthreads();
    if (warp == 0) {
        uint32_t carry = 0;
        for (uint32_t e0 = 0; e0 < experts; e0 += 32) {
            const uint32_t e = e0 + lane;
            const uint32_t n = e < experts ? total[e] : 0;
            uint32_t incl = n;
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                const uint32_t o = __shfl_up_sync(0xffffffffu, incl, off);
                if (lane >= (uint32_t)off) incl += o;
            }
            if (e < experts) {
                total[e] = carry + incl - n;
                offsets[e] = carry + incl - n;
            }
            carry += __shfl_sync(0xffffffffu, incl, 31);
        }
        if (lane == 0) {
            offsets[experts] = carry;
            total[experts] = carry;
        }
    }
    __syncthreads();
    for (uint32_t e = tid; e < experts; e += 1024) {
        uint32_t at = total[e];
        for (int w = 0; w < 32; w++) {
            const uint32_t n = cnt[w * experts + e];
            cnt[w * experts + e] = at;
            at += n;
        }
    }
    __syncthreads();
    auto place_one = [&](uint32_t r, uint32_t e, bool live) {
        const uint32_t peers = same_as(e, live && e < experts);
        if (live && e < experts) {
            const uint32_t rank = __popc(peers & ((1u << lane) - 1));
            const uint32_t at = cnt[warp * experts + e] + rank;
            sorted[at] = r;
            position[r] = at;
        } else if (live) {
            position[r] = 0; // an id that names no expert: the route belongs to no row
        }
        __syncwarp();
        if (live && e < experts && lane == (uint32_t)(__ffs(peers) - 1)) cnt[warp * experts + e] += __popc(peers);
        __syncwarp();
    };
    if (cached) {
#pragma unroll
        for (int i = 0; i < MAP_CACHED; i++)
            if (begin + 32u * i < end) place_one(begin + 32u * i + lane, ev[i], begin + 32u * i + lane < end);
    } else {
        for (uint32_t base = begin; base < end; base += 32) {
            const bool live = base + lane < end;
            place_one(base + lane, live ? ids[base + lane] : 0xffffffffu, live);
        }
    }
    // Rows past the last expert's (only there when some id named no expert) point at route 0.
    for (uint32_t i = total[experts] + tid; i < routes; i += 1024) sorted[i] = 0;
}

// The same map for many routes: a cluster of MAP_CLUSTER blocks, block c owning the contiguous run
// [c * S, (c + 1) * S) of routes (S a multiple of 1024) and its warps contiguous slices of that, so that the order of
// equal experts is the order of the routes, as above.  Every block counts its own routes, the blocks read one
// another's per-expert totals through distributed shared memory, and each then knows where its warps' routes go.
constexpr int MAP_CLUSTER = 8;
constexpr uint32_t MAP_CLUSTER_MIN_ROUTES = 4096;
__global__ void __cluster_dims__(MAP_CLUSTER, 1, 1) __launch_bounds__(1024)
k_moe_map_cluster(const uint32_t *__restrict__ ids, uint32_t experts, uint32_t routes, uint32_t *__restrict__ offsets,
                  uint32_t *__restrict__ sorted, uint32_t *__restrict__ position) {
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    extern __shared__ uint32_t cnt[]; // [32][experts], block totals [experts], expert offsets [experts + 1]
    uint32_t *mine = cnt + 32 * experts, *total = mine + experts;
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, rank = cluster.block_rank();
    const uint32_t per_block = ((routes + MAP_CLUSTER - 1) / MAP_CLUSTER + 1023) / 1024 * 1024, slice = per_block / 32;
    const uint32_t begin = min(routes, rank * per_block + warp * slice), end = min(routes, begin + slice);
    const bool cached = slice <= 32u * MAP_CACHED;
    uint32_t ev[MAP_CACHED];
    if (cached) {
#pragma unroll
        for (int i = 0; i < MAP_CACHED; i++) {
            const uint32_t r = begin + 32u * i + lane;
            ev[i] = r < end ? ids[r] : 0xffffffffu;
        }
    }
    for (uint32_t i = tid; i < 32 * experts; i += 1024) cnt[i] = 0;
    __syncthreads();
    const int id_bits = 32 - __clz((int)experts - 1);
    auto same_as = [&](uint32_t e, bool valid) { // lanes of the warp that hold the same (valid) expert id
        uint32_t peers = __ballot_sync(0xffffffffu, valid);
        for (int b = 0; b < id_bits; b++) {
            const bool bit = (e >> b) & 1u;
            const uint32_t bal = __ballot_sync(0xffffffffu, bit);
            peers &= bit ? bal : ~bal;
        }
        return peers;
    };
    auto count_one = [&](uint32_t e, bool live) {
        const bool valid = live && e < experts;
        const uint32_t peers = same_as(e, valid);
        if (valid && lane == (uint32_t)(__ffs(peers) - 1)) cnt[warp * experts + e] += __popc(peers);
        __syncwarp();
    };
    if (cached) {
#pragma unroll
        for (int i = 0; i < MAP_CACHED; i++)
            if (begin + 32u * i < end) count_one(ev[i], begin + 32u * i + lane < end);
    } else {
        for (uint32_t base = begin; base < end; base += 32) {
            const bool live = base + lane < end;
            count_one(live ? ids[base + lane] : 0xffffffffu, live);
        }
    }
    __syncthreads();
    for (uint32_t e = tid; e < experts; e += 1024) {
        uint32_t n = 0;
        for (int w = 0; w < 32; w++) n += cnt[w * experts + e];
        mine[e] = n;
    }
    cluster.sync(); // every block's totals are in place
    // Per expert: the routes of all blocks, and of the blocks before this one.
    uint32_t before = 0, all = 0; // of expert tid (experts <= 1024 = the block's threads)
    if (tid < experts) {
        for (uint32_t c = 0; c < (uint32_t)MAP_CLUSTER; c++) {
            const uint32_t n = cluster.map_shared_rank(mine, c)[tid];
            if (c < rank) before += n;
            all += n;
        }
    }
    // Exclusive scan of `all` over the experts: within warps by shuffles, across warps through `total`.
    uint32_t incl = all;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        const uint32_t o = __shfl_up_sync(0xffffffffu, incl, off);
        if (lane >= (uint32_t)off) incl += o;
    }
    __shared__ uint32_t warp_sum_of[32];
    if (lane == 31) warp_sum_of[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        uint32_t v = warp_sum_of[lane], inc = v;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const uint32_t o = __shfl_up_sync(0xffffffffu, inc, off);
            if (lane >= (uint32_t)off) inc += o;
        }
        warp_sum_of[lane] = inc - v;
    }
    __syncthreads();
    const uint32_t first = warp_sum_of[warp] + incl - all; // the expert's first row
    if (tid < experts) {
        total[tid] = first;
        if (rank == 0) offsets[tid] = first;
    }
    if (tid == experts - 1) {
        total[experts] = first + all;
        if (rank == 0) offsets[experts] = first + all;
    }
    // Where each warp's next route of the expert goes.
    if (tid < experts) {
        uint32_t at = first + before;
        for (int w = 0; w < 32; w++) {
            const uint32_t n = cnt[w * experts + tid];
            cnt[w * experts + tid] = at;
            at += n;
        }
    }
    __syncthreads();
    auto place_one = [&](uint32_t r, uint32_t e, bool live) {
        const uint32_t peers = same_as(e, live && e < experts);
        if (live && e < experts) {
            const uint32_t at = cnt[warp * experts + e] + __popc(peers & ((1u << lane) - 1));
            sorted[at] = r;
            position[r] = at;
        } else if (live) {
            position[r] = 0; // an id that names no expert: the route belongs to no row
        }
        __syncwarp();
        if (live && e < experts && lane == (uint32_t)(__ffs(peers) - 1)) cnt[warp * experts + e] += __popc(peers);
        __syncwarp();
    };
    if (cached) {
#pragma unroll
        for (int i = 0; i < MAP_CACHED; i++)
            if (begin + 32u * i < end) place_one(begin + 32u * i + lane, ev[i], begin + 32u * i + lane < end);
    } else {
        for (uint32_t base = begin; base < end; base += 32) {
            const bool live = base + lane < end;
            place_one(base + lane, live ? ids[base + lane] : 0xffffffffu, live);
        }
    }
    // Rows past the last expert's (only there when some id named no expert) point at route 0.
    for (uint32_t i = total[experts] + rank * 1024 + tid; i < routes; i += MAP_CLUSTER * 1024) sorted[i] = 0;
    cluster.sync(); // no block leaves while another may still read its totals
}

// The same map for at most 32 routes (a decode step's), by one warp: lane r ranks its route among the others.
__global__ void __launch_bounds__(32)
k_moe_map_small(const uint32_t *__restrict__ ids, uint32_t experts, uint32_t routes, uint32_t *__restrict__ offsets,
                uint32_t *__restrict__ sorted, uint32_t *__restrict__ position) {
    map_small(ids, experts, routes, offsets, sorted, position);
}

// xg[row] = x[sorted[row] / used]
__global__ void k_moe_gather(const float *__restrict__ x, const uint32_t *__restrict__ sorted, uint32_t hidden,
                             uint32_t used, float *__restrict__ xg) {
    const uint32_t row = blockIdx.x;
    const uint32_t token = sorted[row] / used;
    const float *src = x + (size_t)token * hidden;
    float *dst = xg + (size_t)row * hidden;
    if ((hidden & 3u) == 0) {
        for (uint32_t i = threadIdx.x; i < hidden / 4; i += blockDim.x)
            reinterpret_cast<float4 *>(dst)[i] = reinterpret_cast<const float4 *>(src)[i];
    } else {
        for (uint32_t i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = src[i];
    }
}

// out[t][i] = sum_s w[t][s] * down[row(t, s)][i] + gate[t] * shared[t][i]; VEC values of a token per thread.
template <int VEC>
__global__ void __launch_bounds__(256)
k_moe_combine(const float *__restrict__ down, const float *__restrict__ weights,
              const uint32_t *__restrict__ position, const float *__restrict__ shared,
              const float *__restrict__ gate, uint32_t hidden, uint32_t used, uint32_t tokens,
              int identity, float *__restrict__ out) {
    fqk::pdl_trigger();
    fqk::pdl_wait(); // the expert rows and the shared expert's output come from the kernels before
    const size_t gid = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * VEC;
    if (gid >= (size_t)tokens * hidden) return;
    const uint32_t t = gid / hidden, i = gid % hidden;
    float acc[VEC];
#pragma unroll
    for (int v = 0; v < VEC; v++) acc[v] = 0.f;
    for (uint32_t s = 0; s < used; s++) {
        const uint32_t r = t * used + s;
        const uint32_t row = identity ? r : position[r];
        const float w = weights[r];
        const float *src = down + (size_t)row * hidden + i;
        if constexpr (VEC == 4) {
            const float4 d = *reinterpret_cast<const float4 *>(src);
            acc[0] = fmaf(w, d.x, acc[0]);
            acc[1] = fmaf(w, d.y, acc[1]);
            acc[2] = fmaf(w, d.z, acc[2]);
            acc[3] = fmaf(w, d.w, acc[3]);
        } else {
            acc[0] = fmaf(w, src[0], acc[0]);
        }
    }
    const float g = gate[t];
    if constexpr (VEC == 4) {
        const float4 sh = *reinterpret_cast<const float4 *>(shared + gid);
        *reinterpret_cast<float4 *>(out + gid) = make_float4(fmaf(g, sh.x, acc[0]), fmaf(g, sh.y, acc[1]), fmaf(g, sh.z, acc[2]), fmaf(g, sh.w, acc[3]));
    } else {
        out[gid] = fmaf(g, shared[gid], acc[0]);
    }
}

template <typename... Args> void launch_combine(cudaStream_t stream, const float *down, const float *shared, float *out, uint32_t hidden, size_t n, Args... args) {
    const bool vec = hidden % 4 == 0 && (((uintptr_t)down | (uintptr_t)shared | (uintptr_t)out) & 15) == 0;
    if (vec) fqk::launch_pdl(k_moe_combine<4>, dim3((unsigned)((n / 4 + 255) / 256)), dim3(256), 0, stream, args...);
    else fqk::launch_pdl(k_moe_combine<1>, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, args...);
}

// out = g / (1 + exp(-g)) * u
__global__ void k_swiglu(const float *__restrict__ g, const float *__restrict__ u, size_t n, float *__restrict__ y) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) {
        const float x = g[i];
        y[i] = x / (1.f + expf(-x)) * u[i];
    }
}

// The two kernels above with bf16 results, for the tensor-core expert GEMM that follows them.
// `range` (may be null): two row indices; rows outside [range[0], range[stride]) are skipped (the rows of
// experts another rank owns).
__global__ void k_moe_gather_bf16(const float *__restrict__ x, const uint32_t *__restrict__ sorted, uint32_t hidden,
                                  uint32_t used, const uint32_t *__restrict__ range, uint32_t stride, __nv_bfloat16 *__restrict__ xg) {
    const uint32_t row = blockIdx.x;
    if (range && (row < range[0] || row >= range[stride])) return;
    const float *src = x + (size_t)(sorted[row] / used) * hidden;
    __nv_bfloat16 *dst = xg + (size_t)row * hidden;
    if ((hidden & 3u) == 0) {
        for (uint32_t i = threadIdx.x; i < hidden / 4; i += blockDim.x) {
            const float4 v = reinterpret_cast<const float4 *>(src)[i];
            const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
            reinterpret_cast<uint2 *>(dst)[i] = make_uint2(*reinterpret_cast<const uint32_t *>(&a), *reinterpret_cast<const uint32_t *>(&b));
        }
    } else {
        for (uint32_t i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = __float2bfloat16_rn(src[i]);
    }
}

__global__ void k_swiglu_bf16(const float *__restrict__ g, const float *__restrict__ u, size_t n, const uint32_t *__restrict__ range,
                              uint32_t stride, uint32_t width, __nv_bfloat16 *__restrict__ y) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (range && (i < (size_t)range[0] * width || i >= (size_t)range[stride] * width)) return;
    if (i < n) {
        const float x = g[i];
        y[i] = __float2bfloat16_rn(x / (1.f + expf(-x)) * u[i]);
    }
}

// Expert of each expert-sorted row, relative to the first expert this rank stores; rows of other ranks'
// experts get an id no matrix has, which the per-route kernels skip.
__global__ void k_moe_local_ids(const uint32_t *__restrict__ ids, const uint32_t *__restrict__ sorted, uint32_t routes, uint32_t first,
                                uint32_t count, uint32_t *__restrict__ out) {
    const uint32_t row = blockIdx.x * blockDim.x + threadIdx.x;
    if (row >= routes) return;
    const uint32_t e = ids[sorted[row]];
    out[row] = (e >= first && e - first < count) ? e - first : 0xFFFFFFFFu;
}

} // namespace

int fq_launch_moe_gather_bf16(fq_device *dev, const float *x, const uint32_t *sorted, uint32_t hidden, uint32_t used, uint32_t routes,
                              const uint32_t *range, uint32_t stride, void *xg) {
    if (int rc = fq_begin_enqueue(dev)) return rc;
    k_moe_gather_bf16<<<routes, 256, 0, dev->stream>>>(x, sorted, hidden, used, range, stride, (__nv_bfloat16 *)xg);
    return fq_end_enqueue(dev, "moe_gather", 1);
}

int fq_launch_glu_bf16(fq_device *dev, const float *gate, const float *up, size_t n, const uint32_t *range, uint32_t stride, uint32_t width,
                       void *out) {
    if (int rc = fq_begin_enqueue(dev)) return rc;
    k_swiglu_bf16<<<(unsigned)((n + 255) / 256), 256, 0, dev->stream>>>(gate, up, n, range, stride, width, (__nv_bfloat16 *)out);
    return fq_end_enqueue(dev, "glu", 1);
}

int fq_launch_moe_local_ids(fq_device *dev, const uint32_t *ids, const uint32_t *sorted, uint32_t routes, uint32_t first, uint32_t count,
                            uint32_t *out) {
    if (int rc = fq_begin_enqueue(dev)) return rc;
    k_moe_local_ids<<<(routes + 255) / 256, 256, 0, dev->stream>>>(ids, sorted, routes, first, count, out);
    return fq_end_enqueue(dev, "moe_local_ids", 1);
}

extern "C" int fq_moe_route(fq_device *dev, const float *logits, const float *x, const float *shared_w,
                            uint32_t experts, uint32_t used, uint32_t hidden, uint32_t tokens, int sigmoid,
                            int norm, int shared_gate, uint32_t *ids, float *weights, float *gate) {
    return fq_moe_route_map(dev, logits, x, shared_w, experts, used, hidden, tokens, sigmoid, norm, shared_gate, ids, weights, gate, nullptr, nullptr,
                            nullptr);
}

// Routing and, with `offsets`, the expert-major map of the routes (fq_moe_map's outputs): one launch when the
// routes are a decode step's (one block routes them all), else two.
int fq_moe_route_map(fq_device *dev, const float *logits, const float *x, const float *shared_w, uint32_t experts, uint32_t used,
                     uint32_t hidden, uint32_t tokens, int sigmoid, int norm, int shared_gate, uint32_t *ids, float *weights, float *gate,
                     uint32_t *offsets, uint32_t *sorted, uint32_t *position) {
    if (int rc = fq_begin_enqueue(dev)) return rc;
    const bool fused = offsets && tokens <= (uint32_t)ROUTE_WARPS && (size_t)tokens * used <= 32;
    if (fused) {
        const size_t routes = (size_t)tokens * used;
        if (int rc = fq_check_binding(dev, offsets, (size_t)(experts + 1) * 4, "offsets")) return rc;
        if (int rc = fq_check_binding(dev, sorted, routes * 4, "sorted")) return rc;
        if (int rc = fq_check_binding(dev, position, routes * 4, "position")) return rc;
    }
    if (experts == 0 || experts > MAX_EXPERTS || used == 0 || used > experts || tokens == 0)
        return fq_fail(dev, FQ_ERR_SHAPE, "routing %u of %u experts for %u tokens", used, experts, tokens);
    if (int rc = fq_check_binding(dev, logits, (size_t)tokens * experts * 4, "logits")) return rc;
    if (int rc = fq_check_binding(dev, ids, (size_t)tokens * used * 4, "ids")) return rc;
    if (int rc = fq_check_binding(dev, weights, (size_t)tokens * used * 4, "weights")) return rc;
    if (int rc = fq_check_binding(dev, gate, (size_t)tokens * 4, "shared gate")) return rc;
    if (shared_gate) {
        if (int rc = fq_check_binding(dev, x, (size_t)tokens * hidden * 4, "x")) return rc;
        if (int rc = fq_check_binding(dev, shared_w, (size_t)hidden * 4, "shared gate weight")) return rc;
    }
    if (int rc = fq_check_no_alias(dev, ids, (size_t)tokens * used * 4, logits, (size_t)tokens * experts * 4, "ids")) return rc;
    if (int rc = fq_check_no_alias(dev, weights, (size_t)tokens * used * 4, logits, (size_t)tokens * experts * 4, "weights")) return rc;
    if (int rc = fq_check_cuda(dev, fqk::launch_pdl(k_moe_route, dim3((tokens + ROUTE_WARPS - 1) / ROUTE_WARPS), dim3(ROUTE_WARPS * 32),
                                                    (size_t)ROUTE_WARPS * experts * sizeof(float), dev->stream, logits, x, shared_w, experts, used, hidden,
                                                    tokens, sigmoid, norm, shared_gate, ids, weights, gate, dev->status_dev, fused ? offsets : nullptr,
                                                    fused ? sorted : nullptr, fused ? position : nullptr),
                               "moe_route launch"))
        return rc;
    if (int rc = fq_end_enqueue(dev, "moe_route", 1)) return rc;
    if (offsets && !fused) return fq_moe_map(dev, ids, experts, tokens * used, offsets, sorted, position);
    return FQ_OK;
}

extern "C" int fq_moe_map(fq_device *dev, const uint32_t *ids, uint32_t experts, uint32_t routes,
                          uint32_t *offsets, uint32_t *sorted, uint32_t *position) {
    if (int rc = fq_begin_enqueue(dev)) return rc;
    if (experts == 0 || experts > MAX_EXPERTS || routes == 0)
        return fq_fail(dev, FQ_ERR_SHAPE, "map of %u routes over %u experts", routes, experts);
    if (int rc = fq_check_binding(dev, ids, (size_t)routes * 4, "ids")) return rc;
    if (int rc = fq_check_binding(dev, offsets, (size_t)(experts + 1) * 4, "offsets")) return rc;
    if (int rc = fq_check_binding(dev, sorted, (size_t)routes * 4, "sorted")) return rc;
    if (int rc = fq_check_binding(dev, position, (size_t)routes * 4, "position")) return rc;
    if (routes <= 32) {
        k_moe_map_small<<<1, 32, 0, dev->stream>>>(ids, experts, routes, offsets, sorted, position);
        return fq_end_enqueue(dev, "moe_map", 1);
    }
    if (routes >= MAP_CLUSTER_MIN_ROUTES) { // enough routes for eight blocks to beat one
        const size_t smem = ((size_t)34 * experts + 1) * sizeof(uint32_t);
        static bool configured = false;
        if (smem > 48 * 1024 && !configured) {
            cudaError_t e = cudaFuncSetAttribute(k_moe_map_cluster, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return fq_check_cuda(dev, e, "moe_map shared memory");
            configured = true;
        }
        k_moe_map_cluster<<<MAP_CLUSTER, 1024, smem, dev->stream>>>(ids, experts, routes, offsets, sorted, position);
        if (int rc = fq_check_cuda(dev, cudaGetLastError(), "moe_map launch")) return rc;
        return fq_end_enqueue(dev, "moe_map", 1);
    }
    const size_t smem = ((size_t)33 * experts + 1) * sizeof(uint32_t);
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(k_moe_map, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fq_check_cuda(dev, e, "moe_map shared memory");
    }
    k_moe_map<<<1, 1024, smem, dev->stream>>>(ids, experts, routes, offsets, sorted, position);
    return fq_end_enqueue(dev, "moe_map", 1);
}

extern "C" int fq_moe_gather(fq_device *dev, const float *x, const uint32_t *sorted, uint32_t hidden,
                             uint32_t used, uint32_t routes, float *xg) {
    if (int rc = fq_begin_enqueue(dev)) return rc;
    if (hidden == 0 || used == 0 || routes == 0) return fq_fail(dev, FQ_ERR_SHAPE, "gather geometry");
    if (int rc = fq_check_binding(dev, x, (size_t)((routes + used - 1) / used) * hidden * 4, "x")) return rc;
    if (int rc = fq_check_binding(dev, sorted, (size_t)routes * 4, "sorted")) return rc;
    if (int rc = fq_check_binding(dev, xg, (size_t)routes * hidden * 4, "xg")) return rc;
    if (int rc = fq_check_no_alias(dev, xg, (size_t)routes * hidden * 4, x, (size_t)((routes + used - 1) / used) * hidden * 4, "xg")) return rc;
    k_moe_gather<<<routes, 256, 0, dev->stream>>>(x, sorted, hidden, used, xg);
    return fq_end_enqueue(dev, "moe_gather", 1);
}

// Tokens [token0, token0 + tokens): out[t] for those tokens only (`out` is indexed by the token, like the rest).
int fq_launch_moe_combine_range(fq_device *dev, const float *down, const float *weights, const uint32_t *position, const float *shared,
                                const float *gate, uint32_t hidden, uint32_t used, uint32_t token0, uint32_t tokens, float *out) {
    if (int rc = fq_begin_enqueue(dev)) return rc;
    if (tokens == 0) return FQ_OK;
    const size_t n = (size_t)tokens * hidden;
    launch_combine(dev->stream, down, shared + (size_t)token0 * hidden, out + (size_t)token0 * hidden, hidden, n, down,
                   weights + (size_t)token0 * used, position + (size_t)token0 * used, shared + (size_t)token0 * hidden, gate + token0, hidden, used,
                   tokens, 0, out + (size_t)token0 * hidden);
    return fq_end_enqueue(dev, "moe_combine", 1);
}

extern "C" int fq_moe_combine(fq_device *dev, const float *down, const float *weights, const uint32_t *position,
                              const float *shared, const float *gate, uint32_t hidden, uint32_t used,
                              uint32_t tokens, int identity, float *out) {
    if (int rc = fq_begin_enqueue(dev)) return rc;
    if (hidden == 0 || used == 0 || tokens == 0) return fq_fail(dev, FQ_ERR_SHAPE, "combine geometry");
    const size_t routes = (size_t)tokens * used;
    if (int rc = fq_check_binding(dev, down, routes * hidden * 4, "down")) return rc;
    if (int rc = fq_check_binding(dev, weights, routes * 4, "weights")) return rc;
    if (!identity)
        if (int rc = fq_check_binding(dev, position, routes * 4, "position")) return rc;
    if (int rc = fq_check_binding(dev, shared, (size_t)tokens * hidden * 4, "shared")) return rc;
    if (int rc = fq_check_binding(dev, gate, (size_t)tokens * 4, "shared gate")) return rc;
    if (int rc = fq_check_binding(dev, out, (size_t)tokens * hidden * 4, "out")) return rc;
    if (int rc = fq_check_no_alias(dev, out, (size_t)tokens * hidden * 4, down, routes * hidden * 4, "out")) return rc;
    if (int rc = fq_check_no_alias(dev, out, (size_t)tokens * hidden * 4, shared, (size_t)tokens * hidden * 4, "out")) return rc;
    const size_t n = (size_t)tokens * hidden;
    launch_combine(dev->stream, down, shared, out, hidden, n, down, weights, position, shared, gate, hidden, used, tokens, identity, out);
    return fq_end_enqueue(dev, "moe_combine", 1);
}

extern "C" int fq_glu(fq_device *dev, const float *gate, const float *up, size_t n, float *out) {
    if (int rc = fq_begin_enqueue(dev)) return rc;
    if (n == 0) return fq_fail(dev, FQ_ERR_SHAPE, "empty gated unit");
    if (int rc = fq_check_binding(dev, gate, n * 4, "gate")) return rc;
    if (int rc = fq_check_binding(dev, up, n * 4, "up")) return rc;
    if (int rc = fq_check_binding(dev, out, n * 4, "out")) return rc;
    k_swiglu<<<(unsigned)((n + 255) / 256), 256, 0, dev->stream>>>(gate, up, n, out);
    return fq_end_enqueue(dev, "glu", 1);
}
