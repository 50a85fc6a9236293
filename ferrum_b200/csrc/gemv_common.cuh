// Pieces shared by the decode / verify projection kernels (gemv_i8.cu, gemv_nt.cu): programmatic dependent
// launch, load helpers, the warp-level integer MMAs, the 16-bit quantisation of eight activations, and the
// device side of the fused row-shard exchange.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "internal.h"

namespace fqk {

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ uint64_t global_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// u8 (weights) x s8 (activations), 16 rows x 8 columns x 32 k.
__device__ __forceinline__ void mma_u8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// s8 x s8, 16 rows x 8 columns x 16 k.
__device__ __forceinline__ void mma_s8s8_k16(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a0), "r"(a1), "r"(b0));
}

// Prepared activations: written by the kernel before this one (which may still run when this grid
// starts), so ordinary coherent loads after `pdl_wait`; volatile so guarded loads are not speculated.
__device__ __forceinline__ uint4 ldx128(const void *p) {
    uint4 r;
    asm volatile("ld.global.ca.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
    return r;
}
__device__ __forceinline__ uint32_t ldx32(const void *p) {
    uint32_t r;
    asm volatile("ld.global.ca.u32 %0, [%1];" : "=r"(r) : "l"(p));
    return r;
}
// Weights: immutable, read once -> read-only path, no L1 allocation.
__device__ __forceinline__ uint4 ldw128(const void *p) {
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
    return r;
}
__device__ __forceinline__ uint2 ldw64(const void *p) {
    uint2 r;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(r.x), "=r"(r.y) : "l"(p));
    return r;
}
__device__ __forceinline__ uint32_t ldw16(const void *p) {
    uint16_t r;
    asm volatile("ld.global.nc.L1::no_allocate.u16 %0, [%1];" : "=h"(r) : "l"(p));
    return r;
}
// Weights of which one thread takes 4 bytes at a time: the rest of the 32-byte sector is asked for by a later
// instruction of the same warp, so the line is kept in L1.
__device__ __forceinline__ uint32_t ldw32_keep(const void *p) {
    uint32_t r;
    asm volatile("ld.global.nc.u32 %0, [%1];" : "=r"(r) : "l"(p));
    return r;
}
__device__ __forceinline__ uint32_t lop3_select(uint32_t a, uint32_t b, uint32_t mask) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xE4;" : "=r"(r) : "r"(a), "r"(b), "r"(mask)); // (a & mask) | (b & ~mask)
    return r;
}
__device__ __forceinline__ uint32_t lop3_and_xor(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0x6A;" : "=r"(r) : "r"(a), "r"(b), "r"(c)); // (a & b) ^ c
    return r;
}
// Byte i of w, zero- or sign-extended (one PRMT each; a selector nibble with its top bit set replicates the
// sign of the byte it names).
__device__ __forceinline__ int byte_u(uint32_t w, int i) { return (int)__byte_perm(w, 0u, 0x4440u + (uint32_t)i); }
__device__ __forceinline__ int byte_s(uint32_t w, int i) {
    int r;
    asm("prmt.b32 %0, %1, %1, %2;" : "=r"(r) : "r"(w), "r"(0x8880u + (uint32_t)i * 0x1111u));
    return r;
}
__device__ __forceinline__ uint32_t word_of(const uint4 &v, int i) { return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w; }

// Eight activations of one lane (values 8 lane .. 8 lane + 7 of a 256-value superblock handled by one warp) as
// 16-bit integers x' = round(x * s) = 256 hi + lo with both halves signed bytes; s = 2^e is the largest power of
// two with max|x| * s <= 32639 over the superblock (1 when the superblock is all zero or holds a NaN or an
// infinity, in which case `finite` is false and every x' is zero: the caller makes the superblock's factor NaN).
struct Quant8 {
    uint8_t hi[8], lo[8];
    int sum, sum_hi, sum_lo; // over the lane's eight values
    int e;
    bool finite;
};
__device__ __forceinline__ Quant8 quantize8(const float (&v)[8]) {
    Quant8 q;
    float amax = 0.f;
    bool bad = false;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        amax = fmaxf(amax, fabsf(v[i]));
        bad |= !(fabsf(v[i]) < INFINITY);
    }
    q.finite = __ballot_sync(0xffffffffu, bad) == 0u;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
    int e = 0;
    if (amax > 0.f && q.finite) {
        int ex;
        frexpf(amax, &ex);
        e = 15 - ex;
        if (ldexpf(amax, e) > 32639.f) e -= 1;
        e = max(-110, min(110, e));
    }
    q.e = e;
    const float s = ldexpf(1.f, e);
    q.sum = q.sum_hi = q.sum_lo = 0;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        int x = __float2int_rn(fminf(fmaxf(v[i] * s, -32639.f), 32639.f));
        if (!q.finite) x = 0;
        const int h = (x + 128) >> 8, l = x - (h << 8);
        q.hi[i] = (uint8_t)h;
        q.lo[i] = (uint8_t)l;
        q.sum += x;
        q.sum_hi += h;
        q.sum_lo += l;
    }
    return q;
}
// 1 / sqrt(mean(x^2) + eps) of a row of n values (a multiple of 4), by one warp: every lane sums the float4s
// lane, lane + 32, .. in order and the lanes are added by a butterfly, so any warp that calls this on the same row
// gets the same bits (the standalone normalisation and the one fused into activation preparation agree).
__device__ __forceinline__ float row_inv_rms(const float *__restrict__ row, uint32_t n, float eps, uint32_t lane) {
    float ss = 0.f;
    for (uint32_t i = lane; i < n / 4; i += 32) {
        const float4 v = reinterpret_cast<const float4 *>(row)[i];
        ss = fmaf(v.x, v.x, ss);
        ss = fmaf(v.y, v.y, ss);
        ss = fmaf(v.z, v.z, ss);
        ss = fmaf(v.w, v.w, ss);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
    return 1.0f / sqrtf(ss / (float)n + eps);
}
__device__ __forceinline__ uint32_t pack4(const uint8_t *p) { return p[0] | (p[1] << 8) | (p[2] << 16) | ((uint32_t)p[3] << 24); }

// Row-sharded launches (TpPush, internal.h).  tp_seq: the sequence number of this exchange, read by every block
// once the kernel before has finished.  tp_store: one output value to the mirror of every peer, tagged.
// tp_finish: this block's share of the incoming slots, then the bookkeeping by the last block.  A slot that has
// not arrived after P.wait_ns of wall time makes the block record FQ_ERR_TIMEOUT and stop polling for good (its
// remaining slots are looked at once each), so an absent peer costs one limit per block, not one per slot.
__device__ __forceinline__ uint32_t tp_seq(const TpPush &P) { return *(volatile uint32_t *)P.epoch + 1u; }
__device__ __forceinline__ void tp_store(const TpPush &P, uint32_t seq, const float *dst, float v) {
    const size_t off = (size_t)((const uint8_t *)dst - P.peer[P.rank]);
    for (uint32_t p = 0; p < P.world; p++)
        if (p != P.rank)
            asm volatile("st.global.v2.u32 [%0], {%1, %2};" ::"l"(P.peer[p] + P.mirror_off + 2 * off), "r"(__float_as_uint(v)), "r"(seq) : "memory");
}
__device__ __forceinline__ void tp_finish(const TpPush &P, uint32_t seq) {
    __shared__ uint32_t tp_gave_up;
    const uint32_t blocks = gridDim.x * gridDim.y * gridDim.z, block = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
    if (threadIdx.x == 0) tp_gave_up = 0;
    __syncthreads();
    const size_t per_rank = P.covered_bytes / 4, incoming = per_rank * (P.world - 1);
    const size_t lo = incoming * block / blocks, hi = incoming * (block + 1) / blocks;
    uint64_t t0 = 0;
    for (size_t i = lo + threadIdx.x; i < hi; i += blockDim.x) {
        uint32_t p = (uint32_t)(i / per_rank);
        const size_t j = i % per_rank;
        if (p >= P.rank) p++; // the senders, skipping this rank
        const size_t off = P.slice_off + ((size_t)p - P.rank) * P.slice_bytes + 4 * j; // wraps correctly for p < rank
        const uint8_t *slot = P.peer[P.rank] + P.mirror_off + 2 * off;
        uint32_t v = 0, tag = 0;
        bool arrived = false;
        for (uint32_t n = 0;; n++) {
            asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v), "=r"(tag) : "l"(slot) : "memory");
            arrived = tag == seq;
            if (arrived || *(volatile uint32_t *)&tp_gave_up) break;
            if (n > 16) {
                __nanosleep(64);
                if (t0 == 0) t0 = global_ns();
                else if ((n & 15u) == 0 && global_ns() - t0 > P.wait_ns) {
                    tp_gave_up = 1u;
                    break;
                }
            }
        }
        if (arrived) *reinterpret_cast<uint32_t *>(P.peer[P.rank] + off) = v;
        else *(volatile int *)P.status = (int)FQ_ERR_TIMEOUT; // the peer never sent: report, do not hang
    }
    __syncthreads();
    if (threadIdx.x == 0 && atomicAdd(P.counter, 1u) + 1u == blocks) {
        *P.counter = 0;
        *(volatile uint32_t *)P.epoch = seq; // every block has read it by now
    }
}

// ---------------------------------------------------------------- per-warp weight rings
//
// A warp streams the packed superblocks of its 16-row weight tiles through a private ring of stages in shared
// memory with 16-byte asynchronous copies: several superblocks in flight per warp, no registers held, no
// block-wide barrier.  A stage holds one superblock of 16 rows, row r at r * ROW (ROW >= the bytes of a row's
// superblock, padded so that the reads of a kernel's fragment pattern fall on different banks):
//   Q4_K / Q5_K  the 144 / 176 bytes of the block;
//   Q6_K         ql[128] | qh[64] | scales[16] of the device layout (blocks.cuh), and after the 16 rows 4 bytes
//                per row: the aligned word that holds the f16 d of the superblock (its high half for odd b).
// A lane copies the same pieces of every superblock, so their offsets from the tile's first row are worked out
// once per tile (`start_tile`); rows past the end of the matrix read its last row.
__device__ __forceinline__ void cp_async16(void *smem_dst, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async4(void *smem_dst, const void *src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <int FMT, uint32_t ROW> struct WeightRing {
    static constexpr uint32_t SRC = FMT == FQ_Q4_K ? 144 : FMT == FQ_Q5_K ? 176 : 208; // bytes copied per row and superblock
    static constexpr uint32_t PER_ROW = SRC / 16;
    static constexpr uint32_t PIECES = 16 * PER_ROW;
    static constexpr int NP = FMT == FQ_Q6_K ? 7 : (int)((PIECES + 31) / 32);
    static constexpr uint32_t BYTES = 16 * ROW + (FMT == FQ_Q6_K ? 64 : 0);
    static_assert(ROW >= SRC && ROW % 16 == 0, "stage rows hold a row's superblock and stay 16-byte aligned");
    const uint8_t *base = nullptr;
    uint32_t off[NP];
    // Q6_K: pieces 0..127 are ql (row p / 8), 128..191 qh (row / 4), 192..207 the scales, 208..223 the word with d.
    __device__ __forceinline__ uint32_t piece_row(int i, uint32_t lane) const {
        const uint32_t p = lane + 32 * i;
        if constexpr (FMT != FQ_Q6_K) return p / PER_ROW;
        return i < 4 ? p / 8 : i < 6 ? (p - 128) / 4 : (lane & 15);
    }
    // `first_row`: the tile's first weight row; `last`: index of the matrix's last row relative to it.
    __device__ __forceinline__ void start_tile(const uint8_t *first_row, uint32_t last, uint32_t pitch, uint32_t nblk, uint32_t lane) {
        base = first_row;
#pragma unroll
        for (int i = 0; i < NP; i++) {
            const uint32_t p = lane + 32 * i, r = min(piece_row(i, lane), last);
            uint32_t in_row;
            if constexpr (FMT != FQ_Q6_K) in_row = 16 * (p % PER_ROW);
            else in_row = i < 4 ? 16 * (p % 8) : i < 6 ? nblk * 128 + 16 * (p % 4) : lane < 16 ? nblk * 192 : nblk * 208;
            off[i] = r * pitch + in_row;
        }
    }
    // Superblock b of the tile into the stage at `dst`.
    __device__ __forceinline__ void issue(uint8_t *dst, uint32_t b, uint32_t lane) const {
#pragma unroll
        for (int i = 0; i < NP; i++) {
            const uint32_t p = lane + 32 * i;
            if constexpr (FMT != FQ_Q6_K) {
                if (p < PIECES) cp_async16(dst + ROW * (p / PER_ROW) + 16 * (p % PER_ROW), base + (off[i] + b * SRC));
            } else {
                if (i < 4) cp_async16(dst + ROW * (p / 8) + 16 * (p % 8), base + (off[i] + b * 128));
                else if (i < 6) cp_async16(dst + ROW * ((p - 128) / 4) + 128 + 16 * (p % 4), base + (off[i] + b * 64));
                else if (lane < 16) cp_async16(dst + ROW * lane + 192, base + (off[i] + b * 16));
                else cp_async4(dst + 16 * ROW + 4 * (lane - 16), base + (off[i] + (b & ~1u) * 2)); // the aligned 4 bytes that hold d
            }
        }
    }
};

template <typename... KArgs, typename... Args>
cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

} // namespace fqk
