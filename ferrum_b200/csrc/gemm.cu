// Prefill dequant-GEMM on the 5th-generation tensor cores (BF16 activations in, BF16 out, fp32
// accumulation in tensor memory).  The work of the reference's `q4_k_gemm_mpp*`, `q6_k_gemm_mpp`,
// `q8_0_gemm_mpp*` (src/metal/shaders/project_mpp.metal:505-729, 1133-1212, 89-230) and, for shape,
// of `h_mm_*` (src/metal/shaders/hybrid.metal:1411-1469).
//
//   Y[m][n] = sum_k X[m][k] * bf16(W[n][k])        X, Y bf16; W decoded exactly, then rounded to bf16
//
// One block owns 128 weight rows x 256 activation rows and walks K in steps of 64:
//
//   warp 0       one thread issues TMA loads (cp.async.bulk.tensor, 128-byte swizzle) of the
//                64 x 256 activation tile of each stage; the warp also owns the tensor-memory allocation;
//   warp 1       one thread issues tcgen05.mma (M = 128 weight rows, N = 256 activation rows, K = 16,
//                four per stage) with both operands in shared memory and the accumulator in tensor
//                memory, and commits each stage back to the producers;
//   warps 2..9   decode the packed blocks with the exact per-value formula (blocks.cuh), round to
//                bf16 (RNE) and write the 128 x 64 weight tile in the same K-major 128-byte-swizzled
//                layout the TMA produces; afterwards warps 2..5 read the accumulator back
//                (tcgen05.ld, 32 lanes x 32 columns per load), round to bf16 and store Y.
//
// Weights sit on the MMA's M side and tokens on its N side, so a weight tile is decoded once per 256
// tokens.  Every mbarrier wait is bounded: a wait that gives up records FQ_ERR_TIMEOUT in the status
// word, the block stops issuing work, waits (bounded) for what it already issued, frees its tensor
// memory and returns.
//
// Further down: k_gemm_f16g, the persistent fp16 kernel for expert-sorted rows of F32 callers (tokens on the MMA's
// M side as hi + lo terms, 256 weight rows on its N side).
#include <cuda.h>
#include <cuda_fp16.h>

#include <algorithm>

#include "blocks.cuh"
#include "internal.h"

namespace {

constexpr int BM = 128;      // weight rows per block (MMA M)
// Activation rows per block (MMA N): 256 for dense prefill, 64 for expert groups (about 32 rows each).
constexpr int BK = 64;       // k per stage: 64 bf16 = one 128-byte swizzle row
constexpr int PRODUCER_WARPS = 8;
constexpr int PREFETCH = 3;  // k-blocks of packed bytes in flight per producer thread
constexpr int THREADS = (2 + PRODUCER_WARPS) * 32;
constexpr uint32_t A_BYTES = BM * BK * 2;
constexpr uint32_t WAIT_LIMIT = 1u << 24;          // attempts, where a wait only drains what is in flight
constexpr uint32_t WAIT_HINT_NS = 20000;          // how long one attempt may park the thread
constexpr uint64_t WAIT_LIMIT_NS = 2000000000ull; // a wait gives up after two seconds

// Two rings in shared memory.  A: decoded 128 x 64 weight tiles (16 KB each).  B: activation tiles of at most
// 256 rows x 64 (one TMA box, one MMA N extent; a 512-row block uses two per k-block, each released on its own
// so that its reload starts as early as possible).  For the 512-row block the B ring is what keeps the tensor
// pipe fed (64 KB per k-block is about what an SM can take in from L2 in the time the MMAs need), so it gets
// the larger share of the 227 KB.
template <int BN> constexpr int a_stages() { return 4; }
template <int BN> constexpr int b_slots() { return 4; }
template <int BN> constexpr int mma_n() { return BN > 256 ? 256 : BN; }

template <int BN> struct __align__(1024) Smem {
    uint8_t a[a_stages<BN>()][A_BYTES];
    uint8_t b[b_slots<BN>()][mma_n<BN>() * BK * 2];
    uint64_t full_a[a_stages<BN>()], empty_a[a_stages<BN>()], full_b[b_slots<BN>()], empty_b[b_slots<BN>()], accum;
    uint32_t tmem_base;
    uint32_t abort_flag;
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// One attempt; the hardware may park the thread for up to `hint_ns` while the phase is still open, so a
// waiting thread does not burn issue slots that the decoding warps need.
__device__ __forceinline__ bool mbar_try(uint64_t *bar, uint32_t parity, uint32_t hint_ns = 0) {
    uint32_t ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\nselp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok)
                 : "r"(smem_u32(bar)), "r"(parity), "r"(hint_ns)
                 : "memory");
    return ok != 0;
}
__device__ __forceinline__ uint64_t now_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Bounded wait (WAIT_LIMIT_NS of wall time).  On giving up: record the timeout, raise the block's abort
// flag, report failure.
template <class SM, uint32_t HINT_NS = WAIT_HINT_NS> __device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, SM *sm, int *status) {
    if (mbar_try(bar, parity)) return true;
    const uint64_t t0 = now_ns();
    do {
        if (mbar_try(bar, parity, HINT_NS)) return true;
        if (*(volatile uint32_t *)&sm->abort_flag) return false;
    } while (now_ns() - t0 < WAIT_LIMIT_NS);
    *(volatile int *)status = (int)FQ_ERR_TIMEOUT;
    atomicExch(&sm->abort_flag, 1u);
    return false;
}

__device__ __forceinline__ void tma_load_2d(void *dst, const CUtensorMap *map, int x, int y, uint64_t *bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
                 : "memory");
}

// Shared-memory operand descriptor: K-major, 128-byte swizzle, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr) {
    return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
           ((uint64_t)2 << 61);
}
// Instruction descriptor, kind::f16: D = F32, A = B = BF16, both K-major, N = bn, M = 128.
constexpr uint32_t idesc_for(int bn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
                 : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
          "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]),
          "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
          "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi); // .x = lo (low 16 bits), RNE
    return *reinterpret_cast<uint32_t *>(&v);
}

// Small unsigned integer -> float without the conversion unit: the integer placed in the mantissa of 2^23,
// minus 2^23 (+ bias).  Exact, and it keeps the quarter-rate I2F pipe out of the producers' inner loop.
__device__ __forceinline__ float small_to_float(uint32_t q, float bias = 0.f) {
    return __fsub_rn(__uint_as_float(0x4B000000u | q), 8388608.0f + bias);
}

// The packed bytes one producer thread needs for 32 consecutive k values of its weight row (a k-block of 64
// is two of these: part 0 and 1).  Loading and decoding are separate so that the loads of later k-blocks are
// in flight while the current one is decoded: a thread's stream is otherwise bound by memory latency.
template <int FMT> struct Raw;
template <> struct Raw<FQ_Q4_K> { uint4 hdr, q0, q1; };
template <> struct Raw<FQ_Q5_K> { uint4 hdr, q0, q1, h0, h1; };
template <> struct Raw<FQ_Q6_K> { uint4 l0, l1, h0, h1; uint32_t sc, d; };
template <> struct Raw<FQ_Q8_0> { uint32_t q[8]; uint32_t d; };

template <int FMT>
__device__ __forceinline__ Raw<FMT> load_raw(const uint8_t *rowp, uint32_t nblk, uint32_t kb, int part) {
    Raw<FMT> r;
    if constexpr (FMT == FQ_Q4_K) {
        // k-block kb = chunk c of superblock b: part 0 = low nibbles (sub-block 2c), part 1 = high nibbles.
        const uint8_t *blk = rowp + (size_t)(kb >> 2) * 144;
        const uint32_t c = kb & 3;
        r.hdr = *reinterpret_cast<const uint4 *>(blk);
        r.q0 = *reinterpret_cast<const uint4 *>(blk + 16 + 32 * c);
        r.q1 = *reinterpret_cast<const uint4 *>(blk + 32 + 32 * c);
    } else if constexpr (FMT == FQ_Q5_K) {
        // As Q4_K, with the 32 bytes of fifth bits (bit j of qh[l] belongs to value l of sub-block j).
        const uint8_t *blk = rowp + (size_t)(kb >> 2) * 176;
        const uint32_t c = kb & 3;
        r.hdr = *reinterpret_cast<const uint4 *>(blk);
        r.h0 = *reinterpret_cast<const uint4 *>(blk + 16);
        r.h1 = *reinterpret_cast<const uint4 *>(blk + 32);
        r.q0 = *reinterpret_cast<const uint4 *>(blk + 48 + 32 * c);
        r.q1 = *reinterpret_cast<const uint4 *>(blk + 64 + 32 * c);
    } else if constexpr (FMT == FQ_Q6_K) {
        // k-block kb of superblock b: half n = (kb % 4) / 2, 32-groups i = 2 h and 2 h + 1 with h = kb % 2;
        // part selects the group.  Device layout of blocks.cuh.
        const uint32_t b = kb >> 2, n = (kb >> 1) & 1, h = kb & 1, i = 2 * h + part;
        const uint8_t *ql = rowp + (size_t)b * 128 + 64 * n + 32 * (i & 1);
        const uint8_t *qh = rowp + (size_t)nblk * 128 + (size_t)b * 64 + 32 * n;
        r.l0 = *reinterpret_cast<const uint4 *>(ql);
        r.l1 = *reinterpret_cast<const uint4 *>(ql + 16);
        r.h0 = *reinterpret_cast<const uint4 *>(qh);
        r.h1 = *reinterpret_cast<const uint4 *>(qh + 16);
        r.sc = *reinterpret_cast<const uint16_t *>(rowp + (size_t)nblk * 192 + (size_t)b * 16 + 8 * n + 2 * i);
        r.d = *reinterpret_cast<const uint16_t *>(rowp + (size_t)nblk * 208 + (size_t)b * 2);
    } else {
        // Q8_0 (device layout of blocks.cuh): k-block kb = blocks 2 kb and 2 kb + 1; part selects the block.
        const uint32_t b = 2 * kb + part;
        const uint4 q0 = *reinterpret_cast<const uint4 *>(rowp + (size_t)b * 32), q1 = *reinterpret_cast<const uint4 *>(rowp + (size_t)b * 32 + 16);
        r.q[0] = q0.x, r.q[1] = q0.y, r.q[2] = q0.z, r.q[3] = q0.w, r.q[4] = q1.x, r.q[5] = q1.y, r.q[6] = q1.z, r.q[7] = q1.w;
        r.d = *reinterpret_cast<const uint16_t *>(rowp + (size_t)nblk * 32 + (size_t)b * 2);
    }
    return r;
}

// Two decoded weights as a bf16 pair: the values rounded to bf16, or (lo) what that rounding dropped.
__device__ __forceinline__ uint32_t pack_term(float a, float b, bool lo) {
    if (lo) {
        a -= __bfloat162float(__float2bfloat16_rn(a));
        b -= __bfloat162float(__float2bfloat16_rn(b));
    }
    return pack_bf16(a, b);
}

// Raw bytes -> 32 weights decoded exactly and rounded to bf16 (or, with `lo`, the bf16 of the rounding
// residue), two per register.
template <int FMT>
__device__ __forceinline__ void decode_raw(const Raw<FMT> &r, uint32_t kb, int part, bool lo, uint32_t (&out)[16]) {
    if constexpr (FMT == FQ_Q4_K || FMT == FQ_Q5_K) {
        const uint32_t c = kb & 3;
        const uint4 hdr = r.hdr;
        // `get_scale_min_k4` on the three scale words (hdr.y = scales[0..3], .z = [4..7], .w = [8..11]).
        const uint32_t j = 2 * c + part, sh = 8 * (j & 3);
        uint32_t sc, mn;
        if (j < 4) {
            sc = (hdr.y >> sh) & 63u;
            mn = (hdr.z >> sh) & 63u;
        } else {
            sc = ((hdr.w >> sh) & 0xFu) | ((((hdr.y >> sh) >> 6) & 3u) << 4);
            mn = (((hdr.w >> sh) >> 4) & 0xFu) | ((((hdr.z >> sh) >> 6) & 3u) << 4);
        }
        const float d = f16_bits_to_f32((uint16_t)(hdr.x & 0xFFFFu)), dmin = f16_bits_to_f32((uint16_t)(hdr.x >> 16));
        const float ds = __fmul_rn(d, small_to_float(sc)), dm = __fmul_rn(dmin, small_to_float(mn));
        // fl(ds * q) in one FMA: with Q = 2^23 + q (the quant dropped into the mantissa of 2^23),
        // ds * Q - ds * 2^23 is rounded once, and ds * 2^23 is exact, so the result is the correctly rounded
        // product, the same bits as converting q and multiplying.
        const float ds23 = -__fmul_rn(ds, 8388608.0f);
        const uint32_t w[8] = {r.q0.x, r.q0.y, r.q0.z, r.q0.w, r.q1.x, r.q1.y, r.q1.z, r.q1.w};
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const uint32_t v = part ? (w[i] >> 4) : w[i];
            uint32_t n4 = v & 0x0F0F0F0Fu; // one quant per byte; each byte moves into a float mantissa with one PRMT
            if constexpr (FMT == FQ_Q5_K) {
                const uint32_t hw = i == 0 ? r.h0.x : i == 1 ? r.h0.y : i == 2 ? r.h0.z : i == 3 ? r.h0.w : i == 4 ? r.h1.x : i == 5 ? r.h1.y : i == 6 ? r.h1.z : r.h1.w;
                n4 |= ((hw >> j) & 0x01010101u) << 4;
            }
            const float f0 = __fsub_rn(__fmaf_rn(ds, __uint_as_float(__byte_perm(n4, 0x4B000000u, 0x7440)), ds23), dm);
            const float f1 = __fsub_rn(__fmaf_rn(ds, __uint_as_float(__byte_perm(n4, 0x4B000000u, 0x7441)), ds23), dm);
            const float f2 = __fsub_rn(__fmaf_rn(ds, __uint_as_float(__byte_perm(n4, 0x4B000000u, 0x7442)), ds23), dm);
            const float f3 = __fsub_rn(__fmaf_rn(ds, __uint_as_float(__byte_perm(n4, 0x4B000000u, 0x7443)), ds23), dm);
            out[2 * i] = pack_term(f0, f1, lo);
            out[2 * i + 1] = pack_term(f2, f3, lo);
        }
    } else if constexpr (FMT == FQ_Q6_K) {
        const uint32_t h = kb & 1, i = 2 * h + part;
        const float d = f16_bits_to_f32((uint16_t)r.d);
        // signed scale s -> (s ^ 0x80) - 128 without the conversion unit
        const float ds0 = __fmul_rn(d, small_to_float((r.sc & 0xFFu) ^ 0x80u, 128.f));
        const float ds1 = __fmul_rn(d, small_to_float(((r.sc >> 8) & 0xFFu) ^ 0x80u, 128.f));
        const uint32_t lw[8] = {r.l0.x, r.l0.y, r.l0.z, r.l0.w, r.l1.x, r.l1.y, r.l1.z, r.l1.w};
        const uint32_t hw[8] = {r.h0.x, r.h0.y, r.h0.z, r.h0.w, r.h1.x, r.h1.y, r.h1.z, r.h1.w};
#pragma unroll
        for (int j = 0; j < 8; j++) {
            // four 6-bit quants, one per byte: low nibbles from ql, bits 4..5 from qh (one select for all four)
            const uint32_t lo4 = (i < 2) ? lw[j] : (lw[j] >> 4);
            const uint32_t hi4 = i == 0 ? (hw[j] << 4) : i == 1 ? (hw[j] << 2) : i == 2 ? hw[j] : (hw[j] >> 2);
            const uint32_t q4 = ((lo4 & 0x0F0F0F0Fu) | (hi4 & 0x30303030u));
            const float ds = j < 4 ? ds0 : ds1;
            const float f0 = __fmul_rn(ds, small_to_float(__byte_perm(q4, 0, 0x4440), 32.0f)); // q - 32, exact
            const float f1 = __fmul_rn(ds, small_to_float(__byte_perm(q4, 0, 0x4441), 32.0f));
            const float f2 = __fmul_rn(ds, small_to_float(__byte_perm(q4, 0, 0x4442), 32.0f));
            const float f3 = __fmul_rn(ds, small_to_float(__byte_perm(q4, 0, 0x4443), 32.0f));
            out[2 * j] = pack_term(f0, f1, lo);
            out[2 * j + 1] = pack_term(f2, f3, lo);
        }
    } else {
        const float d = f16_bits_to_f32((uint16_t)r.d);
#pragma unroll
        for (int j = 0; j < 8; j++) {
            // signed byte b -> (b ^ 0x80) - 128
            const uint32_t u = r.q[j] ^ 0x80808080u;
            const float f0 = __fmul_rn(small_to_float(__byte_perm(u, 0, 0x4440), 128.f), d);
            const float f1 = __fmul_rn(small_to_float(__byte_perm(u, 0, 0x4441), 128.f), d);
            const float f2 = __fmul_rn(small_to_float(__byte_perm(u, 0, 0x4442), 128.f), d);
            const float f3 = __fmul_rn(small_to_float(__byte_perm(u, 0, 0x4443), 128.f), d);
            out[2 * j] = pack_term(f0, f1, lo);
            out[2 * j + 1] = pack_term(f2, f3, lo);
        }
    }
}

__device__ __forceinline__ void store_out(float *p, float v) { *p = v; }
__device__ __forceinline__ void store_out(__nv_bfloat16 *p, float v) { *p = __float2bfloat16_rn(v); }

// Epilogue, run by the eight producer warps: a warp may read the 32 tensor-memory lanes of
// quarter warp % 4; warps 2..5 take the first half of the accumulator columns, warps 6..9 the second.
// A complete tile is rounded and stored to Y; a partial one (a K range only) goes to `part` as fp32,
// column-major ([col][row]) so that these stores and the fix-up kernel's loads are coalesced.
template <int BN, typename YT>
__device__ __forceinline__ void epilogue(uint32_t tmem, int warp, int lane, uint32_t n0, uint32_t rows, uint32_t m0, uint32_t m_end,
                                      YT *__restrict__ y, float *__restrict__ part) {
    const int quarter = warp & 3, c_begin = warp < 6 ? 0 : BN / 2, c_end = warp < 6 ? BN / 2 : BN;
    const uint32_t row = n0 + 32 * quarter + lane;
    for (int c0 = c_begin; c0 < c_end; c0 += 32) {
        uint32_t acc[32];
        tmem_ld32(tmem + ((uint32_t)(32 * quarter) << 16) + c0, acc);
        if (part) {
            float *mine = part + 32 * quarter + lane;
#pragma unroll
            for (int c = 0; c < 32; c++) mine[(size_t)(c0 + c) * BM] = __uint_as_float(acc[c]);
        } else if (row < rows) {
#pragma unroll
            for (int c = 0; c < 32; c++) {
                const uint32_t tok = m0 + c0 + c;
                if (tok < m_end) store_out(y + (size_t)tok * rows + row, __uint_as_float(acc[c]));
            }
        }
    }
}

// `xmap` describes X as a [m][cols] bf16 tensor, box 64 x min(BN, 256), 128-byte swizzle; `b_bytes` is one box.
//
// Dense (grid.x blocks): tile t covers weight rows (t % tiles_x) * 128.. and activation rows
// (t / tiles_x) * BN...  Blocks 0 .. full_tiles-1 compute one whole tile each (whole waves of the machine: the
// blocks of a wave walk K together, so the activation k-slices they share stay in L2).  The remaining tiles,
// too few to fill a wave, are split along K: block full_tiles + i computes k-blocks [z * per, (z + 1) * per)
// of tile full_tiles + i / splits, z = i % splits, and leaves fp32 partial sums in workspace slot i, which
// k_fixup adds up in split order.
//
// GROUPED (`h_mm_id*`, src/metal/shaders/hybrid.metal:2430-2523; grid (ceil(rows / 128), activation tiles of
// all groups)): group z serves activation rows offsets[z] .. offsets[z+1] with the expert stored at slots[z]
// (or z); one tile per block; a tile that runs past its group reads the next group's rows and does not
// store them.
//
// MODE 2 (dense, F32 callers): near-fp32 products from bf16 operands.  Both operands are split in two bf16
// terms (v = hi + lo, lo = bf16(v - hi)) and every k-block is walked three times: hi x hi, hi x lo, lo x hi
// (w_hi, w_hi, w_lo against x_hi, x_lo, x_hi); the caller lays X out as [m][3 * cols] in that order.  The
// dropped lo x lo term and the residuals are 2^-17 of a product.
// Up to four matrices of one format and width that share X (q|k|v, gate|up): their row tiles are counted
// through, so one launch fills the machine where the small ones alone would not.
struct GemmMany {
    const uint8_t *w[4];
    void *y[4];
    uint32_t rows[4];
    uint32_t tx_end[4]; // row tiles up to and including matrix i
    uint32_t count;     // <= 1: the kernel's own w / rows / y arguments
};

template <int FMT, int BN, typename YT, int MODE>
__global__ void __launch_bounds__(THREADS, MODE == 1 ? 2 : 1) // two expert-tile blocks share an SM: one's set-up and epilogue overlap the other's main loop
k_gemm_tc(const __grid_constant__ CUtensorMap xmap, const uint8_t *__restrict__ w, uint32_t rows, uint32_t cols, uint32_t pitch,
          YT *__restrict__ y, uint32_t m, uint32_t b_bytes, const uint32_t *__restrict__ offsets,
          const uint32_t *__restrict__ slots, uint32_t experts, uint32_t tiles_x, uint32_t full_tiles, uint32_t splits, uint32_t per,
          float *__restrict__ ws, int *status, const __grid_constant__ GemmMany many) {
    constexpr bool GROUPED = MODE == 1, PRECISE = MODE == 2;
    constexpr uint32_t TMEM_COLS = BN < 32 ? 32 : BN;
    constexpr int NSUB = BN > 256 ? BN / 256 : 1, MMA_N = BN / NSUB, A_STAGES = a_stages<BN>(), B_SLOTS = b_slots<BN>();
    constexpr uint32_t IDESC = idesc_for(MMA_N);
    extern __shared__ uint8_t smem_raw[];
    using SM = Smem<BN>;
    SM *sm = reinterpret_cast<SM *>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint32_t k_first = 0, k_iters = cols / BK * (PRECISE ? 3 : 1), n0, m0, m_end = m; // in units: (k-block, term)
    float *partial = nullptr;
    if (GROUPED) {
        // blockIdx.y counts activation tiles over all groups in order; `full_tiles` holds the group count.
        // Every warp finds (group z, tile ty of that group) for itself: 32 groups per step, tile counts
        // prefix-summed with shuffles.
        const uint32_t groups = full_tiles, ft = blockIdx.y;
        uint32_t z = 0, ty = 0, base = 0;
        bool found = false;
        for (uint32_t g0 = 0; g0 < groups && !found; g0 += 32) {
            const uint32_t g = g0 + lane;
            const uint32_t cnt = g < groups ? offsets[g + 1] - offsets[g] : 0u, t = (cnt + BN - 1) / BN;
            uint32_t incl = t;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const uint32_t n = __shfl_up_sync(0xffffffffu, incl, d);
                if (lane >= d) incl += n;
            }
            const uint32_t total = __shfl_sync(0xffffffffu, incl, 31);
            if (ft < base + total) {
                const uint32_t hit = __ballot_sync(0xffffffffu, ft >= base + incl - t && ft < base + incl);
                const int src = __ffs(hit) - 1;
                z = g0 + src;
                ty = ft - (base + __shfl_sync(0xffffffffu, incl - t, src));
                found = true;
            } else {
                base += total;
            }
        }
        if (!found) return; // uniform for the block: nothing was set up yet
        const uint32_t first = offsets[z], count = offsets[z + 1] - first;
        const uint32_t e = slots ? slots[z] : z;
        if (e >= experts) return;
        w += (size_t)e * rows * pitch;
        n0 = blockIdx.x * BM;
        m0 = first + ty * BN;
        m_end = first + count;
    } else {
        uint32_t t = blockIdx.x;
        if (t >= full_tiles) {
            const uint32_t i = t - full_tiles, z = i % splits;
            t = full_tiles + i / splits;
            k_first = z * per;
            if (k_first >= k_iters) return; // the launcher leaves no split without work
            k_iters = min(per, k_iters - k_first);
            partial = ws + (size_t)i * BN * BM;
        }
        uint32_t tx = t % tiles_x;
        if (many.count > 1) { // tiles_x counts the row tiles of all the matrices
            uint32_t which = 0, first = 0;
#pragma unroll
            for (int i = 0; i < 3; i++)
                if ((uint32_t)i + 1 < many.count && tx >= many.tx_end[i]) { which = i + 1; first = many.tx_end[i]; }
            w = many.w[which];
            y = (YT *)many.y[which];
            rows = many.rows[which];
            tx -= first;
        }
        n0 = tx * BM;
        m0 = (t / tiles_x) * BN;
    }
    constexpr uint32_t nblk_div = FMT == FQ_Q8_0 ? 32 : 256;
    const uint32_t nblk = cols / nblk_div;

    if (threadIdx.x == 0) {
        for (int s = 0; s < A_STAGES; s++) {
            mbar_init(&sm->full_a[s], PRODUCER_WARPS * 32);
            mbar_init(&sm->empty_a[s], 1);
        }
        for (int s = 0; s < B_SLOTS; s++) {
            mbar_init(&sm->full_b[s], 1);
            mbar_init(&sm->empty_b[s], 1);
        }
        mbar_init(&sm->accum, 1);
        sm->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&xmap) : "memory");
    }
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm->tmem_base)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *(volatile uint32_t *)&sm->tmem_base;

    if (warp == 0) {
        if (lane == 0) {
            uint32_t issued = 0;
            bool ok = true;
            for (uint32_t it = 0; it < k_iters && ok; it++) {
#pragma unroll
                for (int h = 0; h < NSUB; h++) {
                    const uint32_t ib = it * NSUB + h, s = ib % B_SLOTS;
                    if (!(ok = mbar_wait(&sm->empty_b[s], ((ib / B_SLOTS) & 1) ^ 1, sm, status))) break;
                    mbar_expect_tx(&sm->full_b[s], b_bytes);
                    tma_load_2d(sm->b[s], &xmap, (int)((k_first + it) * BK), (int)(m0 + h * MMA_N), &sm->full_b[s]);
                    issued = ib + 1;
                }
            }
            // On an abort the copies already issued still land: wait for them (bounded) before the
            // block's shared memory goes away.
            if (*(volatile uint32_t *)&sm->abort_flag) {
                for (uint32_t ib = issued > (uint32_t)B_SLOTS ? issued - B_SLOTS : 0; ib < issued; ib++) {
                    const uint32_t s = ib % B_SLOTS;
                    for (uint32_t i = 0; i < WAIT_LIMIT && !mbar_try(&sm->full_b[s], (ib / B_SLOTS) & 1); i++) {}
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            bool ok = true;
            for (uint32_t it = 0; it < k_iters && ok; it++) {
                const int sa = it % A_STAGES;
                if (!mbar_wait(&sm->full_a[sa], (it / A_STAGES) & 1, sm, status)) break;
                const uint64_t adesc = umma_desc(smem_u32(sm->a[sa]));
#pragma unroll
                for (int h = 0; h < NSUB; h++) { // each 256-row part of the activation tile has its own accumulator columns
                    const uint32_t ib = it * NSUB + h, sb = ib % B_SLOTS;
                    if (!(ok = mbar_wait(&sm->full_b[sb], (ib / B_SLOTS) & 1, sm, status))) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint64_t bdesc = umma_desc(smem_u32(sm->b[sb]));
#pragma unroll
                    for (int k = 0; k < BK / 16; k++) // 16 bf16 = 32 bytes = 2 descriptor units along K
                        umma_bf16(tmem + h * MMA_N, adesc + 2 * k, bdesc + 2 * k, IDESC, (it | k) != 0);
                    umma_commit(&sm->empty_b[sb]); // the slot is free once these MMAs have read it
                }
                if (ok) umma_commit(&sm->empty_a[sa]);
            }
            if (ok) umma_commit(&sm->accum); // arrives when every MMA issued so far has completed
        }
    } else {
        // Producers: thread p owns weight row p / 2 of the tile and k part p % 2 of each stage.
        const int p = threadIdx.x - 64, r = p >> 1, part = p & 1;
        const bool live = n0 + r < rows;
        const uint8_t *rowp = w + (size_t)min(n0 + r, rows - 1) * pitch;
        // PREFETCH k-blocks of packed bytes are in flight per thread while one is decoded.
        const uint32_t last = k_first + k_iters - 1;
        Raw<FMT> ring[PREFETCH];
#pragma unroll
        for (int j = 0; j < PREFETCH; j++) ring[j] = load_raw<FMT>(rowp, nblk, min(k_first + j, last) / (PRECISE ? 3 : 1), part);
        bool go = true;
        for (uint32_t it0 = 0; it0 < k_iters && go; it0 += PREFETCH) {
#pragma unroll
            for (int j = 0; j < PREFETCH; j++) {
                const uint32_t it = it0 + j;
                if (it >= k_iters) break;
                const int s = it % A_STAGES;
                uint32_t v[16];
                const uint32_t unit = k_first + it;
                decode_raw<FMT>(ring[j], unit / (PRECISE ? 3 : 1), part, PRECISE && unit % 3 == 2, v);
                ring[j] = load_raw<FMT>(rowp, nblk, min(unit + PREFETCH, last) / (PRECISE ? 3 : 1), part);
                if (!live) {
#pragma unroll
                    for (int i = 0; i < 16; i++) v[i] = 0u;
                }
                if (!mbar_wait(&sm->empty_a[s], ((it / A_STAGES) & 1) ^ 1, sm, status)) { go = false; break; }
                uint8_t *tile_row = sm->a[s] + r * 128;
#pragma unroll
                for (int c = 0; c < 4; c++) { // 16-byte chunk 4 part + c of the row, at its swizzled place
                    const int chunk = (4 * part + c) ^ (r & 7);
                    *reinterpret_cast<uint4 *>(tile_row + 16 * chunk) = make_uint4(v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); // generic-proxy stores -> tensor-core reads
                mbar_arrive(&sm->full_a[s]);
            }
        }
        // Epilogue, all eight producer warps.
        if (!mbar_wait(&sm->accum, 0, sm, status)) atomicExch(&sm->abort_flag, 1u);
        asm volatile("bar.sync 1, 256;" ::: "memory"); // the eight warps agree on whether to go on
        if (*(volatile uint32_t *)&sm->abort_flag == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            epilogue<BN, YT>(tmem, warp, lane, n0, rows, m0, m_end, y, partial);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        // Outstanding MMAs must have finished before the accumulator columns are released.
        if (lane == 0 && *(volatile uint32_t *)&sm->abort_flag)
            for (uint32_t i = 0; i < WAIT_LIMIT && !mbar_try(&sm->accum, 0); i++) {}
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}

typedef CUresult (*EncodeTiled)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encode_fn() {
    static EncodeTiled fn = [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return (EncodeTiled)p;
    }();
    return fn;
}

// X as bf16 when the caller's activations are F32 (the grouped expert path of the hybrid engine).
__global__ void k_to_bf16(const float *__restrict__ x, __nv_bfloat16 *__restrict__ out, size_t n) {
    const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i + 3 < n) {
        const float4 v = *reinterpret_cast<const float4 *>(x + i);
        const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
        *reinterpret_cast<uint2 *>(out + i) = make_uint2(*reinterpret_cast<const uint32_t *>(&a), *reinterpret_cast<const uint32_t *>(&b));
    } else {
        for (size_t j = i; j < n; j++) out[j] = __float2bfloat16_rn(x[j]);
    }
}

// X (fp32) as two bf16 terms laid out for MODE 2: k-block b of a row becomes the three 64-wide blocks
// hi, lo, hi at 3 b, 3 b + 1, 3 b + 2, with hi = bf16(x) and lo = bf16(x - hi).
__global__ void k_split3(const float *__restrict__ x, __nv_bfloat16 *__restrict__ out, uint32_t cols, size_t n) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const size_t row = i / cols;
    const uint32_t k = (uint32_t)(i % cols), b = k / BK, j = k % BK;
    const float v = x[i];
    const __nv_bfloat16 hi = __float2bfloat16_rn(v), lo = __float2bfloat16_rn(v - __bfloat162float(hi));
    __nv_bfloat16 *dst = out + row * (size_t)cols * 3 + (size_t)b * 3 * BK + j;
    dst[0] = hi;
    dst[BK] = lo;
    dst[2 * BK] = hi;
}

// The tiles that were split along K: their fp32 partial sums added in split order (deterministic), rounded and
// stored as Y.  One thread per four consecutive weight rows of one activation row of a split tile.
template <int BN, typename YT>
__global__ void __launch_bounds__(256)
k_fixup(const float *__restrict__ ws, uint32_t full_tiles, uint32_t splits, uint32_t tiles_x, uint32_t rows, uint32_t m, YT *__restrict__ y,
        size_t total, const __grid_constant__ GemmMany many) {
    const size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= total) return;
    const uint32_t r4 = e % (BM / 4), col = (e / (BM / 4)) % BN, i = (uint32_t)(e / ((size_t)(BM / 4) * BN)), tile = full_tiles + i;
    uint32_t tx = tile % tiles_x;
    if (many.count > 1) {
        uint32_t which = 0, first = 0;
#pragma unroll
        for (int q = 0; q < 3; q++)
            if ((uint32_t)q + 1 < many.count && tx >= many.tx_end[q]) { which = q + 1; first = many.tx_end[q]; }
        y = (YT *)many.y[which];
        rows = many.rows[which];
        tx -= first;
    }
    const uint32_t row = tx * BM + 4 * r4, tok = (tile / tiles_x) * BN + col;
    if (tok >= m || row >= rows) return;
    const float *p = ws + (((size_t)i * splits) * BN + col) * BM + 4 * r4;
    float4 sum = __ldcg(reinterpret_cast<const float4 *>(p));
    for (uint32_t z = 1; z < splits; z++) {
        const float4 v = __ldcg(reinterpret_cast<const float4 *>(p + (size_t)z * BN * BM));
        sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
    }
    const float o[4] = {sum.x, sum.y, sum.z, sum.w};
    YT *dst = y + (size_t)tok * rows + row;
#pragma unroll
    for (int j = 0; j < 4; j++)
        if (row + j < rows) store_out(dst + j, o[j]);
}

template <int FMT, int BN, typename YT, int MODE>
int launch(fq_device *dev, const ProjectArgs &a, const CUtensorMap &map, uint32_t b_bytes, uint32_t m_rows, int *status, const GemmMany &many) {
    constexpr bool GROUPED = MODE == 1;
    const size_t smem = sizeof(Smem<BN>) + 1024;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(k_gemm_tc<FMT, BN, YT, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fq_check_cuda(dev, e, "gemm shared memory");
        configured = true;
    }
    const uint32_t tiles_x = many.count > 1 ? many.tx_end[many.count - 1] : (a.rows + BM - 1) / BM, k_iters = a.cols / BK * (MODE == 2 ? 3 : 1);
    if (GROUPED) {
        // At most one partly filled tile per group on top of the full ones (m_rows = all groups' rows).
        const uint32_t per_group = (a.max_rows + BN - 1) / BN;
        const uint32_t tiles_y = (uint32_t)std::min<uint64_t>((uint64_t)per_group * a.groups, (uint64_t)m_rows / BN + a.groups);
        if (tiles_y > 65535) return FQ_ERR_UNSUPPORTED;
        dim3 grid(tiles_x, tiles_y, 1);
        k_gemm_tc<FMT, BN, YT, MODE><<<grid, THREADS, smem, dev->stream>>>(map, a.w, a.rows, a.cols, a.row_bytes, (YT *)a.y, m_rows, b_bytes,
                                                                              a.offsets, a.slots, a.experts, tiles_x, a.groups, 1, k_iters, dev->gemm_ws, status, many);
        return FQ_OK;
    }
    // Whole waves of tiles run one tile per block.  A remainder that would fill less than three quarters of a
    // wave is split along K into about one block per SM, each with at least 8 k-blocks and a workspace slot.
    const uint32_t tiles = tiles_x * ((m_rows + BN - 1) / BN), sms = (uint32_t)dev->sm_count;
    const uint32_t rest = tiles % sms;
    uint32_t full = tiles, splits = 1, per = k_iters;
    if (rest && rest * 4 < sms * 3) {
        const uint32_t cap = (uint32_t)std::min<size_t>(sms / rest, dev->gemm_ws_bytes / ((size_t)rest * BN * BM * sizeof(float)));
        const uint32_t want = std::min({cap, std::max(1u, k_iters / 8), 16u});
        if (want > 1) {
            per = (k_iters + want - 1) / want;
            splits = (k_iters + per - 1) / per; // no split is left without work
            full = tiles - rest;
        }
    }
    const uint32_t blocks = full + (tiles - full) * splits;
    k_gemm_tc<FMT, BN, YT, MODE><<<blocks, THREADS, smem, dev->stream>>>(map, a.w, a.rows, a.cols, a.row_bytes, (YT *)a.y, m_rows, b_bytes,
                                                                            a.offsets, a.slots, a.experts, tiles_x, full, splits, per, dev->gemm_ws, status, many);
    if (splits > 1) {
        const size_t threads = (size_t)(tiles - full) * BN * (BM / 4);
        k_fixup<BN, YT><<<(unsigned)((threads + 255) / 256), 256, 0, dev->stream>>>(dev->gemm_ws, full, splits, tiles_x, a.rows, m_rows, (YT *)a.y, threads, many);
    }
    return FQ_OK;
}

template <int BN, typename YT, int MODE>
int launch_fmt(fq_device *dev, const ProjectArgs &a, const CUtensorMap &map, uint32_t b_bytes, uint32_t m_rows, const GemmMany &many = GemmMany{}) {
    switch (a.format) {
    case FQ_Q4_K: return launch<FQ_Q4_K, BN, YT, MODE>(dev, a, map, b_bytes, m_rows, dev->status_dev, many);
    case FQ_Q5_K: return launch<FQ_Q5_K, BN, YT, MODE>(dev, a, map, b_bytes, m_rows, dev->status_dev, many);
    case FQ_Q6_K: return launch<FQ_Q6_K, BN, YT, MODE>(dev, a, map, b_bytes, m_rows, dev->status_dev, many);
    default: return launch<FQ_Q8_0, BN, YT, MODE>(dev, a, map, b_bytes, m_rows, dev->status_dev, many);
    }
}

int make_map(fq_device *dev, CUtensorMap *map, const void *x, uint32_t cols, uint32_t m_rows, uint32_t bn, uint32_t *b_bytes,
             CUtensorMapDataType type = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16) {
    EncodeTiled encode = encode_fn();
    if (!encode) return FQ_ERR_UNSUPPORTED;
    const cuuint64_t dims[2] = {cols, m_rows};
    const cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    // A box may not be taller than the tensor; rows past the end of a later tile are zero-filled.
    const uint32_t box_rows = m_rows < bn ? m_rows : bn;
    const cuuint32_t box[2] = {BK, box_rows}, elem[2] = {1, 1};
    CUresult r = encode(map, type, 2, const_cast<void *>(x), dims, strides, box, elem,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fq_fail(dev, FQ_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d)", (int)r);
    *b_bytes = box_rows * BK * 2;
    return FQ_OK;
}


// ---------------------------------------------------------------------------------------------------------
// Expert tiles on fp16 products: grouped projections of sixteen rows per expert or more, F32 in and out, for
// which the integer kernel of gemv_nt.cu repeats its per-(row, sub-block) scale arithmetic too often and the
// bf16 GEMM above is both too coarse (2^-9 weights, bf16 activations) and organised for many rows per tile.
//
//   y[t][n] = (sum_k (hi[t][k] + lo[t][k]) * fp16(W[e][n][k])) / s[t]      hi + lo = s[t] x[t] to 22 bits
//
// A tcgen05.mma with M = 128 takes about the same time whatever its N (measured: N = 32, 80 and 128 alike), so the
// few activation rows go on the M side -- 64 rows, each as two MMA rows (hi, lo) -- and 256 weight rows on the
// N side: the widest instruction, the most weights per tensor-core cycle.
//
// The block is persistent (one per SM) and walks work items (activation tile of <= 64 expert-sorted rows,
// 256 weight rows of one of up to two matrix sets) in a strided order:
//
//   warp 0        builds the table of activation tiles from the group offsets, then one thread issues one TMA
//                 load per k-block: the tile's rows with their hi and lo terms interleaved (MMA row 2 c is
//                 activation row c against hi, row 2 c + 1 against lo);
//   warp 1        one thread issues tcgen05.mma (M = 128, N = 256, K = 16, kind::f16) into one of two
//                 accumulators in tensor memory, so that the next item's MMAs run under this item's epilogue;
//   warp 2        (Q4_K) one thread asks the TMA for the packed bytes of the item's 256 weight rows, half a superblock
//                 at a time (plain boxes of the matrix as bytes), three stages ahead, across item borders: loads
//                 by the decoding threads themselves queue behind the SM's load unit and hold up their proxy fences;
//   warps 3..18   decode: a warp owns sixteen weight rows; lane (row, group) reads its packed bytes from the staged
//                 half superblock (Q6_K, whose items here are two superblocks long: from global memory, a
//                 superblock ahead) and writes 32 fp16 weights per k-block in packed half arithmetic (g_decode_*
//                 below) into the K-major, 128-byte-swizzled tile the MMA reads;
//   warps 19..22  epilogue: read the accumulator (lane = MMA row), add the hi and lo rows with a shuffle, undo
//                 the row scale, store y.
//
// Every wait is bounded as in k_gemm_tc.
constexpr int G_PRODUCER_WARPS = 16, G_EPI_WARPS = 4, G_THREADS = (3 + G_PRODUCER_WARPS + G_EPI_WARPS) * 32;
constexpr uint32_t G_TOK = 64;          // activation rows per tile (128 MMA rows)
constexpr uint32_t G_BN = 256;          // weight rows per tile (MMA N)
constexpr uint32_t G_W_BYTES = G_BN * BK * 2, G_X_BYTES = 2 * G_TOK * BK * 2;
constexpr uint32_t G_MAX_TILES = 512;   // activation tiles the table holds

// Q4_K: the packed bytes of a tile's 256 weight rows are staged by TMA half a superblock (two k-blocks) at a time, as
// plain row-major boxes of the matrix seen as bytes: the 16-byte header and the 64 bytes of two chunks per row.
// W_STAGES / X_SLOTS: decoded weight tiles and activation tiles in flight (what fits beside the rest).
template <int FMT> struct GRaw;
template <> struct GRaw<FQ_Q4_K> {
    static constexpr int STAGES = 3, W_STAGES = 3, X_SLOTS = 3;
    static constexpr uint32_t QS = G_BN * 16, BYTES = QS + G_BN * 64;
};
template <> struct GRaw<FQ_Q6_K> { // not staged: the decoding threads fetch their own bytes (see the kernel)
    static constexpr int STAGES = 1, W_STAGES = 4, X_SLOTS = 3;
    static constexpr uint32_t BYTES = 128;
};

template <int FMT> struct __align__(1024) GSmem {
    uint8_t w[GRaw<FMT>::W_STAGES][G_W_BYTES];
    uint8_t x[GRaw<FMT>::X_SLOTS][G_X_BYTES];
    uint8_t raw[GRaw<FMT>::STAGES][GRaw<FMT>::BYTES];
    uint2 tiles[G_MAX_TILES]; // .x = first sorted row, .y = expert << 8 | rows
    uint64_t full_w[GRaw<FMT>::W_STAGES], empty_w[GRaw<FMT>::W_STAGES], full_x[GRaw<FMT>::X_SLOTS], empty_x[GRaw<FMT>::X_SLOTS], acc_full[2], acc_empty[2], drain;
    uint64_t raw_full[GRaw<FMT>::STAGES], raw_empty[GRaw<FMT>::STAGES];
    uint32_t tmem_base, abort_flag, n_tiles;
};

// Tensor maps: the activations, and (Q4_K) the packed weights as bytes ([experts * rows][pitch]) per matrix set, 256
// rows a box: [0] = 16-byte (header), [1] = 64-byte (two chunks) boxes.
struct alignas(64) GMaps {
    CUtensorMap x[3];    // activations: 32-, 64- and 128-row boxes
    CUtensorMap w[2][2];
};

struct GJob {
    const uint8_t *w[2]; // matrix sets sharing the rows (gate and up)
    float *y[2];
    uint32_t tx_end[2];  // 256-row tiles up to and including set i
    uint32_t count;
    uint32_t rows, cols, pitch, experts, groups;
    uint32_t row_begin, row_end; // the expert-sorted rows this launch serves (the fp16 copy holds only these)
    const uint32_t *offsets, *slots;
    const float *inv_scale;      // of rows row_begin ..
    int *status;
    uint32_t box_bytes[3]; // of the 32-, 64- and 128-row activation boxes
};

__device__ __forceinline__ __half2 h2_bits(uint32_t b) { return *reinterpret_cast<__half2 *>(&b); }
__device__ __forceinline__ uint32_t bits_h2(__half2 h) { return *reinterpret_cast<uint32_t *>(&h); }
// Two copies of a small unsigned integer as exact halves: 0x6400 | v is 1024 + v.
__device__ __forceinline__ __half2 small_h2(uint32_t v) {
    return __hsub2(h2_bits(0x64006400u | v | (v << 16)), h2_bits(0x64006400u));
}
// Instruction descriptor, kind::f16: D = F32, A = B = F16, both K-major, M = 128, N = 256.
constexpr uint32_t G_IDESC = (1u << 4) | ((G_BN >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);

// One 32-value group of a superblock as 32 fp16 weights, two per register; `live` false gives zeros (rows past
// the end of the matrix).  A quant enters as the half 0x6400 | q = 1024 + q (one PRMT per pair).  Q4_K:
// u = (1024 + q) sc - 1024 sc = q sc in one fused step (exact: below 2048), then w = u d - fp16(dmin m), rounded
// once.  Q6_K: (1024 + q) - 1056 = q - 32 exactly, times fp16(d scale).  Every weight is within 2^-11 (relative)
// of its exact value, plus 2^-12 of its sub-block's minimum term.
//
// Q4_K: the row's staged header and the 32 bytes of chunk C; sub-block j = 2 C + part is nibble `part` of the chunk.
template <int C>
__device__ __forceinline__ void g_decode_q4k(const uint8_t *hdrp, const uint8_t *chunk, uint32_t part, bool live, uint32_t (&out)[16]) {
    constexpr uint32_t MAGIC = 0x64646464u;
    const uint4 hdr = *reinterpret_cast<const uint4 *>(hdrp);
    const uint4 a = *reinterpret_cast<const uint4 *>(chunk), b = *reinterpret_cast<const uint4 *>(chunk + 16);
    const uint32_t sh = 8 * ((2 * C) & 3) + 8 * part; // `get_scale_min_k4`
    uint32_t sc, mn;
    if (C < 2) {
        sc = (hdr.y >> sh) & 63u;
        mn = (hdr.z >> sh) & 63u;
    } else {
        sc = ((hdr.w >> sh) & 0xFu) | ((((hdr.y >> sh) >> 6) & 3u) << 4);
        mn = (((hdr.w >> sh) >> 4) & 0xFu) | ((((hdr.z >> sh) >> 6) & 3u) << 4);
    }
    const uint32_t dd = live ? hdr.x : 0u;
    const __half2 d2 = h2_bits(__byte_perm(dd, 0, 0x1010)), dmin2 = h2_bits(__byte_perm(dd, 0, 0x3232));
    const __half2 sc2 = small_h2(sc), nsc = __hmul2(sc2, h2_bits(0xE400E400u)); // -1024 sc, exact
    const __half2 ndm = __hneg2(__hmul2(dmin2, small_h2(mn)));
    const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const uint32_t n4 = (w[i] >> (4 * part)) & 0x0F0F0F0Fu;
        const __half2 u0 = __hfma2(h2_bits(__byte_perm(n4, MAGIC, 0x4140)), sc2, nsc);
        const __half2 u1 = __hfma2(h2_bits(__byte_perm(n4, MAGIC, 0x4342)), sc2, nsc);
        out[2 * i] = bits_h2(__hfma2(u0, d2, ndm));
        out[2 * i + 1] = bits_h2(__hfma2(u1, d2, ndm));
    }
}
// Q6_K (device layout of blocks.cuh): group i = 2 H + part of a 128-value half: low (H = 0) or high nibbles of the
// half's ql bytes 32 part .. (l0, l1), bits 2 i .. 2 i + 1 of its 32 qh bytes (h0, h1), the two scales `sc16`
// (one per sixteen values), d as f16 bits.
template <int H>
__device__ __forceinline__ void g_decode_q6k(const uint4 &l0, const uint4 &l1, const uint4 &h0, const uint4 &h1, uint32_t sc16, uint32_t d,
                                             uint32_t part, bool live, uint32_t (&out)[16]) {
    constexpr uint32_t MAGIC = 0x64646464u;
    const uint32_t i = 2 * H + part;
    const uint32_t s0 = (sc16 & 0xFFu) ^ 0x80u, s1 = ((sc16 >> 8) & 0xFFu) ^ 0x80u; // signed scales + 128
    const uint32_t dd = live ? d : 0u;
    const __half2 d2 = h2_bits(dd | (dd << 16)), off = h2_bits(0x64806480u); // 1152 = 1024 + 128
    const __half2 ds0 = __hmul2(__hsub2(h2_bits(0x64006400u | s0 | (s0 << 16)), off), d2);
    const __half2 ds1 = __hmul2(__hsub2(h2_bits(0x64006400u | s1 | (s1 << 16)), off), d2);
    const __half2 bias = h2_bits(0x64206420u); // 1056 = 1024 + 32
    const uint32_t lw[8] = {l0.x, l0.y, l0.z, l0.w, l1.x, l1.y, l1.z, l1.w};
    const uint32_t hw[8] = {h0.x, h0.y, h0.z, h0.w, h1.x, h1.y, h1.z, h1.w};
#pragma unroll
    for (int j = 0; j < 8; j++) {
        const uint32_t lo4 = H == 0 ? lw[j] : (lw[j] >> 4);
        const uint32_t q4 = (lo4 & 0x0F0F0F0Fu) | (((hw[j] >> (2 * i)) & 0x03030303u) << 4);
        const __half2 ds = j < 4 ? ds0 : ds1;
        out[2 * j] = bits_h2(__hmul2(__hsub2(h2_bits(__byte_perm(q4, MAGIC, 0x4140)), bias), ds));
        out[2 * j + 1] = bits_h2(__hmul2(__hsub2(h2_bits(__byte_perm(q4, MAGIC, 0x4342)), bias), ds));
    }
}

// X (fp32) for the fp16 expert-tile kernel below: row r of the sorted set (row src[r] / src_div of x, or r; gated by x_up as `k_swiglu`
// does when given) times a power of two s that brings its largest magnitude into [2^13, 2^14), as two fp16
// terms hi = fp16(s x), lo = fp16(s x - hi) -- 22 bits of every value, no fp16 overflow whatever the row holds.
// Rows row_begin .. row_end - 1 go to out: [row - row_begin][2][cols] (a row's hi term, then its lo term) and
// inv_scale[row - row_begin] = 1 / s.  One warp per row; only rows [range[0], range[range_stride]) -- those some
// group covers -- are written.
__global__ void __launch_bounds__(256)
k_split_f16(const float *__restrict__ x, const float *__restrict__ x_up, const uint32_t *__restrict__ src, uint32_t src_div,
            const uint32_t *__restrict__ range, uint32_t range_stride, uint32_t row_begin, uint32_t row_end, uint32_t cols,
            __half *__restrict__ out, float *__restrict__ inv_scale) {
    const uint32_t r = row_begin + ((blockIdx.x * blockDim.x + threadIdx.x) >> 5), lane = threadIdx.x & 31;
    if (r >= row_end) return;
    if (range && (r < range[0] || r >= range[range_stride])) return;
    const size_t srow = src ? src[r] / src_div : r;
    const float4 *xp = reinterpret_cast<const float4 *>(x + srow * cols), *up = x_up ? reinterpret_cast<const float4 *>(x_up + srow * cols) : nullptr;
    auto value = [&](uint32_t i) {
        float4 v = xp[i];
        if (up) {
            const float4 u = up[i];
            v.x = v.x / (1.f + expf(-v.x)) * u.x;
            v.y = v.y / (1.f + expf(-v.y)) * u.y;
            v.z = v.z / (1.f + expf(-v.z)) * u.z;
            v.w = v.w / (1.f + expf(-v.w)) * u.w;
        }
        return v;
    };
    float amax = 0.f;
    for (uint32_t i = lane; i < cols / 4; i += 32) {
        const float4 v = value(i);
        amax = fmaxf(fmaxf(amax, fmaxf(fabsf(v.x), fabsf(v.y))), fmaxf(fabsf(v.z), fabsf(v.w)));
    }
#pragma unroll
    for (int d = 16; d; d >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, d));
    // fmaxf drops NaNs: a row holding one keeps the scale of its finite values and the NaN travels in hi.
    int e = 0;
    if (amax > 0.f && amax <= 3.0e38f) e = min(max(13 - ilogbf(amax), -100), 100);
    const float s = scalbnf(1.f, e);
    if (lane == 0) inv_scale[r - row_begin] = scalbnf(1.f, -e);
    __half *hi = out + (size_t)2 * (r - row_begin) * cols, *lo = hi + cols;
    for (uint32_t i = lane; i < cols / 4; i += 32) {
        const float4 v = value(i);
        const float a[4] = {v.x * s, v.y * s, v.z * s, v.w * s};
        __half h[4], l[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            h[j] = __float2half_rn(a[j]);
            l[j] = __float2half_rn(a[j] - __half2float(h[j]));
        }
        *reinterpret_cast<uint2 *>(hi + 4 * i) = make_uint2(bits_h2(__halves2half2(h[0], h[1])), bits_h2(__halves2half2(h[2], h[3])));
        *reinterpret_cast<uint2 *>(lo + 4 * i) = make_uint2(bits_h2(__halves2half2(l[0], l[1])), bits_h2(__halves2half2(l[2], l[3])));
    }
}


template <int FMT>
__global__ void __launch_bounds__(G_THREADS, 1)
k_gemm_f16g(const __grid_constant__ GMaps M, const __grid_constant__ GJob J) {
    extern __shared__ uint8_t smem_raw[];
    GSmem<FMT> *sm = reinterpret_cast<GSmem<FMT> *>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t nblk = J.cols / 256, k_iters = J.cols / BK, tiles_x = J.tx_end[J.count - 1];
    constexpr uint32_t TMEM_COLS = 2 * G_BN; // two accumulators
    constexpr int W_STAGES = GRaw<FMT>::W_STAGES;

    if (threadIdx.x == 0) {
        for (int s = 0; s < W_STAGES; s++) {
            mbar_init(&sm->full_w[s], G_PRODUCER_WARPS); // one lane arrives for its warp
            mbar_init(&sm->empty_w[s], 1);
        }
        for (int s = 0; s < GRaw<FMT>::X_SLOTS; s++) {
            mbar_init(&sm->full_x[s], 1);
            mbar_init(&sm->empty_x[s], 1);
        }
        for (int i = 0; i < 2; i++) {
            mbar_init(&sm->acc_full[i], 1);
            mbar_init(&sm->acc_empty[i], G_EPI_WARPS * 32);
        }
        mbar_init(&sm->drain, 1);
        for (int s = 0; s < GRaw<FMT>::STAGES; s++) {
            mbar_init(&sm->raw_full[s], 1);
            mbar_init(&sm->raw_empty[s], G_PRODUCER_WARPS);
        }
        sm->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        for (int i = 0; i < 3; i++) asm volatile("prefetch.tensormap [%0];" ::"l"(&M.x[i]) : "memory");
        if (FMT == FQ_Q4_K)
            for (uint32_t i = 0; i < J.count; i++) asm volatile("prefetch.tensormap [%0];" ::"l"(&M.w[i][0]) : "memory");
    }
    if (warp == 0) {
        // The table of activation tiles: group z contributes ceil(rows / 64) tiles for its rows inside this
        // launch's range; 32 groups per step, tile counts prefix-summed with shuffles.
        uint32_t base = 0;
        for (uint32_t g0 = 0; g0 < J.groups; g0 += 32) {
            const uint32_t g = g0 + lane;
            uint32_t first = 0, cnt = 0, e = 0;
            if (g < J.groups) {
                const uint32_t end = min(J.offsets[g + 1], J.row_end);
                first = max(J.offsets[g], J.row_begin);
                cnt = end > first ? end - first : 0u;
                e = J.slots ? J.slots[g] : g;
                if (e >= J.experts) cnt = 0;
            }
            const uint32_t t = (cnt + G_TOK - 1) / G_TOK;
            uint32_t incl = t;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const uint32_t n = __shfl_up_sync(0xffffffffu, incl, d);
                if (lane >= d) incl += n;
            }
            for (uint32_t j = 0; j < t; j++) {
                const uint32_t at = base + incl - t + j;
                if (at < G_MAX_TILES) sm->tiles[at] = make_uint2(first + j * G_TOK, (e << 8) | min(G_TOK, cnt - j * G_TOK));
            }
            base += __shfl_sync(0xffffffffu, incl, 31);
        }
        if (lane == 0) sm->n_tiles = min(base, G_MAX_TILES); // the launcher admits no more
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm->tmem_base)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *(volatile uint32_t *)&sm->tmem_base;
    const uint32_t n_items = sm->n_tiles * tiles_x;
    const uint32_t my_items = n_items > blockIdx.x ? (n_items - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;

    // Item i of this block: activation tile, matrix set and first weight row.
    struct Item {
        uint32_t m0, cnt, e, set, n0;
    };
    auto item_at = [&](uint32_t i) {
        const uint32_t id = blockIdx.x + i * gridDim.x, a = id / tiles_x;
        uint32_t tx = id - a * tiles_x;
        const uint2 t = sm->tiles[a];
        Item it;
        it.m0 = t.x;
        it.cnt = t.y & 0xFFu;
        it.e = t.y >> 8;
        it.set = (J.count > 1 && tx >= J.tx_end[0]) ? 1u : 0u;
        if (it.set) tx -= J.tx_end[0];
        it.n0 = tx * G_BN;
        return it;
    };

    if (warp == 0) {
        if (lane == 0) {
            uint32_t ix = 0;
            bool ok = true;
            for (uint32_t i = 0; i < my_items && ok; i++) {
                const Item it = item_at(i);
                // One box per k-block: the tile's rows with their hi and lo terms interleaved (32, 64 or 128 tensor
                // rows; a box that runs past the tile reads rows whose results are not stored, or zeros past the
                // end; MMA rows the box does not cover keep what an earlier tile left there).
                const CUtensorMap *map = it.cnt <= 16 ? &M.x[0] : it.cnt <= 32 ? &M.x[1] : &M.x[2];
                const uint32_t bytes = (it.cnt <= 16 ? J.box_bytes[0] : it.cnt <= 32 ? J.box_bytes[1] : J.box_bytes[2]);
                for (uint32_t k = 0; k < k_iters; k++, ix++) {
                    const uint32_t s = ix % GRaw<FMT>::X_SLOTS;
                    if (!(ok = mbar_wait(&sm->empty_x[s], ((ix / GRaw<FMT>::X_SLOTS) & 1) ^ 1, sm, J.status))) break;
                    mbar_expect_tx(&sm->full_x[s], bytes);
                    tma_load_2d(sm->x[s], map, (int)(k * BK), (int)(2 * (it.m0 - J.row_begin)), &sm->full_x[s]);
                }
            }
            // On an abort the copies already issued still land: wait for them (bounded) before the block's
            // shared memory goes away.
            if (*(volatile uint32_t *)&sm->abort_flag)
                for (uint32_t u = ix > (uint32_t)GRaw<FMT>::X_SLOTS ? ix - GRaw<FMT>::X_SLOTS : 0; u < ix; u++)
                    for (uint32_t n = 0; n < WAIT_LIMIT && !mbar_try(&sm->full_x[u % GRaw<FMT>::X_SLOTS], (u / GRaw<FMT>::X_SLOTS) & 1); n++) {}
        }
    } else if (warp == 1) {
        if (lane == 0) {
            uint32_t it_n = 0;
            bool ok = true;
            for (uint32_t i = 0; i < my_items && ok; i++) {
                const uint32_t buf = i & 1, acc = tmem + buf * G_BN;
                if (!(ok = mbar_wait(&sm->acc_empty[buf], ((i >> 1) & 1) ^ 1, sm, J.status))) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                for (uint32_t k = 0; k < k_iters; k++, it_n++) {
                    const uint32_t sw = it_n % W_STAGES, sx = it_n % GRaw<FMT>::X_SLOTS;
                    if (!(ok = mbar_wait(&sm->full_w[sw], (it_n / W_STAGES) & 1, sm, J.status))) break;
                    if (!(ok = mbar_wait(&sm->full_x[sx], (it_n / GRaw<FMT>::X_SLOTS) & 1, sm, J.status))) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint64_t adesc = umma_desc(smem_u32(sm->x[sx])), bdesc = umma_desc(smem_u32(sm->w[sw]));
#pragma unroll
                    for (int kk = 0; kk < BK / 16; kk++) umma_bf16(acc, adesc + 2 * kk, bdesc + 2 * kk, G_IDESC, (k | kk) != 0);
                    umma_commit(&sm->empty_x[sx]);
                    umma_commit(&sm->empty_w[sw]);
                }
                if (ok) umma_commit(&sm->acc_full[buf]);
            }
            umma_commit(&sm->drain); // arrives when every MMA issued so far has completed
        }
    } else if (warp == 2) {
        // Q4_K: one thread asks the TMA for every half superblock of every item's 256 rows, as many stages ahead as
        // the ring holds.  The decoding threads so have no loads of their own in flight (their
        // proxy fence would wait for them), and the copies do not queue behind the SM's load unit.
        if constexpr (FMT == FQ_Q4_K) {
        if (lane == 0) {
            constexpr int RAW = GRaw<FMT>::STAGES;
            uint32_t ir = 0;
            bool ok = true;
            for (uint32_t i = 0; i < my_items && ok; i++) {
                const Item it = item_at(i);
                const int y = (int)(it.e * J.rows + it.n0);
                const CUtensorMap *maps = M.w[it.set];
                for (uint32_t hb = 0; hb < 2 * nblk; hb++, ir++) { // half superblocks
                    const uint32_t s = ir % RAW, sb = hb >> 1, half = hb & 1;
                    if (!(ok = mbar_wait(&sm->raw_empty[s], ((ir / RAW) & 1) ^ 1, sm, J.status))) break;
                    mbar_expect_tx(&sm->raw_full[s], GRaw<FMT>::BYTES);
                    uint8_t *dst = sm->raw[s];
                    tma_load_2d(dst, &maps[0], (int)(sb * 144), y, &sm->raw_full[s]);
                    tma_load_2d(dst + GRaw<FMT>::QS, &maps[1], (int)(sb * 144 + 16 + 64 * half), y, &sm->raw_full[s]);
                }
            }
            if (*(volatile uint32_t *)&sm->abort_flag) // copies already issued still land: wait for them (bounded)
                for (uint32_t u = ir > (uint32_t)RAW ? ir - RAW : 0; u < ir; u++)
                    for (uint32_t n = 0; n < WAIT_LIMIT && !mbar_try(&sm->raw_full[u % RAW], (u / RAW) & 1); n++) {}
        }
        }
    } else if (warp < 3 + G_PRODUCER_WARPS) {
        // Decoding warp pw owns weight rows 16 pw .. 16 pw + 15 of every tile; lane = (row, group of the k-block).
        const uint32_t pw = warp - 3, lrow = lane >> 1, part = lane & 1, r = 16 * pw + lrow;
        uint32_t stage = 0, phase = 1;
        bool go = true, live = false;
        const uint32_t swz = r & 7;
        auto emit = [&](const uint32_t (&v)[16]) {
            // One lane waits and, below, arrives for the warp: hundreds of arrivals on one barrier would
            // serialise in the shared-memory atomics.
            bool ok = true;
            if (lane == 0) ok = mbar_wait(&sm->empty_w[stage], phase, sm, J.status);
            if (!__all_sync(0xffffffffu, ok)) { go = false; return; }
            uint8_t *dst = sm->w[stage] + r * 128;
#pragma unroll
            for (int u = 0; u < 4; u++) // the group's four 16-byte chunks, at their swizzled places
                *reinterpret_cast<uint4 *>(dst + 16 * ((4 * part + u) ^ swz)) = make_uint4(v[4 * u], v[4 * u + 1], v[4 * u + 2], v[4 * u + 3]);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); // generic-proxy stores -> tensor-core reads
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm->full_w[stage]);
            if (++stage == (uint32_t)W_STAGES) {
                stage = 0;
                phase ^= 1;
            }
        };
        uint32_t v[16];
        if constexpr (FMT == FQ_Q4_K) {
            constexpr int RAW = GRaw<FMT>::STAGES;
            uint32_t ir = 0;
            for (uint32_t i = 0; i < my_items && go; i++) {
                live = item_at(i).n0 + r < J.rows;
                for (uint32_t hb = 0; hb < 2 * nblk && go; hb++, ir++) { // half superblocks: two k-blocks each
                    const uint32_t rs = ir % RAW, sb = hb >> 1;
                    bool ok = true;
                    if (lane == 0) ok = mbar_wait(&sm->raw_full[rs], (ir / RAW) & 1, sm, J.status);
                    if (!__all_sync(0xffffffffu, ok)) { go = false; break; }
                    const uint8_t *st = sm->raw[rs];
                    const uint8_t *hdrp = st + 16 * r, *qs = st + GRaw<FMT>::QS + 64 * r;
                    if (hb & 1) {
                        g_decode_q4k<2>(hdrp, qs, part, live, v);
                        emit(v);
                        if (go) { g_decode_q4k<3>(hdrp, qs + 32, part, live, v); emit(v); }
                    } else {
                        g_decode_q4k<0>(hdrp, qs, part, live, v);
                        emit(v);
                        if (go) { g_decode_q4k<1>(hdrp, qs + 32, part, live, v); emit(v); }
                    }
                    __syncwarp(); // every lane is done with the stage
                    if (lane == 0) mbar_arrive(&sm->raw_empty[rs]);
                }
            }
        } else {
            // Q6_K: thread (row, group) fetches its own packed bytes, a superblock ahead and across item borders
            // (items of this format are short -- K = 512 is two superblocks -- and the staging ring above would
            // restart with every item).
            auto row_of = [&](uint32_t i) {
                const Item it = item_at(i);
                return J.w[it.set] + ((size_t)it.e * J.rows + min(it.n0 + r, J.rows - 1)) * J.pitch;
            };
            // The superblock whose bytes are fetched next: one ahead of the one being decoded, across item borders.
            uint32_t n_i = 0, n_sb = 0;
            const uint8_t *n_row = my_items ? row_of(0) : nullptr;
            auto step_next = [&]() {
                if (++n_sb == nblk) {
                    n_sb = 0;
                    if (++n_i < my_items) n_row = row_of(n_i);
                }
            };
            // Per superblock: the sixteen scales and d; per 128-value half: 32 ql bytes (this group's) and 32 qh bytes.
            uint4 sc = make_uint4(0, 0, 0, 0), sc_next = sc, ql[2][2], qh[2][2];
            uint32_t d = 0, d_next = 0;
#pragma unroll
            for (int n = 0; n < 2; n++) ql[n][0] = ql[n][1] = qh[n][0] = qh[n][1] = make_uint4(0, 0, 0, 0);
            auto load_half = [&](const uint8_t *row, uint32_t b, int n) {
                const uint8_t *l = row + (size_t)b * 128 + 64 * n + 32 * part, *h = row + (size_t)nblk * 128 + (size_t)b * 64 + 32 * n;
                ql[n][0] = *reinterpret_cast<const uint4 *>(l);
                ql[n][1] = *reinterpret_cast<const uint4 *>(l + 16);
                qh[n][0] = *reinterpret_cast<const uint4 *>(h);
                qh[n][1] = *reinterpret_cast<const uint4 *>(h + 16);
            };
            if (my_items) {
                sc = *reinterpret_cast<const uint4 *>(n_row + (size_t)nblk * 192);
                d = *reinterpret_cast<const uint16_t *>(n_row + (size_t)nblk * 208);
                load_half(n_row, 0, 0);
                load_half(n_row, 0, 1);
                step_next();
            }
            bool has_next = n_i < my_items;
            const uint8_t *next_row = n_row;
            uint32_t next_sb = n_sb;
            if (has_next) {
                sc_next = *reinterpret_cast<const uint4 *>(next_row + (size_t)nblk * 192 + (size_t)next_sb * 16);
                d_next = *reinterpret_cast<const uint16_t *>(next_row + (size_t)nblk * 208 + (size_t)next_sb * 2);
            }
            for (uint32_t i = 0; i < my_items && go; i++) {
                live = item_at(i).n0 + r < J.rows;
                for (uint32_t sb = 0; sb < nblk && go; sb++) {
                    // scales 8 n + 2 (2 H + part) and + 1: word 2 n + H of the sixteen, half `part` of it
                    const uint32_t shift = 16 * part;
#define FQ_G_HALF(N, W0, W1)                                                                                           \
    if (go) {                                                                                                          \
        g_decode_q6k<0>(ql[N][0], ql[N][1], qh[N][0], qh[N][1], (W0) >> shift, d, part, live, v);                      \
        emit(v);                                                                                                       \
    }                                                                                                                  \
    if (go) {                                                                                                          \
        g_decode_q6k<1>(ql[N][0], ql[N][1], qh[N][0], qh[N][1], (W1) >> shift, d, part, live, v);                      \
        if (has_next) load_half(next_row, next_sb, N);                                                                 \
        emit(v);                                                                                                       \
    }
                    FQ_G_HALF(0, sc.x, sc.y) FQ_G_HALF(1, sc.z, sc.w)
#undef FQ_G_HALF
                    sc = sc_next;
                    d = d_next;
                    if (has_next) {
                        step_next();
                        has_next = n_i < my_items;
                        next_row = n_row;
                        next_sb = n_sb;
                        if (has_next) {
                            sc_next = *reinterpret_cast<const uint4 *>(next_row + (size_t)nblk * 192 + (size_t)next_sb * 16);
                            d_next = *reinterpret_cast<const uint16_t *>(next_row + (size_t)nblk * 208 + (size_t)next_sb * 2);
                        }
                    }
                }
            }
        }
    } else {
        // Epilogue: a warp may read the 32 tensor-memory lanes of quarter warp % 4: MMA rows 32 quarter + lane, i.e.
        // activation row 16 quarter + lane / 2, term lane % 2.  Partner lanes exchange halves of each 32-column
        // chunk, so that the even lane ends up with the sums of columns 0..15 and the odd lane with 16..31.
        const int quarter = warp & 3;
        const uint32_t lanes = (uint32_t)(32 * quarter) << 16, trow = 16 * quarter + (lane >> 1), half = lane & 1;
        for (uint32_t i = 0; i < my_items; i++) {
            const Item it = item_at(i);
            const uint32_t buf = i & 1, acc = tmem + buf * G_BN + lanes;
            if (!mbar_wait(&sm->acc_full[buf], (i >> 1) & 1, sm, J.status)) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const bool valid = trow < it.cnt;
            const float scale = valid ? __ldg(J.inv_scale + (it.m0 - J.row_begin) + trow) : 0.f;
            float *yrow = J.y[it.set] + (size_t)(it.m0 + trow) * J.rows + it.n0 + 16 * half;
            for (uint32_t c0 = 0; c0 < G_BN && it.n0 + c0 < J.rows; c0 += 32) {
                uint32_t v[32];
                tmem_ld32(acc + c0, v);
                float o[16];
#pragma unroll
                for (int j = 0; j < 16; j++) {
                    const float keep = __uint_as_float(half ? v[16 + j] : v[j]), send = __uint_as_float(half ? v[j] : v[16 + j]);
                    o[j] = (keep + __shfl_xor_sync(0xffffffffu, send, 1)) * scale;
                }
                if (valid && it.n0 + c0 + 16 * half < J.rows) { // rows is a multiple of 16
#pragma unroll
                    for (int j = 0; j < 4; j++) *reinterpret_cast<float4 *>(yrow + c0 + 4 * j) = make_float4(o[4 * j], o[4 * j + 1], o[4 * j + 2], o[4 * j + 3]);
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            mbar_arrive(&sm->acc_empty[buf]);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        // Outstanding MMAs must have finished before the accumulator columns are released.
        if (lane == 0)
            for (uint32_t n = 0; n < WAIT_LIMIT && !mbar_try(&sm->drain, 0); n++) {}
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}

// The packed rows of a matrix (or a stack of experts) as a [rows][pitch] tensor of bytes, boxes of `box_bytes` x 256
// rows, no swizzle: what k_gemm_f16g stages per superblock.
int make_byte_map(fq_device *dev, CUtensorMap *map, const void *w, uint32_t pitch, uint64_t rows, uint32_t box_bytes) {
    EncodeTiled encode = encode_fn();
    if (!encode) return FQ_ERR_UNSUPPORTED;
    const cuuint64_t dims[2] = {pitch, rows};
    const cuuint64_t strides[1] = {pitch};
    const cuuint32_t box[2] = {box_bytes, (cuuint32_t)std::min<uint64_t>(rows, 256)}, elem[2] = {1, 1};
    CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(w), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fq_fail(dev, FQ_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d)", (int)r);
    return FQ_OK;
}

} // namespace

// X as bf16 in the handle's scratch (the halves of which successive calls alternate between), or null if
// it does not fit.
static const void *x_as_bf16(fq_device *dev, const void *x, size_t n) {
    if (n * 2 > dev->xprep_bytes / 2) return nullptr;
    dev->xprep_turn ^= 1u;
    __nv_bfloat16 *tmp = (__nv_bfloat16 *)((uint8_t *)dev->xprep + (dev->xprep_turn ? dev->xprep_bytes / 2 : 0));
    k_to_bf16<<<(unsigned)((n / 4 + 255) / 256 + 1), 256, 0, dev->stream>>>((const float *)x, tmp, n);
    return tmp;
}

// Dense projection wider than the verify widths.  BF16 in / BF16 out: one bf16 product per weight (the legacy
// `*_gemm_mpp*` contract: bf16 operands, fp32 accumulation, bf16 RNE out).  F32 in / F32 out: the three-term
// split of k_gemm_tc's MODE 2, in slices of activation rows whose split copy fits the handle's scratch.
int fq_launch_gemm_tc(fq_device *dev, const ProjectArgs &a) {
    if (a.x_dtype != a.y_dtype || a.cols % BK || a.ids || a.offsets) return FQ_ERR_UNSUPPORTED;
    if (a.format != FQ_Q4_K && a.format != FQ_Q5_K && a.format != FQ_Q6_K && a.format != FQ_Q8_0) return FQ_ERR_UNSUPPORTED;
    if (a.format == FQ_Q4_K && (a.row_bytes % 16)) return FQ_ERR_UNSUPPORTED;
    if (a.m <= (uint32_t)FQ_GEMV_MAX_M) return FQ_ERR_UNSUPPORTED; // decode and verify widths: the fp32 kernels serve them
    CUtensorMap map;
    uint32_t b_bytes = 0;
    if (a.x_dtype == FQ_BF16) {
        if (int rc = make_map(dev, &map, a.x, a.cols, a.m, 256, &b_bytes)) return rc;
        // 512 activation rows per block (two accumulators sharing each decoded weight tile) once there are
        // enough rows to fill them; the TMA box stays 256 rows.
        const int rc = a.m >= 384 ? launch_fmt<512, __nv_bfloat16, 0>(dev, a, map, b_bytes, a.m)
                                  : launch_fmt<256, __nv_bfloat16, 0>(dev, a, map, b_bytes, a.m);
        if (rc != FQ_OK) return rc;
        return fq_end_enqueue(dev, "gemm_tc", 1);
    }
    const size_t half = dev->xprep_bytes / 2, row_bytes3 = (size_t)a.cols * 3 * sizeof(__nv_bfloat16);
    uint32_t slice = (uint32_t)std::min<size_t>(a.m, half / row_bytes3);
    if (slice < a.m) slice = slice >= 512 ? (slice & ~511u) : (slice & ~255u); // whole tiles per slice
    if (slice == 0) return FQ_ERR_UNSUPPORTED;
    int kernels = 0;
    for (uint32_t m0 = 0; m0 < a.m; m0 += slice) {
        const uint32_t mm = std::min(slice, a.m - m0);
        dev->xprep_turn ^= 1u;
        __nv_bfloat16 *x3 = (__nv_bfloat16 *)((uint8_t *)dev->xprep + (dev->xprep_turn ? half : 0));
        const size_t n = (size_t)mm * a.cols;
        k_split3<<<(unsigned)((n + 255) / 256), 256, 0, dev->stream>>>((const float *)a.x + (size_t)m0 * a.cols, x3, a.cols, n);
        if (int rc = make_map(dev, &map, x3, a.cols * 3, mm, 256, &b_bytes)) return rc;
        ProjectArgs s = a;
        s.m = mm;
        s.y = (float *)a.y + (size_t)m0 * a.rows;
        const int rc = mm >= 384 ? launch_fmt<512, float, 2>(dev, s, map, b_bytes, mm) : launch_fmt<256, float, 2>(dev, s, map, b_bytes, mm);
        if (rc != FQ_OK) return rc;
        kernels += 2;
    }
    return fq_end_enqueue(dev, "gemm_tc", kernels);
}

// `a[0..count)` share X, m, format and width (no routes): one launch over all their row tiles.  BF16 in / BF16
// out, or F32 in / F32 out on the three-term split when the split copy of X fits one half of the scratch.
int fq_launch_gemm_tc_many(fq_device *dev, const ProjectArgs *a, uint32_t count) {
    if (count < 2 || count > 4) return FQ_ERR_UNSUPPORTED;
    const ProjectArgs &f = a[0];
    const bool wide = f.x_dtype == FQ_F32 && f.y_dtype == FQ_F32;
    if (!wide && (f.x_dtype != FQ_BF16 || f.y_dtype != FQ_BF16)) return FQ_ERR_UNSUPPORTED;
    if (f.cols % BK || f.ids || f.offsets) return FQ_ERR_UNSUPPORTED;
    if (f.format != FQ_Q4_K && f.format != FQ_Q5_K && f.format != FQ_Q6_K && f.format != FQ_Q8_0) return FQ_ERR_UNSUPPORTED;
    if (f.format == FQ_Q4_K && (f.row_bytes % 16)) return FQ_ERR_UNSUPPORTED;
    if (f.m <= (uint32_t)FQ_GEMV_MAX_M) return FQ_ERR_UNSUPPORTED;
    if (wide && (size_t)f.m * f.cols * 3 * sizeof(__nv_bfloat16) > dev->xprep_bytes / 2) return FQ_ERR_UNSUPPORTED;
    GemmMany many{};
    many.count = count;
    uint32_t tx = 0;
    for (uint32_t i = 0; i < count; i++) {
        if (a[i].format != f.format || a[i].cols != f.cols || a[i].x != f.x || a[i].m != f.m || a[i].ids || a[i].offsets ||
            a[i].x_dtype != f.x_dtype || a[i].y_dtype != f.y_dtype || a[i].row_bytes != f.row_bytes)
            return FQ_ERR_UNSUPPORTED;
        many.w[i] = a[i].w;
        many.y[i] = a[i].y;
        many.rows[i] = a[i].rows;
        tx += (a[i].rows + BM - 1) / BM;
        many.tx_end[i] = tx;
    }
    CUtensorMap map;
    uint32_t b_bytes = 0;
    if (wide) {
        dev->xprep_turn ^= 1u;
        __nv_bfloat16 *x3 = (__nv_bfloat16 *)((uint8_t *)dev->xprep + (dev->xprep_turn ? dev->xprep_bytes / 2 : 0));
        const size_t n = (size_t)f.m * f.cols;
        k_split3<<<(unsigned)((n + 255) / 256), 256, 0, dev->stream>>>((const float *)f.x, x3, f.cols, n);
        if (int rc = make_map(dev, &map, x3, f.cols * 3, f.m, 256, &b_bytes)) return rc;
        const int rc = f.m >= 384 ? launch_fmt<512, float, 2>(dev, f, map, b_bytes, f.m, many) : launch_fmt<256, float, 2>(dev, f, map, b_bytes, f.m, many);
        if (rc != FQ_OK) return rc;
        return fq_end_enqueue(dev, "gemm_tc", 2);
    }
    if (int rc = make_map(dev, &map, f.x, f.cols, f.m, 256, &b_bytes)) return rc;
    const int rc = f.m >= 384 ? launch_fmt<512, __nv_bfloat16, 0>(dev, f, map, b_bytes, f.m, many)
                              : launch_fmt<256, __nv_bfloat16, 0>(dev, f, map, b_bytes, f.m, many);
    if (rc != FQ_OK) return rc;
    return fq_end_enqueue(dev, "gemm_tc", 1);
}

// Expert-sorted rows (`project_mm_id_in`): x is [total_rows][cols], F32 (converted to bf16 into the
// handle's scratch first) or BF16; y is F32 or BF16.
int fq_launch_gemm_tc_grouped(fq_device *dev, const ProjectArgs &a, uint32_t total_rows) {
    if (a.cols % BK || !a.offsets) return FQ_ERR_UNSUPPORTED;
    if (a.format != FQ_Q4_K && a.format != FQ_Q5_K && a.format != FQ_Q6_K && a.format != FQ_Q8_0) return FQ_ERR_UNSUPPORTED;
    if (a.format == FQ_Q4_K && (a.row_bytes % 16)) return FQ_ERR_UNSUPPORTED;
    if (a.groups > 65535 || total_rows == 0) return FQ_ERR_UNSUPPORTED;
    const void *xb = a.x;
    int kernels = 1;
    if (a.x_dtype == FQ_F32) {
        if (!(xb = x_as_bf16(dev, a.x, (size_t)total_rows * a.cols))) return FQ_ERR_UNSUPPORTED;
        kernels = 2;
    }
    CUtensorMap map;
    uint32_t b_bytes = 0;
    if (int rc = make_map(dev, &map, xb, a.cols, total_rows, 64, &b_bytes)) return rc;
    int rc = a.y_dtype == FQ_F32 ? launch_fmt<64, float, 1>(dev, a, map, b_bytes, total_rows)
                                 : launch_fmt<64, __nv_bfloat16, 1>(dev, a, map, b_bytes, total_rows);
    if (rc != FQ_OK) return rc;
    return fq_end_enqueue(dev, "gemm_tc_grouped", kernels);
}

// Expert-sorted rows, F32 in and out, on k_gemm_f16g: up to two matrix sets of one shape sharing the rows
// (gate and up); `src`, `src_div`, `a[0].x_up` as for `fq_launch_gemv_nt_grouped`.  The fp16 copy of the rows
// takes the whole activation scratch (this path enqueues plain launches only, so nothing before it still
// reads the scratch and nothing after it writes early); more rows than it holds are served in several launches.
int fq_launch_gemm_f16_grouped(fq_device *dev, const ProjectArgs *a, uint32_t count, uint32_t total_rows, const uint32_t *src, uint32_t src_div) {
    const ProjectArgs &f = a[0];
    if (count == 0 || count > 2 || f.cols % 256 || f.row_bytes % 16 || f.rows % 16 || !f.offsets || f.x_dtype != FQ_F32 || f.y_dtype != FQ_F32 || f.norm_w)
        return FQ_ERR_UNSUPPORTED;
    if (f.format != FQ_Q4_K && f.format != FQ_Q6_K) return FQ_ERR_UNSUPPORTED;
    if (f.groups == 0 || f.groups > 65535 || f.experts > 65535 || total_rows < 16 || (src && src_div == 0)) return FQ_ERR_UNSUPPORTED;
    if (f.format == FQ_Q4_K && (uint64_t)f.experts * f.rows < G_BN) return FQ_ERR_UNSUPPORTED; // a TMA box of 256 weight rows must fit the stack
    for (uint32_t i = 1; i < count; i++)
        if (a[i].format != f.format || a[i].cols != f.cols || a[i].rows != f.rows || a[i].row_bytes != f.row_bytes || a[i].x != f.x ||
            a[i].x_up != f.x_up || a[i].offsets != f.offsets || a[i].slots != f.slots || a[i].groups != f.groups || a[i].experts != f.experts ||
            a[i].x_dtype != FQ_F32 || a[i].y_dtype != FQ_F32 || a[i].norm_w)
            return FQ_ERR_UNSUPPORTED;
    // The fp16 copy of as many rows as the activation scratch holds at a time (whole 64-row steps; a group that
    // straddles two launches is served in two parts).
    const size_t per_row = (size_t)2 * f.cols * sizeof(__half) + sizeof(float);
    uint32_t chunk = (uint32_t)std::min<size_t>(total_rows, dev->xprep_bytes / per_row);
    if (f.groups + 8 > G_MAX_TILES) return FQ_ERR_UNSUPPORTED;
    chunk = std::min<uint32_t>(chunk, (G_MAX_TILES - f.groups) * G_TOK); // the kernel's table of activation tiles holds G_MAX_TILES
    if (chunk < total_rows) chunk &= ~(G_TOK - 1);
    if (chunk < 16) return FQ_ERR_UNSUPPORTED;
    __half *xh = (__half *)dev->xprep;
    float *inv_scale = (float *)((uint8_t *)dev->xprep + (size_t)2 * chunk * f.cols * sizeof(__half));
    GJob J{};
    J.count = count;
    uint32_t tx = 0;
    for (uint32_t i = 0; i < count; i++) {
        J.w[i] = a[i].w;
        J.y[i] = (float *)a[i].y;
        tx += (a[i].rows + G_BN - 1) / G_BN;
        J.tx_end[i] = tx;
    }
    J.rows = f.rows;
    J.cols = f.cols;
    J.pitch = f.row_bytes;
    J.experts = f.experts;
    J.groups = f.groups;
    J.offsets = f.offsets;
    J.slots = f.slots;
    J.inv_scale = inv_scale;
    J.status = dev->status_dev;
    const size_t smem = (f.format == FQ_Q4_K ? sizeof(GSmem<FQ_Q4_K>) : sizeof(GSmem<FQ_Q6_K>)) + 1024;
    GMaps maps;
    for (uint32_t i = 0; i < count; i++) {
        const uint64_t wrows = (uint64_t)a[i].experts * a[i].rows;
        if (f.format == FQ_Q4_K) { // the packed bytes are staged by TMA
            if (int rc = make_byte_map(dev, &maps.w[i][0], a[i].w, f.row_bytes, wrows, 16)) return rc;
            if (int rc = make_byte_map(dev, &maps.w[i][1], a[i].w, f.row_bytes, wrows, 64)) return rc;
        }
    }
    auto kernel = f.format == FQ_Q4_K ? k_gemm_f16g<FQ_Q4_K> : k_gemm_f16g<FQ_Q6_K>;
    static bool configured[2] = {};
    bool &done = configured[f.format == FQ_Q4_K ? 0 : 1];
    if (!done) {
        if (int rc = fq_check_cuda(dev, cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), "gemm shared memory")) return rc;
        done = true;
    }
    int kernels = 0;
    for (uint32_t r0 = 0; r0 < total_rows; r0 += chunk) {
        const uint32_t r1 = std::min(total_rows, r0 + chunk), n = r1 - r0;
        if (n < 16) { // too few rows for a TMA box: the last rows again with the ones before them
            r0 = r1 - 16;
        }
        J.row_begin = r0;
        J.row_end = r1;
        k_split_f16<<<(r1 - r0 + 7) / 8, 256, 0, dev->stream>>>((const float *)f.x, f.x_up, src, src_div, f.offsets, f.groups, r0, r1, f.cols, xh, inv_scale);
        for (int i = 0; i < 3; i++)
            if (int rc = make_map(dev, &maps.x[i], xh, f.cols, 2 * (r1 - r0), 32u << i, &J.box_bytes[i], CU_TENSOR_MAP_DATA_TYPE_FLOAT16)) return rc;
        kernel<<<(unsigned)dev->sm_count, G_THREADS, smem, dev->stream>>>(maps, J);
        if (int rc = fq_check_cuda(dev, cudaGetLastError(), "grouped fp16 gemm launch")) return rc;
        kernels += 2;
        if (r1 == total_rows) break;
    }
    return fq_end_enqueue(dev, "gemm_f16_grouped", kernels);
}
