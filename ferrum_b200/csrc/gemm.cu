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
#include <cuda.h>

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
template <class SM> __device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, SM *sm, int *status) {
    if (mbar_try(bar, parity)) return true;
    const uint64_t t0 = now_ns();
    do {
        if (mbar_try(bar, parity, WAIT_HINT_NS)) return true;
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

int make_map(fq_device *dev, CUtensorMap *map, const void *x, uint32_t cols, uint32_t m_rows, uint32_t bn, uint32_t *b_bytes) {
    EncodeTiled encode = encode_fn();
    if (!encode) return FQ_ERR_UNSUPPORTED;
    const cuuint64_t dims[2] = {cols, m_rows};
    const cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    // A box may not be taller than the tensor; rows past the end of a later tile are zero-filled.
    const uint32_t box_rows = m_rows < bn ? m_rows : bn;
    const cuuint32_t box[2] = {BK, box_rows}, elem[2] = {1, 1};
    CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(x), dims, strides, box, elem,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fq_fail(dev, FQ_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d)", (int)r);
    *b_bytes = box_rows * BK * 2;
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
