// Decode projections of ONE activation row, and per-route expert projections, on the integer tensor path
// (F32 in, F32 out).  The reference's `h_mv_q4_k` / `h_mv_q5_k` / `h_mv_q6_k` (src/metal/shaders/hybrid.metal:
// 688-897) and, with routes, `h_mv_id_*` (:2390-2428).  Two to sixteen rows run in gemv_nt.cu.
//
// A K-quant GEMV on B200 is bound by instruction issue, not by HBM, if every weight costs ALU work.
// Here the packed quants never leave the integer domain:
//
//   A (16 weight rows x 32 k, u8)  = the raw quants: one AND per four Q4_K weights
//                                    (w & 0x0F0F0F0F, (w >> 4) & 0x0F0F0F0F), one more LOP3 for the fifth
//                                    bit of Q5_K, one LOP3 select per four Q6_K weights;
//   B (32 k x 8 columns, s8)       = the activations of ONE row as 16-bit integers
//                                    x' = round(x * s) = 256 * hi + lo, both halves signed bytes,
//                                    s a power of two per (row, superblock).  The four threads of a
//                                    quad own k of four different scale groups, so column c of B holds
//                                    x' only on the k slots of thread c % 4 (plane c / 4) and zeros
//                                    elsewhere: one mma.sync m16n8k32 yields, per weight row, the
//                                    integer dot products of four scale groups times two planes;
//   epilogue (integers)            = sum_groups scale_g * (dot_g [- 32 * sum x' for Q6_K]),
//                                    Q4_K / Q5_K minus dmin * sum_j m_j * sum x'; one I2F and one FMA with
//                                    d / s per row and superblock.
//
// The result is the exact dot product of the decoded weights with the activations rounded to 16 bits
// relative to the largest magnitude of their superblock (error <= 2^-16 of that maximum per
// activation; llama.cpp's CUDA GEMV, which the reference's kernels derive from, rounds to 8 bits per
// 32).  Thread (g = lane / 4, t = lane % 4) owns weight rows g, g + 8 of a 16-row tile.
//
// Two kernels share that arithmetic (`superblock_dot`):
//   k_gemv_i8s  dense matrices, one row: one block of 16 warps per SM; K is cut into slices, a block prepares
//               its slice of the activation row itself (no preparation launch; optionally with the row's
//               rmsnorm), every warp walks 16-row tiles with its own cp.async ring of weight stages; with more
//               than one slice partial sums go through a workspace and the last warp to arrive at a tile adds
//               them in slice order, so results do not depend on timing;
//   k_gemv_i8   per-route expert projections (`project_id`) and the allocation-free entry point: activations
//               prepared by k_prep_i8, weights read with 128-bit loads into registers, warps of a block split K
//               and meet in shared memory in warp order.
#include <algorithm>
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <type_traits>

#include "blocks.cuh"
#include "gemv_common.cuh"
#include "internal.h"

namespace {
using namespace fqk;

constexpr int MAX_WARPS = 16; // warps of a block split K between them; the count is chosen per launch
constexpr int MAX_TARGETS = 4;
constexpr int MAX_TOKENS = 4;


// ---------------------------------------------------------------- prepared activations
//
// Per group (one activation row in expert mode, else all rows) and token:
//   plane[2][cols] s8   hi and lo bytes of x' in natural k order
//   sx32 [cols / 32] s32   sum of x' per 32 values            (Q4_K minimum term)
//   sx16 [2][cols / 16] s16  sum of hi / lo bytes per 16 values (Q6_K "- 32" term)
//   isc  [cols / 256] f32  1 / s
struct PrepI8 {
    uint32_t cols, nblk;
    uint32_t lo_off, sx32_off, sx16_off, isc_off, token_bytes;
};

__host__ __device__ inline PrepI8 prep_i8_layout(uint32_t cols) {
    PrepI8 L;
    L.cols = cols;
    L.nblk = cols / 256;
    L.lo_off = cols;
    L.sx32_off = 2 * cols;
    L.sx16_off = L.sx32_off + cols / 32 * 4;
    L.isc_off = L.sx16_off + 2 * (cols / 16) * 2;
    L.token_bytes = (L.isc_off + L.nblk * 4 + 255u) & ~255u;
    return L;
}

// Superblock b of one activation row, by one warp (lane l owns the eight values at 256 b + 8 l), written in
// the layout above at `base` (global or shared memory).
// With `urow` the activations are the gated unit silu(x) * u, x / (1 + exp(-x)) * u as `k_swiglu` computes it.
// With `norm_w` they are rmsnorm(x) * norm_w (`h_rmsnorm`, src/metal/shaders/hybrid.metal:1563-1575).
// `bsrc` is the superblock of the row that is read, `b` the slot of the layout `L` it is written to (the same
// unless `L` describes a slice of the row); `norm_scale` = row_inv_rms of the whole row when `norm_w` is given.
struct PrepLoad { // the lane's eight values of one superblock, fetched ahead of their use
    float4 v0, v1;
    __device__ __forceinline__ void fetch(const float *__restrict__ xrow, uint32_t bsrc, uint32_t lane) {
        const float4 *src = reinterpret_cast<const float4 *>(xrow + (size_t)bsrc * 256 + lane * 8);
        v0 = src[0];
        v1 = src[1];
    }
};
__device__ __forceinline__ void prep_superblock(const PrepLoad &in, uint32_t bsrc, uint32_t b, uint32_t lane, const PrepI8 &L, uint8_t *base,
                                                const float *__restrict__ urow, const float *__restrict__ norm_w, float norm_scale) {
    const float4 v0 = in.v0, v1 = in.v1;
    float v[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
    if (norm_w) {
        const float scale = norm_scale;
        const float4 *ws = reinterpret_cast<const float4 *>(norm_w + (size_t)bsrc * 256 + lane * 8);
        const float4 w0 = ws[0], w1 = ws[1];
        const float g[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
        for (int i = 0; i < 8; i++) v[i] = v[i] * scale * g[i];
    }
    if (urow) {
        const float4 *us = reinterpret_cast<const float4 *>(urow + (size_t)bsrc * 256 + lane * 8);
        const float4 u0 = us[0], u1 = us[1];
        const float u[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
#pragma unroll
        for (int i = 0; i < 8; i++) v[i] = v[i] / (1.f + expf(-v[i])) * u[i];
    }
    const Quant8 q = quantize8(v);
    const bool finite = q.finite;
    const int e = q.e;
    int sum = q.sum, sum_hi = q.sum_hi, sum_lo = q.sum_lo;
    auto pack8 = [](const uint8_t *p) { return make_uint2(pack4(p), pack4(p + 4)); };
    const uint8_t *hi = q.hi, *lo = q.lo;
    reinterpret_cast<uint2 *>(base)[b * 32 + lane] = pack8(hi);
    reinterpret_cast<uint2 *>(base + L.lo_off)[b * 32 + lane] = pack8(lo);
    // 16-value sums (lane pairs) and 32-value sums (lane quads).
    sum_hi += __shfl_xor_sync(0xffffffffu, sum_hi, 1);
    sum_lo += __shfl_xor_sync(0xffffffffu, sum_lo, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    if ((lane & 1) == 0) {
        int16_t *s16 = reinterpret_cast<int16_t *>(base + L.sx16_off);
        s16[b * 16 + (lane >> 1)] = (int16_t)sum_hi;
        s16[L.cols / 16 + b * 16 + (lane >> 1)] = (int16_t)sum_lo;
    }
    if ((lane & 3) == 0) reinterpret_cast<int *>(base + L.sx32_off)[b * 8 + (lane >> 2)] = sum;
    if (lane == 0) {
        // A non-finite activation anywhere in the block makes the block's factor NaN.
        reinterpret_cast<float *>(base + L.isc_off)[b] = finite ? ldexpf(1.f, -e) : __int_as_float(0x7fc00000);
    }
}

__device__ __forceinline__ void prep_superblock(const float *__restrict__ xrow, uint32_t bsrc, uint32_t b, uint32_t lane, const PrepI8 &L, uint8_t *base,
                                                const float *__restrict__ urow, const float *__restrict__ norm_w, float norm_scale) {
    PrepLoad in;
    in.fetch(xrow, bsrc, lane);
    prep_superblock(in, bsrc, b, lane, L, base, urow, norm_w, norm_scale);
}

// One warp per (activation row, superblock).
__global__ void __launch_bounds__(128)
k_prep_i8(const float *__restrict__ x, const float *__restrict__ x_up, const float *__restrict__ norm_w, float eps, uint32_t xrows, PrepI8 L,
          uint8_t *__restrict__ out) {
    pdl_trigger();
    pdl_wait();
    const uint32_t warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    const uint32_t xr = warp / L.nblk, b = warp % L.nblk;
    if (xr >= xrows) return;
    const float *xrow = x + (size_t)xr * L.cols;
    prep_superblock(xrow, b, b, lane, L, out + (size_t)xr * L.token_bytes, x_up ? x_up + (size_t)xr * L.cols : nullptr, norm_w,
                    norm_w ? row_inv_rms(xrow, L.cols, eps, lane) : 0.f);
}

// ---------------------------------------------------------------- helpers

// Q4_K: the header, 16 bytes of chunk t / 2 and 16 bytes of chunk 2 + t / 2 (bytes 16 (t % 2) .. of each
// chunk's 32), so that the four threads of a quad read 64 contiguous bytes per instruction.
struct Q4Raw {
    uint4 hdr, qa, qb;
    __device__ __forceinline__ void load(const uint8_t *row, uint32_t, uint32_t b, int t) {
        const uint8_t *blk = row + (size_t)b * 144;
        hdr = ldw128(blk);
        qa = ldw128(blk + 16 + 16 * t);
        qb = ldw128(blk + 80 + 16 * t);
    }
    // From a row of a ring stage (shared memory): the block's 144 bytes.
    __device__ __forceinline__ void load_staged(const uint8_t *r, uint32_t, int t) {
        hdr = *reinterpret_cast<const uint4 *>(r);
        qa = *reinterpret_cast<const uint4 *>(r + 16 + 16 * t);
        qb = *reinterpret_cast<const uint4 *>(r + 80 + 16 * t);
    }
};
// Q5_K: as Q4_K, plus the 16 bytes of qh under this thread's run (bit j of qh[l] = fifth bit of value l of sub-block j).
struct Q5Raw {
    uint4 hdr, qa, qb, qh;
    __device__ __forceinline__ void load(const uint8_t *row, uint32_t, uint32_t b, int t) {
        const uint8_t *blk = row + (size_t)b * 176;
        hdr = ldw128(blk);
        qh = ldw128(blk + 16 + 16 * (t & 1));
        qa = ldw128(blk + 48 + 16 * t);
        qb = ldw128(blk + 112 + 16 * t);
    }
    __device__ __forceinline__ void load_staged(const uint8_t *r, uint32_t, int t) {
        hdr = *reinterpret_cast<const uint4 *>(r);
        qh = *reinterpret_cast<const uint4 *>(r + 16 + 16 * (t & 1));
        qa = *reinterpret_cast<const uint4 *>(r + 48 + 16 * t);
        qb = *reinterpret_cast<const uint4 *>(r + 112 + 16 * t);
    }
};
struct Q6Raw;
template <int FMT> struct RawOf { using type = Q6Raw; };
template <> struct RawOf<FQ_Q4_K> { using type = Q4Raw; };
template <> struct RawOf<FQ_Q5_K> { using type = Q5Raw; };
template <int FMT> constexpr bool is_k45 = FMT == FQ_Q4_K || FMT == FQ_Q5_K;
struct Q6Raw { // device layout of blocks.cuh; thread t = (n, lh)
    uint4 q0, q1, qh; // ql of 32-groups 0|2 and 1|3 of half n, qh of half n: run lh (16 bytes each)
    uint2 sc;         // the 8 scales of half t % 2 (the half whose groups this thread sums up)
    uint32_t d;
    __device__ __forceinline__ void load(const uint8_t *row, uint32_t nblk, uint32_t b, int t) {
        const int n = t >> 1, lh = t & 1;
        const uint8_t *ql = row + (size_t)b * 128 + 64 * n + 16 * lh;
        q0 = ldw128(ql);
        q1 = ldw128(ql + 32);
        qh = ldw128(row + (size_t)nblk * 128 + (size_t)b * 64 + 32 * n + 16 * lh);
        sc = ldw64(row + (size_t)nblk * 192 + (size_t)b * 16 + 8 * (t & 1));
        d = ldw16(row + (size_t)nblk * 208 + (size_t)b * 2);
    }
    // From a row of a ring stage: ql[128] | qh[64] | scales[16]; `dword` = the stage's word that holds d.
    __device__ __forceinline__ void load_staged(const uint8_t *r, uint32_t dword, int t) {
        const int n = t >> 1, lh = t & 1;
        q0 = *reinterpret_cast<const uint4 *>(r + 64 * n + 16 * lh);
        q1 = *reinterpret_cast<const uint4 *>(r + 64 * n + 16 * lh + 32);
        qh = *reinterpret_cast<const uint4 *>(r + 128 + 32 * n + 16 * lh);
        sc = *reinterpret_cast<const uint2 *>(r + 192 + 8 * (t & 1));
        d = dword;
    }
};

// The prepared activations of one row that one thread needs for one superblock.
//   Q4_K: xb[0] / xb[1] = the 16 activation bytes under this thread's low / high nibbles of the chunk it
//         feeds (values 64 c + 16 (t % 2) + [0, 16), + 32), sx = sums of sub-blocks 4u .. 4u+3.
//   Q6_K: xb[i] = the 16 bytes under its run of 32-group i, sx = byte sums of 16-groups 8u .. 8u+7.
template <int FMT> struct Act {
    uint4 xb[is_k45<FMT> ? 2 : 4];
    uint4 sx;
    float inv;
    __device__ __forceinline__ void load(const uint8_t *tok, const PrepI8 &L, uint32_t b, int t, int g) { load_at<false>(tok, L, b, t, g); }
    // SH: `tok` is shared memory (plain loads), else global memory written by the kernel before.
    template <bool SH> __device__ __forceinline__ void load_at(const uint8_t *tok, const PrepI8 &L, uint32_t b, int t, int g) {
        auto ld128 = [](const uint8_t *p) { return SH ? *reinterpret_cast<const uint4 *>(p) : ldx128(p); };
        auto ld32 = [](const uint8_t *p) { return SH ? *reinterpret_cast<const uint32_t *>(p) : ldx32(p); };
        const int plane = g >> 2, u = t & 1;
        if constexpr (is_k45<FMT>) {
            const bool feeds = (t >> 1) == (g & 1);
            const int chunk = (((g & 3) >> 1) ? 2 : 0) + (t >> 1);
            const uint8_t *src = tok + (plane ? L.lo_off : 0) + (size_t)b * 256 + 64 * chunk + 16 * (t & 1);
#pragma unroll
            for (int i = 0; i < 2; i++) xb[i] = feeds ? ld128(src + 32 * i) : make_uint4(0, 0, 0, 0);
            sx = ld128(tok + L.sx32_off + (size_t)b * 32 + 16 * u);
        } else {
            const bool feeds = (g & 3) == t;
            const uint8_t *src = tok + (plane ? L.lo_off : 0) + (size_t)b * 256 + 128 * (t >> 1) + 16 * (t & 1);
#pragma unroll
            for (int i = 0; i < 4; i++) xb[i] = feeds ? ld128(src + 32 * i) : make_uint4(0, 0, 0, 0);
            sx = ld128(tok + L.sx16_off + ((t >> 1) ? (L.cols / 16) * 2 : 0) + (size_t)b * 32 + 16 * u);
        }
        inv = __uint_as_float(ld32(tok + L.isc_off + (size_t)b * 4));
    }
};

// One superblock of a 16-row tile against MT prepared activation rows: adds into yacc[m][r] this thread's
// share (its scale groups and plane) of rows g and g + 8.
template <int FMT, int MT, typename RawT>
__device__ __forceinline__ void superblock_dot(const RawT (&cur)[2], const Act<FMT> (&acur)[MT], int t, int g, float (&yacc)[MT][2]) {
    // This thread feeds column g of B (scale group g & 3, plane g >> 2) on its own k slots only, and
    // only if those k slots belong to that scale group; everything else it feeds is zero.
    //   Q6_K: group j = the k slots of quad thread j.
    //   Q4_K: group j = chunk j; thread t holds chunk t / 2 in its first operand word (k slots 4t ..)
    //         and chunk 2 + t / 2 in its second (k slots 16 + 4t ..).
    const bool second = is_k45<FMT> && ((g & 3) >> 1); // Q4_K / Q5_K: the group sits in the second operand word
    // It reads columns 2t, 2t+1 of the accumulators: scale groups 2 (t & 1), 2 (t & 1) + 1, plane t >> 1.
    const int u = t & 1;
    const float plane_weight = (t >> 1) ? 1.f : 256.f;
    (void)second;
    (void)u;
    if constexpr (is_k45<FMT>) {
        // The four scales and minimums of sub-blocks 4u .. 4u+3, one per byte.
        uint32_t sc4[2], mn4[2];
        float dsc[2], dmn[2];
#pragma unroll
        for (int r = 0; r < 2; r++) {
            const uint4 h = cur[r].hdr;
            sc4[r] = u ? ((h.w & 0x0F0F0F0Fu) | ((h.y >> 2) & 0x30303030u)) : (h.y & 0x3F3F3F3Fu);
            mn4[r] = u ? (((h.w >> 4) & 0x0F0F0F0Fu) | ((h.z >> 2) & 0x30303030u)) : (h.z & 0x3F3F3F3Fu);
            dsc[r] = f16_bits_to_f32((uint16_t)(h.x & 0xFFFFu)) * plane_weight;
            dmn[r] = (t >> 1) ? 0.f : f16_bits_to_f32((uint16_t)(h.x >> 16)); // minimum term once per plane pair
        }
        // u8 operands: low nibbles (even sub-block of the chunk) and high nibbles (odd sub-block); words
        // 0..3 from the first chunk, 4..7 from the second.
        uint32_t lo[2][8], hi[2][8];
#pragma unroll
        for (int r = 0; r < 2; r++)
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const uint32_t wd = word_of(i < 4 ? cur[r].qa : cur[r].qb, i & 3);
                lo[r][i] = wd & 0x0F0F0F0Fu;
                hi[r][i] = (wd >> 4) & 0x0F0F0F0Fu;
                if constexpr (FMT == FQ_Q5_K) {
                    // The fifth bits: qa is chunk t / 2 (sub-blocks 2 (t / 2), + 1), qb chunk 2 + t / 2 (four bits on).
                    const uint32_t v = word_of(cur[r].qh, i & 3) >> (2 * (t >> 1) + (i < 4 ? 0 : 4));
                    lo[r][i] |= (v << 4) & 0x10101010u;
                    hi[r][i] |= (v << 3) & 0x10101010u;
                }
            }
#pragma unroll
        for (int m = 0; m < MT; m++) {
            int cl[4] = {0, 0, 0, 0}, ch[4] = {0, 0, 0, 0};
#pragma unroll
            for (int i = 0; i < 4; i++) { // word i of either chunk <-> activation bytes 4i .. 4i+3 of the run
                const uint32_t xl = word_of(acur[m].xb[0], i), xh = word_of(acur[m].xb[1], i);
                mma_u8s8(cl, lo[0][i], lo[1][i], lo[0][4 + i], lo[1][4 + i], second ? 0u : xl, second ? xl : 0u);
                mma_u8s8(ch, hi[0][i], hi[1][i], hi[0][4 + i], hi[1][4 + i], second ? 0u : xh, second ? xh : 0u);
            }
            // Columns 2t, 2t+1 = scale groups 2u, 2u+1: sub-blocks 4u (low), 4u+1 (high), 4u+2, 4u+3.
#pragma unroll
            for (int r = 0; r < 2; r++) {
                const int dot = byte_u(sc4[r], 0) * cl[2 * r] + byte_u(sc4[r], 1) * ch[2 * r] + byte_u(sc4[r], 2) * cl[2 * r + 1] +
                                byte_u(sc4[r], 3) * ch[2 * r + 1];
                const uint4 &sx = acur[m].sx;
                const int mins = byte_u(mn4[r], 0) * (int)sx.x + byte_u(mn4[r], 1) * (int)sx.y +
                                 byte_u(mn4[r], 2) * (int)sx.z + byte_u(mn4[r], 3) * (int)sx.w;
                yacc[m][r] = fmaf(acur[m].inv, dsc[r] * (float)dot - dmn[r] * (float)mins, yacc[m][r]);
            }
        }
    } else {
        // Q6_K: thread t = (n, lh) owns, for i = 0..3, the values 128 n + 32 i + 16 lh + [0, 16).
        uint32_t v4[2][4][4]; // [row][i][word]: four 6-bit quants, one per byte
#pragma unroll
        for (int r = 0; r < 2; r++)
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int wi = 0; wi < 4; wi++) {
                    const uint32_t lw = word_of((i & 1) ? cur[r].q1 : cur[r].q0, wi), hw = word_of(cur[r].qh, wi);
                    const uint32_t lo4 = (i < 2) ? lw : (lw >> 4);
                    const uint32_t hi4 = i == 0 ? (hw << 4) : i == 1 ? (hw << 2) : i == 2 ? hw : (hw >> 2);
                    v4[r][i][wi] = lop3_select(lo4, hi4, 0x0F0F0F0Fu) & 0x3F3F3F3Fu;
                }
        float dd[2];
#pragma unroll
        for (int r = 0; r < 2; r++) dd[r] = f16_bits_to_f32((uint16_t)cur[r].d) * plane_weight;
#pragma unroll
        for (int m = 0; m < MT; m++) {
            int dot[2] = {0, 0};
#pragma unroll
            for (int i = 0; i < 4; i++) {
                int c[4] = {0, 0, 0, 0};
                const uint4 &xv = acur[m].xb[i];
                mma_u8s8(c, v4[0][i][0], v4[1][i][0], v4[0][i][1], v4[1][i][1], xv.x, xv.y);
                mma_u8s8(c, v4[0][i][2], v4[1][i][2], v4[0][i][3], v4[1][i][3], xv.z, xv.w);
                // Columns 2t, 2t+1 = quad threads 2u, 2u+1 = (half u, runs 0 and 1): 16-groups
                // 8u + 2i and 8u + 2i + 1.  (q - 32) is applied as  dot - 32 * sum(x bytes).
                const uint32_t spair = word_of(acur[m].sx, i);
                const int s0 = (int)(int16_t)(spair & 0xFFFFu), s1 = (int)(int16_t)(spair >> 16);
#pragma unroll
                for (int r = 0; r < 2; r++) {
                    const uint32_t scw = (i < 2) ? cur[r].sc.x : cur[r].sc.y;
                    dot[r] += byte_s(scw, 2 * (i & 1)) * (c[2 * r] - 32 * s0) + byte_s(scw, 2 * (i & 1) + 1) * (c[2 * r + 1] - 32 * s1);
                }
            }
#pragma unroll
            for (int r = 0; r < 2; r++) yacc[m][r] = fmaf(acur[m].inv * dd[r], (float)dot[r], yacc[m][r]);
        }
    }
}

struct GemvTargets {
    const uint8_t *w[MAX_TARGETS];
    float *y[MAX_TARGETS];
    uint32_t rows[MAX_TARGETS];
    uint32_t tile_end[MAX_TARGETS];
    uint32_t count;
};

// FMT: FQ_Q4_K / FQ_Q6_K; MT: activation rows (1..4).  grid.x = persistent blocks over the 16-row tiles of all targets;
// grid.y = routes in expert mode (route r: expert ids[r], activation row r / x_div, output row r).
// INP (routes, one activation row): the block prepares its route's activation row itself into shared memory from
// `xin` (and `xup`: the gated unit), so no preparation launch precedes the kernel; else `prep` holds prepared rows.
template <int FMT, int MT, bool INP = false>
__global__ void __launch_bounds__(MT >= 3 ? 256 : MT == 2 ? 384 : MAX_WARPS * 32)
k_gemv_i8(const __grid_constant__ GemvTargets T, uint32_t pitch, const uint8_t *__restrict__ prep, PrepI8 L,
          const uint32_t *__restrict__ ids, uint32_t x_div, uint32_t experts, const __grid_constant__ TpPush P,
          const float *__restrict__ xin, const float *__restrict__ xup, const __grid_constant__ CombineTail C,
          const uint32_t *__restrict__ route_map, uint32_t id_base, bool map_x) {
    using Raw = typename RawOf<FMT>::type;
    static_assert(!INP || MT == 1, "in-kernel preparation serves one activation row per route");
    extern __shared__ __align__(16) uint8_t own_act[]; // INP: the route's prepared row
    __shared__ float red[2][MAX_WARPS - 1][MT * 2][8];
    const int WARPS = blockDim.x >> 5;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;

    // Blocks are persistent: block b takes the 16-row tiles b, b + gridDim.x, ... of the launch (all targets
    // counted through), so that a block's set-up is paid once and the weight stream of its next tile is
    // already in flight while the current one is reduced and stored.
    const uint32_t total_tiles = T.tile_end[T.count - 1];
    size_t expert_off = 0, y_base = 0;
    uint32_t x_row = 0; // the route's activation row
    if (ids) {
        pdl_wait(); // the routing that wrote `ids` (and the map) must have completed
        const uint32_t r = blockIdx.y, src = route_map ? route_map[r] : r;
        const uint32_t e = ids[src] - id_base; // wraps to a value no matrix has when the expert is below id_base
        if (e >= experts) return;
        expert_off = (size_t)e * T.rows[0] * pitch;
        x_row = (map_x ? src : r) / x_div;
        if constexpr (!INP) prep += (size_t)x_row * L.token_bytes;
        y_base = (size_t)r * T.rows[0];
    }
    struct Tile {
        const uint8_t *rowp[2];
        float *y;
        uint32_t rows, tile0;
    };
    auto tile_at = [&](uint32_t tile) {
        uint32_t which = 0, first_block = 0;
#pragma unroll
        for (int i = 0; i < MAX_TARGETS - 1; i++)
            if ((uint32_t)i + 1 < T.count && tile >= T.tile_end[i]) { which = i + 1; first_block = T.tile_end[i]; }
        Tile q;
        q.rows = T.rows[which];
        q.tile0 = tile - first_block;
        q.y = T.y[which];
        const uint8_t *w = T.w[which] + expert_off;
#pragma unroll
        for (int r = 0; r < 2; r++) q.rowp[r] = w + (size_t)min(q.tile0 * 16 + g + r * 8, q.rows - 1) * pitch;
        return q;
    };
    uint32_t tile = blockIdx.x;
    Tile here = tile_at(tile);

    const uint32_t nblk = L.nblk;
    const uint32_t iters = nblk > (uint32_t)warp ? (nblk - warp + WARPS - 1) / WARPS : 0;
    auto block_of = [&](uint32_t it) { return warp + min(it, iters - 1) * WARPS; };
    Raw cur[2], nxt[2];
    if (iters > 0) {
        cur[0].load(here.rowp[0], nblk, block_of(0), t);
        cur[1].load(here.rowp[1], nblk, block_of(0), t);
    }
    // The loads above touch immutable weights only; the rest reads prepared activations and writes y.
    pdl_trigger();
    pdl_wait();
    const uint32_t seq = P.world > 1 ? tp_seq(P) : 0u;
    if constexpr (INP) {
        const size_t xr = (size_t)x_row * L.cols;
        for (uint32_t b = warp; b < nblk; b += WARPS) prep_superblock(xin + xr, b, b, lane, L, own_act, xup ? xup + xr : nullptr, nullptr, 0.f);
        __syncthreads();
        prep = own_act;
    }

    // With one activation row its fragments are fetched one superblock ahead, like the weights; with
    // more rows the registers do not allow that and they are fetched at the top of the iteration.
    constexpr bool AHEAD = MT == 1;
    Act<FMT> acur[MT], anxt[MT]; // anxt is used with AHEAD only
    if (AHEAD && iters > 0) {
#pragma unroll
        for (int m = 0; m < MT; m++) acur[m].template load_at<INP>(prep + (size_t)m * L.token_bytes, L, block_of(0), t, g);
    }

    float yacc[MT][2];
#pragma unroll
    for (int m = 0; m < MT; m++) yacc[m][0] = yacc[m][1] = 0.f;

    for (uint32_t buf = 0;; buf ^= 1u) {
    const uint32_t next_tile = tile + gridDim.x;
    const bool more = next_tile < total_tiles;
    const Tile next = more ? tile_at(next_tile) : here;
    // One superblock: everything the next one needs is requested first (after a tile's last superblock that is
    // the first superblock of the block's next tile), then this one runs from registers.
    auto step = [&](const Raw (&c)[2], Raw (&n)[2], Act<FMT> (&ac)[MT], Act<FMT> (&an)[MT], uint32_t it) {
        const bool wrap = it + 1 == iters && more;
        const uint32_t nb_next = wrap ? block_of(0) : block_of(it + 1);
        n[0].load(wrap ? next.rowp[0] : here.rowp[0], nblk, nb_next, t);
        n[1].load(wrap ? next.rowp[1] : here.rowp[1], nblk, nb_next, t);
#pragma unroll
        for (int m = 0; m < MT; m++) {
            if (AHEAD) an[m].template load_at<INP>(prep + (size_t)m * L.token_bytes, L, nb_next, t, g);
            else ac[m].template load_at<INP>(prep + (size_t)m * L.token_bytes, L, block_of(it), t, g);
        }
        superblock_dot<FMT, MT>(c, ac, t, g, yacc);
    };
    if (is_k45<FMT> && (iters & 1u) == 0) {
        // An even count: the two register sets swap roles instead of being copied (Q4_K only: with Q6_K's larger
        // register sets the second copy of the loop body spills).
        for (uint32_t it = 0; it < iters; it += 2) {
            step(cur, nxt, acur, anxt, it);
            if (AHEAD) step(nxt, cur, anxt, acur, it + 1);
            else step(nxt, cur, acur, anxt, it + 1);
        }
    } else {
        for (uint32_t it = 0; it < iters; it++) {
            step(cur, nxt, acur, anxt, it);
            cur[0] = nxt[0];
            cur[1] = nxt[1];
            if (AHEAD) {
#pragma unroll
                for (int m = 0; m < MT; m++) acur[m] = anxt[m];
            }
        }
    }
    // Quad threads hold partial sums of different scale groups and planes: add them, then the warps.
#pragma unroll
    for (int m = 0; m < MT; m++)
#pragma unroll
        for (int r = 0; r < 2; r++) {
            yacc[m][r] += __shfl_xor_sync(0xffffffffu, yacc[m][r], 1);
            yacc[m][r] += __shfl_xor_sync(0xffffffffu, yacc[m][r], 2);
        }
    if (warp > 0 && t == 0) {
#pragma unroll
        for (int m = 0; m < MT; m++) {
            red[buf][warp - 1][m * 2][g] = yacc[m][0];
            red[buf][warp - 1][m * 2 + 1][g] = yacc[m][1];
        }
    }
    __syncthreads(); // one barrier per tile: the two halves of `red` alternate
    if (warp == 0 && t == 0) {
#pragma unroll
        for (int m = 0; m < MT; m++)
#pragma unroll
            for (int r = 0; r < 2; r++) {
                float v = yacc[m][r];
#pragma unroll
                for (int ww = 0; ww < WARPS - 1; ww++) v += red[buf][ww][m * 2 + r][g];
                const uint32_t row = here.tile0 * 16 + g + r * 8;
                if (row < here.rows) {
                    float *dst = &here.y[y_base + (size_t)m * here.rows + row];
                    *dst = v;
                    if (P.world > 1) tp_store(P, seq, dst, v);
                }
            }
    }
    if (C.counters && warp == 0) {
        // The weighted sum over a token's routes (and the shared expert) for this tile's rows, by the last of the
        // token's route blocks to get here: in route order, so the result does not depend on which block that is.
        __threadfence();
        __syncwarp();
        const uint32_t token = blockIdx.y / C.used;
        uint32_t *counter = C.counters + (size_t)token * total_tiles + here.tile0;
        uint32_t last = 0;
        if (lane == 0) last = atomicAdd(counter, 1u) + 1 == C.used;
        last = __shfl_sync(0xffffffffu, last, 0);
        if (last) {
            if (lane == 0) *counter = 0;
            __threadfence();
            const uint32_t row = here.tile0 * 16 + lane;
            if (lane < 16 && row < here.rows) {
                float acc = 0.f;
                for (uint32_t s2 = 0; s2 < C.used; s2++) {
                    const uint32_t r = token * C.used + s2;
                    acc = fmaf(C.weights[r], __ldcg(&here.y[(size_t)r * here.rows + row]), acc);
                }
                C.out[(size_t)token * here.rows + row] = fmaf(C.gate[token], C.shared[(size_t)token * here.rows + row], acc);
            }
        }
    }
    if (!more) break;
    tile = next_tile;
    here = next;
#pragma unroll
    for (int m = 0; m < MT; m++) yacc[m][0] = yacc[m][1] = 0.f;
    }
    if (P.world > 1) tp_finish(P, seq);
}

// ---------------------------------------------------------------- one activation row, K slices and weight rings
//
// The same arithmetic (superblock_dot) organised for latency and balance: a block of 16 warps quantises ONE K
// slice of the activation row into shared memory itself (no preparation launch: one dependency less between a
// projection and the kernel that produced its input), every warp then takes 16-row tiles against it, streaming
// their packed superblocks through a private ring of asynchronous copies (gemv_common.cuh) -- no block-wide
// barrier in the main loop, the ring running on across tile borders.  K is cut into as many slices as it takes
// for every SM to get its share of warps when rows are few (the 5120 x 17408 down projection: 320 tiles); with
// more than one slice the partial sums go to a workspace and the last warp to arrive at a tile adds them in
// slice order (deterministic).
template <int FMT> struct Stage1; // bytes between the rows of a stage, chosen for the 16-byte fragment reads
template <> struct Stage1<FQ_Q4_K> { static constexpr uint32_t ROW = 192; };
template <> struct Stage1<FQ_Q5_K> { static constexpr uint32_t ROW = 176; };
template <> struct Stage1<FQ_Q6_K> { static constexpr uint32_t ROW = 224; };

struct SlicedJob {
    GemvTargets T;         // tile_end in 16-row tiles
    uint32_t pitch, cols, nblk;
    const float *x, *x_up, *norm_w;
    float norm_eps;
    uint32_t slices, nb_max;
    float *ws;             // partial sums [tile][slice][16 rows]
    uint32_t *counters;    // arrivals per tile
};

template <int FMT, int STAGES>
__global__ void __launch_bounds__(512, 1)
k_gemv_i8s(const __grid_constant__ SlicedJob J, const __grid_constant__ TpPush P) {
    using Raw = typename RawOf<FMT>::type;
    using Ring = WeightRing<FMT, Stage1<FMT>::ROW>;
    constexpr uint32_t ROW = Stage1<FMT>::ROW;
    extern __shared__ __align__(128) uint8_t s1_smem[];
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5, W = blockDim.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const uint32_t slice = blockIdx.x % J.slices;
    const uint32_t b0 = (uint32_t)((uint64_t)slice * J.nblk / J.slices), nb = (uint32_t)((uint64_t)(slice + 1) * J.nblk / J.slices) - b0;
    // Tiles are dealt out across the blocks of a slice first, then across their warps: when there are fewer tiles
    // than warps the idle warps are spread over all SMs instead of leaving whole SMs without work.
    const uint32_t first = warp * (gridDim.x / J.slices) + blockIdx.x / J.slices, stride = (gridDim.x / J.slices) * W;
    const uint32_t total_tiles = J.T.tile_end[J.T.count - 1];
    const PrepI8 L = prep_i8_layout(J.nb_max * 256); // the slice's activations, laid out like a short row
    uint8_t *act = s1_smem, *ring = s1_smem + L.token_bytes + (size_t)warp * STAGES * Ring::BYTES;

    struct Tile {
        const uint8_t *w;
        float *y;
        uint32_t rows, row0;
    };
    auto tile_at = [&](uint32_t tile) {
        uint32_t which = 0, first_tile = 0;
#pragma unroll
        for (int i = 0; i < MAX_TARGETS - 1; i++)
            if ((uint32_t)i + 1 < J.T.count && tile >= J.T.tile_end[i]) { which = i + 1; first_tile = J.T.tile_end[i]; }
        Tile q;
        q.rows = J.T.rows[which];
        q.row0 = (tile - first_tile) * 16;
        q.w = J.T.w[which];
        q.y = J.T.y[which];
        return q;
    };
    // Producer side of the warp's ring: item = (tile, superblock of the slice), in the order they are consumed.
    Ring wr;
    uint32_t p_tile = first, p_bb = 0, p_stage = 0;
    auto start_tile = [&](uint32_t tile) {
        const Tile q = tile_at(tile);
        wr.start_tile(q.w + (size_t)q.row0 * J.pitch, q.rows - 1 - q.row0, J.pitch, J.nblk, lane);
    };
    if (p_tile < total_tiles) start_tile(p_tile);
    auto issue = [&]() {
        if (p_tile < total_tiles) {
            wr.issue(ring + (size_t)p_stage * Ring::BYTES, b0 + p_bb, lane);
            if (++p_bb == nb) {
                p_bb = 0;
                p_tile += stride;
                if (p_tile < total_tiles) start_tile(p_tile);
            }
        }
        cp_async_commit();
        p_stage = p_stage + 1 == STAGES ? 0 : p_stage + 1;
    };
#pragma unroll
    for (int i = 0; i < STAGES - 1; i++) issue();
    // The copies above read immutable weights only; the rest reads activations and writes y.
    pdl_trigger();
    pdl_wait();
    const uint32_t seq = P.world > 1 ? tp_seq(P) : 0u;
    {
        const float scale = J.norm_w ? row_inv_rms(J.x, J.cols, J.norm_eps, lane) : 0.f;
        // A warp's superblocks two at a time, both fetched before either is worked on (the fetch is an L2 round
        // trip; the widest slice of the 27B layer set gives a warp two superblocks).
        for (uint32_t bb = warp; bb < nb; bb += 2 * W) {
            PrepLoad in0, in1;
            const bool two = bb + W < nb;
            in0.fetch(J.x, b0 + bb, lane);
            if (two) in1.fetch(J.x, b0 + bb + W, lane);
            prep_superblock(in0, b0 + bb, bb, lane, L, act, J.x_up, J.norm_w, scale);
            if (two) prep_superblock(in1, b0 + bb + W, bb + W, lane, L, act, J.x_up, J.norm_w, scale);
        }
    }
    __syncthreads();

    uint32_t c_stage = 0;
    for (uint32_t tile = first; tile < total_tiles; tile += stride) {
        const Tile here = tile_at(tile);
        float yacc[1][2] = {{0.f, 0.f}};
        for (uint32_t bb = 0; bb < nb; bb++) {
            issue();
            cp_async_wait<STAGES - 1>();
            __syncwarp();
            const uint8_t *stage = ring + (size_t)c_stage * Ring::BYTES;
            Raw cur[2];
            Act<FMT> a[1];
#pragma unroll
            for (int r = 0; r < 2; r++) {
                uint32_t dword = 0;
                if constexpr (FMT == FQ_Q6_K) {
                    dword = *reinterpret_cast<const uint32_t *>(stage + 16 * ROW + 4 * (g + 8 * r));
                    dword = ((b0 + bb) & 1u) ? dword >> 16 : dword & 0xFFFFu;
                }
                cur[r].load_staged(stage + (g + 8 * r) * ROW, dword, t);
            }
            a[0].template load_at<true>(act, L, bb, t, g);
            superblock_dot<FMT, 1>(cur, a, t, g, yacc);
            __syncwarp();
            c_stage = c_stage + 1 == STAGES ? 0 : c_stage + 1;
        }
        // Quad threads hold partial sums of different scale groups and planes.
        float v[2];
#pragma unroll
        for (int r = 0; r < 2; r++) {
            v[r] = yacc[0][r];
            v[r] += __shfl_xor_sync(0xffffffffu, v[r], 1);
            v[r] += __shfl_xor_sync(0xffffffffu, v[r], 2);
        }
        bool store = true;
        if (J.slices > 1) {
            float *part = J.ws + (size_t)tile * J.slices * 16;
            if (t == 0) {
                part[slice * 16 + g] = v[0];
                part[slice * 16 + g + 8] = v[1];
            }
            __threadfence();
            __syncwarp();
            uint32_t arrived = 0;
            if (lane == 0) arrived = atomicAdd(J.counters + tile, 1u);
            arrived = __shfl_sync(0xffffffffu, arrived, 0);
            store = arrived + 1 == J.slices;
            if (store) {
                __threadfence();
                if (lane == 0) J.counters[tile] = 0;
                v[0] = v[1] = 0.f;
                if (t == 0)
                    for (uint32_t s = 0; s < J.slices; s++) {
                        v[0] += __ldcg(&part[s * 16 + g]);
                        v[1] += __ldcg(&part[s * 16 + g + 8]);
                    }
            }
        }
        if (store && t == 0) {
#pragma unroll
            for (int r = 0; r < 2; r++) {
                const uint32_t row = here.row0 + g + r * 8;
                if (row < here.rows) {
                    float *dst = &here.y[row];
                    *dst = v[r];
                    if (P.world > 1) tp_store(P, seq, dst, v[r]);
                }
            }
        }
    }
    cp_async_wait<0>();
    if (P.world > 1) tp_finish(P, seq);
}

// One activation row, no routes.  cudaErrorNotSupported when the shape does not fit this kernel.
template <int FMT> cudaError_t launch_sliced(fq_device *dev, const ProjectArgs *a, uint32_t count) {
    using Ring = WeightRing<FMT, Stage1<FMT>::ROW>;
    // 16 warps in one block per SM and a ring of two stages (one superblock in flight per warp beside the one
    // being used): deeper rings and smaller blocks measured slower on every shape of the 27B layer set.
    constexpr uint32_t SMEM_MAX = 222 * 1024, WARPS = 16, STAGES = 2;
    SlicedJob J{};
    J.T.count = count;
    uint32_t tiles = 0;
    for (uint32_t i = 0; i < count; i++) {
        J.T.w[i] = a[i].w;
        J.T.y[i] = (float *)a[i].y;
        J.T.rows[i] = a[i].rows;
        tiles += (a[i].rows + 15) / 16;
        J.T.tile_end[i] = tiles;
    }
    J.pitch = a[0].row_bytes;
    J.cols = a[0].cols;
    J.nblk = a[0].cols / 256;
    J.x = (const float *)a[0].x;
    J.x_up = a[0].x_up;
    J.norm_w = a[0].norm_w;
    J.norm_eps = a[0].norm_eps;
    // Slices: estimated time in units of one superblock of one tile = rounds of tiles per warp x (superblocks per
    // slice + a fixed cost per run, larger when partial sums are exchanged) + the block's preparation of its slice.
    const uint32_t sms = (uint32_t)dev->sm_count, nblk = J.nblk;
    double best = 1e30;
    uint32_t slices = 1;
    for (uint32_t s = 1; s <= std::min(nblk, sms); s++) {
        const uint32_t per_slice = (sms / s) * WARPS, nbm = (nblk + s - 1) / s, rounds = (tiles + per_slice - 1) / per_slice;
        const double cost = rounds * (nbm + (s > 1 ? 1.0 : 0.3)) + 1.3 * ((nbm + WARPS - 1) / WARPS);
        if (cost < best - 1e-9) { best = cost; slices = s; }
    }
    J.slices = slices;
    J.nb_max = (nblk + slices - 1) / slices;
    const size_t act = prep_i8_layout(J.nb_max * 256).token_bytes;
    const size_t smem = act + (size_t)WARPS * STAGES * Ring::BYTES;
    if (smem > SMEM_MAX) return cudaErrorNotSupported;
    J.ws = (float *)dev->nt_ws;
    J.counters = dev->nt_counters;
    if (slices > 1 && ((size_t)tiles * slices * 16 * sizeof(float) > dev->nt_ws_bytes || tiles > dev->nt_counter_count)) return cudaErrorNotSupported;
    auto kernel = k_gemv_i8s<FMT, STAGES>;
    static bool configured = false;
    if (!configured) {
        const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_MAX);
        if (e != cudaSuccess) return e;
        configured = true;
    }
    TpPush push{};
    if (dev->tp_push) { // one launch covers every target: it can do the exchange itself
        push = *dev->tp_push;
        dev->tp_push = nullptr;
        dev->tp_pushed = true;
    }
    // Blocks per slice: every SM's share, unless the tiles fill fewer than half of their warps -- a small matrix
    // then takes only the blocks it can use and leaves the other SMs to whatever runs beside it (a block of this
    // kernel takes an SM's whole register file: the shared expert of an MoE block beside the routed chain).
    uint32_t per = std::max(1u, sms / slices);
    const uint32_t need = (tiles + WARPS - 1) / WARPS;
    if (need * 2 <= per) per = need;
    return launch_pdl(kernel, dim3(per * slices), dim3(WARPS * 32), smem, dev->stream, J, push);
}

template <int FMT, int MT, bool INP = false>
cudaError_t launch(fq_device *dev, const ProjectArgs *a, uint32_t count, const uint8_t *prep, const PrepI8 &L, bool expert) {
    GemvTargets T{};
    T.count = count;
    uint32_t blocks = 0;
    for (uint32_t i = 0; i < count; i++) {
        T.w[i] = a[i].w;
        T.y[i] = (float *)a[i].y;
        T.rows[i] = a[i].rows;
        blocks += (a[i].rows + 15) / 16;
        T.tile_end[i] = blocks;
    }
    dim3 grid(blocks, expert ? a[0].m : 1);
    // Warps per block = ways K is split: enough warps in the grid to keep every SM's schedulers and
    // memory pipeline busy (about 32 per SM), at least two superblocks per warp, and among the counts
    // that satisfy this the one that wastes the fewest warp-iterations on an uneven split.
    const uint32_t nblk = L.nblk, want = (uint32_t)dev->sm_count * 32u;
    const uint32_t reg_cap = MT >= 3 ? 8u : MT == 2 ? 12u : (uint32_t)MAX_WARPS; // wider variants need more registers per thread
    const uint32_t max_k = std::max(1u, std::min(reg_cap, nblk / 2));
    const uint32_t need = std::min(max_k, std::max(1u, (uint32_t)((want + (uint64_t)blocks * grid.y - 1) / ((uint64_t)blocks * grid.y))));
    uint32_t warps = need;
    uint64_t best = ~0ull;
    for (uint32_t k = need; k <= max_k; k++) {
        // prefer small k on ties, and an even count per warp (its register sets then swap instead of being copied)
        const uint64_t per = (nblk + k - 1) / k, waste = (per * k - nblk) * 1000 / nblk + (k - need) + ((per & 1) && nblk % k == 0 ? 2 : 0);
        if (waste < best) { best = waste; warps = k; }
    }
    // Persistent blocks: as many as stay resident at once (fewer with routes in grid.y), each walking its tiles.
    static int occupancy[MAX_WARPS + 1] = {};
    if (!occupancy[warps]) {
        int occ = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, k_gemv_i8<FMT, MT, INP>, (int)warps * 32, INP ? L.token_bytes : 0) != cudaSuccess || occ < 1) occ = 1;
        occupancy[warps] = occ;
    }
    const uint32_t resident = (uint32_t)dev->sm_count * (uint32_t)occupancy[warps];
    grid.x = std::min(blocks, std::max(1u, resident / grid.y));
    TpPush push{};
    if (dev->tp_push && !expert) { // one launch covers every target: it can do the exchange itself
        push = *dev->tp_push;
        dev->tp_push = nullptr;
        dev->tp_pushed = true;
    }
    CombineTail tail{};
    if (expert && a[0].combine) tail = *a[0].combine;
    return launch_pdl(k_gemv_i8<FMT, MT, INP>, grid, dim3(warps * 32), INP ? L.token_bytes : 0, dev->stream, T, a[0].row_bytes, prep, L, a[0].ids,
                      a[0].x_div, a[0].experts, push, (const float *)a[0].x, a[0].x_up, tail, a[0].route_map, a[0].id_base, a[0].map_x);
}

} // namespace

// `a[0..count)` share x, format and width; one activation row, or routes (expert mode: one activation row per route).
int fq_launch_gemv_i8_many(fq_device *dev, const ProjectArgs *a, uint32_t count) {
    if (count == 0 || count > (uint32_t)MAX_TARGETS) return FQ_ERR_UNSUPPORTED;
    const ProjectArgs &f = a[0];
    if ((f.format != FQ_Q4_K && f.format != FQ_Q5_K && f.format != FQ_Q6_K) || f.x_dtype != FQ_F32 || f.y_dtype != FQ_F32) return FQ_ERR_UNSUPPORTED;
    if (f.cols % 256 || f.row_bytes % 16) return FQ_ERR_UNSUPPORTED;
    for (uint32_t i = 1; i < count; i++)
        if (a[i].format != f.format || a[i].cols != f.cols || a[i].x != f.x || a[i].x_up != f.x_up || a[i].norm_w != f.norm_w || a[i].m != f.m || a[i].ids != f.ids ||
            a[i].x_div != f.x_div || a[i].experts != f.experts || (f.ids && a[i].rows != f.rows) || a[i].x_dtype != FQ_F32 ||
            a[i].y_dtype != FQ_F32 || a[i].route_map != f.route_map || a[i].id_base != f.id_base || a[i].map_x != f.map_x)
            return FQ_ERR_UNSUPPORTED; // with routes the targets are expert stacks of one shape (gate and up)
    const bool expert = f.ids != nullptr;
    if (!expert && (f.route_map || f.id_base)) return FQ_ERR_UNSUPPORTED;
    if (f.combine && (!expert || count != 1 || f.x_div != 1 || f.norm_w || prep_i8_layout(f.cols).token_bytes > 40 * 1024 ||
                      (size_t)(f.m / f.combine->used) * ((f.rows + 15) / 16) > FQ_COMBINE_COUNTERS))
        return FQ_ERR_UNSUPPORTED; // the caller combines with a kernel of its own
    uint32_t xrows, m;
    if (expert) {
        if (f.m > 65535) return FQ_ERR_UNSUPPORTED;
        xrows = f.m / f.x_div; // the caller checked that x holds routes / x_div rows
        m = 1;
    } else {
        if (f.m != 1) return FQ_ERR_UNSUPPORTED; // 2..16 activation rows: gemv_nt.cu
        xrows = m = f.m;
    }
    if (!expert) {
        const cudaError_t e = f.format == FQ_Q4_K ? launch_sliced<FQ_Q4_K>(dev, a, count)
                            : f.format == FQ_Q5_K ? launch_sliced<FQ_Q5_K>(dev, a, count) : launch_sliced<FQ_Q6_K>(dev, a, count);
        if (e != cudaErrorNotSupported) {
            if (int rc = fq_check_cuda(dev, e, "gemv launch")) return rc;
            return fq_end_enqueue(dev, "gemv_i8s", 1);
        }
    }
    const PrepI8 L = prep_i8_layout(f.cols);
    if (expert && !f.norm_w && L.token_bytes <= 40 * 1024) {
        // Routes: every block prepares its route's activation row itself (a few KB): one launch, one dependency less.
        cudaError_t e;
        if (f.format == FQ_Q4_K) e = launch<FQ_Q4_K, 1, true>(dev, a, count, nullptr, L, true);
        else if (f.format == FQ_Q5_K) e = launch<FQ_Q5_K, 1, true>(dev, a, count, nullptr, L, true);
        else e = launch<FQ_Q6_K, 1, true>(dev, a, count, nullptr, L, true);
        if (int rc = fq_check_cuda(dev, e, "gemv launch")) return rc;
        return fq_end_enqueue(dev, "gemv_i8", 1);
    }
    // Successive projections use alternate halves of the scratch, so a preparation kernel that starts
    // early never writes what the previous projection may still be reading from a cache.
    if ((size_t)xrows * L.token_bytes > dev->xprep_bytes / 2) return FQ_ERR_UNSUPPORTED;
    dev->xprep_turn ^= 1u;
    uint8_t *prep = (uint8_t *)dev->xprep + (dev->xprep_turn ? dev->xprep_bytes / 2 : 0);
    const uint32_t warps = xrows * L.nblk;
    if (int rc = fq_check_cuda(dev, launch_pdl(k_prep_i8, dim3((warps + 3) / 4), dim3(128), 0, dev->stream, (const float *)f.x, f.x_up, f.norm_w, f.norm_eps, xrows, L, prep),
                               "activation preparation launch"))
        return rc;
    cudaError_t e;
    if (f.format == FQ_Q4_K) e = launch<FQ_Q4_K, 1>(dev, a, count, prep, L, expert);
    else if (f.format == FQ_Q5_K) e = launch<FQ_Q5_K, 1>(dev, a, count, prep, L, expert);
    else e = launch<FQ_Q6_K, 1>(dev, a, count, prep, L, expert);
    if (int rc = fq_check_cuda(dev, e, "gemv launch")) return rc;
    return fq_end_enqueue(dev, "gemv_i8", 2);
}

// ---------------------------------------------------------------- allocation-free entry point
//
// `fq_gemv_q4k_static` is for callers that must not allocate device memory at all: code running
// inside a memory pool that has already handed every byte to the model, a plugin loaded into a
// process whose allocator is owned by someone else, or a call site between the begin and end of a
// phase in which cudaMalloc would serialise the device.  `fq_device_create` and `fq_matrix_create`
// both allocate, so this entry point takes neither handle: the caller passes device pointers to the
// packed Q4_K rows (GGUF bytes, 16-byte aligned), to the activations and to the output, plus a stream.
// The prepared activations, which the handle-based path keeps in scratch it allocated at creation,
// live here in a fixed array that is part of the library image.
constexpr size_t STATIC_SCRATCH_BYTES = FQ_STATIC_SCRATCH_BYTES;
static __device__ __align__(256) uint8_t g_static_scratch[STATIC_SCRATCH_BYTES];

namespace {

// Device address of g_static_scratch per device ordinal.  In host code the array's name is only a
// stand-in for the symbol; the address a kernel can use comes from cudaGetSymbolAddress, taken once
// per device with that device current.
// Published with release / read with acquire: a host thread that sees the address also sees the SM count
// stored before it, so two threads may make a device's first call at the same time.
constexpr int MAX_DEVICES = 64;
std::atomic<uint8_t *> g_static_ptr[MAX_DEVICES];
int g_static_sms[MAX_DEVICES];

int static_fail(char *err, size_t err_len, int status, const char *fmt, ...) {
    if (err && err_len) {
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(err, err_len, fmt, ap);
        va_end(ap);
    }
    return status;
}

template <int MT>
cudaError_t launch_static(const uint8_t *w, uint32_t rows, uint32_t pitch, float *y, const uint8_t *prep, const PrepI8 &L,
                          int sm_count, cudaStream_t stream) {
    GemvTargets T{};
    T.count = 1;
    T.w[0] = w;
    T.y[0] = y;
    T.rows[0] = rows;
    const uint32_t blocks = (rows + 15) / 16;
    T.tile_end[0] = blocks;
    // Same choice of warps per block as the handle-based path.
    const uint32_t nblk = L.nblk, want = (uint32_t)sm_count * 32u;
    const uint32_t reg_cap = MT >= 3 ? 8u : MT == 2 ? 12u : (uint32_t)MAX_WARPS;
    const uint32_t max_k = std::max(1u, std::min(reg_cap, nblk / 2));
    const uint32_t need = std::min(max_k, std::max(1u, (want + blocks - 1) / blocks));
    uint32_t warps = need;
    uint64_t best = ~0ull;
    for (uint32_t k = need; k <= max_k; k++) {
        const uint64_t per = (nblk + k - 1) / k, waste = (per * k - nblk) * 1000 / nblk + (k - need);
        if (waste < best) { best = waste; warps = k; }
    }
    k_gemv_i8<FQ_Q4_K, MT><<<dim3(blocks, 1), dim3(warps * 32), 0, stream>>>(T, pitch, prep, L, nullptr, 1u, 1u, TpPush{}, nullptr, nullptr, CombineTail{},
                                                                             nullptr, 0u, false);
    return cudaGetLastError();
}

} // namespace

extern "C" int fq_gemv_q4k_static(const void *w_packed, uint64_t rows, uint64_t cols, const float *x, uint32_t m, float *y,
                                  void *cuda_stream, char *err, size_t err_len) {
    if (!w_packed || !x || !y) return static_fail(err, err_len, FQ_ERR_RANGE, "null binding");
    if (((uintptr_t)w_packed | (uintptr_t)x | (uintptr_t)y) & 15u)
        return static_fail(err, err_len, FQ_ERR_RANGE, "bindings must be 16-byte aligned");
    if (rows == 0 || rows > 0x7fffffffull || cols == 0 || cols % 256 || cols > FQ_MAX_COLS)
        return static_fail(err, err_len, FQ_ERR_SHAPE, "Q4_K geometry %llu x %llu (cols must be a multiple of 256)",
                           (unsigned long long)rows, (unsigned long long)cols);
    if (m == 0 || m > (uint32_t)MAX_TOKENS)
        return static_fail(err, err_len, FQ_ERR_SHAPE, "%u activation rows; this entry point serves 1..%d", m, MAX_TOKENS);
    const PrepI8 L = prep_i8_layout((uint32_t)cols);
    if ((size_t)m * L.token_bytes > STATIC_SCRATCH_BYTES)
        return static_fail(err, err_len, FQ_ERR_SHAPE,
                           "%u rows of %llu activations need %zu bytes of prepared activations; the fixed scratch holds %zu",
                           m, (unsigned long long)cols, (size_t)m * L.token_bytes, STATIC_SCRATCH_BYTES);
    {
        // The three bindings must not overlap one another (the handle-based path checks the same).
        const uintptr_t wa = (uintptr_t)w_packed, wb = wa + (size_t)rows * (cols / 256 * 144), xa = (uintptr_t)x, xb = xa + (size_t)m * cols * 4,
                        ya = (uintptr_t)y, yb = ya + (size_t)m * rows * 4;
        if ((ya < xb && xa < yb) || (ya < wb && wa < yb)) return static_fail(err, err_len, FQ_ERR_ALIAS, "the output overlaps an input");
    }
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= MAX_DEVICES)
        return static_fail(err, err_len, FQ_ERR_DEVICE, "no current CUDA device: %s", cudaGetErrorString(e));
    uint8_t *prep = g_static_ptr[dev].load(std::memory_order_acquire);
    if (!prep) {
        // First call on this device: resolve the array's device address (and the SM count).
        uint8_t *p = nullptr;
        e = cudaGetSymbolAddress((void **)&p, g_static_scratch);
        if (e != cudaSuccess || !p)
            return static_fail(err, err_len, FQ_ERR_CUDA, "cudaGetSymbolAddress(static scratch): %s", cudaGetErrorString(e));
        int sms = 0;
        e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess || sms <= 0) return static_fail(err, err_len, FQ_ERR_CUDA, "SM count: %s", cudaGetErrorString(e));
        g_static_sms[dev] = sms;
        g_static_ptr[dev].store(p, std::memory_order_release);
        prep = p;
    }
    cudaStream_t stream = (cudaStream_t)cuda_stream;
    const uint32_t warps = m * L.nblk;
    cudaGetLastError(); // an error the caller left behind is not this call's
    // Every byte the GEMV reads from the scratch is rewritten here first, so nothing has to start at zero.
    k_prep_i8<<<(warps + 3) / 4, 128, 0, stream>>>(x, nullptr, nullptr, 0.f, m, L, prep);
    if ((e = cudaGetLastError()) != cudaSuccess)
        return static_fail(err, err_len, FQ_ERR_CUDA, "activation preparation launch: %s", cudaGetErrorString(e));
    const uint32_t pitch = (uint32_t)(cols / 256 * 144);
    const uint8_t *w = (const uint8_t *)w_packed;
    e = m == 1 ? launch_static<1>(w, (uint32_t)rows, pitch, y, prep, L, g_static_sms[dev], stream)
      : m == 2 ? launch_static<2>(w, (uint32_t)rows, pitch, y, prep, L, g_static_sms[dev], stream)
      : m == 3 ? launch_static<3>(w, (uint32_t)rows, pitch, y, prep, L, g_static_sms[dev], stream)
               : launch_static<4>(w, (uint32_t)rows, pitch, y, prep, L, g_static_sms[dev], stream);
    if (e != cudaSuccess) return static_fail(err, err_len, FQ_ERR_CUDA, "gemv launch: %s", cudaGetErrorString(e));
    return FQ_OK;
}
