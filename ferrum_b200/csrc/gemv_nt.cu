// Verify-width projections (2..16 activation rows) and grouped expert projections with few rows per expert,
// on the integer tensor path with the ACTIVATION ROWS ON THE MMA's N SIDE (F32 in, F32 out).  The reference's
// `h_mvb_*` / `h_mms_*` (src/metal/shaders/hybrid.metal:1330-1394, 1419-1495; dispatch
// src/hybrid/engine.rs:3438-3460) and, over expert-sorted rows, `h_mm_id_*` (hybrid.metal:2430-2523).
//
// Every packed weight is unpacked once and serves eight or sixteen activation rows:
//
//   A (16 weight rows x k)  Q4_K: one 32-value sub-block, raw nibbles as u8 (one AND per four weights, a shift
//                           more for the high nibbles); Q6_K: one 16-value scale group as s8 = 4 (q - 32)
//                           (two shifts and two LOP3 per four weights; the factor 4 goes into d);
//   B (k x 8 rows of x)     the activations as 16-bit integers x' = round(x * s) = 256 hi + lo, both halves
//                           signed bytes, s a power of two per (row, superblock): two MMAs (hi, lo) on the same A;
//   per scale group         acc_hi += scale * c_hi, acc_lo += scale * c_lo in integers (and, Q4_K, the minimums
//                           times the activation sums); once per superblock one conversion and FMA with d / s.
//
// The result is the exact dot product of the decoded weights with activations rounded to 16 bits relative to the
// largest magnitude of their superblock, as in gemv_i8.cu.
//
// Organisation: the activations are prepared once per projection by k_prep_nt (16-bit integers in the order the
// B fragments are read; optionally the row's rmsnorm, the gated unit of two inputs, or only the rows of the
// experts a rank owns).  A block keeps the prepared activations of ONE K slice (dense) or of one tile of up to 32
// expert-sorted rows (grouped: rows picked by index, so the expert-major gather costs nothing) resident in shared
// memory, copied there asynchronously, and its warps each take 16-row weight tiles against them.  A warp streams
// the packed superblocks of its tiles through a private ring in shared memory with 16-byte asynchronous copies
// (several superblocks in flight per warp, no registers held, no block-wide barrier in the main loop; the ring
// runs on across tile borders) and reads MMA fragments from there: thread (g = lane / 4, t = lane % 4) owns
// weight rows g, g + 8 and, since the k order inside a scale group is free, the bytes 8t.. (Q4_K) or 4t.. (Q6_K)
// of each run, so that shared-memory reads are conflict-free.  Dense launches cut K into as many slices as it
// takes for a slice of activations to fit and for every SM to get its share of warps; with more than one slice
// the partial sums go to a workspace and the last warp to arrive at a tile adds them in slice order
// (deterministic).  A grouped block runs the tile loop for 8, 16 or 32 live rows, chosen by the rows its tile holds.
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <type_traits>

#include "blocks.cuh"
#include "gemv_common.cuh"
#include "internal.h"

namespace {
using namespace fqk;

constexpr int NT_MAX_TARGETS = 4;
constexpr uint32_t NT_SMEM_MAX = 222 * 1024;

// A stage of a warp's ring: the packed bytes of one superblock of 16 weight rows.  ROW = bytes between rows in
// shared memory (Q4_K: 160, so that the 8-byte reads of rows g .. g + 3 fall on different banks).
template <int FMT> struct StageNT;
template <> struct StageNT<FQ_Q4_K> {
    static constexpr uint32_t ROW = 160, BYTES = WeightRing<FQ_Q4_K, 160>::BYTES;
};
template <> struct StageNT<FQ_Q5_K> {
    static constexpr uint32_t ROW = 176, BYTES = WeightRing<FQ_Q5_K, 176>::BYTES;
};
template <> struct StageNT<FQ_Q6_K> { // per row ql[128] | qh[64] | scales[16]; then 4 bytes per row holding d
    static constexpr uint32_t ROW = 208, BYTES = WeightRing<FQ_Q6_K, 208>::BYTES;
};

struct NtJob {
    const uint8_t *w[NT_MAX_TARGETS];
    float *y[NT_MAX_TARGETS];
    uint32_t rows[NT_MAX_TARGETS];     // rows of one target (of one expert slice when grouped)
    uint32_t tile_end[NT_MAX_TARGETS]; // 16-row tiles, counted through the targets
    uint32_t count;
    uint32_t pitch, cols, nblk;
    const uint8_t *prep;   // prepared activations (k_prep_nt), row r at r * 544 nblk
    uint32_t m;            // dense: activation rows
    uint32_t slices;       // dense: K slices
    uint32_t nb_max;       // superblocks of the longest slice
    float4 *ws;            // partial sums [tile][slice][lane][NT]
    uint32_t *counters;    // arrivals per tile
    // grouped: activation rows [offsets[i], offsets[i + 1]) belong to expert slots ? slots[i] : i
    const uint32_t *offsets, *slots;
    uint32_t groups, total_rows;
    // grouped: sorted row r reads prepared row src[r] / src_div (the gather of expert-sorted routes), or r itself
    const uint32_t *src;
    uint32_t src_div;
};

// MMAs whose accumulator starts at zero (the zero register four times: nothing to initialise).
__device__ __forceinline__ void mma_u8s8_z(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}
__device__ __forceinline__ void mma_s8s8_k16_z(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
                 : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
                 : "r"(a0), "r"(a1), "r"(b0), "r"(0));
}

// Prepared activations.  In global memory (written once per projection by k_prep_nt), per activation row:
//   frag [nblk][8 groups of 32][4 threads][16 bytes]   what thread t of a quad feeds for a group:
//                                                      Q4_K  values 8t .. 8t+7:               hi[8] | lo[8]
//                                                      Q6_K  values 4t .. 4t+3 of each half:  hi[4] | lo[4] | hi[4] | lo[4]
//   rec  [nblk][32 bytes]   per superblock: the sums of x' per 32 values as three signed base-256 digits, most
//                           significant first, 8 bytes each (the B operand of the MMA that multiplies them with
//                           the eight Q4_K minimums), then 1 / s as f32, then 4 spare bytes.
// A block copies the superblocks of its slice of TOK = 8 NT rows into shared memory: frag rows with stride
// 512 nb + 64 (rows g, g + 1 of a quarter-warp on different banks), rec rows with a stride of 4 words mod 32.
struct PrepNT {
    uint32_t cols, nblk, rec_off, token_bytes;
};
__host__ __device__ inline PrepNT prep_nt_layout(uint32_t cols) {
    PrepNT L;
    L.cols = cols;
    L.nblk = cols / 256;
    L.rec_off = L.nblk * 512;
    L.token_bytes = L.nblk * 544;
    return L;
}
struct ActSmem {
    uint8_t *frag;
    uint8_t *rec;
    uint32_t row_stride, rec_stride;
};
// 16 bytes past a multiple of 128: rows stay 16-byte aligned for the copies, and the eight rows a warp reads
// records of fall on different banks.
__host__ __device__ inline uint32_t nt_rec_stride(uint32_t nb) { return 32 * nb + ((16 + 128 - (32 * nb) % 128) % 128); } // bytes
// Bytes of the resident set (a multiple of 16: the warps' rings follow it).
__host__ __device__ inline uint32_t nt_act_bytes(uint32_t tok, uint32_t nb) {
    return (tok * (nb * 512 + 64) + tok * nt_rec_stride(nb) + 15u) & ~15u;
}

// One warp per (activation row, superblock); lane l owns the eight values at 256 b + 8 l.
//   src    (may be null) row i of the prepared set is row src[i] / src_div of x (expert-sorted routes);
//   range  (may be null) only rows [range[0], range[range_stride]) are prepared (the experts one rank owns);
//   x_up   (may be null) the activations are the gated unit silu(x) * x_up, as `k_swiglu` computes it;
//   norm_w (may be null) the activations are rmsnorm(x) * norm_w.
template <int FMT>
__global__ void __launch_bounds__(128)
k_prep_nt(const float *__restrict__ x, const float *__restrict__ x_up, const float *__restrict__ norm_w, float eps, uint32_t xrows,
          const uint32_t *__restrict__ src, uint32_t src_div, const uint32_t *__restrict__ range, uint32_t range_stride, PrepNT L,
          uint8_t *__restrict__ out) {
    pdl_trigger();
    pdl_wait();
    const uint32_t warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    const uint32_t xr = warp / L.nblk, b = warp % L.nblk;
    if (xr >= xrows) return;
    if (range && (xr < range[0] || xr >= range[range_stride])) return;
    const size_t srow = src ? src[xr] / src_div : xr;
    const float4 *sp = reinterpret_cast<const float4 *>(x + srow * L.cols + (size_t)b * 256 + lane * 8);
    const float4 v0 = sp[0], v1 = sp[1];
    float v[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
    if (norm_w) { // rmsnorm(x) * norm_w, as `h_rmsnorm` computes it
        const float scale = row_inv_rms(x + srow * L.cols, L.cols, eps, lane);
        const float4 *ws = reinterpret_cast<const float4 *>(norm_w + (size_t)b * 256 + lane * 8);
        const float4 w0 = ws[0], w1 = ws[1];
        const float g[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
        for (int i = 0; i < 8; i++) v[i] = v[i] * scale * g[i];
    }
    if (x_up) {
        const float4 *us = reinterpret_cast<const float4 *>(x_up + srow * L.cols + (size_t)b * 256 + lane * 8);
        const float4 u0 = us[0], u1 = us[1];
        const float u[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
#pragma unroll
        for (int i = 0; i < 8; i++) v[i] = v[i] / (1.f + expf(-v[i])) * u[i];
    }
    const Quant8 q = quantize8(v);
    uint8_t *base = out + (size_t)xr * L.token_bytes, *frag = base + (size_t)b * 512, *rec = base + L.rec_off + (size_t)b * 32;
    if constexpr (FMT == FQ_Q4_K) {
        // 32-value group lane / 4, thread lane % 4
        *reinterpret_cast<uint4 *>(frag + 16 * lane) = make_uint4(pack4(q.hi), pack4(q.hi + 4), pack4(q.lo), pack4(q.lo + 4));
    } else {
        // The lane's values sit in half (lane % 4) / 2 of the group; its first four belong to thread
        // 2 (lane % 2), the other four to the thread after it.
        uint8_t *dst = frag + 64 * (lane >> 2) + 8 * ((lane & 3) >> 1) + 32 * (lane & 1);
        *reinterpret_cast<uint2 *>(dst) = make_uint2(pack4(q.hi), pack4(q.lo));
        *reinterpret_cast<uint2 *>(dst + 16) = make_uint2(pack4(q.hi + 4), pack4(q.lo + 4));
    }
    int sum = q.sum;
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    if ((lane & 3) == 0) { // three signed base-256 digits of the sum
        const int p0 = ((sum + 128) & 0xFF) - 128, rem = (sum - p0) >> 8, p1 = ((rem + 128) & 0xFF) - 128, p2 = (rem - p1) >> 8;
        rec[lane >> 2] = (uint8_t)p2;
        rec[8 + (lane >> 2)] = (uint8_t)p1;
        rec[16 + (lane >> 2)] = (uint8_t)p0;
    }
    // A non-finite activation anywhere in the superblock makes its factor NaN.
    if (lane == 0) {
        *reinterpret_cast<float *>(rec + 24) = q.finite ? ldexpf(1.f, -q.e) : __int_as_float(0x7fc00000);
        *reinterpret_cast<uint32_t *>(rec + 28) = 0u;
    }
}

// One superblock (index `bb` within the block's slice) of a 16-row tile whose packed bytes lie in `stage`,
// against NT tiles of eight activation rows: adds into yacc[nt][i], i = 2 r + c, the contribution to weight row
// g + 8 r and activation row 8 nt + 2 t + c.
template <int FMT, int NT>
__device__ __forceinline__ void superblock_nt(const uint8_t *stage, const ActSmem &A, uint32_t bb, bool odd_b, int g, int t, float (&yacc)[NT][4]) {
    int ah[NT][4], al[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; nt++)
#pragma unroll
        for (int i = 0; i < 4; i++) ah[nt][i] = al[nt][i] = 0;
    const uint8_t *fragp[NT];
#pragma unroll
    for (int nt = 0; nt < NT; nt++) fragp[nt] = A.frag + (size_t)(8 * nt + g) * A.row_stride + (size_t)bb * 512 + 16 * t;
    if constexpr (FMT == FQ_Q4_K || FMT == FQ_Q5_K) {
        constexpr uint32_t ROW = StageNT<FMT>::ROW, QS = FMT == FQ_Q4_K ? 16 : 48;
        const uint8_t *r0 = stage + g * ROW, *r1 = r0 + 8 * ROW;
        uint2 h0 = make_uint2(0u, 0u), h1 = make_uint2(0u, 0u); // Q5_K: qh under this thread's eight values of every sub-block
        if constexpr (FMT == FQ_Q5_K) {
            h0 = *reinterpret_cast<const uint2 *>(r0 + 16 + 8 * t);
            h1 = *reinterpret_cast<const uint2 *>(r1 + 16 + 8 * t);
        }
        // Scales and minimums of sub-blocks 0..3 and 4..7, one per byte (`get_scale_min_k4`).
        uint32_t sc4[2][2], mn4[2][2];
        float d[2], dmin[2];
#pragma unroll
        for (int r = 0; r < 2; r++) {
            const uint4 h = *reinterpret_cast<const uint4 *>(r ? r1 : r0);
            sc4[r][0] = h.y & 0x3F3F3F3Fu;
            mn4[r][0] = h.z & 0x3F3F3F3Fu;
            sc4[r][1] = (h.w & 0x0F0F0F0Fu) | ((h.y >> 2) & 0x30303030u);
            mn4[r][1] = ((h.w >> 4) & 0x0F0F0F0Fu) | ((h.z >> 2) & 0x30303030u);
            d[r] = f16_bits_to_f32((uint16_t)(h.x & 0xFFFFu));
            dmin[r] = f16_bits_to_f32((uint16_t)(h.x >> 16));
        }
        // The minimum term sum_j m_j * sx_j by three MMAs per tile: A holds the eight minimums of each row on
        // k slots 0..7 (threads 0 and 1 of a quad), B the digits of the sums.
        int am[NT][4];
        {
            const uint32_t ma0 = t == 0 ? mn4[0][0] : t == 1 ? mn4[0][1] : 0u, ma1 = t == 0 ? mn4[1][0] : t == 1 ? mn4[1][1] : 0u;
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                const uint8_t *sp = A.rec + (size_t)(8 * nt + g) * A.rec_stride + (size_t)bb * 32 + 4 * (t & 1);
                int c2[4], c1[4], c0[4];
                mma_u8s8_z(c2, ma0, ma1, 0u, 0u, *reinterpret_cast<const uint32_t *>(sp), 0u);
                mma_u8s8_z(c1, ma0, ma1, 0u, 0u, *reinterpret_cast<const uint32_t *>(sp + 8), 0u);
                mma_u8s8_z(c0, ma0, ma1, 0u, 0u, *reinterpret_cast<const uint32_t *>(sp + 16), 0u);
#pragma unroll
                for (int i = 0; i < 4; i++) am[nt][i] = (c2[i] * 256 + c1[i]) * 256 + c0[i];
            }
        }
#pragma unroll
        for (int c = 0; c < 4; c++) {
            const uint2 q0 = *reinterpret_cast<const uint2 *>(r0 + QS + 32 * c + 8 * t), q1 = *reinterpret_cast<const uint2 *>(r1 + QS + 32 * c + 8 * t);
#pragma unroll
            for (int half = 0; half < 2; half++) { // low nibbles = sub-block 2c, high nibbles = sub-block 2c + 1
                const int j = 2 * c + half;
                uint32_t a0 = (half ? q0.x >> 4 : q0.x) & 0x0F0F0F0Fu, a1 = (half ? q1.x >> 4 : q1.x) & 0x0F0F0F0Fu;
                uint32_t a2 = (half ? q0.y >> 4 : q0.y) & 0x0F0F0F0Fu, a3 = (half ? q1.y >> 4 : q1.y) & 0x0F0F0F0Fu;
                if constexpr (FMT == FQ_Q5_K) { // bit j of the qh bytes becomes bit 4
                    auto fifth = [j](uint32_t hw) { return (j < 4 ? hw << (4 - j) : hw >> (j - 4)) & 0x10101010u; };
                    a0 |= fifth(h0.x);
                    a1 |= fifth(h1.x);
                    a2 |= fifth(h0.y);
                    a3 |= fifth(h1.y);
                }
                const int s0 = byte_u(sc4[0][j >> 2], j & 3), s1 = byte_u(sc4[1][j >> 2], j & 3);
#pragma unroll
                for (int nt = 0; nt < NT; nt++) {
                        const uint4 f = *reinterpret_cast<const uint4 *>(fragp[nt] + 64 * j);
                    int ch[4], cl[4];
                    mma_u8s8_z(ch, a0, a1, a2, a3, f.x, f.y);
                    mma_u8s8_z(cl, a0, a1, a2, a3, f.z, f.w);
                    ah[nt][0] += s0 * ch[0];
                    ah[nt][1] += s0 * ch[1];
                    ah[nt][2] += s1 * ch[2];
                    ah[nt][3] += s1 * ch[3];
                    al[nt][0] += s0 * cl[0];
                    al[nt][1] += s0 * cl[1];
                    al[nt][2] += s1 * cl[2];
                    al[nt][3] += s1 * cl[3];
                }
            }
        }
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const float inv = *reinterpret_cast<const float *>(A.rec + (size_t)(8 * nt + 2 * t + (i & 1)) * A.rec_stride + (size_t)bb * 32 + 24);
                const float dot = fmaf(256.f, (float)ah[nt][i], (float)al[nt][i]);
                yacc[nt][i] = fmaf(inv, d[i >> 1] * dot - dmin[i >> 1] * (float)am[nt][i], yacc[nt][i]);
            }
    } else {
        const uint8_t *r0 = stage + g * 208, *r1 = r0 + 8 * 208;
        float d4[2];
#pragma unroll
        for (int r = 0; r < 2; r++) {
            const uint32_t dd = *reinterpret_cast<const uint32_t *>(stage + 16 * 208 + 4 * (g + 8 * r));
            d4[r] = f16_bits_to_f32((uint16_t)(odd_b ? dd >> 16 : dd & 0xFFFFu)) * 0.25f;
        }
        const uint4 sc0 = *reinterpret_cast<const uint4 *>(r0 + 192), sc1 = *reinterpret_cast<const uint4 *>(r1 + 192);
#pragma unroll
        for (int n = 0; n < 2; n++) {
            uint32_t hw[2][2]; // [row][lh]
#pragma unroll
            for (int lh = 0; lh < 2; lh++) {
                hw[0][lh] = *reinterpret_cast<const uint32_t *>(r0 + 128 + 32 * n + 16 * lh + 4 * t);
                hw[1][lh] = *reinterpret_cast<const uint32_t *>(r1 + 128 + 32 * n + 16 * lh + 4 * t);
            }
#pragma unroll
            for (int i = 0; i < 4; i++) { // 32 values 128 n + 32 i ..: scale groups 8n + 2i (first 16) and 8n + 2i + 1
                uint4 f[NT];
#pragma unroll
                for (int nt = 0; nt < NT; nt++) f[nt] = *reinterpret_cast<const uint4 *>(fragp[nt] + 64 * (4 * n + i));
#pragma unroll
                for (int lh = 0; lh < 2; lh++) {
                    uint32_t a[2];
#pragma unroll
                    for (int r = 0; r < 2; r++) {
                        const uint32_t lw = *reinterpret_cast<const uint32_t *>((r ? r1 : r0) + 64 * n + 32 * (i & 1) + 16 * lh + 4 * t);
                        const uint32_t lo4 = (i < 2) ? (lw << 2) : (lw >> 2); // the nibble in bits 2..5
                        const uint32_t h = hw[r][lh];
                        const uint32_t hi2 = i == 0 ? (h << 6) : i == 1 ? (h << 4) : i == 2 ? (h << 2) : h; // the two high bits in bits 6..7
                        // ((q ^ 32) << 2) read as s8 = 4 (q - 32)
                        a[r] = lop3_and_xor(lop3_select(lo4, hi2, 0x3C3C3C3Cu), 0xFCFCFCFCu, 0x80808080u);
                    }
                    const int gidx = 8 * n + 2 * i + lh;
                    const int s0 = byte_s(word_of(sc0, gidx >> 2), gidx & 3), s1 = byte_s(word_of(sc1, gidx >> 2), gidx & 3);
#pragma unroll
                    for (int nt = 0; nt < NT; nt++) {
                                int ch[4], cl[4];
                        mma_s8s8_k16_z(ch, a[0], a[1], lh ? f[nt].z : f[nt].x);
                        mma_s8s8_k16_z(cl, a[0], a[1], lh ? f[nt].w : f[nt].y);
                        ah[nt][0] += s0 * ch[0];
                        ah[nt][1] += s0 * ch[1];
                        ah[nt][2] += s1 * ch[2];
                        ah[nt][3] += s1 * ch[3];
                        al[nt][0] += s0 * cl[0];
                        al[nt][1] += s0 * cl[1];
                        al[nt][2] += s1 * cl[2];
                        al[nt][3] += s1 * cl[3];
                    }
                }
            }
        }
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const float inv = *reinterpret_cast<const float *>(A.rec + (size_t)(8 * nt + 2 * t + (i & 1)) * A.rec_stride + (size_t)bb * 32 + 24);
                yacc[nt][i] = fmaf(inv * d4[i >> 1], fmaf(256.f, (float)ah[nt][i], (float)al[nt][i]), yacc[nt][i]);
            }
    }
}

// FMT: FQ_Q4_K / FQ_Q6_K; NT: tiles of eight activation rows; STAGES: superblocks in flight per warp;
// GROUPED: block = (expert, tile of 8 NT expert-sorted rows), else block = (K slice, share of the row tiles).
template <int FMT, int NT, int STAGES, bool GROUPED>
__global__ void __launch_bounds__(NT > 2 ? 384 : 512, 1)
k_nt(const __grid_constant__ NtJob J, const __grid_constant__ TpPush P) {
    using St = StageNT<FMT>;
    constexpr uint32_t TOK = 8 * NT;
    extern __shared__ __align__(128) uint8_t nt_smem[];
    __shared__ uint32_t job_group, job_row0, job_cnt, job_src[TOK];
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5, W = blockDim.x >> 5;
    const int g = lane >> 2, t = lane & 3;

    // The block's job.
    uint32_t b0 = 0, nb = J.nblk, slice = 0, first, stride, m = J.m, xrow0 = 0;
    size_t expert_off = 0; // rows to skip in every target
    if constexpr (GROUPED) {
        pdl_wait(); // the routing map is the output of an earlier kernel of the stream
        if (warp == 0) {
            // Tile blockIdx.x of all groups' row tiles, counted through the groups (32 at a time).
            uint32_t base = 0, found = 0xffffffffu, row0 = 0, cnt = 0;
            for (uint32_t g0 = 0; g0 < J.groups && found == 0xffffffffu; g0 += 32) {
                const uint32_t gi = g0 + lane;
                const uint32_t lo = gi < J.groups ? J.offsets[gi] : 0, hi = gi < J.groups ? J.offsets[gi + 1] : 0;
                const uint32_t n = hi > lo ? (hi - lo + TOK - 1) / TOK : 0;
                uint32_t incl = n;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const uint32_t v = __shfl_up_sync(0xffffffffu, incl, o);
                    if ((int)lane >= o) incl += v;
                }
                const uint32_t excl = base + incl - n;
                const bool mine = blockIdx.x >= excl && blockIdx.x < excl + n;
                const uint32_t who = __ballot_sync(0xffffffffu, mine);
                if (who) {
                    const int src_lane = __ffs(who) - 1;
                    found = g0 + src_lane;
                    const uint32_t tile_in = blockIdx.x - __shfl_sync(0xffffffffu, excl, src_lane);
                    const uint32_t glo = __shfl_sync(0xffffffffu, lo, src_lane), ghi = __shfl_sync(0xffffffffu, hi, src_lane);
                    row0 = glo + tile_in * TOK;
                    cnt = min(TOK, ghi - row0);
                }
                base += __shfl_sync(0xffffffffu, incl, 31);
            }
            if (lane == 0) {
                job_group = found;
                job_row0 = row0;
                job_cnt = cnt;
            }
            // The prepared row behind each of the tile's sorted rows.
            for (uint32_t i = lane; i < TOK; i += 32) job_src[i] = i < cnt ? (J.src ? J.src[row0 + i] / J.src_div : row0 + i) : 0u;
        }
        __syncthreads();
        if (job_group == 0xffffffffu) return; // more blocks than tiles
        const uint32_t e = J.slots ? J.slots[job_group] : job_group;
        expert_off = (size_t)e * J.rows[0];
        m = job_cnt;
        xrow0 = job_row0;
        first = warp;
        stride = W;
    } else {
        slice = blockIdx.x % J.slices;
        b0 = (uint32_t)((uint64_t)slice * J.nblk / J.slices);
        nb = (uint32_t)((uint64_t)(slice + 1) * J.nblk / J.slices) - b0;
        first = (blockIdx.x / J.slices) * W + warp;
        stride = (gridDim.x / J.slices) * W;
    }
    const uint32_t total_tiles = J.tile_end[J.count - 1];

    ActSmem A;
    A.row_stride = J.nb_max * 512 + 64;
    A.rec_stride = nt_rec_stride(J.nb_max);
    A.frag = nt_smem;
    A.rec = nt_smem + (size_t)TOK * A.row_stride;
    uint8_t *ring = nt_smem + nt_act_bytes(TOK, J.nb_max) + (size_t)warp * STAGES * St::BYTES;

    struct Tile {
        const uint8_t *w; // first row of the target (of the expert's slice of it)
        float *y;
        uint32_t rows, row0;
    };
    auto tile_at = [&](uint32_t tile) {
        uint32_t which = 0, first_tile = 0;
#pragma unroll
        for (int i = 0; i < NT_MAX_TARGETS - 1; i++)
            if ((uint32_t)i + 1 < J.count && tile >= J.tile_end[i]) { which = i + 1; first_tile = J.tile_end[i]; }
        Tile q;
        q.rows = J.rows[which];
        q.row0 = (tile - first_tile) * 16;
        q.w = J.w[which] + expert_off * J.pitch; // grouped targets share one shape
        q.y = J.y[which];
        return q;
    };

    // Producer side of the warp's ring: item = (tile, superblock of the slice), in the order they are consumed.
    WeightRing<FMT, St::ROW> wr;
    uint32_t p_tile = first, p_bb = 0, p_stage = 0;
    auto start_tile = [&](uint32_t tile) {
        const Tile q = tile_at(tile);
        wr.start_tile(q.w + (size_t)q.row0 * J.pitch, q.rows - 1 - q.row0, J.pitch, J.nblk, lane);
    };
    if (p_tile < total_tiles) start_tile(p_tile);
    auto issue = [&]() {
        if (p_tile < total_tiles) {
            wr.issue(ring + (size_t)p_stage * St::BYTES, b0 + p_bb, lane);
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
    if constexpr (!GROUPED) pdl_wait();
    const uint32_t seq = P.world > 1 ? tp_seq(P) : 0u;

    // The block's resident activations: 16-byte pieces of the prepared rows (per row 32 nb of fragments and
    // 2 nb of records), copied asynchronously; rows the job does not have are zero.
    {
        // Rows the tile loop will read: all of them, or (grouped tiles of 32) as many eights as it will take.
        const uint32_t rows_used = (GROUPED && NT == 4) ? (m <= 8 ? 8u : m <= 16 ? 16u : 32u) : TOK;
        const uint32_t per_row = 34 * nb, pieces = rows_used * per_row;
        const size_t tok_bytes = (size_t)J.nblk * 544;
        for (uint32_t i = threadIdx.x; i < pieces; i += blockDim.x) {
            const uint32_t tok = i / per_row, p = i - tok * per_row;
            uint8_t *dst = p < 32 * nb ? A.frag + (size_t)tok * A.row_stride + 16 * p : A.rec + (size_t)tok * A.rec_stride + 16 * (p - 32 * nb);
            if (tok < m) {
                size_t prow = xrow0 + tok;
                if constexpr (GROUPED) prow = job_src[tok];
                const uint8_t *row = J.prep + prow * tok_bytes;
                cp_async16(dst, p < 32 * nb ? row + (size_t)b0 * 512 + 16 * p : row + (size_t)J.nblk * 512 + (size_t)b0 * 32 + 16 * (p - 32 * nb));
            } else {
                *reinterpret_cast<uint4 *>(dst) = make_uint4(0u, 0u, 0u, 0u);
            }
        }
        cp_async_commit();
        cp_async_wait<0>();
    }
    __syncthreads();

    // The tile loop for NTU tiles of eight activation rows.  A grouped block picks NTU by the rows its tile holds
    // (the resident layout does not depend on it), so a nearly empty tile does not pay for a full one.
    uint32_t c_stage = 0;
    auto run = [&](auto ntu) {
        constexpr int NTU = decltype(ntu)::value;
        for (uint32_t tile = first; tile < total_tiles; tile += stride) {
            const Tile here = tile_at(tile);
            float yacc[NTU][4];
    #pragma unroll
            for (int nt = 0; nt < NTU; nt++)
    #pragma unroll
                for (int i = 0; i < 4; i++) yacc[nt][i] = 0.f;
            for (uint32_t bb = 0; bb < nb; bb++) {
                issue();
                cp_async_wait<STAGES - 1>();
                __syncwarp();
                superblock_nt<FMT, NTU>(ring + (size_t)c_stage * St::BYTES, A, bb, ((b0 + bb) & 1u) != 0, g, t, yacc);
                __syncwarp();
                c_stage = c_stage + 1 == STAGES ? 0 : c_stage + 1;
            }
            bool store = true;
            if (!GROUPED && J.slices > 1) {
                // Partial sums of this slice; the last warp to arrive at the tile adds all slices in slice order.
                float4 *part = J.ws + ((size_t)tile * J.slices) * 32 * NTU;
    #pragma unroll
                for (int nt = 0; nt < NTU; nt++) part[((size_t)slice * 32 + lane) * NTU + nt] = make_float4(yacc[nt][0], yacc[nt][1], yacc[nt][2], yacc[nt][3]);
                __threadfence();
                __syncwarp();
                uint32_t arrived = 0;
                if (lane == 0) arrived = atomicAdd(J.counters + tile, 1u);
                arrived = __shfl_sync(0xffffffffu, arrived, 0);
                store = arrived + 1 == J.slices;
                if (store) {
                    __threadfence();
                    if (lane == 0) J.counters[tile] = 0;
    #pragma unroll
                    for (int nt = 0; nt < NTU; nt++) {
                        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
                        for (uint32_t s = 0; s < J.slices; s++) {
                            const float4 p = __ldcg(&part[((size_t)s * 32 + lane) * NTU + nt]);
                            acc.x += p.x;
                            acc.y += p.y;
                            acc.z += p.z;
                            acc.w += p.w;
                        }
                        yacc[nt][0] = acc.x;
                        yacc[nt][1] = acc.y;
                        yacc[nt][2] = acc.z;
                        yacc[nt][3] = acc.w;
                    }
                }
            }
            if (store) {
    #pragma unroll
                for (int nt = 0; nt < NTU; nt++)
    #pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const uint32_t row = here.row0 + g + (i >> 1) * 8, tok = 8 * nt + 2 * t + (i & 1);
                        if (row < here.rows && tok < m) {
                            float *dst = &here.y[(size_t)(xrow0 + tok) * here.rows + row];
                            *dst = yacc[nt][i];
                            if (!GROUPED && P.world > 1) tp_store(P, seq, dst, yacc[nt][i]);
                        }
                    }
            }
        }
    };
    if constexpr (GROUPED && NT == 4) {
        if (m <= 8) run(std::integral_constant<int, 1>{});
        else if (m <= 16) run(std::integral_constant<int, 2>{});
        else run(std::integral_constant<int, 4>{});
    } else {
        run(std::integral_constant<int, NT>{});
    }
    cp_async_wait<0>();
    if (!GROUPED && P.world > 1) tp_finish(P, seq);
}

struct NtShape {
    uint32_t warps, stages, slices, nb_max, smem, grid;
};

template <int FMT, int NT, bool GROUPED> void (*nt_kernel(int stages))(NtJob, TpPush) {
    return stages >= 4 ? k_nt<FMT, NT, 4, GROUPED> : stages == 3 ? k_nt<FMT, NT, 3, GROUPED> : k_nt<FMT, NT, 2, GROUPED>;
}

// Chooses warps per block, ring depth and K slices for `tiles16` 16-row tiles of `nblk` superblocks.
template <int FMT, int NT> bool nt_shape(const fq_device *dev, uint32_t tiles16, uint32_t nblk, bool grouped, NtShape &S) {
    using St = StageNT<FMT>;
    constexpr uint32_t TOK = 8 * NT;
    S.warps = NT > 2 ? 12 : 16; // wider tiles hold more accumulators per thread: fewer, fatter warps
    // Fewest slices: a slice of activations must fit beside a ring of two stages per warp.
    const uint32_t ring2 = S.warps * 2 * St::BYTES;
    uint32_t nb_fit = 0;
    while (nb_fit < nblk && nt_act_bytes(TOK, nb_fit + 1) + ring2 <= NT_SMEM_MAX) nb_fit++;
    if (nb_fit == 0) return false;
    uint32_t slices = (nblk + nb_fit - 1) / nb_fit;
    if (grouped) {
        if (slices > 1) return false; // an expert's whole K is resident
    } else {
        // More slices give more warps a tile when rows are few, at the price of a shorter run per tile with a fixed
        // cost per run (and, beyond one slice, the partial sums).  Estimated time in units of one superblock of
        // one tile: rounds of tiles per warp x (superblocks per slice + overhead) + the block's preparation.
        const uint32_t sms = (uint32_t)dev->sm_count;
        double best = 1e30;
        uint32_t pick = slices;
        for (uint32_t s = slices; s <= std::min(nblk, sms); s++) {
            const uint32_t per_slice = (sms / s) * S.warps, nbm = (nblk + s - 1) / s;
            const uint32_t rounds = (tiles16 + per_slice - 1) / per_slice;
            const double cost = rounds * (nbm + (s > 1 ? 1.5 : 0.3)) + 0.25 * nbm * TOK / 16.0;
            if (cost < best - 1e-9) { best = cost; pick = s; }
        }
        slices = pick;
    }
    S.slices = slices;
    S.nb_max = (nblk + slices - 1) / slices;
    const size_t act = nt_act_bytes(TOK, S.nb_max);
    S.stages = (uint32_t)std::min<size_t>(4, (NT_SMEM_MAX - act) / ((size_t)S.warps * St::BYTES));
    if (S.stages < 2) return false;
    S.smem = (uint32_t)(act + (size_t)S.warps * S.stages * St::BYTES);
    S.grid = grouped ? 0 : std::max(1u, (uint32_t)dev->sm_count / slices) * slices;
    return true;
}

template <int FMT, int NT, bool GROUPED> cudaError_t nt_launch(fq_device *dev, const NtJob &J, const NtShape &S, uint32_t grid, const TpPush &push) {
    auto kernel = nt_kernel<FMT, NT, GROUPED>((int)S.stages);
    static bool configured[5] = {};
    if (!configured[S.stages]) {
        const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)NT_SMEM_MAX);
        if (e != cudaSuccess) return e;
        configured[S.stages] = true;
    }
    return launch_pdl(kernel, dim3(grid), dim3(S.warps * 32), S.smem, dev->stream, J, push);
}

// Prepares `xrows` activation rows into the handle's scratch (its two halves alternate, so a preparation that
// starts early never writes what the projection before may still be reading) and returns where, or null when
// they do not fit.
uint8_t *launch_prep(fq_device *dev, int format, const ProjectArgs &f, uint32_t xrows, const uint32_t *src, uint32_t src_div, const uint32_t *range,
                     uint32_t range_stride, cudaError_t &e) {
    const PrepNT L = prep_nt_layout(f.cols);
    if ((size_t)xrows * L.token_bytes > dev->xprep_bytes / 2) return nullptr;
    dev->xprep_turn ^= 1u;
    uint8_t *prep = (uint8_t *)dev->xprep + (dev->xprep_turn ? dev->xprep_bytes / 2 : 0);
    const uint32_t warps = xrows * L.nblk;
    if (format == FQ_Q4_K || format == FQ_Q5_K) // the same fragment order
        e = launch_pdl(k_prep_nt<FQ_Q4_K>, dim3((warps + 3) / 4), dim3(128), 0, dev->stream, (const float *)f.x, f.x_up, f.norm_w, f.norm_eps, xrows, src, src_div, range, range_stride, L, prep);
    else
        e = launch_pdl(k_prep_nt<FQ_Q6_K>, dim3((warps + 3) / 4), dim3(128), 0, dev->stream, (const float *)f.x, f.x_up, f.norm_w, f.norm_eps, xrows, src, src_div, range, range_stride, L, prep);
    return prep;
}

template <int FMT, int NT> int launch_dense(fq_device *dev, const ProjectArgs *a, uint32_t count) {
    NtJob J{};
    J.count = count;
    uint32_t tiles = 0;
    for (uint32_t i = 0; i < count; i++) {
        J.w[i] = a[i].w;
        J.y[i] = (float *)a[i].y;
        J.rows[i] = a[i].rows;
        tiles += (a[i].rows + 15) / 16;
        J.tile_end[i] = tiles;
    }
    J.pitch = a[0].row_bytes;
    J.cols = a[0].cols;
    J.nblk = a[0].cols / 256;
    J.m = a[0].m;
    NtShape S;
    if (!nt_shape<FMT, NT>(dev, tiles, J.nblk, false, S)) return FQ_ERR_UNSUPPORTED;
    J.slices = S.slices;
    J.nb_max = S.nb_max;
    J.ws = (float4 *)dev->nt_ws;
    J.counters = dev->nt_counters;
    if (S.slices > 1 && ((size_t)tiles * S.slices * 32 * NT * sizeof(float4) > dev->nt_ws_bytes || tiles > dev->nt_counter_count))
        return FQ_ERR_UNSUPPORTED;
    cudaError_t e = cudaSuccess;
    if (!(J.prep = launch_prep(dev, FMT, a[0], a[0].m, nullptr, 1, nullptr, 0, e))) return FQ_ERR_UNSUPPORTED;
    if (int rc = fq_check_cuda(dev, e, "activation preparation launch")) return rc;
    TpPush push{};
    if (dev->tp_push) { // one launch covers every target: it can do the exchange itself
        push = *dev->tp_push;
        dev->tp_push = nullptr;
        dev->tp_pushed = true;
    }
    if (int rc = fq_check_cuda(dev, nt_launch<FMT, NT, false>(dev, J, S, S.grid, push), "gemv launch")) return rc;
    return fq_end_enqueue(dev, "gemv_nt", 2);
}

} // namespace

// `a[0..count)` share x, m (2..16), format and width.
int fq_launch_gemv_nt_many(fq_device *dev, const ProjectArgs *a, uint32_t count) {
    if (count == 0 || count > (uint32_t)NT_MAX_TARGETS) return FQ_ERR_UNSUPPORTED;
    const ProjectArgs &f = a[0];
    if ((f.format != FQ_Q4_K && f.format != FQ_Q5_K && f.format != FQ_Q6_K) || f.x_dtype != FQ_F32 || f.y_dtype != FQ_F32) return FQ_ERR_UNSUPPORTED;
    if (f.cols % 256 || f.row_bytes % 16 || f.ids || f.m < 2 || f.m > 16) return FQ_ERR_UNSUPPORTED;
    for (uint32_t i = 1; i < count; i++)
        if (a[i].format != f.format || a[i].cols != f.cols || a[i].x != f.x || a[i].x_up != f.x_up || a[i].norm_w != f.norm_w || a[i].m != f.m || a[i].ids ||
            a[i].x_dtype != FQ_F32 || a[i].y_dtype != FQ_F32)
            return FQ_ERR_UNSUPPORTED;
    if (f.format == FQ_Q4_K) return f.m <= 8 ? launch_dense<FQ_Q4_K, 1>(dev, a, count) : launch_dense<FQ_Q4_K, 2>(dev, a, count);
    if (f.format == FQ_Q5_K) return f.m <= 8 ? launch_dense<FQ_Q5_K, 1>(dev, a, count) : launch_dense<FQ_Q5_K, 2>(dev, a, count);
    return f.m <= 8 ? launch_dense<FQ_Q6_K, 1>(dev, a, count) : launch_dense<FQ_Q6_K, 2>(dev, a, count);
}

// Grouped expert projection over expert-sorted rows (F32 in, F32 out), up to two expert stacks of one shape
// sharing the rows (gate and up).  `src` (may be null): row r of the sorted set is row src[r] / src_div of x, so
// the gather needs no pass of its own; `a[0].x_up`: the activations are the gated unit silu(x) * x_up.
int fq_launch_gemv_nt_grouped(fq_device *dev, const ProjectArgs *a, uint32_t count, uint32_t total_rows, const uint32_t *src, uint32_t src_div) {
    if (count == 0 || count > 2) return FQ_ERR_UNSUPPORTED;
    const ProjectArgs &f = a[0];
    if ((f.format != FQ_Q4_K && f.format != FQ_Q5_K && f.format != FQ_Q6_K) || f.x_dtype != FQ_F32 || f.y_dtype != FQ_F32) return FQ_ERR_UNSUPPORTED;
    if (f.cols % 256 || f.row_bytes % 16 || !f.offsets || f.groups == 0 || total_rows == 0) return FQ_ERR_UNSUPPORTED;
    for (uint32_t i = 1; i < count; i++)
        if (a[i].format != f.format || a[i].cols != f.cols || a[i].rows != f.rows || a[i].x != f.x || a[i].offsets != f.offsets ||
            a[i].slots != f.slots || a[i].groups != f.groups || a[i].experts != f.experts)
            return FQ_ERR_UNSUPPORTED;
    NtJob J{};
    J.count = count;
    uint32_t tiles = 0;
    for (uint32_t i = 0; i < count; i++) {
        J.w[i] = a[i].w;
        J.y[i] = (float *)a[i].y;
        J.rows[i] = a[i].rows;
        tiles += (a[i].rows + 15) / 16;
        J.tile_end[i] = tiles;
    }
    J.pitch = f.row_bytes;
    J.cols = f.cols;
    J.nblk = f.cols / 256;
    J.slices = 1;
    J.offsets = f.offsets;
    J.slots = f.slots;
    J.groups = f.groups;
    J.total_rows = total_rows;
    NtShape S;
    constexpr int GNT = 4; // grouped blocks take tiles of 32 expert-sorted rows
    const bool ok = f.format == FQ_Q4_K ? nt_shape<FQ_Q4_K, GNT>(dev, tiles, J.nblk, true, S)
                  : f.format == FQ_Q5_K ? nt_shape<FQ_Q5_K, GNT>(dev, tiles, J.nblk, true, S) : nt_shape<FQ_Q6_K, GNT>(dev, tiles, J.nblk, true, S);
    if (!ok) return FQ_ERR_UNSUPPORTED;
    J.nb_max = S.nb_max;
    cudaError_t e = cudaSuccess;
    // With a gather (`src`) every row of x is prepared once and the blocks pick rows by index; else the rows of
    // the experts in `offsets` (a rank's share when the matrices hold only some experts).
    if (src) {
        if (src_div == 0) return FQ_ERR_UNSUPPORTED;
        J.src = src;
        J.src_div = src_div;
        J.prep = launch_prep(dev, (int)f.format, f, (total_rows + src_div - 1) / src_div, nullptr, 1, nullptr, 0, e);
    } else {
        J.prep = launch_prep(dev, (int)f.format, f, total_rows, nullptr, 1, f.offsets, f.groups, e);
    }
    if (!J.prep) return FQ_ERR_UNSUPPORTED;
    if (int rc = fq_check_cuda(dev, e, "activation preparation launch")) return rc;
    // Every group has at most ceil(rows / 32) <= rows / 32 + 1 tiles.
    const uint32_t grid = total_rows / (8 * GNT) + f.groups;
    e = f.format == FQ_Q4_K ? nt_launch<FQ_Q4_K, GNT, true>(dev, J, S, grid, TpPush{})
      : f.format == FQ_Q5_K ? nt_launch<FQ_Q5_K, GNT, true>(dev, J, S, grid, TpPush{}) : nt_launch<FQ_Q6_K, GNT, true>(dev, J, S, grid, TpPush{});
    if (int rc = fq_check_cuda(dev, e, "grouped gemv launch")) return rc;
    return fq_end_enqueue(dev, "gemv_nt_grouped", 2);
}
