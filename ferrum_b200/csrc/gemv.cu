// Decode / speculative-verify projections (M = 1..16, F32 in, F32 out) with the packed weights
// streamed once.  The work of `h_mv_*`, `h_mvb_*` and `h_mms_*` in the reference
// (src/metal/shaders/hybrid.metal:688-756, 838-897, 1330-1394, 1419-1495).
//
// On B200 a K-quant GEMV is bound by instruction issue before HBM, so the multiply runs on the
// tensor cores even at M = 1 (warp-level mma.sync m16n8k16, f16 operands, fp32 accumulators in
// registers):
//
//   A (16 weight rows x 16 k)    = the scaled integer quants as f16, built from the packed bits with
//                                  a LOP3 (bits into the mantissa of a power of two) and one HFMA2
//                                  per two weights:  Q4_K  sc * q  (exact, <= 63 * 15);
//                                                    Q6_K  scale * (q - 32)  (one f16 rounding
//                                                    when the product exceeds 11 bits);
//   B (16 k x 8 columns)         = the activations as f16, split x = hi + lo so the product keeps
//                                  fp32-level accuracy.  With M <= 4 the hi parts sit in columns
//                                  0..3 and the lo parts in columns 4..7 of ONE MMA; otherwise
//                                  columns are activation rows and hi / lo take two MMAs;
//   per superblock (Q4_K):  y += (1/s) * (d * acc - dmin * sum_j m_j * Sx_j)
//   per superblock (Q6_K):  y += (1/s) *  d * acc
//
// the factored forms of the reference's `mv_q4_K` / `mv_q6_K`.  A preparation kernel turns the fp32
// activations into the B fragments (already in the register order of the MMA), the per-32 sums Sx
// and a power-of-two scale s per (activation row, superblock) that keeps every f16 operand in range
// whatever the magnitude of x.
//
// Thread (g = lane / 4, t = lane % 4) of a warp owns weight rows g and g + 8 of a 16-row tile and a
// fixed quarter of each superblock's packed bytes (Q4_K: chunk t = sub-blocks 2t, 2t+1; Q6_K: half
// n = t / 2, 16-value run t % 2 of every 32-group).  The MMA's k order is free as long as A and B
// agree, so nothing is exchanged between lanes.  Each thread reads its bytes with 128-bit loads that do
// not allocate in L1 and always has the next superblock's loads in flight while it computes on the
// current one; L1 is left to the prepared activations, which every block re-reads.
#include <cstdlib>
#include <type_traits>

#include "blocks.cuh"
#include "internal.h"

namespace {

constexpr int WARPS = 4;   // warps of a thread block split K between them
constexpr int THREADS = WARPS * 32;

// Programmatic dependent launch: a kernel launched with the stream-serialization attribute may start
// while its predecessor in the stream is still running; `pdl_wait` blocks until the predecessor has
// completed and its writes are visible, `pdl_trigger` lets the successor start its own prologue.
// Every kernel here waits before it reads activations or writes anything, so the stream's total
// order is preserved; only weight prefetch (immutable data) runs ahead.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---------------------------------------------------------------- prepared activations
//
// One group holds `cols_n` columns (activation rows, or hi / lo halves of up to 4 of them):
//   x0  [nblk][8 u][cols_n][4 t] x 16 B   unit (b,u,col,t) = eight f16 values x[k0 + {0,2,1,3,4,6,5,7}]
//        Q4_K: u = 4 h + q, k0 = 256 b + 64 t + 32 h + 8 q
//        Q6_K: u = 2 i + v, k0 = 256 b + 128 (t / 2) + 32 i + 16 (t % 2) + 8 v
//   x1  the same for the lo parts (unused in split-column mode)
//   sx0 [nblk][cols_n][4 t] x 4 B         half2(Sx of sub-blocks 2t, 2t+1), hi part (Q4_K only)
//   sx1 the lo parts (unused in split-column mode)
//   isc [nblk][8] x 4 B                   1 / s per activation row (indexed by column)
struct PrepLayout {
    uint32_t nblk, cols_n, split, fmt;
    uint32_t x1_off, sx0_off, sx1_off, isc_off, group_bytes;
};

PrepLayout prep_layout(uint32_t fmt, uint32_t cols, uint32_t cols_n, bool split) {
    PrepLayout L;
    L.nblk = cols / 256;
    L.cols_n = cols_n;
    L.split = split;
    L.fmt = fmt;
    const uint32_t xbytes = L.nblk * 8 * cols_n * 4 * 16, sbytes = L.nblk * cols_n * 4 * 4;
    L.x1_off = xbytes;
    L.sx0_off = 2 * xbytes;
    L.sx1_off = L.sx0_off + sbytes;
    L.isc_off = L.sx1_off + sbytes;
    L.group_bytes = (L.isc_off + L.nblk * cols_n * 4 + 255u) & ~255u;
    return L;
}

__device__ __forceinline__ uint4 pack_perm(const __half *p) {
    uint4 r;
    r.x = (uint32_t)__half_as_ushort(p[0]) | ((uint32_t)__half_as_ushort(p[2]) << 16);
    r.y = (uint32_t)__half_as_ushort(p[1]) | ((uint32_t)__half_as_ushort(p[3]) << 16);
    r.z = (uint32_t)__half_as_ushort(p[4]) | ((uint32_t)__half_as_ushort(p[6]) << 16);
    r.w = (uint32_t)__half_as_ushort(p[5]) | ((uint32_t)__half_as_ushort(p[7]) << 16);
    return r;
}

// One warp per (activation row, superblock); lane l owns the eight values at 256 b + 8 l.
__global__ void __launch_bounds__(128)
k_prep_x(const float *__restrict__ x, uint32_t cols, uint32_t xrows, uint32_t rows_per_group, PrepLayout L,
         uint8_t *__restrict__ out) {
    pdl_trigger();
    pdl_wait();
    const uint32_t warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    const uint32_t xr = warp / L.nblk, b = warp % L.nblk;
    if (xr >= xrows) return;
    const uint32_t group = xr / rows_per_group, tok = xr % rows_per_group;
    const float4 *src = reinterpret_cast<const float4 *>(x + (size_t)xr * cols + (size_t)b * 256 + lane * 8);
    const float4 v0 = src[0], v1 = src[1];
    float v[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 8; i++) amax = fmaxf(amax, fabsf(v[i]));
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
    // s = 2^e with amax * s in [512, 1024); 1 when the block is all zero or not finite.
    int e = 0;
    if (amax > 0.f && amax < INFINITY) {
        int ex;
        frexpf(amax, &ex);
        e = max(-100, min(100, 10 - ex));
    }
    const float s = ldexpf(1.f, e), inv = ldexpf(1.f, -e);
    __half hi[8], lo[8];
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const float xs = v[i] * s;
        hi[i] = __float2half_rn(xs);
        lo[i] = __float2half_rn(xs - __half2float(hi[i]));
        sum += xs;
    }
    uint8_t *base = out + (size_t)group * L.group_bytes;
    uint32_t t, u;
    if (L.fmt == FQ_Q4_K) {
        t = lane >> 3;
        u = lane & 7; // 4 h + q
    } else {
        t = (lane >> 4) * 2 + ((lane >> 1) & 1);
        u = ((lane >> 2) & 3) * 2 + (lane & 1); // 2 i + v
    }
    const uint32_t col_hi = tok, col_lo = L.split ? tok + 4 : tok;
    uint4 *xh = reinterpret_cast<uint4 *>(base), *xl = reinterpret_cast<uint4 *>(base + (L.split ? 0 : L.x1_off));
    xh[(((size_t)b * 8 + u) * L.cols_n + col_hi) * 4 + t] = pack_perm(hi);
    xl[(((size_t)b * 8 + u) * L.cols_n + col_lo) * 4 + t] = pack_perm(lo);
    if (L.fmt == FQ_Q4_K) {
        // Sub-block j = lane / 4 sums its four lanes; lane 8 t collects sub-blocks 2t and 2t + 1.
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        const float odd = __shfl_down_sync(0xffffffffu, sum, 4);
        if ((lane & 7) == 0) {
            const __half eh = __float2half_rn(sum), oh = __float2half_rn(odd);
            const __half el = __float2half_rn(sum - __half2float(eh)), ol = __float2half_rn(odd - __half2float(oh));
            uint32_t *s0 = reinterpret_cast<uint32_t *>(base + L.sx0_off);
            uint32_t *s1 = reinterpret_cast<uint32_t *>(base + (L.split ? L.sx0_off : L.sx1_off));
            s0[((size_t)b * L.cols_n + col_hi) * 4 + (lane >> 3)] = (uint32_t)__half_as_ushort(eh) | ((uint32_t)__half_as_ushort(oh) << 16);
            s1[((size_t)b * L.cols_n + col_lo) * 4 + (lane >> 3)] = (uint32_t)__half_as_ushort(el) | ((uint32_t)__half_as_ushort(ol) << 16);
        }
    }
    if (lane == 0) {
        float *isc = reinterpret_cast<float *>(base + L.isc_off);
        isc[(size_t)b * L.cols_n + col_hi] = inv;
        if (L.split) isc[(size_t)b * L.cols_n + col_lo] = inv;
    }
}

// ---------------------------------------------------------------- small device helpers

__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// The prepared activations are written by the kernel just before this one, which may still be running
// when this grid starts (programmatic dependent launch), so they are read with ordinary coherent
// loads after `pdl_wait`, never through the read-only path.
// (volatile: a load guarded by a condition must not be speculated for the lanes that skip it).
__device__ __forceinline__ uint4 ldg128(const void *p) {
    uint4 r;
    asm volatile("ld.global.ca.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
    return r;
}
__device__ __forceinline__ uint32_t ldg32(const void *p) {
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

__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t mask, uint32_t orv) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(mask), "r"(orv)); // (a & mask) | orv
    return r;
}
__device__ __forceinline__ uint32_t lop3_select(uint32_t a, uint32_t b, uint32_t mask) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xE4;" : "=r"(r) : "r"(a), "r"(b), "r"(mask)); // (a & mask) | (b & ~mask)
    return r;
}
__device__ __forceinline__ uint32_t hfma2_u32(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t r;
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
    return r;
}
__device__ __forceinline__ uint32_t hmul2_u32(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
__device__ __forceinline__ uint32_t h2_as_u32(__half2 v) { return *reinterpret_cast<uint32_t *>(&v); }
__device__ __forceinline__ uint32_t h2_bits(float v) { return h2_as_u32(__float2half2_rn(v)); }

// ---------------------------------------------------------------- Q4_K

// One superblock of one row as thread t needs it: the header and the 32 packed bytes of chunk t.
struct Q4Raw {
    uint4 hdr, qa, qb;
    __device__ __forceinline__ void load(const uint8_t *row, uint32_t /*nblk*/, uint32_t b, int t) {
        const uint8_t *blk = row + (size_t)b * 144;
        hdr = ldw128(blk);
        qa = ldw128(blk + 16 + 32 * t);
        qb = ldw128(blk + 32 + 32 * t);
    }
};

// Per (row, superblock) factors of the two sub-blocks thread t owns, kept packed.
struct Q4Scales {
    uint32_t sc;   // half2(sc_{2t}, sc_{2t+1})
    uint32_t mins; // half2(m_{2t}, m_{2t+1})
    float d, dmin;
};

__device__ __forceinline__ Q4Scales q4_scales(const uint4 hdr, int t) {
    const int sh = (t & 1) * 16;
    const uint32_t A = (hdr.y >> sh) & 0xFFFFu, B = (hdr.z >> sh) & 0xFFFFu, C = (hdr.w >> sh) & 0xFFFFu;
    uint32_t sc16, m16;
    if (t < 2) {
        sc16 = A & 0x3F3Fu;
        m16 = B & 0x3F3Fu;
    } else {
        sc16 = (C & 0x0F0Fu) | ((A >> 2) & 0x3030u);
        m16 = ((C >> 4) & 0x0F0Fu) | ((B >> 2) & 0x3030u);
    }
    // byte pair -> half2 of the two integers: each byte into the mantissa of 1024.0, minus 1024.
    const uint32_t k1024 = 0x64006400u;
    Q4Scales r;
    uint32_t scw = __byte_perm(sc16, 0, 0x4140) | k1024, mw = __byte_perm(m16, 0, 0x4140) | k1024;
    asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(r.sc) : "r"(scw), "r"(k1024));
    asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(r.mins) : "r"(mw), "r"(k1024));
    r.d = f16_bits_to_f32((uint16_t)(hdr.x & 0xFFFFu));
    r.dmin = f16_bits_to_f32((uint16_t)(hdr.x >> 16));
    return r;
}

// ---------------------------------------------------------------- Q6_K (device layout of blocks.cuh)

struct Q6Raw {
    uint4 q0, q1, qh; // ql of 32-groups 0|2 and 1|3 of half n, qh of half n: 16 values each (run lh)
    uint2 sc;         // the 8 scales of half n
    uint32_t d;       // f16 bits
    __device__ __forceinline__ void load(const uint8_t *row, uint32_t nblk, uint32_t b, int t) {
        const int n = t >> 1, lh = t & 1;
        const uint8_t *ql = row + (size_t)b * 128 + 64 * n + 16 * lh;
        q0 = ldw128(ql);
        q1 = ldw128(ql + 32);
        qh = ldw128(row + (size_t)nblk * 128 + (size_t)b * 64 + 32 * n + 16 * lh);
        sc = ldw64(row + (size_t)nblk * 192 + (size_t)b * 16 + 8 * n);
        d = ldw16(row + (size_t)nblk * 208 + (size_t)b * 2);
    }
};

// ---------------------------------------------------------------- the kernel
//
// FMT: FQ_Q4_K / FQ_Q6_K.  NT: 8-column tiles (1, or 2 for 9..16 activation rows).  RT: 16-row tiles
// per block.  SPLIT: hi / lo parts in columns c and c + 4 of one tile (M <= 4, NT = 1).
// Block = WARPS warps; warp w takes the superblocks b = w, w + WARPS, ...; partial sums meet in
// shared memory in a fixed order.  grid.x = ceil(rows / (16 RT)); grid.y = routes (expert mode) or 1.
// Up to MAX_TARGETS matrices of one format and width share the prepared activations and one launch
// (q|k|v, gate|up): block x covers row tiles [tile_end[i-1], tile_end[i]) of matrix i.
constexpr int MAX_TARGETS = 4;
struct GemvTargets {
    const uint8_t *w[MAX_TARGETS];
    float *y[MAX_TARGETS];
    uint32_t rows[MAX_TARGETS];
    uint32_t tile_end[MAX_TARGETS]; // in blocks of RT row tiles
    uint32_t count;
};

template <int FMT, int NT, int RT, bool SPLIT>
__global__ void __launch_bounds__(THREADS)
k_gemv(const __grid_constant__ GemvTargets T, uint32_t pitch, const uint8_t *__restrict__ prep, PrepLayout L, uint32_t m,
       const uint32_t *__restrict__ ids, uint32_t x_div, uint32_t experts) {
    uint32_t which = 0, first_block = 0;
#pragma unroll
    for (int i = 0; i < MAX_TARGETS - 1; i++)
        if ((uint32_t)i + 1 < T.count && blockIdx.x >= T.tile_end[i]) { which = i + 1; first_block = T.tile_end[i]; }
    const uint8_t *__restrict__ w = T.w[which];
    float *__restrict__ y = T.y[which];
    const uint32_t rows = T.rows[which];
    constexpr int ROWS = RT * 2;
    using Raw = std::conditional_t<FMT == FQ_Q4_K, Q4Raw, Q6Raw>;
    __shared__ float red[WARPS - 1][RT * NT * 4][32];

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    size_t y_base = 0;
    if (ids) { // expert mode: route r = blockIdx.y, one activation row per route
        pdl_wait(); // the routing that wrote `ids` must have completed
        const uint32_t r = blockIdx.y;
        const uint32_t e = ids[r];
        if (e >= experts) return;
        w += (size_t)e * rows * pitch;
        prep += (size_t)(r / x_div) * L.group_bytes;
        y_base = (size_t)r * rows;
    }
    const uint4 *x0 = reinterpret_cast<const uint4 *>(prep);
    const uint4 *x1 = reinterpret_cast<const uint4 *>(prep + L.x1_off);
    const uint32_t *sx0 = reinterpret_cast<const uint32_t *>(prep + L.sx0_off);
    const uint32_t *sx1 = reinterpret_cast<const uint32_t *>(prep + L.sx1_off);
    const float *isc = reinterpret_cast<const float *>(prep + L.isc_off);

    const uint32_t tile0 = (blockIdx.x - first_block) * RT;
    const uint8_t *rowp[ROWS];
#pragma unroll
    for (int rr = 0; rr < ROWS; rr++) {
        const uint32_t r = min((tile0 + (rr >> 1)) * 16 + g + (rr & 1) * 8, rows - 1);
        rowp[rr] = w + (size_t)r * pitch;
    }
    // Columns this thread feeds (B fragment, column 8 nt + g) and owns in the accumulators (2t, 2t+1).
    bool live[NT];
#pragma unroll
    for (int nt = 0; nt < NT; nt++) live[nt] = SPLIT ? (uint32_t)(g & 3) < m : (uint32_t)(8 * nt + g) < m;

    // Columns nothing was prepared for are never read (their accumulators stay zero).
    auto col_live = [&](uint32_t c) { return SPLIT ? (c & 3u) < m : c < m; };

    const uint32_t nblk = L.nblk;
    const uint32_t iters = nblk > (uint32_t)warp ? (nblk - warp + WARPS - 1) / WARPS : 0;
    // Superblock `it` of this warp; the index is clamped so the prefetch of the last iteration is a
    // harmless re-read instead of a branch.
    auto block_of = [&](uint32_t it) { return warp + min(it, iters - 1) * WARPS; };
    Raw cur[ROWS], nxt[ROWS];
    if (iters > 0) {
#pragma unroll
        for (int rr = 0; rr < ROWS; rr++) cur[rr].load(rowp[rr], nblk, block_of(0), t);
    }
    // The weight loads above touch immutable data only; everything below reads the prepared
    // activations and writes y, so it waits for the preceding kernels.
    pdl_trigger();
    pdl_wait();

    float yacc[RT][NT][4];
#pragma unroll
    for (int rt = 0; rt < RT; rt++)
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
#pragma unroll
            for (int i = 0; i < 4; i++) yacc[rt][nt][i] = 0.f;

    for (uint32_t it = 0; it < iters; it++) {
        const uint32_t b = warp + it * WARPS;
        // Next superblock's weights first (HBM latency), then all of this superblock's activation
        // fragments, sums and scales (L1 / L2 latency), then the arithmetic on the current registers.
#pragma unroll
        for (int rr = 0; rr < ROWS; rr++) nxt[rr].load(rowp[rr], nblk, block_of(it + 1), t);
        uint4 bfrag[SPLIT ? 1 : 2][8][NT];
        uint32_t sfrag[SPLIT ? 1 : 2][NT];
        float inv[NT][2];
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
#pragma unroll
            for (int u = 0; u < 8; u++) {
                const size_t unit = (((size_t)b * 8 + u) * L.cols_n + 8 * nt + g) * 4 + t;
                bfrag[0][u][nt] = live[nt] ? ldg128(x0 + unit) : make_uint4(0, 0, 0, 0);
                if (!SPLIT) bfrag[SPLIT ? 0 : 1][u][nt] = live[nt] ? ldg128(x1 + unit) : make_uint4(0, 0, 0, 0);
            }
            if (FMT == FQ_Q4_K) {
                const size_t unit = ((size_t)b * L.cols_n + 8 * nt + g) * 4 + t;
                sfrag[0][nt] = live[nt] ? ldg32(sx0 + unit) : 0u;
                if (!SPLIT) sfrag[SPLIT ? 0 : 1][nt] = live[nt] ? ldg32(sx1 + unit) : 0u;
            }
            const uint32_t c0 = 8 * nt + 2 * t;
            inv[nt][0] = col_live(c0) ? __uint_as_float(ldg32(isc + (size_t)b * L.cols_n + c0)) : 0.f;
            inv[nt][1] = col_live(c0 + 1) ? __uint_as_float(ldg32(isc + (size_t)b * L.cols_n + c0 + 1)) : 0.f;
        }

        float acc[RT][NT][4];
#pragma unroll
        for (int rt = 0; rt < RT; rt++)
#pragma unroll
            for (int nt = 0; nt < NT; nt++)
#pragma unroll
                for (int i = 0; i < 4; i++) acc[rt][nt][i] = 0.f;

        if constexpr (FMT == FQ_Q4_K) {
            Q4Scales rs[ROWS];
#pragma unroll
            for (int rr = 0; rr < ROWS; rr++) rs[rr] = q4_scales(cur[rr].hdr, t);
#pragma unroll
            for (int h = 0; h < 2; h++) { // low nibbles (sub-block 2t), then high nibbles (sub-block 2t + 1)
                const uint32_t mask = h ? 0x00F000F0u : 0x000F000Fu;
                uint32_t scv[ROWS], bias[ROWS];
#pragma unroll
                for (int rr = 0; rr < ROWS; rr++) {
                    // low nibbles: q * sc = (1024 + q) * sc - 1024 sc;  high nibbles, read in place as
                    // 16 q:  (1024 + 16 q) * (sc / 16) - 64 sc
                    const uint32_t s2 = h ? __byte_perm(rs[rr].sc, 0, 0x3232) : __byte_perm(rs[rr].sc, 0, 0x1010);
                    scv[rr] = h ? hmul2_u32(s2, h2_bits(0.0625f)) : s2;
                    bias[rr] = hmul2_u32(s2, h ? h2_bits(-64.f) : h2_bits(-1024.f));
                }
#pragma unroll
                for (int half = 0; half < 2; half++) { // bytes 0..15 / 16..31 of the chunk: pieces q = 2 half, 2 half + 1
                    uint4 qw[ROWS];
#pragma unroll
                    for (int rr = 0; rr < ROWS; rr++) qw[rr] = half ? cur[rr].qb : cur[rr].qa;
#pragma unroll
                    for (int qq = 0; qq < 2; qq++) {
                        const int u = 4 * h + 2 * half + qq;
#pragma unroll
                        for (int rt = 0; rt < RT; rt++) {
#pragma unroll
                            for (int jj = 0; jj < 2; jj++) {
                                uint32_t a[4];
#pragma unroll
                                for (int r = 0; r < 2; r++) {
                                    const uint4 &src = qw[rt * 2 + r];
                                    const int wi = qq * 2 + jj;
                                    const uint32_t wd = wi == 0 ? src.x : wi == 1 ? src.y : wi == 2 ? src.z : src.w;
                                    a[r] = hfma2_u32(lop3_and_or(wd, mask, 0x64006400u), scv[rt * 2 + r], bias[rt * 2 + r]);
                                    a[2 + r] = hfma2_u32(lop3_and_or(wd >> 8, mask, 0x64006400u), scv[rt * 2 + r], bias[rt * 2 + r]);
                                }
#pragma unroll
                                for (int nt = 0; nt < NT; nt++) {
                                    const uint4 &bh = bfrag[0][h * 4 + 2 * half + qq][nt];
                                    mma16816(acc[rt][nt], a[0], a[1], a[2], a[3], jj ? bh.z : bh.x, jj ? bh.w : bh.y);
                                    if (!SPLIT) {
                                        const uint4 &bl = bfrag[SPLIT ? 0 : 1][h * 4 + 2 * half + qq][nt];
                                        mma16816(acc[rt][nt], a[0], a[1], a[2], a[3], jj ? bl.z : bl.x, jj ? bl.w : bl.y);
                                    }
                                }
                            }
                        }
                        (void)u;
                    }
                }
            }
            // Minimum term and per-superblock factors.
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                const uint32_t s_hi = sfrag[0][nt], s_lo = sfrag[SPLIT ? 0 : 1][nt];
                const float inv0 = inv[nt][0], inv1 = inv[nt][1];
#pragma unroll
                for (int rt = 0; rt < RT; rt++) {
                    float cm[4] = {0.f, 0.f, 0.f, 0.f};
                    mma16816(cm, rs[rt * 2].mins, rs[rt * 2 + 1].mins, 0u, 0u, s_hi, 0u);
                    if (!SPLIT) mma16816(cm, rs[rt * 2].mins, rs[rt * 2 + 1].mins, 0u, 0u, s_lo, 0u);
                    const float *c = acc[rt][nt];
                    const Q4Scales &r0 = rs[rt * 2], &r1 = rs[rt * 2 + 1];
                    yacc[rt][nt][0] = fmaf(inv0, r0.d * c[0] - r0.dmin * cm[0], yacc[rt][nt][0]);
                    yacc[rt][nt][1] = fmaf(inv1, r0.d * c[1] - r0.dmin * cm[1], yacc[rt][nt][1]);
                    yacc[rt][nt][2] = fmaf(inv0, r1.d * c[2] - r1.dmin * cm[2], yacc[rt][nt][2]);
                    yacc[rt][nt][3] = fmaf(inv1, r1.d * c[3] - r1.dmin * cm[3], yacc[rt][nt][3]);
                }
            }
        } else {
            // Q6_K.  Thread t = (n, lh) owns, for i = 0..3, the values 128 n + 32 i + 16 lh + [0, 16).
            const int lh = t & 1;
            uint32_t scv[ROWS][4], bias[ROWS][4];
            float dd[ROWS];
#pragma unroll
            for (int rr = 0; rr < ROWS; rr++) {
                const uint2 s = cur[rr].sc;
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    // scale byte lh + 2 i of the half: word i / 2, byte 2 (i % 2) + lh
                    const uint32_t wsel = (i < 2) ? s.x : s.y;
                    const int sc = (int)(int8_t)((wsel >> (16 * (i & 1) + 8 * lh)) & 0xFFu);
                    const __half hs = __int2half_rn(sc);
                    const __half2 s2 = __half2half2(hs);
                    scv[rr][i] = h2_as_u32(s2);
                    // (64 + q) * sc - 96 sc = (q - 32) * sc;  96 sc is exact in f16
                    bias[rr][i] = hmul2_u32(h2_as_u32(s2), h2_bits(-96.f));
                }
                dd[rr] = f16_bits_to_f32((uint16_t)cur[rr].d);
            }
#pragma unroll
            for (int i = 0; i < 4; i++) {
#pragma unroll
                for (int v = 0; v < 2; v++) { // words 2v, 2v + 1: values 8 v .. 8 v + 7 of the run
                    const int u = 2 * i + v;
#pragma unroll
                    for (int rt = 0; rt < RT; rt++) {
#pragma unroll
                        for (int jj = 0; jj < 2; jj++) {
                            const int wi = 2 * v + jj;
                            uint32_t a[4];
#pragma unroll
                            for (int r = 0; r < 2; r++) {
                                const int rr = rt * 2 + r;
                                const uint4 &l4 = (i & 1) ? cur[rr].q1 : cur[rr].q0;
                                const uint32_t lw = wi == 0 ? l4.x : wi == 1 ? l4.y : wi == 2 ? l4.z : l4.w;
                                const uint4 &h4 = cur[rr].qh;
                                const uint32_t hw = wi == 0 ? h4.x : wi == 1 ? h4.y : wi == 2 ? h4.z : h4.w;
                                // four 6-bit values, one per byte (bits 6, 7 of each byte are junk, masked below)
                                const uint32_t lo4 = (i < 2) ? lw : (lw >> 4);
                                const uint32_t hi4 = i == 0 ? (hw << 4) : i == 1 ? (hw << 2) : i == 2 ? hw : (hw >> 2);
                                const uint32_t v4 = lop3_select(lo4, hi4, 0x0F0F0F0Fu);
                                // bytes 0, 2 and bytes 1, 3 into the mantissa of 64.0 (ulp 1/16): 64 + q
                                const uint32_t e02 = lop3_and_or(v4 << 4, 0x03F003F0u, 0x54005400u);
                                const uint32_t e13 = lop3_and_or(v4 >> 4, 0x03F003F0u, 0x54005400u);
                                a[r] = hfma2_u32(e02, scv[rr][i], bias[rr][i]);
                                a[2 + r] = hfma2_u32(e13, scv[rr][i], bias[rr][i]);
                            }
#pragma unroll
                            for (int nt = 0; nt < NT; nt++) {
                                const uint4 &bh = bfrag[0][u][nt];
                                mma16816(acc[rt][nt], a[0], a[1], a[2], a[3], jj ? bh.z : bh.x, jj ? bh.w : bh.y);
                                if (!SPLIT) {
                                    const uint4 &bl = bfrag[SPLIT ? 0 : 1][u][nt];
                                    mma16816(acc[rt][nt], a[0], a[1], a[2], a[3], jj ? bl.z : bl.x, jj ? bl.w : bl.y);
                                }
                            }
                        }
                    }
                }
            }
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                const float inv0 = inv[nt][0], inv1 = inv[nt][1];
#pragma unroll
                for (int rt = 0; rt < RT; rt++) {
                    const float *c = acc[rt][nt];
                    yacc[rt][nt][0] = fmaf(inv0 * dd[rt * 2], c[0], yacc[rt][nt][0]);
                    yacc[rt][nt][1] = fmaf(inv1 * dd[rt * 2], c[1], yacc[rt][nt][1]);
                    yacc[rt][nt][2] = fmaf(inv0 * dd[rt * 2 + 1], c[2], yacc[rt][nt][2]);
                    yacc[rt][nt][3] = fmaf(inv1 * dd[rt * 2 + 1], c[3], yacc[rt][nt][3]);
                }
            }
        }
#pragma unroll
        for (int rr = 0; rr < ROWS; rr++) cur[rr] = nxt[rr];
    }
    // Warps 1.. hand their partial sums to warp 0, which adds them in warp order, so the result does
    // not depend on timing.
    if (warp > 0) {
#pragma unroll
        for (int rt = 0; rt < RT; rt++)
#pragma unroll
            for (int nt = 0; nt < NT; nt++)
#pragma unroll
                for (int i = 0; i < 4; i++) red[warp - 1][(rt * NT + nt) * 4 + i][lane] = yacc[rt][nt][i];
    }
    __syncthreads();
    if (warp == 0) {
#pragma unroll
        for (int rt = 0; rt < RT; rt++)
#pragma unroll
            for (int nt = 0; nt < NT; nt++)
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    float v = yacc[rt][nt][i];
#pragma unroll
                    for (int ww = 0; ww < WARPS - 1; ww++) v += red[ww][(rt * NT + nt) * 4 + i][lane];
                    if (SPLIT) v += __shfl_xor_sync(0xffffffffu, v, 2); // column c (hi) + column c + 4 (lo)
                    const uint32_t row = (tile0 + rt) * 16 + g + (i >> 1) * 8;
                    const uint32_t tok = 8 * nt + 2 * t + (i & 1);
                    if (row < rows && tok < m && (!SPLIT || t < 2)) y[y_base + (size_t)tok * rows + row] = v;
                }
    }
}

template <typename... KArgs, typename... Args>
cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    // FQ_PDL=0 turns programmatic dependent launch off (plain stream order), for A/B measurements.
    static const bool pdl = [] { const char *e = getenv("FQ_PDL"); return !(e && e[0] == '0'); }();
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

template <int FMT, int NT, int RT, bool SPLIT>
int launch(fq_device *dev, const ProjectArgs *a, uint32_t count, const uint8_t *prep, const PrepLayout &L, uint32_t m, bool expert) {
    GemvTargets T{};
    T.count = count;
    uint32_t blocks = 0;
    for (uint32_t i = 0; i < count; i++) {
        T.w[i] = a[i].w;
        T.y[i] = (float *)a[i].y;
        T.rows[i] = a[i].rows;
        blocks += (a[i].rows + 16 * RT - 1) / (16 * RT);
        T.tile_end[i] = blocks;
    }
    dim3 grid(blocks, expert ? a[0].m : 1);
    cudaError_t e = launch_pdl(k_gemv<FMT, NT, RT, SPLIT>, grid, dim3(THREADS), 0, dev->stream, T, a[0].row_bytes, prep, L, m,
                               a[0].ids, a[0].x_div, a[0].experts);
    return fq_check_cuda(dev, e, "gemv launch");
}

} // namespace

size_t fq_gemv_scratch_bytes() { return (size_t)96 << 20; }

// `a[0..count)` share x, m, format and width (checked here); expert mode takes one matrix.
int fq_launch_gemv_fast_many(fq_device *dev, const ProjectArgs *a, uint32_t count) {
    if (count == 0 || count > (uint32_t)MAX_TARGETS) return FQ_ERR_UNSUPPORTED;
    const ProjectArgs &f = a[0];
    if ((f.format != FQ_Q4_K && f.format != FQ_Q6_K) || f.x_dtype != FQ_F32 || f.y_dtype != FQ_F32) return FQ_ERR_UNSUPPORTED;
    if (f.cols % 256 || f.row_bytes % 16) return FQ_ERR_UNSUPPORTED;
    for (uint32_t i = 1; i < count; i++)
        if (a[i].format != f.format || a[i].cols != f.cols || a[i].x != f.x || a[i].m != f.m || a[i].ids || f.ids ||
            a[i].x_dtype != FQ_F32 || a[i].y_dtype != FQ_F32)
            return FQ_ERR_UNSUPPORTED;
    const bool expert = f.ids != nullptr;
    uint32_t xrows, rows_per_group, m;
    if (expert) {
        if (f.m > 65535) return FQ_ERR_UNSUPPORTED;
        xrows = f.m / f.x_div; // the caller checked that x holds routes / x_div rows
        rows_per_group = 1;
        m = 1;
    } else {
        if (f.m > (uint32_t)FQ_GEMV_MAX_M) return FQ_ERR_UNSUPPORTED;
        xrows = f.m;
        rows_per_group = f.m;
        m = f.m;
    }
    const bool split = m <= 4;
    const uint32_t cols_n = m <= 8 ? 8 : 16;
    const PrepLayout L = prep_layout(f.format, f.cols, cols_n, split);
    const size_t groups = expert ? xrows : 1;
    // Successive projections use alternate halves of the scratch, so a preparation kernel that starts
    // early never writes what the previous projection may still be reading from a cache.
    if (groups * L.group_bytes > dev->xprep_bytes / 2) return FQ_ERR_UNSUPPORTED;
    dev->xprep_turn ^= 1u;
    uint8_t *prep = (uint8_t *)dev->xprep + (dev->xprep_turn ? dev->xprep_bytes / 2 : 0);
    const uint32_t warps = xrows * L.nblk;
    if (int rc = fq_check_cuda(dev, launch_pdl(k_prep_x, dim3((warps + 3) / 4), dim3(128), 0, dev->stream, (const float *)f.x,
                                               f.cols, xrows, rows_per_group, L, prep), "prep launch"))
        return rc;
    int rc;
    if (f.format == FQ_Q4_K) {
        if (split) rc = launch<FQ_Q4_K, 1, 1, true>(dev, a, count, prep, L, m, expert);
        else if (m <= 8) rc = launch<FQ_Q4_K, 1, 1, false>(dev, a, count, prep, L, m, expert);
        else rc = launch<FQ_Q4_K, 2, 1, false>(dev, a, count, prep, L, m, expert);
    } else {
        if (split) rc = launch<FQ_Q6_K, 1, 1, true>(dev, a, count, prep, L, m, expert);
        else if (m <= 8) rc = launch<FQ_Q6_K, 1, 1, false>(dev, a, count, prep, L, m, expert);
        else rc = launch<FQ_Q6_K, 2, 1, false>(dev, a, count, prep, L, m, expert);
    }
    if (rc != FQ_OK) return rc;
    return fq_end_enqueue(dev, "gemv", 2);
}

int fq_launch_gemv_fast(fq_device *dev, const ProjectArgs &a) { return fq_launch_gemv_fast_many(dev, &a, 1); }
