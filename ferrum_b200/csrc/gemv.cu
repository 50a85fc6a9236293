// Decode / speculative-verify projections (M = 1..16, F32 in, F32 out) with the packed weights
// streamed once.  The work of `h_mv_*`, `h_mvb_*` and `h_mms_*` in the reference
// (src/metal/shaders/hybrid.metal:688-756, 1330-1394, 1419-1495).
//
// On B200 a Q4_K GEMV is bound by instruction issue before HBM, so the multiply runs on the
// tensor cores even at M = 1 (warp-level mma.sync m16n8k16, f16 operands, fp32 accumulators in
// registers):
//
//   A (16 weight rows x 16 k)  = sc * q as exact f16 integers (<= 63 * 15), built from the packed
//                                nibbles with one LOP3 + one HFMA2 per two weights;
//   B (16 k x 8 activation rows) = the activations as f16, split x = hi + lo so the product keeps
//                                fp32-level accuracy (two MMAs);
//   per superblock:  y += (1/s) * (d * acc - dmin * sum_j m_j * Sx_j)
//
// which is the factored form of the reference's `mv_q4_K` (d*sc*sum(q x) - dmin*m*sum(x)).  A small
// preparation kernel turns the fp32 activations into the B fragments (already in the register
// order of the MMA), the per-32 sums Sx and a power-of-two scale s per (activation row, superblock)
// that keeps every f16 operand in range whatever the magnitude of x.
//
// Thread (g = lane / 4, t = lane % 4) of a warp owns weight rows g and g + 8 of a 16-row tile and,
// inside a superblock, the 32 packed bytes of chunk t (values 64t .. 64t+63: low nibbles are
// sub-block 2t, high nibbles sub-block 2t + 1), which it reads with two 128-bit loads.  The MMA's
// k order is free as long as A and B agree, so nothing is shuffled between lanes.
#include "blocks.cuh"
#include "internal.h"

namespace {

constexpr int WARPS = 4; // warps of a thread block split K between them

// Layout of the prepared activations for one group of TP activation rows (all offsets in bytes):
//   xh   [nblk][2 h][4 q][TP][4 t] x 16 B   f16 "hi" parts, unit (b,h,q,tok,t) holds the values at
//        k0 = 256 b + 64 t + 32 h + 8 q in the order k0+{0,2,1,3,4,6,5,7}
//   xl   the same for the "lo" parts
//   sx   [nblk][TP][4 t] x 8 B             half2 hi (Sx of sub-blocks 2t, 2t+1), half2 lo
//   isc  [nblk][TP] x 4 B                  1 / s
struct PrepLayout {
    uint32_t nblk, tp;
    size_t xl_off, sx_off, isc_off, group_bytes;
};

__host__ __device__ inline PrepLayout prep_layout(uint32_t cols, uint32_t tp) {
    PrepLayout L;
    L.nblk = cols / 256;
    L.tp = tp;
    const size_t xbytes = (size_t)L.nblk * 8 * tp * 4 * 16;
    L.xl_off = xbytes;
    L.sx_off = 2 * xbytes;
    L.isc_off = L.sx_off + (size_t)L.nblk * tp * 4 * 8;
    L.group_bytes = (L.isc_off + (size_t)L.nblk * tp * 4 + 255) & ~(size_t)255;
    return L;
}

// One warp per (activation row, superblock).
__global__ void __launch_bounds__(128)
k_prep_x(const float *__restrict__ x, uint32_t cols, uint32_t xrows, uint32_t rows_per_group, PrepLayout L,
         uint8_t *__restrict__ out) {
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
    const uint32_t t = lane >> 3, h = (lane >> 2) & 1, q = lane & 3;
    const size_t unit = ((((size_t)b * 2 + h) * 4 + q) * L.tp + tok) * 4 + t;
    auto pack = [](const __half *p) {
        uint4 r;
        r.x = (uint32_t)__half_as_ushort(p[0]) | ((uint32_t)__half_as_ushort(p[2]) << 16);
        r.y = (uint32_t)__half_as_ushort(p[1]) | ((uint32_t)__half_as_ushort(p[3]) << 16);
        r.z = (uint32_t)__half_as_ushort(p[4]) | ((uint32_t)__half_as_ushort(p[6]) << 16);
        r.w = (uint32_t)__half_as_ushort(p[5]) | ((uint32_t)__half_as_ushort(p[7]) << 16);
        return r;
    };
    reinterpret_cast<uint4 *>(base)[unit] = pack(hi);
    reinterpret_cast<uint4 *>(base + L.xl_off)[unit] = pack(lo);
    // Sub-block j = lane / 4 sums its four lanes.
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    const float odd = __shfl_down_sync(0xffffffffu, sum, 4); // sub-block j + 1
    if ((lane & 7) == 0) {
        const __half eh = __float2half_rn(sum), oh = __float2half_rn(odd);
        const __half el = __float2half_rn(sum - __half2float(eh)), ol = __float2half_rn(odd - __half2float(oh));
        uint2 r;
        r.x = (uint32_t)__half_as_ushort(eh) | ((uint32_t)__half_as_ushort(oh) << 16);
        r.y = (uint32_t)__half_as_ushort(el) | ((uint32_t)__half_as_ushort(ol) << 16);
        reinterpret_cast<uint2 *>(base + L.sx_off)[((size_t)b * L.tp + tok) * 4 + t] = r;
    }
    if (lane == 0) reinterpret_cast<float *>(base + L.isc_off)[(size_t)b * L.tp + tok] = inv;
}

__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ldg128(const void *p) {
    uint4 r;
    asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
    return r;
}

__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t mask, uint32_t orv) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(mask), "r"(orv)); // (a & mask) | orv
    return r;
}

__device__ __forceinline__ uint32_t hfma2_u32(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t r;
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
    return r;
}

__device__ __forceinline__ uint32_t h2_as_u32(__half2 v) { return *reinterpret_cast<uint32_t *>(&v); }

// Per (row, superblock) factors of the two sub-blocks thread t owns.
struct RowScales {
    uint32_t sc_lo, bias_lo; // half2(sc_{2t}), half2(-1024 sc_{2t})       : low nibbles
    uint32_t sc_hi, bias_hi; // half2(sc_{2t+1} / 16), half2(-64 sc_{2t+1}) : high nibbles, read in place
    uint32_t mins;           // half2(m_{2t}, m_{2t+1})
    float d, dmin;
};

__device__ __forceinline__ RowScales row_scales(const uint4 hdr, int t) {
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
    // byte pair -> half2 of the two integers: place each byte in a mantissa of 1024.0, subtract 1024.
    const __half2 k1024 = __float2half2_rn(1024.f);
    uint32_t scw = __byte_perm(sc16, 0, 0x4140) | 0x64006400u;
    uint32_t mw = __byte_perm(m16, 0, 0x4140) | 0x64006400u;
    const __half2 sc = __hsub2(*reinterpret_cast<__half2 *>(&scw), k1024);
    const __half2 mn = __hsub2(*reinterpret_cast<__half2 *>(&mw), k1024);
    const __half2 s_lo = __low2half2(sc), s_hi = __high2half2(sc);
    RowScales r;
    r.sc_lo = h2_as_u32(s_lo);
    r.bias_lo = h2_as_u32(__hmul2(s_lo, __float2half2_rn(-1024.f)));
    r.sc_hi = h2_as_u32(__hmul2(s_hi, __float2half2_rn(0.0625f)));
    r.bias_hi = h2_as_u32(__hmul2(s_hi, __float2half2_rn(-64.f)));
    r.mins = h2_as_u32(mn);
    r.d = f16_bits_to_f32((uint16_t)(hdr.x & 0xFFFFu));
    r.dmin = f16_bits_to_f32((uint16_t)(hdr.x >> 16));
    return r;
}

// Q4_K, M <= 8 * NT.  Block = WARPS warps sharing RT row tiles of 16 rows; warp w takes the
// superblocks b = w, w + WARPS, ...; partial sums meet in shared memory.
// grid.x = ceil(rows / (16 RT)); grid.y = routes (expert mode) or 1.
template <int NT, int RT>
__global__ void __launch_bounds__(WARPS * 32)
k_gemv_q4k(const uint8_t *__restrict__ w, uint32_t rows, uint32_t row_bytes, const uint8_t *__restrict__ prep,
           PrepLayout L, float *__restrict__ y, uint32_t m, const uint32_t *__restrict__ ids, uint32_t x_div,
           uint32_t experts) {
    __shared__ float red[WARPS - 1][RT * NT * 4][32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    size_t y_base = 0;
    uint32_t y_stride = rows;
    if (ids) { // expert mode: route r = blockIdx.y, one activation row per route
        const uint32_t r = blockIdx.y;
        const uint32_t e = ids[r];
        if (e >= experts) return;
        w += (size_t)e * rows * row_bytes;
        prep += (size_t)(r / x_div) * L.group_bytes;
        y_base = (size_t)r * rows;
    }
    const uint4 *xh = reinterpret_cast<const uint4 *>(prep);
    const uint4 *xl = reinterpret_cast<const uint4 *>(prep + L.xl_off);
    const uint2 *sx = reinterpret_cast<const uint2 *>(prep + L.sx_off);
    const float *isc = reinterpret_cast<const float *>(prep + L.isc_off);

    const uint32_t tile0 = blockIdx.x * RT;
    const uint8_t *rowp[RT][2];
#pragma unroll
    for (int rt = 0; rt < RT; rt++) {
        const uint32_t r0 = min((tile0 + rt) * 16 + g, rows - 1), r1 = min((tile0 + rt) * 16 + g + 8, rows - 1);
        rowp[rt][0] = w + (size_t)r0 * row_bytes;
        rowp[rt][1] = w + (size_t)r1 * row_bytes;
    }
    float yacc[RT][NT][4];
#pragma unroll
    for (int rt = 0; rt < RT; rt++)
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
#pragma unroll
            for (int i = 0; i < 4; i++) yacc[rt][nt][i] = 0.f;
    bool live[NT];
#pragma unroll
    for (int nt = 0; nt < NT; nt++) live[nt] = (uint32_t)(8 * nt + g) < m;

    for (uint32_t b = warp; b < L.nblk; b += WARPS) {
        uint4 hdr[RT][2], qa[RT][2], qb[RT][2];
#pragma unroll
        for (int rt = 0; rt < RT; rt++)
#pragma unroll
            for (int r = 0; r < 2; r++) {
                const uint8_t *blk = rowp[rt][r] + (size_t)b * 144;
                hdr[rt][r] = ldg128(blk);
                qa[rt][r] = ldg128(blk + 16 + 32 * t);
                qb[rt][r] = ldg128(blk + 32 + 32 * t);
            }
        RowScales rs[RT][2];
        float acc[RT][NT][4];
#pragma unroll
        for (int rt = 0; rt < RT; rt++) {
            rs[rt][0] = row_scales(hdr[rt][0], t);
            rs[rt][1] = row_scales(hdr[rt][1], t);
#pragma unroll
            for (int nt = 0; nt < NT; nt++)
#pragma unroll
                for (int i = 0; i < 4; i++) acc[rt][nt][i] = 0.f;
        }
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const uint32_t mask = h ? 0x00F000F0u : 0x000F000Fu;
#pragma unroll
            for (int q = 0; q < 4; q++) {
                uint4 bh[NT], bl[NT];
#pragma unroll
                for (int nt = 0; nt < NT; nt++) {
                    bh[nt] = make_uint4(0, 0, 0, 0);
                    bl[nt] = make_uint4(0, 0, 0, 0);
                    if (live[nt]) {
                        const size_t unit = ((((size_t)b * 2 + h) * 4 + q) * L.tp + 8 * nt + g) * 4 + t;
                        bh[nt] = ldg128(xh + unit);
                        bl[nt] = ldg128(xl + unit);
                    }
                }
#pragma unroll
                for (int rt = 0; rt < RT; rt++) {
#pragma unroll
                    for (int jj = 0; jj < 2; jj++) { // the two words of piece q
                        uint32_t wd[2];
#pragma unroll
                        for (int r = 0; r < 2; r++) {
                            const uint4 &src = (q < 2) ? qa[rt][r] : qb[rt][r];
                            const int wi = (q & 1) * 2 + jj;
                            wd[r] = wi == 0 ? src.x : wi == 1 ? src.y : wi == 2 ? src.z : src.w;
                        }
                        uint32_t a[4];
#pragma unroll
                        for (int r = 0; r < 2; r++) {
                            const uint32_t sc = h ? rs[rt][r].sc_hi : rs[rt][r].sc_lo;
                            const uint32_t bias = h ? rs[rt][r].bias_hi : rs[rt][r].bias_lo;
                            a[r] = hfma2_u32(lop3_and_or(wd[r], mask, 0x64006400u), sc, bias);          // bytes 0, 2
                            a[2 + r] = hfma2_u32(lop3_and_or(wd[r] >> 8, mask, 0x64006400u), sc, bias); // bytes 1, 3
                        }
#pragma unroll
                        for (int nt = 0; nt < NT; nt++) {
                            const uint32_t bh0 = jj ? bh[nt].z : bh[nt].x, bh1 = jj ? bh[nt].w : bh[nt].y;
                            const uint32_t bl0 = jj ? bl[nt].z : bl[nt].x, bl1 = jj ? bl[nt].w : bl[nt].y;
                            mma16816(acc[rt][nt], a[0], a[1], a[2], a[3], bh0, bh1);
                            mma16816(acc[rt][nt], a[0], a[1], a[2], a[3], bl0, bl1);
                        }
                    }
                }
            }
        }
        // Minimum term and per-superblock factors.
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
            uint2 s2 = make_uint2(0, 0);
            if (live[nt]) s2 = sx[((size_t)b * L.tp + 8 * nt + g) * 4 + t];
            float inv0 = 0.f, inv1 = 0.f;
            const uint32_t tok = 8 * nt + 2 * t;
            if (tok < m) inv0 = isc[(size_t)b * L.tp + tok];
            if (tok + 1 < m) inv1 = isc[(size_t)b * L.tp + tok + 1];
#pragma unroll
            for (int rt = 0; rt < RT; rt++) {
                float cm[4] = {0.f, 0.f, 0.f, 0.f};
                mma16816(cm, rs[rt][0].mins, rs[rt][1].mins, 0u, 0u, s2.x, 0u);
                mma16816(cm, rs[rt][0].mins, rs[rt][1].mins, 0u, 0u, s2.y, 0u);
                const float *c = acc[rt][nt];
                yacc[rt][nt][0] = fmaf(inv0, rs[rt][0].d * c[0] - rs[rt][0].dmin * cm[0], yacc[rt][nt][0]);
                yacc[rt][nt][1] = fmaf(inv1, rs[rt][0].d * c[1] - rs[rt][0].dmin * cm[1], yacc[rt][nt][1]);
                yacc[rt][nt][2] = fmaf(inv0, rs[rt][1].d * c[2] - rs[rt][1].dmin * cm[2], yacc[rt][nt][2]);
                yacc[rt][nt][3] = fmaf(inv1, rs[rt][1].d * c[3] - rs[rt][1].dmin * cm[3], yacc[rt][nt][3]);
            }
        }
    }
    // Warps 1.. hand their partial sums to warp 0 in a fixed order, so the result does not depend
    // on timing.
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
                    const uint32_t row = (tile0 + rt) * 16 + g + (i >> 1) * 8;
                    const uint32_t tok = 8 * nt + 2 * t + (i & 1);
                    if (row < rows && tok < m) y[y_base + (size_t)tok * y_stride + row] = v;
                }
    }
}

} // namespace

size_t fq_gemv_scratch_bytes() { return (size_t)32 << 20; }

int fq_launch_gemv_fast(fq_device *dev, const ProjectArgs &a) {
    if (a.format != FQ_Q4_K || a.x_dtype != FQ_F32 || a.y_dtype != FQ_F32) return FQ_ERR_UNSUPPORTED;
    if (a.cols % 256 || a.row_bytes % 16) return FQ_ERR_UNSUPPORTED;
    const bool expert = a.ids != nullptr;
    uint32_t xrows, rows_per_group, tp, m;
    if (expert) {
        if (a.m > 65535) return FQ_ERR_UNSUPPORTED;
        xrows = a.m / a.x_div; // checked by the caller: x holds routes / x_div rows
        rows_per_group = 1;
        tp = 1;
        m = 1;
    } else {
        if (a.m > (uint32_t)FQ_GEMV_MAX_M) return FQ_ERR_UNSUPPORTED;
        xrows = a.m;
        rows_per_group = a.m;
        tp = a.m == 1 ? 1 : (a.m <= 8 ? 8 : 16);
        m = a.m;
    }
    const PrepLayout L = prep_layout(a.cols, tp);
    const size_t groups = expert ? xrows : 1;
    if (groups * L.group_bytes > dev->xprep_bytes) return FQ_ERR_UNSUPPORTED;
    const uint32_t warps = xrows * L.nblk;
    k_prep_x<<<(warps + 3) / 4, 128, 0, dev->stream>>>((const float *)a.x, a.cols, xrows, rows_per_group, L,
                                                      (uint8_t *)dev->xprep);
    const uint8_t *prep = (const uint8_t *)dev->xprep;
    float *y = (float *)a.y;
    if (m <= 8) {
        constexpr int RT = 1;
        dim3 grid((a.rows + 16 * RT - 1) / (16 * RT), expert ? a.m : 1);
        k_gemv_q4k<1, RT><<<grid, WARPS * 32, 0, dev->stream>>>(a.w, a.rows, a.row_bytes, prep, L, y, m, a.ids, a.x_div,
                                                                a.experts);
    } else {
        constexpr int RT = 1;
        dim3 grid((a.rows + 16 * RT - 1) / (16 * RT), 1);
        k_gemv_q4k<2, RT><<<grid, WARPS * 32, 0, dev->stream>>>(a.w, a.rows, a.row_bytes, prep, L, y, m, a.ids, a.x_div,
                                                                a.experts);
    }
    return fq_end_enqueue(dev, "gemv_q4k", 2);
}
