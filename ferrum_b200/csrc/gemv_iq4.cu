// IQ4_NL / IQ4_XS decode projections for 1..4 activation rows per launch (F32 in, F32 out): the reference's
// `h_mv_iq4_nl` / `h_mv_iq4_xs` and their batched forms (src/metal/shaders/hybrid.metal:900-1000, 1317-1323,
// 1385).  The 4-bit indices go through the 16-entry codebook to signed bytes with byte permutes (four at a time,
// no memory lookup), and from there the arithmetic is that of the Q8_0 kernel (gemv_q8.cu): dp4a against the two
// byte planes of activations rounded to 16 bits per block of 32 -- the granularity of both formats' scales --
// one conversion and FMA with d (ls - 32) / s per sub-block.
//
// Device layout of a row (blocks.cuh): the nibbles of all blocks first (cols / 2 bytes, natural order), then per
// block the f16 d (IQ4_NL) or the 8 bytes d | scales_h | scales_l (IQ4_XS).  Byte j of a 16-byte run holds values
// j and j + 16 of its 32.
#include <algorithm>
#include <cstdlib>

#include "blocks.cuh"
#include "gemv_common.cuh"
#include "internal.h"

namespace {

constexpr int WARPS = 8;
constexpr uint32_t MAX_COLS_IQ4 = 16384; // 2 planes x 4 activation rows x cols bytes of shared memory

// Four codebook values for the four 4-bit indices of `n` (the low 16 bits: nibble i -> result byte i).
__device__ __forceinline__ uint32_t iq4_lookup4(uint32_t n) {
    // codebook bytes: entries 0-3, 4-7, 8-11, 12-15
    constexpr uint32_t T0 = 0xBFAD9881u, T1 = 0xF6EADDCFu, T2 = 0x26190D01u, T3 = 0x71594535u;
    const uint32_t low3 = n & 0x7777u; // a permute selector: three bits per result byte
    const uint32_t a = __byte_perm(T0, T1, low3), b = __byte_perm(T2, T3, low3);
    // bit 3 of an index picks the upper half of the codebook: byte i of the result comes from a (selector i) or b (4 + i)
    return __byte_perm(a, b, 0x3210u + ((n >> 1) & 0x4444u));
}

// Shared memory: hi[MT][cols], lo[MT][cols] (signed bytes), isc[MT][cols / 32] (1 / s).
template <int FMT, int MT>
__global__ void __launch_bounds__(WARPS * 32)
k_gemv_iq4(const uint8_t *__restrict__ w, uint32_t rows, uint32_t cols, uint32_t pitch, const float *__restrict__ x,
           float *__restrict__ y, const uint32_t *__restrict__ ids, uint32_t x_div, uint32_t experts) {
    extern __shared__ __align__(16) uint8_t iq4_smem[];
    int8_t *hi = reinterpret_cast<int8_t *>(iq4_smem), *lo = hi + (size_t)MT * cols;
    float *isc = reinterpret_cast<float *>(lo + (size_t)MT * cols);
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nb32 = cols / 32;
    fqk::pdl_trigger();
    fqk::pdl_wait(); // x (and the routing) may be the output of the kernel before this one
    if (ids) {
        // Routes (`project_id`, MT = 1): route blockIdx.y uses expert ids[route] (`rows` rows each), activation row
        // route / x_div, output row route.
        const uint32_t r = blockIdx.y, e = ids[r];
        if (e >= experts) return;
        w += (size_t)e * rows * pitch;
        x += (size_t)(r / x_div) * cols;
        y += (size_t)r * rows;
    }

    // 1. Activations -> 16-bit integers, one warp per (activation row, block of 32), lane = value (as in gemv_q8.cu).
    for (uint32_t i = warp; i < MT * nb32; i += WARPS) {
        const uint32_t mrow = i / nb32, b = i % nb32;
        const float v = x[(size_t)mrow * cols + 32 * b + lane];
        float amax = fabsf(v);
        const bool finite = __ballot_sync(0xffffffffu, !(fabsf(v) < INFINITY)) == 0u;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
        int e = 0;
        if (amax > 0.f && finite) {
            const int ex = (int)(__float_as_uint(amax) >> 23) - 126;
            e = max(-110, min(110, 15 - ex));
            if (amax * __uint_as_float((uint32_t)(127 + e) << 23) > 32639.f) e -= 1;
        }
        int q = __float2int_rn(fminf(fmaxf(v * __uint_as_float((uint32_t)(127 + e) << 23), -32639.f), 32639.f));
        if (!finite) q = 0; // the block's factor below is NaN in that case
        const int h = (q + 128) >> 8;
        // Within a run the bytes sit where the permuted codebook values of the weights fall: a byte pair (2p, 2p + 1)
        // of nibbles decodes to values 2p, 2p + 16, 2p + 1, 2p + 17 in that order.
        const uint32_t l = lane & 15u, pos = 4 * (l >> 1) + 2 * (l & 1u) + (lane >> 4);
        hi[(size_t)mrow * cols + 32 * b + pos] = (int8_t)h;
        lo[(size_t)mrow * cols + 32 * b + pos] = (int8_t)(q - (h << 8));
        if (lane == 0) isc[mrow * nb32 + b] = finite ? __uint_as_float((uint32_t)(127 - e) << 23) : __int_as_float(0x7fc00000);
    }
    __syncthreads();

    // 2. Rows.  A warp takes RPW weight rows at a time, strided over the grid, the loads of all of them in flight
    // together; lane l reads 16 bytes = one run of 32 values (an IQ4_NL block, an IQ4_XS sub-block) of every
    // 1024-value chunk.
    constexpr int RPW = 4;
    const uint32_t chunks = (cols + 1023) / 1024, groups = (rows + RPW - 1) / RPW;
    for (uint32_t g = blockIdx.x * WARPS + warp; g < groups; g += gridDim.x * WARPS) {
        const uint32_t row0 = g * RPW;
        const uint8_t *rp[RPW];
#pragma unroll
        for (int r = 0; r < RPW; r++) rp[r] = w + (size_t)min(row0 + r, rows - 1) * pitch;
        float acc[RPW][MT];
#pragma unroll
        for (int r = 0; r < RPW; r++)
#pragma unroll
            for (int t = 0; t < MT; t++) acc[r][t] = 0.f;
        for (uint32_t c = 0; c < chunks; c++) {
            const uint32_t run = 32 * c + lane; // index of the 32-value run
            const bool live = run < nb32;
            const uint32_t rr = live ? run : 0;
            uint4 q[RPW];
            float d[RPW];
#pragma unroll
            for (int r = 0; r < RPW; r++) q[r] = fqk::ldw128(rp[r] + (size_t)rr * 16);
#pragma unroll
            for (int r = 0; r < RPW; r++) {
                const uint8_t *hdr = rp[r] + cols / 2;
                if constexpr (FMT == FQ_IQ4_XS) {
                    const uint8_t *h8 = hdr + (size_t)(rr / 8) * 8;
                    d[r] = load_f16(h8) * (float)iq4xs_scale(h8, (int)(rr % 8));
                } else {
                    d[r] = load_f16(hdr + (size_t)rr * 2);
                }
            }
#pragma unroll
            for (int r = 0; r < RPW; r++) {
                // byte pairs of nibbles -> four signed bytes each, in the order the activations were laid down
                const uint32_t qw[4] = {q[r].x, q[r].y, q[r].z, q[r].w};
                uint32_t vl[4], vh[4]; // pairs 2 i and 2 i + 1
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    vl[i] = iq4_lookup4(qw[i]);
                    vh[i] = iq4_lookup4(qw[i] >> 16);
                }
#pragma unroll
                for (int t = 0; t < MT; t++) {
                    const int4 *xh = reinterpret_cast<const int4 *>(hi + (size_t)t * cols + (size_t)rr * 32);
                    const int4 *xl = reinterpret_cast<const int4 *>(lo + (size_t)t * cols + (size_t)rr * 32);
                    const int4 h0 = xh[0], h1 = xh[1], l0 = xl[0], l1 = xl[1];
                    int dh = __dp4a((int)vl[0], h0.x, 0), dl = __dp4a((int)vl[0], l0.x, 0);
                    dh = __dp4a((int)vh[0], h0.y, dh), dl = __dp4a((int)vh[0], l0.y, dl);
                    dh = __dp4a((int)vl[1], h0.z, dh), dl = __dp4a((int)vl[1], l0.z, dl);
                    dh = __dp4a((int)vh[1], h0.w, dh), dl = __dp4a((int)vh[1], l0.w, dl);
                    dh = __dp4a((int)vl[2], h1.x, dh), dl = __dp4a((int)vl[2], l1.x, dl);
                    dh = __dp4a((int)vh[2], h1.y, dh), dl = __dp4a((int)vh[2], l1.y, dl);
                    dh = __dp4a((int)vl[3], h1.z, dh), dl = __dp4a((int)vl[3], l1.z, dl);
                    dh = __dp4a((int)vh[3], h1.w, dh), dl = __dp4a((int)vh[3], l1.w, dl);
                    const float s = live ? isc[t * nb32 + rr] : 0.f; // lanes past the row's end contribute nothing
                    acc[r][t] = fmaf((float)(dh * 256 + dl), d[r] * s, acc[r][t]);
                }
            }
        }
#pragma unroll
        for (int r = 0; r < RPW; r++)
#pragma unroll
            for (int t = 0; t < MT; t++) {
                float v = acc[r][t];
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
                if (lane == 0 && row0 + r < rows) y[(size_t)t * rows + row0 + r] = v;
            }
    }
}

template <int FMT, int MT> cudaError_t launch(fq_device *dev, const ProjectArgs &a, const float *x, float *y, uint32_t routes = 0) {
    const size_t smem = (size_t)2 * MT * a.cols + (size_t)MT * (a.cols / 32) * sizeof(float);
    static size_t configured = 48 * 1024;
    if (smem > configured) {
        const size_t most = (size_t)MT * (2 * MAX_COLS_IQ4 + MAX_COLS_IQ4 / 8);
        cudaError_t e = cudaFuncSetAttribute(k_gemv_iq4<FMT, MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)most);
        if (e != cudaSuccess) return e;
        configured = most;
    }
    const uint32_t need = (a.rows + WARPS * 4 - 1) / (WARPS * 4);
    const uint32_t grid = std::min<uint32_t>(need, (uint32_t)dev->sm_count * 4);
    return fqk::launch_pdl(k_gemv_iq4<FMT, MT>, dim3(grid, routes ? routes : 1), dim3(WARPS * 32), smem, dev->stream, a.w, a.rows, a.cols, a.row_bytes, x, y,
                           routes ? a.ids : (const uint32_t *)nullptr, routes ? a.x_div : 1u, a.experts);
}

template <int FMT> cudaError_t launch_m(fq_device *dev, const ProjectArgs &a, const float *x, float *y, uint32_t mt) {
    switch (mt) {
    case 1: return launch<FMT, 1>(dev, a, x, y);
    case 2: return launch<FMT, 2>(dev, a, x, y);
    case 3: return launch<FMT, 3>(dev, a, x, y);
    default: return launch<FMT, 4>(dev, a, x, y);
    }
}

} // namespace

// IQ4_NL / IQ4_XS, F32 in / F32 out: up to FQ_GEMV_MAX_M activation rows (four per launch), or routes (`a.ids`: one
// activation row per route, `a.m` routes, `a.rows` rows per expert); FQ_ERR_UNSUPPORTED otherwise.
int fq_launch_gemv_iq4(fq_device *dev, const ProjectArgs &a) {
    if ((a.format != FQ_IQ4_NL && a.format != FQ_IQ4_XS) || a.x_dtype != FQ_F32 || a.y_dtype != FQ_F32 || a.offsets || a.norm_w || a.x_up)
        return FQ_ERR_UNSUPPORTED;
    if (a.m == 0 || a.cols > MAX_COLS_IQ4 || a.cols % 256 || a.row_bytes % 16) return FQ_ERR_UNSUPPORTED;
    if (a.ids) {
        if (a.m > 65535 || a.x_div == 0) return FQ_ERR_UNSUPPORTED;
        const cudaError_t e = a.format == FQ_IQ4_XS ? launch<FQ_IQ4_XS, 1>(dev, a, (const float *)a.x, (float *)a.y, a.m)
                                                    : launch<FQ_IQ4_NL, 1>(dev, a, (const float *)a.x, (float *)a.y, a.m);
        if (int rc = fq_check_cuda(dev, e, "gemv_iq4 launch")) return rc;
        return fq_end_enqueue(dev, "gemv_iq4", 1);
    }
    if (a.m > (uint32_t)FQ_GEMV_MAX_M) return FQ_ERR_UNSUPPORTED;
    int launches = 0;
    for (uint32_t m0 = 0; m0 < a.m; m0 += 4, launches++) {
        const uint32_t mt = a.m - m0 < 4 ? a.m - m0 : 4;
        const float *x = (const float *)a.x + (size_t)m0 * a.cols;
        float *y = (float *)a.y + (size_t)m0 * a.rows;
        const cudaError_t e = a.format == FQ_IQ4_XS ? launch_m<FQ_IQ4_XS>(dev, a, x, y, mt) : launch_m<FQ_IQ4_NL>(dev, a, x, y, mt);
        if (int rc = fq_check_cuda(dev, e, "gemv_iq4 launch")) return rc;
    }
    return fq_end_enqueue(dev, "gemv_iq4", launches);
}
