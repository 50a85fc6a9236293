// Q8_0 decode projections for 1..4 activation rows per launch (F32 in, F32 out): the reference's
// `h_mv_q8_0` / `h_mvb_q8_0` (src/metal/shaders/hybrid.metal:640-686, 1330-1394).  In the 35B-A3B-class
// model every matrix that is not an expert matrix is Q8_0 (attention, router, shared expert, lm_head).
//
// The weights are signed bytes already, so the dot products stay in the integer domain (dp4a):
//
//   1. every block quantises the activations itself, into shared memory: per activation row and per
//      32 values (one Q8_0 block) x' = round(x * s) = 256 * hi + lo, both halves signed bytes, s the
//      largest power of two with max|x| * s <= 32639.  No separate preparation launch.
//   2. a warp owns RPW weight rows; lane l reads bytes [16 l, 16 l + 16) of every 512-byte chunk of the
//      row (half a block) with one 128-bit load, the chunks of all its rows in flight together;
//   3. per half block and activation row: 4 + 4 dp4a (hi, lo planes), 256 * dot_hi + dot_lo, one
//      conversion and one FMA with d / s.
//
// The result is the exact dot product of the decoded weights with activations rounded to 16 bits relative
// to the largest magnitude of their block of 32.  Sums run in a fixed order: a row's value does not depend
// on the launch geometry, so a row-sharded matrix returns the same bits as the whole one.
//
// Device layout of a Q8_0 row (blocks.cuh): the quants of all blocks first (cols bytes, natural order),
// then the f16 scales (2 bytes per block).
#include <algorithm>
#include <cstdlib>

#include "blocks.cuh"
#include "internal.h"

namespace {

constexpr int WARPS = 8;
constexpr uint32_t MAX_COLS_Q8 = 16384; // 2 planes x 4 activation rows x cols bytes of shared memory

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ uint4 ldg_stream(const uint8_t *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// Shared memory: hi[MT][cols], lo[MT][cols] (signed bytes), isc[MT][cols / 32] (1 / s).
template <int MT, int RPW>
__global__ void __launch_bounds__(WARPS * 32)
k_gemv_q8(const uint8_t *__restrict__ w, uint32_t rows, uint32_t cols, uint32_t pitch, const float *__restrict__ x,
          float *__restrict__ y) {
    extern __shared__ __align__(16) uint8_t smem[];
    int8_t *hi = reinterpret_cast<int8_t *>(smem), *lo = hi + (size_t)MT * cols;
    float *isc = reinterpret_cast<float *>(lo + (size_t)MT * cols);
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nb = cols / 32;
    pdl_trigger();
    pdl_wait(); // x may be the output of the kernel before this one

    // 1. Activations -> 16-bit integers, one warp per (activation row, block of 32), lane = value.
    for (uint32_t i = warp; i < MT * nb; i += WARPS) {
        const uint32_t mrow = i / nb, b = i % nb;
        const float v = x[(size_t)mrow * cols + 32 * b + lane];
        float amax = fabsf(v);
        const bool finite = __ballot_sync(0xffffffffu, !(fabsf(v) < INFINITY)) == 0u;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
        // s = 2^e, the largest power of two with amax * s <= 32639: amax = f * 2^ex with f in [0.5, 1), so
        // e = 15 - ex, one less when f * 2^15 > 32639.  Exponents straight from the float's bits.
        int e = 0;
        if (amax > 0.f && finite) {
            const int ex = (int)(__float_as_uint(amax) >> 23) - 126;
            e = max(-110, min(110, 15 - ex));
            if (amax * __uint_as_float((uint32_t)(127 + e) << 23) > 32639.f) e -= 1;
        }
        int q = __float2int_rn(fminf(fmaxf(v * __uint_as_float((uint32_t)(127 + e) << 23), -32639.f), 32639.f));
        if (!finite) q = 0; // the block's factor below is NaN in that case
        const int h = (q + 128) >> 8;
        hi[(size_t)mrow * cols + 32 * b + lane] = (int8_t)h;
        lo[(size_t)mrow * cols + 32 * b + lane] = (int8_t)(q - (h << 8));
        if (lane == 0) isc[mrow * nb + b] = finite ? __uint_as_float((uint32_t)(127 - e) << 23) : __int_as_float(0x7fc00000);
    }
    __syncthreads();

    // 2. Rows.  A warp takes groups of RPW rows, strided over the grid (the grid is a few blocks per SM, so
    // the quantisation above is paid once per many rows).  Lane l: bytes 16 l .. 16 l + 15 of each 512-byte
    // chunk = half of block 16 c + l / 2.
    const uint32_t groups = (rows + RPW - 1) / RPW, chunks = (cols + 511) / 512;
    for (uint32_t g = blockIdx.x * WARPS + warp; g < groups; g += gridDim.x * WARPS) {
        const uint32_t row0 = g * RPW;
        float acc[RPW][MT];
#pragma unroll
        for (int r = 0; r < RPW; r++)
#pragma unroll
            for (int t = 0; t < MT; t++) acc[r][t] = 0.f;
        const uint8_t *rp[RPW];
#pragma unroll
        for (int r = 0; r < RPW; r++) rp[r] = w + (size_t)min(row0 + r, rows - 1) * pitch;
#pragma unroll 2
        for (uint32_t c = 0; c < chunks; c++) {
            const uint32_t k = 512 * c + 16 * lane;
            const bool live = k < cols;
            const uint32_t kk = live ? k : 0, b = kk / 32;
            uint4 q[RPW];
            float d[RPW];
#pragma unroll
            for (int r = 0; r < RPW; r++) q[r] = ldg_stream(rp[r] + kk);
#pragma unroll
            for (int r = 0; r < RPW; r++) d[r] = load_f16(rp[r] + cols + 2 * b);
#pragma unroll
            for (int t = 0; t < MT; t++) {
                const int4 xh = *reinterpret_cast<const int4 *>(hi + (size_t)t * cols + kk);
                const int4 xl = *reinterpret_cast<const int4 *>(lo + (size_t)t * cols + kk);
                const float s = live ? isc[t * nb + b] : 0.f; // lanes past the row's end contribute nothing
#pragma unroll
                for (int r = 0; r < RPW; r++) {
                    int dh = __dp4a((int)q[r].x, xh.x, 0), dl = __dp4a((int)q[r].x, xl.x, 0);
                    dh = __dp4a((int)q[r].y, xh.y, dh), dl = __dp4a((int)q[r].y, xl.y, dl);
                    dh = __dp4a((int)q[r].z, xh.z, dh), dl = __dp4a((int)q[r].z, xl.z, dl);
                    dh = __dp4a((int)q[r].w, xh.w, dh), dl = __dp4a((int)q[r].w, xl.w, dl);
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

template <typename... KArgs, typename... Args>
cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
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

template <int MT, int RPW>
cudaError_t launch(fq_device *dev, const ProjectArgs &a, const float *x, float *y) {
    const size_t smem = (size_t)2 * MT * a.cols + (size_t)MT * (a.cols / 32) * sizeof(float);
    static size_t configured = 48 * 1024;
    if (smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(k_gemv_q8<MT, RPW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(MT * (2 * MAX_COLS_Q8 + MAX_COLS_Q8 / 8)));
        if (e != cudaSuccess) return e;
        configured = MT * (2 * MAX_COLS_Q8 + MAX_COLS_Q8 / 8);
    }
    const uint32_t per_block = WARPS * RPW, need = (a.rows + per_block - 1) / per_block;
    const uint32_t grid = std::min<uint32_t>(need, (uint32_t)dev->sm_count * 4);
    return launch_pdl(k_gemv_q8<MT, RPW>, dim3(grid), dim3(WARPS * 32), smem, dev->stream, a.w, a.rows, a.cols, a.row_bytes, x, y);
}

template <int RPW> cudaError_t launch_m(fq_device *dev, const ProjectArgs &a, const float *x, float *y, uint32_t mt) {
    switch (mt) {
    case 1: return launch<1, RPW>(dev, a, x, y);
    case 2: return launch<2, RPW>(dev, a, x, y);
    case 3: return launch<3, RPW>(dev, a, x, y);
    default: return launch<4, RPW>(dev, a, x, y);
    }
}

} // namespace

// Q8_0, F32 in / F32 out, up to FQ_GEMV_MAX_M activation rows (four per launch); FQ_ERR_UNSUPPORTED otherwise.
int fq_launch_gemv_q8(fq_device *dev, const ProjectArgs &a) {
    if (a.format != FQ_Q8_0 || a.x_dtype != FQ_F32 || a.y_dtype != FQ_F32 || a.ids || a.offsets) return FQ_ERR_UNSUPPORTED;
    if (a.m == 0 || a.m > (uint32_t)FQ_GEMV_MAX_M || a.cols > MAX_COLS_Q8 || a.cols % 32 || a.row_bytes % 16) return FQ_ERR_UNSUPPORTED;
    // Four rows per warp once that still leaves every SM several blocks.
    const bool wide = a.rows >= (uint32_t)dev->sm_count * WARPS * 4 * 4;
    int launches = 0;
    for (uint32_t m0 = 0; m0 < a.m; m0 += 4, launches++) {
        const uint32_t mt = a.m - m0 < 4 ? a.m - m0 : 4;
        const float *x = (const float *)a.x + (size_t)m0 * a.cols;
        float *y = (float *)a.y + (size_t)m0 * a.rows;
        const cudaError_t e = wide ? launch_m<4>(dev, a, x, y, mt) : launch_m<1>(dev, a, x, y, mt);
        if (int rc = fq_check_cuda(dev, e, "gemv_q8 launch")) return rc;
    }
    return fq_end_enqueue(dev, "gemv_q8", launches);
}
