// Exact-decode kernels: embedding lookup (`h_get_rows_*`) and the fp32 projections that decode
// every weight with the reference's per-value formula.  They serve `fq_get_rows`, the handle's
// exact mode (the reference's FERRUM_HYBRID_EXACT), and every shape the tensor-core kernels do
// not cover.  One warp owns one weight row; lanes stride over the values of each block; up to
// MT activation rows share one decode.
#include "blocks.cuh"
#include "internal.h"

namespace {

constexpr int WARPS = 4; // weight rows per thread block
constexpr int MT = 8;    // activation rows sharing one decode

template <int FMT, typename XT>
__device__ __forceinline__ void row_dot(const uint8_t *wrow, uint32_t cols, const XT *x, size_t x_stride,
                                        int tokens, int lane, float (&acc)[MT]) {
    constexpr int EL = BlockTraits<FMT>::EL;
    const uint32_t blocks = cols / EL;
#pragma unroll
    for (int t = 0; t < MT; t++) acc[t] = 0.f;
    for (uint32_t b = 0; b < blocks; b++) {
#pragma unroll
        for (int i = 0; i < EL / 32; i++) {
            const int idx = i * 32 + lane;
            const float w = decode_at<FMT>(wrow, blocks, b, idx);
            const size_t k = (size_t)b * EL + idx;
#pragma unroll
            for (int t = 0; t < MT; t++)
                if (t < tokens) acc[t] = fmaf(w, load_act<XT>(x + (size_t)t * x_stride + k), acc[t]);
        }
    }
#pragma unroll
    for (int t = 0; t < MT; t++)
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) acc[t] += __shfl_xor_sync(0xffffffffu, acc[t], off);
}

// y[t][row] for t in a tile of MT activation rows; grid (ceil(rows / WARPS), ceil(m / MT)).
template <int FMT, typename XT, typename YT>
__global__ void __launch_bounds__(WARPS * 32)
k_project_exact(const uint8_t *__restrict__ w, uint32_t rows, uint32_t cols, uint32_t row_bytes,
                const XT *__restrict__ x, YT *__restrict__ y, uint32_t m) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t row = blockIdx.x * WARPS + warp;
    const uint32_t t0 = blockIdx.y * MT;
    if (row >= rows) return;
    const int tokens = min((uint32_t)MT, m - t0);
    float acc[MT];
    row_dot<FMT, XT>(w + (size_t)row * row_bytes, cols, x + (size_t)t0 * cols, cols, tokens, lane, acc);
    if (lane == 0)
        for (int t = 0; t < tokens; t++) store_act<YT>(y + (size_t)(t0 + t) * rows + row, acc[t]);
}

// Route r = blockIdx.x: expert ids[r], activation row r / x_div, output row r.
template <int FMT>
__global__ void __launch_bounds__(WARPS * 32)
k_project_id_exact(const uint8_t *__restrict__ w, uint32_t rows_e, uint32_t cols, uint32_t row_bytes,
                   const float *__restrict__ x, const uint32_t *__restrict__ ids, uint32_t x_div,
                   uint32_t experts, float *__restrict__ y) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t row = blockIdx.y * WARPS + warp;
    const uint32_t r = blockIdx.x;
    if (row >= rows_e) return;
    const uint32_t e = ids[r];
    if (e >= experts) return; // a route naming no stored expert writes nothing
    float acc[MT];
    row_dot<FMT, float>(w + ((size_t)e * rows_e + row) * row_bytes, cols, x + (size_t)(r / x_div) * cols,
                        cols, 1, lane, acc);
    if (lane == 0) y[(size_t)r * rows_e + row] = acc[0];
}

// Group z = blockIdx.z: rows offsets[z]..offsets[z+1] of x / y, expert slots[z] (or z).
template <int FMT, typename XT, typename YT>
__global__ void __launch_bounds__(WARPS * 32)
k_project_grouped_exact(const uint8_t *__restrict__ w, uint32_t rows_e, uint32_t cols, uint32_t row_bytes,
                        const XT *__restrict__ x, const uint32_t *__restrict__ offsets,
                        const uint32_t *__restrict__ slots, uint32_t experts, YT *__restrict__ y) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t row = blockIdx.x * WARPS + warp;
    const uint32_t z = blockIdx.z;
    const uint32_t first = offsets[z], count = offsets[z + 1] - first;
    const uint32_t t0 = blockIdx.y * MT;
    if (row >= rows_e || t0 >= count) return;
    const uint32_t e = slots ? slots[z] : z;
    if (e >= experts) return;
    const int tokens = min((uint32_t)MT, count - t0);
    float acc[MT];
    row_dot<FMT, XT>(w + ((size_t)e * rows_e + row) * row_bytes, cols, x + (size_t)(first + t0) * cols, cols,
                     tokens, lane, acc);
    if (lane == 0)
        for (int t = 0; t < tokens; t++) store_act<YT>(y + (size_t)(first + t0 + t) * rows_e + row, acc[t]);
}

// y[t][c] = decode(W[ids[t]][c]); grid (tokens, ceil(cols / 256)).
template <int FMT, typename YT>
__global__ void __launch_bounds__(256)
k_get_rows(const uint8_t *__restrict__ w, uint32_t rows, uint32_t cols, uint32_t row_bytes,
           const uint32_t *__restrict__ ids, YT *__restrict__ y) {
    constexpr int EL = BlockTraits<FMT>::EL;
    const uint32_t c = blockIdx.y * 256 + threadIdx.x;
    const uint32_t t = blockIdx.x;
    if (c >= cols) return;
    const uint32_t r = ids[t];
    // An id beyond the matrix decodes nothing; the row is written as zeros.
    const float v = r < rows ? decode_at<FMT>(w + (size_t)r * row_bytes, cols / EL, c / EL, c % EL) : 0.f;
    store_act<YT>(y + (size_t)t * cols + c, v);
}

template <typename F> int dispatch_format(fq_device *dev, uint32_t format, F &&f) {
    switch (format) {
    case FQ_Q4_K: f(std::integral_constant<int, FQ_Q4_K>{}); return FQ_OK;
    case FQ_Q5_K: f(std::integral_constant<int, FQ_Q5_K>{}); return FQ_OK;
    case FQ_Q6_K: f(std::integral_constant<int, FQ_Q6_K>{}); return FQ_OK;
    case FQ_Q8_0: f(std::integral_constant<int, FQ_Q8_0>{}); return FQ_OK;
    case FQ_IQ4_NL: f(std::integral_constant<int, FQ_IQ4_NL>{}); return FQ_OK;
    case FQ_IQ4_XS: f(std::integral_constant<int, FQ_IQ4_XS>{}); return FQ_OK;
    default: return fq_fail(dev, FQ_ERR_UNSUPPORTED, "format %u has no kernel", format);
    }
}

template <typename F> int dispatch_dtypes(fq_device *dev, int xd, int yd, F &&f) {
    if (xd == FQ_F32 && yd == FQ_F32) { f((float *)nullptr, (float *)nullptr); return FQ_OK; }
    if (xd == FQ_BF16 && yd == FQ_BF16) { f((__nv_bfloat16 *)nullptr, (__nv_bfloat16 *)nullptr); return FQ_OK; }
    if (xd == FQ_BF16 && yd == FQ_F32) { f((__nv_bfloat16 *)nullptr, (float *)nullptr); return FQ_OK; }
    if (xd == FQ_F32 && yd == FQ_BF16) { f((float *)nullptr, (__nv_bfloat16 *)nullptr); return FQ_OK; }
    return fq_fail(dev, FQ_ERR_UNSUPPORTED, "activation dtype %d / output dtype %d", xd, yd);
}

} // namespace

int fq_launch_project_exact(fq_device *dev, const ProjectArgs &a) {
    int inner = FQ_OK;
    int rc = dispatch_format(dev, a.format, [&](auto fmt) {
        inner = dispatch_dtypes(dev, a.x_dtype, a.y_dtype, [&](auto *xt, auto *yt) {
            using XT = std::remove_pointer_t<decltype(xt)>;
            using YT = std::remove_pointer_t<decltype(yt)>;
            dim3 grid((a.rows + WARPS - 1) / WARPS, (a.m + MT - 1) / MT);
            k_project_exact<decltype(fmt)::value, XT, YT><<<grid, WARPS * 32, 0, dev->stream>>>(
                a.w, a.rows, a.cols, a.row_bytes, (const XT *)a.x, (YT *)a.y, a.m);
        });
    });
    return rc != FQ_OK ? rc : inner;
}

int fq_launch_project_id_exact(fq_device *dev, const ProjectArgs &a) {
    return dispatch_format(dev, a.format, [&](auto fmt) {
        dim3 grid(a.m, (a.rows + WARPS - 1) / WARPS);
        k_project_id_exact<decltype(fmt)::value><<<grid, WARPS * 32, 0, dev->stream>>>(
            a.w, a.rows, a.cols, a.row_bytes, (const float *)a.x, a.ids, a.x_div, a.experts, (float *)a.y);
    });
}

int fq_launch_project_grouped_exact(fq_device *dev, const ProjectArgs &a) {
    int inner = FQ_OK;
    int rc = dispatch_format(dev, a.format, [&](auto fmt) {
        inner = dispatch_dtypes(dev, a.x_dtype, a.y_dtype, [&](auto *xt, auto *yt) {
            using XT = std::remove_pointer_t<decltype(xt)>;
            using YT = std::remove_pointer_t<decltype(yt)>;
            dim3 grid((a.rows + WARPS - 1) / WARPS, (a.max_rows + MT - 1) / MT, a.groups);
            k_project_grouped_exact<decltype(fmt)::value, XT, YT><<<grid, WARPS * 32, 0, dev->stream>>>(
                a.w, a.rows, a.cols, a.row_bytes, (const XT *)a.x, a.offsets, a.slots, a.experts, (YT *)a.y);
        });
    });
    return rc != FQ_OK ? rc : inner;
}

int fq_launch_get_rows(fq_device *dev, const fq_matrix *w, const uint32_t *ids, uint32_t tokens, void *y,
                       int y_dtype) {
    return dispatch_format(dev, w->format, [&](auto fmt) {
        dim3 grid(tokens, ((uint32_t)w->cols + 255) / 256);
        if (y_dtype == FQ_BF16)
            k_get_rows<decltype(fmt)::value, __nv_bfloat16><<<grid, 256, 0, dev->stream>>>(
                w->data, (uint32_t)w->rows, (uint32_t)w->cols, (uint32_t)w->pitch, ids, (__nv_bfloat16 *)y);
        else
            k_get_rows<decltype(fmt)::value, float><<<grid, 256, 0, dev->stream>>>(
                w->data, (uint32_t)w->rows, (uint32_t)w->cols, (uint32_t)w->pitch, ids, (float *)y);
    });
}


// ------------------------------------------------------------------ read-only stream probe
//
// What a kernel that does nothing but read can stream from HBM on this device: every thread reads 16 bytes
// per step with the loads the projection kernels use for weights, grid-stride, and folds them into one word
// that is (almost) never written.  The ceiling a weight-streaming projection is measured against, as the
// reference measures its own (`h_bw_read`, src/hybrid/bench.rs:140-167).
namespace {
__global__ void __launch_bounds__(256) k_read_stream(const uint4 *__restrict__ p, size_t n16, uint32_t *sink) {
    uint32_t acc = 0;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += (size_t)gridDim.x * blockDim.x) {
        uint4 v;
        asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p + i));
        acc ^= v.x ^ v.y ^ v.z ^ v.w;
    }
    if (acc == 0x9E3779B9u) *sink = acc;
}
} // namespace

extern "C" int fq_probe_read_stream(fq_device *dev, const void *data, size_t bytes, uint32_t blocks_per_sm) {
    if (int rc = fq_begin_enqueue(dev)) return rc;
    if (bytes < 16 || blocks_per_sm == 0 || blocks_per_sm > 32) return fq_fail(dev, FQ_ERR_PARAM, "stream probe of %zu bytes, %u blocks per SM", bytes, blocks_per_sm);
    if (int rc = fq_check_binding(dev, data, bytes, "data")) return rc;
    k_read_stream<<<dev->sm_count * blocks_per_sm, 256, 0, dev->stream>>>((const uint4 *)data, bytes / 16, (uint32_t *)dev->status_dev + 8);
    return fq_end_enqueue(dev, "read_stream", 1);
}
