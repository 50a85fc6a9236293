// GGUF block layouts and the exact per-value decoders (device side).
//
// Layouts (little-endian, f16 = IEEE binary16), as in the reference's `block_q4_K`, `block_q6_K`,
// `block_q8_0` (src/metal/shaders/hybrid.metal:23-26) and src/quantization.rs:50-73:
//   Q4_K  144 B / 256 values: f16 d @0, f16 dmin @2, scales[12] @4, qs[128] @16
//   Q5_K  176 B / 256 values: f16 d @0, f16 dmin @2, scales[12] @4, qh[32] @16, qs[128] @48
//   Q6_K  210 B / 256 values: ql[128] @0, qh[64] @128, int8 scales[16] @192, f16 d @208
//   Q8_0   34 B /  32 values: f16 d @0, int8 qs[32] @2
//   IQ4_NL 18 B /  32 values: f16 d @0, qs[16] @2 (byte j = values j and j + 16, indices into a 16-entry codebook)
//   IQ4_XS 136 B / 256 values: f16 d @0, u16 scales_h @2, scales_l[4] @4, qs[128] @8 (`block_iq4_xs`, hybrid.metal:27)
// On the device Q6_K, Q8_0 and the IQ4 formats are regrouped by field per row (see each decoder), so that the
// quants can be read with aligned 16-byte loads.
//
// The decoders reproduce the CPU formulas the reference tests against
// (src/diffusion/tests.rs:795-864, src/hybrid/draft/gguf.rs:336-343) as explicit round-to-nearest
// single-precision operations, so the compiler cannot contract them into FMAs and the decoded
// weights are bit-identical to the CPU decode.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include "../../include/ferrum_b200.h"

template <int FMT> struct BlockTraits;
template <> struct BlockTraits<FQ_Q4_K> { static constexpr int EL = 256, BB = 144; };
template <> struct BlockTraits<FQ_Q5_K> { static constexpr int EL = 256, BB = 176; };
template <> struct BlockTraits<FQ_Q6_K> { static constexpr int EL = 256, BB = 210; };
template <> struct BlockTraits<FQ_Q8_0> { static constexpr int EL = 32, BB = 34; };
template <> struct BlockTraits<FQ_IQ4_NL> { static constexpr int EL = 32, BB = 18; };
template <> struct BlockTraits<FQ_IQ4_XS> { static constexpr int EL = 256, BB = 136; };

__device__ __forceinline__ float f16_bits_to_f32(uint16_t bits) {
    return __half2float(__ushort_as_half(bits));
}
// Blocks of Q6_K and Q8_0 are only 2-byte aligned, so f16 fields are read as two bytes' worth.
__device__ __forceinline__ float load_f16(const uint8_t *p) {
    return f16_bits_to_f32(*reinterpret_cast<const uint16_t *>(p));
}

// Q4_K sub-block j's 6-bit scale and minimum (`get_scale_min_k4`, hybrid.metal:417-420).
__device__ __forceinline__ void q4k_scale_min(const uint8_t *s, int j, uint32_t &sc, uint32_t &mn) {
    if (j < 4) {
        sc = s[j] & 63u;
        mn = s[j + 4] & 63u;
    } else {
        sc = (s[j + 4] & 0xFu) | ((uint32_t)(s[j - 4] >> 6) << 4);
        mn = (uint32_t)(s[j + 4] >> 4) | ((uint32_t)(s[j] >> 6) << 4);
    }
}

// ((d * sc) * q) - (dmin * m), each operation rounded on its own.
__device__ __forceinline__ float q4k_value(float d, float dmin, uint32_t sc, uint32_t mn, uint32_t q) {
    return __fsub_rn(__fmul_rn(__fmul_rn(d, (float)sc), (float)q), __fmul_rn(dmin, (float)mn));
}
// (d * scale) * (q - 32)
__device__ __forceinline__ float q6k_value(float d, int scale, uint32_t q) {
    return __fmul_rn(__fmul_rn(d, (float)scale), (float)q - 32.0f);
}

// Device layouts.  Q4_K and Q5_K rows are the GGUF bytes.  Q6_K and Q8_0 rows are the same bytes regrouped by
// field at load time so that every field is 16-byte aligned (210- and 34-byte blocks are not): with nb
// blocks in the row,
//   Q6_K: ql of block b at 128 b, qh at 128 nb + 64 b, scales at 192 nb + 16 b, d at 208 nb + 2 b,
//   Q8_0: qs of block b at 32 b, d at 32 nb + 2 b,
// and the row pitch is the packed row size (210 nb, 34 nb) rounded up to 16 bytes.
__host__ __device__ inline uint32_t fq_row_pitch(int format, uint32_t cols) {
    switch (format) {
    case FQ_Q4_K: return cols / 256 * 144;
    case FQ_Q5_K: return cols / 256 * 176;
    case FQ_Q6_K: return (cols / 256 * 210 + 15u) & ~15u;
    case FQ_IQ4_NL: return (cols / 32 * 18 + 15u) & ~15u;
    case FQ_IQ4_XS: return (cols / 256 * 136 + 15u) & ~15u;
    default: return (cols / 32 * 34 + 15u) & ~15u;
    }
}

// Value `idx` (0 .. EL-1, in the format's logical order) of block `b` of a row with `nb` blocks.
template <int FMT> __device__ __forceinline__ float decode_at(const uint8_t *row, uint32_t nb, uint32_t b, int idx);

template <> __device__ __forceinline__ float decode_at<FQ_Q4_K>(const uint8_t *row, uint32_t, uint32_t b, int idx) {
    const uint8_t *blk = row + (size_t)b * 144;
    const int j = idx >> 5, l = idx & 31;
    uint32_t sc, mn;
    q4k_scale_min(blk + 4, j, sc, mn);
    const uint8_t v = blk[16 + 32 * (j >> 1) + l];
    const uint32_t q = (j & 1) ? (v >> 4) : (v & 0xFu);
    return q4k_value(load_f16(blk), load_f16(blk + 2), sc, mn, q);
}

// Q5_K (`q45_k` with the high bits, src/diffusion/tests.rs:811-840): bit j of qh[l] is the fifth bit of value l of
// sub-block j.
template <> __device__ __forceinline__ float decode_at<FQ_Q5_K>(const uint8_t *row, uint32_t, uint32_t b, int idx) {
    const uint8_t *blk = row + (size_t)b * 176;
    const int j = idx >> 5, l = idx & 31;
    uint32_t sc, mn;
    q4k_scale_min(blk + 4, j, sc, mn);
    const uint8_t v = blk[48 + 32 * (j >> 1) + l];
    const uint32_t q = ((j & 1) ? (v >> 4) : (v & 0xFu)) + (((blk[16 + l] >> j) & 1u) << 4);
    return q4k_value(load_f16(blk), load_f16(blk + 2), sc, mn, q);
}

template <> __device__ __forceinline__ float decode_at<FQ_Q6_K>(const uint8_t *row, uint32_t nb, uint32_t b, int idx) {
    const uint8_t *ql = row + (size_t)b * 128, *qh = row + (size_t)nb * 128 + (size_t)b * 64;
    const uint8_t *sc = row + (size_t)nb * 192 + (size_t)b * 16, *d = row + (size_t)nb * 208 + (size_t)b * 2;
    const int n = idx >> 7, r = idx & 127, i = r >> 5, l = r & 31;
    const uint8_t lo = ql[64 * n + l + 32 * (i & 1)];
    const uint32_t nib = (i < 2) ? (lo & 0xFu) : (lo >> 4);
    const uint32_t hi = (qh[32 * n + l] >> (2 * i)) & 3u;
    const int scale = (int)(int8_t)sc[8 * n + (l >> 4) + 2 * i];
    return q6k_value(load_f16(d), scale, nib | (hi << 4));
}

// The non-linear 4-bit codebook of the IQ4 formats (`kvalues_iq4nl_f`, hybrid.metal:34-37) as two 64-bit words of
// signed bytes.
__device__ __forceinline__ float iq4_value(uint32_t q) {
    const uint64_t table = q < 8 ? 0xF6EADDCFBFAD9881ull : 0x7159453526190D01ull;
    return (float)(int)(int8_t)(table >> (8 * (q & 7u)));
}

// IQ4_NL (`dequant_iq4_nl`, src/hybrid/iq_tests.rs:1606-1618): d * codebook[q], byte j = values j and j + 16.
// Device layout of a row: the nibbles of all blocks (16 bytes each), then the f16 scales.
template <> __device__ __forceinline__ float decode_at<FQ_IQ4_NL>(const uint8_t *row, uint32_t nb, uint32_t b, int idx) {
    const uint8_t v = row[(size_t)b * 16 + (idx & 15)];
    return __fmul_rn(load_f16(row + (size_t)nb * 16 + (size_t)b * 2), iq4_value(idx < 16 ? (v & 15u) : (v >> 4)));
}

// IQ4_XS (`dequantize_iq4_xs`, hybrid.metal:580-596): (d * (ls - 32)) * codebook[q] with the sub-block's 6-bit ls.
// Device layout of a row: the nibbles of all blocks (128 bytes each), then the 8-byte headers d | scales_h | scales_l.
__device__ __forceinline__ int iq4xs_scale(const uint8_t *hdr, int ib) {
    const uint32_t scales_h = hdr[2] | ((uint32_t)hdr[3] << 8);
    return ((int)((hdr[4 + ib / 2] >> (4 * (ib % 2))) & 15u) | (int)(((scales_h >> (2 * ib)) & 3u) << 4)) - 32;
}
template <> __device__ __forceinline__ float decode_at<FQ_IQ4_XS>(const uint8_t *row, uint32_t nb, uint32_t b, int idx) {
    const uint8_t *hdr = row + (size_t)nb * 128 + (size_t)b * 8;
    const int ib = idx >> 5, l = idx & 31;
    const uint8_t v = row[(size_t)b * 128 + 16 * ib + (l & 15)];
    return __fmul_rn(__fmul_rn(load_f16(hdr), (float)iq4xs_scale(hdr, ib)), iq4_value(l < 16 ? (v & 15u) : (v >> 4)));
}

template <> __device__ __forceinline__ float decode_at<FQ_Q8_0>(const uint8_t *row, uint32_t nb, uint32_t b, int idx) {
    return __fmul_rn((float)(int)(int8_t)row[(size_t)b * 32 + idx], load_f16(row + (size_t)nb * 32 + (size_t)b * 2));
}

// Round to nearest even (src/hybrid/draft/gguf.rs:362-369).  cvt.rn.bf16.f32 agrees for every
// non-NaN input; a NaN stays a quiet NaN but its payload is the canonical one.
__device__ __forceinline__ __nv_bfloat16 to_bf16_rne(float v) { return __float2bfloat16_rn(v); }

template <typename T> __device__ __forceinline__ float load_act(const T *p);
template <> __device__ __forceinline__ float load_act<float>(const float *p) { return *p; }
template <> __device__ __forceinline__ float load_act<__nv_bfloat16>(const __nv_bfloat16 *p) {
    return __bfloat162float(*p);
}
template <typename T> __device__ __forceinline__ void store_act(T *p, float v);
template <> __device__ __forceinline__ void store_act<float>(float *p, float v) { *p = v; }
template <> __device__ __forceinline__ void store_act<__nv_bfloat16>(__nv_bfloat16 *p, float v) {
    *p = to_bf16_rne(v);
}
