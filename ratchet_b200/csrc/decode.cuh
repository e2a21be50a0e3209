// Element decoders for every lhs storage kind, shared by the general-purpose kernels and by the
// dequantise kernels.  The arithmetic is the reference's:
//   Q8_0F  (i8)q * d in f32                     crates/ratchet-core/src/quant.rs:114-120
//   Q8_0H  f16(q) * d rounded to f16            crates/ratchet-core/src/ops/gemm.rs:400-406
//   Q4_K   (d*sc)*q - (dmin*m), separate f32 roundings (GGUF Q4_K; block struct
//          crates/ratchet-loader/src/k_quants.rs:95-103)
#pragma once
#include "common.cuh"

namespace rt {

enum LhsKind : int { LK_F32 = 0, LK_F16 = 1, LK_BF16 = 2, LK_Q8H = 3, LK_Q8F = 4, LK_Q4K = 5 };

__device__ __forceinline__ void q4k_scale_min(int j, const uint8_t *s, int &sc, int &m) {
    if (j < 4) {
        sc = s[j] & 63;
        m = s[j + 4] & 63;
    } else {
        sc = (s[j + 4] & 0x0F) | ((s[j - 4] >> 6) << 4);
        m = (s[j + 4] >> 4) | ((s[j] >> 6) << 4);
    }
}

// value of flat element `idx` of a Q4_K tensor
__device__ __forceinline__ float q4k_element(const uint8_t *base, long long idx) {
    const uint8_t *blk = base + (idx >> 8) * 144;
    const int within = (int)(idx & 255), j = within >> 5, l = within & 31;
    const float d = __half2float(*reinterpret_cast<const __half *>(blk));
    const float dmin = __half2float(*reinterpret_cast<const __half *>(blk + 2));
    int sc, m;
    q4k_scale_min(j, blk + 4, sc, m);
    const uint8_t q = blk[16 + 32 * (j >> 1) + l];
    const int code = (j & 1) ? (q >> 4) : (q & 0x0F);
    const float ds = __fmul_rn(d, (float)sc);
    const float dm = __fmul_rn(dmin, (float)m);
    return __fsub_rn(__fmul_rn(ds, (float)code), dm);
}

// Value of lhs element at flat index `idx` (row-major within one batch slice).
template <int KIND>
__device__ __forceinline__ float lhs_element(const void *lhs, const void *scales, long long idx) {
    if (KIND == LK_F32) return ((const float *)lhs)[idx];
    if (KIND == LK_F16) return __half2float(((const __half *)lhs)[idx]);
    if (KIND == LK_BF16) return __bfloat162float(((const __nv_bfloat16 *)lhs)[idx]);
    if (KIND == LK_Q8H) {
        const float q = (float)((const int8_t *)lhs)[idx];
        const float d = __half2float(((const __half *)scales)[idx >> 5]);
        return __half2float(__float2half_rn(__fmul_rn(q, d))); // q*d is exact in f32; one rounding to f16
    }
    if (KIND == LK_Q8F) {
        const float q = (float)((const int8_t *)lhs)[idx];
        return __fmul_rn(q, ((const float *)scales)[idx >> 5]);
    }
    return q4k_element((const uint8_t *)lhs, idx);
}

} // namespace rt
