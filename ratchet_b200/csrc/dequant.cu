// Dequantise a block-format tensor on the device: the parity hook for "bit-exact dequantised
// weights" and the weight pre-pass of the large-M tensor-core GEMM.
// Arithmetic per element: see decode.cuh (quant.rs:114-120, gemm.rs:400-406 of the reference).
#include <algorithm>

#include "decode.cuh"
#include "kernels.hpp"

namespace rt {

namespace {

template <int KIND, typename OutT>
__global__ void __launch_bounds__(256) dequant_kernel(const void *src, const void *scales, OutT *dst, long long numel) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < numel; i += stride)
        dst[i] = from_f32<OutT>(lhs_element<KIND>(src, scales, i));
}

// Q8_0H -> f16, 16 codes per thread: the pre-pass form (same values as the element-wise kernel).
__global__ void __launch_bounds__(256) dequant_q8h_f16_vec_kernel(const uint4 *codes, const __half *scales, uint4 *dst,
                                                                 long long n16) {
    // the next kernel may start its prologue now; this one's stream predecessor may still be reading what it writes
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += stride) {
        const uint4 w = __ldg(codes + i);
        const __half2 d = __half2half2(__ldg(scales + (i >> 1)));
        __half2 h[8];
        codes4_to_half2(w.x, h[0], h[1]);
        codes4_to_half2(w.y, h[2], h[3]);
        codes4_to_half2(w.z, h[4], h[5]);
        codes4_to_half2(w.w, h[6], h[7]);
#pragma unroll
        for (int j = 0; j < 8; j++) h[j] = __hmul2(h[j], d); // f16(q) * d rounded to f16
        dst[2 * i] = make_uint4(h2_as_u32(h[0]), h2_as_u32(h[1]), h2_as_u32(h[2]), h2_as_u32(h[3]));
        dst[2 * i + 1] = make_uint4(h2_as_u32(h[4]), h2_as_u32(h[5]), h2_as_u32(h[6]), h2_as_u32(h[7]));
    }
}

// Q4_K -> f16, sixteen quant bytes per thread: their low nibbles are sixteen values of sub-block 2p, their
// high nibbles sixteen values of sub-block 2p + 1 (GGUF block_q4_K: d, dmin, 12 bytes of 6-bit scales and
// mins, 128 bytes of nibbles).  Same arithmetic, value by value, as q4k_element: (d * sc) * q - dmin * m
// with every step rounded to f32, then one rounding to f16.
__global__ void __launch_bounds__(256) dequant_q4k_f16_vec_kernel(const uint8_t *src, __half *dst, long long n_units) {
    // the next kernel may start its prologue now; this one's stream predecessor may still be reading what it writes
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long u = (long long)blockIdx.x * blockDim.x + threadIdx.x; u < n_units; u += stride) {
        const long long blk_i = u >> 3;           // super-block of 256 values
        const int p = (int)(u & 7) >> 1;          // pair of sub-blocks
        const int h = (int)(u & 1);               // which sixteen of the pair's thirty-two bytes
        const uint8_t *blk = src + blk_i * 144;
        const uint4 head = __ldg(reinterpret_cast<const uint4 *>(blk));
        const uint4 qs = __ldg(reinterpret_cast<const uint4 *>(blk + 16 + 32 * p + 16 * h));
        const __half2 dd = *reinterpret_cast<const __half2 *>(&head.x);
        const float d = __low2float(dd), dmin = __high2float(dd);
        const uint8_t *sb = reinterpret_cast<const uint8_t *>(&head) + 4;
        int sc0, m0, sc1, m1;
        q4k_scale_min(2 * p, sb, sc0, m0);
        q4k_scale_min(2 * p + 1, sb, sc1, m1);
        const float ds0 = __fmul_rn(d, (float)sc0), dm0 = __fmul_rn(dmin, (float)m0);
        const float ds1 = __fmul_rn(d, (float)sc1), dm1 = __fmul_rn(dmin, (float)m1);
        const uint32_t w[4] = {qs.x, qs.y, qs.z, qs.w};
        uint32_t lo[8], hi[8];
#pragma unroll
        for (int i = 0; i < 4; i++) {
#pragma unroll
            for (int b = 0; b < 4; b += 2) {
                const uint32_t q0 = (w[i] >> (8 * b)) & 0xFFu, q1 = (w[i] >> (8 * b + 8)) & 0xFFu;
                const __half2 l2 = __halves2half2(__float2half_rn(__fsub_rn(__fmul_rn(ds0, (float)(q0 & 15u)), dm0)),
                                                  __float2half_rn(__fsub_rn(__fmul_rn(ds0, (float)(q1 & 15u)), dm0)));
                const __half2 h2 = __halves2half2(__float2half_rn(__fsub_rn(__fmul_rn(ds1, (float)(q0 >> 4)), dm1)),
                                                  __float2half_rn(__fsub_rn(__fmul_rn(ds1, (float)(q1 >> 4)), dm1)));
                lo[i * 2 + b / 2] = *reinterpret_cast<const uint32_t *>(&l2);
                hi[i * 2 + b / 2] = *reinterpret_cast<const uint32_t *>(&h2);
            }
        }
        __half *o = dst + blk_i * 256 + (2 * p) * 32 + 16 * h;
        reinterpret_cast<uint4 *>(o)[0] = make_uint4(lo[0], lo[1], lo[2], lo[3]);
        reinterpret_cast<uint4 *>(o)[1] = make_uint4(lo[4], lo[5], lo[6], lo[7]);
        reinterpret_cast<uint4 *>(o + 32)[0] = make_uint4(hi[0], hi[1], hi[2], hi[3]);
        reinterpret_cast<uint4 *>(o + 32)[1] = make_uint4(hi[4], hi[5], hi[6], hi[7]);
    }
}

// the largest finite magnitude among eight bf16 values (0 when none is finite)
__device__ __forceinline__ float finite_amax8(const uint4 v) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    float m = 0.f;
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const float lo = fabsf(__uint_as_float(w[j] << 16)), hi = fabsf(__uint_as_float(w[j] & 0xFFFF0000u));
        if (lo <= 3.0e38f) m = fmaxf(m, lo); // false for infinities and NaNs
        if (hi <= 3.0e38f) m = fmaxf(m, hi);
    }
    return m;
}
// eight bf16 values times a power of two, as f16
__device__ __forceinline__ uint4 scaled_f16x8(const uint4 v, float down) {
    uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; j++)
        w[j] = h2_as_u32(__floats2half2_rn(__uint_as_float(w[j] << 16) * down, __uint_as_float(w[j] & 0xFFFF0000u) * down));
    return make_uint4(w[0], w[1], w[2], w[3]);
}

// bf16 rows to f16 rows with one power-of-two factor per row.  f16 keeps every bit of a bf16 mantissa but not its
// exponent range, so each row is first multiplied by 2^-sh, sh chosen from the row's largest finite magnitude m so
// that m * 2^-sh lies in [2^14, 2^15): nothing saturates, and only elements more than 2^29 below the row's largest lose
// bits (in the f16 subnormals).  scale[row] = 2^sh goes back onto the f32 accumulators in the GEMM's epilogue: both
// multiplications are exact.  Infinities and NaNs pass through as they are; a row without a finite non-zero element
// has the factor 1.
__global__ void __launch_bounds__(256) cast_bf16_f16_rows_kernel(const __nv_bfloat16 *__restrict__ src, __half *__restrict__ dst,
                                                                 float *__restrict__ scale, long long rows, int K) {
    // the next kernel may start its prologue now; this one's stream predecessor may still be reading what it writes
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // One warp per row: the row's largest magnitude needs shuffles only, and rows of up to 4096 values (16 loads of
    // 16 bytes per lane, all in flight together) stay in registers between the two steps; longer rows are read a
    // second time, out of L2.
    constexpr int HOLD = 16;
    const int lane = threadIdx.x & 31;
    const long long warp = (long long)blockIdx.x * 8 + (threadIdx.x >> 5), n_warps = (long long)gridDim.x * 8;
    const bool vec = (K % 8) == 0; // then every row starts on a 16-byte boundary
    const int n8 = vec ? K / 8 : 0;
    const bool held = n8 <= HOLD * 32;
    for (long long r = warp; r < rows; r += n_warps) {
        const __nv_bfloat16 *s = src + r * K;
        __half *d = dst + r * K;
        float m = 0.f;
        uint4 keep[HOLD];
        if (held) {
#pragma unroll
            for (int j = 0; j < HOLD; j++) {
                const int i = lane + 32 * j;
                keep[j] = i < n8 ? __ldg(reinterpret_cast<const uint4 *>(s) + i) : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int j = 0; j < HOLD; j++) m = fmaxf(m, finite_amax8(keep[j]));
        } else {
            for (int i = lane; i < n8; i += 32) m = fmaxf(m, finite_amax8(__ldg(reinterpret_cast<const uint4 *>(s) + i)));
        }
        for (int i = n8 * 8 + lane; i < K; i += 32) {
            const float a = fabsf(__bfloat162float(s[i]));
            if (a <= 3.0e38f) m = fmaxf(m, a);
        }
#pragma unroll
        for (int o = 16; o; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        int sh = 0;
        if (m > 0.f) {
            int e;
            frexpf(m, &e); // m = f * 2^e, f in [0.5, 1)
            sh = min(max(e - 15, -126), 112); // 2^126 and 2^-126 are still normal f32 values
        }
        const float down = ldexpf(1.f, -sh);
        if (held) {
#pragma unroll
            for (int j = 0; j < HOLD; j++) {
                const int i = lane + 32 * j;
                if (i < n8) reinterpret_cast<uint4 *>(d)[i] = scaled_f16x8(keep[j], down);
            }
        } else {
            for (int i = lane; i < n8; i += 32)
                reinterpret_cast<uint4 *>(d)[i] = scaled_f16x8(__ldg(reinterpret_cast<const uint4 *>(s) + i), down);
        }
        for (int i = n8 * 8 + lane; i < K; i += 32) d[i] = __float2half_rn(__bfloat162float(s[i]) * down);
        if (lane == 0) scale[r] = ldexpf(1.f, sh);
    }
}

// [stack][rows][cols] -> [stack][cols][dst_ld], 32 x 32 tiles through padded shared memory so that both
// the reads and the writes run along the contiguous dimension; dst_ld >= rows, the columns past `rows`
// of every output row are zero.  T: a 2- or 4-byte element.
template <typename T>
__global__ void __launch_bounds__(256) transpose_kernel(const T *__restrict__ src, T *__restrict__ dst, int rows, int cols, int dst_ld) {
    __shared__ T tile[32][33];
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const long long base = (long long)blockIdx.z * rows * cols, dbase = (long long)blockIdx.z * cols * dst_ld;
    const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5; // 32 x 8
#pragma unroll
    for (int j = 0; j < 32; j += 8) {
        const int r = r0 + ty + j, c = c0 + tx;
        tile[ty + j][tx] = (r < rows && c < cols) ? src[base + (long long)r * cols + c] : T(0);
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < 32; j += 8) {
        const int c = c0 + ty + j, r = r0 + tx;
        if (c < cols && r < dst_ld) dst[dbase + (long long)c * dst_ld + r] = tile[tx][ty + j];
    }
}

// rows of `k` 16-bit elements -> rows of `k_pad` (a multiple of 8), zero filled: one 16-byte store per thread
__global__ void __launch_bounds__(256) pad_rows16_kernel(const uint16_t *__restrict__ src, uint4 *__restrict__ dst, long long rows, int k, int k_pad) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int groups = k_pad / 8;
    const long long total = rows * groups;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / groups;
        const int c0 = (int)(i - r * groups) * 8;
        const uint16_t *s = src + r * k + c0;
        uint16_t v[8];
#pragma unroll
        for (int j = 0; j < 8; j++) v[j] = c0 + j < k ? s[j] : (uint16_t)0;
        dst[i] = make_uint4(v[0] | ((uint32_t)v[1] << 16), v[2] | ((uint32_t)v[3] << 16), v[4] | ((uint32_t)v[5] << 16),
                            v[6] | ((uint32_t)v[7] << 16));
    }
}

} // namespace

// src [stacks][rows][cols] -> dst [stacks][cols][dst_ld], dst_ld >= rows (zero filled beyond rows); elem_size 2 or 4.
cudaError_t launch_transpose(const void *src, void *dst, int stacks, int rows, int cols, int dst_ld, int elem_size, cudaStream_t stream) {
    if (stacks <= 0 || rows <= 0 || cols <= 0) return cudaSuccess;
    if (dst_ld < rows || stacks > 65535 || (dst_ld + 31) / 32 > 65535) return cudaErrorInvalidValue;
    const dim3 grid((cols + 31) / 32, (dst_ld + 31) / 32, stacks);
    if (elem_size == 2)
        return launch_pdl(transpose_kernel<uint16_t>, grid, dim3(256), 0, stream, (const uint16_t *)src, (uint16_t *)dst, rows, cols, dst_ld);
    if (elem_size == 4)
        return launch_pdl(transpose_kernel<uint32_t>, grid, dim3(256), 0, stream, (const uint32_t *)src, (uint32_t *)dst, rows, cols, dst_ld);
    return cudaErrorInvalidValue;
}

// [rows][k] 16-bit -> [rows][k_pad], k_pad a multiple of 8 and >= k, zero filled; dst 16-byte aligned.
cudaError_t launch_pad_rows16(const void *src, void *dst, long long rows, int k, int k_pad, int sm_count, cudaStream_t stream) {
    if (rows <= 0 || k <= 0) return cudaSuccess;
    if (k_pad < k || k_pad % 8 != 0) return cudaErrorInvalidValue;
    const long long total = rows * (k_pad / 8);
    const int blocks = (int)std::min<long long>((total + 255) / 256, (long long)sm_count * 16);
    return launch_pdl(pad_rows16_kernel, dim3(blocks), dim3(256), 0, stream, (const uint16_t *)src, (uint4 *)dst, rows, k, k_pad);
}

// [rows][2*ff] (gate | up, as the plain Linear node leaves them) -> [rows][ff] = up * cast(silu(full(gate)))
template <typename T>
__global__ void __launch_bounds__(256) silu_mul_kernel(const T *__restrict__ full, T *__restrict__ out, long long rows, int ff) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const long long n = rows * ff, stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const long long r = i / ff;
        const int c = (int)(i - r * ff);
        const T *row = full + r * 2 * ff;
        out[i] = silu_mul_value<T>(row[c], row[ff + c]);
    }
}

cudaError_t launch_silu_mul(const void *full, void *out, long long rows, int ff, rt_dtype dt, int sm_count, cudaStream_t stream) {
    const long long n = rows * ff;
    if (n == 0) return cudaSuccess;
    const long long want = (n + 255) / 256;
    const int blocks = (int)(want < (long long)sm_count * 16 ? want : (long long)sm_count * 16);
    switch (dt) {
    case RT_F16: return launch_pdl(silu_mul_kernel<__half>, dim3(blocks), dim3(256), 0, stream, (const __half *)full, (__half *)out, rows, ff);
    case RT_BF16:
        return launch_pdl(silu_mul_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (const __nv_bfloat16 *)full,
                          (__nv_bfloat16 *)out, rows, ff);
    case RT_F32: return launch_pdl(silu_mul_kernel<float>, dim3(blocks), dim3(256), 0, stream, (const float *)full, (float *)out, rows, ff);
    default: return cudaErrorInvalidValue;
    }
}

cudaError_t launch_cast_bf16_f16_rows(const void *src, void *dst, float *scale, long long rows, int K, int sm_count, cudaStream_t stream) {
    if (rows == 0 || K == 0) return cudaSuccess;
    const long long want = (rows + 7) / 8; // eight rows (warps) per block
    const int blocks = (int)(want < (long long)sm_count * 8 ? want : (long long)sm_count * 8);
    return launch_pdl(cast_bf16_f16_rows_kernel, dim3(blocks), dim3(256), 0, stream, (const __nv_bfloat16 *)src, (__half *)dst, scale, rows, K);
}

cudaError_t launch_dequant(rt_dtype dt, long long numel, const void *src, const void *scales, void *dst, rt_dtype out_dt,
                           int sm_count, cudaStream_t stream) {
    if (numel == 0) return cudaSuccess;
    const int threads = 256;
    long long want = (numel + threads - 1) / threads;
    const int blocks = (int)(want < (long long)sm_count * 16 ? want : (long long)sm_count * 16);
    if (dt == RT_Q8_0H && out_dt == RT_F16) {
        if (numel % 16 == 0 && (reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) % 16 == 0) {
            long long n16 = numel / 16;
            long long w2 = (n16 + threads - 1) / threads;
            const int b2 = (int)(w2 < (long long)sm_count * 16 ? w2 : (long long)sm_count * 16);
            return launch_pdl(dequant_q8h_f16_vec_kernel, dim3(b2), dim3(threads), 0, stream, (const uint4 *)src, (const __half *)scales, (uint4 *)dst, n16);
        } else {
            dequant_kernel<LK_Q8H, __half><<<blocks, threads, 0, stream>>>(src, scales, (__half *)dst, numel);
        }
    } else if (dt == RT_Q8_0H && out_dt == RT_F32) {
        dequant_kernel<LK_Q8H, float><<<blocks, threads, 0, stream>>>(src, scales, (float *)dst, numel);
    } else if (dt == RT_Q8_0F && out_dt == RT_F32) {
        dequant_kernel<LK_Q8F, float><<<blocks, threads, 0, stream>>>(src, scales, (float *)dst, numel);
    } else if (dt == RT_Q4_K && out_dt == RT_F32) {
        dequant_kernel<LK_Q4K, float><<<blocks, threads, 0, stream>>>(src, scales, (float *)dst, numel);
    } else if (dt == RT_Q4_K && out_dt == RT_F16) {
        if (numel % 256 == 0 && (reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) % 16 == 0) {
            const long long n_units = numel / 32;
            const long long w2 = (n_units + threads - 1) / threads;
            const int b2 = (int)(w2 < (long long)sm_count * 16 ? w2 : (long long)sm_count * 16);
            return launch_pdl(dequant_q4k_f16_vec_kernel, dim3(b2), dim3(threads), 0, stream, (const uint8_t *)src, (__half *)dst, n_units);
        } else {
            dequant_kernel<LK_Q4K, __half><<<blocks, threads, 0, stream>>>(src, scales, (__half *)dst, numel);
        }
    } else {
        return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

} // namespace rt
