// Device-side helpers shared by the Matmul kernels: operand decode, the reference's epilogue
// chain, and the launch parameter block.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cuda/std/type_traits>

#include "ratchet_b200.h"

namespace rt {

// Bias addressing (gemm.rs:468-476, gemv.rs:476-490 of the reference)
enum BiasMode : int { BIAS_NONE = 0, BIAS_PER_N = 1, BIAS_PER_M = 2 };

// Everything a kernel needs to know about one Matmul node.  M/N/K are the extents of
// op(lhs) [M,K] and op(rhs) [K,N]; the output is [stacks][M][N], or [stacks][N][M] when
// trans_out.  Batch b reads lhs[b % lhs_stack] and rhs[b % rhs_stack] (gemm.rs:359-361).
struct MatmulParams {
    const void *lhs;        // codes / values of the lhs
    const void *lhs_scales; // Q8_0: scales segment (lhs + align256(numel)); else null
    const void *rhs;
    const void *bias;
    void *out;
    int M, N, K;
    int stacks, lhs_stack, rhs_stack;
    int trans_lhs, trans_rhs, trans_out;
    int bias_mode;
    int bias_dt; // rt_dtype of the bias
    int epilogue;
    long long lhs_batch_elems; // M*K
    long long lhs_batch_scale_bytes;
};

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// tanh GELU of ops/unary.rs:97-119 in f32.  tanh(u) = 1 - 2/(1+exp(2u)); saturates to +-1 for
// |u| large exactly as the reference's safe_tanh does at |u| >= 10.
__device__ __forceinline__ float gelu_tanh_f32(float v) {
    float u = v * fmaf(0.035677407f, v * v, 0.7978846f);
    float e = __expf(2.0f * u);
    float t = 1.0f - __fdividef(2.0f, 1.0f + e);
    return v * fmaf(0.5f, t, 0.5f);
}

__device__ __forceinline__ float load_bias(const void *bias, int bias_dt, int idx) {
    switch (bias_dt) {
    case RT_F16: return __half2float(((const __half *)bias)[idx]);
    case RT_BF16: return __bfloat162float(((const __nv_bfloat16 *)bias)[idx]);
    default: return ((const float *)bias)[idx];
    }
}

// The reference's epilogue: val = dt(acc) + bias evaluated in dt (gemm.rs:485, gemv.rs:480);
// the optional GELU is the cast -> f32 GELU -> cast chain of whisper/mlp.rs:18-22.
// bf16 outputs are this library's extension (the reference has no bf16 Matmul): bias and GELU are
// applied to the f32 accumulator and the result is rounded once.  A bf16 rounding is 2^-9
// relative, so the reference's round-then-add chain would by itself cost more than the path's
// 1e-3 rel-L2 budget.
template <typename OutT>
__device__ __forceinline__ OutT epilogue_value(float acc, bool has_bias, float bias, int epilogue) {
    if (sizeof(OutT) == 2 && !cuda::std::is_same<OutT, __half>::value) {
        float v = has_bias ? acc + bias : acc;
        if (epilogue == RT_EPILOGUE_GELU_TANH) v = gelu_tanh_f32(v);
        return from_f32<OutT>(v);
    }
    OutT v = from_f32<OutT>(acc);
    if (has_bias) v = from_f32<OutT>(to_f32(v) + bias); // one rounding of the f32 sum == the add in dt
    if (epilogue == RT_EPILOGUE_GELU_TANH) v = from_f32<OutT>(gelu_tanh_f32(to_f32(v)));
    return v;
}

// sigmoid and silu of ops/unary.rs:121-131,165-175 in f32, branch for branch: exp(v) / (1 + exp(v)) for
// v >= 0 (which is NaN once exp(v) overflows, v > 88.7, as it is in the reference's shader), 1 / (1 + exp(-v))
// below zero.
__device__ __forceinline__ float silu_ref_f32(float v) {
    const float sg = v >= 0.f ? expf(v) / (1.0f + expf(v)) : 1.0f / (1.0f + expf(-v));
    return v * sg;
}

// up * cast(silu(full(gate))) of crates/ratchet-models/src/phi3/mlp.rs:36 on values already rounded to the
// output dtype: f16 rounds silu and then the product (the f32 product of two f16 values is exact, so one
// rounding of it is the f16 multiply); f32 needs no rounding; bf16 (no reference counterpart) rounds the
// product only.
template <typename OutT> __device__ __forceinline__ OutT silu_mul_value(OutT gate, OutT up) {
    const float sv = silu_ref_f32(to_f32(gate));
    if (cuda::std::is_same<OutT, __half>::value) return from_f32<OutT>(to_f32(up) * to_f32(from_f32<OutT>(sv)));
    return from_f32<OutT>(to_f32(up) * sv);
}

// Four int8 codes in a 32-bit word -> two half2 {c0,c1}, {c2,c3}, exact for every int8 value.
// (code ^ 0x80) is the byte of 1024 + (code + 128) in binary16 (0x6400 | byte); subtracting 1152
// leaves the signed code.
__device__ __forceinline__ void codes4_to_half2(uint32_t w, __half2 &lo, __half2 &hi) {
    uint32_t x = w ^ 0x80808080u;
    uint32_t a = __byte_perm(x, 0x64646464u, 0x4140); // bytes: x0, 0x64, x1, 0x64
    uint32_t b = __byte_perm(x, 0x64646464u, 0x4342); // bytes: x2, 0x64, x3, 0x64
    const __half2 bias = __half2half2(__ushort_as_half((unsigned short)0x6480)); // 1152.0
    lo = __hsub2(*reinterpret_cast<__half2 *>(&a), bias);
    hi = __hsub2(*reinterpret_cast<__half2 *>(&b), bias);
}

// Named barrier `id` over `nthreads` threads that also returns the OR of every thread's `pred`: all of them
// take the same decision (to leave a loop after a bounded wait ran out, say), so none is left behind at the
// next barrier.
__device__ __forceinline__ bool bar_red_or(int id, int nthreads, bool pred) {
    int r;
    asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.s32 p, %3, 0;\n\tbarrier.cta.red.or.pred q, %1, %2, p;\n\tselp.s32 %0, 1, 0, q;\n\t}\n"
                 : "=r"(r) : "r"(id), "r"(nthreads), "r"((int)pred) : "memory");
    return r != 0;
}

__device__ __forceinline__ uint32_t h2_as_u32(__half2 h) { return *reinterpret_cast<uint32_t *>(&h); }

} // namespace rt
