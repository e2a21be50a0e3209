// A Linear-shaped Q8_0 GEMM that never allocates device memory.
//
// The regular path (rt_matmul_plan) gives each plan its own cudaMalloc'ed buffer for the
// dequantised weights.  Some hosts cannot accept that: a runtime that hands the whole device
// to its own planner (as ratchet-core's BufferAllocator does for a resolved graph) and forbids
// allocations behind its back, or a latency-critical serving loop where cudaMalloc's implicit
// device synchronisation is not tolerable.  For them this file keeps the scratch in a fixed
// array that is part of the loaded module: every GPU that loads the library carries
// RT_STATIC_SCRATCH_BYTES of it until the process exits, and no call here reaches cudaMalloc,
// cudaFree or any allocating library routine.
//
// The array's name in host code is only a handle for the runtime, not an address a kernel can
// use.  Its device address is looked up once per device with cudaGetSymbolAddress, with that
// device current, and that address is what the kernels receive.
#include <cuda_runtime.h>

#include <mutex>
#include <string>

#include "kernels.hpp"
#include "ratchet_b200.h"
#include "spec.hpp"

using namespace rt;

static __device__ __align__(256) unsigned char g_static_scratch[RT_STATIC_SCRATCH_BYTES];

namespace {
constexpr int MAX_DEVICES = 64;
std::mutex g_setup_mu;
void *g_scratch_addr[MAX_DEVICES] = {};
} // namespace

extern "C" rt_status rt_linear_q8_0_static_scratch(rt_device *dev, const void *w, const void *x, const void *bias, void *out,
                                                   int64_t rows, int64_t n, int64_t k, int32_t epilogue, void *stream) {
    if (!dev || !w || !x || !out) return fail(RT_ERR_ARG, "rt_linear_q8_0_static_scratch: null argument");
    if (epilogue != RT_EPILOGUE_NONE && epilogue != RT_EPILOGUE_GELU_TANH)
        return fail(RT_ERR_ARG, "rt_linear_q8_0_static_scratch: invalid epilogue");
    if (rows < 1 || n < 1 || k < 32 || k % 32 != 0 || rows >= (int64_t(1) << 31) || n >= (int64_t(1) << 31) || k >= (int64_t(1) << 31))
        return fail(RT_ERR_SHAPE, "rt_linear_q8_0_static_scratch: rows, n >= 1 and k a positive multiple of 32 are required");
    const uint64_t need = (uint64_t)n * (uint64_t)k * 2;
    if (need > (uint64_t)RT_STATIC_SCRATCH_BYTES)
        return fail(RT_ERR_UNSUPPORTED, "rt_linear_q8_0_static_scratch: the weight needs " + std::to_string(need) +
                                            " bytes of scratch, the built-in array holds " +
                                            std::to_string((uint64_t)RT_STATIC_SCRATCH_BYTES) +
                                            "; use rt_matmul_plan for larger weights");
    const int ordinal = rt_device_ordinal(dev), sm_count = rt_device_sm_count(dev);
    if (ordinal < 0 || ordinal >= MAX_DEVICES) return fail(RT_ERR_ARG, "device ordinal out of range");
    if (out == w || out == x || out == bias) return fail(RT_ERR_INVARIANT, "Matmul is never in place: out aliases an operand");
    // the dequantising pass and the GEMM's tensor maps read 16 bytes at a time
    if ((reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(x)) % 16 != 0)
        return fail(RT_ERR_ARG, "rt_linear_q8_0_static_scratch: w and x must be 16-byte aligned");
    cudaError_t e = cudaSetDevice(ordinal);
    if (e != cudaSuccess) return fail(RT_ERR_CUDA, std::string("cudaSetDevice: ") + cudaGetErrorString(e));
    void *scratch = nullptr;
    {
        // one-time set-up per device (the first call on a device; make it before any stream capture)
        std::lock_guard<std::mutex> lk(g_setup_mu);
        if (!g_scratch_addr[ordinal]) {
            void *p = nullptr;
            e = cudaGetSymbolAddress(&p, g_static_scratch);
            if (e != cudaSuccess || !p)
                return fail(RT_ERR_CUDA, std::string("cudaGetSymbolAddress(static scratch): ") + cudaGetErrorString(e));
            g_scratch_addr[ordinal] = p;
        }
        scratch = g_scratch_addr[ordinal];
    }
    if (!umma_gemm_supported(k)) return fail(RT_ERR_UNSUPPORTED, "the tensor-core GEMM is not available for this k");
    cudaStream_t st = stream ? (cudaStream_t)stream : (cudaStream_t)rt_device_stream(dev);
    // codes | pad to 256 | f16 scales (crates/ratchet-core/src/dtype/blocks.rs:61-74 of the reference)
    const uint64_t numel = (uint64_t)n * (uint64_t)k;
    const void *scales = (const char *)w + (numel + 255) / 256 * 256;
    // every element of the first n*k halves is rewritten before the GEMM reads it, and the GEMM's
    // tensor map stops at n*k: nothing left over from an earlier call is ever read, nothing needs zeroing
    e = launch_dequant(RT_Q8_0H, (long long)numel, w, scales, scratch, RT_F16, sm_count, st);
    if (e == cudaSuccess) {
        const int bn = umma_pick_bn(rows, n, 1, sm_count);
        e = launch_gemm_umma(x, RT_F16, scratch, RT_F16, out, RT_F16, (int)rows, (int)n, (int)k, 1, 1, 1, bias, RT_F16,
                             bias ? BIAS_PER_N : BIAS_NONE, epilogue, bn, sm_count, st);
    }
    if (e != cudaSuccess) return fail(RT_ERR_CUDA, std::string("rt_linear_q8_0_static_scratch launch: ") + cudaGetErrorString(e));
    return RT_OK;
}
