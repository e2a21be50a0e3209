// Launchers of the device kernels (one translation unit each).
#pragma once
#include <mutex>
#include <string>
#include <vector>
#include <cuda_runtime.h>

#include "common.cuh"

namespace rt {

// Launch with programmatic stream serialisation: the kernel may start (and run whatever precedes its
// griddepcontrol.wait) while its stream predecessor is still running.
template <typename... KArgs, typename... Args>
cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args &&...args) {
    cudaLaunchConfig_t lc = {};
    lc.gridDim = grid;
    lc.blockDim = block;
    lc.dynamicSmemBytes = smem;
    lc.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = attr;
    lc.numAttrs = 1;
    return cudaLaunchKernelEx(&lc, kernel, static_cast<KArgs>(args)...);
}

// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) acts on the current device only, and launches may come from
// several host threads: one record per device ordinal of the largest size set so far, under a mutex.
class SmemAttr {
    std::mutex mu_;
    size_t set_[64] = {};

  public:
    template <typename Kernel> cudaError_t ensure(Kernel kernel, size_t bytes) {
        int dev = 0;
        cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess) return e;
        if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
        std::lock_guard<std::mutex> lk(mu_);
        if (bytes <= set_[dev]) return cudaSuccess;
        e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
        if (e == cudaSuccess) set_[dev] = bytes;
        return e;
    }
};

// General CUDA-core kernels: any legal node.
cudaError_t launch_matmul_simt(const MatmulParams &p, rt_dtype lhs_dt, rt_dtype act_dt, bool gemv, cudaStream_t stream);
// one row of a dense lhs against a dense rhs stored [K][N] of the same dtype (M == 1, no transposes)
int rowvec_mat_chunks(int N, int K, int stacks, int sm_count); // CTAs that share the k rows (1: no partial sums)
cudaError_t launch_rowvec_mat(const MatmulParams &p, rt_dtype dt, int chunks, float *partial, cudaStream_t stream);

// Q8_0 x f16 GEMV / skinny GEMM on warp MMAs.  nv = columns of op(rhs), 1..16 (rhs stored [nv][K]).
// pick_split returns the K split (cluster size), or 0 when the shape does not fit the kernel.
// lhs_constant: the weight bytes are not written by any work in flight on the stream, so the
// kernel may request them before it waits for its stream predecessor.
int q8_gemv_mma_pick_split(int M, int K, int sm_count, int scale_size);
cudaError_t launch_q8_gemv_mma(const MatmulParams &p, bool f32_scales, int nv, int split, bool lhs_constant, cudaStream_t stream);
cudaError_t gemv_take_error(int *site, cudaStream_t stream);

// Q8_0H x f16 GEMV on tcgen05 kind::i8 (one activation vector, stacks == 1, K % 256 == 0).
struct GemvUmmaConfig {
    int split, clusters, rb, rb8, ks, ring, stage_bytes, b_bytes;
    size_t smem_bytes;
};
bool q8_gemv_umma_config(int M, int K, int sm_count, GemvUmmaConfig *cfg);
cudaError_t launch_q8_gemv_umma(const MatmulParams &p, const GemvUmmaConfig &cfg, bool lhs_constant, cudaStream_t stream);
cudaError_t gemv_umma_take_error(int *site, cudaStream_t stream);

// A list of such GEMVs (constant weights, node l+1 may read what node l wrote) as one persistent
// cooperative kernel with grid barriers between the nodes.  gemv_chain_create returns cudaSuccess
// with *out == nullptr and a reason when the list is not one the kernel takes.
struct GemvChain;
cudaError_t gemv_chain_create(const std::vector<MatmulParams> &nodes, int device, int sm_count, GemvChain **out, std::string *why);
cudaError_t gemv_chain_launch(GemvChain *chain, cudaStream_t stream);
void gemv_chain_destroy(GemvChain *chain);
const char *gemv_chain_name(const GemvChain *chain);
cudaError_t gemv_chain_take_error(int *site, cudaStream_t stream);

// Q4_K x f16 GEMV / skinny GEMM on warp MMAs.  nv = columns of op(rhs), 1..16 (rhs stored [nv][K]).
int q4k_gemv_pick_split(int M, int K, int nv, int stacks, int sm_count); // split | groups per CTA << 8 | weight buffers << 16, or 0
cudaError_t launch_q4k_gemv(const MatmulParams &p, int nv, int config, bool lhs_constant, cudaStream_t stream);
cudaError_t gemv_q4k_take_error(int *site, cudaStream_t stream);

// Q4_K GEMV / skinny GEMM through tensor memory (gemv_q4k_umma.cu): raw super-blocks by TMA, nibbles to int8 codes
// in shared memory, tcgen05.mma kind::i8 against block-floating digits of the activations.
struct Q4kUmmaConfig {
    int split, clusters, rb, rb8, ks, raw_ring, a_ring, nvmax, b_bytes;
    size_t smem_bytes;
};
bool q4k_gemv_umma_config(int M, int K, int nv, int sm_count, Q4kUmmaConfig *cfg);
cudaError_t launch_q4k_gemv_umma(const MatmulParams &p, int nv, const Q4kUmmaConfig &cfg, bool lhs_constant, cudaStream_t stream);
cudaError_t gemv_q4k_umma_take_error(int *site, cudaStream_t stream);

// Dense f32 GEMM on the tensor cores, three TF32 MMAs per product (f32-class accuracy): D[R][S] = P[R][K] . Q[S][K]^T.
bool umma_tf32_supported(long long K);
int umma_tf32_pick_bn(int R, int S, int stacks, int sm_count);
bool umma_tf32_presplit_pays(int S, int bn);
cudaError_t launch_gemm_umma_tf32x3(const void *P, const void *Q, void *out, int R, int S, int K, int stacks, int p_stack, int q_stack,
                                    const void *bias, int bias_dt, int bias_mode, int epilogue, int bn, void *p_split, int sm_count,
                                    cudaStream_t stream);
cudaError_t umma_tf32_take_error(int *site, cudaStream_t stream);

// Tensor-core GEMM (tcgen05): D[R][S] = P[R][K] . Q[S][K]^T, 16-bit K-major operands, bias along S.
// Several destinations for one result: see UmmaParams in gemm_umma.cu.  p_scale [p_stack][R] / q_scale [q_stack][S]:
// optional f32 factors per row of P / of Q, multiplied onto the accumulators before bias and epilogue.
struct UmmaScatter {
    int n_out;
    void *outs[RT_MAX_PEERS];
    long long out_ld, out_col;
};
bool umma_gemm_supported(long long K);
// Tile width: 128 or 256 columns on one CTA per SM, or UMMA_BN_PAIR: 256 x 256 tiles on pairs of CTAs (cta_group::2)
constexpr int UMMA_BN_PAIR = 512;
int umma_pick_bn(long long R, long long S, long long stacks, int sm_count);
cudaError_t launch_gemm_umma(const void *P, rt_dtype p_dt, const void *Q, rt_dtype q_dt, void *out, rt_dtype out_dt,
                             int R, int S, int K, int stacks, int p_stack, int q_stack, const void *bias, int bias_dt,
                             int bias_mode, int epilogue, int bn, int sm_count, cudaStream_t stream,
                             const UmmaScatter *scatter = nullptr, const float *p_scale = nullptr, const float *q_scale = nullptr);
// Reads and clears the device flag a kernel sets when one of its bounded waits expires.
cudaError_t umma_take_error(int *site, cudaStream_t stream);

// Block-format tensor -> f32 / f16 values.
cudaError_t launch_dequant(rt_dtype dt, long long numel, const void *src, const void *scales, void *dst, rt_dtype out_dt,
                           int sm_count, cudaStream_t stream);

// bf16 [rows][K] -> f16 [rows][K] * 2^-sh(row) with scale[row] = 2^sh(row): the activations of a quantised-weight
// tensor-core GEMM, brought into f16's exponent range row by row (nothing saturates; infinities and NaNs pass through).
cudaError_t launch_cast_bf16_f16_rows(const void *src, void *dst, float *scale, long long rows, int K, int sm_count, cudaStream_t stream);
// [rows][2*ff] (gate | up) -> [rows][ff] = up * silu(gate), the second launch of a RT_EPILOGUE_SILU_MUL node on the routes
// that do not fuse it
cudaError_t launch_silu_mul(const void *full, void *out, long long rows, int ff, rt_dtype dt, int sm_count, cudaStream_t stream);
// [stacks][rows][cols] -> [stacks][cols][dst_ld] (zero filled past `rows`), elements of 2 or 4 bytes: the pass that
// makes an operand K-major; launch_pad_rows16 gives 16-bit rows a length that is a multiple of 8
cudaError_t launch_transpose(const void *src, void *dst, int stacks, int rows, int cols, int dst_ld, int elem_size, cudaStream_t stream);
cudaError_t launch_pad_rows16(const void *src, void *dst, long long rows, int k, int k_pad, int sm_count, cudaStream_t stream);

} // namespace rt
