// General-purpose Matmul kernels on the CUDA cores: every dtype pair, transpose combination,
// batch broadcast, ragged extent and bias / GELU option of the node.  They cover what the
// specialised kernels do not (f32 operands, transposed lhs, non-transposed rhs, odd extents) with
// f32 products and f32 accumulation.
//
// Roles in the reference: the scalar GEMM of crates/ratchet-core/src/ops/gemm.rs:342-492 and the
// workgroup GEMV of crates/ratchet-core/src/ops/gemv.rs:181-331.
#include <algorithm>

#include "decode.cuh"
#include "kernels.hpp"

namespace rt {

namespace {

constexpr int BM = 64, BN = 64, BK = 16;

template <typename ActT>
__device__ __forceinline__ float rhs_element(const void *rhs, long long idx) {
    return to_f32(((const ActT *)rhs)[idx]);
}

template <int KIND, typename ActT>
__global__ void __launch_bounds__(256) gemm_simt_kernel(MatmulParams p) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Bs[BK][BN + 4];
    const int t = threadIdx.x, tx = t & 15, ty = t >> 4;
    const int batch = blockIdx.z;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const long long abase = (long long)(batch % p.lhs_stack) * p.M * p.K;
    const long long bbase = (long long)(batch % p.rhs_stack) * p.K * p.N;

    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < p.K; k0 += BK) {
#pragma unroll
        for (int i = 0; i < 4; i++) {
            int ml, kl;
            if (p.trans_lhs) { ml = t & 63; kl = (t >> 6) + 4 * i; }
            else             { kl = t & 15; ml = (t >> 4) + 16 * i; }
            const int m = m0 + ml, k = k0 + kl;
            float v = 0.f;
            if (m < p.M && k < p.K)
                v = lhs_element<KIND>(p.lhs, p.lhs_scales, abase + (p.trans_lhs ? (long long)k * p.M + m : (long long)m * p.K + k));
            As[kl][ml] = v;
        }
#pragma unroll
        for (int i = 0; i < 4; i++) {
            int nl, kl;
            if (p.trans_rhs) { kl = t & 15; nl = (t >> 4) + 16 * i; }
            else             { nl = t & 63; kl = (t >> 6) + 4 * i; }
            const int n = n0 + nl, k = k0 + kl;
            float v = 0.f;
            if (n < p.N && k < p.K)
                v = rhs_element<ActT>(p.rhs, bbase + (p.trans_rhs ? (long long)n * p.K + k : (long long)k * p.N + n));
            Bs[kl][nl] = v;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; kk++) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; i++) a[i] = As[kk][ty + 16 * i];
#pragma unroll
            for (int j = 0; j < 4; j++) b[j] = Bs[kk][tx + 16 * j];
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }

    const bool has_bias = p.bias_mode != BIAS_NONE;
    ActT *out = (ActT *)p.out + (long long)batch * p.M * p.N;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int m = m0 + ty + 16 * i;
        if (m >= p.M) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int n = n0 + tx + 16 * j;
            if (n >= p.N) continue;
            float bias = 0.f;
            if (has_bias) bias = load_bias(p.bias, p.bias_dt, p.bias_mode == BIAS_PER_M ? m : n);
            const ActT v = epilogue_value<ActT>(acc[i][j], has_bias, bias, p.epilogue);
            out[p.trans_out ? (long long)n * p.M + m : (long long)m * p.N + n] = v;
        }
    }
}

// y[r] = sum_k lhs[r][k] * x[k]: a warp takes GEMV_ROWS consecutive rows, lanes stride over K.  Several rows per
// warp keep that many independent 16-byte loads in flight per lane and share the loads of x: with one row per
// warp a short row (the Whisper logits, K = 384) is one or two dependent loads and a shuffle reduction, and the
// kernel ran at the same 16.5 us for 40 MB (f16) as for 80 MB (f32).
// GEMV_ROWS is 8 when that still gives two CTAs per SM, else 2 (a [2560, 10240] node has only 2560 rows).
template <int KIND, typename ActT, int GEMV_ROWS>
__global__ void __launch_bounds__(256) gemv_simt_kernel(MatmulParams p) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row0 = (blockIdx.x * 8 + warp) * GEMV_ROWS;
    const int batch = blockIdx.z;
    if (row0 >= p.M) return;
    const long long lbase = (long long)(batch % p.lhs_stack) * p.M * p.K;
    const ActT *x = (const ActT *)p.rhs + (long long)(batch % p.rhs_stack) * p.K;
    float acc[GEMV_ROWS];
    long long abase[GEMV_ROWS];
#pragma unroll
    for (int r = 0; r < GEMV_ROWS; r++) {
        acc[r] = 0.f;
        abase[r] = lbase + (long long)min(row0 + r, p.M - 1) * p.K; // rows past the end repeat the last one; not stored
    }
    constexpr bool dense16 = (KIND == LK_F16 || KIND == LK_BF16) && sizeof(ActT) == 2;
    constexpr bool dense32 = KIND == LK_F32 && sizeof(ActT) == 4;
    // every row starts on a 16-byte boundary when the first one does and K is a multiple of 8 (4 for f32)
    const bool aligned = ((lbase * (long long)sizeof(ActT)) % 16 == 0) && (p.K % 8 == 0) &&
                         ((reinterpret_cast<uintptr_t>(p.lhs) | reinterpret_cast<uintptr_t>(x)) % 16 == 0);
    if ((dense16 || dense32) && aligned) {
        if (dense16) {
            const ActT *w = (const ActT *)p.lhs;
            for (int k = lane * 8; k < p.K; k += 256) {
                uint4 wv[GEMV_ROWS];
#pragma unroll
                for (int r = 0; r < GEMV_ROWS; r++) wv[r] = __ldg(reinterpret_cast<const uint4 *>(w + abase[r] + k));
                const uint4 xv = __ldg(reinterpret_cast<const uint4 *>(x + k));
                const ActT *xp = reinterpret_cast<const ActT *>(&xv);
#pragma unroll
                for (int r = 0; r < GEMV_ROWS; r++) {
                    const ActT *wp = reinterpret_cast<const ActT *>(&wv[r]);
#pragma unroll
                    for (int i = 0; i < 8; i++) acc[r] = fmaf(to_f32(wp[i]), to_f32(xp[i]), acc[r]);
                }
            }
        } else {
            const float *w = (const float *)p.lhs;
            const float *xf = (const float *)x;
            for (int k = lane * 4; k < p.K; k += 128) {
                float4 wv[GEMV_ROWS];
#pragma unroll
                for (int r = 0; r < GEMV_ROWS; r++) wv[r] = __ldg(reinterpret_cast<const float4 *>(w + abase[r] + k));
                const float4 xv = __ldg(reinterpret_cast<const float4 *>(xf + k));
#pragma unroll
                for (int r = 0; r < GEMV_ROWS; r++) {
                    acc[r] = fmaf(wv[r].x, xv.x, acc[r]);
                    acc[r] = fmaf(wv[r].y, xv.y, acc[r]);
                    acc[r] = fmaf(wv[r].z, xv.z, acc[r]);
                    acc[r] = fmaf(wv[r].w, xv.w, acc[r]);
                }
            }
        }
    } else if ((KIND == LK_Q8H || KIND == LK_Q8F) && p.K % 32 == 0 && lbase % 16 == 0 &&
               (reinterpret_cast<uintptr_t>(p.lhs) | reinterpret_cast<uintptr_t>(x)) % 16 == 0) {
        // Q8_0 against activations this file's tensor-core kernels do not take (f32, the reference's
        // (Q8_0F, F32) pair; bf16): a lane takes 16 codes of a row per step (one 16-byte load, half a block),
        // the 16 activations are loaded once for all the warp's rows, and every element is dequantised with
        // the rounding of lhs_element before it meets its activation.
        const int8_t *codes = (const int8_t *)p.lhs;
        for (int k = lane * 16; k < p.K; k += 512) {
            uint4 qv[GEMV_ROWS];
            float d[GEMV_ROWS];
#pragma unroll
            for (int r = 0; r < GEMV_ROWS; r++) {
                qv[r] = __ldg(reinterpret_cast<const uint4 *>(codes + abase[r] + k));
                const long long blk = (abase[r] + k) >> 5;
                d[r] = KIND == LK_Q8F ? __ldg((const float *)p.lhs_scales + blk) : __half2float(__ldg((const __half *)p.lhs_scales + blk));
            }
            ActT xv[16];
#pragma unroll
            for (int j = 0; j < (int)(16 * sizeof(ActT) / 16); j++)
                reinterpret_cast<uint4 *>(xv)[j] = __ldg(reinterpret_cast<const uint4 *>(x + k) + j);
#pragma unroll
            for (int r = 0; r < GEMV_ROWS; r++) {
                const int8_t *q = reinterpret_cast<const int8_t *>(&qv[r]);
#pragma unroll
                for (int i = 0; i < 16; i++) {
                    const float qd = __fmul_rn((float)q[i], d[r]);
                    const float v = KIND == LK_Q8F ? qd : __half2float(__float2half_rn(qd));
                    acc[r] = fmaf(v, to_f32(xv[i]), acc[r]);
                }
            }
        }
    } else {
        for (int k = lane; k < p.K; k += 32) {
            const float xk = to_f32(x[k]);
#pragma unroll
            for (int r = 0; r < GEMV_ROWS; r++) acc[r] = fmaf(lhs_element<KIND>(p.lhs, p.lhs_scales, abase[r] + k), xk, acc[r]);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
#pragma unroll
        for (int r = 0; r < GEMV_ROWS; r++) acc[r] += __shfl_xor_sync(0xffffffffu, acc[r], o);
    if (lane < GEMV_ROWS && row0 + lane < p.M) {
        const int row = row0 + lane;
        float sum = acc[0];
#pragma unroll
        for (int r = 1; r < GEMV_ROWS; r++) sum = lane == r ? acc[r] : sum;
        const bool has_bias = p.bias_mode != BIAS_NONE;
        float bias = 0.f;
        if (has_bias) bias = load_bias(p.bias, p.bias_dt, p.bias_mode == BIAS_PER_M ? row : 0);
        ((ActT *)p.out)[(long long)batch * p.M + row] = epilogue_value<ActT>(sum, has_bias, bias, p.epilogue);
    }
}

// y[n] = sum_k x[k] * B[k][n] per stack: one row of op(lhs) against a dense rhs stored [K][N] (the decode step's
// attention products: q.kT with one query row, softmax.v with one row of weights).  A CTA takes ROWVEC_COLS
// columns; its eight warps take the k rows 8 apart, every lane four adjacent columns of a row (one 8- or
// 16-byte load, a warp reads a contiguous run of B), and the warps' sums meet in shared memory in warp order.
// With few columns and many k rows (softmax.v of a decode step: 80 columns, K = the cache length) the k rows
// are also split over gridDim.z CTAs, which leave f32 partial sums in `partial` [stack][chunk][N] for
// rowvec_reduce_kernel to add in chunk order (deterministic) and finish.
constexpr int ROWVEC_COLS = 128;
template <typename T, bool PARTIAL>
__global__ void __launch_bounds__(256) rowvec_mat_kernel(MatmulParams p, float *partial, int k_chunk) {
    __shared__ float part[8][ROWVEC_COLS];
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int batch = blockIdx.y;
    const int k_begin = PARTIAL ? (int)blockIdx.z * k_chunk : 0;
    const int k_end = PARTIAL ? min(p.K, k_begin + k_chunk) : p.K;
    const int n0 = blockIdx.x * ROWVEC_COLS + lane * 4;
    const T *x = (const T *)p.lhs + (long long)(batch % p.lhs_stack) * p.K;
    const T *B = (const T *)p.rhs + (long long)(batch % p.rhs_stack) * p.K * p.N;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    const bool vec = (p.N % 4 == 0) && (reinterpret_cast<uintptr_t>(p.rhs) % 16 == 0) && n0 + 3 < p.N;
    if (vec) {
#pragma unroll 4
        for (int k = k_begin + warp; k < k_end; k += 8) {
            const float xk = to_f32(x[k]);
            T v[4];
            if (sizeof(T) == 2) *reinterpret_cast<uint2 *>(v) = __ldg(reinterpret_cast<const uint2 *>(B + (long long)k * p.N + n0));
            else *reinterpret_cast<uint4 *>(v) = __ldg(reinterpret_cast<const uint4 *>(B + (long long)k * p.N + n0));
#pragma unroll
            for (int j = 0; j < 4; j++) acc[j] = fmaf(xk, to_f32(v[j]), acc[j]);
        }
    } else {
        for (int k = k_begin + warp; k < k_end; k += 8) {
            const float xk = to_f32(x[k]);
#pragma unroll
            for (int j = 0; j < 4; j++)
                if (n0 + j < p.N) acc[j] = fmaf(xk, to_f32(B[(long long)k * p.N + n0 + j]), acc[j]);
        }
    }
#pragma unroll
    for (int j = 0; j < 4; j++) part[warp][lane * 4 + j] = acc[j];
    __syncthreads();
    if (threadIdx.x < ROWVEC_COLS) {
        const int n = blockIdx.x * ROWVEC_COLS + threadIdx.x;
        if (n < p.N) {
            float sum = 0.f;
#pragma unroll
            for (int w = 0; w < 8; w++) sum += part[w][threadIdx.x];
            if (PARTIAL) {
                partial[((long long)batch * gridDim.z + blockIdx.z) * p.N + n] = sum;
            } else {
                const bool has_bias = p.bias_mode != BIAS_NONE;
                float bias = 0.f;
                if (has_bias) bias = load_bias(p.bias, p.bias_dt, p.bias_mode == BIAS_PER_N ? n : 0);
                ((T *)p.out)[(long long)batch * p.N + n] = epilogue_value<T>(sum, has_bias, bias, p.epilogue);
            }
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(256) rowvec_reduce_kernel(MatmulParams p, const float *partial, int chunks) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)p.stacks * p.N) return;
    const int batch = (int)(i / p.N), n = (int)(i - (long long)batch * p.N);
    float sum = 0.f;
    for (int c = 0; c < chunks; c++) sum += partial[((long long)batch * chunks + c) * p.N + n];
    const bool has_bias = p.bias_mode != BIAS_NONE;
    float bias = 0.f;
    if (has_bias) bias = load_bias(p.bias, p.bias_dt, p.bias_mode == BIAS_PER_N ? n : 0);
    ((T *)p.out)[i] = epilogue_value<T>(sum, has_bias, bias, p.epilogue);
}

template <int KIND, typename ActT>
cudaError_t launch_kind_act(const MatmulParams &p, bool gemv, cudaStream_t stream) {
    if (gemv) {
        int sms = 148;
        int dev = 0;
        if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if ((long long)((p.M + 63) / 64) * p.stacks >= 2LL * sms) {
            dim3 grid((p.M + 63) / 64, 1, p.stacks);
            gemv_simt_kernel<KIND, ActT, 8><<<grid, 256, 0, stream>>>(p);
        } else {
            dim3 grid((p.M + 15) / 16, 1, p.stacks);
            gemv_simt_kernel<KIND, ActT, 2><<<grid, 256, 0, stream>>>(p);
        }
    } else {
        dim3 grid((p.N + BN - 1) / BN, (p.M + BM - 1) / BM, p.stacks);
        gemm_simt_kernel<KIND, ActT><<<grid, 256, 0, stream>>>(p);
    }
    return cudaGetLastError();
}

template <int KIND>
cudaError_t launch_kind(const MatmulParams &p, rt_dtype act, bool gemv, cudaStream_t stream) {
    switch (act) {
    case RT_F32: return launch_kind_act<KIND, float>(p, gemv, stream);
    case RT_F16: return launch_kind_act<KIND, __half>(p, gemv, stream);
    case RT_BF16: return launch_kind_act<KIND, __nv_bfloat16>(p, gemv, stream);
    default: return cudaErrorInvalidValue;
    }
}

template <typename T>
cudaError_t launch_rowvec_t(const MatmulParams &p, int chunks, float *partial, cudaStream_t stream) {
    const int col_blocks = (p.N + ROWVEC_COLS - 1) / ROWVEC_COLS;
    if (chunks <= 1)
        return launch_pdl(rowvec_mat_kernel<T, false>, dim3(col_blocks, p.stacks, 1), dim3(256), 0, stream, p, (float *)nullptr, p.K);
    const int k_chunk = ((p.K + chunks - 1) / chunks + 7) & ~7;
    cudaError_t e = launch_pdl(rowvec_mat_kernel<T, true>, dim3(col_blocks, p.stacks, chunks), dim3(256), 0, stream, p, partial, k_chunk);
    if (e != cudaSuccess) return e;
    const long long total = (long long)p.stacks * p.N;
    return launch_pdl(rowvec_reduce_kernel<T>, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, p, (const float *)partial, chunks);
}

} // namespace

// How many CTAs share the k rows of one column block: enough to put about two CTAs on every SM, at least 64 rows each.
int rowvec_mat_chunks(int N, int K, int stacks, int sm_count) {
    const long long col_ctas = (long long)((N + ROWVEC_COLS - 1) / ROWVEC_COLS) * stacks;
    const long long want = (2LL * sm_count + col_ctas - 1) / col_ctas;
    return (int)std::max<long long>(1, std::min<long long>(want, K / 64));
}

// One row of a dense lhs against a dense rhs [K][N] of the same dtype (M == 1, no transposes; with M == 1 the
// output is the same memory with or without trans_out).  chunks > 1: `partial` holds stacks * chunks * N floats.
cudaError_t launch_rowvec_mat(const MatmulParams &p, rt_dtype dt, int chunks, float *partial, cudaStream_t stream) {
    if (p.M != 1 || p.stacks > 65535 || chunks > 65535 || (chunks > 1 && !partial)) return cudaErrorInvalidValue;
    switch (dt) {
    case RT_F32: return launch_rowvec_t<float>(p, chunks, partial, stream);
    case RT_F16: return launch_rowvec_t<__half>(p, chunks, partial, stream);
    case RT_BF16: return launch_rowvec_t<__nv_bfloat16>(p, chunks, partial, stream);
    default: return cudaErrorInvalidValue;
    }
}

cudaError_t launch_matmul_simt(const MatmulParams &p, rt_dtype lhs_dt, rt_dtype act_dt, bool gemv, cudaStream_t stream) {
    switch (lhs_dt) {
    case RT_F32: return launch_kind<LK_F32>(p, act_dt, gemv, stream);
    case RT_F16: return launch_kind<LK_F16>(p, act_dt, gemv, stream);
    case RT_BF16: return launch_kind<LK_BF16>(p, act_dt, gemv, stream);
    case RT_Q8_0H: return launch_kind<LK_Q8H>(p, act_dt, gemv, stream);
    case RT_Q8_0F: return launch_kind<LK_Q8F>(p, act_dt, gemv, stream);
    case RT_Q4_K: return launch_kind<LK_Q4K>(p, act_dt, gemv, stream);
    default: return cudaErrorInvalidValue;
    }
}

} // namespace rt
