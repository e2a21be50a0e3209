// Q8_0 GEMV / skinny GEMM for f16 activations: y[v][r] = sum_k W[r][k] * x[v][k], 1..8 vectors.
//
// Takes the role of the reference's subgroup GEMV (crates/ratchet-core/src/ops/gemv.rs:333-558)
// for the (Q8_0H, F16) pair, and of its GEMM (ops/gemm.rs:342-492) when op(rhs) has at most 8
// columns, where the problem is bound by streaming the weight bytes once.
//
// Design (HBM-bound: 1 byte per weight, ~1.06 with scales):
//  * a CTA owns 16 consecutive rows of W and a slice of K; its 8 warps interleave over the
//    32-wide Q8_0 blocks of that slice, so one warp instruction streams 16 rows x 32 codes;
//  * each lane issues 8-byte loads (4 lanes cover one block of one row = one 32-B sector) and
//    keeps UNROLL blocks in flight;
//  * codes become exact f16 values with two byte-permutes and one packed subtract per four codes;
//    the 16x32 code tile times the 32xNV activation tile goes through two m16n8k16 tensor-core
//    MMAs with f32 accumulation (products and sums are exact up to f32 rounding);
//  * the per-block scale d multiplies the block's partial sum: sum_k (q*d)*x = d * sum_k q*x;
//  * warps are reduced through shared memory in a fixed order; when K is split over a thread-block
//    cluster, rank 0 gathers the other CTAs' partials through distributed shared memory, also in
//    a fixed order, so results are deterministic;
//  * epilogue = the reference's: f16(acc) + bias in f16, optional fused GELU.
#include <cooperative_groups.h>

#include "common.cuh"
#include "kernels.hpp"

namespace cg = cooperative_groups;

namespace rt {

namespace {

constexpr int WARPS = 8;
constexpr int ROWS = 16;
constexpr int UNROLL = 4;

__device__ __forceinline__ void mma_m16n8k16_f16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint2 ldg_stream_u2(const void *p) {
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];\n" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}

__device__ __forceinline__ float scale_to_f32(__half s) { return __half2float(s); }
__device__ __forceinline__ float scale_to_f32(float s) { return s; }

// ScaleT: __half (Q8_0H) or float (Q8_0F).  NV: number of activation vectors (1..8).
// SPLIT: K is split over a cluster of gridDim.y CTAs.
template <typename ScaleT, int NV, bool SPLIT>
__global__ void __launch_bounds__(WARPS * 32) q8_gemv_mma_kernel(MatmulParams p, int blocks_per_cta) {
    __shared__ float red[WARPS][ROWS][8];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, c = lane & 3;
    const int batch = blockIdx.z;
    const int nblk = p.K >> 5;
    const int split = SPLIT ? (int)blockIdx.y : 0;
    const int blk_begin = split * blocks_per_cta;
    const int blk_end = min(nblk, blk_begin + blocks_per_cta);

    const int row0 = blockIdx.x * ROWS + g;
    // rows past the end re-read the last row; their results are never stored
    const int ra = min(row0, p.M - 1), rb = min(row0 + 8, p.M - 1);
    const long long lb = batch % p.lhs_stack;
    const uint8_t *codes = (const uint8_t *)p.lhs + lb * p.lhs_batch_elems;
    const ScaleT *scales = (const ScaleT *)((const uint8_t *)p.lhs_scales + lb * p.lhs_batch_scale_bytes);
    const uint8_t *qa = codes + (long long)ra * p.K + c * 8;
    const uint8_t *qb = codes + (long long)rb * p.K + c * 8;
    const ScaleT *sa = scales + (long long)ra * nblk;
    const ScaleT *sb = scales + (long long)rb * nblk;
    // activation vectors: op(rhs) is [K][NV]; both storage orders of a vector batch are handled
    // by the element strides below (NV == 1: contiguous K)
    const int vec = NV == 1 ? 0 : min(g, NV - 1);
    const long long rbatch = batch % p.rhs_stack;
    const __half *x = (const __half *)p.rhs + rbatch * (long long)p.K * NV + (long long)vec * p.K + c * 8;

    float acc[4] = {0.f, 0.f, 0.f, 0.f};

    for (int blk0 = blk_begin + warp; blk0 < blk_end; blk0 += WARPS * UNROLL) {
        uint2 wa[UNROLL], wb[UNROLL];
        uint4 xv[UNROLL];
        float da[UNROLL], db[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; u++) {
            const int blk = blk0 + u * WARPS;
            if (blk < blk_end) {
                wa[u] = ldg_stream_u2(qa + blk * 32);
                wb[u] = ldg_stream_u2(qb + blk * 32);
                da[u] = scale_to_f32(__ldg(sa + blk));
                db[u] = scale_to_f32(__ldg(sb + blk));
                xv[u] = __ldg(reinterpret_cast<const uint4 *>(x + blk * 32));
            } else {
                wa[u] = make_uint2(0x0u, 0x0u);
                wb[u] = make_uint2(0x0u, 0x0u);
                da[u] = db[u] = 0.f;
                xv[u] = make_uint4(0u, 0u, 0u, 0u);
            }
        }
#pragma unroll
        for (int u = 0; u < UNROLL; u++) {
            __half2 a01, a23, a45, a67, b01, b23, b45, b67;
            codes4_to_half2(wa[u].x, a01, a23);
            codes4_to_half2(wa[u].y, a45, a67);
            codes4_to_half2(wb[u].x, b01, b23);
            codes4_to_half2(wb[u].y, b45, b67);
            float t[4] = {0.f, 0.f, 0.f, 0.f};
            // The k index inside a block is permuted identically for W and x: lane c owns
            // elements c*8..c*8+7; the first MMA consumes 0..3 of them, the second 4..7.
            uint32_t fa[4] = {h2_as_u32(a01), h2_as_u32(b01), h2_as_u32(a23), h2_as_u32(b23)};
            mma_m16n8k16_f16(t, fa, xv[u].x, xv[u].y);
            uint32_t fb[4] = {h2_as_u32(a45), h2_as_u32(b45), h2_as_u32(a67), h2_as_u32(b67)};
            mma_m16n8k16_f16(t, fb, xv[u].z, xv[u].w);
            acc[0] = fmaf(da[u], t[0], acc[0]);
            acc[1] = fmaf(da[u], t[1], acc[1]);
            acc[2] = fmaf(db[u], t[2], acc[2]);
            acc[3] = fmaf(db[u], t[3], acc[3]);
        }
    }

    // C fragment: acc[0],acc[1] -> (row g, cols 2c,2c+1); acc[2],acc[3] -> (row g+8, same cols)
    red[warp][g][2 * c] = acc[0];
    red[warp][g][2 * c + 1] = acc[1];
    red[warp][g + 8][2 * c] = acc[2];
    red[warp][g + 8][2 * c + 1] = acc[3];
    __syncthreads();

    const int r = threadIdx.x >> 3, v = threadIdx.x & 7; // first 128 threads: one (row, vector) each
    float sum = 0.f;
    if (threadIdx.x < ROWS * 8) {
#pragma unroll
        for (int w = 0; w < WARPS; w++) sum += red[w][r][v];
    }
    if (SPLIT) {
        cg::cluster_group cluster = cg::this_cluster();
        __syncthreads();
        if (threadIdx.x < ROWS * 8) red[0][r][v] = sum;
        cluster.sync();
        if (cluster.block_rank() == 0 && threadIdx.x < ROWS * 8) {
            const unsigned n = cluster.num_blocks();
            for (unsigned k = 1; k < n; k++) {
                const float *remote = cluster.map_shared_rank(&red[0][0][0], k);
                sum += remote[r * 8 + v];
            }
        }
        cluster.sync(); // keep every CTA's shared memory alive until rank 0 has read it
        if (cluster.block_rank() != 0) return;
    }
    if (threadIdx.x < ROWS * 8 && v < NV) {
        const int row = blockIdx.x * ROWS + r;
        if (row < p.M) {
            const bool has_bias = p.bias_mode != BIAS_NONE;
            float bias = 0.f;
            if (has_bias) bias = load_bias(p.bias, p.bias_dt, p.bias_mode == BIAS_PER_M ? row : v);
            __half o = epilogue_value<__half>(sum, has_bias, bias, p.epilogue);
            // out is [stacks][M][NV] or, transposed, [stacks][NV][M]
            const long long ob = (long long)batch * p.M * NV;
            const long long idx = p.trans_out ? ob + (long long)v * p.M + row : ob + (long long)row * NV + v;
            ((__half *)p.out)[idx] = o;
        }
    }
}

template <typename ScaleT, int NV>
cudaError_t launch_nv(const MatmulParams &p, int split, cudaStream_t stream) {
    const int nblk = p.K / 32;
    const int bpc = (nblk + split - 1) / split;
    dim3 grid((p.M + ROWS - 1) / ROWS, split, p.stacks), block(WARPS * 32);
    if (split == 1) {
        q8_gemv_mma_kernel<ScaleT, NV, false><<<grid, block, 0, stream>>>(p, bpc);
        return cudaGetLastError();
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = split;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, q8_gemv_mma_kernel<ScaleT, NV, true>, p, bpc);
}

template <typename ScaleT>
cudaError_t launch_scale(const MatmulParams &p, int nv, int split, cudaStream_t stream) {
    switch (nv) {
    case 1: return launch_nv<ScaleT, 1>(p, split, stream);
    case 2: return launch_nv<ScaleT, 2>(p, split, stream);
    case 3: return launch_nv<ScaleT, 3>(p, split, stream);
    case 4: return launch_nv<ScaleT, 4>(p, split, stream);
    case 5: return launch_nv<ScaleT, 5>(p, split, stream);
    case 6: return launch_nv<ScaleT, 6>(p, split, stream);
    case 7: return launch_nv<ScaleT, 7>(p, split, stream);
    case 8: return launch_nv<ScaleT, 8>(p, split, stream);
    }
    return cudaErrorInvalidValue;
}

} // namespace

int q8_gemv_mma_pick_split(int M, int K, int sm_count) {
    const int nblk = K / 32;
    const int groups = (M + ROWS - 1) / ROWS;
    const int want = 4 * sm_count; // CTAs needed to keep every SM's load queue full
    int split = 1;
    // split K while the grid is short and every warp still gets at least two blocks
    while (split < 8 && groups * split < want && nblk / (split * 2) >= 2 * WARPS) split *= 2;
    return split;
}

cudaError_t launch_q8_gemv_mma(const MatmulParams &p, bool f32_scales, int nv, int split, cudaStream_t stream) {
    return f32_scales ? launch_scale<float>(p, nv, split, stream) : launch_scale<__half>(p, nv, split, stream);
}

} // namespace rt
