// Q8_0 GEMV / skinny GEMM for f16 activations: y[v][r] = sum_k W[r][k] * x[v][k], 1..16 vectors.
//
// Takes the role of the reference's subgroup GEMV (crates/ratchet-core/src/ops/gemv.rs:333-558)
// for the (Q8_0H, F16) pair, and of its GEMM (ops/gemm.rs:342-492) when op(rhs) has at most 8
// columns, where the problem is bound by streaming the weight bytes once.
//
// Design (HBM-bound: 1 byte per weight, ~1.06 with scales; the whole problem is one wave):
//  * a CTA owns 16 consecutive rows of W and a slice of K.  At kernel entry one thread asks the
//    TMA engine for the CTA's whole share of the codes (one bulk copy per row into padded
//    shared-memory rows, completion counted on an mbarrier) and the other threads fetch the
//    block scales.  Up to five CTAs fit one SM, so every byte of W is in flight within the
//    first microsecond and no register is spent on latency hiding;
//  * the weight requests are issued BEFORE the kernel waits on its stream predecessor
//    (programmatic dependent launch) when the caller states that the weights are constants, so
//    layer i+1 streams its weights while layer i is still finishing; the activations, which the
//    predecessor produces, are only read after that wait;
//  * 8 warps interleave over the 32-wide Q8_0 blocks.  Codes become exact f16 values with two
//    byte-permutes and one packed subtract per four codes; a 16x32 code tile times the 32xNV
//    activation tile goes through two m16n8k16 tensor-core MMAs with f32 accumulation (products
//    and sums exact up to f32 rounding); the block scale multiplies the block's partial sum:
//    sum_k (q*d)*x = d * sum_k q*x;
//  * warps are reduced through shared memory in a fixed order; when K is split over a
//    thread-block cluster, rank 0 gathers the other CTAs' partials through distributed shared
//    memory, also in a fixed order: results are deterministic;
//  * epilogue = the reference's: f16(acc) + bias in f16, optional fused GELU.
#include <cooperative_groups.h>

#include "common.cuh"
#include "kernels.hpp"

namespace cg = cooperative_groups;

namespace rt {

__device__ int g_gemv_error = 0;

namespace {

constexpr int WARPS = 8;
constexpr int THREADS = WARPS * 32;
constexpr int ROWS = 16;
constexpr unsigned long long WAIT_LIMIT_CYCLES = 4000000000ull; // about 2 s at the SM clock

__device__ __forceinline__ void mma_m16n8k16_f16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

// The SM's own cycle counter bounds the waits: it is a register read, where %globaltimer is a
// long-latency access that would sit on the critical path of every stage hand-over.
__device__ __forceinline__ unsigned long long wait_clock() { return (unsigned long long)clock64(); }

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}

__device__ __forceinline__ float scale_to_f32(__half s) { return __half2float(s); }
__device__ __forceinline__ float scale_to_f32(float s) { return s; }

// Row stride of the staged codes: a multiple of 16 (bulk-copy alignment) that is 32 mod 128, so the
// eight rows a half-warp reads start 32 bytes apart in bank space (conflict-free 8-byte reads).
__host__ __device__ inline int code_row_stride(int ks) { return ks + ((32 - ks % 128) + 128) % 128; }
__host__ __device__ inline int scale_row_stride(int nblk_slice) { return nblk_slice | 1; }

// Shared memory: [codes 16 x cstride][scales 16 x sstride][mbarrier]; the first 4 KB double as the
// cross-warp reduction buffer once the codes have been consumed (the mbarrier lies beyond it).
__host__ __device__ inline size_t bar_offset(int blocks_per_cta, int scale_size, int cols) {
    const size_t codes = (size_t)ROWS * code_row_stride(blocks_per_cta * 32);
    const size_t scales = ((size_t)ROWS * scale_row_stride(blocks_per_cta) * scale_size + 15) & ~(size_t)15;
    const size_t red = (size_t)WARPS * ROWS * cols * sizeof(float);
    return codes + scales < red ? red : codes + scales;
}

// ScaleT: __half (Q8_0H) or float (Q8_0F).  NV: number of activation vectors, 1..8, or 16 = two groups of eight
// MMA columns holding nv_rt (9..16) vectors.  SPLIT: K is split over a cluster of gridDim.y CTAs.
template <typename ScaleT, int NV, bool SPLIT>
__global__ void __launch_bounds__(THREADS, 5) q8_gemv_bulk_kernel(MatmulParams p, int blocks_per_cta, int lhs_constant, int nv_rt) {
    constexpr int NVG = NV > 8 ? 2 : 1, COLS = NVG * 8;
    const int nvv = NV > 8 ? nv_rt : NV;
    extern __shared__ __align__(128) uint8_t smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, c = lane & 3;
    const int batch = blockIdx.z;
    const int nblk = p.K >> 5;
    const int split = SPLIT ? (int)blockIdx.y : 0;
    const int blk_begin = split * blocks_per_cta;
    const int blk_cnt = max(0, min(nblk, blk_begin + blocks_per_cta) - blk_begin);
    const int ks = blocks_per_cta * 32;
    const int cstride = code_row_stride(ks);
    const int sstride = scale_row_stride(blocks_per_cta);
    uint8_t *codes_s = smem;
    ScaleT *scales_s = reinterpret_cast<ScaleT *>(smem + ROWS * cstride);
    uint64_t *bar = reinterpret_cast<uint64_t *>(smem + bar_offset(blocks_per_cta, (int)sizeof(ScaleT), COLS));
    const uint32_t bar_addr = smem_u32(bar);

    const int row_base = blockIdx.x * ROWS;
    const int rows_here = min(ROWS, p.M - row_base);
    const long long lb = batch % p.lhs_stack;
    const uint8_t *codes = (const uint8_t *)p.lhs + lb * p.lhs_batch_elems;
    const ScaleT *scales = (const ScaleT *)((const uint8_t *)p.lhs_scales + lb * p.lhs_batch_scale_bytes);

    if (threadIdx.x == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar_addr) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // let the next kernel in the stream start its own prologue and weight requests
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (!lhs_constant) asm volatile("griddepcontrol.wait;" ::: "memory");
    __syncthreads();

    // ---- weight requests: codes through the TMA engine, scales through the load/store unit
    const uint32_t row_bytes = (uint32_t)blk_cnt * 32u;
    if (threadIdx.x == 0 && row_bytes > 0) {
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar_addr), "r"(row_bytes * (uint32_t)rows_here) : "memory");
        for (int r = 0; r < rows_here; r++) {
            const uint8_t *src = codes + (long long)(row_base + r) * p.K + (long long)blk_begin * 32;
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                         ::"r"(smem_u32(codes_s + r * cstride)), "l"(src), "r"(row_bytes), "r"(bar_addr) : "memory");
        }
    }
    {
        // 16 threads per row, no division: thread t stages scales t%16, t%16+16, ... of row t/16
        const int r = threadIdx.x >> 4;
        const int row = min(row_base + r, p.M - 1);
        const ScaleT *src = scales + (long long)row * nblk + blk_begin;
        ScaleT *dst = scales_s + r * sstride;
        for (int j = threadIdx.x & 15; j < blk_cnt; j += 16) dst[j] = __ldg(src + j);
    }
    if (lhs_constant) asm volatile("griddepcontrol.wait;" ::: "memory");

    // ---- activations: written by the stream predecessor, so only touched after the wait
    const long long rbatch = batch % p.rhs_stack;
    const __half *x[NVG]; // MMA column g of group j is vector j*8 + g (clamped: columns past the last vector repeat it)
#pragma unroll
    for (int j = 0; j < NVG; j++) {
        const int vec = NV == 1 ? 0 : min(j * 8 + g, nvv - 1);
        x[j] = (const __half *)p.rhs + rbatch * (long long)p.K * nvv + (long long)vec * p.K + (long long)blk_begin * 32 + c * 8;
    }
    {
        // warm L1 with this CTA's slice of x while the weights are still on their way
        const char *xb = (const char *)((const __half *)p.rhs + rbatch * (long long)p.K * nvv + (long long)blk_begin * 32);
        for (int v = 0; v < nvv; v++)
            for (int off = threadIdx.x * 128; off < blk_cnt * 64; off += THREADS * 128)
                asm volatile("prefetch.global.L1 [%0];" ::"l"(xb + (long long)v * p.K * 2 + off));
    }
    __syncthreads(); // scales staged

    // ---- wait for the codes (bounded)
    bool ok = true;
    if (row_bytes > 0 && !mbar_try_wait(bar_addr, 0)) {
        const unsigned long long t0 = wait_clock();
        while (!mbar_try_wait(bar_addr, 0)) {
            if (wait_clock() - t0 > WAIT_LIMIT_CYCLES) {
                ok = false;
                atomicCAS(&g_gemv_error, 0, 1);
                break;
            }
        }
    }

    float acc[NVG][4];
#pragma unroll
    for (int j = 0; j < NVG; j++)
#pragma unroll
        for (int i = 0; i < 4; i++) acc[j][i] = 0.f;
    if (ok) {
        const uint8_t *qa = codes_s + g * cstride + c * 8;
        const uint8_t *qb = codes_s + (g + 8) * cstride + c * 8;
        const ScaleT *sa = scales_s + g * sstride, *sb = scales_s + (g + 8) * sstride;
#pragma unroll 2
        for (int blk = warp; blk < blk_cnt; blk += WARPS) {
            const uint2 wa = *reinterpret_cast<const uint2 *>(qa + blk * 32);
            const uint2 wb = *reinterpret_cast<const uint2 *>(qb + blk * 32);
            const float da = scale_to_f32(sa[blk]), db = scale_to_f32(sb[blk]);
            __half2 a01, a23, a45, a67, b01, b23, b45, b67;
            codes4_to_half2(wa.x, a01, a23);
            codes4_to_half2(wa.y, a45, a67);
            codes4_to_half2(wb.x, b01, b23);
            codes4_to_half2(wb.y, b45, b67);
            // The k index inside a block is permuted identically for W and x: lane c owns
            // elements c*8..c*8+7; the first MMA consumes 0..3 of them, the second 4..7.
            const uint32_t fa[4] = {h2_as_u32(a01), h2_as_u32(b01), h2_as_u32(a23), h2_as_u32(b23)};
            const uint32_t fb[4] = {h2_as_u32(a45), h2_as_u32(b45), h2_as_u32(a67), h2_as_u32(b67)};
#pragma unroll
            for (int j = 0; j < NVG; j++) {
                const uint4 xv = *reinterpret_cast<const uint4 *>(x[j] + blk * 32);
                float t[4] = {0.f, 0.f, 0.f, 0.f};
                mma_m16n8k16_f16(t, fa, xv.x, xv.y);
                mma_m16n8k16_f16(t, fb, xv.z, xv.w);
                acc[j][0] = fmaf(da, t[0], acc[j][0]);
                acc[j][1] = fmaf(da, t[1], acc[j][1]);
                acc[j][2] = fmaf(db, t[2], acc[j][2]);
                acc[j][3] = fmaf(db, t[3], acc[j][3]);
            }
        }
    }
    __syncthreads(); // every warp is done with the staged codes: the region becomes the reduction buffer

    // C fragment: acc[0],acc[1] -> (row g, cols 2c,2c+1); acc[2],acc[3] -> (row g+8, same cols)
    float *red = reinterpret_cast<float *>(smem); // [WARPS][ROWS][COLS]
#pragma unroll
    for (int j = 0; j < NVG; j++) {
        red[(warp * ROWS + g) * COLS + j * 8 + 2 * c] = acc[j][0];
        red[(warp * ROWS + g) * COLS + j * 8 + 2 * c + 1] = acc[j][1];
        red[(warp * ROWS + g + 8) * COLS + j * 8 + 2 * c] = acc[j][2];
        red[(warp * ROWS + g + 8) * COLS + j * 8 + 2 * c + 1] = acc[j][3];
    }
    __syncthreads();

    const int r = threadIdx.x / COLS, v = threadIdx.x % COLS; // the first ROWS * COLS threads: one (row, vector) each
    float sum = 0.f;
    if (threadIdx.x < ROWS * COLS) {
#pragma unroll
        for (int w = 0; w < WARPS; w++) sum += red[(w * ROWS + r) * COLS + v];
    }
    if (SPLIT) {
        cg::cluster_group cluster = cg::this_cluster();
        __syncthreads();
        if (threadIdx.x < ROWS * COLS) red[r * COLS + v] = sum;
        cluster.sync();
        if (cluster.block_rank() == 0 && threadIdx.x < ROWS * COLS) {
            const unsigned n = cluster.num_blocks();
            for (unsigned k = 1; k < n; k++) {
                const float *remote = cluster.map_shared_rank(red, k);
                sum += remote[r * COLS + v];
            }
        }
        cluster.sync(); // keep every CTA's shared memory alive until rank 0 has read it
        if (cluster.block_rank() != 0) return;
    }
    if (threadIdx.x < ROWS * COLS && v < nvv) {
        const int row = row_base + r;
        if (row < p.M) {
            const bool has_bias = p.bias_mode != BIAS_NONE;
            float bias = 0.f;
            if (has_bias) bias = load_bias(p.bias, p.bias_dt, p.bias_mode == BIAS_PER_M ? row : v);
            __half o = epilogue_value<__half>(sum, has_bias, bias, p.epilogue);
            // out is [stacks][M][NV] or, transposed, [stacks][NV][M]
            const long long ob = (long long)batch * p.M * nvv;
            const long long idx = p.trans_out ? ob + (long long)v * p.M + row : ob + (long long)row * nvv + v;
            ((__half *)p.out)[idx] = o;
        }
    }
}

size_t smem_bytes(int blocks_per_cta, int scale_size, int cols = 8) { return bar_offset(blocks_per_cta, scale_size, cols) + 16; }

template <typename ScaleT, int NV>
cudaError_t launch_nv(const MatmulParams &p, int nv, int split, bool lhs_constant, cudaStream_t stream) {
    const int nblk = p.K / 32;
    const int bpc = (nblk + split - 1) / split;
    const size_t smem = smem_bytes(bpc, (int)sizeof(ScaleT), NV > 8 ? 16 : 8);
    auto kernel = split == 1 ? q8_gemv_bulk_kernel<ScaleT, NV, false> : q8_gemv_bulk_kernel<ScaleT, NV, true>;
    static SmemAttr smem_attr[2];
    if (smem > 48 * 1024) {
        cudaError_t e = smem_attr[split != 1].ensure(kernel, smem);
        if (e != cudaSuccess) return e;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((p.M + ROWS - 1) / ROWS, split, p.stacks);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n = 0;
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    n++;
    if (split > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = 1;
        attr[n].val.clusterDim.y = split;
        attr[n].val.clusterDim.z = 1;
        n++;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    return cudaLaunchKernelEx(&cfg, kernel, p, bpc, lhs_constant ? 1 : 0, nv);
}

template <typename ScaleT>
cudaError_t launch_scale(const MatmulParams &p, int nv, int split, bool lhs_constant, cudaStream_t stream) {
    switch (nv) {
    case 1: return launch_nv<ScaleT, 1>(p, nv, split, lhs_constant, stream);
    case 2: return launch_nv<ScaleT, 2>(p, nv, split, lhs_constant, stream);
    case 3: return launch_nv<ScaleT, 3>(p, nv, split, lhs_constant, stream);
    case 4: return launch_nv<ScaleT, 4>(p, nv, split, lhs_constant, stream);
    case 5: return launch_nv<ScaleT, 5>(p, nv, split, lhs_constant, stream);
    case 6: return launch_nv<ScaleT, 6>(p, nv, split, lhs_constant, stream);
    case 7: return launch_nv<ScaleT, 7>(p, nv, split, lhs_constant, stream);
    case 8: return launch_nv<ScaleT, 8>(p, nv, split, lhs_constant, stream);
    }
    if (nv >= 9 && nv <= 16) return launch_nv<ScaleT, 16>(p, nv, split, lhs_constant, stream);
    return cudaErrorInvalidValue;
}

} // namespace

// K split over a cluster: as few CTAs per row group as keep (a) the CTA's share of W within the
// shared memory of one of five co-resident CTAs and (b) the grid long enough to fill every SM.
// Returns 0 when even an eight-way split does not fit one SM's shared memory.
int q8_gemv_mma_pick_split(int M, int K, int sm_count, int scale_size) {
    const int nblk = K / 32;
    const int groups = (M + ROWS - 1) / ROWS;
    const size_t per_cta_target = 44 * 1024, per_cta_max = 200 * 1024;
    int split = 1;
    while (split < 8 && smem_bytes((nblk + split - 1) / split, scale_size) > per_cta_target) split *= 2;
    // more K slices while the machine is not full, but never past the CTAs that are resident at once (five
    // per SM): a second wave costs more than the finer split gains ([3072,3072]: 768 CTAs on 740 slots)
    while (split < 8 && groups * split < 4 * sm_count && groups * split * 2 <= 5 * sm_count && nblk / (split * 2) >= 2 * WARPS) split *= 2;
    if (smem_bytes((nblk + split - 1) / split, scale_size) > per_cta_max) return 0;
    return split;
}

cudaError_t launch_q8_gemv_mma(const MatmulParams &p, bool f32_scales, int nv, int split, bool lhs_constant, cudaStream_t stream) {
    return f32_scales ? launch_scale<float>(p, nv, split, lhs_constant, stream)
                      : launch_scale<__half>(p, nv, split, lhs_constant, stream);
}

cudaError_t gemv_take_error(int *site, cudaStream_t stream) {
    int zero = 0;
    cudaError_t e = cudaMemcpyFromSymbolAsync(site, g_gemv_error, sizeof(int), 0, cudaMemcpyDeviceToHost, stream);
    if (e != cudaSuccess) return e;
    e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess) return e;
    if (*site != 0) e = cudaMemcpyToSymbolAsync(g_gemv_error, &zero, sizeof(int), 0, cudaMemcpyHostToDevice, stream);
    return e;
}

} // namespace rt
