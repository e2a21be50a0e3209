// Q8_0 GEMV (one activation vector) on the 5th-generation tensor cores: y[r] = sum_k W[r][k] * x[k].
//
// Takes the role of the reference's subgroup GEMV (crates/ratchet-core/src/ops/gemv.rs:333-558) for
// the (Q8_0H, F16) pair at decode shapes.  The problem is bound by reading every weight byte once
// (1.06 bytes per weight); what has to be kept off the critical path is the instruction stream.
// Converting int8 codes to f16 in registers costs more than one instruction per code, which at
// 26 M codes per launch is more issue time than the 4.3 us HBM budget.  Here no code ever passes
// through a register:
//
//  * the int8 codes go from HBM to shared memory by TMA (128-byte swizzle) and are consumed there
//    by tcgen05.mma kind::i8 (M = 128 weight rows, N = 16, K = 32 = one Q8_0 block), one
//    instruction per block, issued by four threads (two blocks of every stage each), s32 accumulators in
//    tensor memory;
//  * the activation vector is turned once per CTA into block-floating-point int8 digits: per block
//    of 32 a power-of-two scale xs and a 15-bit integer m = hi*256 + lo per element, stored as
//    two int8 rows (hi, lo) of the MMA's B operand; |x - m*xs| <= 2^-15 of the block's largest
//    element, far inside the path's 1e-3 bar (f16 inputs carry 11 bits);
//  * per block the epilogue warps (lane = weight row) read the two s32 sums from tensor memory and
//    add d[row][block] * xs[block] * (256*hi + lo) to the row's f32 accumulator: the only per-row
//    work, about ten instructions per block per warp of 32 rows;
//  * a CTA owns a contiguous range of at most 128 rows (N / #CTAs, so all SMs get equal bytes) and,
//    for fat weights, a slice of K: the CTAs of a thread-block cluster split K and rank 0 adds the
//    slices' row sums through distributed shared memory in rank order (deterministic);
//  * the producer warp keeps a small ring of stages full, and it starts before the kernel waits for
//    its stream predecessor when the caller states that the weights are constants (programmatic
//    dependent launch).  A CTA needs less than half of an SM's shared memory and half of its tensor
//    memory, so the next layer's CTAs are resident with their first stages loaded while this layer
//    computes.  (Asking for the whole share with cp.async.bulk.prefetch.L2 as well measured 3 %
//    slower: the requests compete with the running layer's refills.)
// Every wait is bounded (about two seconds of SM cycles); on expiry the kernel sets a device flag,
// leaves its loops, frees tensor memory and returns; the next rt_device_sync reports it.
#include <cooperative_groups.h>
#include <cuda.h>

#include "common.cuh"
#include "kernels.hpp"
#include "umma_gemv.cuh"

namespace cg = cooperative_groups;

namespace rt {

__device__ int g_gemv_umma_error = 0;

namespace {

constexpr int THREADS = 288;          // warp 0: TMA producer, warps 1, 6, 7, 8: MMA issuers, warps 2-5: digits + epilogue
constexpr int N_ISSUE = 4;
constexpr int STAGE_K = 256;          // bytes of K per ring stage = 8 Q8_0 blocks = two 128-byte swizzle rows
constexpr int TMEM_COLS = 256;        // half of an SM's tensor memory
constexpr int TG_COLS = 128;          // tensor-memory columns per stage: 32 per issuing thread (see the MMA issuers)
constexpr int TGROUPS = TMEM_COLS / TG_COLS;

struct UmmaGemvParams {
    MatmulParams p;
    int rb;            // weight rows per cluster (<= 128)
    int rb8;           // rb rounded up to 8: rows of a staged sub-tile
    int ks;            // bytes of K per CTA (multiple of 256)
    int nstages_k;     // ks / 256
    int ring;          // ring stages
    int stage_bytes;   // 2 * rb8 * 128
    int b_bytes;       // digit tiles (and read-past guard), multiple of 1024
    int split;         // cluster size along K
    int lhs_constant;
};

using namespace umma_gemv;

__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, int site) {
    return mbar_wait_flag(bar, parity, abort_flag, site, &g_gemv_umma_error);
}

// Shared-memory map (all offsets from a 1024-byte aligned base):
//   [ring: stages of {A0: rb8 x 128, A1: rb8 x 128}][B digits: (ks/128) tiles of 8 rows x 128 B, at least
//   (128 - rb8) x 128 bytes because the MMAs read 128 rows from every sub-tile][scales: ring x rb8 x 16]
//   [xs: ks/32 floats][red: split x 128 floats][barriers]
__global__ void __launch_bounds__(THREADS, 2)
q8_gemv_umma_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_s, const UmmaGemvParams up) {
    extern __shared__ uint8_t smem_raw[];
    const MatmulParams &p = up.p;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rank = up.split > 1 ? (int)(blockIdx.x % up.split) : 0;
    const int cluster_id = (int)(blockIdx.x / up.split);
    const int row_begin = cluster_id * up.rb;
    if (row_begin >= p.M) return; // the whole cluster leaves together: nothing has been set up yet

    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int n_ksteps = up.ks / 128;
    uint8_t *ring = smem;                                            // [ring][2 sub-tiles][rb8 x 128]
    uint8_t *b_tiles = ring + (size_t)up.ring * up.stage_bytes;      // [ks/128][8 rows x 128]; also absorbs MMA reads past a sub-tile's last row
    uint8_t *scales_s = b_tiles + up.b_bytes;                        // [ring][rb8 x 16]
    float *xs = reinterpret_cast<float *>(scales_s + (size_t)up.ring * up.rb8 * 16);
    float *red = xs + up.ks / 32;
    uint64_t *bars = reinterpret_cast<uint64_t *>(red + 128 * up.split);
    // bars: [0..R) full, [R..2R) empty, then TGROUPS tmem_full, TGROUPS tmem_empty, digits ready, K-slice sums arrived
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * up.ring + 2 * TGROUPS + 2);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    unsigned int *badmask = tmem_slot + 2; // [4]: blocks of this CTA's K slice that hold a NaN or an infinity, then [1]: any
    const uint32_t bar_full = smem_u32(bars), bar_empty = smem_u32(bars + up.ring);
    const uint32_t bar_tfull = smem_u32(bars + 2 * up.ring), bar_tempty = smem_u32(bars + 2 * up.ring + TGROUPS);
    const uint32_t bar_x = smem_u32(bars + 2 * up.ring + 2 * TGROUPS), bar_red = smem_u32(bars + 2 * up.ring + 2 * TGROUPS + 1);

    if (threadIdx.x == 0) {
        for (int s = 0; s < up.ring; s++) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, N_ISSUE + 4); // the issuers' commits + the four epilogue warps (they read the stage's scales)
        }
        for (int a = 0; a < TGROUPS; a++) {
            mbar_init(bar_tfull + 8 * a, N_ISSUE);
            mbar_init(bar_tempty + 8 * a, 4);
        }
        mbar_init(bar_x, 4);
        mbar_init(bar_red, (up.split > 1 ? up.split - 1 : 1) * 128); // one arrival per row of every other K slice
        *abort_flag = 0;
        for (int i = 0; i < 5; i++) badmask[i] = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "n"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // the next kernel in the stream may start its prologue and its weight requests
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    // every CTA of the cluster has initialised its barriers before any other may arrive on them
    if (up.split > 1) cg::this_cluster().sync();
    const uint32_t tmem_base = *tmem_slot;
    const int k_begin = rank * up.ks; // first byte of K of this CTA
    const int rows_here = min(up.rb, p.M - row_begin);

    if (warp == 0) {
        // ------------------------------------------------------------------ producer
        if (!up.lhs_constant) asm volatile("griddepcontrol.wait;" ::: "memory");
        if (lane == 0) {
            int slot = 0;
            uint32_t phase = 0;
            const uint32_t tx = (uint32_t)up.rb * (2 * 128 + 16);
            for (int s = 0; s < up.nstages_k; s++) {
                if (!mbar_wait(bar_empty + 8 * slot, phase ^ 1, abort_flag, 1)) break;
                const uint32_t st = smem_u32(ring + (size_t)slot * up.stage_bytes);
                const uint32_t full = bar_full + 8 * slot;
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(full), "r"(tx) : "memory");
                const int kb = k_begin + s * STAGE_K;
                tma_load_2d(st, &map_w, kb, row_begin, full);
                tma_load_2d(st + up.rb8 * 128, &map_w, kb + 128, row_begin, full);
                tma_load_2d(smem_u32(scales_s + (size_t)slot * up.rb8 * 16), &map_s, kb / 32, row_begin, full);
                if (++slot == up.ring) { slot = 0; phase ^= 1; }
            }
        }
    } else if (warp == 1 || warp >= 6) {
        // ------------------------------------------------------------------ MMA issuers: each takes two of a stage's eight
        // blocks.  One thread issues a tcgen05.mma about every 130 cycles beside the other warps of two resident CTAs (70
        // on an idle SM), which for the 80 MMAs of a Phi-2 sized share was most of the launch.
        if (lane == 0) {
            const int issuer = warp == 1 ? 0 : warp - 5; // 0..3
            const int kk = issuer >> 1, j0 = (issuer & 1) * 2; // sub-tile, first block of the sub-tile
            // instruction descriptor: s32 accumulate, signed 8-bit A and B, K-major, N = 16, M = 128
            const uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) | ((16u >> 3) << 17) | ((128u >> 4) << 24);
            const uint64_t a_desc_ring = umma_desc_sw128(smem_u32(ring), 1024), b_desc_base = umma_desc_sw128(smem_u32(b_tiles), 0);
            bool ok = mbar_wait(bar_x, 0, abort_flag, 2);
            int slot = 0, tg = 0;
            uint32_t phase = 0, tphase = 0;
            for (int s = 0; s < up.nstages_k && ok; s++) {
                if (!mbar_wait(bar_tempty + 8 * tg, tphase ^ 1, abort_flag, 3)) break;
                if (!mbar_wait(bar_full + 8 * slot, phase, abort_flag, 4)) break;
                tc_fence_after();
                // descriptors differ only in their 16-byte address field: one add per operand per MMA keeps the
                // issuing thread, which is the pace-maker of this kernel, short
                const uint64_t a_desc = a_desc_ring + (uint64_t)((uint32_t)(slot * up.stage_bytes) >> 4);
                const uint64_t b_desc = b_desc_base + (uint64_t)(s * 2 * (1024 >> 4));
                const uint32_t d0 = tmem_base + tg * TG_COLS;
                {
                    const uint64_t ak = a_desc + (uint64_t)((uint32_t)(kk * up.rb8 * 128) >> 4), bk = b_desc + (uint64_t)(kk * (1024 >> 4));
                    // Each MMA writes 16 columns: a block's two sums (the hi and lo digit rows of B) followed by columns it
                    // does not need.  MMAs of one thread execute in issue order and this thread's second block starts two
                    // columns after its first, so its quarter of the stage's group begins hi, lo, hi, lo.  The other
                    // threads' MMAs are not ordered against these, hence a quarter of 32 columns per thread.
#pragma unroll
                    for (int j = 0; j < 2; j++) umma_i8(d0 + issuer * 32 + j * 2, ak + 2 * (j0 + j), bk + 2 * (j0 + j), idesc);
                }
                umma_commit(bar_empty + 8 * slot);
                umma_commit(bar_tfull + 8 * tg);
                if (++slot == up.ring) { slot = 0; phase ^= 1; }
                if (++tg == TGROUPS) { tg = 0; tphase ^= 1; }
            }
        }
    } else {
        // ------------------------------------------------------------------ digits, then epilogue (warps 2..5)
        const int q = warp & 3;          // tensor-memory lane quarter of this warp
        const int et = threadIdx.x - 64; // 0..127
        // zero the B tiles: rows 2..7 of every tile stay zero, rows 0 and 1 receive the digits
        for (int i = et; i < n_ksteps * 1024 / 16; i += 128) reinterpret_cast<uint4 *>(b_tiles)[i] = make_uint4(0u, 0u, 0u, 0u);
        asm volatile("bar.sync 1, 128;" ::: "memory");
        // the activations are the stream predecessor's output
        asm volatile("griddepcontrol.wait;" ::: "memory");
        {
            const __half *x = (const __half *)p.rhs + k_begin;
            const int sub = et & 3; // 4 threads per block of 32 elements, 8 elements each
            constexpr int MAX_IT = 3072 / 32 / 32; // blocks per thread quad at the largest K slice
            uint4 pre[MAX_IT];
#pragma unroll
            for (int it = 0; it < MAX_IT; it++) { // all loads first: one L2 round trip, not one per iteration
                const int blk = (et >> 2) + it * 32;
                pre[it] = blk < up.ks / 32 ? *reinterpret_cast<const uint4 *>(x + blk * 32 + sub * 8) : make_uint4(0u, 0u, 0u, 0u);
            }
#pragma unroll
            for (int it = 0; it < MAX_IT; it++) {
                const int blk = (et >> 2) + it * 32;
                if (blk >= up.ks / 32) break;
                if (digits_of_quarter_block(pre[it], blk, sub, b_tiles, xs) && sub == 0) {
                    atomicOr(badmask + (blk >> 5), 1u << (blk & 31));
                    badmask[4] = 1u;
                }
            }
        }
        // the MMAs read the tiles through the async proxy
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("bar.sync 1, 128;" ::: "memory"); // xs visible to all epilogue warps
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_x);

        const int row_local = q * 32 + lane;
        float acc = 0.f;
        int slot = 0, tg = 0;
        uint32_t phase = 0, tphase = 0;
        for (int s = 0; s < up.nstages_k; s++) {
            if (!mbar_wait(bar_full + 8 * slot, phase, abort_flag, 5)) break;
            const uint4 sc = *reinterpret_cast<const uint4 *>(scales_s + (size_t)slot * up.rb8 * 16 + min(row_local, up.rb8 - 1) * 16);
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_empty + 8 * slot);
            if (!mbar_wait(bar_tfull + 8 * tg, tphase, abort_flag, 6)) break;
            tc_fence_after();
            int dq[N_ISSUE][8]; // per issuing thread: hi, lo of its two blocks (the upper four values are not loaded)
#pragma unroll
            for (int i = 0; i < N_ISSUE; i++) tmem_ld4_nowait(tmem_base + tg * TG_COLS + 32 * i + ((uint32_t)(q * 32) << 16), dq[i]);
            tmem_ld_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_tempty + 8 * tg);
            const __half2 *d2 = reinterpret_cast<const __half2 *>(&sc);
            const float4 xa = *reinterpret_cast<const float4 *>(xs + s * 8), xb = *reinterpret_cast<const float4 *>(xs + s * 8 + 4);
            const float xsv[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const float d = (j & 1) ? __high2float(d2[j >> 1]) : __low2float(d2[j >> 1]);
                acc = add_block(acc, d, xsv[j], dq[j >> 1][2 * (j & 1)], dq[j >> 1][2 * (j & 1) + 1]); // block j: issuer j / 2
            }
            if (++slot == up.ring) { slot = 0; phase ^= 1; }
            if (++tg == TGROUPS) { tg = 0; tphase ^= 1; }
        }
        // blocks of the activations that hold NaN or infinities were left out above (zero digits): their
        // products, formed as the reference forms them
        if (badmask[4] && row_local < rows_here) {
            const int row = row_begin + row_local;
            for (int w = 0; w < (up.ks / 32 + 31) / 32; w++) {
                unsigned int m = badmask[w];
                while (m) {
                    const int blk = w * 32 + __ffs(m) - 1;
                    m &= m - 1;
                    const __half d = ((const __half *)p.lhs_scales)[(size_t)row * (p.K / 32) + k_begin / 32 + blk];
                    acc += nonfinite_block_products((const int8_t *)p.lhs + (size_t)row * p.K + k_begin + blk * 32, d,
                                                    (const __half *)p.rhs + k_begin + blk * 32, nullptr);
                }
            }
        }
        red[row_local] = acc;
    }

    // ---------------------------------------------------------------------- K slices meet, epilogue, teardown
    tc_fence_before();
    __syncthreads();
    if (up.split > 1) {
        // Ranks 1.. push their row sums into rank 0's shared memory and arrive on its barrier (release);
        // rank 0 waits for them and adds in rank order.  Nobody waits for rank 0, so only it stays behind.
        cg::cluster_group cluster = cg::this_cluster();
        if (rank != 0) {
            if (threadIdx.x < 128) {
                float *dst = cluster.map_shared_rank(red, 0) + rank * 128 + threadIdx.x;
                *dst = red[threadIdx.x];
                uint32_t remote_bar;
                asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote_bar) : "r"(bar_red), "r"(0));
                asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(remote_bar) : "memory");
            }
        } else if (threadIdx.x < 128) {
            uint32_t done = 0;
            const unsigned long long t0 = wait_clock();
            while (!done) {
                asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], 0;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
                             : "=r"(done) : "r"(bar_red) : "memory");
                if (!done && wait_clock() - t0 > WAIT_LIMIT_CYCLES) {
                    *abort_flag = 1;
                    atomicCAS(&g_gemv_umma_error, 0, 7);
                    break;
                }
            }
            float sum = red[threadIdx.x];
            for (int r = 1; r < up.split; r++) sum += red[r * 128 + threadIdx.x];
            red[threadIdx.x] = sum; // only this thread touches its entry from here on
        }
    }
    if (rank == 0 && threadIdx.x < rows_here && !*abort_flag) {
        const int row = row_begin + threadIdx.x;
        const bool has_bias = p.bias_mode != BIAS_NONE;
        float bias = 0.f;
        if (has_bias) bias = load_bias(p.bias, p.bias_dt, p.bias_mode == BIAS_PER_M ? row : 0);
        ((__half *)p.out)[row] = epilogue_value<__half>(red[threadIdx.x], has_bias, bias, p.epilogue);
    }
    if (*abort_flag) {
        const unsigned long long t0 = wait_clock();
        while (wait_clock() - t0 < 400000ull) __nanosleep(1000);
    }
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "n"(TMEM_COLS) : "memory");
    }
}

int b_region_bytes(int ks, int rb8) {
    int b = (ks / 128) * 1024;
    const int guard = (128 - rb8) * 128;
    if (b < guard) b = guard;
    return (b + 1023) & ~1023;
}

size_t smem_for(int ks, int rb8, int ring, int stage_bytes, int split) {
    return 1024 + (size_t)ring * stage_bytes + b_region_bytes(ks, rb8) + (size_t)ring * rb8 * 16 + (size_t)(ks / 32) * 4 +
           (size_t)split * 128 * 4 + (size_t)(2 * ring + 2 * TGROUPS + 2) * 8 + 64;
}

} // namespace

// Work split for a [M][K] Q8_0H weight: K slices per cluster, rows per cluster, ring depth.  False when
// the shape is not one this kernel takes (the plan then uses the warp-MMA GEMV).
bool q8_gemv_umma_config(int M, int K, int sm_count, GemvUmmaConfig *cfg) {
    if (M < 1 || K < 256 || K % 256 != 0 || !encode_tiled_fn()) return false;
    int split = 1;
    while (split < 8 && (K / split > 3072 || (K / split) % 256 != 0)) split *= 2;
    if (K % (split * 256) != 0 || K / split > 3072) return false;
    int clusters = sm_count / split;
    if (clusters < 1) return false;
    int rb = (M + clusters - 1) / clusters;
    if (rb > 128) return false;
    const int rb8 = (rb + 7) & ~7;
    const int ks = K / split;
    const int stage_bytes = 2 * rb8 * 128;
    const size_t budget = 112 * 1024; // two CTAs (this layer's and the next one's) share an SM
    int ring = 8;
    while (ring > 2 && smem_for(ks, rb8, ring, stage_bytes, split) > budget) ring--;
    if (smem_for(ks, rb8, ring, stage_bytes, split) > 200 * 1024) return false;
    if (ring > ks / STAGE_K) ring = ks / STAGE_K < 2 ? 2 : ks / STAGE_K;
    cfg->split = split; cfg->clusters = clusters; cfg->rb = rb; cfg->rb8 = rb8; cfg->ks = ks; cfg->ring = ring;
    cfg->stage_bytes = stage_bytes;
    cfg->b_bytes = b_region_bytes(ks, rb8);
    cfg->smem_bytes = smem_for(ks, rb8, ring, stage_bytes, split);
    return true;
}

cudaError_t launch_q8_gemv_umma(const MatmulParams &p, const GemvUmmaConfig &cfg, bool lhs_constant, cudaStream_t stream) {
    CUtensorMap map_w, map_s;
    {
        cuuint64_t dims[2] = {(cuuint64_t)p.K, (cuuint64_t)p.M};
        cuuint64_t strides[1] = {(cuuint64_t)p.K};
        cuuint32_t box[2] = {128, (cuuint32_t)cfg.rb};
        cuuint32_t estr[2] = {1, 1};
        if (encode_tiled_fn()(&map_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(p.lhs), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return cudaErrorInvalidValue;
    }
    {
        cuuint64_t dims[2] = {(cuuint64_t)(p.K / 32), (cuuint64_t)p.M};
        cuuint64_t strides[1] = {(cuuint64_t)(p.K / 32) * 2};
        cuuint32_t box[2] = {8, (cuuint32_t)cfg.rb};
        cuuint32_t estr[2] = {1, 1};
        if (encode_tiled_fn()(&map_s, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void *>(p.lhs_scales), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return cudaErrorInvalidValue;
    }
    UmmaGemvParams up{};
    up.p = p;
    up.rb = cfg.rb; up.rb8 = cfg.rb8; up.ks = cfg.ks; up.nstages_k = cfg.ks / STAGE_K; up.ring = cfg.ring;
    up.stage_bytes = cfg.stage_bytes; up.b_bytes = cfg.b_bytes; up.split = cfg.split; up.lhs_constant = lhs_constant ? 1 : 0;
    static SmemAttr smem_attr;
    {
        cudaError_t e = smem_attr.ensure(q8_gemv_umma_kernel, cfg.smem_bytes);
        if (e != cudaSuccess) return e;
    }
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3(cfg.clusters * cfg.split);
    lc.blockDim = dim3(THREADS);
    lc.dynamicSmemBytes = cfg.smem_bytes;
    lc.stream = stream;
    cudaLaunchAttribute attr[2];
    int n = 0;
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    n++;
    if (cfg.split > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = cfg.split;
        attr[n].val.clusterDim.y = 1;
        attr[n].val.clusterDim.z = 1;
        n++;
    }
    lc.attrs = attr;
    lc.numAttrs = n;
    return cudaLaunchKernelEx(&lc, q8_gemv_umma_kernel, map_w, map_s, up);
}

cudaError_t gemv_umma_take_error(int *site, cudaStream_t stream) {
    int zero = 0;
    cudaError_t e = cudaMemcpyFromSymbolAsync(site, g_gemv_umma_error, sizeof(int), 0, cudaMemcpyDeviceToHost, stream);
    if (e != cudaSuccess) return e;
    e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess) return e;
    if (*site != 0) e = cudaMemcpyToSymbolAsync(g_gemv_umma_error, &zero, sizeof(int), 0, cudaMemcpyHostToDevice, stream);
    return e;
}

} // namespace rt
