// Dense f32 GEMM on the 5th-generation tensor cores with f32-class accuracy (three TF32 MMAs per product).
//
// Takes the role of the reference's tiled GEMM shader (crates/ratchet-core/src/ops/gemm.rs, the generic
// f32 path of build_gemm_scalar / vectorized) for nn::Linear-shaped f32 nodes: D[R][S] = P[R][K] . Q[S][K]^T,
// both operands K-major.  The path's bar for f32 is rel-L2 <= 1e-5 against fp64, which one TF32 MMA
// (10 explicit mantissa bits) misses by two orders of magnitude.  Every operand value is therefore
// split in shared memory into hi = the value with its low 13 mantissa bits cleared (exactly a TF32
// number, so the tensor core reads it without rounding) and lo = value - hi (exact in f32; the tensor
// core keeps its leading 11 bits), and the product is accumulated as hi.hi + hi.lo + lo.hi in f32:
// the dropped lo.lo term and the rounding of lo are below 2^-21 of the product.  The tensor core's own
// f32 accumulation is not round-to-nearest, and its error grows with the number of MMAs added into one
// accumulator (measured: 2.9e-5 rel-L2 at K = 4096); so an accumulator only ever takes CHUNK stages
// (K = 128: 48 MMAs), and the chunks are added in registers with ordinary f32 adds.
//
//   warp 0      TMA producer: 128-byte-swizzled boxes of 128 x 32 f32 (P) and BN x 32 f32 (Q) per stage
//   warps 1, 10 MMA issuers: per stage 3 x 4 tcgen05.mma kind::tf32 (128 x BN x 8), six per issuer, each issuer
//               into accumulators of its own (one thread issues an MMA about every 75 cycles, which for twelve
//               is longer than they run); two accumulator pairs alternate by chunk
//   warps 2-9   per stage: split the raw tiles in place into hi and write the lo tiles beside them
//               (element-wise, so the swizzled layout carries over unchanged); per chunk: add the finished
//               accumulator pair into BN / 2 registers per thread (one chunk behind the splitting, so the
//               MMAs never wait for it); per output tile: bias / GELU, store f32 rows
// Two things keep the SMs busy on Linear-shaped problems (few rows of P, many of Q).  The tile width BN
// (128, 96, 80 or 64 rows of Q) is the one whose tiles take the fewest waves x width: 10240 rows are 80
// tiles of 128 on 148 SMs, but 128 tiles of 80.  And when P spans more than one tile column its split is
// done once, by a pass of its own into a scratch pair (hi, lo) that the TMA producer then loads directly,
// instead of by every CTA of the tile row again: the per-stage split then only covers the BN rows of Q.
// Every wait is bounded; on expiry the kernel records the site, frees tensor memory and returns.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <algorithm>
#include <cstdlib>

#include "common.cuh"
#include "kernels.hpp"
#include "umma_gemv.cuh"

namespace rt {

__device__ int g_umma_tf32_error = 0;

namespace {

using namespace umma_gemv; // smem_u32, mbarrier helpers, fences, encode_tiled_fn

constexpr int BM = 128;                // rows of P per tile (the MMA's M)
constexpr int BK = 32;                 // 32 f32 = one 128-byte swizzle row
constexpr int UMMA_K = 8;              // TF32: 8 elements = 32 bytes per instruction
constexpr int P_TILE = BM * BK * 4;    // 16 KB
constexpr int SPLIT_WARPS = 8;
constexpr int ISSUERS = 2;             // MMA-issuing threads (warp 1 and the last warp), each with accumulators of its own
constexpr int NUM_THREADS = 64 + SPLIT_WARPS * 32 + 32;
constexpr int ISSUER_B_WARP = 2 + SPLIT_WARPS;
constexpr int ACC_STRIDE = 128;        // tensor-memory columns between accumulators
constexpr int TMEM_COLS = 2 * ISSUERS * ACC_STRIDE; // per chunk parity one accumulator per issuer: one pair collects a chunk while the other is drained
constexpr int CHUNK = 4;               // stages per accumulator: K = 128

// BN: rows of Q per tile (the MMA's N), a multiple of 16 up to 128.  A stage holds P hi, P lo, Q hi, Q lo.
template <int BN> struct TileCfg {
    static_assert(BN % 16 == 0 && BN >= 32 && BN <= 128, "BN");
    static constexpr int Q_TILE = BN * BK * 4;
    static constexpr int STAGE_BYTES = 2 * P_TILE + 2 * Q_TILE;
    static constexpr int STAGES_FIT = (227 * 1024 - 1024 - 256) / STAGE_BYTES;
    static constexpr int STAGES = STAGES_FIT < 6 ? STAGES_FIT : 6;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
};

struct Tf32Params {
    int R, S, K;
    int stacks, p_stack, q_stack;
    float *out;
    const void *bias;
    int bias_dt, bias_mode;
    int epilogue;
    int tiles_r, tiles_s;
};

// tcgen05.ld of 8 consecutive columns of this warp's 32 lanes, no wait
__device__ __forceinline__ void tmem_ld8_f32(uint32_t taddr, uint32_t (&v)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];\n"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
                 : "r"(taddr)
                 : "memory");
}

__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, int site) {
    return mbar_wait_flag(bar, parity, abort_flag, site, &g_umma_tf32_error);
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *map, int c0, int c1, int c2, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                 ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2), "r"(bar)
                 : "memory");
}

// hi = the value with its 13 low mantissa bits cleared (what a TF32 operand keeps), lo = value - hi.  An infinity goes
// into lo alone (hi = 0): with hi = inf, lo would be inf - inf, and hi would meet the other operand's lo part, whose
// sign is arbitrary.  As lo it meets only the other operand's hi part, so inf * w comes out +-inf by w's sign (NaN
// against w = 0), as in one f32 product.  (Two infinities at the same k on both sides meet a zero hi part each: NaN.)
__device__ __forceinline__ void split_tf32(float v, float &h, float &l) {
    const uint32_t bits = __float_as_uint(v);
    const bool inf = (bits << 1) == 0xFF000000u;
    h = __uint_as_float(inf ? 0u : bits & 0xFFFFE000u);
    l = inf ? v : v - h;
}

__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}\n"
                 ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
                 : "memory");
}

// P_PRE: P arrives already split (map_p = its hi parts, map_plo = its lo parts, written by
// split_tf32_kernel): every CTA of a tile row would otherwise repeat the same split.
template <int BN, bool P_PRE>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_umma_tf32x3_kernel(const __grid_constant__ CUtensorMap map_p, const __grid_constant__ CUtensorMap map_plo,
                        const __grid_constant__ CUtensorMap map_q, const Tf32Params prm) {
    using Cfg = TileCfg<BN>;
    constexpr int STAGES = Cfg::STAGES, STAGE_BYTES = Cfg::STAGE_BYTES, Q_TILE = Cfg::Q_TILE;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *tiles = smem;
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + STAGES * STAGE_BYTES);
    // bars: [0..S) full (TMA landed), [S..2S) split (hi/lo tiles ready), [2S..3S) empty, 2 accumulator complete, 2 accumulator drained
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 3 * STAGES + 4);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t bar_full = smem_u32(bars), bar_split = smem_u32(bars + STAGES), bar_empty = smem_u32(bars + 2 * STAGES);
    const uint32_t bar_tfull = smem_u32(bars + 3 * STAGES), bar_tempty = smem_u32(bars + 3 * STAGES + 2);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_split + 8 * s, SPLIT_WARPS);
            mbar_init(bar_empty + 8 * s, ISSUERS);
        }
        for (int a = 0; a < 2; a++) {
            mbar_init(bar_tfull + 8 * a, ISSUERS);
            mbar_init(bar_tempty + 8 * a, SPLIT_WARPS);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "n"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // programmatic dependent launch: everything above overlapped the stream predecessor (the split pass or the
    // previous node); its results are read, and this kernel's output written, only after this wait
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");

    const int num_k = (prm.K + BK - 1) / BK;
    const int tiles_per_batch = prm.tiles_r * prm.tiles_s;
    const int total_tiles = tiles_per_batch * prm.stacks;

    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                const int b = tile / tiles_per_batch, rem = tile % tiles_per_batch;
                const int r0 = (rem % prm.tiles_r) * BM, s0 = (rem / prm.tiles_r) * BN;
                const int bp = b % prm.p_stack, bq = b % prm.q_stack;
                for (int kb = 0; kb < num_k; kb++) {
                    if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1, abort_flag, 1)) { ok = false; break; }
                    const uint32_t dst = smem_u32(tiles + stage * STAGE_BYTES);
                    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar_full + 8 * stage),
                                 "r"((P_PRE ? 2 : 1) * P_TILE + Q_TILE) : "memory");
                    tma_load_3d(dst, &map_p, kb * BK, r0, bp, bar_full + 8 * stage);
                    if (P_PRE) tma_load_3d(dst + P_TILE, &map_plo, kb * BK, r0, bp, bar_full + 8 * stage);
                    tma_load_3d(dst + 2 * P_TILE, &map_q, kb * BK, s0, bq, bar_full + 8 * stage);
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1 || warp == ISSUER_B_WARP) {
        // ---------------------------------------------------------------- MMA issuers
        // One thread issues a tcgen05.mma about every 75 cycles here (descriptors included), so the twelve
        // MMAs of a stage would take longer to issue than to run.  Two threads issue six each, into
        // accumulators of their own (the first MMA of a chunk overwrites its accumulator, and nothing
        // orders the MMAs of two threads); the drain adds the two.
        if (lane == 0) {
            const int who = warp == 1 ? 0 : 1;
            // instruction descriptor: f32 accumulate, TF32 A and B, K-major, N >> 3 at bit 17, M >> 4 at bit 24
            const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
            int stage = 0, chunk = 0; // chunk counts over all tiles: accumulator pair chunk & 1
            uint32_t phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                for (int kb = 0; kb < num_k; kb++) {
                    const int buf = chunk & 1;
                    if (kb % CHUNK == 0) {
                        // the accumulators' previous chunk has been added into registers
                        if (!mbar_wait(bar_tempty + 8 * buf, ((chunk >> 1) & 1) ^ 1, abort_flag, 5)) { ok = false; break; }
                        tc_fence_after();
                    }
                    if (!mbar_wait(bar_split + 8 * stage, phase, abort_flag, 3)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t d_tmem = tmem_base + (buf * ISSUERS + who) * ACC_STRIDE;
                    const uint32_t p_hi = smem_u32(tiles + stage * STAGE_BYTES), p_lo = p_hi + P_TILE;
                    const uint32_t q_hi = p_hi + 2 * P_TILE, q_lo = q_hi + Q_TILE;
                    // the stage's twelve MMAs in the order lo.hi (k = 0..3), hi.lo (0..3), hi.hi (0..3): small terms
                    // first; issuer 0 takes the first six, issuer 1 the last six
                    // descriptors of the four tiles at k = 0; a step of 8 elements (32 bytes) adds 2 to the address field
                    const uint64_t d_phi = umma_desc_sw128(p_hi, 1024), d_plo = umma_desc_sw128(p_lo, 1024);
                    const uint64_t d_qhi = umma_desc_sw128(q_hi, 1024), d_qlo = umma_desc_sw128(q_lo, 1024);
                    const uint32_t first = (kb % CHUNK) != 0 ? 1u : 0u;
                    if (who == 0) {
                        umma_tf32(d_tmem, d_plo + 0, d_qhi + 0, idesc, first);
                        umma_tf32(d_tmem, d_plo + 2, d_qhi + 2, idesc, 1u);
                        umma_tf32(d_tmem, d_plo + 4, d_qhi + 4, idesc, 1u);
                        umma_tf32(d_tmem, d_plo + 6, d_qhi + 6, idesc, 1u);
                        umma_tf32(d_tmem, d_phi + 0, d_qlo + 0, idesc, 1u);
                        umma_tf32(d_tmem, d_phi + 2, d_qlo + 2, idesc, 1u);
                    } else {
                        umma_tf32(d_tmem, d_phi + 4, d_qlo + 4, idesc, first);
                        umma_tf32(d_tmem, d_phi + 6, d_qlo + 6, idesc, 1u);
                        umma_tf32(d_tmem, d_phi + 0, d_qhi + 0, idesc, 1u);
                        umma_tf32(d_tmem, d_phi + 2, d_qhi + 2, idesc, 1u);
                        umma_tf32(d_tmem, d_phi + 4, d_qhi + 4, idesc, 1u);
                        umma_tf32(d_tmem, d_phi + 6, d_qhi + 6, idesc, 1u);
                    }
                    umma_commit(bar_empty + 8 * stage); // stage reusable once both issuers' MMAs have read it
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                    if (kb % CHUNK == CHUNK - 1 || kb == num_k - 1) {
                        umma_commit(bar_tfull + 8 * buf); // chunk complete (both issuers)
                        chunk++;
                    }
                }
            }
        }
    } else if (warp >= 2 && warp < 2 + SPLIT_WARPS) {
        // ---------------------------------------------------------------- split (per stage), epilogue (per tile)
        const int q = warp & 3;             // the tensor-memory lane quarter this warp may read
        const int half = (warp - 2) >> 2;   // which half of the tile's columns it stores
        const int st_tid = threadIdx.x - 64; // 0..255
        int stage = 0, chunk = 0; // chunk: the next chunk to be drained, counted over all tiles
        uint32_t phase = 0;
        bool ok = true;
        constexpr int HC = BN / 2; // columns of a row that one thread keeps
        // adds accumulator (chunk & 1), columns [half * HC, half * HC + HC) of this thread's row, into racc and
        // hands the accumulator back
        auto drain = [&](float (&racc)[HC]) -> bool {
            const int buf = chunk & 1;
            if (!mbar_wait(bar_tfull + 8 * buf, (chunk >> 1) & 1, abort_flag, 4)) return false;
            tc_fence_after();
#pragma unroll
            for (int who = 0; who < ISSUERS; who++) {
                uint32_t v[HC / 8][8];
#pragma unroll
                for (int j = 0; j < HC / 8; j++)
                    tmem_ld8_f32(tmem_base + (buf * ISSUERS + who) * ACC_STRIDE + half * HC + j * 8 + ((uint32_t)(q * 32) << 16), v[j]);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int j = 0; j < HC / 8; j++)
#pragma unroll
                    for (int i = 0; i < 8; i++) racc[j * 8 + i] += __uint_as_float(v[j][i]);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_tempty + 8 * buf);
            chunk++;
            return true;
        };
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
            const int b = tile / tiles_per_batch, rem = tile % tiles_per_batch;
            const int r0 = (rem % prm.tiles_r) * BM, s0 = (rem / prm.tiles_r) * BN;
            float racc[HC];
#pragma unroll
            for (int i = 0; i < HC; i++) racc[i] = 0.f;
            int pending = 0; // chunks of this tile whose stages are split but which are not drained yet
            for (int kb = 0; kb < num_k; kb++) {
                if (!mbar_wait(bar_full + 8 * stage, phase, abort_flag, 2)) { ok = false; break; }
                // the raw tiles (P unless it came split, and Q): thread t takes float4 number t, t + 256, ... of each
                uint8_t *base = tiles + stage * STAGE_BYTES;
#pragma unroll
                for (int op = P_PRE ? 1 : 0; op < 2; op++) {
                    float4 *raw = reinterpret_cast<float4 *>(base + op * 2 * P_TILE);
                    float4 *lo = reinterpret_cast<float4 *>(base + op * 2 * P_TILE + (op == 0 ? P_TILE : Q_TILE));
                    const int n4 = (op == 0 ? P_TILE : Q_TILE) / 16;
#pragma unroll
                    for (int i = 0; i < (P_TILE / 16 + SPLIT_WARPS * 32 - 1) / (SPLIT_WARPS * 32); i++) {
                        const int idx = st_tid + i * (SPLIT_WARPS * 32);
                        if (idx >= n4) break;
                        const float4 v = raw[idx];
                        float4 h, l;
                        h.x = __uint_as_float(__float_as_uint(v.x) & 0xFFFFE000u); l.x = v.x - h.x;
                        h.y = __uint_as_float(__float_as_uint(v.y) & 0xFFFFE000u); l.y = v.y - h.y;
                        h.z = __uint_as_float(__float_as_uint(v.z) & 0xFFFFE000u); l.z = v.z - h.z;
                        h.w = __uint_as_float(__float_as_uint(v.w) & 0xFFFFE000u); l.w = v.w - h.w;
                        // P (the activations of a Linear) gets the careful split; Q (its weights) is split by
                        // every CTA of a tile column in this loop, which is what bounds the kernel, so an infinite
                        // value of Q comes out as NaN (hi = inf, lo = inf - inf)
                        const float probe = op == 0 ? (l.x + l.y) + (l.z + l.w) : 0.f;
                        if (op == 0 && probe != probe) { // an infinity (lo = inf - inf) or a NaN among the four
                            split_tf32(v.x, h.x, l.x);
                            split_tf32(v.y, h.y, l.y);
                            split_tf32(v.z, h.z, l.z);
                            split_tf32(v.w, h.w, l.w);
                        }
                        raw[idx] = h;
                        lo[idx] = l;
                    }
                }
                // the MMAs read the tiles through the async proxy
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_split + 8 * stage);
                if (++stage == STAGES) { stage = 0; phase ^= 1; }
                if (kb % CHUNK == CHUNK - 1 || kb == num_k - 1) {
                    // this chunk's MMAs are only being issued now: drain the one before it, which is long complete
                    if (pending == 1 && !drain(racc)) { ok = false; break; }
                    pending = 1;
                }
            }
            if (!ok) break;
            if (pending == 1 && !drain(racc)) break;
            const int row = r0 + q * 32 + lane;
            const bool has_bias = prm.bias_mode != BIAS_NONE;
            float row_bias = 0.f;
            if (prm.bias_mode == BIAS_PER_M && row < prm.R) row_bias = load_bias(prm.bias, prm.bias_dt, row);
            float *orow = prm.out + (long long)b * prm.R * prm.S + (long long)row * prm.S;
            const bool vec_ok = (prm.S % 4 == 0) && (reinterpret_cast<uintptr_t>(prm.out) % 16 == 0);
            {
                const int col0 = s0 + half * HC;
                if (row < prm.R && col0 < prm.S) {
                    if (vec_ok && col0 + HC <= prm.S) {
#pragma unroll
                        for (int g = 0; g < HC / 4; g++) {
                            float4 o;
                            float *op = reinterpret_cast<float *>(&o);
#pragma unroll
                            for (int j = 0; j < 4; j++) {
                                const int i = g * 4 + j;
                                const float bv = prm.bias_mode == BIAS_PER_N ? load_bias(prm.bias, prm.bias_dt, col0 + i) : row_bias;
                                op[j] = epilogue_value<float>(racc[i], has_bias, bv, prm.epilogue);
                            }
                            *reinterpret_cast<float4 *>(orow + col0 + g * 4) = o;
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < HC; i++) {
                            if (col0 + i < prm.S) {
                                const float bv = prm.bias_mode == BIAS_PER_N ? load_bias(prm.bias, prm.bias_dt, col0 + i) : row_bias;
                                orow[col0 + i] = epilogue_value<float>(racc[i], has_bias, bv, prm.epilogue);
                            }
                        }
                    }
                }
            }
        }
    }

    // ---------------------------------------------------------------- teardown
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        const unsigned long long t0 = wait_clock();
        while (wait_clock() - t0 < 400000ull) __nanosleep(1000);
    }
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "n"(TMEM_COLS) : "memory");
    }
}

// hi = the value with the 13 low mantissa bits cleared (what a TF32 operand keeps), lo = value - hi
__global__ void split_tf32_kernel(const float4 *__restrict__ in, float4 *__restrict__ hi, float4 *__restrict__ lo, long long n4) {
    // programmatic dependent launch: the GEMM behind this pass may set itself up now; this pass reads what its
    // own stream predecessor wrote (and overwrites the scratch that predecessor's GEMM may still read)
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
        const float4 v = in[i];
        float4 h, l;
        split_tf32(v.x, h.x, l.x);
        split_tf32(v.y, h.y, l.y);
        split_tf32(v.z, h.z, l.z);
        split_tf32(v.w, h.w, l.w);
        hi[i] = h;
        lo[i] = l;
    }
}

// [stack][rows][K] f32 row-major -> boxes of box_rows rows x 32 elements, 128-byte swizzle, zero fill
bool make_map_f32(CUtensorMap *map, const void *base, long long K, long long rows, long long stack, int box_rows) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    cuuint64_t dims[3] = {(cuuint64_t)K, (cuuint64_t)rows, (cuuint64_t)stack};
    cuuint64_t strides[2] = {(cuuint64_t)K * 4, (cuuint64_t)K * 4 * (cuuint64_t)rows};
    cuuint32_t box[3] = {(cuuint32_t)BK, (cuuint32_t)box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int BN, bool P_PRE>
cudaError_t launch_t(const CUtensorMap &mp, const CUtensorMap &mplo, const CUtensorMap &mq, Tf32Params prm, int sm_count, cudaStream_t stream) {
    auto kernel = gemm_umma_tf32x3_kernel<BN, P_PRE>;
    static SmemAttr smem_attr;
    {
        cudaError_t e = smem_attr.ensure(kernel, TileCfg<BN>::SMEM_BYTES);
        if (e != cudaSuccess) return e;
    }
    prm.tiles_s = (prm.S + BN - 1) / BN;
    const long long total = (long long)prm.tiles_r * prm.tiles_s * prm.stacks;
    const int grid = (int)(total < sm_count ? total : sm_count);
    return launch_pdl(kernel, dim3(grid), dim3(NUM_THREADS), TileCfg<BN>::SMEM_BYTES, stream, mp, mplo, mq, prm);
}

} // namespace

// K * 4 bytes must be a multiple of 16 (tensor-map strides), and the operands 16-byte aligned.
bool umma_tf32_supported(long long K) { return K >= 4 && K % 4 == 0 && encode_tiled_fn() != nullptr; }

// Rows of Q per tile: the width whose tiles take the fewest waves x width on sm_count SMs (each SM
// holds one CTA); ties go to the wider tile.
int umma_tf32_pick_bn(int R, int S, int stacks, int sm_count) {
    static const int forced = [] { const char *e = std::getenv("RT_TF32_BN"); return e ? std::atoi(e) : 0; }();
    if (forced == 128 || forced == 96 || forced == 80 || forced == 64) return forced;
    static const int widths[] = {128, 96, 80, 64};
    int best = 128;
    long long best_cost = -1;
    for (int bn : widths) {
        const long long tiles = (long long)((R + BM - 1) / BM) * ((S + bn - 1) / bn) * stacks;
        const long long cost = ((tiles + sm_count - 1) / sm_count) * bn;
        if (best_cost < 0 || cost < best_cost) best = bn, best_cost = cost;
    }
    return best;
}

// Whether splitting P ahead of the GEMM pays: every tile column repeats P's split otherwise.
bool umma_tf32_presplit_pays(int S, int bn) {
    static const int allow = [] { const char *e = std::getenv("RT_TF32_PRESPLIT"); return e ? std::atoi(e) : 1; }();
    return allow != 0 && (S + bn - 1) / bn >= 2;
}

// P: [p_stack][R][K] f32, Q: [q_stack][S][K] f32; out [stacks][R][S] f32.  p_split: nullptr, or room for
// 2 * p_stack * R * K floats, in which P is split into its hi and lo parts by a pass of its own.
cudaError_t launch_gemm_umma_tf32x3(const void *P, const void *Q, void *out, int R, int S, int K, int stacks, int p_stack, int q_stack,
                                    const void *bias, int bias_dt, int bias_mode, int epilogue, int bn, void *p_split, int sm_count,
                                    cudaStream_t stream) {
    if ((reinterpret_cast<uintptr_t>(P) | reinterpret_cast<uintptr_t>(Q) | reinterpret_cast<uintptr_t>(p_split)) % 16 != 0)
        return cudaErrorInvalidValue;
    const long long p_elems = (long long)p_stack * R * K;
    const float *p_hi = static_cast<const float *>(P), *p_lo = p_hi;
    if (p_split) {
        float *hi = static_cast<float *>(p_split), *lo = hi + p_elems;
        const long long n4 = p_elems / 4; // K % 4 == 0
        const int blocks = (int)std::min<long long>((n4 + 255) / 256, (long long)sm_count * 8);
        cudaError_t e = launch_pdl(split_tf32_kernel, dim3(blocks), dim3(256), 0, stream, static_cast<const float4 *>(P),
                                   reinterpret_cast<float4 *>(hi), reinterpret_cast<float4 *>(lo), n4);
        if (e != cudaSuccess) return e;
        p_hi = hi, p_lo = lo;
    }
    CUtensorMap mp, mplo, mq;
    if (!make_map_f32(&mp, p_hi, K, R, p_stack, BM) || !make_map_f32(&mplo, p_lo, K, R, p_stack, BM) ||
        !make_map_f32(&mq, Q, K, S, q_stack, bn))
        return cudaErrorInvalidValue;
    Tf32Params prm{};
    prm.R = R; prm.S = S; prm.K = K;
    prm.stacks = stacks; prm.p_stack = p_stack; prm.q_stack = q_stack;
    prm.out = static_cast<float *>(out);
    prm.bias = bias; prm.bias_dt = bias_dt; prm.bias_mode = bias_mode;
    prm.epilogue = epilogue;
    prm.tiles_r = (R + BM - 1) / BM;
    const bool pre = p_split != nullptr;
    switch (bn) {
    case 128: return pre ? launch_t<128, true>(mp, mplo, mq, prm, sm_count, stream) : launch_t<128, false>(mp, mplo, mq, prm, sm_count, stream);
    case 96: return pre ? launch_t<96, true>(mp, mplo, mq, prm, sm_count, stream) : launch_t<96, false>(mp, mplo, mq, prm, sm_count, stream);
    case 80: return pre ? launch_t<80, true>(mp, mplo, mq, prm, sm_count, stream) : launch_t<80, false>(mp, mplo, mq, prm, sm_count, stream);
    case 64: return pre ? launch_t<64, true>(mp, mplo, mq, prm, sm_count, stream) : launch_t<64, false>(mp, mplo, mq, prm, sm_count, stream);
    default: return cudaErrorInvalidValue;
    }
}

cudaError_t umma_tf32_take_error(int *site, cudaStream_t stream) {
    int zero = 0;
    cudaError_t e = cudaMemcpyFromSymbolAsync(site, g_umma_tf32_error, sizeof(int), 0, cudaMemcpyDeviceToHost, stream);
    if (e != cudaSuccess) return e;
    e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess) return e;
    if (*site != 0) e = cudaMemcpyToSymbolAsync(g_umma_tf32_error, &zero, sizeof(int), 0, cudaMemcpyHostToDevice, stream);
    return e;
}

} // namespace rt
