// Q4_K GEMV / skinny GEMM (1..16 activation vectors) on the 5th-generation tensor cores:
// y[v][r] = sum_k W[r][k] * x[v][k], W raw GGUF Q4_K super-blocks, x and y f16.
//
// The reference declares the Q4_K block (crates/ratchet-loader/src/k_quants.rs:95-103) and has no kernel for it;
// this is the route its Q8_0 GEMV (crates/ratchet-core/src/ops/gemv.rs:333-558) takes in this library
// (gemv_q8_umma.cu), given to the 4-bit format.  The problem is bound by reading 0.5625 bytes per weight once;
// what has to stay off the critical path is the instruction stream.  Turning nibbles into f16 values in registers
// and applying the sub-block scales per weight (gemv_q4k_mma.cu) costs 6.7 instructions per weight, more issue
// time than the HBM time.  Here a weight costs under one:
//
//  * a super-block is 144 bytes = {f16 d, f16 dmin, 12 bytes of 6-bit (scale, min) pairs, 128 bytes of nibbles},
//    value = (d * sc_j) * q - dmin * m_j for sub-block j of 32.  With the activations written per block of 32
//    as block-floating int8 digits, x = xs * (256 hi + lo) (umma_gemv.cuh),
//        sum_k W x = sum_j [ (d sc_j) xs_j (256 sum q hi + sum q lo)  -  (dmin m_j) sum_{k in j} x_k ]
//    and the two integer sums are what tcgen05.mma kind::i8 gives for the codes q against the digit rows;
//  * the producer warp brings raw super-blocks (one per row and stage) into a ring with TMA; eight warps turn
//    nibbles into int8 codes, sixteen at a time (one 16-byte load, six logic instructions, two 16-byte stores
//    into the 128-byte-swizzled K-major operand tile) and copy the 16-byte headers aside; one thread issues the
//    MMAs (M = 128 rows, N = 16 or 32 digit rows, K = 32 = one sub-block), s32 sums in tensor memory;
//  * eight epilogue warps (lane = weight row, two warps per tensor-memory lane quarter taking four sub-blocks
//    each) decode a row's header once per super-block and add the sub-block terms to f32 accumulators, one per
//    vector; integer sums become floats by the 1.5 * 2^23 trick (two full-rate instructions) because the
//    conversion instruction runs at a quarter of the rate;
//  * a CTA owns up to 128 consecutive rows (so an MMA is nearly full) and a slice of K; the CTAs of a cluster
//    split K and rank 0 adds the slices' row sums through distributed shared memory in rank order;
//  * weights flagged constant are requested before the kernel waits for its stream predecessor.
// A block of activations that holds a NaN or an infinity has no digits: its products are formed in f32 from
// the decoded weights instead, so that they come out as IEEE arithmetic gives them.
// Every wait is bounded; on expiry the kernel sets a device flag, leaves its loops, frees tensor memory and
// returns; the next rt_device_sync reports it.
#include <cooperative_groups.h>
#include <cuda.h>

#include "common.cuh"
#include "decode.cuh"
#include "kernels.hpp"
#include "umma_gemv.cuh"

namespace cg = cooperative_groups;

namespace rt {

__device__ int g_gemv_q4k_umma_error = 0;

namespace {

using namespace umma_gemv;

constexpr int N_ISSUE = 2;      // MMA-issuing warps: warp 1 takes the first 128 values of every super-block, warp 2 the second
constexpr int UNPACK_WARPS = 8; // warps 4..11
constexpr int FIRST_UNPACK = 4, FIRST_EPI = FIRST_UNPACK + UNPACK_WARPS;
constexpr int SB_BYTES = 144;
constexpr int MAX_KS = 4096; // K elements per CTA at most (128 blocks: four mask words per vector)

// Epilogue warps: four (one per tensor-memory lane quarter, all eight sub-blocks each) up to eight vectors, eight
// (two per quarter, four sub-blocks each) beyond.
template <int NV> struct Roles {
    static constexpr int EPI_WARPS = NV <= 8 ? 4 : 8;
    static constexpr int THREADS = 32 * (FIRST_EPI + EPI_WARPS);
    static constexpr int BLOCKS_PER_WARP = 32 / EPI_WARPS; // sub-blocks of a super-block one epilogue warp takes
    static constexpr int NB = NV <= 8 ? 16 : 32;           // N of the MMA = accumulator columns per sub-block
    // Digit rows stored per 128 bytes of K: up to four vectors fill one 8-row group, which the MMA reads twice (group
    // stride 0: its columns 8..15 repeat 0..7 and are never read).
    static constexpr int B_ROWS = NV <= 4 ? 8 : NB;
    // Up to four vectors a CTA takes half of an SM's tensor memory (two super-blocks in flight) and, up to two, at most
    // half of its shared memory and registers, so that the next launch's CTA is resident beside it with its first
    // weights loaded while this one computes.
    static constexpr int TMEM_COLS = NV <= 4 ? 256 : 512;
    static constexpr int CTAS_PER_SM = NV <= 2 ? 2 : 1;
    static constexpr int LD_COLS = 2 * NV < 16 ? 2 * NV : 16;   // columns per tensor-memory load
    static constexpr int LOADS = 2 * NV / LD_COLS;              // loads per sub-block (two for sixteen vectors)
    // sub-blocks whose sums a warp fetches before it waits once and does their arithmetic: 32 registers' worth
    static constexpr int BATCH = (32 / (2 * NV) < 1 ? 1 : 32 / (2 * NV)) < BLOCKS_PER_WARP ? (32 / (2 * NV) < 1 ? 1 : 32 / (2 * NV)) : BLOCKS_PER_WARP;
};

struct Q4kUmmaParams {
    MatmulParams p;
    int nv;            // activation vectors, 1..16
    int rb, rb8;       // rows per cluster, rounded up to 8
    int ks, nsb;       // K elements per CTA, super-blocks per CTA
    int split;         // cluster size along K
    int raw_ring, a_ring;
    int raw_stage_bytes; // rb8 * 144
    int a_stage_bytes;   // 2 * rb8 * 128
    int b_bytes;         // digit tiles (also the guard behind the code ring), multiple of 1024
    int inv_rb8_q20;     // ceil(2^20 / rb8): idx / rb8 == (idx * this) >> 20 for idx < 9 * rb8 (rb8 <= 128)
    int lhs_constant;
};

__device__ __forceinline__ bool mbar_wait_hot(uint32_t bar, uint32_t parity, volatile int *abort_flag, int site) {
    return mbar_wait_flag(bar, parity, abort_flag, site, &g_gemv_q4k_umma_error);
}

// Bounded wait.  The waiting warp sleeps between tries: a spinning warp's tries go through the same shared-memory
// instruction queue as the loads and stores of the warps that unpack nibbles, and take issue slots from the MMA
// issuers, whose instruction chains are this kernel's pace-makers.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, int site) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = wait_clock();
    while (true) {
#pragma unroll 1
        for (int i = 0; i < 64; i++) {
            __nanosleep(32);
            if (mbar_try_wait(bar, parity)) return true;
        }
        if (*abort_flag) return false;
        if (wait_clock() - t0 > WAIT_LIMIT_CYCLES) {
            *abort_flag = 1;
            atomicCAS(&g_gemv_q4k_umma_error, 0, site);
            return false;
        }
    }
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *map, int c0, int c1, int c2, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                 ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2), "r"(bar) : "memory");
}

// N consecutive accumulator columns of this warp's 32 lanes into v[0..N), no wait (N = 2, 4, 8 or 16).
template <int N> __device__ __forceinline__ void tmem_ld_cols(uint32_t taddr, int *v) {
    if constexpr (N == 2) {
        asm volatile("tcgen05.ld.sync.aligned.32x32b.x2.b32 {%0, %1}, [%2];" : "=r"(v[0]), "=r"(v[1]) : "r"(taddr) : "memory");
    } else if constexpr (N == 4) {
        asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]) : "r"(taddr) : "memory");
    } else if constexpr (N == 8) {
        asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                     : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]) : "r"(taddr) : "memory");
    } else {
        static_assert(N == 16, "column count");
        asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                     : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
                       "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
                     : "r"(taddr) : "memory");
    }
}

// An s32 of magnitude below 2^22 as a float, without the (quarter-rate) conversion instruction: the integer is
// added into the mantissa of 1.5 * 2^23, whose unit in the last place is one.
__device__ __forceinline__ float small_int_to_float(int v) { return __int_as_float(0x4B400000 + v) - 12582912.0f; }

// Shared-memory map (offsets from a 1024-byte aligned base):
//   [code ring: a_ring x {chunk 0: rb8 x 128, chunk 1: rb8 x 128}][digit tiles: (ks/128) x 2 NV rows x 128; at least
//   (128 - rb8) x 128 bytes, because every MMA reads 128 rows][raw ring: raw_ring x rb8 x 144][headers: a_ring x
//   rb8 x 16][xs: NV x 128][sumx: NV x 128][part: 2 x NV x 128][red: split x NV x 128][mask][barriers]
template <int NV>
__global__ void __launch_bounds__(Roles<NV>::THREADS, Roles<NV>::CTAS_PER_SM)
q4k_gemv_umma_kernel(const __grid_constant__ CUtensorMap map_w, const Q4kUmmaParams up) {
    extern __shared__ uint8_t smem_raw[];
    const MatmulParams &p = up.p;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rank = up.split > 1 ? (int)(blockIdx.x % up.split) : 0;
    const int cluster_id = (int)(blockIdx.x / up.split);
    const int row_begin = cluster_id * up.rb;
    if (row_begin >= p.M) return; // the whole cluster leaves together: nothing has been set up yet

    constexpr int EPI_WARPS = Roles<NV>::EPI_WARPS, BPW = Roles<NV>::BLOCKS_PER_WARP;
    constexpr int NB = Roles<NV>::NB, B_ROWS = Roles<NV>::B_ROWS, TMEM_COLS = Roles<NV>::TMEM_COLS;
    constexpr int LD_COLS = Roles<NV>::LD_COLS, LOADS = Roles<NV>::LOADS, BATCH = Roles<NV>::BATCH;
    constexpr int TG_COLS = 8 * NB;         // one super-block's sums
    constexpr int TGROUPS = TMEM_COLS / TG_COLS;
    const int nblk = up.ks / 32, nv = up.nv;

    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *a_ring = smem;
    uint8_t *b_tiles = a_ring + (size_t)up.a_ring * up.a_stage_bytes;
    uint8_t *raw_ring = b_tiles + up.b_bytes;
    uint8_t *hdr = raw_ring + (size_t)up.raw_ring * up.raw_stage_bytes;
    float *xs = reinterpret_cast<float *>(hdr + (size_t)up.a_ring * up.rb8 * 16);
    float *sumx = xs + NV * (MAX_KS / 32);
    float *part = sumx + NV * (MAX_KS / 32);
    float *red = part + 2 * NV * 128;
    unsigned int *badmask = reinterpret_cast<unsigned int *>(red + up.split * NV * 128); // [NV][4], then [1]: any
    uint64_t *bars = reinterpret_cast<uint64_t *>(badmask + NV * 4 + 2);
    // bars: raw_full[R], raw_empty[R], a_full[A], a_empty[A], tmem_full[TGROUPS], tmem_empty[TGROUPS], digits ready, slices arrived
    const int n_bars = 2 * up.raw_ring + 2 * up.a_ring + 2 * TGROUPS + 2;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + n_bars);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    const uint32_t bar_rfull = smem_u32(bars), bar_rempty = bar_rfull + 8 * up.raw_ring;
    const uint32_t bar_afull = bar_rempty + 8 * up.raw_ring, bar_aempty = bar_afull + 8 * up.a_ring;
    const uint32_t bar_tfull = bar_aempty + 8 * up.a_ring, bar_tempty = bar_tfull + 8 * TGROUPS;
    const uint32_t bar_x = bar_tempty + 8 * TGROUPS, bar_red = bar_x + 8;

    if (threadIdx.x == 0) {
        for (int s = 0; s < up.raw_ring; s++) {
            mbar_init(bar_rfull + 8 * s, 1);
            mbar_init(bar_rempty + 8 * s, UNPACK_WARPS);
        }
        for (int s = 0; s < up.a_ring; s++) {
            mbar_init(bar_afull + 8 * s, UNPACK_WARPS);
            mbar_init(bar_aempty + 8 * s, N_ISSUE + EPI_WARPS); // the issuers' commits and the epilogue warps (they read the stage's headers)
        }
        for (int a = 0; a < TGROUPS; a++) {
            mbar_init(bar_tfull + 8 * a, N_ISSUE);
            mbar_init(bar_tempty + 8 * a, EPI_WARPS);
        }
        mbar_init(bar_x, EPI_WARPS);
        mbar_init(bar_red, (up.split > 1 ? up.split - 1 : 1) * 128);
        *abort_flag = 0;
        for (int i = 0; i < NV * 4 + 1; i++) badmask[i] = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "n"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (up.split > 1) cg::this_cluster().sync(); // every CTA's barriers exist before another arrives on them
    const uint32_t tmem_base = *tmem_slot;
    const int k_begin = rank * up.ks;
    const int sb_begin = k_begin >> 8;
    const int rows_here = min(up.rb, p.M - row_begin);

    if (warp == 0) {
        // ------------------------------------------------------------------ producer: one super-block per row and stage
        if (!up.lhs_constant) asm volatile("griddepcontrol.wait;" ::: "memory");
        if (lane == 0) {
            int slot = 0;
            uint32_t phase = 0;
            const uint32_t tx = (uint32_t)up.rb * SB_BYTES;
            for (int s = 0; s < up.nsb; s++) {
                if (!mbar_wait(bar_rempty + 8 * slot, phase ^ 1, abort_flag, 1)) break;
                const uint32_t full = bar_rfull + 8 * slot;
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(full), "r"(tx) : "memory");
                tma_load_3d(smem_u32(raw_ring + (size_t)slot * up.raw_stage_bytes), &map_w, 0, sb_begin + s, row_begin, full);
                if (++slot == up.raw_ring) { slot = 0; phase ^= 1; }
            }
        }
    } else if (warp <= N_ISSUE) {
        // ------------------------------------------------------------------ MMA issuers (warps 1, 2): one 128-value chunk each
        if (lane == 0) {
            const int c = warp - 1;
            // instruction descriptor: s32 accumulate, signed 8-bit A and B, K-major, N = NB, M = 128
            const uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(NB >> 3) << 17) | ((128u >> 4) << 24);
            const uint64_t a_desc_ring = umma_desc_sw128(smem_u32(a_ring) + c * up.rb8 * 128, 1024);
            const uint64_t b_desc_base = umma_desc_sw128(smem_u32(b_tiles) + c * B_ROWS * 128, B_ROWS == 8 ? 0 : 1024);
            bool ok = mbar_wait(bar_x, 0, abort_flag, 2);
            int slot = 0, tg = 0;
            uint32_t phase = 0, tphase = 0;
            for (int s = 0; s < up.nsb && ok; s++) {
                if (!mbar_wait_hot(bar_tempty + 8 * tg, tphase ^ 1, abort_flag, 3)) break;
                if (!mbar_wait_hot(bar_afull + 8 * slot, phase, abort_flag, 4)) break;
                tc_fence_after();
                const uint64_t ak = a_desc_ring + (uint64_t)((uint32_t)(slot * up.a_stage_bytes) >> 4);
                const uint64_t bk = b_desc_base + (uint64_t)((uint32_t)(s * 2 * B_ROWS * 128) >> 4);
                const uint32_t d0 = tmem_base + tg * TG_COLS + c * 4 * NB;
                // sub-block j of the chunk: 32 bytes further along K in both operands; its NB sums get their own columns
#pragma unroll
                for (int j = 0; j < 4; j++) umma_i8(d0 + j * NB, ak + 2 * j, bk + 2 * j, idesc);
                umma_commit(bar_aempty + 8 * slot);
                umma_commit(bar_tfull + 8 * tg);
                if (++slot == up.a_ring) { slot = 0; phase ^= 1; }
                if (++tg == TGROUPS) { tg = 0; tphase ^= 1; }
            }
        }
    } else if (warp < FIRST_UNPACK) {
        // warp 3: no role (keeps the unpacking and epilogue warps spread evenly over the four schedulers)
    } else if (warp < FIRST_EPI) {
        // ------------------------------------------------------------------ nibbles -> int8 codes (warps 4..11)
        // Warp t takes the t-th 16-byte group of nibbles of every row (rows lane, lane + 32, ..): no index arithmetic
        // beyond a row stride, and eight consecutive lanes touch eight consecutive rows, which are 144 bytes apart in
        // the raw stage and 128 bytes apart (16-byte chunks XOR-swizzled by row) in the tile: no bank conflicts on
        // either side.  Warps 0..3 also copy the rows' 16-byte headers.
        const int t = warp - FIRST_UNPACK;
        // group g = t / 2 of 64 values: bytes 16 (t % 2) .. of its 32 hold values 64 g + 16 (t % 2) .. in their low
        // nibbles and the values 32 further on in their high nibbles
        const int g = t >> 1, unit = (g & 1) * 4 + (t & 1);
        const int lo_off = (unit ^ (lane & 7)) << 4, hi_off = ((unit + 2) ^ (lane & 7)) << 4; // row & 7 == lane & 7
        const int chunk_off = (g >> 1) * (up.rb8 * 128);
        int rslot = 0, aslot = 0;
        uint32_t rphase = 0, aphase = 0;
        for (int s = 0; s < up.nsb; s++) {
            if (!mbar_wait_hot(bar_rfull + 8 * rslot, rphase, abort_flag, 5)) break;
            if (!mbar_wait_hot(bar_aempty + 8 * aslot, aphase ^ 1, abort_flag, 6)) break;
            const uint8_t *raw = raw_ring + (size_t)rslot * up.raw_stage_bytes + lane * SB_BYTES;
            uint8_t *a_st = a_ring + (size_t)aslot * up.a_stage_bytes + chunk_off + lane * 128;
            uint8_t *h_st = hdr + (size_t)aslot * up.rb8 * 16 + lane * 16;
            uint4 w[4], hd = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
            for (int i = 0; i < 4; i++) // all loads first: one trip through shared memory, not four
                w[i] = lane + 32 * i < up.rb8 ? *reinterpret_cast<const uint4 *>(raw + i * 32 * SB_BYTES + 16 + t * 16) : make_uint4(0u, 0u, 0u, 0u);
            if (t < 4 && lane + 32 * t < up.rb8) hd = *reinterpret_cast<const uint4 *>(raw + t * 32 * SB_BYTES);
#pragma unroll
            for (int i = 0; i < 4; i++) {
                if (lane + 32 * i < up.rb8) {
                    const uint4 lo = make_uint4(w[i].x & 0x0F0F0F0Fu, w[i].y & 0x0F0F0F0Fu, w[i].z & 0x0F0F0F0Fu, w[i].w & 0x0F0F0F0Fu);
                    const uint4 hi = make_uint4((w[i].x >> 4) & 0x0F0F0F0Fu, (w[i].y >> 4) & 0x0F0F0F0Fu, (w[i].z >> 4) & 0x0F0F0F0Fu,
                                                (w[i].w >> 4) & 0x0F0F0F0Fu);
                    *reinterpret_cast<uint4 *>(a_st + i * 32 * 128 + lo_off) = lo;
                    *reinterpret_cast<uint4 *>(a_st + i * 32 * 128 + hi_off) = hi;
                }
            }
            if (t < 4 && lane + 32 * t < up.rb8) *reinterpret_cast<uint4 *>(h_st + t * 32 * 16) = hd;
            // the MMAs read the tile through the async proxy
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(bar_afull + 8 * aslot);
                mbar_arrive(bar_rempty + 8 * rslot);
            }
            if (++rslot == up.raw_ring) { rslot = 0; rphase ^= 1; }
            if (++aslot == up.a_ring) { aslot = 0; aphase ^= 1; }
        }
    } else {
        // ------------------------------------------------------------------ digits, then epilogue (warps 12..)
        const int et = threadIdx.x - 32 * FIRST_EPI;  // 0 .. 32 EPI_WARPS - 1
        const int q = warp & 3;                        // tensor-memory lane quarter of this warp
        const int half = (warp - FIRST_EPI) >> 2;      // with eight warps: sub-blocks 0..3 or 4..7 of every super-block
        // the activations are the stream predecessor's output
        asm volatile("griddepcontrol.wait;" ::: "memory");
        {
            const int sub = et & 3; // 4 threads per block of 32 elements, 8 elements each
            const int n_items = nv * nblk; // a multiple of 8: a warp's eight quads stay together
#pragma unroll 2
            for (int i = et >> 2; i < n_items; i += 8 * EPI_WARPS) {
                const int v = i / nblk, blk = i - v * nblk;
                const uint4 raw = *reinterpret_cast<const uint4 *>((const __half *)p.rhs + (size_t)v * p.K + k_begin + blk * 32 + sub * 8);
                uint2 hi8, lo8;
                float inv;
                bool nonfinite;
                quantize_quarter_block(raw, hi8, lo8, inv, nonfinite);
                // the block's sum of x, taken from the digits so that it is the sum of exactly what the MMAs see
                int sm = 256 * (__dp4a((int)hi8.x, 0x01010101, 0) + __dp4a((int)hi8.y, 0x01010101, 0)) +
                         __dp4a((int)lo8.x, 0x01010101, 0) + __dp4a((int)lo8.y, 0x01010101, 0);
                sm += __shfl_xor_sync(0xffffffffu, sm, 1);
                sm += __shfl_xor_sync(0xffffffffu, sm, 2);
                uint8_t *tile = b_tiles + (size_t)(blk >> 2) * (B_ROWS * 128) + ((2 * v) >> 3) * 1024;
                const int kpos = (blk & 3) * 32 + sub * 8;
                store_digits8(tile, (2 * v) & 7, kpos, hi8);
                store_digits8(tile, ((2 * v) & 7) + 1, kpos, lo8);
                if (sub == 0) {
                    xs[v * (MAX_KS / 32) + blk] = inv;
                    sumx[v * (MAX_KS / 32) + blk] = inv * (float)sm;
                    if (nonfinite) {
                        atomicOr(badmask + v * 4 + (blk >> 5), 1u << (blk & 31));
                        badmask[NV * 4] = 1u;
                    }
                }
            }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("bar.sync 1, %0;" ::"n"(32 * EPI_WARPS) : "memory"); // xs, sumx visible to all epilogue warps
        if (lane == 0) mbar_arrive(bar_x);

        const int row_local = q * 32 + lane;
        float acc[NV];
#pragma unroll
        for (int v = 0; v < NV; v++) acc[v] = 0.f;
        int slot = 0, tg = 0;
        uint32_t phase = 0, tphase = 0;
        for (int s = 0; s < up.nsb; s++) {
            if (!mbar_wait(bar_afull + 8 * slot, phase, abort_flag, 7)) break;
            const uint4 h = *reinterpret_cast<const uint4 *>(hdr + (size_t)slot * up.rb8 * 16 + min(row_local, up.rb8 - 1) * 16);
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_aempty + 8 * slot);
            const __half2 dd = *reinterpret_cast<const __half2 *>(&h.x);
            const float d = __low2float(dd), dmin = __high2float(dd);
            if (!mbar_wait(bar_tfull + 8 * tg, tphase, abort_flag, 8)) break;
            tc_fence_after();
#pragma unroll
            for (int j0 = 0; j0 < BPW; j0 += BATCH) {
                // the batch's sums first (one wait for all of them), then their arithmetic
                int dv[BATCH][2 * NV];
#pragma unroll
                for (int jj = 0; jj < BATCH; jj++) {
                    const int jb = (BPW == 8 ? 0 : half * 4) + j0 + jj; // sub-block of the super-block
                    const uint32_t taddr = tmem_base + tg * TG_COLS + jb * NB + ((uint32_t)(q * 32) << 16);
#pragma unroll
                    for (int l = 0; l < LOADS; l++) tmem_ld_cols<LD_COLS>(taddr + l * LD_COLS, &dv[jj][l * LD_COLS]);
                }
                tmem_ld_wait();
                if (j0 + BATCH >= BPW) {
                    // this warp has read its part of the stage's sums
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar_tempty + 8 * tg);
                }
#pragma unroll
                for (int jj = 0; jj < BATCH; jj++) {
                    const int jw = j0 + jj, jb = (BPW == 8 ? 0 : half * 4) + jw;
                    float dsc, dmn; // (d * sc, dmin * m), each one f32 rounding as the decoders form them
                    {
                        // get_scale_min_k4 of the format: bytes jb % 4 of the three words of packed scales
                        const int j = jw & 3;
                        const bool upper = BPW == 8 ? jw >= 4 : half != 0;
                        const unsigned int b0 = (h.y >> (8 * j)) & 0xFFu, b1 = (h.z >> (8 * j)) & 0xFFu, b2 = (h.w >> (8 * j)) & 0xFFu;
                        const int sc = !upper ? (int)(b0 & 63u) : (int)((b2 & 0x0Fu) | ((b0 >> 6) << 4));
                        const int m = !upper ? (int)(b1 & 63u) : (int)((b2 >> 4) | ((b1 >> 6) << 4));
                        dsc = __fmul_rn(d, small_int_to_float(sc));
                        dmn = __fmul_rn(dmin, small_int_to_float(m));
                    }
                    const int blk = s * 8 + jb;
#pragma unroll
                    for (int v = 0; v < NV; v++) {
                        if (v < nv) {
                            const float t = fmaf(256.0f, small_int_to_float(dv[jj][2 * v]), small_int_to_float(dv[jj][2 * v + 1]));
                            acc[v] = fmaf(dsc * xs[v * (MAX_KS / 32) + blk], t, acc[v]);
                            acc[v] = fmaf(-dmn, sumx[v * (MAX_KS / 32) + blk], acc[v]);
                        }
                    }
                }
            }
            if (++slot == up.a_ring) { slot = 0; phase ^= 1; }
            if (++tg == TGROUPS) { tg = 0; tphase ^= 1; }
        }
        // blocks of activations that hold NaN or infinities were left out above (zero digits, zero sums): their
        // products from the decoded weights, in f32
        if (badmask[NV * 4] && half == 0 && row_local < rows_here) {
            const long long row = row_begin + row_local;
#pragma unroll
            for (int v = 0; v < NV; v++) { // unrolled: a runtime index would put the accumulators into local memory
                if (v >= nv) continue;
                for (int w = 0; w < (nblk + 31) / 32; w++) {
                    unsigned int m = badmask[v * 4 + w];
                    while (m) {
                        const int blk = w * 32 + __ffs(m) - 1;
                        m &= m - 1;
                        const __half *xv = (const __half *)p.rhs + (size_t)v * p.K + k_begin + blk * 32;
                        float sum = 0.f;
                        for (int i = 0; i < 32; i++)
                            sum += q4k_element((const uint8_t *)p.lhs, row * p.K + k_begin + blk * 32 + i) * __half2float(xv[i]);
                        acc[v] += sum;
                    }
                }
            }
        }
        if (EPI_WARPS == 8) {
#pragma unroll
            for (int v = 0; v < NV; v++) part[(half * NV + v) * 128 + row_local] = acc[v];
            asm volatile("bar.sync 1, %0;" ::"n"(32 * EPI_WARPS) : "memory");
            if (half == 0) {
#pragma unroll
                for (int v = 0; v < NV; v++) red[v * 128 + row_local] = part[v * 128 + row_local] + part[(NV + v) * 128 + row_local];
            }
        } else {
#pragma unroll
            for (int v = 0; v < NV; v++) red[v * 128 + row_local] = acc[v];
        }
    }

    // ---------------------------------------------------------------------- K slices meet, epilogue, teardown
    tc_fence_before();
    __syncthreads();
    if (up.split > 1) {
        // Ranks 1.. push their row sums into rank 0's shared memory and arrive on its barrier (release); rank 0 waits
        // for them and adds in rank order.  Nobody waits for rank 0, so only it stays behind.
        cg::cluster_group cluster = cg::this_cluster();
        if (rank != 0) {
            if (threadIdx.x < 128) {
                float *dst = cluster.map_shared_rank(red, 0) + rank * NV * 128 + threadIdx.x;
                for (int v = 0; v < nv; v++) dst[v * 128] = red[v * 128 + threadIdx.x];
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
                    atomicCAS(&g_gemv_q4k_umma_error, 0, 9);
                    break;
                }
            }
            for (int v = 0; v < nv; v++) {
                float sum = red[v * 128 + threadIdx.x];
                for (int r = 1; r < up.split; r++) sum += red[(r * NV + v) * 128 + threadIdx.x];
                red[v * 128 + threadIdx.x] = sum; // only this thread touches its entries from here on
            }
        }
    }
    if (rank == 0 && threadIdx.x < rows_here && !*abort_flag) {
        const int row = row_begin + threadIdx.x;
        const bool has_bias = p.bias_mode != BIAS_NONE;
        for (int v = 0; v < nv; v++) {
            float bias = 0.f;
            if (has_bias) bias = load_bias(p.bias, p.bias_dt, p.bias_mode == BIAS_PER_M ? row : v);
            const __half o = epilogue_value<__half>(red[v * 128 + threadIdx.x], has_bias, bias, p.epilogue);
            ((__half *)p.out)[p.trans_out ? (long long)v * p.M + row : (long long)row * nv + v] = o;
        }
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

int b_region_bytes(int ks, int rb8, int b_rows) {
    int b = (ks / 128) * b_rows * 128;
    const int guard = (128 - rb8) * 128;
    if (b < guard) b = guard;
    return (b + 1023) & ~1023;
}

int b_rows_for(int nvmax) { return nvmax <= 4 ? 8 : nvmax <= 8 ? 16 : 32; }

size_t smem_for(int ks, int rb8, int nvmax, int split, int raw_ring, int a_ring) {
    const int nb = nvmax <= 8 ? 16 : 32, tgroups = (nvmax <= 4 ? 256 : 512) / (8 * nb);
    return 1024 + (size_t)a_ring * 2 * rb8 * 128 + b_region_bytes(ks, rb8, b_rows_for(nvmax)) + (size_t)raw_ring * rb8 * SB_BYTES +
           (size_t)a_ring * rb8 * 16 + (size_t)2 * nvmax * (MAX_KS / 32) * 4 + (size_t)2 * nvmax * 128 * 4 + (size_t)split * nvmax * 128 * 4 +
           (size_t)(nvmax * 4 + 2) * 4 + (size_t)(2 * raw_ring + 2 * a_ring + 2 * tgroups + 2) * 8 + 64;
}

} // namespace

// Work split for a [M][K] Q4_K weight against nv vectors: the K slices per cluster, rows per cluster and ring
// depths.  False when the shape is not one this kernel takes (the plan then uses gemv_q4k_mma.cu).
bool q4k_gemv_umma_config(int M, int K, int nv, int sm_count, Q4kUmmaConfig *cfg) {
    if (M < 1 || K < 256 || K % 256 != 0 || nv < 1 || nv > 16 || !encode_tiled_fn()) return false;
    const int nvmax = nv <= 1 ? 1 : nv <= 2 ? 2 : nv <= 4 ? 4 : nv <= 8 ? 8 : 16; // the kernel's template parameter
    // the split whose clusters own the most rows (fullest MMAs) among those that fit
    int best = 0, best_rb = 0;
    for (int split = 1; split <= 8; split *= 2) {
        if (K % (split * 256) != 0 || K / split > MAX_KS) continue;
        const int clusters = sm_count / split;
        if (clusters < 1) continue;
        const int rb = (M + clusters - 1) / clusters;
        if (rb > 128) continue;
        const int rb8 = (rb + 7) & ~7;
        if (smem_for(K / split, rb8, nvmax, split, 2, 2) > 227 * 1024) continue;
        if (rb > best_rb) { best = split; best_rb = rb; }
    }
    if (!best) return false;
    const int split = best, rb = best_rb, rb8 = (rb + 7) & ~7, ks = K / split, nsb = ks / 256;
    int raw_ring, a_ring = 2;
    if (nvmax <= 2 && smem_for(ks, rb8, nvmax, split, 2, 2) <= 113 * 1024) {
        // two CTAs per SM (this launch's and the next one's): two stages of each ring, a third raw one if it fits
        raw_ring = nsb > 2 && smem_for(ks, rb8, nvmax, split, 3, 2) <= 113 * 1024 ? 3 : 2;
    } else {
        // the SM to itself: all of the CTA's weights are requested at once when they fit (nothing waits for a slot), two
        // stages of codes suffice, a third takes what is left
        raw_ring = std::max(2, std::min(12, nsb));
        while (raw_ring > 2 && smem_for(ks, rb8, nvmax, split, raw_ring, a_ring) > 227 * 1024) raw_ring--;
        if (smem_for(ks, rb8, nvmax, split, raw_ring, a_ring) > 227 * 1024) return false;
        if (nsb > 2 && smem_for(ks, rb8, nvmax, split, raw_ring, 3) <= 227 * 1024) a_ring = 3;
    }
    cfg->split = split; cfg->clusters = sm_count / split; cfg->rb = rb; cfg->rb8 = rb8; cfg->ks = ks;
    cfg->raw_ring = raw_ring; cfg->a_ring = a_ring; cfg->nvmax = nvmax;
    cfg->b_bytes = b_region_bytes(ks, rb8, b_rows_for(nvmax));
    cfg->smem_bytes = smem_for(ks, rb8, nvmax, split, raw_ring, a_ring);
    return true;
}

cudaError_t launch_q4k_gemv_umma(const MatmulParams &p, int nv, const Q4kUmmaConfig &cfg, bool lhs_constant, cudaStream_t stream) {
    CUtensorMap map_w;
    {
        // [M][K/256][144] bytes; a box is one super-block of rb rows
        cuuint64_t dims[3] = {(cuuint64_t)SB_BYTES, (cuuint64_t)(p.K / 256), (cuuint64_t)p.M};
        cuuint64_t strides[2] = {(cuuint64_t)SB_BYTES, (cuuint64_t)(p.K / 256) * SB_BYTES};
        cuuint32_t box[3] = {(cuuint32_t)SB_BYTES, 1, (cuuint32_t)cfg.rb};
        cuuint32_t estr[3] = {1, 1, 1};
        if (encode_tiled_fn()(&map_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void *>(p.lhs), dims, strides, box, estr,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return cudaErrorInvalidValue;
    }
    Q4kUmmaParams up{};
    up.p = p;
    up.nv = nv;
    up.rb = cfg.rb; up.rb8 = cfg.rb8; up.ks = cfg.ks; up.nsb = cfg.ks / 256; up.split = cfg.split;
    up.raw_ring = cfg.raw_ring; up.a_ring = cfg.a_ring;
    up.raw_stage_bytes = cfg.rb8 * SB_BYTES;
    up.a_stage_bytes = 2 * cfg.rb8 * 128;
    up.b_bytes = cfg.b_bytes;
    up.inv_rb8_q20 = ((1 << 20) + cfg.rb8 - 1) / cfg.rb8;
    up.lhs_constant = lhs_constant ? 1 : 0;
    static SmemAttr smem_attr[5];
    void (*kernel)(CUtensorMap, Q4kUmmaParams) = nullptr;
    int slot = 0, threads = 0;
    switch (cfg.nvmax) {
    case 1: kernel = q4k_gemv_umma_kernel<1>; slot = 0; threads = Roles<1>::THREADS; break;
    case 2: kernel = q4k_gemv_umma_kernel<2>; slot = 1; threads = Roles<2>::THREADS; break;
    case 4: kernel = q4k_gemv_umma_kernel<4>; slot = 2; threads = Roles<4>::THREADS; break;
    case 8: kernel = q4k_gemv_umma_kernel<8>; slot = 3; threads = Roles<8>::THREADS; break;
    case 16: kernel = q4k_gemv_umma_kernel<16>; slot = 4; threads = Roles<16>::THREADS; break;
    default: return cudaErrorInvalidValue;
    }
    {
        cudaError_t e = smem_attr[slot].ensure(kernel, cfg.smem_bytes);
        if (e != cudaSuccess) return e;
    }
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3(cfg.clusters * cfg.split);
    lc.blockDim = dim3(threads);
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
    return cudaLaunchKernelEx(&lc, kernel, map_w, up);
}

cudaError_t gemv_q4k_umma_take_error(int *site, cudaStream_t stream) {
    int zero = 0;
    cudaError_t e = cudaMemcpyFromSymbolAsync(site, g_gemv_q4k_umma_error, sizeof(int), 0, cudaMemcpyDeviceToHost, stream);
    if (e != cudaSuccess) return e;
    e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess) return e;
    if (*site != 0) e = cudaMemcpyToSymbolAsync(g_gemv_q4k_umma_error, &zero, sizeof(int), 0, cudaMemcpyHostToDevice, stream);
    return e;
}

} // namespace rt
