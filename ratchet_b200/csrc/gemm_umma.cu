// Tensor-core GEMM for sm_100a: D[R][S] = P[R][K] . Q[S][K]^T with both operands K-major and
// 16-bit (f16 / bf16), f32 accumulation in tensor memory, fused bias / GELU epilogue.
//
// Takes the role of the reference's tiled GEMM (crates/ratchet-core/src/ops/gemm.rs:342-492) for
// the nn::Linear form W.gemm(X, b, false, true, true) (crates/ratchet-nn/src/linear.rs:23), where
// both W [N,K] and X [M,K] are K-major.  With trans_out the activations are P and the weight is Q
// (output [M][N]); without it the roles swap (output [N][M]).  Quantised weights reach this
// kernel as 16-bit values: the dequantise pre-pass (dequant.cu) writes them to a scratch buffer
// owned by the plan with the reference's rounding (f16(q) * d rounded to f16, gemm.rs:400-406).
//
// Structure (one persistent CTA per SM, 320 threads):
//   warp 0      TMA producer: 128B-swizzled tiles of P (128 x 64) and Q (BN x 64) into a
//               multi-stage shared-memory ring, completion on mbarriers
//   warp 1      allocates tensor memory; one lane issues tcgen05.mma (128 x BN x 16 per
//               instruction), tcgen05.commit releases ring stages and publishes accumulators
//   warps 2-9   epilogue: tcgen05.ld of one of two accumulator buffers (so the next tile's MMAs
//               overlap), the reference's epilogue chain, stores staged through shared memory so
//               that every store instruction writes whole 128-byte lines
// Every wait is bounded (about two seconds of SM cycles); on expiry the kernel records the wait site in a device
// flag, all roles leave their loops, tensor memory is freed and the kernel returns.  The host
// reads the flag at the next rt_device_sync.
#include <cuda.h>

#include <algorithm>
#include <unordered_map>
#include <string>
#include <mutex>
#include <cstdlib>
#include <cstring>

#include "common.cuh"
#include "kernels.hpp"

namespace rt {

__device__ int g_umma_error = 0;

namespace {

constexpr int BM = 128;
constexpr int BK = 64; // 64 x 16-bit = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int TILE_GROUP_ROWS = 2048;     // rows per group of the tile order (see tile_coords), when it is grouped
constexpr int EPI_WARPS = 8;             // two per tensor-memory lane quarter, alternating 64-column rounds
constexpr int NUM_THREADS = 64 + EPI_WARPS * 32;
constexpr int STG_ROW_BYTES = 128;       // 64 outputs of 2 bytes; 16-byte chunks XOR-swizzled by row: conflict-free both ways
constexpr unsigned long long WAIT_LIMIT_CYCLES = 4000000000ull; // about 2 s at the SM clock

struct UmmaParams {
    int R, S, K;
    int stacks, p_stack, q_stack;
    void *out;
    long long out_batch_stride;
    // Output placement: element (r, s) of batch b goes to outs[d][b*out_batch_stride + r*out_ld + out_col + s] for
    // every destination d.  One destination with out_ld = S, out_col = 0 is the plain case; several
    // destinations are the N-sharded form, where each GPU writes its column slice straight into
    // every GPU's full-width output through peer-mapped pointers (plain stores over NVLink).
    int n_out;
    void *outs[RT_MAX_PEERS];
    long long out_ld, out_col;
    const void *bias;
    int bias_dt, bias_mode; // BIAS_PER_N: index along S; BIAS_PER_M: index along R
    int epilogue;
    // RT_EPILOGUE_SILU_MUL: Q is [2*ff][K], gate rows then up rows.  A tile's BN accumulator columns are BN/2 gate
    // rows and the BN/2 up rows that pair with them (one 4-D copy whose third extent steps from the gate half to
    // the up half), and the epilogue writes BN/2 output columns up * silu(gate): pair = 1, s_out = ff, and tiles
    // advance by BN/2 output columns.  Otherwise pair = 0 and s_out = S.
    int pair, s_out;
    int tiles_r, tiles_s;
    int group_r; // tile rows per group of the tile order (tile_coords); tiles_r: plain order, tile rows fastest
    int tma_store; // CTA-pair kernel: the epilogue hands its staged 32 x 64 blocks to TMA stores (one per destination)
    uint32_t idesc;
    // Factors that were taken out of an operand's rows before the product (bf16 activations brought into f16's range):
    // p_scale [p_stack][R], q_scale [q_stack][S], either may be null; they go back onto the f32 accumulators.
    const float *p_scale, *q_scale;
};

template <int BN> struct Cfg {
    static constexpr int STAGES = BN == 256 ? 4 : 6;
    static constexpr int A_BYTES = BM * BK * 2;
    static constexpr int B_BYTES = BN * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int TMEM_COLS = 2 * BN; // two accumulator buffers
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment*/ + 256 /*barriers*/ + BN * 4 /*bias*/ +
                                      EPI_WARPS * 32 * STG_ROW_BYTES /*store staging*/;
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

// The SM's own cycle counter bounds the waits: it is a register read, where %globaltimer is a
// long-latency access that would sit on the critical path of every stage hand-over.
__device__ __forceinline__ unsigned long long wait_clock() { return (unsigned long long)clock64(); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}

// Bounded wait.  Returns false when the wait expired or another role already gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, int site) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = wait_clock();
    while (true) {
#pragma unroll 1
        for (int i = 0; i < 32; i++)
            if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (wait_clock() - t0 > WAIT_LIMIT_CYCLES) {
            *abort_flag = 1;
            atomicCAS(&g_umma_error, 0, site);
            return false;
        }
    }
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *map, int c0, int c1, int c2, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                 ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2), "r"(bar)
                 : "memory");
}

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap *map, int c0, int c1, int c2, int c3, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
                 ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar)
                 : "memory");
}

// Shared-memory matrix descriptor: K-major tile, 128-byte swizzle, rows of 128 bytes, 8-row
// groups 1024 bytes apart (the layout a 128B-swizzled TMA box produces).
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;            // leading byte offset: unused for swizzled K-major
    d |= (uint64_t)(1024 >> 4) << 32;  // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;            // descriptor version of sm_100
    d |= (uint64_t)2 << 61;            // 128-byte swizzle
    return d;
}

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
                 ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
                 : "memory");
}

__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
          "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Order of a batch's tiles: groups of `group_r` tile rows; inside a group the tile rows run fastest, then the tile
// columns.  The CTAs working at the same time then share a few tiles of each operand (which stay in L2) instead of one
// operand's single tile against a whole sweep of the other (row-major order reads [32768][2560] activations again for
// every one of 40 tile columns: 6.7 GB instead of 0.9 GB).
__device__ __forceinline__ void tile_coords(int rem, int tiles_r, int tiles_s, int group_r, int &tr, int &ts) {
    const int per_group = group_r * tiles_s;
    const int g = rem / per_group, first_r = g * group_r;
    const int rows = min(group_r, tiles_r - first_r);
    const int in = rem - g * per_group;
    ts = in / rows;
    tr = first_r + in - ts * rows;
}

template <typename OutT> __device__ __forceinline__ uint32_t pack2(float a, float b);
template <> __device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
    __half2 h = __halves2half2(__float2half_rn(a), __float2half_rn(b));
    return *reinterpret_cast<uint32_t *>(&h);
}
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
    __nv_bfloat162 h = __halves2bfloat162(__float2bfloat16_rn(a), __float2bfloat16_rn(b));
    return *reinterpret_cast<uint32_t *>(&h);
}

// epilogue_value over 32 accumulator columns of one row, results into the row's staging line (chunk h*4+g, XOR-swizzled
// by the row).  BIAS: 0 none, 1 per column (bias32 = this round's 32 values in shared memory), 2 per row.  The f16
// form is epilogue_value<__half> step by step (round the accumulator, add the bias in f32 and round, GELU in f32 and
// round) on pairs, so that each rounding is one packed conversion; the bf16 form rounds once, at the end.
template <typename OutT, int BIAS, bool GELU>
__device__ __forceinline__ void epilogue_math32(const uint32_t (&v)[32], const float *bias32, float row_bias, uint8_t *row_stg, int h, int lane) {
#pragma unroll
    for (int g = 0; g < 4; g++) {
        uint32_t w[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int i0 = g * 8 + j * 2;
            float2 f = make_float2(__uint_as_float(v[i0]), __uint_as_float(v[i0 + 1]));
            float2 b = make_float2(row_bias, row_bias);
            if (BIAS == 1) b = *reinterpret_cast<const float2 *>(bias32 + i0);
            if (cuda::std::is_same<OutT, __half>::value) {
                __half2 hh = __floats2half2_rn(f.x, f.y);
                if (BIAS != 0) {
                    f = __half22float2(hh);
                    hh = __floats2half2_rn(f.x + b.x, f.y + b.y);
                }
                if (GELU) {
                    f = __half22float2(hh);
                    hh = __floats2half2_rn(gelu_tanh_f32(f.x), gelu_tanh_f32(f.y));
                }
                w[j] = *reinterpret_cast<uint32_t *>(&hh);
            } else {
                if (BIAS != 0) { f.x += b.x; f.y += b.y; }
                if (GELU) { f.x = gelu_tanh_f32(f.x); f.y = gelu_tanh_f32(f.y); }
                w[j] = pack2<OutT>(f.x, f.y);
            }
        }
        *reinterpret_cast<uint4 *>(row_stg + (((h * 4 + g) ^ (lane & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
    }
}

// The plain epilogue of one accumulator tile (128 rows x BN columns of this CTA's tensor memory at `tmem_acc`): 64
// columns per round: two tensor-memory loads, the epilogue arithmetic, then through a per-warp staging buffer so that
// global stores run along rows: 8 lanes x 16 B = one full 128-byte line per row (this matters most when the destination
// is a peer GPU over NVLink).  `bar_done` (this CTA's barrier, or with REMOTE_DONE the shared::cluster address of the
// leading CTA's) gets one arrival per warp once the warp has read its part of the accumulator.
__device__ __forceinline__ void arrive_cluster(uint32_t bar_cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}

// One tensor map per destination of the output ([stacks][R][window end] of 16-bit values, 128-byte swizzle, boxes of 64
// columns x 32 rows: what one epilogue warp stages per round).
struct OutMaps {
    CUtensorMap m[RT_MAX_PEERS];
};
__device__ __forceinline__ void tma_store_3d(const CUtensorMap *map, int c0, int c1, int c2, uint32_t src) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%1, %2, %3}], [%4];"
                 ::"l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2), "r"(src) : "memory");
}

// Operand factors (UmmaParams::p_scale, q_scale) exist for bf16 activations only, and those have bf16 outputs: the
// f16 kernels carry none of that code.
template <typename OutT> constexpr bool HAS_OPERAND_FACTORS = !cuda::std::is_same<OutT, __half>::value;

template <int BN, typename OutT, bool REMOTE_DONE, bool TMA_STORE = false>
__device__ __forceinline__ void epilogue_tile(const UmmaParams &prm, uint32_t tmem_acc, uint32_t bar_done, int r0, int s0, int b, int q, int half,
                                              int lane, uint8_t *stg, const float *bias_s, bool has_bias, float row_bias, float row_mul,
                                              bool vec_ok, bool pair_ok, const OutMaps *omaps = nullptr) {
#pragma unroll 1
    for (int cc = half; cc < BN / 64; cc += 2) {
        const int colbase = s0 + cc * 64;
        if (TMA_STORE && prm.tma_store) {
            // the stores of the previous round have read the staging block
            if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
            __syncwarp();
        }
        // not unrolled: a CTA with one tile runs this code once, straight from a cold instruction cache (a fifth of the
        // warps' stall cycles of a one-tile launch were instruction fetches), so half the code is half of those misses
#pragma unroll 1
        for (int h = 0; h < 2; h++) {
            const int c = cc * 2 + h;
            uint32_t v[32];
            tmem_ld32(tmem_acc + c * 32 + ((uint32_t)(q * 32) << 16), v);
            if (HAS_OPERAND_FACTORS<OutT>) {
#pragma unroll
                for (int i = 0; i < 32; i++) v[i] = __float_as_uint(__uint_as_float(v[i]) * row_mul); // 1 where P has no factors
                if (prm.q_scale) {
                    const float *qs = prm.q_scale + (long long)(b % prm.q_stack) * prm.S;
#pragma unroll
                    for (int i = 0; i < 32; i++) v[i] = __float_as_uint(__uint_as_float(v[i]) * __ldg(qs + min(s0 + c * 32 + i, prm.S - 1)));
                }
            }
            if (cc + 2 >= BN / 64 && h == 1) {
                // the accumulator has been read completely: hand it back to the MMA warp now
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    if (REMOTE_DONE) arrive_cluster(bar_done);
                    else mbar_arrive(bar_done);
                }
            }
            {
                // the arithmetic of 32 columns, compiled once per (bias, GELU) form: with the two switches tested for every
                // element the eight epilogue warps took 0.8 us per 32 columns without GELU and 2.1 us with it, which is
                // most of a one-tile launch
                uint8_t *row_stg = stg + lane * STG_ROW_BYTES;
                const float *b32 = bias_s + c * 32;
                const int form = (has_bias ? (prm.bias_mode == BIAS_PER_N ? 2 : 4) : 0) | (prm.epilogue == RT_EPILOGUE_GELU_TANH ? 1 : 0);
                switch (form) {
                case 0: epilogue_math32<OutT, 0, false>(v, b32, row_bias, row_stg, h, lane); break;
                case 1: epilogue_math32<OutT, 0, true>(v, b32, row_bias, row_stg, h, lane); break;
                case 2: epilogue_math32<OutT, 1, false>(v, b32, row_bias, row_stg, h, lane); break;
                case 3: epilogue_math32<OutT, 1, true>(v, b32, row_bias, row_stg, h, lane); break;
                case 4: epilogue_math32<OutT, 2, false>(v, b32, row_bias, row_stg, h, lane); break;
                default: epilogue_math32<OutT, 2, true>(v, b32, row_bias, row_stg, h, lane); break;
                }
            }
        }
        __syncwarp();
        if (TMA_STORE && prm.tma_store) {
            // The staged block is the image a 128-byte-swizzled TMA box wants (16-byte chunks XOR the row index, the
            // warp's block on a 1024-byte boundary): one bulk store per destination, clipped by the map at the tensor's
            // last row and at the end of this shard's column window.
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) {
                for (int d = 0; d < prm.n_out; d++)
                    tma_store_3d(&omaps->m[d], (int)prm.out_col + colbase, r0 + q * 32, b, smem_u32(stg));
                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            }
        } else if (vec_ok) {
            const int colv = colbase + (lane & 7) * 8;
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const int rl = 4 * i + (lane >> 3);
                const int rg = r0 + q * 32 + rl;
                if (rg < prm.R && colv < prm.s_out) {
                    const uint4 pk = *reinterpret_cast<const uint4 *>(stg + rl * STG_ROW_BYTES + (((lane & 7) ^ (rl & 7)) << 4));
                    const long long off = (long long)b * prm.out_batch_stride + (long long)rg * prm.out_ld + prm.out_col + colv;
                    for (int d = 0; d < prm.n_out; d++) *reinterpret_cast<uint4 *>(reinterpret_cast<OutT *>(prm.outs[d]) + off) = pk;
                }
            }
        } else if (pair_ok) {
            // rows that start on 4-byte but not on 16-byte boundaries: a warp writes the round's 64
            // columns of one row as 32 element pairs per instruction
#pragma unroll 4
            for (int rl = 0; rl < 32; rl++) {
                const int rg = r0 + q * 32 + rl;
                if (rg >= prm.R) break;
                const int col = 2 * lane;
                if (colbase + col < prm.s_out) {
                    const uint32_t o2 = *reinterpret_cast<const uint32_t *>(stg + rl * STG_ROW_BYTES + (((col >> 3) ^ (rl & 7)) << 4) + (col & 7) * 2);
                    const long long off = (long long)b * prm.out_batch_stride + (long long)rg * prm.out_ld + prm.out_col + colbase + col;
                    for (int d = 0; d < prm.n_out; d++) *reinterpret_cast<uint32_t *>(reinterpret_cast<OutT *>(prm.outs[d]) + off) = o2;
                }
            }
        } else {
            // any other row alignment: element stores, still along the rows
#pragma unroll 4
            for (int rl = 0; rl < 32; rl++) {
                const int rg = r0 + q * 32 + rl;
                if (rg >= prm.R) break;
                const long long off = (long long)b * prm.out_batch_stride + (long long)rg * prm.out_ld + prm.out_col + colbase;
#pragma unroll
                for (int k = 0; k < 2; k++) {
                    const int col = lane + 32 * k;
                    if (colbase + col < prm.s_out) {
                        const OutT o = *reinterpret_cast<const OutT *>(stg + rl * STG_ROW_BYTES + (((col >> 3) ^ (rl & 7)) << 4) + (col & 7) * 2);
                        for (int d = 0; d < prm.n_out; d++) reinterpret_cast<OutT *>(prm.outs[d])[off + col] = o;
                    }
                }
            }
        }
        __syncwarp();
    }
}

// PAIR: the gate/up fold of RT_EPILOGUE_SILU_MUL (see UmmaParams::pair), compiled only into the kernels that run it
template <int BN, typename OutT, bool PAIR>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_umma_kernel(const __grid_constant__ CUtensorMap map_p, const __grid_constant__ CUtensorMap map_q, const UmmaParams prm) {
    using C = Cfg<BN>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *tiles = smem;
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + C::STAGES * C::STAGE_BYTES);
    // bars[0..S): full, [S..2S): empty, [2S..2S+2): tmem_full, [2S+2..2S+4): tmem_empty
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * C::STAGES + 4);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    float *bias_s = reinterpret_cast<float *>(smem + C::STAGES * C::STAGE_BYTES + 256);
    uint8_t *stage_out = smem + C::STAGES * C::STAGE_BYTES + 256 + BN * 4;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t bar_full = smem_u32(bars), bar_empty = smem_u32(bars + C::STAGES);
    const uint32_t bar_tfull = smem_u32(bars + 2 * C::STAGES), bar_tempty = smem_u32(bars + 2 * C::STAGES + 2);

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::STAGES; s++) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, 1);
        }
        for (int a = 0; a < 2; a++) {
            mbar_init(bar_tfull + 8 * a, 1);
            mbar_init(bar_tempty + 8 * a, EPI_WARPS); // one arrival per epilogue warp
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(C::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // Everything so far touched no global data: it ran beside the stream predecessor (programmatic dependent
    // launch).  Operands, bias and output wait for it; the successor may start its own prologue.
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
                int tr, ts;
                tile_coords(rem, prm.tiles_r, prm.tiles_s, prm.group_r, tr, ts);
                const int r0 = tr * BM, s0 = ts * (PAIR ? BN / 2 : BN);
                const int bp = b % prm.p_stack, bq = b % prm.q_stack;
                for (int kb = 0; kb < num_k; kb++) {
                    if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1, abort_flag, 1)) { ok = false; break; }
                    const uint32_t a_dst = smem_u32(tiles + stage * C::STAGE_BYTES);
                    mbar_expect_tx(bar_full + 8 * stage, C::STAGE_BYTES);
                    tma_load_3d(a_dst, &map_p, kb * BK, r0, bp, bar_full + 8 * stage);
                    if (PAIR) tma_load_4d(a_dst + C::A_BYTES, &map_q, kb * BK, s0, 0, bq, bar_full + 8 * stage);
                    else tma_load_3d(a_dst + C::A_BYTES, &map_q, kb * BK, s0, bq, bar_full + 8 * stage);
                    if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            int stage = 0, acc = 0;
            uint32_t phase = 0, acc_phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                if (!mbar_wait(bar_tempty + 8 * acc, acc_phase ^ 1, abort_flag, 2)) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int kb = 0; kb < num_k; kb++) {
                    if (!mbar_wait(bar_full + 8 * stage, phase, abort_flag, 3)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(tiles + stage * C::STAGE_BYTES);
                    const uint32_t b_addr = a_addr + C::A_BYTES;
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; k++) {
                        umma_f16(d_tmem, umma_desc_sw128(a_addr + k * UMMA_K * 2), umma_desc_sw128(b_addr + k * UMMA_K * 2),
                                 prm.idesc, (kb | k) != 0 ? 1u : 0u);
                    }
                    umma_commit(bar_empty + 8 * stage); // stage reusable once these MMAs have read it
                    if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
                umma_commit(bar_tfull + 8 * acc); // accumulator complete
                if (++acc == 2) { acc = 0; acc_phase ^= 1; }
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue (warps 2..9)
        const int q = warp & 3;            // the tensor-memory lane quarter this warp may read
        const int half = (warp - 2) >> 2;  // which of the alternating 64-column rounds it takes
        const int ep_tid = threadIdx.x - 64;
        int acc = 0;
        uint32_t acc_phase = 0;
        bool vec_ok = (prm.s_out % 8 == 0) && (prm.out_ld % 8 == 0) && (prm.out_col % 8 == 0) && (prm.out_batch_stride % 8 == 0);
        bool pair_ok = (prm.s_out % 2 == 0) && (prm.out_ld % 2 == 0) && (prm.out_col % 2 == 0) && (prm.out_batch_stride % 2 == 0);
        for (int d = 0; d < prm.n_out; d++) {
            vec_ok = vec_ok && (reinterpret_cast<uintptr_t>(prm.outs[d]) % 16 == 0);
            pair_ok = pair_ok && (reinterpret_cast<uintptr_t>(prm.outs[d]) % 4 == 0);
        }
        bool gave_up = false; // a wait of this warp ran out: it skips its work but stays in step with the other warps
        for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
            const int b = tile / tiles_per_batch, rem = tile % tiles_per_batch;
            int tr, ts;
            tile_coords(rem, prm.tiles_r, prm.tiles_s, prm.group_r, tr, ts);
            const int r0 = tr * BM, s0 = ts * (PAIR ? BN / 2 : BN);
            // The eight warps leave together: the barrier hands every thread the OR of what each of them saw, so
            // none is left waiting at a barrier for a warp that has gone.
            if (bar_red_or(1, EPI_WARPS * 32, gave_up || *abort_flag != 0)) break;
            // bias values of this tile's columns, shared by the epilogue warps
            if (prm.bias_mode == BIAS_PER_N) {
                for (int j = ep_tid; j < BN; j += EPI_WARPS * 32) {
                    // paired tiles: accumulator column j holds weight row (j / (BN/2)) * ff + s0 + j % (BN/2)
                    const int jj = PAIR ? j % (BN / 2) : j;
                    const int wrow = PAIR ? (j / (BN / 2)) * prm.s_out + s0 + jj : s0 + j;
                    bias_s[j] = (s0 + jj < prm.s_out) ? load_bias(prm.bias, prm.bias_dt, wrow) : 0.f;
                }
            }
            asm volatile("bar.sync 1, %0;" ::"n"(EPI_WARPS * 32) : "memory");
            if (!mbar_wait(bar_tfull + 8 * acc, acc_phase, abort_flag, 4)) { gave_up = true; continue; }
            tc_fence_after();
            const int row = r0 + q * 32 + lane;
            const bool has_bias = prm.bias_mode != BIAS_NONE;
            float row_bias = 0.f;
            if (prm.bias_mode == BIAS_PER_M && row < prm.R) row_bias = load_bias(prm.bias, prm.bias_dt, row);
            const float row_mul = (HAS_OPERAND_FACTORS<OutT> && prm.p_scale && row < prm.R) ? __ldg(prm.p_scale + (long long)(b % prm.p_stack) * prm.R + row) : 1.f;
            // 64 columns per round: two tensor-memory loads, the epilogue arithmetic, then through a
            // per-warp staging buffer so that global stores run along rows: 8 lanes x 16 B = one full
            // 128-byte line per row (this matters most when the destination is a peer GPU over NVLink)
            uint8_t *stg = stage_out + (warp - 2) * (32 * STG_ROW_BYTES);
            if (PAIR) {
                // 32 output columns per round: the gate accumulators, the up accumulators BN/2 columns further on,
                // up * silu(gate), then out through the staging rows (four 16-byte chunks each)
#pragma unroll 1
                for (int cc = half; cc < BN / 64; cc += 2) {
                    const int colbase = s0 + cc * 32;
                    uint32_t vg[32], vu[32];
                    tmem_ld32(tmem_base + acc * BN + cc * 32 + ((uint32_t)(q * 32) << 16), vg);
                    tmem_ld32(tmem_base + acc * BN + BN / 2 + cc * 32 + ((uint32_t)(q * 32) << 16), vu);
                    if (cc + 2 >= BN / 64) {
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(bar_tempty + 8 * acc);
                    }
#pragma unroll
                    for (int g = 0; g < 4; g++) {
                        uint32_t w[4];
#pragma unroll
                        for (int j = 0; j < 4; j++) {
                            float o[2];
#pragma unroll
                            for (int e = 0; e < 2; e++) {
                                const int i = g * 8 + j * 2 + e;
                                const float bg = has_bias ? bias_s[cc * 32 + i] : 0.f;
                                const float bu = has_bias ? bias_s[BN / 2 + cc * 32 + i] : 0.f;
                                const float ga = HAS_OPERAND_FACTORS<OutT> ? __uint_as_float(vg[i]) * row_mul : __uint_as_float(vg[i]);
                                const float ua = HAS_OPERAND_FACTORS<OutT> ? __uint_as_float(vu[i]) * row_mul : __uint_as_float(vu[i]);
                                const OutT gv = epilogue_value<OutT>(ga, has_bias, bg, RT_EPILOGUE_NONE);
                                const OutT uv = epilogue_value<OutT>(ua, has_bias, bu, RT_EPILOGUE_NONE);
                                o[e] = to_f32(silu_mul_value<OutT>(gv, uv));
                            }
                            w[j] = pack2<OutT>(o[0], o[1]);
                        }
                        *reinterpret_cast<uint4 *>(stg + lane * STG_ROW_BYTES + ((g ^ (lane & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                    __syncwarp();
                    if (vec_ok) {
                        const int colv = colbase + (lane & 3) * 8;
#pragma unroll
                        for (int i = 0; i < 4; i++) {
                            const int rl = 8 * i + (lane >> 2);
                            const int rg = r0 + q * 32 + rl;
                            if (rg < prm.R && colv < prm.s_out) {
                                const uint4 pk = *reinterpret_cast<const uint4 *>(stg + rl * STG_ROW_BYTES + (((lane & 3) ^ (rl & 7)) << 4));
                                const long long off = (long long)b * prm.out_batch_stride + (long long)rg * prm.out_ld + prm.out_col + colv;
                                for (int d = 0; d < prm.n_out; d++) *reinterpret_cast<uint4 *>(reinterpret_cast<OutT *>(prm.outs[d]) + off) = pk;
                            }
                        }
                    } else {
#pragma unroll 4
                        for (int rl = 0; rl < 32; rl++) {
                            const int rg = r0 + q * 32 + rl;
                            if (rg >= prm.R) break;
                            if (colbase + lane < prm.s_out) {
                                const OutT o = *reinterpret_cast<const OutT *>(stg + rl * STG_ROW_BYTES + (((lane >> 3) ^ (rl & 7)) << 4) + (lane & 7) * 2);
                                const long long off = (long long)b * prm.out_batch_stride + (long long)rg * prm.out_ld + prm.out_col + colbase + lane;
                                for (int d = 0; d < prm.n_out; d++) reinterpret_cast<OutT *>(prm.outs[d])[off] = o;
                            }
                        }
                    }
                    __syncwarp();
                }
                if (++acc == 2) { acc = 0; acc_phase ^= 1; }
                continue;
            }
            epilogue_tile<BN, OutT, false>(prm, tmem_base + acc * BN, bar_tempty + 8 * acc, r0, s0, b, q, half, lane, stg, bias_s, has_bias, row_bias,
                                    row_mul, vec_ok, pair_ok);
            if (++acc == 2) { acc = 0; acc_phase ^= 1; }
        }
    }

    // ---------------------------------------------------------------- teardown
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        // give copies that may still be in flight time to land before the CTA's memory is released
        const unsigned long long t0 = wait_clock();
        while (wait_clock() - t0 < 400000ull) __nanosleep(1000);
    }
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(C::TMEM_COLS) : "memory");
    }
}

// ------------------------------------------------------------------------------------------ CTA pairs
// The same GEMM with two CTAs (a cluster of two SMs) on one 256 x 256 tile: tcgen05.mma cta_group::2.  Each CTA
// stages its own 128 rows of P and HALF of the tile's 256 rows of Q (every copy is a plain TMA load into the CTA's own
// shared memory whose completion is counted on the leading CTA's barrier; no copy is multicast), the leading CTA's
// thread issues one MMA for both SMs, which read both halves of Q, and each SM's tensor memory receives its own 128 rows
// of the tile.  Per MMA cycle an SM then takes 64 bytes of operands from shared memory instead of 96, and a stage is 32 KB
// instead of 48: six stages in flight instead of four.
//   full[s]      leading CTA: its producer's arrival with the byte count of both CTAs' copies
//   empty[s]     both CTAs: the leading CTA's tcgen05.commit, multicast to both
//   tmem_full    both CTAs: the same commit after a tile's last MMA
//   tmem_empty   leading CTA: one arrival per epilogue warp of both CTAs
constexpr int P2_STAGES = 6;
constexpr int P2_BN = 256;
constexpr int P2_A_BYTES = BM * BK * 2, P2_B_BYTES = (P2_BN / 2) * BK * 2, P2_STAGE_BYTES = P2_A_BYTES + P2_B_BYTES;
constexpr int P2_SMEM_BYTES = P2_STAGES * P2_STAGE_BYTES + 1024 + 256 + P2_BN * 4 + EPI_WARPS * 32 * STG_ROW_BYTES;

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t cta) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(cta));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// A tile into this CTA's shared memory, its bytes counted on the barrier at `bar_cluster` (the leading CTA's)
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const CUtensorMap *map, int c0, int c1, int c2, uint32_t bar_cluster) {
    asm volatile("cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                 ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2), "r"(bar_cluster)
                 : "memory");
}
__device__ __forceinline__ void umma_f16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
                 ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
                 : "memory");
}
// arrives on the barrier at this offset in both CTAs of the pair once the MMAs issued so far are complete
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
    asm volatile("{\n\t.reg .b16 m;\n\tmov.b16 m, 3;\n\t"
                 "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], m;\n\t}\n" ::"r"(bar)
                 : "memory");
}

template <typename OutT>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_umma_pair_kernel(const __grid_constant__ CUtensorMap map_p, const __grid_constant__ CUtensorMap map_q, const __grid_constant__ OutMaps omaps,
                      const UmmaParams prm) {
    constexpr int BN = P2_BN;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *tiles = smem;
    // the store staging follows the ring, so each warp's 4 KB block sits on a 1024-byte boundary (the TMA stores' swizzle)
    uint8_t *stage_out = smem + P2_STAGES * P2_STAGE_BYTES;
    uint64_t *bars = reinterpret_cast<uint64_t *>(stage_out + EPI_WARPS * 32 * STG_ROW_BYTES);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * P2_STAGES + 4);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    float *bias_s = reinterpret_cast<float *>(reinterpret_cast<uint8_t *>(bars) + 256);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank(); // 0: the leading CTA
    const uint32_t bar_full = smem_u32(bars), bar_empty = smem_u32(bars + P2_STAGES);
    const uint32_t bar_tfull = smem_u32(bars + 2 * P2_STAGES), bar_tempty = smem_u32(bars + 2 * P2_STAGES + 2);

    if (threadIdx.x == 0) {
        for (int s = 0; s < P2_STAGES; s++) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, 1);
        }
        for (int a = 0; a < 2; a++) {
            mbar_init(bar_tfull + 8 * a, 1);
            mbar_init(bar_tempty + 8 * a, 2 * EPI_WARPS); // the epilogue warps of both CTAs
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) { // the same warp of both CTAs: the allocation is one operation of the pair
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "n"(2 * P2_BN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all(); // both CTAs' barriers exist before either signals the other's
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");

    const int num_k = (prm.K + BK - 1) / BK;
    const int tiles_per_batch = prm.tiles_r * prm.tiles_s; // tiles of 256 x 256
    const int total_tiles = tiles_per_batch * prm.stacks;
    const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;

    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer (both CTAs)
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int tile = pair; tile < total_tiles && ok; tile += num_pairs) {
                const int b = tile / tiles_per_batch, rem = tile % tiles_per_batch;
                int tr, ts;
                tile_coords(rem, prm.tiles_r, prm.tiles_s, prm.group_r, tr, ts);
                const int r0 = tr * 2 * BM + (int)rank * BM, s0 = ts * BN + (int)rank * (BN / 2);
                const int bp = b % prm.p_stack, bq = b % prm.q_stack;
                for (int kb = 0; kb < num_k; kb++) {
                    if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1, abort_flag, 1)) { ok = false; break; }
                    const uint32_t a_dst = smem_u32(tiles + stage * P2_STAGE_BYTES);
                    if (rank == 0) mbar_expect_tx(bar_full + 8 * stage, 2 * P2_STAGE_BYTES);
                    const uint32_t full0 = map_to_cta(bar_full + 8 * stage, 0);
                    tma_load_3d_pair(a_dst, &map_p, kb * BK, r0, bp, full0);
                    tma_load_3d_pair(a_dst + P2_A_BYTES, &map_q, kb * BK, s0, bq, full0);
                    if (++stage == P2_STAGES) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer (the leading CTA only)
        if (lane == 0 && rank == 0) {
            int stage = 0, acc = 0;
            uint32_t phase = 0, acc_phase = 0;
            bool ok = true;
            for (int tile = pair; tile < total_tiles && ok; tile += num_pairs) {
                if (!mbar_wait(bar_tempty + 8 * acc, acc_phase ^ 1, abort_flag, 2)) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int kb = 0; kb < num_k; kb++) {
                    if (!mbar_wait(bar_full + 8 * stage, phase, abort_flag, 3)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(tiles + stage * P2_STAGE_BYTES);
                    const uint32_t b_addr = a_addr + P2_A_BYTES;
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; k++) {
                        umma_f16_pair(d_tmem, umma_desc_sw128(a_addr + k * UMMA_K * 2), umma_desc_sw128(b_addr + k * UMMA_K * 2), prm.idesc,
                                      (kb | k) != 0 ? 1u : 0u);
                    }
                    umma_commit_pair(bar_empty + 8 * stage); // both CTAs' stages are reusable once these MMAs have read them
                    if (++stage == P2_STAGES) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
                umma_commit_pair(bar_tfull + 8 * acc); // both CTAs' accumulators are complete
                if (++acc == 2) { acc = 0; acc_phase ^= 1; }
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue (warps 2..9 of both CTAs)
        const int q = warp & 3;
        const int half = (warp - 2) >> 2;
        const int ep_tid = threadIdx.x - 64;
        int acc = 0;
        uint32_t acc_phase = 0;
        bool vec_ok = (prm.s_out % 8 == 0) && (prm.out_ld % 8 == 0) && (prm.out_col % 8 == 0) && (prm.out_batch_stride % 8 == 0);
        bool pair_ok = (prm.s_out % 2 == 0) && (prm.out_ld % 2 == 0) && (prm.out_col % 2 == 0) && (prm.out_batch_stride % 2 == 0);
        for (int d = 0; d < prm.n_out; d++) {
            vec_ok = vec_ok && (reinterpret_cast<uintptr_t>(prm.outs[d]) % 16 == 0);
            pair_ok = pair_ok && (reinterpret_cast<uintptr_t>(prm.outs[d]) % 4 == 0);
        }
        const uint32_t tempty0 = map_to_cta(bar_tempty, 0);
        bool gave_up = false;
        for (int tile = pair; tile < total_tiles; tile += num_pairs) {
            const int b = tile / tiles_per_batch, rem = tile % tiles_per_batch;
            int tr, ts;
            tile_coords(rem, prm.tiles_r, prm.tiles_s, prm.group_r, tr, ts);
            const int r0 = tr * 2 * BM + (int)rank * BM, s0 = ts * BN;
            if (bar_red_or(1, EPI_WARPS * 32, gave_up || *abort_flag != 0)) break;
            if (prm.bias_mode == BIAS_PER_N) {
                for (int j = ep_tid; j < BN; j += EPI_WARPS * 32)
                    bias_s[j] = (s0 + j < prm.S) ? load_bias(prm.bias, prm.bias_dt, s0 + j) : 0.f;
            }
            asm volatile("bar.sync 1, %0;" ::"n"(EPI_WARPS * 32) : "memory");
            if (!mbar_wait(bar_tfull + 8 * acc, acc_phase, abort_flag, 4)) { gave_up = true; continue; }
            tc_fence_after();
            const int row = r0 + q * 32 + lane;
            const bool has_bias = prm.bias_mode != BIAS_NONE;
            float row_bias = 0.f;
            if (prm.bias_mode == BIAS_PER_M && row < prm.R) row_bias = load_bias(prm.bias, prm.bias_dt, row);
            const float row_mul = (HAS_OPERAND_FACTORS<OutT> && prm.p_scale && row < prm.R) ? __ldg(prm.p_scale + (long long)(b % prm.p_stack) * prm.R + row) : 1.f;
            uint8_t *stg = stage_out + (warp - 2) * (32 * STG_ROW_BYTES);
            epilogue_tile<BN, OutT, true, true>(prm, tmem_base + acc * BN, tempty0 + 8 * acc, r0, s0, b, q, half, lane, stg, bias_s, has_bias, row_bias,
                                                row_mul, vec_ok, pair_ok, &omaps);
            if (++acc == 2) { acc = 0; acc_phase ^= 1; }
        }
        // the warp's bulk stores are complete (written, not only read) before the CTA goes
        if (prm.tma_store && lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    }

    // ---------------------------------------------------------------- teardown
    tc_fence_before();
    __syncthreads();
    cluster_sync_all(); // neither CTA leaves while the other may still signal its barriers or read its shared memory
    if (*abort_flag) {
        const unsigned long long t0 = wait_clock();
        while (wait_clock() - t0 < 400000ull) __nanosleep(1000);
    }
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "n"(2 * P2_BN) : "memory");
    }
}

// ------------------------------------------------------------------------------------------ host side

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) != cudaSuccess ||
            qres != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

// A tensor map is a pure function of its description, and a step launches the same few descriptions again and again
// (the reference compiles a node once and dispatches it many times, op.rs:304-362): the encoded maps are kept, so a launch
// outside a CUDA graph does not pay the driver's encoder each time.
CUresult encode_cached(CUtensorMap *map, CUtensorMapDataType dt, cuuint32_t rank, void *base, const cuuint64_t *dims, const cuuint64_t *strides,
                       const cuuint32_t *box, CUtensorMapL2promotion l2) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return CUDA_ERROR_NOT_SUPPORTED;
    std::string key;
    auto put = [&key](unsigned long long v) { key.append(reinterpret_cast<const char *>(&v), sizeof(v)); };
    put((unsigned long long)dt); put(rank); put((unsigned long long)(uintptr_t)base); put((unsigned long long)l2);
    for (cuuint32_t i = 0; i < rank; i++) { put(dims[i]); put(box[i]); }
    for (cuuint32_t i = 0; i + 1 < rank; i++) put(strides[i]);
    static std::mutex mu;
    static std::unordered_map<std::string, CUtensorMap> cache;
    {
        std::lock_guard<std::mutex> lk(mu);
        auto it = cache.find(key);
        if (it != cache.end()) {
            *map = it->second;
            return CUDA_SUCCESS;
        }
    }
    const cuuint32_t estr[5] = {1, 1, 1, 1, 1};
    const CUresult r = fn(map, dt, rank, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, l2,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r == CUDA_SUCCESS) {
        std::lock_guard<std::mutex> lk(mu);
        if (cache.size() >= 8192) cache.clear(); // bounded: addresses of freed buffers would otherwise pile up
        cache.emplace(std::move(key), *map);
    }
    return r;
}

// [stack][rows][K] 16-bit row-major -> boxes of box_rows x 64 elements, 128-byte swizzle, zero fill
bool make_map(CUtensorMap *map, const void *base, rt_dtype dt, long long K, long long rows, long long stack, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[3] = {(cuuint64_t)K, (cuuint64_t)rows, (cuuint64_t)stack};
    cuuint64_t strides[2] = {(cuuint64_t)K * 2, (cuuint64_t)K * 2 * (cuuint64_t)rows};
    cuuint32_t box[3] = {(cuuint32_t)BK, (cuuint32_t)box_rows, 1};
    return encode_cached(map, dt == RT_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void *>(base),
                         dims, strides, box, CU_TENSOR_MAP_L2_PROMOTION_L2_256B) == CUDA_SUCCESS;
}

// Q = [stack][2*ff][K] seen as [stack][2][ff][K]: one box of (64, box_rows, 2) brings box_rows gate rows and the
// box_rows up rows ff further on, the gate rows first in shared memory; rows past ff read as zero
bool make_pair_map(CUtensorMap *map, const void *base, rt_dtype dt, long long K, long long ff, long long stack, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[4] = {(cuuint64_t)K, (cuuint64_t)ff, 2, (cuuint64_t)stack};
    cuuint64_t strides[3] = {(cuuint64_t)K * 2, (cuuint64_t)K * 2 * (cuuint64_t)ff, (cuuint64_t)K * 4 * (cuuint64_t)ff};
    cuuint32_t box[4] = {(cuuint32_t)BK, (cuuint32_t)box_rows, 2, 1};
    return encode_cached(map, dt == RT_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void *>(base),
                         dims, strides, box, CU_TENSOR_MAP_L2_PROMOTION_L2_256B) == CUDA_SUCCESS;
}

// The grouped tile order pays when the row operand does not stay in L2 across a sweep of the tile columns (measured:
// [32768][2560] 16-bit rows, 168 MB: 1512 -> 1364 us; [8192][2560], 42 MB: 327 -> 347 us, so smaller ones keep the
// plain order).
bool grouped_order(const UmmaParams &prm) { return (long long)prm.R * prm.K * 2 > (64ll << 20); }

template <int BN, typename OutT>
cudaError_t launch_bn(const CUtensorMap &mp, const CUtensorMap &mq, UmmaParams prm, int sm_count, cudaStream_t stream) {
    using C = Cfg<BN>;
    static SmemAttr smem_attr;
    static SmemAttr smem_attr_pair;
    auto kernel = prm.pair ? gemm_umma_kernel<BN, OutT, true> : gemm_umma_kernel<BN, OutT, false>;
    {
        cudaError_t e = (prm.pair ? smem_attr_pair : smem_attr).ensure(kernel, C::SMEM_BYTES);
        if (e != cudaSuccess) return e;
    }
    prm.tiles_r = (prm.R + BM - 1) / BM;
    prm.group_r = grouped_order(prm) ? TILE_GROUP_ROWS / BM : prm.tiles_r;
    prm.tiles_s = prm.pair ? (prm.s_out + BN / 2 - 1) / (BN / 2) : (prm.S + BN - 1) / BN;
    // instruction descriptor: f32 accumulate, K-major A and B, N >> 3 at bit 17, M >> 4 at bit 24
    prm.idesc |= (1u << 4) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
    const long long total = (long long)prm.tiles_r * prm.tiles_s * prm.stacks;
    const int grid = (int)(total < sm_count ? total : sm_count);
    return launch_pdl(kernel, dim3(grid), dim3(NUM_THREADS), C::SMEM_BYTES, stream, mp, mq, prm);
}

// The output as the epilogue's TMA stores see it: [stacks][R][columns up to the end of this launch's window].
bool make_out_maps(OutMaps *om, const UmmaParams &prm, rt_dtype dt) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    if (prm.out_ld % 8 != 0 || prm.out_col % 8 != 0 || prm.out_batch_stride % 8 != 0) return false;
    for (int d = 0; d < prm.n_out; d++) {
        if (reinterpret_cast<uintptr_t>(prm.outs[d]) % 16 != 0) return false;
        cuuint64_t dims[3] = {(cuuint64_t)(prm.out_col + prm.s_out), (cuuint64_t)prm.R, (cuuint64_t)prm.stacks};
        cuuint64_t strides[2] = {(cuuint64_t)prm.out_ld * 2, (cuuint64_t)prm.out_batch_stride * 2};
        cuuint32_t box[3] = {64, 32, 1};
        if (encode_cached(&om->m[d], dt == RT_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, prm.outs[d], dims,
                          strides, box, CU_TENSOR_MAP_L2_PROMOTION_NONE) != CUDA_SUCCESS)
            return false;
    }
    return true;
}

template <typename OutT>
cudaError_t launch_pair(const CUtensorMap &mp, const CUtensorMap &mq, UmmaParams prm, int sm_count, cudaStream_t stream, rt_dtype out_dt) {
    static SmemAttr smem_attr;
    auto kernel = gemm_umma_pair_kernel<OutT>;
    {
        cudaError_t e = smem_attr.ensure(kernel, P2_SMEM_BYTES);
        if (e != cudaSuccess) return e;
    }
    prm.tiles_r = (prm.R + 2 * BM - 1) / (2 * BM);
    prm.group_r = grouped_order(prm) ? TILE_GROUP_ROWS / (2 * BM) : prm.tiles_r;
    prm.tiles_s = (prm.S + P2_BN - 1) / P2_BN;
    // instruction descriptor: f32 accumulate, K-major A and B, N = 256, M = 256 over the two CTAs
    prm.idesc |= (1u << 4) | ((uint32_t)(P2_BN >> 3) << 17) | ((uint32_t)((2 * BM) >> 4) << 24);
    const long long total = (long long)prm.tiles_r * prm.tiles_s * prm.stacks;
    const int pairs = (int)std::min<long long>(total, sm_count / 2);
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3(2 * pairs);
    lc.blockDim = dim3(NUM_THREADS);
    lc.dynamicSmemBytes = P2_SMEM_BYTES;
    lc.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = 2;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    lc.attrs = attr;
    lc.numAttrs = 2;
    // RT_GEMM_TMA_STORE=0 keeps the epilogue on the SM's own stores (A/B timing)
    static const bool tma_store_wanted = [] { const char *v = getenv("RT_GEMM_TMA_STORE"); return !(v && v[0] == '0'); }();
    OutMaps om;
    memset(&om, 0, sizeof(om));
    prm.tma_store = tma_store_wanted && make_out_maps(&om, prm, out_dt) ? 1 : 0;
    return cudaLaunchKernelEx(&lc, kernel, mp, mq, om, prm);
}

} // namespace

bool umma_gemm_supported(long long K) { return K >= 8 && K % 8 == 0 && encode_fn() != nullptr; }

int umma_pick_bn(long long R, long long S, long long stacks, int sm_count) {
    // 128 x 256 tiles need 96 bytes of operands per MMA cycle, 128 x 128 tiles 128: the narrow tile is bound by
    // the copies into shared memory, so the wide one is taken as soon as it fills half of the SMs
    const long long t256 = ((R + BM - 1) / BM) * ((S + 255) / 256) * stacks;
    return 2 * t256 >= sm_count ? 256 : 128;
}

// P: [p_stack][R][K] of p_dt, Q: [q_stack][S][K] of q_dt (f16 or bf16 each); out [stacks][R][S] of out_dt.
cudaError_t launch_gemm_umma(const void *P, rt_dtype p_dt, const void *Q, rt_dtype q_dt, void *out, rt_dtype out_dt,
                             int R, int S, int K, int stacks, int p_stack, int q_stack, const void *bias, int bias_dt,
                             int bias_mode, int epilogue, int bn, int sm_count, cudaStream_t stream, const UmmaScatter *scatter,
                             const float *p_scale, const float *q_scale) {
    // kind::f16 wants one format for both operands: an instruction descriptor that mixes f16 and
    // bf16 is an illegal instruction on sm_100a
    if (p_dt != q_dt || (p_dt != RT_F16 && p_dt != RT_BF16)) return cudaErrorInvalidValue;
    const bool pair = epilogue == RT_EPILOGUE_SILU_MUL;
    if (pair && (S % 2 != 0 || bias_mode == BIAS_PER_M || (scatter && scatter->n_out > 0))) return cudaErrorInvalidValue;
    CUtensorMap mp, mq;
    if (!make_map(&mp, P, p_dt, K, R, p_stack, BM)) return cudaErrorInvalidValue;
    if (bn == UMMA_BN_PAIR && pair) return cudaErrorInvalidValue; // the CTA-pair kernel has no gate/up fold
    if (!(pair ? make_pair_map(&mq, Q, q_dt, K, S / 2, q_stack, bn / 2)
               : make_map(&mq, Q, q_dt, K, S, q_stack, bn == UMMA_BN_PAIR ? P2_BN / 2 : bn)))
        return cudaErrorInvalidValue;
    UmmaParams prm{};
    prm.R = R; prm.S = S; prm.K = K;
    prm.pair = pair ? 1 : 0;
    prm.s_out = pair ? S / 2 : S;
    prm.stacks = stacks; prm.p_stack = p_stack; prm.q_stack = q_stack;
    prm.out = out;
    if (scatter && scatter->n_out > 0) {
        if (scatter->n_out > RT_MAX_PEERS) return cudaErrorInvalidValue;
        prm.n_out = scatter->n_out;
        // The destinations are written in an order that starts at this shard's own index (out_col / S for equal shards):
        // at any moment the GPUs of a group then store to different peers, instead of all to GPU 0, then all to GPU 1, ..
        const int first = S > 0 ? (int)((scatter->out_col / S) % scatter->n_out) : 0;
        for (int d = 0; d < scatter->n_out; d++) prm.outs[d] = scatter->outs[(first + d) % scatter->n_out];
        prm.out_ld = scatter->out_ld;
        prm.out_col = scatter->out_col;
        prm.out_batch_stride = (long long)R * scatter->out_ld;
    } else {
        prm.n_out = 1;
        prm.outs[0] = out;
        prm.out_ld = prm.s_out;
        prm.out_col = 0;
        prm.out_batch_stride = (long long)R * prm.s_out;
    }
    prm.bias = bias; prm.bias_dt = bias_dt; prm.bias_mode = bias_mode;
    prm.epilogue = epilogue;
    prm.p_scale = p_scale; prm.q_scale = q_scale;
    if (pair && q_scale) return cudaErrorInvalidValue; // the gate/up fold has the weights as Q
    if ((p_scale || q_scale) && out_dt != RT_BF16) return cudaErrorInvalidValue; // only those kernels hold the code
    prm.idesc = ((p_dt == RT_BF16 ? 1u : 0u) << 7) | ((q_dt == RT_BF16 ? 1u : 0u) << 10);
    if (bn == UMMA_BN_PAIR) {
        if (out_dt == RT_F16) return launch_pair<__half>(mp, mq, prm, sm_count, stream, out_dt);
        if (out_dt == RT_BF16) return launch_pair<__nv_bfloat16>(mp, mq, prm, sm_count, stream, out_dt);
        return cudaErrorInvalidValue;
    }
    if (out_dt == RT_F16)
        return bn == 256 ? launch_bn<256, __half>(mp, mq, prm, sm_count, stream) : launch_bn<128, __half>(mp, mq, prm, sm_count, stream);
    if (out_dt == RT_BF16)
        return bn == 256 ? launch_bn<256, __nv_bfloat16>(mp, mq, prm, sm_count, stream)
                         : launch_bn<128, __nv_bfloat16>(mp, mq, prm, sm_count, stream);
    return cudaErrorInvalidValue;
}

// Reads and clears the wait-expiry flag (0 = no kernel gave up a wait).
cudaError_t umma_take_error(int *site, cudaStream_t stream) {
    int zero = 0;
    cudaError_t e = cudaMemcpyFromSymbolAsync(site, g_umma_error, sizeof(int), 0, cudaMemcpyDeviceToHost, stream);
    if (e != cudaSuccess) return e;
    e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess) return e;
    if (*site != 0) e = cudaMemcpyToSymbolAsync(g_umma_error, &zero, sizeof(int), 0, cudaMemcpyHostToDevice, stream);
    return e;
}

} // namespace rt
