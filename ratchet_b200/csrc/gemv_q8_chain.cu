// A chain of Q8_0 GEMVs (one activation vector each) as ONE persistent cooperative kernel.
//
// Decode runs the reference's Executable::dispatch_operations (crates/ratchet-core/src/executable.rs:25-54)
// over a list of GEMV nodes (crates/ratchet-core/src/ops/gemv.rs:333-558) in which node l+1 reads what
// node l wrote.  Launched one kernel per node, every node pays the kernel boundary twice: HBM idles
// while the boundary, the conversion of the activations and the first fetches go by, and a CTA
// can only hold the part of its weights that fits beside its predecessor's.  Here the whole list is one
// launch of one CTA per SM:
//
//  * the producer warp streams the CTA's share of EVERY node's weights through one ring of TMA stages
//    that fills nearly all of shared memory (the share of a Phi-2 sized node fits whole), bounded only by
//    free slots: weights are constants, so it runs ahead into the next nodes while the current one
//    computes and while the CTAs meet, and HBM never waits for the dependency;
//  * nodes are separated by a grid barrier (one atomic counter; arrival after the node's outputs are
//    fenced, an acquire poll before the next node's activations are read), not by a launch;
//  * the arithmetic is that of the single-launch kernel (gemv_q8_umma.cu, shared code in umma_gemv.cuh):
//    int8 codes straight from shared memory into tcgen05.mma kind::i8 against block-floating int8 digits
//    of the activations, s32 sums in tensor memory, per-block rescale by four epilogue warps.  K slices of
//    fat weights meet in global memory: each slice's CTA stores its row sums and counts itself in, and the
//    one that arrives last adds the slices in rank order and writes the rows (thread-block clusters would
//    do this in shared memory, but clusters of four leave 16 of the 148 SMs without a CTA).  Results are
//    bit-identical to launching the nodes one by one;
//  * with the SM to itself a CTA owns all 512 tensor-memory columns: every block of a stage gets its own
//    16-column accumulator (no overlapping writes), so two warps can issue MMAs for alternate stages.
// Every wait is bounded; a wait that runs out records its site, raises the CTA's abort flag and the CTA
// leaves its loops, frees tensor memory and returns; the other CTAs run into their own limits.
#include <cuda.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "common.cuh"
#include "kernels.hpp"
#include "umma_gemv.cuh"

namespace rt {

__device__ int g_gemv_chain_error = 0;

namespace {

using namespace umma_gemv;

constexpr int N_ISSUE = 2;                               // MMA-issuing warps (stage g belongs to issuer g % N_ISSUE)
constexpr int THREADS = 64 + 128 + 32 * (N_ISSUE - 1);   // warp 0 producer, warp 1 issuer 0, warps 2-5 epilogue, warps 6.. issuers 1..
constexpr int STAGE_K = 256;                             // bytes of K per ring stage = 8 Q8_0 blocks
constexpr int TMEM_COLS = 512;
constexpr int TG_COLS = 128;                             // 8 blocks x 16 columns
constexpr int TGROUPS = TMEM_COLS / TG_COLS;
constexpr int MAX_KS = 3072;                             // bytes of K per CTA and node
constexpr size_t SMEM_LIMIT = 227 * 1024;

struct alignas(64) ChainNodeDev {
    CUtensorMap map_w; // codes  [M][K] u8, box 128 x rb, 128-byte swizzle
    CUtensorMap map_s; // scales [M][K/32] f16, box 8 x rb
    const void *rhs;
    void *out;
    const void *bias;
    int M, K;
    int rb, rb8, ks, nstages, split;
    int bias_mode, bias_dt, epilogue;
};

struct ChainParams {
    const ChainNodeDev *nodes;
    int n_nodes;
    int ring;            // stages in the ring
    int slot_bytes;      // codes of one stage: 2 sub-tiles of rb8_max x 128
    int scale_slot_bytes;
    int b_bytes;         // digit tiles (and the guard for MMA reads past a sub-tile's last row)
    int n_issue;         // MMA-issuing warps in use (<= N_ISSUE)
    unsigned long long *counter; // grid barrier: arrivals so far
    unsigned int *unit_count;    // [n_nodes][gridDim.x]: K slices of a unit that have stored their row sums
    float *partial;              // [max split][partial_ld]: row sums of the K slices of the node in flight
    int partial_ld;
};

__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, int site) {
    return mbar_wait_flag(bar, parity, abort_flag, site, &g_gemv_chain_error);
}

__global__ void __launch_bounds__(THREADS, 1) q8_gemv_chain_kernel(const ChainParams cp) {
    extern __shared__ uint8_t smem_raw[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *ring = smem;                                         // [ring][2 sub-tiles][rb8 x 128]
    uint8_t *b_tiles = ring + (size_t)cp.ring * cp.slot_bytes;    // [MAX_KS/128][8 rows x 128]
    uint8_t *scales_s = b_tiles + cp.b_bytes;                     // [ring][rb8 x 16]
    float *xs = reinterpret_cast<float *>(scales_s + (size_t)cp.ring * cp.scale_slot_bytes);
    uint64_t *bars = reinterpret_cast<uint64_t *>(xs + MAX_KS / 32);
    // bars: [0..R) full, [R..2R) empty, TGROUPS tmem_full, TGROUPS tmem_empty, digits ready
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * cp.ring + 2 * TGROUPS + 2);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    volatile unsigned int *arrived_before = reinterpret_cast<volatile unsigned int *>(tmem_slot + 2);
    const uint32_t bar_full = smem_u32(bars), bar_empty = smem_u32(bars + cp.ring);
    const uint32_t bar_tfull = smem_u32(bars + 2 * cp.ring), bar_tempty = smem_u32(bars + 2 * cp.ring + TGROUPS);
    const uint32_t bar_x = smem_u32(bars + 2 * cp.ring + 2 * TGROUPS);

    if (threadIdx.x == 0) {
        for (int s = 0; s < cp.ring; s++) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, 5); // the MMAs' commit + the four epilogue warps (they read the stage's scales)
        }
        for (int a = 0; a < TGROUPS; a++) {
            mbar_init(bar_tfull + 8 * a, 1);
            mbar_init(bar_tempty + 8 * a, 4);
        }
        mbar_init(bar_x, 4);
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

    if (warp == 0) {
        // ------------------------------------------------------------------ producer: all nodes, one ring
        if (lane == 0) {
            int slot = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int l = 0; l < cp.n_nodes && ok; l++) {
                const ChainNodeDev &nd = cp.nodes[l];
                const int unit = (int)blockIdx.x / nd.split, rank = (int)blockIdx.x % nd.split;
                const int row_begin = unit * nd.rb;
                if (row_begin >= nd.M) continue;
                const int k_begin = rank * nd.ks;
                const uint32_t tx = (uint32_t)nd.rb * (2 * 128 + 16);
                const int nstages = nd.nstages, rb8 = nd.rb8;
                const CUtensorMap *map_w = &nd.map_w, *map_s = &nd.map_s;
                // the maps live in global memory (written by the host before the launch): the tensor-map proxy
                // has to acquire them before this CTA's first copy through them
                asm volatile("fence.proxy.tensormap::generic.acquire.sys [%0], 128;" ::"l"(map_w) : "memory");
                asm volatile("fence.proxy.tensormap::generic.acquire.sys [%0], 128;" ::"l"(map_s) : "memory");
                for (int s = 0; s < nstages; s++) {
                    if (!mbar_wait(bar_empty + 8 * slot, phase ^ 1, abort_flag, 1)) { ok = false; break; }
                    const uint32_t st = smem_u32(ring + (size_t)slot * cp.slot_bytes);
                    const uint32_t full = bar_full + 8 * slot;
                    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(full), "r"(tx) : "memory");
                    const int kb = k_begin + s * STAGE_K;
                    tma_load_2d(st, map_w, kb, row_begin, full);
                    tma_load_2d(st + rb8 * 128, map_w, kb + 128, row_begin, full);
                    tma_load_2d(smem_u32(scales_s + (size_t)slot * cp.scale_slot_bytes), map_s, kb / 32, row_begin, full);
                    if (++slot == cp.ring) { slot = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1 || warp >= 6) {
        // ------------------------------------------------------------------ MMA issuers
        const int issuer = warp == 1 ? 0 : warp - 5;
        if (lane == 0) {
            // instruction descriptor: s32 accumulate, signed 8-bit A and B, K-major, N = 16, M = 128
            const uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) | ((16u >> 3) << 17) | ((128u >> 4) << 24);
            const uint64_t a_desc_ring = umma_desc_sw128(smem_u32(ring), 1024), b_desc_base = umma_desc_sw128(smem_u32(b_tiles), 0);
            int slot = 0, tg = 0, turn = 0;
            uint32_t phase = 0, tphase = 0, xphase = 0;
            bool ok = true;
            for (int l = 0; l < cp.n_nodes && ok; l++) {
                const ChainNodeDev &nd = cp.nodes[l];
                const int unit = (int)blockIdx.x / nd.split;
                if (unit * nd.rb >= nd.M) continue;
                // this node's digits are in place (one phase of bar_x per node that has rows here)
                if (!mbar_wait(bar_x, xphase, abort_flag, 2)) break;
                xphase ^= 1;
                const int rb8 = nd.rb8, nstages = nd.nstages;
                for (int s = 0; s < nstages; s++) {
                    if (turn == issuer) {
                        if (!mbar_wait(bar_tempty + 8 * tg, tphase ^ 1, abort_flag, 3)) { ok = false; break; }
                        if (!mbar_wait(bar_full + 8 * slot, phase, abort_flag, 4)) { ok = false; break; }
                        tc_fence_after();
                        const uint64_t a_desc = a_desc_ring + (uint64_t)((uint32_t)(slot * cp.slot_bytes) >> 4);
                        const uint64_t b_desc = b_desc_base + (uint64_t)(s * 2 * (1024 >> 4));
                        const uint32_t d0 = tmem_base + tg * TG_COLS;
#pragma unroll
                        for (int kk = 0; kk < 2; kk++) {
                            const uint64_t ak = a_desc + (uint64_t)((uint32_t)(kk * rb8 * 128) >> 4), bk = b_desc + (uint64_t)(kk * (1024 >> 4));
                            // block jj of the stage owns columns [16 jj, 16 jj + 16): its two sums (the hi and lo digit
                            // rows of B) and fourteen columns nobody reads
#pragma unroll
                            for (int j = 0; j < 4; j++) umma_i8(d0 + (kk * 4 + j) * 16, ak + 2 * j, bk + 2 * j, idesc);
                        }
                        umma_commit(bar_empty + 8 * slot);
                        umma_commit(bar_tfull + 8 * tg);
                    }
                    if (++turn == cp.n_issue) turn = 0;
                    if (++slot == cp.ring) { slot = 0; phase ^= 1; }
                    if (++tg == TGROUPS) { tg = 0; tphase ^= 1; }
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ digits, epilogue, grid barrier (warps 2..5)
        const int q = warp & 3;          // tensor-memory lane quarter of this warp
        const int et = threadIdx.x - 64; // 0..127
        const int row_local = q * 32 + lane;
        // rows 2..7 of every digit tile stay zero for the whole kernel, rows 0 and 1 receive each node's digits
        for (int i = et; i < cp.b_bytes / 16; i += 128) reinterpret_cast<uint4 *>(b_tiles)[i] = make_uint4(0u, 0u, 0u, 0u);
        asm volatile("bar.sync 1, 128;" ::: "memory");
        int slot = 0, tg = 0;
        uint32_t phase = 0, tphase = 0;
        bool ok = true;
        for (int l = 0; l < cp.n_nodes && ok; l++) {
            const ChainNodeDev &nd = cp.nodes[l];
            const int split = nd.split, unit = (int)blockIdx.x / split, rank = (int)blockIdx.x % split;
            const int row_begin = unit * nd.rb;
            const bool has_rows = row_begin < nd.M;
            if (l > 0) {
                // node l-1 is complete on every CTA: (l) * gridDim.x arrivals
                if (et == 0) {
                    const unsigned long long target = (unsigned long long)l * gridDim.x;
                    const unsigned long long t0 = wait_clock();
                    while (true) {
                        unsigned long long v;
                        asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(cp.counter) : "memory");
                        if (v >= target) break;
                        if (*abort_flag) break;
                        if (wait_clock() - t0 > WAIT_LIMIT_CYCLES) {
                            *abort_flag = 1;
                            atomicCAS(&g_gemv_chain_error, 0, 8);
                            break;
                        }
                    }
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (*abort_flag) break;
            }
            if (has_rows) {
                const int ks = nd.ks, nstages = nd.nstages, scale_row = min(row_local, nd.rb8 - 1) * 16;
                const int k_begin = rank * ks;
                const int rows_here = min(nd.rb, nd.M - row_begin);
                {
                    // another SM wrote these activations during this launch: read them from L2
                    const __half *x = (const __half *)nd.rhs + k_begin;
                    const int sub = et & 3; // 4 threads per block of 32 elements, 8 elements each
                    constexpr int MAX_IT = MAX_KS / 32 / 32;
                    uint4 pre[MAX_IT];
#pragma unroll
                    for (int it = 0; it < MAX_IT; it++) { // all loads first: one L2 round trip, not one per iteration
                        const int blk = (et >> 2) + it * 32;
                        pre[it] = blk < ks / 32 ? __ldcg(reinterpret_cast<const uint4 *>(x + blk * 32 + sub * 8)) : make_uint4(0u, 0u, 0u, 0u);
                    }
#pragma unroll
                    for (int it = 0; it < MAX_IT; it++) {
                        const int blk = (et >> 2) + it * 32;
                        if (blk >= ks / 32) break;
                        digits_of_quarter_block(pre[it], blk, sub, b_tiles, xs);
                    }
                }
                // the MMAs read the tiles through the async proxy
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                asm volatile("bar.sync 1, 128;" ::: "memory"); // xs visible to all epilogue warps
                if (lane == 0) mbar_arrive(bar_x);

                float acc = 0.f;
                for (int s = 0; s < nstages; s++) {
                    if (!mbar_wait(bar_full + 8 * slot, phase, abort_flag, 5)) { ok = false; break; }
                    const uint4 sc = *reinterpret_cast<const uint4 *>(scales_s + (size_t)slot * cp.scale_slot_bytes + scale_row);
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar_empty + 8 * slot);
                    if (!mbar_wait(bar_tfull + 8 * tg, tphase, abort_flag, 6)) { ok = false; break; }
                    tc_fence_after();
                    int hi[8], lo[8];
                    const uint32_t t0 = tmem_base + tg * TG_COLS + ((uint32_t)(q * 32) << 16);
#pragma unroll
                    for (int j = 0; j < 8; j++) tmem_ld2_nowait(t0 + j * 16, hi[j], lo[j]);
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
                        acc = add_block(acc, d, xsv[j], hi[j], lo[j]);
                    }
                    if (++slot == cp.ring) { slot = 0; phase ^= 1; }
                    if (++tg == TGROUPS) { tg = 0; tphase ^= 1; }
                }
                if (!ok) break;
                bool writes_rows = true;
                if (split > 1) {
                    // K slices meet: store this slice's row sums, count it in; the slice that arrives last adds all
                    // of them in rank order (the order of the single-launch kernel) and writes the rows.
                    if (row_local < rows_here) cp.partial[(size_t)rank * cp.partial_ld + row_begin + row_local] = acc;
                    __threadfence();
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    if (et == 0) *arrived_before = atomicAdd(cp.unit_count + (size_t)l * gridDim.x + unit, 1u);
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    writes_rows = *arrived_before == (unsigned int)(split - 1);
                    if (writes_rows && row_local < rows_here) {
                        __threadfence();
                        const float *pr = cp.partial + row_begin + row_local;
                        acc = __ldcg(pr);
                        for (int r = 1; r < split; r++) acc += __ldcg(pr + (size_t)r * cp.partial_ld);
                    }
                }
                if (writes_rows && row_local < rows_here) { // this thread holds the sum of tensor-memory lane row_local
                    const int row = row_begin + row_local;
                    const bool has_bias = nd.bias_mode != BIAS_NONE;
                    float bias = 0.f;
                    if (has_bias) bias = load_bias(nd.bias, nd.bias_dt, nd.bias_mode == BIAS_PER_M ? row : 0);
                    ((__half *)nd.out)[row] = epilogue_value<__half>(acc, has_bias, bias, nd.epilogue);
                }
            }
            if (l + 1 < cp.n_nodes) {
                // publish: this CTA's part of node l is in memory (and its reads of node l's inputs are over)
                __threadfence();
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (et == 0) atomicAdd(cp.counter, 1ull);
            }
        }
    }

    // ---------------------------------------------------------------------- teardown
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

int split_for(int K) {
    int split = 1;
    while (split < 8 && (K / split > MAX_KS || (K / split) % STAGE_K != 0)) split *= 2;
    if (K % (split * STAGE_K) != 0 || K / split > MAX_KS) return 0;
    return split;
}

size_t smem_for(int ring, int slot_bytes, int scale_slot_bytes, int b_bytes) {
    return 1024 + (size_t)ring * (slot_bytes + scale_slot_bytes) + b_bytes + (size_t)(MAX_KS / 32) * 4 +
           (size_t)(2 * ring + 2 * TGROUPS + 2) * 8 + 64;
}

} // namespace

struct GemvChain {
    int device = 0;
    ChainParams cp{};
    ChainNodeDev *d_nodes = nullptr;
    unsigned char *d_counters = nullptr; // grid barrier counter (8 bytes), then the per-unit slice counts
    size_t counters_bytes = 0;
    float *d_partial = nullptr;
    int grid = 0;
    size_t smem = 0;
    std::string name;
};

const char *gemv_chain_name(const GemvChain *c) { return c ? c->name.c_str() : ""; }

void gemv_chain_destroy(GemvChain *c) {
    if (!c) return;
    cudaSetDevice(c->device);
    if (c->d_nodes) cudaFree(c->d_nodes);
    if (c->d_counters) cudaFree(c->d_counters);
    if (c->d_partial) cudaFree(c->d_partial);
    delete c;
}

// Builds the chain for `nodes` (each a Q8_0H [M][K] x f16 [K] GEMV with constant weights).  Returns
// cudaSuccess with *out == nullptr and a reason in *why when the list is not one this kernel takes.
cudaError_t gemv_chain_create(const std::vector<MatmulParams> &nodes, int device, int sm_count, GemvChain **out, std::string *why) {
    *out = nullptr;
    EncodeTiledFn encode = encode_tiled_fn();
    if (!encode) { *why = "no cuTensorMapEncodeTiled"; return cudaSuccess; }
    if (nodes.size() < 2) { *why = "fewer than two nodes"; return cudaSuccess; }
    std::vector<int> splits;
    int max_split = 1, partial_ld = 0;
    for (const MatmulParams &p : nodes) {
        const int s = p.K >= STAGE_K ? split_for(p.K) : 0;
        if (s == 0) { *why = "K is not a multiple of 256 per slice"; return cudaSuccess; }
        splits.push_back(s);
        if (s > max_split) max_split = s;
        if (s > 1 && p.M > partial_ld) partial_ld = p.M;
    }

    cudaError_t e = cudaSetDevice(device);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(q8_gemv_chain_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_LIMIT);
    if (e != cudaSuccess) return e;
    // how many CTAs can be resident at once decides the grid (a cooperative launch takes no more)
    int grid = 0;
    {
        int per_sm = 0;
        e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, q8_gemv_chain_kernel, THREADS, SMEM_LIMIT);
        if (e != cudaSuccess) { cudaGetLastError(); *why = std::string("occupancy query: ") + cudaGetErrorString(e); return cudaSuccess; }
        grid = per_sm >= 1 ? sm_count : 0;
    }
    if (grid < 1) { *why = "no resident CTA"; return cudaSuccess; }

    std::vector<ChainNodeDev> host(nodes.size());
    int rb8_max = 8;
    for (size_t i = 0; i < nodes.size(); i++) {
        const MatmulParams &p = nodes[i];
        ChainNodeDev &nd = host[i];
        std::memset(&nd, 0, sizeof(nd));
        const int units = grid / splits[i];
        const int rb = (p.M + units - 1) / units;
        if (rb > 128 || rb < 8) { *why = "rows per CTA outside 8..128"; return cudaSuccess; }
        nd.M = p.M; nd.K = p.K; nd.rb = rb; nd.rb8 = (rb + 7) & ~7; nd.split = splits[i];
        nd.ks = p.K / splits[i]; nd.nstages = nd.ks / STAGE_K;
        nd.rhs = p.rhs; nd.out = p.out; nd.bias = p.bias;
        nd.bias_mode = p.bias_mode; nd.bias_dt = p.bias_dt; nd.epilogue = p.epilogue;
        if (nd.rb8 > rb8_max) rb8_max = nd.rb8;
        if ((reinterpret_cast<uintptr_t>(p.lhs) | reinterpret_cast<uintptr_t>(p.rhs) | reinterpret_cast<uintptr_t>(p.lhs_scales)) % 16 != 0) {
            *why = "operands not 16-byte aligned";
            return cudaSuccess;
        }
        {
            cuuint64_t dims[2] = {(cuuint64_t)p.K, (cuuint64_t)p.M};
            cuuint64_t strides[1] = {(cuuint64_t)p.K};
            cuuint32_t box[2] = {128, (cuuint32_t)rb};
            cuuint32_t estr[2] = {1, 1};
            if (encode(&nd.map_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(p.lhs), dims, strides, box, estr,
                       CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                       CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) { *why = "tensor map (codes)"; return cudaSuccess; }
        }
        {
            cuuint64_t dims[2] = {(cuuint64_t)(p.K / 32), (cuuint64_t)p.M};
            cuuint64_t strides[1] = {(cuuint64_t)(p.K / 32) * 2};
            cuuint32_t box[2] = {8, (cuuint32_t)rb};
            cuuint32_t estr[2] = {1, 1};
            if (encode(&nd.map_s, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void *>(p.lhs_scales), dims, strides, box, estr,
                       CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                       CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) { *why = "tensor map (scales)"; return cudaSuccess; }
        }
    }
    GemvChain *c = new GemvChain();
    c->device = device;
    c->grid = grid;
    ChainParams &cp = c->cp;
    cp.n_nodes = (int)nodes.size();
    {
        const char *v = getenv("RT_CHAIN_ISSUERS");
        cp.n_issue = v ? std::max(1, std::min(N_ISSUE, atoi(v))) : N_ISSUE;
    }
    cp.slot_bytes = 2 * rb8_max * 128;
    cp.scale_slot_bytes = rb8_max * 16;
    cp.b_bytes = (MAX_KS / 128) * 1024; // 24 KB >= the 128 - rb8 rows an MMA may read past the ring's last sub-tile
    int ring = 16;
    while (ring > 2 && smem_for(ring, cp.slot_bytes, cp.scale_slot_bytes, cp.b_bytes) > SMEM_LIMIT) ring--;
    if (smem_for(ring, cp.slot_bytes, cp.scale_slot_bytes, cp.b_bytes) > SMEM_LIMIT) {
        delete c;
        *why = "ring does not fit";
        return cudaSuccess;
    }
    cp.ring = ring;
    c->smem = smem_for(ring, cp.slot_bytes, cp.scale_slot_bytes, cp.b_bytes);
    c->counters_bytes = 8 + sizeof(unsigned int) * nodes.size() * (size_t)grid;
    partial_ld = (partial_ld + 31) & ~31;
    e = cudaMalloc(&c->d_nodes, host.size() * sizeof(ChainNodeDev));
    if (e == cudaSuccess) e = cudaMalloc(&c->d_counters, c->counters_bytes);
    if (e == cudaSuccess && partial_ld > 0) e = cudaMalloc(&c->d_partial, sizeof(float) * (size_t)max_split * partial_ld);
    if (e == cudaSuccess) e = cudaMemcpy(c->d_nodes, host.data(), host.size() * sizeof(ChainNodeDev), cudaMemcpyHostToDevice);
    if (e != cudaSuccess) {
        gemv_chain_destroy(c);
        return e;
    }
    cp.nodes = c->d_nodes;
    cp.counter = reinterpret_cast<unsigned long long *>(c->d_counters);
    cp.unit_count = reinterpret_cast<unsigned int *>(c->d_counters + 8);
    cp.partial = c->d_partial;
    cp.partial_ld = partial_ld;
    c->name = "q8_gemv_chain_h_nodes" + std::to_string(cp.n_nodes) + "_grid" + std::to_string(grid) + "_maxsplit" + std::to_string(max_split) +
              "_ring" + std::to_string(ring);
    *out = c;
    return cudaSuccess;
}

// One dispatch of the whole chain: the counters start from zero, then one cooperative launch.
cudaError_t gemv_chain_launch(GemvChain *c, cudaStream_t stream) {
    cudaError_t e = cudaMemsetAsync(c->d_counters, 0, c->counters_bytes, stream);
    if (e != cudaSuccess) return e;
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3(c->grid);
    lc.blockDim = dim3(THREADS);
    lc.dynamicSmemBytes = c->smem;
    lc.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative; // all CTAs resident at once: they wait for one another
    attr[0].val.cooperative = 1;
    lc.attrs = attr;
    lc.numAttrs = 1;
    return cudaLaunchKernelEx(&lc, q8_gemv_chain_kernel, c->cp);
}

cudaError_t gemv_chain_take_error(int *site, cudaStream_t stream) {
    int zero = 0;
    cudaError_t e = cudaMemcpyFromSymbolAsync(site, g_gemv_chain_error, sizeof(int), 0, cudaMemcpyDeviceToHost, stream);
    if (e != cudaSuccess) return e;
    e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess) return e;
    if (*site != 0) e = cudaMemcpyToSymbolAsync(g_gemv_chain_error, &zero, sizeof(int), 0, cudaMemcpyHostToDevice, stream);
    return e;
}

} // namespace rt
