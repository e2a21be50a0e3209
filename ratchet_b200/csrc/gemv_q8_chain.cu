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
//  * nodes are separated neither by a launch nor by a barrier: every output row is also written as one
//    32-bit word {f16 value, 16-bit tag of this dispatch} into an exchange buffer of its node, and the
//    next node's CTAs poll exactly the words they convert until the tags are this dispatch's.  A word
//    is its own flag, so no fence and no counter is on the path (a fence costs about 1.5 us while the
//    SM's weight stream is in flight);
//  * the arithmetic is that of the single-launch kernel (gemv_q8_umma.cu, shared code in umma_gemv.cuh):
//    int8 codes straight from shared memory into tcgen05.mma kind::i8 against block-floating int8 digits
//    of the activations, s32 sums in tensor memory, per-block rescale by eight epilogue warps.  K slices of
//    fat weights meet in global memory the same way: slices 1.. store {f32 sum, 32-bit tag} words, slice 0
//    polls them, adds in rank order and writes the rows (thread-block clusters would do this in shared
//    memory, but clusters of four leave 16 of the 148 SMs without a CTA).  The products are those of
//    launching the nodes one by one; the f32 sums are taken in another order;
//  * with the SM to itself a CTA owns all 512 tensor-memory columns: four regions of 128, one per stage in
//    flight, so no stage of a node waits for the epilogue of another.  Up to four warps issue a stage's MMAs,
//    tile by tile (a single thread issues a tcgen05.mma every 54 cycles; the pipe takes this shape every 41),
//    each with one tcgen05.commit per stage onto one barrier that says both "sums ready" and "slot free";
//  * a node's MMAs take 128 consecutive rows of the stage's row stream, whichever 128-byte chunks of K they
//    belong to (see ChainNodeDev): every MMA is full, 48 per Phi-2 node instead of 80;
//  * the producer spaces its copies (cp.pace): bursts of copy writes and the MMAs' operand reads would meet
//    at the shared-memory port; it sleeps in between, because it shares a scheduler with epilogue warps.
// The dispatch is only legal as a cooperative launch: CTAs wait for one another, so all must be resident.
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

constexpr int N_ISSUE = 4;                               // MMA-issuing warps at most: tile t of a stage belongs to issuer t % n_issue
constexpr int THREADS = 64 + 256 + 32 * (N_ISSUE - 1);   // warp 0 producer, warp 1 issuer 0, warps 2-9 epilogue, warps 10.. issuers 1..
constexpr int CHUNK_K = 128;                             // bytes of K per sub-tile row (one swizzle row) = 4 Q8_0 blocks
constexpr int MAX_S = 8;                                 // sub-tiles (chunks) per ring stage
constexpr int MAX_TILES = 3;                             // 128-row MMA tiles per stage
constexpr int TMEM_COLS = 512;
constexpr int TG_COLS = 128;                             // columns of one stage's accumulators (see col_stride)
constexpr int TGROUPS = TMEM_COLS / TG_COLS;
constexpr int MAX_KS = 3072;                             // bytes of K per CTA and node
constexpr int GUARD_BYTES = 16384;                       // an MMA tile may read up to 128 rows past its stage
constexpr size_t SMEM_LIMIT = 227 * 1024;

// How a node's weights sit in a ring stage, and how the MMAs tile them.
//
// A stage holds S consecutive chunks of K (128 bytes each) for the CTA's rb rows: S sub-tiles of rb8
// rows x 128 bytes, one after the other, i.e. a stream of S * rb8 rows of 128 bytes.  An MMA takes 128
// consecutive rows of that stream as its A operand, whatever sub-tiles they belong to: tile t covers
// stream rows [128 t, 128 t + 128), which are rows of chunks c0[t] .. c1[t].  Its B operand holds, for
// every one of those chunks d = c - c0[t], the chunk's hi digits in row 2d and its lo digits in row
// 2d + 1, so accumulator columns (2d, 2d + 1) of the lanes that hold chunk c's rows are that chunk's
// sums; the other columns of those lanes pair weights with another chunk's activations and are never
// read.  With rb = 70 a 128-row MMA is full instead of 55 % full: 48 MMAs per node instead of 80.
struct alignas(16) ChainNodeInfo { // 128 bytes: what the warps other than the producer need of a node
    const void *rhs;
    void *out;
    const void *bias;
    int M, K;
    int rb, rb8, ks, split;
    int S, nstages, tiles;       // chunks per stage, stages per node, MMA tiles per stage
    int b_tile_bytes;            // 1024 (8 digit rows: at most 4 chunks per tile) or 2048 (16 rows)
    int c0[4], c1[4];
    int bias_mode, bias_dt, epilogue;
    int inv_S_q16;               // ceil(65536 / S): chunk / S without a division
    int col_stride;              // tensor-memory columns between two MMAs' accumulators: 8 or 16
    int x_off;                   // this node's output words in the exchange buffer (32-bit words)
    int p_off;                   // this node's K-slice sums in the slice buffer (64-bit words), rank-major, ld = M
    int pad[1];
};
static_assert(sizeof(ChainNodeInfo) == 128, "ChainNodeInfo is copied as 32 words");

struct alignas(64) ChainNodeDev : ChainNodeInfo {
    CUtensorMap map_w; // codes  [M][K] u8, box 128 x rb, 128-byte swizzle
    CUtensorMap map_s; // scales [M][K/32] f16, box (ks/32) x rb
    const void *lhs;   // the same tensors as plain pointers: only the path for NaN / infinite activations reads them
    const void *lhs_scales;
};

struct ChainParams {
    const ChainNodeDev *nodes;
    int n_nodes;
    int ring;            // stages in the ring
    int slot_bytes;      // codes of one stage (the largest S * rb8 * 128 of the chain)
    int b_bytes;         // digit tiles, and the guard behind the ring
    int scale_buf_bytes; // one node's scales: rb8 rows of ks/32 f16 (two buffers)
    int n_issue;         // MMA-issuing warps in use (<= N_ISSUE)
    unsigned int *xbuf;          // every node's output rows as {f16 value, 16-bit tag} words
    unsigned long long *pbuf;    // K-sliced nodes: the slices' row sums as {f32 sum, 32-bit tag} words
    unsigned int tag;            // this dispatch's tag: 1..65535, never the previous dispatch's
    unsigned int publish_tag;    // the tag written with the rows: `tag`, except under the bounded-wait test hook
    unsigned long long poll_limit; // cycles the readers wait for rows and K-slice sums
    int pace;            // least number of cycles between two chunk copies of the producer (0: none)
    int skip_tempty;     // no node has more stages than tensor-memory regions: a region is only reused by a later node
};

__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, int site) {
    return mbar_wait_flag(bar, parity, abort_flag, site, &g_gemv_chain_error);
}

__global__ void __launch_bounds__(THREADS, 1) q8_gemv_chain_kernel(const ChainParams cp) {
    extern __shared__ uint8_t smem_raw[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *ring = smem;                                         // [ring][S sub-tiles][rb8 x 128]
    uint8_t *b_tiles = ring + (size_t)cp.ring * cp.slot_bytes;    // [nstages][tiles][8 or 16 rows x 128]
    uint8_t *scales_s = b_tiles + cp.b_bytes;                     // [2][rb8][ks/32] f16
    float *xs = reinterpret_cast<float *>(scales_s + 2 * (size_t)cp.scale_buf_bytes);
    float *part = xs + MAX_KS / 32;                               // [2 block pairs][MAX_TILES x 128 stream rows]: row sums
    ChainNodeInfo *info = reinterpret_cast<ChainNodeInfo *>(part + 2 * MAX_TILES * 128); // [2]: this node's and the next one's
    uint64_t *bars = reinterpret_cast<uint64_t *>(info + 2);
    // bars: [0..R) full, [R..2R) done (the stage's MMAs are complete: its sums are in tensor memory AND its slot is
    // free - one tcgen05.commit per stage, a commit costs the tensor pipe about as much as an MMA), TGROUPS
    // unused, TGROUPS tmem_empty, digits ready, 2 scales full, 2 scales empty
    const int n_bars = 2 * cp.ring + 2 * TGROUPS + 1 + 4;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + n_bars);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    unsigned int *badmask = tmem_slot + 2; // [2][4]: blocks of the K slice with a NaN or an infinity, by node parity; then [2]: any
    const uint32_t bar_full = smem_u32(bars), bar_done = smem_u32(bars + cp.ring);
    const uint32_t bar_tempty = smem_u32(bars + 2 * cp.ring + TGROUPS);
    const uint32_t bar_x = smem_u32(bars + 2 * cp.ring + 2 * TGROUPS);
    const uint32_t bar_sfull = bar_x + 8, bar_sempty = bar_x + 24;

    if (threadIdx.x == 0) {
        for (int s = 0; s < cp.ring; s++) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_done + 8 * s, cp.n_issue); // one commit per issuer
        }
        for (int a = 0; a < TGROUPS; a++) {
            mbar_init(bar_tempty + 8 * a, 8);
        }
        mbar_init(bar_x, 8);
        for (int a = 0; a < 2; a++) {
            mbar_init(bar_sfull + 8 * a, 1);
            mbar_init(bar_sempty + 8 * a, 8);
        }
        *abort_flag = 0;
        for (int i = 0; i < 12; i++) badmask[i] = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "n"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (warp == 2) reinterpret_cast<int *>(info)[lane] = reinterpret_cast<const int *>(static_cast<const ChainNodeInfo *>(cp.nodes))[lane];
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------------ producer: all nodes, one ring
        if (lane == 0) {
            int slot = 0, sbuf = 0;
            uint32_t phase = 0, sphase = 0;
            long long last_copy = clock64();
            bool ok = true;
            for (int l = 0; l < cp.n_nodes && ok; l++) {
                const ChainNodeDev &nd = cp.nodes[l];
                const int unit = (int)blockIdx.x / nd.split, rank = (int)blockIdx.x % nd.split;
                const int row_begin = unit * nd.rb;
                if (row_begin >= nd.M) continue;
                const int k_begin = rank * nd.ks;
                const int nstages = nd.nstages, rb8 = nd.rb8, S = nd.S;
                const CUtensorMap *map_w = &nd.map_w, *map_s = &nd.map_s;
                // the maps live in global memory (written by the host before the launch): the tensor-map proxy
                // has to acquire them before this CTA's first copy through them
                asm volatile("fence.proxy.tensormap::generic.acquire.sys [%0], 128;" ::"l"(map_w) : "memory");
                asm volatile("fence.proxy.tensormap::generic.acquire.sys [%0], 128;" ::"l"(map_s) : "memory");
                // the node's scales: one copy, into the buffer the node before the previous one has left
                if (!mbar_wait(bar_sempty + 8 * sbuf, sphase ^ 1, abort_flag, 9)) break;
                {
                    const uint32_t full = bar_sfull + 8 * sbuf;
                    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(full), "r"((uint32_t)(nd.rb * (nd.ks / 16))) : "memory");
                    tma_load_2d(smem_u32(scales_s + (size_t)sbuf * cp.scale_buf_bytes), map_s, k_begin / 32, row_begin, full);
                    if (++sbuf == 2) { sbuf = 0; sphase ^= 1; }
                }
                const uint32_t tx = (uint32_t)nd.rb * 128u * (uint32_t)S;
                for (int s = 0; s < nstages; s++) {
                    if (!mbar_wait(bar_done + 8 * slot, phase ^ 1, abort_flag, 1)) { ok = false; break; }
                    const uint32_t st = smem_u32(ring + (size_t)slot * cp.slot_bytes);
                    const uint32_t full = bar_full + 8 * slot;
                    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(full), "r"(tx) : "memory");
                    const int kb = k_begin + s * S * CHUNK_K;
                    for (int c = 0; c < S; c++) {
                        // Copies are spread over the node's time instead of bursting when the MMAs free the slots:
                        // MMA operand reads (about 100 bytes per cycle) and copy writes share the shared-memory port.
                        if (cp.pace > 0) {
                            while (clock64() - last_copy < cp.pace) __nanosleep(40); // no hot spin: the scheduler is shared with epilogue warps
                            last_copy = clock64();
                        }
                        tma_load_2d(st + c * rb8 * 128, map_w, kb + c * CHUNK_K, row_begin, full);
                    }
                    if (++slot == cp.ring) { slot = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1 || warp >= 10) {
        // ------------------------------------------------------------------ MMA issuers
        const int issuer = warp == 1 ? 0 : warp - 9;
        if (lane == 0 && issuer < cp.n_issue) {
            // instruction descriptor: s32 accumulate, signed 8-bit A and B, K-major, N = 16, M = 128
            const uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) | ((16u >> 3) << 17) | ((128u >> 4) << 24);
            const uint64_t a_desc_ring = umma_desc_sw128(smem_u32(ring), 1024);
            int slot = 0, tg = 0;
            uint32_t phase = 0, tphase = 0, xphase = 0;
            bool ok = true;
            for (int l = 0; l < cp.n_nodes && ok; l++) {
                // the epilogue warps put node l's description into shared memory while node l-1 ran
                const ChainNodeInfo &nd = info[l & 1];
                const int unit = (int)blockIdx.x / nd.split;
                const bool has_rows = unit * nd.rb < nd.M;
                const int nstages = nd.nstages, tiles = nd.tiles, btb = nd.b_tile_bytes, cstride = nd.col_stride;
                // one phase of bar_x per node: the node's digits are in place (and the next node's description)
                if (!mbar_wait(bar_x, xphase, abort_flag, 2)) break;
                xphase ^= 1;
                if (!has_rows) continue;
                // 16-row digit tiles are two 8-row groups 1024 bytes apart; 8-row tiles repeat their group (stride 0)
                const uint64_t b_desc_base = umma_desc_sw128(smem_u32(b_tiles), btb == 2048 ? 1024 : 0);
                const int tile_cols = 4 * cstride + (cstride == 8 ? 8 : 0);
                for (int s = 0; s < nstages; s++) {
                    // the region's previous sums have been read (when a node has no more stages than there are regions,
                    // the previous user was an earlier node, which the epilogue warps had left before this node's digits)
                    if (!cp.skip_tempty && !mbar_wait(bar_tempty + 8 * tg, tphase ^ 1, abort_flag, 3)) { ok = false; break; }
                    if (!mbar_wait(bar_full + 8 * slot, phase, abort_flag, 4)) { ok = false; break; }
                    tc_fence_after();
                    const uint64_t a_desc = a_desc_ring + (uint64_t)((uint32_t)(slot * cp.slot_bytes) >> 4);
                    const uint32_t d0 = tmem_base + tg * TG_COLS;
                    // The issuers share a stage tile by tile.  Tile t: 128 stream rows; block j of the chunks: 32 bytes
                    // further along K in both operands.  An MMA writes 16 columns, of which at most the first
                    // 2 * (chunks of the tile) are ever read; with a stride of 8 the next MMA of the same thread
                    // overwrites the unread upper half (the tensor pipe runs one thread's MMAs in issue order), and a
                    // gap of 8 columns behind a tile keeps another thread's tile out of reach.  So four stages fit into
                    // tensor memory and no stage of a node waits for the epilogue of another.
                    for (int t = issuer; t < tiles; t += cp.n_issue) {
                        const uint64_t at = a_desc + (uint64_t)(t * (128 * 128 >> 4));
                        const uint64_t bt = b_desc_base + (uint64_t)((uint32_t)((s * tiles + t) * btb) >> 4);
#pragma unroll
                        for (int j = 0; j < 4; j++) umma_i8(d0 + t * tile_cols + j * cstride, at + 2 * j, bt + 2 * j, idesc);
                    }
                    umma_commit(bar_done + 8 * slot); // this issuer's part of the stage (possibly nothing)
                    if (++slot == cp.ring) { slot = 0; phase ^= 1; }
                    if (++tg == TGROUPS) { tg = 0; tphase ^= 1; }
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ digits, epilogue, grid barrier (warps 2..9)
        // Two warps per tensor-memory lane quarter: the first takes blocks 0 and 1 of every chunk, the second
        // blocks 2 and 3.
        const int q = warp & 3;               // tensor-memory lane quarter of this warp
        const int half = (warp - 2) >> 2;     // which two blocks of every chunk
        const int et = threadIdx.x - 64;      // 0..255
        const int row_local = q * 32 + lane;  // this thread's tensor-memory lane
        int tg = 0, sbuf = 0, prev_x_off = 0, slot = 0;
        uint32_t sphase = 0, phase = 0;
        bool gave_up = false; // a wait of this warp ran out: it skips work but stays in step with the others up to the next barrier
        // The eight warps leave together, and only at a node's last barrier.  Before it ONE thread copies the CTA's
        // abort flag into one of two words (taken in turn, so that a thread still reading the last node's word is not
        // overtaken); after the barrier all threads test that copy, hence take the same decision.  A warp whose own wait
        // ran out (which raised the flag) skips its work, and every later wait of the CTA returns at once, until that
        // barrier shows the flag to everybody.
        volatile unsigned int *abort_seen = badmask + 10;
        int barriers = 0;
        auto sync_and_check = [&]() -> bool {
            if (et == 0) abort_seen[barriers & 1] = (unsigned int)*abort_flag;
            asm volatile("bar.sync 1, 256;" ::: "memory");
            return abort_seen[(barriers++) & 1] != 0u;
        };
        for (int l = 0; l < cp.n_nodes; l++) {
            const ChainNodeInfo &nd = info[l & 1];
            const int split = nd.split, unit = (int)blockIdx.x / split, rank = (int)blockIdx.x % split;
            const int row_begin = unit * nd.rb;
            const bool has_rows = row_begin < nd.M;
            // the next node's description, fetched while this node waits and computes (nobody reads the other
            // copy any more: node l-1 is over for every warp of this CTA once its sums were taken)
            int next_word = 0;
            // (asked for here, stored after the digits: a warp issues in order, and a store right behind the load would
            // hold up the whole warp, and with it the node's digits, until the word has come from memory)
            if (warp == 2 && l + 1 < cp.n_nodes) next_word = __ldcg(reinterpret_cast<const int *>(static_cast<const ChainNodeInfo *>(cp.nodes + l + 1)) + lane);
            if (!has_rows) {
                if (warp == 2 && l + 1 < cp.n_nodes) reinterpret_cast<int *>(info + ((l + 1) & 1))[lane] = next_word;
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_x);
            }
            if (has_rows) {
                const int ks = nd.ks, nstages = nd.nstages, rb8 = nd.rb8, S = nd.S, tiles = nd.tiles, btb = nd.b_tile_bytes, cstride = nd.col_stride;
                const int k_begin = rank * ks, inv_S = nd.inv_S_q16;
                const int rows_here = min(nd.rb, nd.M - row_begin);
                int c0[MAX_TILES], c1[MAX_TILES];
#pragma unroll
                for (int t = 0; t < MAX_TILES; t++) { c0[t] = nd.c0[t]; c1[t] = nd.c1[t]; }
                // where this thread's lane sits in the stage's row stream, tile by tile (worked out before the wait for the
                // activations: afterwards the issuing warps need the schedulers)
                int my_cl[MAX_TILES], my_row[MAX_TILES], my_k[MAX_TILES], col0[MAX_TILES];
                bool mine[MAX_TILES], warp_has[MAX_TILES];
                float acc[MAX_TILES];
                int sc_off[MAX_TILES], xs_off[MAX_TILES];
                const bool narrow = rb8 >= 32; // a warp's 32 lanes then belong to at most two chunks: two column pairs do
#pragma unroll
                for (int t = 0; t < MAX_TILES; t++) {
                    const int pos = 128 * t + row_local, pos_w = 128 * t + q * 32;
                    my_cl[t] = pos / rb8;
                    my_row[t] = pos - my_cl[t] * rb8;
                    warp_has[t] = t < tiles && pos_w < S * rb8;
                    mine[t] = t < tiles && pos < S * rb8 && my_row[t] < rows_here;
                    // first of the column pairs this warp loads: two pairs (narrow) or four, inside the MMA's cstride columns
                    const int d_first = min(pos_w / rb8 - c0[t], cstride / 2 - (narrow ? 2 : 4));
                    col0[t] = 2 * d_first;
                    my_k[t] = my_cl[t] - c0[t] - d_first;
                    acc[t] = 0.f;
                    // where this lane's scales and activation scales are (lanes outside the stage read some valid
                    // place: their sums are dropped)
                    const int cl_in = min(my_cl[t], S - 1), row_in = min(my_row[t], rb8 - 1);
                    sc_off[t] = row_in * (ks / 16) + (cl_in * 4 + half * 2) * 2;
                    xs_off[t] = cl_in * 4 + half * 2;
                }
                {
                    const int sub = et & 3; // 4 threads per block of 32 elements, 8 elements each
                    constexpr int MAX_IT = (MAX_KS / 32 + 63) / 64;
                    uint4 pre[MAX_IT];
                    if (l == 0) {
                        // the first node's activations were there before the launch
                        const __half *x = (const __half *)nd.rhs + k_begin;
#pragma unroll
                        for (int it = 0; it < MAX_IT; it++) {
                            const int blk = (et >> 2) + it * 64;
                            pre[it] = blk < ks / 32 ? __ldcg(reinterpret_cast<const uint4 *>(x + blk * 32 + sub * 8)) : make_uint4(0u, 0u, 0u, 0u);
                        }
                    } else {
                        // The previous node's rows arrive as {f16, tag} words from the CTAs that compute them: poll the
                        // eight words of each of this thread's quarter blocks until all carry this dispatch's tag.
                        const unsigned int *xw = cp.xbuf + prev_x_off + k_begin;
                        const unsigned long long t0 = wait_clock();
#pragma unroll
                        for (int it = 0; it < MAX_IT; it++) {
                            const int blk = (et >> 2) + it * 64;
                            pre[it] = make_uint4(0u, 0u, 0u, 0u);
                            if (blk >= ks / 32) continue;
                            const unsigned int *src = xw + blk * 32 + sub * 8;
                            while (true) {
                                uint4 a, b;
                                asm volatile("ld.relaxed.gpu.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(a.x), "=r"(a.y), "=r"(a.z), "=r"(a.w) : "l"(src) : "memory");
                                asm volatile("ld.relaxed.gpu.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(b.x), "=r"(b.y), "=r"(b.z), "=r"(b.w) : "l"(src + 4) : "memory");
                                const unsigned int want = cp.tag << 16;
                                const unsigned int miss = ((a.x ^ want) | (a.y ^ want) | (a.z ^ want) | (a.w ^ want) | (b.x ^ want) | (b.y ^ want) | (b.z ^ want) | (b.w ^ want)) >> 16;
                                if (miss == 0) {
                                    pre[it] = make_uint4((a.x & 0xFFFFu) | (a.y << 16), (a.z & 0xFFFFu) | (a.w << 16), (b.x & 0xFFFFu) | (b.y << 16), (b.z & 0xFFFFu) | (b.w << 16));
                                    break;
                                }
                                if (*abort_flag) break;
                                if (wait_clock() - t0 > cp.poll_limit) {
                                    *abort_flag = 1;
                                    atomicCAS(&g_gemv_chain_error, 0, 8);
                                    break;
                                }
                            }
                        }
                    }
#pragma unroll
                    for (int it = 0; it < MAX_IT; it++) {
                        const int blk = (et >> 2) + it * 64;
                        if (blk >= ks / 32) break;
                        uint2 hi8, lo8;
                        float inv;
                        bool nonfinite;
                        quantize_quarter_block(pre[it], hi8, lo8, inv, nonfinite);
                        if (sub == 0) {
                            xs[blk] = inv;
                            if (nonfinite) {
                                atomicOr(badmask + (l & 1) * 4 + (blk >> 5), 1u << (blk & 31));
                                badmask[8 + (l & 1)] = 1u;
                            }
                        }
                        // the chunk's digits go into every MMA tile that holds some of the chunk's rows
                        const int chunk = blk >> 2, stage = (chunk * inv_S) >> 16, cl = chunk - stage * S;
                        const int kpos = (blk & 3) * 32 + sub * 8;
#pragma unroll
                        for (int t = 0; t < MAX_TILES; t++) {
                            if (t < tiles && cl >= c0[t] && cl <= c1[t]) {
                                const int row = 2 * (cl - c0[t]);
                                uint8_t *tile = b_tiles + (size_t)(stage * tiles + t) * btb + (row >> 3) * 1024;
                                store_digits8(tile, row & 7, kpos, hi8);
                                store_digits8(tile, (row & 7) + 1, kpos, lo8);
                            }
                        }
                    }
                }
                // the MMAs read the tiles through the async proxy
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                asm volatile("bar.sync 1, 256;" ::: "memory"); // xs visible to all epilogue warps
                if (lane == 0) mbar_arrive(bar_x);
                if (warp == 2 && l + 1 < cp.n_nodes) reinterpret_cast<int *>(info + ((l + 1) & 1))[lane] = next_word;
                if (et < 4) badmask[((l + 1) & 1) * 4 + et] = 0u; // the next node's mask and flag (node l-1's readers are two barriers back)
                if (et == 4) badmask[8 + ((l + 1) & 1)] = 0u;

                const uint8_t *scales_n = scales_s + (size_t)sbuf * cp.scale_buf_bytes;
                const int srow = ks / 16; // bytes per row of the node's scales
                if (!mbar_wait(bar_sfull + 8 * sbuf, sphase, abort_flag, 10)) gave_up = true;
                for (int s = 0; s < nstages && !gave_up; s++) {
                    // the stage's weight scales and activation scales do not wait for the MMAs
                    __half2 d2[MAX_TILES];
                    float2 xv[MAX_TILES];
#pragma unroll
                    for (int t = 0; t < MAX_TILES; t++) {
                        d2[t] = *reinterpret_cast<const __half2 *>(scales_n + sc_off[t] + s * S * 8);
                        xv[t] = *reinterpret_cast<const float2 *>(xs + xs_off[t] + s * S * 4);
                    }
                    if (!mbar_wait(bar_done + 8 * slot, phase, abort_flag, 6)) { gave_up = true; break; }
                    tc_fence_after();
                    const uint32_t t0 = tmem_base + tg * TG_COLS + ((uint32_t)(q * 32) << 16) + half * 2 * cstride;
                    const int tile_cols = 4 * cstride + (cstride == 8 ? 8 : 0);
                    // all of the stage's loads first (one wait), then the arithmetic
                    int v[MAX_TILES][2][8]; // tiles the warp has no rows in stay unset: their sums are dropped
                    if (narrow) {
#pragma unroll
                        for (int t = 0; t < MAX_TILES; t++) {
                            if (!warp_has[t]) continue;
#pragma unroll
                            for (int j = 0; j < 2; j++) tmem_ld4_nowait(t0 + t * tile_cols + j * cstride + col0[t], v[t][j]);
                        }
                    } else {
#pragma unroll
                        for (int t = 0; t < MAX_TILES; t++) {
                            if (!warp_has[t]) continue;
#pragma unroll
                            for (int j = 0; j < 2; j++) tmem_ld8_nowait(t0 + t * tile_cols + j * cstride + col0[t], v[t][j]);
                        }
                    }
                    tmem_ld_wait();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar_tempty + 8 * tg); // the sums are in registers: the MMAs may reuse the columns
                    // no branches from here to the end of the stage: three independent chains the scheduler can interleave
#pragma unroll
                    for (int t = 0; t < MAX_TILES; t++) {
                        const int k = my_k[t];
#pragma unroll
                        for (int j = 0; j < 2; j++) {
                            int hi, lo;
                            if (narrow) {
                                hi = k == 0 ? v[t][j][0] : v[t][j][2];
                                lo = k == 0 ? v[t][j][1] : v[t][j][3];
                            } else {
                                hi = k == 0 ? v[t][j][0] : k == 1 ? v[t][j][2] : k == 2 ? v[t][j][4] : v[t][j][6];
                                lo = k == 0 ? v[t][j][1] : k == 1 ? v[t][j][3] : k == 2 ? v[t][j][5] : v[t][j][7];
                            }
                            const float d = j ? __high2float(d2[t]) : __low2float(d2[t]);
                            acc[t] = add_block(acc[t], d, j ? xv[t].y : xv[t].x, hi, lo);
                        }
                    }
                    if (++tg == TGROUPS) tg = 0;
                    if (++slot == cp.ring) { slot = 0; phase ^= 1; }
                }
                // the scales buffer is free for the node after the next one
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_sempty + 8 * sbuf);
                if (++sbuf == 2) { sbuf = 0; sphase ^= 1; }
                // a row's chunks and block pairs were summed by different threads: add them in a fixed order
#pragma unroll
                for (int t = 0; t < MAX_TILES; t++)
                    if (mine[t]) part[half * (MAX_TILES * 128) + 128 * t + row_local] = acc[t];
                asm volatile("bar.sync 1, 256;" ::: "memory");
                const bool my_rows = et < rows_here; // from here on thread et of the first four warps owns row et
                float sum = 0.f;
                if (my_rows) {
                    for (int c = 0; c < S; c++) sum += part[c * rb8 + et] + part[MAX_TILES * 128 + c * rb8 + et];
                    // blocks of the activations that hold NaN or infinities were left out above (zero digits): their
                    // products over this CTA's K slice, formed as the reference forms them
                    if (badmask[8 + (l & 1)]) {
                        const ChainNodeDev &dev = cp.nodes[l];
                        const int row = row_begin + et;
                        for (int w = 0; w < (ks / 32 + 31) / 32; w++) {
                            unsigned int m = badmask[(l & 1) * 4 + w];
                            while (m) {
                                const int blk = w * 32 + __ffs(m) - 1;
                                m &= m - 1;
                                const __half d = ((const __half *)dev.lhs_scales)[(size_t)row * (nd.K / 32) + k_begin / 32 + blk];
                                sum += nonfinite_block_products((const int8_t *)dev.lhs + (size_t)row * nd.K + k_begin + blk * 32, d,
                                                                l == 0 ? (const __half *)nd.rhs + k_begin + blk * 32 : nullptr,
                                                                l == 0 ? nullptr : cp.xbuf + prev_x_off + k_begin + blk * 32);
                            }
                        }
                    }
                }
                bool writes_rows = true;
                if (split > 1) {
                    // K slices meet: slices 1.. store {sum, tag} words, slice 0 polls them and adds in rank order
                    unsigned long long *pw = cp.pbuf + nd.p_off + row_begin + et;
                    if (rank != 0) {
                        writes_rows = false;
                        if (my_rows) {
                            const unsigned long long word = ((unsigned long long)cp.tag << 32) | __float_as_uint(sum);
                            asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(pw + (size_t)rank * nd.M), "l"(word) : "memory");
                        }
                    } else if (my_rows) {
                        const unsigned long long t0 = wait_clock();
                        unsigned long long w1 = 0, w2 = 0, w3 = 0;
                        if (split == 4) {
                            // the common case, all three slices asked for at once: one L2 round trip per try, not three
                            while (true) {
                                asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(w1) : "l"(pw + (size_t)1 * nd.M) : "memory");
                                asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(w2) : "l"(pw + (size_t)2 * nd.M) : "memory");
                                asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(w3) : "l"(pw + (size_t)3 * nd.M) : "memory");
                                if ((unsigned int)(w1 >> 32) == cp.tag && (unsigned int)(w2 >> 32) == cp.tag && (unsigned int)(w3 >> 32) == cp.tag) break;
                                if (*abort_flag) break;
                                if (wait_clock() - t0 > cp.poll_limit) {
                                    *abort_flag = 1;
                                    atomicCAS(&g_gemv_chain_error, 0, 7);
                                    break;
                                }
                            }
                            sum += __uint_as_float((unsigned int)w1); // rank order
                            sum += __uint_as_float((unsigned int)w2);
                            sum += __uint_as_float((unsigned int)w3);
                        } else {
                            for (int r = 1; r < split; r++) {
                                while (true) {
                                    unsigned long long word;
                                    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(word) : "l"(pw + (size_t)r * nd.M) : "memory");
                                    if ((unsigned int)(word >> 32) == cp.tag) {
                                        sum += __uint_as_float((unsigned int)word);
                                        break;
                                    }
                                    if (*abort_flag) break;
                                    if (wait_clock() - t0 > cp.poll_limit) {
                                        *abort_flag = 1;
                                        atomicCAS(&g_gemv_chain_error, 0, 7);
                                        break;
                                    }
                                }
                            }
                        }
                    }
                }
                if (writes_rows && my_rows) {
                    const int row = row_begin + et;
                    const bool has_bias = nd.bias_mode != BIAS_NONE;
                    float bias = 0.f;
                    if (has_bias) bias = load_bias(nd.bias, nd.bias_dt, nd.bias_mode == BIAS_PER_M ? row : 0);
                    const __half y = epilogue_value<__half>(sum, has_bias, bias, nd.epilogue);
                    // for the next node: value and tag in one word, so the word is its own "ready" flag
                    const unsigned int word = (cp.publish_tag << 16) | (unsigned int)__half_as_ushort(y);
                    asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(cp.xbuf + nd.x_off + row), "r"(word) : "memory");
                    ((__half *)nd.out)[row] = y; // for the caller, after the kernel
                }
            }
            prev_x_off = nd.x_off;
            // every warp is done with node l's description, digits scales and sums before the next node's are written
            if (sync_and_check()) break;
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
    while (split < 8 && (K / split > MAX_KS || (K / split) % 256 != 0)) split *= 2;
    if (K % (split * 256) != 0 || K / split > MAX_KS) return 0;
    return split;
}

// Chunks per stage: the divisor of the node's chunk count that needs the fewest MMAs (ties: the smaller
// stage), under the limits of the stage (64 KB), of tensor memory (MAX_TILES tiles) and of the digit tiles
// (at most 8 chunks per MMA tile).
bool pick_stage(ChainNodeDev &nd) {
    const int nchunks = nd.ks / CHUNK_K;
    int best_cost = 1 << 30;
    nd.S = 0;
    for (int S = 1; S <= MAX_S && S <= nchunks; S++) {
        if (nchunks % S != 0) continue;
        const int rows = S * nd.rb8, tiles = (rows + 127) / 128;
        if (tiles > MAX_TILES || rows * 128 > 64 * 1024) continue;
        // a stage's accumulators have TG_COLS columns: 8 per MMA (and 8 more behind the last) when no tile holds
        // rows of more than four chunks, else 16 per MMA
        int span = 1;
        for (int t = 0; t < tiles; t++) span = std::max(span, std::min(S - 1, (128 * t + 127) / nd.rb8) - (128 * t) / nd.rb8 + 1);
        if (span > 8) continue;
        if ((span <= 4 ? tiles * (4 * 8 + 8) : tiles * 4 * 16) > TG_COLS) continue;
        const int cost = (nchunks / S) * tiles;
        if (cost < best_cost) { best_cost = cost; nd.S = S; }
    }
    if (nd.S == 0) return false;
    nd.nstages = nchunks / nd.S;
    nd.inv_S_q16 = (65536 + nd.S - 1) / nd.S;
    nd.tiles = (nd.S * nd.rb8 + 127) / 128;
    int span = 1;
    for (int t = 0; t < MAX_TILES; t++) {
        nd.c0[t] = nd.c1[t] = 0;
        if (t >= nd.tiles) continue;
        nd.c0[t] = (128 * t) / nd.rb8;
        nd.c1[t] = std::min(nd.S - 1, (128 * t + 127) / nd.rb8);
        span = std::max(span, nd.c1[t] - nd.c0[t] + 1);
    }
    if (span > 8) return false;
    nd.b_tile_bytes = span > 4 ? 2048 : 1024;
    nd.col_stride = span > 4 ? 16 : 8;
    return true;
}

size_t smem_for(int ring, int slot_bytes, int b_bytes, int scale_buf_bytes) {
    return 1024 + (size_t)ring * slot_bytes + b_bytes + 2 * (size_t)scale_buf_bytes + (size_t)(MAX_KS / 32) * 4 + (size_t)2 * MAX_TILES * 128 * 4 +
           2 * sizeof(ChainNodeInfo) + (size_t)(2 * ring + 2 * TGROUPS + 5) * 8 + 64;
}

} // namespace

struct GemvChain {
    int device = 0;
    ChainParams cp{};
    ChainNodeDev *d_nodes = nullptr;
    unsigned int *d_xbuf = nullptr;        // {f16, tag} words of every node's output rows
    unsigned long long *d_pbuf = nullptr;  // {f32, tag} words of the K slices' row sums
    unsigned int tag = 0;                  // the last dispatch's tag
    bool wrong_tag_once = false;           // bounded-wait test hook: the next dispatch publishes a tag nobody waits for
    int grid = 0;
    size_t smem = 0;
    std::string name;
};

const char *gemv_chain_name(const GemvChain *c) { return c ? c->name.c_str() : ""; }

void gemv_chain_destroy(GemvChain *c) {
    if (!c) return;
    cudaSetDevice(c->device);
    if (c->d_nodes) cudaFree(c->d_nodes);
    if (c->d_xbuf) cudaFree(c->d_xbuf);
    if (c->d_pbuf) cudaFree(c->d_pbuf);
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
    int max_split = 1;
    for (size_t i = 0; i < nodes.size(); i++) {
        const MatmulParams &p = nodes[i];
        const int s = p.K >= 256 ? split_for(p.K) : 0;
        if (s == 0) { *why = "K is not a multiple of 256 per slice"; return cudaSuccess; }
        splits.push_back(s);
        if (s > max_split) max_split = s;
        // the nodes hand their rows on through tagged words: node i must read exactly what node i-1 wrote
        if (i > 0 && (p.rhs != nodes[i - 1].out || p.K != nodes[i - 1].M)) { *why = "not a chain: a node does not read its predecessor's output"; return cudaSuccess; }
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
    int slot_bytes = 0, b_bytes = GUARD_BYTES, scale_buf_bytes = 0, mmas = 0;
    size_t x_words = 0, p_words = 0;
    int max_stages = 0;
    for (size_t i = 0; i < nodes.size(); i++) {
        const MatmulParams &p = nodes[i];
        ChainNodeDev &nd = host[i];
        std::memset(&nd, 0, sizeof(nd));
        const int units = grid / splits[i];
        const int rb = (p.M + units - 1) / units;
        if (rb > 128 || rb < 9) { *why = "rows per CTA outside 9..128"; return cudaSuccess; }
        nd.M = p.M; nd.K = p.K; nd.rb = rb; nd.rb8 = (rb + 7) & ~7; nd.split = splits[i];
        nd.ks = p.K / splits[i];
        if (!pick_stage(nd)) { *why = "no stage shape for this node"; return cudaSuccess; }
        nd.rhs = p.rhs; nd.out = p.out; nd.bias = p.bias;
        nd.lhs = p.lhs; nd.lhs_scales = p.lhs_scales;
        nd.bias_mode = p.bias_mode; nd.bias_dt = p.bias_dt; nd.epilogue = p.epilogue;
        slot_bytes = std::max(slot_bytes, nd.S * nd.rb8 * 128);
        b_bytes = std::max(b_bytes, nd.nstages * nd.tiles * nd.b_tile_bytes);
        scale_buf_bytes = std::max(scale_buf_bytes, nd.rb8 * (nd.ks / 16));
        mmas = std::max(mmas, nd.nstages * nd.tiles * 4);
        max_stages = std::max(max_stages, nd.nstages);
        nd.x_off = (int)x_words;
        x_words += (size_t)((p.M + 31) & ~31);
        nd.p_off = (int)p_words;
        if (nd.split > 1) p_words += (size_t)nd.split * p.M;
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
            cuuint32_t box[2] = {(cuuint32_t)(nd.ks / 32), (cuuint32_t)rb};
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
        cp.n_issue = v ? std::max(1, std::min(N_ISSUE, atoi(v))) : 3;
        const char *pv = getenv("RT_CHAIN_PACE");
        cp.pace = pv ? std::max(0, atoi(pv)) : 300;
        cp.skip_tempty = max_stages <= TGROUPS ? 1 : 0;

    }
    cp.slot_bytes = (slot_bytes + 1023) & ~1023;
    cp.b_bytes = (b_bytes + 1023) & ~1023;
    cp.scale_buf_bytes = (scale_buf_bytes + 127) & ~127;
    int ring = 16;
    while (ring > 2 && smem_for(ring, cp.slot_bytes, cp.b_bytes, cp.scale_buf_bytes) > SMEM_LIMIT) ring--;
    if (smem_for(ring, cp.slot_bytes, cp.b_bytes, cp.scale_buf_bytes) > SMEM_LIMIT) {
        delete c;
        *why = "ring does not fit";
        return cudaSuccess;
    }
    cp.ring = ring;
    c->smem = smem_for(ring, cp.slot_bytes, cp.b_bytes, cp.scale_buf_bytes);
    e = cudaMalloc(&c->d_nodes, host.size() * sizeof(ChainNodeDev));
    if (e == cudaSuccess) e = cudaMalloc(&c->d_xbuf, sizeof(unsigned int) * x_words);
    if (e == cudaSuccess) e = cudaMemset(c->d_xbuf, 0, sizeof(unsigned int) * x_words); // tag 0: no dispatch
    if (e == cudaSuccess && p_words > 0) e = cudaMalloc(&c->d_pbuf, sizeof(unsigned long long) * p_words);
    if (e == cudaSuccess && p_words > 0) e = cudaMemset(c->d_pbuf, 0, sizeof(unsigned long long) * p_words);
    if (e == cudaSuccess) e = cudaMemcpy(c->d_nodes, host.data(), host.size() * sizeof(ChainNodeDev), cudaMemcpyHostToDevice);
    if (e != cudaSuccess) {
        gemv_chain_destroy(c);
        return e;
    }
    cp.nodes = c->d_nodes;
    {
        // where the dispatch tags start (a test hook: the tag wraps from 65535 to 1)
        const char *tv = getenv("RT_CHAIN_TAG_START");
        if (tv) c->tag = (unsigned int)std::max(0, std::min(65535, atoi(tv)));
        // two more test hooks: a short budget for the readers' waits, and one dispatch whose rows carry a tag no
        // reader waits for, so that those waits run out (nothing faults or spins past the budget)
        const char *wv = getenv("RT_CHAIN_WAIT_CYCLES");
        cp.poll_limit = wv ? (unsigned long long)std::max(1000ll, atoll(wv)) : WAIT_LIMIT_CYCLES;
        const char *bv = getenv("RT_CHAIN_TEST_WRONG_TAG");
        c->wrong_tag_once = bv && bv[0] == '1';
    }
    cp.xbuf = c->d_xbuf;
    cp.pbuf = c->d_pbuf;
    c->name = "q8_gemv_chain_h_nodes" + std::to_string(cp.n_nodes) + "_grid" + std::to_string(grid) + "_maxsplit" + std::to_string(max_split) +
              "_ring" + std::to_string(ring) + "x" + std::to_string(cp.slot_bytes / 1024) + "k_mma" + std::to_string(mmas);
    *out = c;
    return cudaSuccess;
}

// One dispatch of the whole chain: a new tag, one cooperative launch.
cudaError_t gemv_chain_launch(GemvChain *c, cudaStream_t stream) {
    c->tag = c->tag >= 65535u ? 1u : c->tag + 1u;
    c->cp.tag = c->tag;
    c->cp.publish_tag = c->tag;
    if (c->wrong_tag_once) {
        c->cp.publish_tag = c->tag ^ 0x8000u;
        c->wrong_tag_once = false;
    }
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
