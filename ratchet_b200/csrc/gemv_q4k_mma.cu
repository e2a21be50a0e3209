// Q4_K GEMV / skinny GEMM for f16 activations: y[v][r] = sum_k W[r][k] * x[v][k], 1..16 vectors.
//
// The reference declares the Q4_K block (crates/ratchet-loader/src/k_quants.rs:95-103) but has no
// kernel for it; this kernel gives the format the same decode path Q8_0 has.  W is raw GGUF
// super-blocks: 144 bytes per 256 values = {f16 d, f16 dmin, 12 bytes of 6-bit (scale, min) pairs,
// 128 bytes of nibbles}; value = (d*sc_j)*q - dmin*m_j for sub-block j of 32.
//
// Design (HBM-bound: 0.5625 bytes per weight):
//  * a CTA owns 16 consecutive rows and a slice of K.  At entry one thread asks the TMA engine for
//    the CTA's whole share (one bulk copy per row into padded shared-memory rows) before the kernel
//    waits for its stream predecessor when the weights are constants; the activations are staged
//    after that wait, permuted to the order in which nibbles leave a 32-bit word, together with
//    their per-sub-block sums;
//  * all threads decode the super-block headers once into a table of (s1, s3) per (row, sub-block)
//    with s1 = d*sc and s3 = 1024*s1 + dmin*m;
//  * 8 warps interleave over pairs of sub-blocks (one 8-byte load per row holds both: low and high
//    nibbles).  A nibble q becomes the f16 value 1024+q with one shift and one AND/OR; a 16x32 tile
//    meets the activations in two m16n8k16 tensor-core MMAs (f32 accumulate), and
//    sum_k (s1*q - dmin*m) x = s1 * sum_k (1024+q) x - s3 * sum_k x;
//  * warps are reduced through shared memory in a fixed order and K slices through distributed
//    shared memory in rank order: deterministic results;
//  * with more than four vectors the staged activations outweigh one row group's weights, so a CTA
//    then keeps them and walks several row groups, the next group's super-blocks already in flight
//    into a second buffer while the current one is multiplied;
//  * epilogue = the reference's: f16(acc) + bias in f16, optional fused GELU.
#include <algorithm>
#include <cstdlib>
#include <cooperative_groups.h>

#include "common.cuh"
#include "decode.cuh"
#include "kernels.hpp"

namespace cg = cooperative_groups;

namespace rt {

__device__ int g_gemv_q4k_error = 0;

namespace {

constexpr int WARPS_ONCE = 8;  // a CTA that handles one row group (up to four such CTAs per SM)
constexpr int WARPS_WALK = 16; // a CTA that walks several row groups (one or two per SM)
constexpr int ROWS = 16;
constexpr int SB_BYTES = 144;
constexpr unsigned long long WAIT_LIMIT_CYCLES = 4000000000ull;

__device__ __forceinline__ void mma_m16n8k16_f16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}

// row stride of the staged super-blocks: a multiple of 16 that is 32 mod 128 (conflict-free 8-byte reads by 8 rows)
__host__ __device__ inline int row_stride(int nsb) { const int b = nsb * SB_BYTES; return b + ((32 - b % 128) + 128) % 128; }

// halves between two staged activation vectors: 64 bytes past a multiple of 128, so that the 16-byte
// reads of the two vectors (B-fragment columns) in one quarter-warp fall in different banks
__host__ __device__ inline int x_stride(int nsb) { return nsb * 256 + 32; }

struct Q4kLayout {
    int codes, table, slot, x, xsum, red, bar, total; // byte offsets (slot: bytes per half-CTA table)
};
__host__ __device__ inline Q4kLayout layout(int nsb, int nv, int nbuf) {
    const int WARPS = nbuf > 1 ? WARPS_WALK : WARPS_ONCE;
    Q4kLayout l;
    l.codes = 0;                                             // nbuf buffers of ROWS padded rows
    const int cols = nv <= 8 ? 8 : 16;
    l.slot = ROWS * (nsb * 8 + 1) * 8;                       // float2 [ROWS][nsb*8 + 1]
    l.table = nbuf * ROWS * row_stride(nsb);                 // one table per half-CTA when walking
    l.x = l.table + (nbuf > 1 ? 2 : 1) * l.slot;             // half [nv][x_stride], permuted
    l.xsum = l.x + nv * x_stride(nsb) * 2;                   // float [nsb*8][cols]
    l.red = l.xsum + nsb * 8 * cols * 4;                     // float [WARPS][ROWS][cols]
    l.bar = l.red + WARPS * ROWS * cols * 4;
    l.total = l.bar + 8 * 4; // up to four buffers, one barrier each
    return l;
}

// NVG: groups of 8 activation vectors (1 or 2).  SPLIT: K is split over a cluster of gridDim.y CTAs.
// WARPS: WARPS_WALK when the CTA walks gpc > 1 row groups through nbuf buffers, else WARPS_ONCE.
// HALVES: 2 = the two halves of the CTA's warps work on alternate row groups at the same time,
// each with its own header table, partial sums and named barrier, sharing the activations and the
// buffers (like two CTAs per SM, without staging the activations twice); not with SPLIT, whose
// cluster barrier needs the whole CTA.
// n consecutive Q4_K values of one row (from global memory, starting at a super-block) against one staged activation
// vector, element by element in f32: IEEE's rules for infinities and NaNs decide the result, not the order of the sum.
// Kept out of line so that the kernel's registers are those of its main path.
__device__ __forceinline__ float exact_dot(const uint8_t *row, const __half *xv, int n) {
    float acc = 0.f;
    for (int k = 0; k < n; k++) {
        const int pos = (k & ~7) | ((0x75643120u >> (4 * (k & 7))) & 7); // the staged order 0,2,1,3,4,6,5,7
        acc += q4k_element(row, k) * __half2float(xv[pos]);
    }
    return acc;
}

// Registers: a walking CTA (512 threads) is given all the registers one CTA per SM can have (70 .. 96 are used): held to
// 64 for two CTAs per SM it was up to 7 % slower with 9 .. 16 vectors and no faster with fewer.  The one-row-group CTAs
// keep the compiler's own choice (64 or fewer: four per SM).
template <int NVG, bool SPLIT, int WARPS, int HALVES>
__global__ void __launch_bounds__(WARPS * 32, WARPS == WARPS_WALK ? 1 : 0) q4k_gemv_kernel(MatmulParams p, int nv, int sb_per_cta, int lhs_constant, int gpc, int nbuf) {
    static_assert(HALVES == 1 || !SPLIT, "the cluster barrier needs every thread");
    constexpr int THREADS = WARPS * 32;
    constexpr int WH = WARPS / HALVES, TH = WH * 32; // warps and threads that share a row group
    extern __shared__ __align__(128) uint8_t smem[];
    const int lane = threadIdx.x & 31;
    const int half = HALVES == 2 ? (int)(threadIdx.x / TH) : 0;
    const int t = (int)threadIdx.x - half * TH;       // thread index within the half
    const int warp = t >> 5;                          // warp index within the half
    auto half_sync = [&]() {
        if (HALVES == 1) __syncthreads();
        else asm volatile("bar.sync %0, %1;" ::"r"(1 + half), "r"(TH) : "memory");
    };
    const int g = lane >> 2, c = lane & 3;
    const int batch = blockIdx.z;
    const int nsb_total = p.K >> 8;
    const int split = SPLIT ? (int)blockIdx.y : 0;
    const int sb_begin = split * sb_per_cta;
    const int nsb = max(0, min(nsb_total, sb_begin + sb_per_cta) - sb_begin);
    const Q4kLayout L = layout(sb_per_cta, nv, nbuf);
    const int rstride = row_stride(sb_per_cta);
    uint8_t *codes_s = smem + L.codes;
    const int tstride = sb_per_cta * 8 + 1;
    float2 *table = reinterpret_cast<float2 *>(smem + L.table + half * L.slot);
    __half *x_s = reinterpret_cast<__half *>(smem + L.x);
    float *xsum = reinterpret_cast<float *>(smem + L.xsum);
    constexpr int COLS = NVG * 8;
    float *red = reinterpret_cast<float *>(smem + L.red) + half * WH * ROWS * COLS;
    const uint32_t bar_addr = smem_u32(smem + L.bar); // one barrier per buffer, 8 bytes apart

    // this CTA's row groups: gpc consecutive groups of ROWS rows
    const int group0 = blockIdx.x * gpc;
    const int my_groups = max(0, min(gpc, (p.M + ROWS - 1) / ROWS - group0));
    const uint8_t *w = (const uint8_t *)p.lhs + (long long)(batch % p.lhs_stack) * p.M * nsb_total * SB_BYTES;
    const uint32_t row_bytes = (uint32_t)nsb * SB_BYTES;

    // one thread: ask for row group `it` of this CTA (into buffer it % nbuf)
    auto request = [&](int it) {
        const int buf = it % nbuf;
        const int rb = (group0 + it) * ROWS;
        const int rows = min(ROWS, p.M - rb);
        const uint32_t bar = bar_addr + 8u * buf;
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(row_bytes * (uint32_t)rows) : "memory");
        for (int r = 0; r < rows; r++) {
            const uint8_t *src = w + ((long long)(rb + r) * nsb_total + sb_begin) * SB_BYTES;
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                         ::"r"(smem_u32(codes_s + (buf * ROWS + r) * rstride)), "l"(src), "r"(row_bytes), "r"(bar) : "memory");
        }
    };

    if (threadIdx.x == 0) {
        for (int b = 0; b < nbuf; b++) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar_addr + 8u * b) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (!lhs_constant) asm volatile("griddepcontrol.wait;" ::: "memory");
    __syncthreads();

    if (threadIdx.x == 0 && row_bytes > 0) {
        for (int it = 0; it < min(nbuf, my_groups); it++) request(it);
    }
    if (lhs_constant) asm volatile("griddepcontrol.wait;" ::: "memory");

    // ---- activations of this K slice: permuted copy and per-sub-block sums
    // Within every 8 consecutive elements the order becomes 0,2,1,3,4,6,5,7: the order in which the
    // nibbles of two 32-bit words leave the AND / shift sequence below as f16 pairs.
    const int kslice = nsb * 256;
    const long long rbatch = batch % p.rhs_stack;
    // eight independent 16-byte loads per thread are in flight at a time: the activations come from L2
    // and a dependent load per iteration would cost one L2 round trip each.  kslice / 8 is a multiple
    // of 32, so a warp is either wholly inside or wholly outside the range.
    constexpr int XU = 8;
    const int x_items = nv * (kslice / 8);
    auto x_load = [&](int i0, uint4 (&raw)[XU]) {
#pragma unroll
        for (int u = 0; u < XU; u++) {
            const int i = i0 + u * THREADS;
            if (i < x_items) {
                const int v = i / (kslice / 8), o = i - v * (kslice / 8);
                raw[u] = *reinterpret_cast<const uint4 *>((const __half *)p.rhs + (rbatch * nv + v) * (long long)p.K +
                                                          (long long)sb_begin * 256 + o * 8);
            }
        }
    };
    auto x_store = [&](int i0, const uint4 (&raw)[XU]) {
#pragma unroll
        for (int u = 0; u < XU; u++) {
            const int i = i0 + u * THREADS;
            if (i < x_items) {
                const int v = i / (kslice / 8), o = i - v * (kslice / 8);
                const __half *h = reinterpret_cast<const __half *>(&raw[u]);
                __half out[8] = {h[0], h[2], h[1], h[3], h[4], h[6], h[5], h[7]};
                *reinterpret_cast<uint4 *>(x_s + (long long)v * x_stride(sb_per_cta) + o * 8) = *reinterpret_cast<const uint4 *>(out);
                float s = 0.f;
#pragma unroll
                for (int j = 0; j < 8; j++) s += __half2float(h[j]);
                s += __shfl_xor_sync(0xffffffffu, s, 1);
                s += __shfl_xor_sync(0xffffffffu, s, 2);
                if ((o & 3) == 0) xsum[(o >> 2) * COLS + v] = s; // four consecutive 8-element groups = one sub-block
            }
        }
    };

    bool ok = true;
    // waits (bounded) for row group `it` and builds its header table: (s1, s3) per (row, sub-block).
    // One thread per (row, super-block): the 16-byte header in one load, its eight 6-bit (scale, min)
    // pairs unpacked in registers (the packing of q4k_scale_min, decode.cuh).
    auto prepare = [&](int it) {
        const int buf = it % nbuf;
        const uint32_t bar = bar_addr + 8u * buf;
        const uint32_t parity = (uint32_t)(it / nbuf) & 1u; // how often this buffer has been filled before
        const int rows_here = min(ROWS, p.M - (group0 + it) * ROWS);
        const uint8_t *codes_b = codes_s + buf * ROWS * rstride;
        if (ok && row_bytes > 0 && !mbar_try_wait(bar, parity)) {
            const unsigned long long t0 = (unsigned long long)clock64();
            while (!mbar_try_wait(bar, parity)) {
                if ((unsigned long long)clock64() - t0 > WAIT_LIMIT_CYCLES) {
                    ok = false;
                    atomicCAS(&g_gemv_q4k_error, 0, 1);
                    break;
                }
            }
        }
        if (!ok) return;
        for (int item = t; item < ROWS * nsb; item += TH) {
            const int r = item / nsb, sb = item - r * nsb;
            float2 *dst = table + r * tstride + sb * 8;
            if (r < rows_here) {
                const uint4 h = *reinterpret_cast<const uint4 *>(codes_b + r * rstride + sb * SB_BYTES);
                const float d = __half2float(__ushort_as_half((unsigned short)(h.x & 0xFFFFu)));
                const float dmin = __half2float(__ushort_as_half((unsigned short)(h.x >> 16)));
                // scale bytes s[0..3] = h.y, s[4..7] = h.z, s[8..11] = h.w
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const uint32_t a = (h.y >> (8 * j)) & 0xFFu, b = (h.z >> (8 * j)) & 0xFFu, c8 = (h.w >> (8 * j)) & 0xFFu;
                    const float s_lo = d * (float)(a & 63u);                          // sub-block j
                    dst[j] = make_float2(s_lo, fmaf(1024.f, s_lo, dmin * (float)(b & 63u)));
                    const float s_hi = d * (float)((c8 & 0x0Fu) | ((a >> 6) << 4));   // sub-block j + 4
                    dst[j + 4] = make_float2(s_hi, fmaf(1024.f, s_hi, dmin * (float)((c8 >> 4) | ((b >> 6) << 4))));
                }
            } else {
#pragma unroll
                for (int j = 0; j < 8; j++) dst[j] = make_float2(0.f, 0.f);
            }
        }
    };

    {
        uint4 raw[XU];
        x_load(threadIdx.x, raw);
        // a CTA with one row group builds its table while the first activation loads are in flight
        if (WARPS == WARPS_ONCE && my_groups > 0) prepare(0);
        x_store(threadIdx.x, raw);
        for (int i0 = threadIdx.x + THREADS * XU; i0 < x_items; i0 += THREADS * XU) {
            x_load(i0, raw);
            x_store(i0, raw);
        }
    }
    // vectors past nv (the MMA has 8 or 16 columns) read vector nv-1 and a zero sum is not needed: their outputs are dropped

    if (HALVES == 2) __syncthreads(); // the activations are staged by all warps and read by both halves

#pragma unroll 1
    for (int it = half; it < my_groups; it += HALVES) {
    const int buf = it % nbuf;
    const int row_base = (group0 + it) * ROWS;
    const uint8_t *codes_b = codes_s + buf * ROWS * rstride;
    if (WARPS != WARPS_ONCE) prepare(it);
    half_sync();

    float acc[NVG][4];
#pragma unroll
    for (int n = 0; n < NVG; n++)
#pragma unroll
        for (int i = 0; i < 4; i++) acc[n][i] = 0.f;

    if (ok) {
        const uint8_t *qa = codes_b + g * rstride + 16 + c * 8;
        const uint8_t *qb = codes_b + (g + 8) * rstride + 16 + c * 8;
        const float2 *ta = table + g * tstride, *tb = table + (g + 8) * tstride;
        // B fragment column n = g <-> activation vector (clamped); one pointer per group of 8 vectors
        const __half *xl[NVG];
#pragma unroll
        for (int n = 0; n < NVG; n++) xl[n] = x_s + (long long)min(n * 8 + g, nv - 1) * x_stride(sb_per_cta) + c * 8;
        const uint32_t magic = 0x64006400u, mask = 0x000F000Fu;
#pragma unroll 1
        for (int pr = warp; pr < nsb * 4; pr += WH) { // a pair = sub-blocks 2*pr (low nibbles) and 2*pr+1 (high nibbles)
            const int sb = pr >> 2, jp = pr & 3;
            const int off = sb * SB_BYTES + jp * 32;
            const uint2 wa = *reinterpret_cast<const uint2 *>(qa + off);
            const uint2 wb = *reinterpret_cast<const uint2 *>(qb + off);
#pragma unroll
            for (int hl = 0; hl < 2; hl++) { // 0: low nibbles, 1: high nibbles
                const int sub = pr * 2 + hl;  // sub-block index inside the slice
                const int sh = hl * 4;
                uint32_t fa[4], fb[4];
                fa[0] = ((wa.x >> sh) & mask) | magic;        // row g   : elements 0,2
                fa[2] = ((wa.x >> (sh + 8)) & mask) | magic;  // row g   : elements 1,3
                fa[1] = ((wb.x >> sh) & mask) | magic;        // row g+8 : elements 0,2
                fa[3] = ((wb.x >> (sh + 8)) & mask) | magic;
                fb[0] = ((wa.y >> sh) & mask) | magic;        // elements 4,6
                fb[2] = ((wa.y >> (sh + 8)) & mask) | magic;  // elements 5,7
                fb[1] = ((wb.y >> sh) & mask) | magic;
                fb[3] = ((wb.y >> (sh + 8)) & mask) | magic;
                const float2 ea = ta[sub], eb = tb[sub];
#pragma unroll
                for (int n = 0; n < NVG; n++) {
                    const uint4 xv = *reinterpret_cast<const uint4 *>(xl[n] + sub * 32);
                    float t[4] = {0.f, 0.f, 0.f, 0.f};
                    mma_m16n8k16_f16(t, fa, xv.x, xv.y);
                    mma_m16n8k16_f16(t, fb, xv.z, xv.w);
                    const float2 xs2 = *reinterpret_cast<const float2 *>(xsum + sub * COLS + n * 8 + 2 * c);
                    acc[n][0] += ea.x * t[0] - ea.y * xs2.x;
                    acc[n][1] += ea.x * t[1] - ea.y * xs2.y;
                    acc[n][2] += eb.x * t[2] - eb.y * xs2.x;
                    acc[n][3] += eb.x * t[3] - eb.y * xs2.y;
                }
            }
        }
    }

    // C fragment: acc[n][0..1] -> (row g, cols n*8 + 2c, +1); acc[n][2..3] -> (row g+8, same cols)
#pragma unroll
    for (int n = 0; n < NVG; n++) {
        red[(warp * ROWS + g) * COLS + n * 8 + 2 * c] = acc[n][0];
        red[(warp * ROWS + g) * COLS + n * 8 + 2 * c + 1] = acc[n][1];
        red[(warp * ROWS + g + 8) * COLS + n * 8 + 2 * c] = acc[n][2];
        red[(warp * ROWS + g + 8) * COLS + n * 8 + 2 * c + 1] = acc[n][3];
    }
    half_sync();
    // every warp is done with this buffer and with the table: refill the buffer for nbuf groups ahead
    if (t == 0 && ok && row_bytes > 0 && it + nbuf < my_groups) {
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        request(it + nbuf);
    }
    const int r = (t >> 4) & 15, v = t < 256 ? (t & 15) : COLS; // one (row, vector) per thread of the first 256
    float sum = 0.f;
    if (v < COLS) {
#pragma unroll
        for (int w8 = 0; w8 < WH; w8++) sum += red[(w8 * ROWS + r) * COLS + v];
    }
    // An infinity among the activations makes s1 * sum((1024+q) x) - s3 * sum(x) = inf - inf: a NaN here is either
    // the product's own or that one, so the slice is summed again for this (row, vector), element by element.
    if (sum != sum && ok && v < nv && row_base + r < p.M)
        sum = exact_dot(w + ((long long)(row_base + r) * nsb_total + sb_begin) * SB_BYTES,
                        x_s + (long long)v * x_stride(sb_per_cta), nsb * 256);
    bool writer = true;
    if (SPLIT) {
        cg::cluster_group cluster = cg::this_cluster();
        __syncthreads();
        if (v < COLS) red[r * COLS + v] = sum;
        cluster.sync();
        if (cluster.block_rank() == 0 && v < COLS) {
            const unsigned n = cluster.num_blocks();
            for (unsigned k = 1; k < n; k++) sum += cluster.map_shared_rank(red, k)[r * COLS + v];
        }
        cluster.sync(); // keep every CTA's shared memory alive until rank 0 has read it
        writer = cluster.block_rank() == 0;
    }
    if (writer && v < nv && ok) {
        const int row = row_base + r;
        if (row < p.M) {
            const bool has_bias = p.bias_mode != BIAS_NONE;
            float bias = 0.f;
            if (has_bias) bias = load_bias(p.bias, p.bias_dt, p.bias_mode == BIAS_PER_M ? row : v);
            const __half o = epilogue_value<__half>(sum, has_bias, bias, p.epilogue);
            const long long ob = (long long)batch * p.M * nv;
            ((__half *)p.out)[p.trans_out ? ob + (long long)v * p.M + row : ob + (long long)row * nv + v] = o;
        }
    }
    } // row groups
}

template <int NVG>
cudaError_t launch_g(const MatmulParams &p, int nv, int split, int gpc, int nbuf, bool lhs_constant, cudaStream_t stream) {
    const int nsb_total = p.K / 256;
    const int spc = (nsb_total + split - 1) / split;
    const size_t smem = (size_t)layout(spc, nv, nbuf).total;
    const bool walk = nbuf > 1;
    auto kernel = walk ? (split == 1 ? q4k_gemv_kernel<NVG, false, WARPS_WALK, 2> : q4k_gemv_kernel<NVG, true, WARPS_WALK, 1>)
                       : (split == 1 ? q4k_gemv_kernel<NVG, false, WARPS_ONCE, 1> : q4k_gemv_kernel<NVG, true, WARPS_ONCE, 1>);
    static SmemAttr smem_attr[4];
    const int slot = (walk ? 2 : 0) + (split != 1 ? 1 : 0);
    if (smem > 48 * 1024) {
        cudaError_t e = smem_attr[slot].ensure(kernel, smem);
        if (e != cudaSuccess) return e;
    }
    const int groups = (p.M + ROWS - 1) / ROWS;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((groups + gpc - 1) / gpc, split, p.stacks);
    cfg.blockDim = dim3((walk ? WARPS_WALK : WARPS_ONCE) * 32);
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
    return cudaLaunchKernelEx(&cfg, kernel, p, nv, spc, lhs_constant ? 1 : 0, gpc, nbuf);
}

} // namespace

// The launch shape for [M][K] x nv vectors: the K split over a cluster (1, 2, 4 or 8) in bits 0-7,
// the row groups one CTA walks in bits 8-15 and its weight buffers in bits 16-23; 0 when the shape
// does not fit the kernel.
int q4k_gemv_pick_split(int M, int K, int nv, int stacks, int sm_count) {
    if (K < 256 || K % 256 != 0 || nv < 1 || nv > 16 || M < 1) return 0;
    const int nsb = K / 256;
    const int groups = (M + ROWS - 1) / ROWS;
    const size_t limit = 200 * 1024, whole_sm = 226 * 1024;
    static const int walk_from = [] { const char *e = std::getenv("RT_Q4K_WALK_FROM"); return e ? std::atoi(e) : 2; }();
    if (nv >= walk_from) {
        // keep the activations and walk row groups, one CTA of WARPS_WALK warps per SM (its registers
        // leave no room for a second): the smallest split that fits at least two weight buffers,
        // then as many buffers (up to four) as fit, since the bytes in flight hide the DRAM latency
        for (int split = 1; split <= 8 && nsb / split >= 1; split *= 2) {
            const int spc = (nsb + split - 1) / split;
            if ((size_t)layout(spc, nv, 2).total > whole_sm) continue;
            const int clusters = std::max(1, sm_count / split / std::max(1, stacks));
            const int gpc = std::min(255, (groups + clusters - 1) / clusters);
            if (gpc < 2) break;
            int nbuf = std::min(4, gpc);
            while (nbuf > 2 && (size_t)layout(spc, nv, nbuf).total > whole_sm) nbuf--;
            return split | (gpc << 8) | (nbuf << 16);
        }
    }
    const size_t target = 56 * 1024; // four CTAs per SM
    int split = 1;
    while (split < 8 && (size_t)layout((nsb + split - 1) / split, nv, 1).total > target) split *= 2;
    while (split < 8 && groups * split < 3 * sm_count && nsb / (split * 2) >= 2) split *= 2;
    if ((size_t)layout((nsb + split - 1) / split, nv, 1).total > limit) return 0;
    return split | (1 << 8) | (1 << 16);
}

cudaError_t launch_q4k_gemv(const MatmulParams &p, int nv, int config, bool lhs_constant, cudaStream_t stream) {
    const int split = config & 0xff, gpc = std::max(1, (config >> 8) & 0xff), nbuf = std::max(1, (config >> 16) & 0xff);
    return nv <= 8 ? launch_g<1>(p, nv, split, gpc, nbuf, lhs_constant, stream)
                   : launch_g<2>(p, nv, split, gpc, nbuf, lhs_constant, stream);
}

cudaError_t gemv_q4k_take_error(int *site, cudaStream_t stream) {
    int zero = 0;
    cudaError_t e = cudaMemcpyFromSymbolAsync(site, g_gemv_q4k_error, sizeof(int), 0, cudaMemcpyDeviceToHost, stream);
    if (e != cudaSuccess) return e;
    e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess) return e;
    if (*site != 0) e = cudaMemcpyToSymbolAsync(g_gemv_q4k_error, &zero, sizeof(int), 0, cudaMemcpyHostToDevice, stream);
    return e;
}

} // namespace rt
