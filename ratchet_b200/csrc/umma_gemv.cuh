// Device helpers shared by the tcgen05 Q8_0 GEMV kernels (single launch and persistent chain): mbarrier,
// TMA, tcgen05 wrappers, and the conversion of a slice of the f16 activation vector into the
// block-floating-point int8 digit tiles the MMAs read as their B operand.  Both kernels must
// produce the same bits for the same node, so the arithmetic lives here once.
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace rt {
namespace umma_gemv {

// cuTensorMapEncodeTiled through the runtime's driver entry point (no link against libcuda)
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
inline EncodeTiledFn encode_tiled_fn() {
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

constexpr unsigned long long WAIT_LIMIT_CYCLES = 4000000000ull;

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ unsigned long long wait_clock() { return (unsigned long long)clock64(); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
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
// Bounded wait: gives up after WAIT_LIMIT_CYCLES, or as soon as the CTA's abort flag is up; the first
// site that gives up is recorded in *error_word (a __device__ int the host reads at its next sync).
__device__ __forceinline__ bool mbar_wait_flag(uint32_t bar, uint32_t parity, volatile int *abort_flag, int site, int *error_word) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = wait_clock();
    while (true) {
#pragma unroll 1
        for (int i = 0; i < 32; i++)
            if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (wait_clock() - t0 > WAIT_LIMIT_CYCLES) {
            *abort_flag = 1;
            atomicCAS(error_word, 0, site);
            return false;
        }
    }
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int c0, int c1, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(bar) : "memory");
}

// K-major operand tile, 128-byte swizzle, 8-row groups `group_stride` bytes apart.  The digit tiles
// hold 8 rows and use a stride of 0: rows 8..15 of the N = 16 operand repeat rows 0..7, which only
// duplicates accumulator columns that the next block overwrites (see the MMA issuer).
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr, uint32_t group_stride) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(group_stride >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

__device__ __forceinline__ void umma_i8(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc) {
    // the predicate is false: the accumulator slot is overwritten, every block starts from zero
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, 0, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}\n"
                 ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, int (&v)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                   "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
                 : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Four accumulator columns (two hi / lo pairs) of one MMA, no wait; the upper four values are left alone.
__device__ __forceinline__ void tmem_ld4_nowait(uint32_t taddr, int (&v)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]) : "r"(taddr) : "memory");
}
// Eight accumulator columns (four hi / lo pairs) of one MMA, no wait.
__device__ __forceinline__ void tmem_ld8_nowait(uint32_t taddr, int (&v)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
                 : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Eight consecutive activations (one quarter of a Q8_0 block; the four threads of a quad hold one
// block) -> their hi / lo int8 digits (eight bytes each) and the block's power-of-two scale.
//   m = round(x / xs), |m| <= 16383, m = 256 * hi + lo with lo in [-128, 127];  x ~ m * xs.
// A block that holds a NaN or an infinity cannot be written as digits: it gets zero digits and a zero
// scale (it then adds nothing to any row) and `nonfinite` is set for all four threads of the quad, so
// that the caller can add the block's products the way the reference forms them (nonfinite_block_products).
__device__ __forceinline__ void quantize_quarter_block(const uint4 raw, uint2 &hi8, uint2 &lo8, float &xs_of_block, bool &nonfinite) {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
    const __half2 *h2 = reinterpret_cast<const __half2 *>(&raw);
    float v[8];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const float2 f = __half22float2(h2[i]);
        v[2 * i] = f.x;
        v[2 * i + 1] = f.y;
    }
    // the largest magnitude as a bit pattern (f16 magnitudes order like integers; NaN and infinities, whose
    // exponent field is all ones, come out on top, which a floating-point maximum would not guarantee)
    uint32_t amax_bits = 0u;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const uint32_t a = w[i] & 0x7FFF7FFFu;
        amax_bits = max(amax_bits, max(a & 0xFFFFu, a >> 16));
    }
    amax_bits = max(amax_bits, __shfl_xor_sync(0xffffffffu, amax_bits, 1));
    amax_bits = max(amax_bits, __shfl_xor_sync(0xffffffffu, amax_bits, 2));
    nonfinite = amax_bits >= 0x7C00u;
    const float amax = nonfinite ? 0.f : __half2float(__ushort_as_half((unsigned short)amax_bits));
    // amax < 2^(E-126) for its exponent field E: scale it below 2^14
    const int E = (int)((__float_as_uint(amax) >> 23) & 0xFFu);
    const float scale = amax > 0.f ? __uint_as_float((uint32_t)(140 - E + 127) << 23) : 0.f;
    xs_of_block = amax > 0.f ? __uint_as_float((uint32_t)(E - 13) << 23) : 0.f;
    uint32_t hi_w[2] = {0u, 0u}, lo_w[2] = {0u, 0u};
#pragma unroll
    for (int i = 0; i < 8; i++) {
        int m = __float2int_rn(v[i] * scale);
        m = max(-16383, min(16383, m));
        const int hi = (m + 128) >> 8;
        const int lo = m - (hi << 8);
        hi_w[i >> 2] |= (uint32_t)(hi & 0xFF) << (8 * (i & 3));
        lo_w[i >> 2] |= (uint32_t)(lo & 0xFF) << (8 * (i & 3));
    }
    hi8 = make_uint2(hi_w[0], hi_w[1]);
    lo8 = make_uint2(lo_w[0], lo_w[1]);
}

// One 32-wide block's contribution to one weight row, formed the way the reference's GEMV forms it
// (crates/ratchet-core/src/ops/gemv.rs:470-480: code times scale rounded to f16, times x in f16, widened to
// f32 and added), so that NaN and infinities in x come out as IEEE arithmetic gives them.  Only blocks that
// quantize_quarter_block flagged take this path.  The activations are either plain f16 (`x_plain`) or the
// low halves of 32-bit words (`x_words`, the chain kernels' exchange format); the other pointer is null.
__device__ __forceinline__ float nonfinite_block_products(const int8_t *codes, __half d, const __half *x_plain, const unsigned int *x_words) {
    float sum = 0.f;
    for (int i = 0; i < 32; i++) {
        const __half xv = x_plain ? x_plain[i] : __ushort_as_half((unsigned short)(__ldcg(x_words + i) & 0xFFFFu));
        const __half w = __hmul(__int2half_rn((int)codes[i]), d);
        sum += __half2float(__hmul(w, xv));
    }
    return sum;
}

// Stores eight digit bytes at byte `kpos` (a multiple of 8 below 128) of row `row` (0..7) of a K-major
// 8-row x 128-byte operand tile with the 128-byte swizzle: 16-byte chunks XOR the row index.
__device__ __forceinline__ void store_digits8(uint8_t *tile, int row, int kpos, uint2 v) {
    const int chunk = kpos >> 4, within = kpos & 15;
    *reinterpret_cast<uint2 *>(tile + row * 128 + ((chunk ^ row) << 4) + within) = v;
}

// The single-launch kernel's layout: one 8-row tile per 128 bytes of K, row 0 = hi, row 1 = lo, rows
// 2..7 zero.  `blk` is the block index inside the CTA's K slice, `sub` the quarter (0..3).
__device__ __forceinline__ bool digits_of_quarter_block(const uint4 raw, int blk, int sub, uint8_t *b_tiles, float *xs) {
    uint2 hi8, lo8;
    float inv;
    bool nonfinite;
    quantize_quarter_block(raw, hi8, lo8, inv, nonfinite);
    uint8_t *tile = b_tiles + (size_t)(blk >> 2) * 1024;
    const int kpos = (blk & 3) * 32 + sub * 8;
    store_digits8(tile, 0, kpos, hi8);
    store_digits8(tile, 1, kpos, lo8);
    if (sub == 0) xs[blk] = inv;
    return nonfinite;
}

// One block's contribution to a row: d = weight scale, xsv = activation scale, (hi, lo) = the MMA's two sums.
__device__ __forceinline__ float add_block(float acc, float d, float xsv, int hi, int lo) {
    // 256 * hi + lo fits an int (|hi|, |lo| < 2^20): one exact integer add, one rounding to f32 - the same
    // value as fmaf(256, hi, lo)
    const float t = (float)(hi * 256 + lo);
    return fmaf(d * xsv, t, acc);
}

} // namespace umma_gemv
} // namespace rt
