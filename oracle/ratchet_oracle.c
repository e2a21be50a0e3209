/*
 * CPU oracle for ratchet-core's Matmul path.  TEST INFRASTRUCTURE ONLY: it is
 * imported by the tests, by the smoke check and by the benchmark's cpu_baseline /
 * reference legs as the checker and the timed CPU baseline.  The product library
 * never links, loads or calls anything in this file.
 *
 * It restates, in plain C, the arithmetic of the reference (FL33TW00D/ratchet,
 * paths relative to that project):
 *   - Q8_0 quantise / dequantise      crates/ratchet-core/src/quant.rs:26-124
 *   - Q8_0 device layout (segments)   crates/ratchet-core/src/dtype/blocks.rs:61-74,
 *                                     crates/ratchet-core/src/gpu/align.rs:23-40
 *   - GGUF Q8_0 -> ratchet transcode  crates/ratchet-loader/src/gguf/dtype.rs:44-110
 *   - code unpack                     crates/ratchet-core/src/gpu/wgsl/kernel_builder.rs:222-240
 *   - GEMM arithmetic                 crates/ratchet-core/src/ops/gemm.rs:342-492
 *   - GEMV arithmetic                 crates/ratchet-core/src/ops/gemv.rs:333-558
 *   - tanh-GELU                       crates/ratchet-core/src/ops/unary.rs:75-119
 *   - Q4_K block struct (format only) crates/ratchet-loader/src/k_quants.rs:95-103
 *
 * Parity pin: the reference is Rust + WebGPU and cannot be built or run here and holds
 * no golden vectors for Matmul; its tests compare against torch.matmul at run time
 * (crates/ratchet-core/src/ops/matmul.rs:663-718).  This oracle is pinned the same way:
 * against torch.matmul / F.gelu(approximate="tanh") and against the gguf Python
 * package's Q8_0 / Q4_K decoders, through the fixtures in tests/golden/.
 * Q4_K matmul is NOT implemented by the reference: "parity unpinned" for that format;
 * the Q4_K decoder below is pinned bit-exactly to gguf-py's decoder only.
 *
 * Two matmul oracles:
 *   orc_matmul_truth     fp64 accumulation, result left in fp64 (caller rounds once)
 *   orc_matmul_faithful  products rounded to the activation dtype, f32 accumulation in
 *                        K order, accumulator -> dtype, bias added in dtype (what the
 *                        reference's shaders do)
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define QK8_0 32
#define QK_K 256
#define Q4K_BLOCK_BYTES 144

/* ---------------------------------------------------------------- f16 helpers */

typedef _Float16 f16_t;

static inline float f16_bits_to_f32(uint16_t h) {
    f16_t v;
    memcpy(&v, &h, 2);
    return (float)v;
}

static inline uint16_t f32_to_f16_bits(float f) {
    f16_t v = (f16_t)f; /* round to nearest even */
    uint16_t h;
    memcpy(&h, &v, 2);
    return h;
}

static inline float round_f16(float f) { return (float)(f16_t)f; }

void orc_f32_to_f16(const float *src, uint16_t *dst, int64_t n) {
    for (int64_t i = 0; i < n; i++) dst[i] = f32_to_f16_bits(src[i]);
}

void orc_f16_to_f32(const uint16_t *src, float *dst, int64_t n) {
    for (int64_t i = 0; i < n; i++) dst[i] = f16_bits_to_f32(src[i]);
}

/* f64 -> f16 with a single rounding (double -> _Float16 is a direct conversion) */
void orc_f64_to_f16(const double *src, uint16_t *dst, int64_t n) {
    for (int64_t i = 0; i < n; i++) {
        f16_t v = (f16_t)src[i];
        memcpy(&dst[i], &v, 2);
    }
}

/* f64 -> bf16 bits with a single rounding: f64 -> f32 with round-to-odd (keeps the
 * sticky information), then f32 -> bf16 round to nearest even. */
void orc_f64_to_bf16(const double *src, uint16_t *dst, int64_t n) {
    for (int64_t i = 0; i < n; i++) {
        double x = src[i];
        if (isnan(x)) { dst[i] = 0x7fc0; continue; }
        float f = (float)x;
        uint32_t u;
        if ((double)f != x) {
            if (fabs((double)f) > fabs(x)) f = nextafterf(f, 0.0f);
            memcpy(&u, &f, 4);
            u |= 1u;
        } else {
            memcpy(&u, &f, 4);
        }
        u += 0x7fffu + ((u >> 16) & 1u);
        dst[i] = (uint16_t)(u >> 16);
    }
}

/* ---------------------------------------------------------------- layout */

/* align.rs:23-40  align_for_offset: round up to a multiple of 256 */
static inline int64_t align256(int64_t n) {
    int64_t r = n % 256;
    return r == 0 ? n : n + 256 - r;
}

/* blocks.rs:61-74: two segments, codes then scales, each padded to 256 bytes.
 * scale_bytes is 2 (Q8_0H) or 4 (Q8_0F).  out[4] = {qs_off, qs_len, d_off, d_len}. */
void orc_q8_segments(int64_t numel, int scale_bytes, int64_t out[4]) {
    int64_t qs = align256(numel);
    int64_t ds = align256((numel / QK8_0) * (int64_t)scale_bytes);
    out[0] = 0;
    out[1] = qs;
    out[2] = qs;
    out[3] = ds;
}

int64_t orc_q8_nbytes(int64_t numel, int scale_bytes) {
    int64_t s[4];
    orc_q8_segments(numel, scale_bytes, s);
    return s[1] + s[3];
}

/* ---------------------------------------------------------------- Q8_0 quantiser */

/* Rust `f32 as i32`: NaN -> 0, saturating. */
static inline int32_t rust_f32_as_i32(float v) {
    if (isnan(v)) return 0;
    if (v >= 2147483648.0f) return INT32_MAX;
    if (v <= -2147483648.0f) return INT32_MIN;
    return (int32_t)v;
}

/* quant.rs:26-79  sint8_quantize: per 32 elements d = max|x| / 127 (f32);
 * code = round(x / d) (half away from zero) & 0xFF, four codes per little-endian u32.
 * Output buffer = codes padded to 256 B, then f32 scales padded to 256 B (Q8_0F). */
void orc_q8_quantize_f(const float *x, int64_t numel, uint8_t *out) {
    int64_t seg[4];
    orc_q8_segments(numel, 4, seg);
    memset(out, 0, (size_t)(seg[1] + seg[3]));
    uint32_t *qs = (uint32_t *)out;
    float *ds = (float *)(out + seg[2]);
    float d = -INFINITY;
    for (int64_t i = 0; i < numel; i += 4) {
        if (i % QK8_0 == 0) {
            float amax = -INFINITY;
            for (int j = 0; j < QK8_0; j++) {
                float a = fabsf(x[i + j]);
                /* f32::max ignores NaN operands */
                if (!(a <= amax)) amax = isnan(a) ? amax : a;
            }
            d = amax / 127.0f;
        }
        uint32_t packed = 0;
        for (int j = 0; j < 4; j++) {
            int32_t q = rust_f32_as_i32(roundf(x[i + j] / d)) & 0xFF;
            packed |= (uint32_t)q << (8 * j);
        }
        qs[i / 4] = packed;
        ds[i / QK8_0] = d;
    }
}

/* The Q8_0H form of a synthetic weight: same codes, scale rounded to f16
 * (what the loader holds for a GGUF file: gguf/dtype.rs:80-109 keeps d as f16). */
void orc_q8_f_to_h(const uint8_t *qf, int64_t numel, uint8_t *out) {
    int64_t sf[4], sh[4];
    orc_q8_segments(numel, 4, sf);
    orc_q8_segments(numel, 2, sh);
    memset(out, 0, (size_t)(sh[1] + sh[3]));
    memcpy(out, qf, (size_t)numel);
    const float *df = (const float *)(qf + sf[2]);
    uint16_t *dh = (uint16_t *)(out + sh[2]);
    for (int64_t b = 0; b < numel / QK8_0; b++) dh[b] = f32_to_f16_bits(df[b]);
}

/* quant.rs:81-124 sint8_dequantize: (i8)q * d in f32 */
void orc_q8_dequantize_f(const uint8_t *buf, int64_t numel, float *out) {
    int64_t seg[4];
    orc_q8_segments(numel, 4, seg);
    const int8_t *qs = (const int8_t *)buf;
    const float *ds = (const float *)(buf + seg[2]);
    for (int64_t i = 0; i < numel; i++) out[i] = (float)qs[i] * ds[i / QK8_0];
}

/* Q8_0H dequant as the shaders do it: f16(q) * d, product rounded to f16
 * (gemm.rs:400-406, gemv.rs:509, kernel_builder.rs:222-231).  Result as f16 bits. */
void orc_q8_dequantize_h(const uint8_t *buf, int64_t numel, uint16_t *out) {
    int64_t seg[4];
    orc_q8_segments(numel, 2, seg);
    const int8_t *qs = (const int8_t *)buf;
    const uint16_t *ds = (const uint16_t *)(buf + seg[2]);
    for (int64_t i = 0; i < numel; i++) {
        float v = (float)qs[i] * f16_bits_to_f32(ds[i / QK8_0]); /* exact in f32 */
        out[i] = f32_to_f16_bits(v);
    }
}

/* gguf/dtype.rs:44-73 (F) and 80-109 (H): GGUF BlockQ8_0 {f16 d; i8 qs[32]} (34 bytes)
 * -> codes segment, scales segment.  */
void orc_q8_transcode_gguf(const uint8_t *blocks, int64_t n_blocks, int scale_bytes, uint8_t *out) {
    int64_t numel = n_blocks * QK8_0;
    int64_t seg[4];
    orc_q8_segments(numel, scale_bytes, seg);
    memset(out, 0, (size_t)(seg[1] + seg[3]));
    for (int64_t b = 0; b < n_blocks; b++) {
        const uint8_t *blk = blocks + b * 34;
        uint16_t d;
        memcpy(&d, blk, 2);
        memcpy(out + b * QK8_0, blk + 2, QK8_0);
        if (scale_bytes == 2) {
            memcpy(out + seg[2] + b * 2, &d, 2);
        } else {
            float f = f16_bits_to_f32(d);
            memcpy(out + seg[2] + b * 4, &f, 4);
        }
    }
}

/* ---------------------------------------------------------------- Q4_K */

/* Block = {f16 d; f16 dmin; u8 scales[12]; u8 qs[128]} (k_quants.rs:95-103), 256 values.
 * Eight sub-blocks of 32 four-bit codes; sub-block j has a 6-bit scale sc_j and a 6-bit
 * min m_j packed into the 12 scale bytes; value = (d*sc_j)*q - (dmin*m_j), every
 * product and the difference rounded to f32 separately (that order is what the gguf
 * Python decoder computes, and the fixtures pin it bit-exactly). */
static inline void q4k_scale_min(int j, const uint8_t *s, uint8_t *sc, uint8_t *m) {
    if (j < 4) {
        *sc = s[j] & 63;
        *m = s[j + 4] & 63;
    } else {
        *sc = (uint8_t)((s[j + 4] & 0x0F) | ((s[j - 4] >> 6) << 4));
        *m = (uint8_t)((s[j + 4] >> 4) | ((s[j] >> 6) << 4));
    }
}

void orc_q4k_dequantize(const uint8_t *blocks, int64_t numel, float *out) {
    int64_t nb = numel / QK_K;
    for (int64_t b = 0; b < nb; b++) {
        const uint8_t *blk = blocks + b * Q4K_BLOCK_BYTES;
        uint16_t dh, dmh;
        memcpy(&dh, blk, 2);
        memcpy(&dmh, blk + 2, 2);
        float d = f16_bits_to_f32(dh), dmin = f16_bits_to_f32(dmh);
        const uint8_t *scales = blk + 4;
        const uint8_t *qs = blk + 16;
        float *y = out + b * QK_K;
        for (int j = 0; j < 8; j++) {
            uint8_t sc, m;
            q4k_scale_min(j, scales, &sc, &m);
            volatile float ds = d * (float)sc;   /* volatile: forbid fused multiply-add */
            volatile float dm = dmin * (float)m;
            const uint8_t *q = qs + 32 * (j / 2);
            for (int l = 0; l < 32; l++) {
                int code = (j & 1) ? (q[l] >> 4) : (q[l] & 0x0F);
                volatile float p = ds * (float)code;
                y[j * 32 + l] = p - dm;
            }
        }
    }
}

/* Encoder (ours; the reference has none): per sub-block affine fit x ~ s*q - m with
 * q in 0..15, m >= 0; super-block d = max s / 63, dmin = max m / 63 held as f16. */
void orc_q4k_quantize(const float *x, int64_t numel, uint8_t *out) {
    int64_t nb = numel / QK_K;
    for (int64_t b = 0; b < nb; b++) {
        const float *xb = x + b * QK_K;
        uint8_t *blk = out + b * Q4K_BLOCK_BYTES;
        float s[8], m[8];
        float smax = 0.f, mmax = 0.f;
        for (int j = 0; j < 8; j++) {
            float lo = xb[j * 32], hi = xb[j * 32];
            for (int l = 1; l < 32; l++) {
                float v = xb[j * 32 + l];
                if (v < lo) lo = v;
                if (v > hi) hi = v;
            }
            if (lo > 0.f) lo = 0.f;
            if (hi < lo) hi = lo;
            s[j] = (hi - lo) / 15.0f;
            m[j] = -lo;
            if (s[j] > smax) smax = s[j];
            if (m[j] > mmax) mmax = m[j];
        }
        uint16_t dh = f32_to_f16_bits(smax / 63.0f), dmh = f32_to_f16_bits(mmax / 63.0f);
        float d = f16_bits_to_f32(dh), dmin = f16_bits_to_f32(dmh);
        uint8_t sc[8], mq[8];
        for (int j = 0; j < 8; j++) {
            int a = d > 0.f ? (int)lrintf(s[j] / d) : 0;
            int c = dmin > 0.f ? (int)lrintf(m[j] / dmin) : 0;
            sc[j] = (uint8_t)(a < 0 ? 0 : a > 63 ? 63 : a);
            mq[j] = (uint8_t)(c < 0 ? 0 : c > 63 ? 63 : c);
        }
        memcpy(blk, &dh, 2);
        memcpy(blk + 2, &dmh, 2);
        uint8_t *sb = blk + 4;
        memset(sb, 0, 12);
        for (int j = 0; j < 4; j++) {
            sb[j] = (uint8_t)((sc[j] & 63) | ((sc[j + 4] >> 4) << 6));
            sb[j + 4] = (uint8_t)((mq[j] & 63) | ((mq[j + 4] >> 4) << 6));
            sb[j + 8] = (uint8_t)((sc[j + 4] & 0x0F) | ((mq[j + 4] & 0x0F) << 4));
        }
        uint8_t *qs = blk + 16;
        memset(qs, 0, 128);
        for (int j = 0; j < 8; j++) {
            float ds = d * (float)sc[j], dm = dmin * (float)mq[j];
            for (int l = 0; l < 32; l++) {
                int q = 0;
                if (ds > 0.f) {
                    q = (int)lrintf((xb[j * 32 + l] + dm) / ds);
                    q = q < 0 ? 0 : q > 15 ? 15 : q;
                }
                if (j & 1) qs[32 * (j / 2) + l] |= (uint8_t)(q << 4);
                else qs[32 * (j / 2) + l] |= (uint8_t)q;
            }
        }
    }
}

/* ---------------------------------------------------------------- GELU */

/* unary.rs:75-76,97-119: x*(0.5+0.5*safe_tanh(x*(0.035677407*x*x+0.7978846))),
 * safe_tanh(x) = sign(x) if |x| >= 10 else tanh(x); evaluated in f32. */
static inline float gelu_f32(float v) {
    float t = v * (0.035677407f * (v * v) + 0.7978846f);
    float th = fabsf(t) >= 10.0f ? (t > 0.f ? 1.0f : (t < 0.f ? -1.0f : 0.0f)) : tanhf(t);
    return v * (0.5f + 0.5f * th);
}

static inline double gelu_f64(double v) {
    double t = v * (0.035677407 * (v * v) + 0.7978846);
    double th = fabs(t) >= 10.0 ? (t > 0 ? 1.0 : (t < 0 ? -1.0 : 0.0)) : tanh(t);
    return v * (0.5 + 0.5 * th);
}

void orc_gelu_f32(const float *x, float *y, int64_t n) {
    for (int64_t i = 0; i < n; i++) y[i] = gelu_f32(x[i]);
}

/* ---------------------------------------------------------------- matmul */

/* Operand conventions (gemm.rs:359-361, 395-447, 466-489; matmul.rs:284-361):
 *   A: [a_stack][M][K], or [a_stack][K][M] when trans_a
 *   B: [b_stack][K][N], or [b_stack][N][K] when trans_b
 *   out: [stacks][M][N], or [stacks][N][M] when trans_out
 *   batch b reads A[b % a_stack], B[b % b_stack]
 *   bias index: column n, or row m when trans_out (gemm.rs:468-476)
 * A and B are given as f32 arrays holding the exact operand values (f16 and
 * dequantised values are exactly representable in f32). */

static inline int64_t a_index(int64_t m, int64_t k, int64_t M, int64_t K, int trans_a) {
    return trans_a ? k * M + m : m * K + k;
}
static inline int64_t b_index(int64_t k, int64_t n, int64_t K, int64_t N, int trans_b) {
    return trans_b ? n * K + k : k * N + n;
}

/* epilogue: 0 none, 1 tanh-GELU */
void orc_matmul_truth(const float *A, const float *B, const float *bias, double *out,
                      int64_t stacks, int64_t a_stack, int64_t b_stack,
                      int64_t M, int64_t N, int64_t K,
                      int trans_a, int trans_b, int trans_out, int epilogue) {
#pragma omp parallel for collapse(2) schedule(static)
    for (int64_t b = 0; b < stacks; b++) {
        for (int64_t m = 0; m < M; m++) {
            const float *Ab = A + (b % a_stack) * M * K;
            const float *Bb = B + (b % b_stack) * K * N;
            double *Ob = out + b * M * N;
            for (int64_t n = 0; n < N; n++) {
                double acc = 0.0;
                for (int64_t k = 0; k < K; k++)
                    acc += (double)Ab[a_index(m, k, M, K, trans_a)] *
                           (double)Bb[b_index(k, n, K, N, trans_b)];
                if (bias) acc += (double)bias[trans_out ? m : n];
                if (epilogue == 1) acc = gelu_f64(acc);
                Ob[trans_out ? n * M + m : m * N + n] = acc;
            }
        }
    }
}

/* Shader-faithful oracle.  act_dt: 0 = f32, 1 = f16.
 * f16: product rounded to f16 (gemm.rs:441-444), accumulated in f32 in K order,
 * val = f16(acc) + bias in f16 (gemm.rs:485); with epilogue 1 the chain is
 * f16 -> f32 -> GELU in f32 -> f16 (crates/ratchet-models/src/whisper/mlp.rs:18-22).
 * Output is f32-valued (exact f16 values on the f16 path). */
void orc_matmul_faithful(const float *A, const float *B, const float *bias, float *out,
                         int64_t stacks, int64_t a_stack, int64_t b_stack,
                         int64_t M, int64_t N, int64_t K,
                         int trans_a, int trans_b, int trans_out, int epilogue, int act_dt) {
#pragma omp parallel for collapse(2) schedule(static)
    for (int64_t b = 0; b < stacks; b++) {
        for (int64_t m = 0; m < M; m++) {
            const float *Ab = A + (b % a_stack) * M * K;
            const float *Bb = B + (b % b_stack) * K * N;
            float *Ob = out + b * M * N;
            for (int64_t n = 0; n < N; n++) {
                float acc = 0.0f;
                if (act_dt == 1) {
                    for (int64_t k = 0; k < K; k++) {
                        float p = Ab[a_index(m, k, M, K, trans_a)] * Bb[b_index(k, n, K, N, trans_b)];
                        acc += round_f16(p);
                    }
                } else {
                    for (int64_t k = 0; k < K; k++) {
                        volatile float p = Ab[a_index(m, k, M, K, trans_a)] * Bb[b_index(k, n, K, N, trans_b)];
                        acc += p;
                    }
                }
                float v;
                if (act_dt == 1) {
                    v = round_f16(acc);
                    if (bias) v = round_f16(v + bias[trans_out ? m : n]);
                    if (epilogue == 1) v = round_f16(gelu_f32(v));
                } else {
                    v = acc;
                    if (bias) v = v + bias[trans_out ? m : n];
                    if (epilogue == 1) v = gelu_f32(v);
                }
                Ob[trans_out ? n * M + m : m * N + n] = v;
            }
        }
    }
}

/* Shader-faithful GEMV (gemv.rs:492-553): 32 lanes, lane l accumulates K elements
 * 4l..4l+3 of every 128-wide step in its own f32 partial, then the partials are summed
 * (subgroupAdd; order unspecified by WGSL, summed here lane 0..31), then dt(acc)+bias[row].
 * W: [N][K] values (dequantised), x: [K].  act_dt as above. */
void orc_gemv_faithful(const float *W, const float *x, const float *bias, float *out,
                       int64_t N, int64_t K, int act_dt) {
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < N; r++) {
        float part[32];
        for (int l = 0; l < 32; l++) part[l] = 0.f;
        for (int64_t k0 = 0; k0 < K; k0 += 128) {
            for (int l = 0; l < 32; l++) {
                for (int t = 0; t < 4; t++) {
                    int64_t k = k0 + 4 * l + t;
                    if (k >= K) continue;
                    float p = W[r * K + k] * x[k];
                    part[l] += (act_dt == 1) ? round_f16(p) : p;
                }
            }
        }
        float acc = 0.f;
        for (int l = 0; l < 32; l++) acc += part[l];
        float v = (act_dt == 1) ? round_f16(acc) : acc;
        if (bias) v = (act_dt == 1) ? round_f16(v + bias[r]) : v + bias[r];
        out[r] = v;
    }
}

/* ---------------------------------------------------------------- timed CPU baselines
 * Same arithmetic as the faithful oracles, but reading the packed weights directly and
 * blocked for throughput; used only as the benchmark's CPU baseline. */

/* Q8_0H GEMV: y[r] = f16( sum_k f16( f16(q*d) * x[k] ) ) + bias  */
void orc_q8h_gemv_packed(const uint8_t *wbuf, int64_t N, int64_t K, const uint16_t *x16,
                         const uint16_t *bias16, uint16_t *y16) {
    int64_t seg[4];
    orc_q8_segments(N * K, 2, seg);
    const int8_t *qs = (const int8_t *)wbuf;
    const uint16_t *ds = (const uint16_t *)(wbuf + seg[2]);
    float *xf = (float *)malloc(sizeof(float) * (size_t)K);
    for (int64_t k = 0; k < K; k++) xf[k] = f16_bits_to_f32(x16[k]);
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < N; r++) {
        float acc = 0.f;
        const int8_t *q = qs + r * K;
        const uint16_t *d = ds + r * (K / QK8_0);
        for (int64_t kb = 0; kb < K / QK8_0; kb++) {
            f16_t dv;
            memcpy(&dv, &d[kb], 2);
            for (int j = 0; j < QK8_0; j++) {
                f16_t w = (f16_t)((float)q[kb * QK8_0 + j] * (float)dv);
                acc += (float)(f16_t)((float)w * xf[kb * QK8_0 + j]);
            }
        }
        f16_t v = (f16_t)acc;
        if (bias16) {
            f16_t bv;
            memcpy(&bv, &bias16[r], 2);
            v = (f16_t)((float)v + (float)bv);
        }
        memcpy(&y16[r], &v, 2);
    }
    free(xf);
}

/* The launcher of a multi-process run may export OMP_NUM_THREADS=1; the timed baseline sets its own count. */
void orc_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

int orc_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
