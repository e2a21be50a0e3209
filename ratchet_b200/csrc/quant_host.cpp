// Host-side block formats: layouts, Q8_0 quantiser / dequantiser, GGUF transcode, Q4_K codec.
// Restates crates/ratchet-core/src/quant.rs:26-124, crates/ratchet-core/src/dtype/blocks.rs:61-74,
// crates/ratchet-core/src/gpu/align.rs:23-40 and crates/ratchet-loader/src/gguf/dtype.rs:44-110.
// In the reference these run on the CPU as well (weights are quantised / transcoded on the host
// and uploaded once), so this is the product's host code, not a fallback for a device kernel.
#include <cmath>
#include <cstring>

#include "half_host.hpp"
#include "spec.hpp"

namespace rt {

static inline uint64_t align_up(uint64_t n, uint64_t a) { return (n + a - 1) / a * a; }

Status dtype_segments(rt_dtype dt, uint64_t numel, rt_segment *segs, int *n) {
    switch (dt) {
    case RT_Q8_0H:
    case RT_Q8_0F: {
        if (numel % 32 != 0) return Status::Err(RT_ERR_SHAPE, "Q8_0 tensors hold a multiple of 32 values");
        uint64_t sb = dt == RT_Q8_0H ? 2 : 4;
        segs[0] = {0, align_up(numel, 256)};                 // blocks.rs:66-67
        segs[1] = {segs[0].size, align_up(numel / 32 * sb, 256)}; // blocks.rs:68-71
        *n = 2;
        return Status::Ok();
    }
    case RT_Q4_K:
        if (numel % 256 != 0) return Status::Err(RT_ERR_SHAPE, "Q4_K tensors hold a multiple of 256 values");
        segs[0] = {0, numel / 256 * 144};
        *n = 1;
        return Status::Ok();
    default: {
        uint64_t bytes = numel * dtype_size(dt);
        if (bytes < 16) bytes = 16;                           // MIN_STORAGE_BUFFER_SIZE (dtype/mod.rs:90)
        segs[0] = {0, align_up(bytes, 4)};                    // align_for_copy
        *n = 1;
        return Status::Ok();
    }
    }
}

// Rust `f32 as i32`: NaN -> 0, saturating.
static inline int32_t f32_as_i32(float v) {
    if (std::isnan(v)) return 0;
    if (v >= 2147483648.0f) return INT32_MAX;
    if (v <= -2147483648.0f) return INT32_MIN;
    return (int32_t)v;
}

// quant.rs:26-79
Status quantize_q8_0(const float *x, uint64_t numel, rt_dtype dt, uint8_t *out) {
    rt_segment seg[2];
    int n;
    Status st = dtype_segments(dt, numel, seg, &n);
    if (!st.ok()) return st;
    std::memset(out, 0, seg[0].size + seg[1].size);
    float d = -INFINITY;
    for (uint64_t i = 0; i < numel; i += 4) {
        if (i % 32 == 0) {
            float amax = -INFINITY;
            for (int j = 0; j < 32; j++) {
                float a = std::fabs(x[i + j]);
                if (a > amax) amax = a; // f32::max drops NaN operands; NaN > amax is false
            }
            d = amax / 127.0f;
            if (dt == RT_Q8_0H) {
                uint16_t h = f32_to_f16(d);
                std::memcpy(out + seg[1].offset + (i / 32) * 2, &h, 2);
            } else {
                std::memcpy(out + seg[1].offset + (i / 32) * 4, &d, 4);
            }
        }
        for (int j = 0; j < 4; j++) {
            int32_t q = f32_as_i32(std::round(x[i + j] / d)) & 0xFF; // f32::round: half away from zero
            out[i + j] = (uint8_t)q;
        }
    }
    return Status::Ok();
}

// quant.rs:81-124; the f16 form is the shaders' f16(q) * d (gemm.rs:400-406).
Status dequantize_q8_0(const uint8_t *src, uint64_t numel, rt_dtype dt, float *out) {
    rt_segment seg[2];
    int n;
    Status st = dtype_segments(dt, numel, seg, &n);
    if (!st.ok()) return st;
    const int8_t *qs = (const int8_t *)src;
    for (uint64_t i = 0; i < numel; i++) {
        if (dt == RT_Q8_0H) {
            uint16_t h;
            std::memcpy(&h, src + seg[1].offset + (i / 32) * 2, 2);
            float v = (float)qs[i] * f16_to_f32(h); // exact in f32
            out[i] = f16_to_f32(f32_to_f16(v));     // one rounding to f16
        } else {
            float d;
            std::memcpy(&d, src + seg[1].offset + (i / 32) * 4, 4);
            out[i] = (float)qs[i] * d;
        }
    }
    return Status::Ok();
}

// gguf/dtype.rs:44-73 (f32 scales) and 80-109 (f16 scales)
Status transcode_gguf_q8_0(const uint8_t *blocks, uint64_t n_blocks, rt_dtype dt, uint8_t *out) {
    rt_segment seg[2];
    int n;
    Status st = dtype_segments(dt, n_blocks * 32, seg, &n);
    if (!st.ok()) return st;
    std::memset(out, 0, seg[0].size + seg[1].size);
    for (uint64_t b = 0; b < n_blocks; b++) {
        const uint8_t *blk = blocks + b * 34;
        uint16_t d;
        std::memcpy(&d, blk, 2);
        std::memcpy(out + b * 32, blk + 2, 32);
        if (dt == RT_Q8_0H) {
            std::memcpy(out + seg[1].offset + b * 2, &d, 2);
        } else {
            float f = f16_to_f32(d);
            std::memcpy(out + seg[1].offset + b * 4, &f, 4);
        }
    }
    return Status::Ok();
}

// Q4_K super-block: {f16 d; f16 dmin; u8 scales[12]; u8 qs[128]} (k_quants.rs:95-103).
static inline void q4k_scale_min(int j, const uint8_t *s, uint8_t *sc, uint8_t *m) {
    if (j < 4) {
        *sc = s[j] & 63;
        *m = s[j + 4] & 63;
    } else {
        *sc = (uint8_t)((s[j + 4] & 0x0F) | ((s[j - 4] >> 6) << 4));
        *m = (uint8_t)((s[j + 4] >> 4) | ((s[j] >> 6) << 4));
    }
}

// value = (d*sc)*q - (dmin*m), each operation rounded to f32 on its own
Status dequantize_q4_k(const uint8_t *src, uint64_t numel, float *out) {
    if (numel % 256 != 0) return Status::Err(RT_ERR_SHAPE, "Q4_K tensors hold a multiple of 256 values");
    for (uint64_t b = 0; b < numel / 256; b++) {
        const uint8_t *blk = src + b * 144;
        uint16_t dh, dmh;
        std::memcpy(&dh, blk, 2);
        std::memcpy(&dmh, blk + 2, 2);
        float d = f16_to_f32(dh), dmin = f16_to_f32(dmh);
        for (int j = 0; j < 8; j++) {
            uint8_t sc, m;
            q4k_scale_min(j, blk + 4, &sc, &m);
            volatile float ds = d * (float)sc;
            volatile float dm = dmin * (float)m;
            const uint8_t *q = blk + 16 + 32 * (j / 2);
            for (int l = 0; l < 32; l++) {
                int code = (j & 1) ? (q[l] >> 4) : (q[l] & 0x0F);
                volatile float p = ds * (float)code;
                out[b * 256 + j * 32 + l] = p - dm;
            }
        }
    }
    return Status::Ok();
}

// Encoder: per sub-block affine fit x ~ s*q - m (q in 0..15, m >= 0), 6-bit s and m against the
// super-block's f16 d = max s / 63 and dmin = max m / 63.
Status quantize_q4_k(const float *x, uint64_t numel, uint8_t *out) {
    if (numel % 256 != 0) return Status::Err(RT_ERR_SHAPE, "Q4_K tensors hold a multiple of 256 values");
    for (uint64_t b = 0; b < numel / 256; b++) {
        const float *xb = x + b * 256;
        uint8_t *blk = out + b * 144;
        float s[8], m[8], smax = 0.f, mmax = 0.f;
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
        uint16_t dh = f32_to_f16(smax / 63.0f), dmh = f32_to_f16(mmax / 63.0f);
        float d = f16_to_f32(dh), dmin = f16_to_f32(dmh);
        uint8_t sc[8], mq[8];
        for (int j = 0; j < 8; j++) {
            long a = d > 0.f ? std::lrintf(s[j] / d) : 0;
            long c = dmin > 0.f ? std::lrintf(m[j] / dmin) : 0;
            sc[j] = (uint8_t)(a < 0 ? 0 : a > 63 ? 63 : a);
            mq[j] = (uint8_t)(c < 0 ? 0 : c > 63 ? 63 : c);
        }
        std::memcpy(blk, &dh, 2);
        std::memcpy(blk + 2, &dmh, 2);
        uint8_t *sb = blk + 4;
        for (int j = 0; j < 4; j++) {
            sb[j] = (uint8_t)((sc[j] & 63) | ((sc[j + 4] >> 4) << 6));
            sb[j + 4] = (uint8_t)((mq[j] & 63) | ((mq[j + 4] >> 4) << 6));
            sb[j + 8] = (uint8_t)((sc[j + 4] & 0x0F) | ((mq[j + 4] & 0x0F) << 4));
        }
        uint8_t *qs = blk + 16;
        std::memset(qs, 0, 128);
        for (int j = 0; j < 8; j++) {
            float ds = d * (float)sc[j], dm = dmin * (float)mq[j];
            for (int l = 0; l < 32; l++) {
                long q = 0;
                if (ds > 0.f) {
                    q = std::lrintf((xb[j * 32 + l] + dm) / ds);
                    q = q < 0 ? 0 : q > 15 ? 15 : q;
                }
                qs[32 * (j / 2) + l] |= (uint8_t)((j & 1) ? (q << 4) : q);
            }
        }
    }
    return Status::Ok();
}

} // namespace rt
