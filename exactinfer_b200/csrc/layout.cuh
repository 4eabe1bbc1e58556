// Index arithmetic of the tiled weight layouts (described in common.cuh), usable from host and device code:
// the permutation file layout -> tiled layout, one output byte at a time, and the element access that decodes a
// value back out of a tile. The host versions exist so that the permutation can be checked without a GPU.
#pragma once

#include "common.cuh"

namespace elb {

#ifdef __CUDA_ARCH__
#define ELB_FMUL(a, b) __fmul_rn(a, b)
#define ELB_FSUB(a, b) __fsub_rn(a, b)
#else
#define ELB_FMUL(a, b) ((a) * (b))
#define ELB_FSUB(a, b) ((a) - (b))
#endif
#define ELB_HD __host__ __device__ __forceinline__

ELB_HD float h2f16(uint32_t h16) { return __half2float(__ushort_as_half((unsigned short)h16)); }

// source row (in the uploaded bytes) of tiled row R; -1 when R is padding. Paired weights (gate then up, `rows`
// counting both) put gate rows 8T..8T+7 in rows 0..7 of tile T and the matching up rows in rows 8..15.
ELB_HD int64_t src_row(int64_t R, int64_t rows, bool pair) {
    if (!pair) return R < rows ? R : -1;
    const int64_t half_rows = rows / 2, T = R / 16, rr = R % 16;
    const int64_t r = 8 * T + (rr & 7);
    if (r >= half_rows) return -1;
    return rr < 8 ? r : half_rows + r;
}

// low 4 bits and high 2 bits of value k (0..255) of a Q6_K block in file layout (src/quant.cpp:35-60 of the reference)
ELB_HD int q6k_lo(const uint8_t* blk, int k) {
    const int h = k >> 7, kk = k & 127, grp = kk >> 5, l = kk & 31;
    const uint8_t b = blk[64 * h + 32 * (grp & 1) + l];
    return grp >= 2 ? b >> 4 : b & 0xF;
}
ELB_HD int q6k_hi(const uint8_t* blk, int k) {
    const int h = k >> 7, kk = k & 127, grp = kk >> 5, l = kk & 31;
    return (blk[128 + 32 * h + l] >> (2 * grp)) & 3;
}

// byte o of the tiled Q4_K weight (nb = 256-blocks per row)
ELB_HD uint8_t tile_byte_q4k(const uint8_t* src, int64_t o, int64_t rows, int64_t nb, bool pair) {
    const int64_t unit = o / Q4K_UNIT, T = unit / nb, b = unit % nb;
    const int w = int(o % Q4K_UNIT);
    int rr, byte;
    if (w < 256) {
        rr = w / 32 + 8 * ((w % 32) / 16);
        byte = w % 16;
    } else {
        const int v = w - 256, j = v / 512, lane = (v % 512) / 16, q = v % 16;
        rr = lane / 4 + 8 * (q / 8);
        byte = 16 + 32 * j + 8 * (lane % 4) + q % 8;
    }
    const int64_t r = src_row(16 * T + rr, rows, pair);
    return r < 0 ? uint8_t(0) : src[(r * nb + b) * Q4_K_BYTES + byte];
}

// byte o of the tiled Q8_0 weight (nb32 = 32-blocks per row, a multiple of 4)
ELB_HD uint8_t tile_byte_q8(const uint8_t* src, int64_t o, int64_t rows, int64_t nb32, bool pair) {
    const int64_t upt = nb32 / Q8_GROUP, unit = o / Q8_UNIT, T = unit / upt, u = unit % upt;
    const int w = int(o % Q8_UNIT);
    int rr, blk, byte;
    if (w < 128) {
        const int g = w / 16, q = w % 16;
        rr = g + 8 * (q / 8);
        blk = (q % 8) / 2;
        byte = q % 2;
    } else {
        const int v = w - 128, lane = (v % 512) / 16, q = v % 16;
        blk = v / 512;
        rr = lane / 4 + 8 * (q / 8);
        byte = 2 + 8 * (lane % 4) + q % 8;
    }
    const int64_t r = src_row(16 * T + rr, rows, pair);
    return r < 0 ? uint8_t(0) : src[(r * nb32 + u * Q8_GROUP + blk) * Q8_0_BYTES + byte];
}

// byte o of the tiled Q6_K weight
ELB_HD uint8_t tile_byte_q6k(const uint8_t* src, int64_t o, int64_t rows, int64_t nb, bool pair) {
    const int64_t unit = o / Q6K_UNIT, T = unit / nb, b = unit % nb;
    const int w = int(o % Q6K_UNIT);
    uint8_t out = 0;
    if (w < 32) {
        const int idx = w / 2, rr = idx / 2 + 8 * (idx % 2);
        const int64_t r = src_row(16 * T + rr, rows, pair);
        if (r >= 0) out = src[(r * nb + b) * Q6_K_BYTES + 208 + w % 2];
    } else if (w < 288) {
        const int v = w - 32, rr = v / 32 + 8 * ((v % 32) / 16);
        const int64_t r = src_row(16 * T + rr, rows, pair);
        if (r >= 0) out = src[(r * nb + b) * Q6_K_BYTES + 192 + v % 16];
    } else if (w < 2336) {
        const int v = w - 288, c = v / 512, lane = (v % 512) / 16, q = v % 16, i = q / 4, j = q % 4;
        const int g = lane / 4, t = lane % 4, k = 16 * (4 * c + i) + 4 * t + j;
        const int64_t r0 = src_row(16 * T + g, rows, pair), r1 = src_row(16 * T + g + 8, rows, pair);
        const int lo = r0 < 0 ? 0 : q6k_lo(src + (r0 * nb + b) * Q6_K_BYTES, k);
        const int hi = r1 < 0 ? 0 : q6k_lo(src + (r1 * nb + b) * Q6_K_BYTES, k);
        out = uint8_t(lo | (hi << 4));
    } else {
        const int v = w - 2336, c = v / 256, lane = (v % 256) / 8, q = v % 8, half = q / 4, j = q % 4;
        const int g = lane / 4, t = lane % 4;
        const int64_t r = src_row(16 * T + g + 8 * half, rows, pair);
        if (r >= 0) {
            const uint8_t* blk = src + (r * nb + b) * Q6_K_BYTES;
            for (int i = 0; i < 4; ++i) out |= uint8_t(q6k_hi(blk, 16 * (4 * c + i) + 4 * t + j) << (2 * i));
        }
    }
    return out;
}

struct QElem {
    int q;       // integer part: Q4_K 0..15, Q6_K -32..31, Q8_0 -128..127
    int sc;      // integer sub-block scale (Q8_0: 1)
    int mn;      // Q4_K 6-bit min (else 0)
    float d;     // block scale
    float dmin;  // Q4_K
};

// element (tiled row R, column k) of a quantized weight in tiled layout
ELB_HD QElem tiled_elem(int type, const uint8_t* tiled, int64_t n, int64_t R, int64_t k) {
    QElem e{0, 1, 0, 0.f, 0.f};
    const int64_t T = R / 16;
    const int rr = int(R % 16), g = rr & 7, half = rr >> 3;
    if (type == ELB_Q4_K) {
        const int64_t nb = n / QK_K, b = k / QK_K;
        const int kk = int(k % QK_K), sub = kk / 32, idx = kk % 32, t = idx / 8, byte = idx % 8;
        const uint8_t* u = tiled + (T * nb + b) * Q4K_UNIT;
        const uint8_t* hdr = u + g * 32 + half * 16;
        e.d = h2f16(hdr[0] | (hdr[1] << 8));
        e.dmin = h2f16(hdr[2] | (hdr[3] << 8));
        q4k_scale_min(sub, hdr + 4, e.sc, e.mn);
        const uint8_t v = u[256 + (sub / 2) * 512 + (4 * g + t) * 16 + half * 8 + byte];
        e.q = (sub & 1) ? v >> 4 : v & 0xF;
    } else if (type == ELB_Q6_K) {
        const int64_t nb = n / QK_K, b = k / QK_K;
        const int kk = int(k % QK_K), s = kk / 16, c = s / 4, i = s % 4, idx = kk % 16, t = idx / 4, j = idx % 4;
        const uint8_t* u = tiled + (T * nb + b) * Q6K_UNIT;
        const uint8_t* dp = u + (2 * g + half) * 2;
        e.d = h2f16(dp[0] | (dp[1] << 8));
        e.sc = reinterpret_cast<const int8_t*>(u + 32 + g * 32 + half * 16)[s];
        const uint8_t lo = u[288 + c * 512 + (4 * g + t) * 16 + i * 4 + j];
        const uint8_t hi = u[2336 + c * 256 + (4 * g + t) * 8 + half * 4 + j];
        e.q = int((half ? lo >> 4 : lo & 0xF) | (((hi >> (2 * i)) & 3) << 4)) - 32;
    } else {  // Q8_0
        const int64_t upt = n / (QK8_0 * Q8_GROUP), blk = k / QK8_0, un = blk / Q8_GROUP;
        const int i = int(blk % Q8_GROUP), idx = int(k % QK8_0), t = idx / 8, byte = idx % 8;
        const uint8_t* u = tiled + (T * upt + un) * Q8_UNIT;
        const uint8_t* dp = u + g * 16 + half * 8 + i * 2;
        e.d = h2f16(dp[0] | (dp[1] << 8));
        e.q = reinterpret_cast<const int8_t*>(u)[128 + i * 512 + (4 * g + t) * 16 + half * 8 + byte];
    }
    return e;
}

// fp32 value with the reference decoders' operation order (src/quant.cpp:7-60 of the reference)
ELB_HD float elem_value(int type, const QElem& e) {
    if (type == ELB_Q4_K) {
        const float d1 = ELB_FMUL(e.d, float(e.sc)), m1 = ELB_FMUL(e.dmin, float(e.mn));
        return ELB_FSUB(ELB_FMUL(d1, float(e.q)), m1);
    }
    if (type == ELB_Q6_K) return ELB_FMUL(ELB_FMUL(e.d, float(e.sc)), float(e.q));
    return ELB_FMUL(float(e.q), e.d);
}

}  // namespace elb
