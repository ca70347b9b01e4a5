/*
 * kq_oracle.c -- CPU restatement of Kernelcore's quantized-LLM arithmetic.
 *
 * TEST INFRASTRUCTURE ONLY (see kq_oracle.h).  Build with -ffp-contract=off:
 * the reference's mirror rounds every fp32 product before the next add, and a
 * fused multiply-add would change the bits.
 *
 * Citations "ref:" are into llm/llm_reference.cpp of the reference project.
 */
#include "kq_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

/* ---- small helpers ------------------------------------------------------- */

static uint16_t ld16(const uint8_t* p) { return (uint16_t)(p[0] | (p[1] << 8)); }
static int32_t ld32(const uint8_t* p) {
    int32_t v;
    memcpy(&v, p, 4);
    return v;
}
static int32_t asr(int32_t v, int s) { return v >> s; }                              /* arithmetic shift */
static int32_t lsl(int32_t v, int s) { return (int32_t)((uint32_t)v << s); }         /* no UB */
static int32_t sbyte(int32_t w, int i) { return asr(lsl(w, 24 - 8 * i), 24); }       /* signed byte i */

/* u8 x s8 four-way dot product, the reference's dp4a (ref:106-112). */
static int32_t dot4_u8s8(int32_t a, int32_t b, int32_t c) {
    for (int i = 0; i < 4; ++i) c += ((a >> (8 * i)) & 255) * (int8_t)((uint32_t)b >> (8 * i));
    return c;
}

/* ---- fp16 conversions ------------------------------------------------------ */

/* ref:284-309 -- exact widening, subnormals renormalised, inf/nan kept. */
float kqo_f16_to_f32(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    const uint32_t ex = (h >> 10) & 0x1Fu, man = h & 0x3FFu;
    uint32_t bits;
    if (ex == 0) {
        if (man == 0) {
            bits = sign;
        } else {
            uint32_t m = man;
            int e = -1;
            do {
                ++e;
                m <<= 1;
            } while (!(m & 0x400u));
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((m & 0x3FFu) << 13);
        }
    } else if (ex == 31) {
        bits = sign | 0x7F800000u | (man << 13);
    } else {
        bits = sign | ((ex + 112u) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* ref:730-739 -- round to nearest even by float arithmetic; >= 65520 saturates to
 * 0x7bff and -0 becomes +0 (both are the kernel's documented deviations from IEEE). */
uint16_t kqo_f32_to_f16(float x) {
    const uint32_t sign = x < 0.0f ? 0x8000u : 0u;
    const float a = fabsf(x);
    if (!(a < 65520.0f)) return (uint16_t)(sign | 0x7bffu);
    if (a < 6.103515625e-05f) return (uint16_t)(sign | (uint32_t)nearbyintf(a * 16777216.0f));
    int e = 0;
    const float f = frexpf(a, &e);
    const uint32_t m = (uint32_t)nearbyintf((f * 2.0f - 1.0f) * 1024.0f);
    return (uint16_t)(sign | (((uint32_t)(e - 1 + 15) << 10) + m));
}

/* ---- GGUF K-quant dequantisation ------------------------------------------- */

/* ref:329-337 -- the j-th 6-bit scale and min of a Q4_K super-block's 12 packed bytes. */
static void q4k_scale_min(int j, const uint8_t* p, int* sc, int* mn) {
    if (j < 4) {
        *sc = p[j] & 63;
        *mn = p[j + 4] & 63;
    } else {
        *sc = (p[j + 4] & 0xF) | ((p[j - 4] >> 6) << 4);
        *mn = (p[j + 4] >> 4) | ((p[j] >> 6) << 4);
    }
}

/* ref:342-359 -- w = (d*sc)*q - (dmin*m), each product rounded on its own. */
void kqo_dequant_row_q4k(const uint8_t* src, int k, float* out) {
    for (int s = 0; s < k / 256; ++s) {
        const uint8_t* blk = src + (size_t)s * 144;
        const float d = kqo_f16_to_f32(ld16(blk)), dmin = kqo_f16_to_f32(ld16(blk + 2));
        const uint8_t* packed = blk + 4;
        const uint8_t* qs = blk + 16;
        float* y = out + (size_t)s * 256;
        for (int c = 0; c < 4; ++c) {
            int sc, mn;
            q4k_scale_min(2 * c, packed, &sc, &mn);
            const float dl = d * (float)sc, ml = dmin * (float)mn;
            q4k_scale_min(2 * c + 1, packed, &sc, &mn);
            const float dh = d * (float)sc, mh = dmin * (float)mn;
            for (int l = 0; l < 32; ++l) y[64 * c + l] = dl * (float)(qs[32 * c + l] & 0xF) - ml;
            for (int l = 0; l < 32; ++l) y[64 * c + 32 + l] = dh * (float)(qs[32 * c + l] >> 4) - mh;
        }
    }
}

/* ref:361-383 -- w = d*float(sc)*float(q6-32), multiplied left to right. */
void kqo_dequant_row_q6k(const uint8_t* src, int k, float* out) {
    for (int s = 0; s < k / 256; ++s) {
        const uint8_t* blk = src + (size_t)s * 210;
        const uint8_t *ql = blk, *qh = blk + 128;
        const int8_t* sc = (const int8_t*)(blk + 192);
        const float d = kqo_f16_to_f32(ld16(blk + 208));
        float* y = out + (size_t)s * 256;
        for (int n = 0; n < 2; ++n)
            for (int l = 0; l < 32; ++l) {
                const int is = l / 16;
                const int h = qh[32 * n + l];
                const int q1 = (int)((ql[64 * n + l] & 0xF) | (((h >> 0) & 3) << 4)) - 32;
                const int q2 = (int)((ql[64 * n + l + 32] & 0xF) | (((h >> 2) & 3) << 4)) - 32;
                const int q3 = (int)((ql[64 * n + l] >> 4) | (((h >> 4) & 3) << 4)) - 32;
                const int q4 = (int)((ql[64 * n + l + 32] >> 4) | (((h >> 6) & 3) << 4)) - 32;
                y[128 * n + l] = d * (float)sc[8 * n + is + 0] * (float)q1;
                y[128 * n + l + 32] = d * (float)sc[8 * n + is + 2] * (float)q2;
                y[128 * n + l + 64] = d * (float)sc[8 * n + is + 4] * (float)q3;
                y[128 * n + l + 96] = d * (float)sc[8 * n + is + 6] * (float)q4;
            }
    }
}

/* ---- activation quantizers -------------------------------------------------- */

static float absmax_run(const float* x, int n) { /* max as "a > b ? a : b" (ref:83-87) */
    float amax = 0.0f;
    for (int i = 0; i < n; ++i) {
        const float a = x[i] > 0.0f - x[i] ? x[i] : 0.0f - x[i];
        amax = amax > a ? amax : a;
    }
    return amax;
}
static int round_clamp(float t) { /* half away from zero, clamp to +-127 (ref:95-96) */
    int q = t >= 0.0f ? (int)(t + 0.5f) : (int)(t - 0.5f);
    return q > 127 ? 127 : q < -127 ? -127 : q;
}

/* ref:79-104 -- per 32 values: d = amax/127, 8 packed words, {d, float(sum q)}. */
void kqo_quantize_q8x4(const float* x, int32_t* xq, float* xd, int count) {
    for (int b = 0; b < count; ++b) {
        const float* xb = x + (size_t)b * 32;
        const float d = absmax_run(xb, 32) / 127.0f;
        const float id = d > 0.0f ? 1.0f / d : 0.0f;
        int sum = 0;
        for (int w = 0; w < 8; ++w) {
            uint32_t word = 0;
            for (int i = 0; i < 4; ++i) {
                const int q = round_clamp(xb[w * 4 + i] * id);
                sum += q;
                word |= ((uint32_t)q & 255u) << (8 * i);
            }
            xq[(size_t)b * 8 + w] = (int32_t)word;
        }
        xd[(size_t)b * 2] = d;
        xd[(size_t)b * 2 + 1] = (float)sum;
    }
}

/* ref:491-527 -- one scale per 256; slot = [64 nsb words | nsb f32 | 16 nsb sums of 16 |
 * 4 nsb words holding the sums of 32 split into bytes (B >> 6, then B & 63)]. */
void kqo_quantize_q8k(const float* x, int32_t* q, int nsb) {
    float* scale = (float*)(q + (size_t)nsb * 64);
    int32_t* sum16 = q + (size_t)nsb * 65;
    for (int s = 0; s < nsb; ++s) {
        const float* xs = x + (size_t)s * 256;
        const float d = absmax_run(xs, 256) / 127.0f;
        const float id = d > 0.0f ? 1.0f / d : 0.0f;
        for (int g = 0; g < 16; ++g) {
            int sum = 0;
            for (int w = 0; w < 4; ++w) {
                uint32_t word = 0;
                for (int i = 0; i < 4; ++i) {
                    const int v = round_clamp(xs[g * 16 + w * 4 + i] * id);
                    sum += v;
                    word |= ((uint32_t)v & 255u) << (8 * i);
                }
                q[(size_t)s * 64 + g * 4 + w] = (int32_t)word;
            }
            sum16[(size_t)s * 16 + g] = sum;
        }
        scale[s] = d;
        uint32_t pw[4] = {0, 0, 0, 0};
        for (int i = 0; i < 8; ++i) {
            const int b = sum16[(size_t)s * 16 + 2 * i] + sum16[(size_t)s * 16 + 2 * i + 1];
            pw[i / 4] |= ((uint32_t)asr(b, 6) & 255u) << (8 * (i % 4));
            pw[2 + i / 4] |= (uint32_t)(b & 63) << (8 * (i % 4));
        }
        for (int i = 0; i < 4; ++i) q[(size_t)nsb * 81 + (size_t)s * 4 + i] = (int32_t)pw[i];
    }
}

/* ---- K-quant matvecs on Q8 activations -------------------------------------- */

/* The 8 scales and 8 mins of a Q4_K block as four words of bytes (ref:422-425). */
static void q4k_scale_words(const uint8_t* blk, int32_t* sclo, int32_t* schi, int32_t* mlo, int32_t* mhi) {
    const int32_t s0 = ld32(blk + 4), s1 = ld32(blk + 8), s2 = ld32(blk + 12);
    *sclo = s0 & 0x3F3F3F3F;
    *mlo = s1 & 0x3F3F3F3F;
    *schi = (s2 & 0x0F0F0F0F) | (asr(s0, 2) & 0x30303030);
    *mhi = (asr(s2, 4) & 0x0F0F0F0F) | (asr(s1, 2) & 0x30303030);
}

/* ref:413-445 */
void kqo_matvec_q4k_q8(const uint8_t* w, const int32_t* xq, const float* xd, float* y, int rows, int k) {
    const int nsb = k / 256;
    for (int row = 0; row < rows; ++row) {
        float acc = 0.0f;
        for (int s = 0; s < nsb; ++s) {
            const uint8_t* blk = w + ((size_t)row * nsb + s) * 144;
            const float d = kqo_f16_to_f32(ld16(blk)), dmin = kqo_f16_to_f32(ld16(blk + 2));
            int32_t sclo, schi, mlo, mhi;
            q4k_scale_words(blk, &sclo, &schi, &mlo, &mhi);
            float fd = 0.0f, fm = 0.0f;
            for (int j = 0; j < 4; ++j) {
                const int b = s * 8 + j * 2;
                int32_t da = 0, db = 0;
                for (int t = 0; t < 8; ++t) {
                    const int32_t q = ld32(blk + 16 + 4 * (j * 8 + t));
                    da = dot4_u8s8(q & 0x0F0F0F0F, xq[b * 8 + t], da);
                    db = dot4_u8s8(asr(q, 4) & 0x0F0F0F0F, xq[b * 8 + 8 + t], db);
                }
                const int sh = 16 * (j & 1);
                const int32_t scw = j < 2 ? sclo : schi, mw = j < 2 ? mlo : mhi;
                const int sca = asr(scw, sh) & 255, scb = asr(scw, sh + 8) & 255;
                const int ma = asr(mw, sh) & 255, mb = asr(mw, sh + 8) & 255;
                fd += (float)(sca * da) * xd[b * 2] + (float)(scb * db) * xd[b * 2 + 2];
                fm += (float)ma * (xd[b * 2] * xd[b * 2 + 1]) + (float)mb * (xd[b * 2 + 2] * xd[b * 2 + 3]);
            }
            acc += d * fd - dmin * fm;
        }
        y[row] = acc;
    }
}

/* ref:447-489 */
void kqo_matvec_q6k_q8(const uint8_t* w, const int32_t* xq, const float* xd, float* y, int rows, int k) {
    const int nsb = k / 256;
    for (int row = 0; row < rows; ++row) {
        float acc = 0.0f;
        for (int s = 0; s < nsb; ++s) {
            const uint8_t* blk = w + ((size_t)row * nsb + s) * 210;
            const float d = kqo_f16_to_f32(ld16(blk + 208));
            for (int n = 0; n < 2; ++n) {
                const int b = s * 8 + n * 4;
                int32_t da[4] = {0, 0, 0, 0}, db[4] = {0, 0, 0, 0}, sa[4] = {0, 0, 0, 0};
                for (int t8 = 0; t8 < 8; ++t8) {
                    const int32_t qa = ld32(blk + 4 * (16 * n + t8)), qc = ld32(blk + 4 * (16 * n + 8 + t8));
                    const int32_t h = ld32(blk + 128 + 4 * (8 * n + t8));
                    const int32_t q[4] = {(qa & 0x0F0F0F0F) | (lsl(h, 4) & 0x30303030),
                                          (qc & 0x0F0F0F0F) | (lsl(h, 2) & 0x30303030),
                                          (asr(qa, 4) & 0x0F0F0F0F) | (h & 0x30303030),
                                          (asr(qc, 4) & 0x0F0F0F0F) | (asr(h, 2) & 0x30303030)};
                    for (int t = 0; t < 4; ++t) {
                        const int32_t xw = xq[b * 8 + 8 * t + t8];
                        if (t8 < 4) {
                            da[t] = dot4_u8s8(q[t], xw, da[t]);
                            sa[t] = dot4_u8s8(0x01010101, xw, sa[t]);
                        } else {
                            db[t] = dot4_u8s8(q[t], xw, db[t]);
                        }
                    }
                }
                const int32_t sw0 = ld32(blk + 192 + 8 * n), sw1 = ld32(blk + 196 + 8 * n);
                int32_t is[4];
                for (int t = 0; t < 4; ++t) {
                    const int32_t sw = t < 2 ? sw0 : sw1;
                    const int lo = 2 * (t & 1);
                    const int32_t sb = (int32_t)xd[(b + t) * 2 + 1] - sa[t];
                    is[t] = sbyte(sw, lo) * (da[t] - 32 * sa[t]) + sbyte(sw, lo + 1) * (db[t] - 32 * sb);
                }
                acc += d * ((float)is[0] * xd[b * 2] + (float)is[1] * xd[b * 2 + 2] + (float)is[2] * xd[b * 2 + 4] +
                            (float)is[3] * xd[b * 2 + 6]);
            }
        }
        y[row] = acc;
    }
}

/* ref:529-562 -- integer accumulation over a whole super-block, one fp step per 256. */
void kqo_matvec_q4k_q8k(const uint8_t* w, const int32_t* xq, float* y, int rows, int k) {
    const int nsb = k / 256;
    const float* xd = (const float*)(xq + (size_t)nsb * 64);
    const int32_t* bs = xq + (size_t)nsb * 65;
    for (int row = 0; row < rows; ++row) {
        float acc = 0.0f;
        for (int s = 0; s < nsb; ++s) {
            const uint8_t* blk = w + ((size_t)row * nsb + s) * 144;
            const float d = kqo_f16_to_f32(ld16(blk)), dmin = kqo_f16_to_f32(ld16(blk + 2));
            int32_t sclo, schi, mlo, mhi;
            q4k_scale_words(blk, &sclo, &schi, &mlo, &mhi);
            int32_t is = 0, im = 0;
            for (int j = 0; j < 4; ++j) {
                const int32_t* xs = xq + (size_t)s * 64 + j * 16;
                int32_t da = 0, db = 0;
                for (int t = 0; t < 8; ++t) {
                    const int32_t q = ld32(blk + 16 + 4 * (j * 8 + t));
                    da = dot4_u8s8(q & 0x0F0F0F0F, xs[t], da);
                    db = dot4_u8s8(asr(q, 4) & 0x0F0F0F0F, xs[8 + t], db);
                }
                const int sh = 16 * (j & 1);
                const int32_t scw = j < 2 ? sclo : schi, mw = j < 2 ? mlo : mhi;
                is += (asr(scw, sh) & 255) * da + (asr(scw, sh + 8) & 255) * db;
                const int32_t* b = bs + (size_t)s * 16 + j * 4;
                im += (asr(mw, sh) & 255) * (b[0] + b[1]) + (asr(mw, sh + 8) & 255) * (b[2] + b[3]);
            }
            acc += (d * xd[s]) * (float)is - (dmin * xd[s]) * (float)im;
        }
        y[row] = acc;
    }
}

/* ref:564-596 */
void kqo_matvec_q6k_q8k(const uint8_t* w, const int32_t* xq, float* y, int rows, int k) {
    const int nsb = k / 256;
    const float* xd = (const float*)(xq + (size_t)nsb * 64);
    const int32_t* bs = xq + (size_t)nsb * 65;
    for (int row = 0; row < rows; ++row) {
        float acc = 0.0f;
        for (int s = 0; s < nsb; ++s) {
            const uint8_t* blk = w + ((size_t)row * nsb + s) * 210;
            const float d = kqo_f16_to_f32(ld16(blk + 208));
            int32_t is = 0;
            for (int n = 0; n < 2; ++n)
                for (int t = 0; t < 4; ++t) {
                    const int32_t* xs = xq + (size_t)s * 64 + (n * 4 + t) * 8;
                    int32_t da = 0, db = 0;
                    for (int t8 = 0; t8 < 8; ++t8) {
                        const int32_t qa = ld32(blk + 4 * (16 * n + 8 * (t & 1) + t8));
                        const int32_t h = ld32(blk + 128 + 4 * (8 * n + t8));
                        const int32_t q = (asr(qa, 4 * (t >> 1)) & 0x0F0F0F0F) | (lsl(asr(h, 2 * t), 4) & 0x30303030);
                        if (t8 < 4) da = dot4_u8s8(q, xs[t8], da);
                        else db = dot4_u8s8(q, xs[t8], db);
                    }
                    const int32_t sw = ld32(blk + 192 + 4 * (2 * n + (t >> 1)));
                    const int lo = 2 * (t & 1);
                    const int32_t* b = bs + (size_t)s * 16 + (n * 4 + t) * 2;
                    is += sbyte(sw, lo) * (da - 32 * b[0]) + sbyte(sw, lo + 1) * (db - 32 * b[1]);
                }
            acc += (d * xd[s]) * (float)is;
        }
        y[row] = acc;
    }
}

/* tests/test_llm_kernels.cpp:228-236 -- the "dequantized floats" product. */
void kqo_matvec_dequant_f64(const uint8_t* w, const float* x, float* y, int rows, int k, int q6) {
    float* row = (float*)malloc((size_t)k * sizeof(float));
    const size_t row_bytes = (size_t)(k / 256) * (q6 ? 210 : 144);
    for (int r = 0; r < rows; ++r) {
        if (q6) kqo_dequant_row_q6k(w + (size_t)r * row_bytes, k, row);
        else kqo_dequant_row_q4k(w + (size_t)r * row_bytes, k, row);
        double s = 0;
        for (int i = 0; i < k; ++i) s += (double)row[i] * x[i];
        y[r] = (float)s;
    }
    free(row);
}

/* ---- glue --------------------------------------------------------------------- */

/* ref:153-162 -- y = x * r * w with r = 1/sqrt(mean(x^2) + eps); two multiplies in that order. */
void kqo_rms_norm(const float* x, const float* w, float* y, int n, int rows, float eps) {
    for (int row = 0; row < rows; ++row) {
        const float* xr = x + (size_t)row * n;
        float* yr = y + (size_t)row * n;
        float ss = 0.0f;
        for (int j = 0; j < n; ++j) ss += xr[j] * xr[j];
        const float r = 1.0f / sqrtf(ss / (float)n + eps);
        for (int j = 0; j < n; ++j) yr[j] = xr[j] * r * w[j];
    }
}

void kqo_add(float* x, const float* t, int n) { /* ref:232-234 */
    for (int i = 0; i < n; ++i) x[i] = x[i] + t[i];
}

void kqo_add_rms_norm(float* x, const float* t, const float* w, float* y, int n, float eps) { /* ref:240-243 */
    kqo_add(x, t, n);
    kqo_rms_norm(x, w, y, n, 1, eps);
}

/* ref:255-267 -- x += t; per-32 partial sums of squares go to q[nb*10 ..]. */
void kqo_add_sumsq(float* x, const float* t, int32_t* q, int nb) {
    float* ss = (float*)(q + nb * 10);
    for (int b = 0; b < nb; ++b) {
        float s = 0.0f;
        for (int i = 0; i < 32; ++i) {
            const float v = x[b * 32 + i] + t[b * 32 + i];
            x[b * 32 + i] = v;
            s += v * v;
        }
        ss[b] = s;
    }
}

/* ref:269-276 -- partial sums added in block order, then norm * w quantized per 32. */
void kqo_norm_q8x4(const float* x, const float* w, int32_t* q, int nb, float eps) {
    const float* ss = (const float*)(q + nb * 10);
    float tot = 0.0f;
    for (int j = 0; j < nb; ++j) tot += ss[j];
    const float r = 1.0f / sqrtf(tot / (float)(nb * 32) + eps);
    float* h = (float*)malloc((size_t)nb * 32 * sizeof(float));
    for (int i = 0; i < nb * 32; ++i) h[i] = x[i] * r * w[i];
    kqo_quantize_q8x4(h, q, (float*)(q + nb * 8), nb);
    free(h);
}

/* The reference evaluates sin/cos of (theta * 1/(2 pi)) * 2 pi in float, a quirk of its
 * kernel compiler that the mirror reproduces (ref:168-174). */
static void rot(float theta, float* a, float* b, float x0, float x1) {
    const float turns = theta * 0.159154943f;
    const float c = cosf(turns * 6.28318548f), s = sinf(turns * 6.28318548f);
    *a = x0 * c - x1 * s;
    *b = x0 * s + x1 * c;
}

void kqo_rope(float* x, int pairs_per_head, int pos, int count, float log2_base) { /* ref:164-180 */
    for (int idx = 0; idx < count; ++idx) {
        const int i = idx % pairs_per_head;
        const float theta = (float)pos * exp2f(-(float)i / (float)pairs_per_head * log2_base);
        rot(theta, &x[2 * idx], &x[2 * idx + 1], x[2 * idx], x[2 * idx + 1]);
    }
}

void kqo_rope_ff(float* x, const float* ff, int pairs_per_head, int pos, int count, float log2_base) { /* ref:598-610 */
    for (int idx = 0; idx < count; ++idx) {
        const int i = idx % pairs_per_head;
        const float theta = (float)pos * exp2f(-(float)i / (float)pairs_per_head * log2_base) / ff[i];
        rot(theta, &x[2 * idx], &x[2 * idx + 1], x[2 * idx], x[2 * idx + 1]);
    }
}

/* ref:620-635 -- per-token positions; NORM pairs (2i, 2i+1) or NEOX pairs (i, i + D/2). */
void kqo_rope_ggml(const float* x, float* y, const int32_t* pos, const float* ff, int head_dim, int n_head,
                   int n_tokens, float log2_base, int neox) {
    const int pairs = head_dim / 2, count = pairs * n_head * n_tokens;
    for (int idx = 0; idx < count; ++idx) {
        const int t = idx / (pairs * n_head), i = idx % pairs;
        const float theta = (float)pos[t] * exp2f(-(float)i / (float)pairs * log2_base) / ff[i];
        const int head = idx / pairs;
        const int a = neox ? head * head_dim + i : 2 * idx, b = neox ? a + pairs : a + 1;
        rot(theta, &y[a], &y[b], x[a], x[b]);
    }
}

void kqo_append_kv(const float* k, const float* v, float* kt, float* vc, int n, int k_stride, int pos) { /* ref:182-187 */
    for (int j = 0; j < n; ++j) {
        kt[(size_t)j * k_stride + pos] = k[j];
        vc[(size_t)pos * n + j] = v[j];
    }
}

void kqo_attn_scores(const float* q, const float* kt, float* scores, const kqo_attn_dims* d, float scale) { /* ref:189-199 */
    for (int h = 0; h < d->n_heads; ++h) {
        const float* qh = q + (size_t)h * d->head_dim;
        const size_t kb = (size_t)(h / d->group) * d->head_dim;
        for (int t = 0; t < d->ctx; ++t) {
            float s = 0.0f;
            for (int i = 0; i < d->head_dim; ++i) s += qh[i] * kt[(kb + i) * d->k_stride + t];
            scores[(size_t)h * d->ctx_pad + t] = s * scale;
        }
    }
}

void kqo_softmax(float* x, int n, int stride, int rows) { /* ref:201-215 */
    for (int row = 0; row < rows; ++row) {
        float* xr = x + (size_t)row * stride;
        float m = xr[0];
        for (int j = 1; j < n; ++j) m = m < xr[j] ? xr[j] : m;
        float sum = 0.0f;
        for (int j = 0; j < n; ++j) {
            const float e = exp2f((xr[j] - m) * 1.44269504f);
            xr[j] = e;
            sum += e;
        }
        const float inv = 1.0f / sum;
        for (int j = 0; j < n; ++j) xr[j] = xr[j] * inv;
    }
}

void kqo_attn_values(const float* p, const float* v, float* out, const kqo_attn_dims* d) { /* ref:217-226 */
    for (int h = 0; h < d->n_heads; ++h)
        for (int i = 0; i < d->head_dim; ++i) {
            const size_t vo = (size_t)(h / d->group) * d->head_dim + i;
            float s = 0.0f;
            for (int t = 0; t < d->ctx; ++t) s += p[(size_t)h * d->ctx_pad + t] * v[(size_t)t * d->kv_stride + vo];
            out[(size_t)h * d->head_dim + i] = s;
        }
}

static float swiglu1(float g, float u) { return g / (1.0f + exp2f(-g * 1.44269504f)) * u; } /* ref:228-230 */

void kqo_silu_mul(const float* g, const float* u, float* out, int count) {
    for (int i = 0; i < count; ++i) out[i] = swiglu1(g[i], u[i]);
}

void kqo_silu_mul_q8x4(const float* g, const float* u, int32_t* xq, float* xd, int count) { /* ref:245-249 */
    float* h = (float*)malloc((size_t)count * 32 * sizeof(float));
    kqo_silu_mul(g, u, h, count * 32);
    kqo_quantize_q8x4(h, xq, xd, count);
    free(h);
}

void kqo_mul_rows(const float* x, const float* w, float* y, int n, int count) { /* ref:616-618 */
    for (int i = 0; i < count; ++i) y[i] = x[i] * w[i % n];
}

/* One block of 32 quantized into row slot qr (ref:641-650). */
static void quantize_block_into(const float* y, int32_t* qr, int nb, int bl) {
    int32_t words[8];
    float xd[2];
    kqo_quantize_q8x4(y, words, xd, 1);
    for (int i = 0; i < 8; ++i) qr[bl * 8 + i] = words[i];
    float* d = (float*)(qr + nb * 8);
    d[bl * 2] = xd[0];
    d[bl * 2 + 1] = xd[1];
}

void kqo_add_sumsq_f(const float* a, const float* b, float* out, int32_t* q, int n, int rows) { /* ref:653-668 */
    const int nb = n / 32;
    for (int row = 0; row < rows; ++row) {
        float* ss = (float*)(q + (size_t)row * nb * 11 + nb * 10);
        for (int bl = 0; bl < nb; ++bl) {
            float s = 0.0f;
            for (int i = 0; i < 32; ++i) {
                const size_t o = (size_t)row * n + (size_t)bl * 32 + i;
                const float v = a[o] + b[o];
                out[o] = v;
                s += v * v;
            }
            ss[bl] = s;
        }
    }
}

void kqo_sumsq_part(const float* x, int32_t* q, int n, int rows) { /* ref:670-683 */
    const int nb = n / 32;
    for (int row = 0; row < rows; ++row) {
        float* ss = (float*)(q + (size_t)row * nb * 11 + nb * 10);
        for (int bl = 0; bl < nb; ++bl) {
            float s = 0.0f;
            for (int i = 0; i < 32; ++i) {
                const float v = x[(size_t)row * n + (size_t)bl * 32 + i];
                s += v * v;
            }
            ss[bl] = s;
        }
    }
}

static float row_rinv(const float* ss, int nb, int n, float eps) {
    float tot = 0.0f;
    for (int j = 0; j < nb; ++j) tot += ss[j];
    return 1.0f / sqrtf(tot / (float)n + eps);
}

void kqo_norm_mul_q8(const float* x, const float* w, float* y, int32_t* q, int n, int rows, float eps) { /* ref:685-701 */
    const int nb = n / 32;
    for (int row = 0; row < rows; ++row) {
        int32_t* qr = q + (size_t)row * nb * 11;
        const float r = row_rinv((const float*)(qr + nb * 10), nb, n, eps);
        for (int bl = 0; bl < nb; ++bl) {
            float* yb = y + (size_t)row * n + (size_t)bl * 32;
            const float* xb = x + (size_t)row * n + (size_t)bl * 32;
            for (int i = 0; i < 32; ++i) yb[i] = xb[i] * r * w[bl * 32 + i];
            quantize_block_into(yb, qr, nb, bl);
        }
    }
}

void kqo_norm_mul_q8k(const float* x, const float* w, float* y, int32_t* q, const int32_t* sq, int n, int rows,
                      float eps) { /* ref:703-712 */
    const int nb = n / 32;
    for (int row = 0; row < rows; ++row) {
        const float r = row_rinv((const float*)(sq + (size_t)row * nb * 11 + nb * 10), nb, n, eps);
        for (int i = 0; i < n; ++i) y[(size_t)row * n + i] = x[(size_t)row * n + i] * r * w[i];
        kqo_quantize_q8k(y + (size_t)row * n, q + (size_t)row * (n / 256 * 85), n / 256);
    }
}

void kqo_silu_mul_q8k(const float* g, const float* u, float* y, int32_t* q, int n, int cols) { /* ref:713-716 */
    for (size_t i = 0; i < (size_t)n * cols; ++i) y[i] = swiglu1(g[i], u[i]);
    for (int c = 0; c < cols; ++c) kqo_quantize_q8k(y + (size_t)c * n, q + (size_t)c * (n / 256 * 85), n / 256);
}

void kqo_silu_mul_q8f(const float* g, const float* u, float* y, int32_t* q, int n, int cols) { /* ref:717-727 */
    const int nb = n / 32;
    for (int c = 0; c < cols; ++c) {
        int32_t* qc = q + (size_t)c * nb * 11;
        for (int bl = 0; bl < nb; ++bl) {
            const size_t o = (size_t)c * n + (size_t)bl * 32;
            for (int i = 0; i < 32; ++i) y[o + i] = swiglu1(g[o + i], u[o + i]);
            quantize_block_into(y + o, qc, nb, bl);
        }
    }
}

/* ---- fp16 KV-cache path ------------------------------------------------------- */

/* ref:765-772 -- row index read as the low 32 bits of an int64; out-of-range rows skipped. */
void kqo_set_rows_f16(const float* src, const int64_t* idx, uint16_t* dst, int pairs, int rows, int src_row,
                      int dst_row, int dst_rows) {
    for (int r = 0; r < rows; ++r) {
        const int row = (int)idx[r];
        if (row < 0 || row >= dst_rows) continue;
        for (int j = 0; j < 2 * pairs; ++j)
            dst[(size_t)row * dst_row * 2 + j] = kqo_f32_to_f16(src[(size_t)r * src_row + j]);
    }
}

/* ref:773-798 -- strides of K, V and mask are in 32-bit words (two fp16). */
void kqo_flash_attn_f16(const float* q, const uint16_t* k, const uint16_t* v, const uint16_t* mask, float* out,
                        const kqo_fa_dims* d, float scale) {
    float* s = (float*)malloc((size_t)d->T * sizeof(float));
    for (int i = 0; i < d->N; ++i)
        for (int h = 0; h < d->H; ++h) {
            const int kvh = h / d->group;
            const float* qh = q + (size_t)i * d->q_tok + (size_t)h * d->q_head;
            float mx = -INFINITY;
            for (int t = 0; t < d->T; ++t) {
                const uint16_t* kr = k + ((size_t)t * d->k_row + (size_t)kvh * d->k_head) * 2;
                float a = 0.0f;
                for (int j = 0; j < d->D; ++j) a += qh[j] * kqo_f16_to_f32(kr[j]);
                const float mv = d->has_mask ? kqo_f16_to_f32(mask[(size_t)i * d->m_row * 2 + t]) : 0.0f;
                s[t] = a * scale + mv;
                mx = mx < s[t] ? s[t] : mx;
            }
            float sum = 0.0f;
            for (int t = 0; t < d->T; ++t) sum += (s[t] = exp2f((s[t] - mx) * 1.44269504f));
            for (int dd = 0; dd < d->D; ++dd) {
                float a = 0.0f;
                for (int t = 0; t < d->T; ++t)
                    a += s[t] * kqo_f16_to_f32(v[((size_t)t * d->v_row + (size_t)kvh * d->v_head) * 2 + dd]);
                out[((size_t)i * d->H + h) * d->D + dd] = a / sum;
            }
        }
    free(s);
}

/* ---- synthetic 8-bit / 4-bit formats of the reference's own benchmark models and fp16 weights --------- */

/* ref:10-23 -- int8 weights [rows][k], one float scale per 32. */
void kqo_matvec_q8w(const int8_t* q, const float* scales, const float* x, float* y, int rows, int k) {
    const int nb = k / 32;
    for (int row = 0; row < rows; ++row) {
        float acc = 0.0f;
        for (int b = 0; b < nb; ++b) {
            float s = 0.0f;
            for (int j = 0; j < 32; ++j) s += (float)q[(size_t)row * k + (size_t)b * 32 + j] * x[(size_t)b * 32 + j];
            acc += s * scales[(size_t)row * nb + b];
        }
        y[row] = acc;
    }
}

/* ref:25-42 -- 4-bit weights, ggml Q4_0 nibble order with a float scale: byte j of a block holds weight j
 * (low nibble) and j + 16 (high), each biased by 8. */
void kqo_matvec_q4w(const uint8_t* qs, const float* scales, const float* x, float* y, int rows, int k) {
    const int nb = k / 32;
    for (int row = 0; row < rows; ++row) {
        float acc = 0.0f;
        for (int b = 0; b < nb; ++b) {
            float s = 0.0f;
            const uint8_t* qb = qs + (size_t)row * (k / 2) + (size_t)b * 16;
            for (int j = 0; j < 16; ++j) {
                s += (float)((qb[j] & 15) - 8) * x[(size_t)b * 32 + j];
                s += (float)((qb[j] >> 4) - 8) * x[(size_t)b * 32 + j + 16];
            }
            acc += s * scales[(size_t)row * nb + b];
        }
        y[row] = acc;
    }
}

/* ref:66-77 -- the same blocks interleaved over groups of 8 rows: byte j of row l of block (g, b) at
 * qs8[((g*nb + b)*16 + j)*8 + l], its scale at scales8[(g*nb + b)*8 + l]. */
void kqo_repack_q4x8(const uint8_t* qs, const float* scales, uint8_t* qs8, float* scales8, int rows, int k) {
    const int nb = k / 32;
    for (int row = 0; row < rows; ++row)
        for (int b = 0; b < nb; ++b) {
            const size_t blk = (size_t)(row / 8) * nb + b;
            for (int j = 0; j < 16; ++j) qs8[(blk * 16 + j) * 8 + row % 8] = qs[(size_t)row * (k / 2) + (size_t)b * 16 + j];
            scales8[blk * 8 + row % 8] = scales[(size_t)row * nb + b];
        }
}

/* ref:44-64 -- four partial sums per block, combined as (s0 + s2) + (s1 + s3). */
void kqo_matvec_q4x8(const uint8_t* qs8, const float* scales8, const float* x, float* y, int rows, int k) {
    const int nb = k / 32;
    for (int row = 0; row < rows; ++row) {
        float acc = 0.0f;
        for (int b = 0; b < nb; ++b) {
            const size_t blk = (size_t)(row / 8) * nb + b;
            const uint8_t* qb = qs8 + blk * 128 + row % 8;
            const float* xb = x + (size_t)b * 32;
            float s0 = 0.0f, s1 = 0.0f, s2 = 0.0f, s3 = 0.0f;
            for (int j = 0; j < 16; j += 2) {
                const int v0 = qb[j * 8], v1 = qb[j * 8 + 8];
                s0 += (float)((v0 & 15) - 8) * xb[j];
                s1 += (float)((v0 >> 4) - 8) * xb[j + 16];
                s2 += (float)((v1 & 15) - 8) * xb[j + 1];
                s3 += (float)((v1 >> 4) - 8) * xb[j + 17];
            }
            acc += ((s0 + s2) + (s1 + s3)) * scales8[blk * 8 + row % 8];
        }
        y[row] = acc;
    }
}

/* ref:137-152 -- 40 words per (8-row group, block): 4 x 8 quant words (word w of row l at [w*8 + l]), then the
 * 8 float scales. */
void kqo_repack_q4x8_q8(const uint8_t* qs, const float* scales, int32_t* qw, int rows, int k) {
    const int nb = k / 32;
    for (int row = 0; row < rows; ++row)
        for (int b = 0; b < nb; ++b) {
            int32_t* blk = qw + ((size_t)(row / 8) * nb + b) * 40;
            const uint8_t* src = qs + (size_t)row * (k / 2) + (size_t)b * 16;
            for (int w = 0; w < 4; ++w) blk[w * 8 + row % 8] = ld32(src + 4 * w);
            memcpy(blk + 32 + row % 8, &scales[(size_t)row * nb + b], 4);
        }
}

/* ref:114-135 -- integer dot against Q8 activations; the +8 bias leaves through the activation sum. */
void kqo_matvec_q4x8_q8(const int32_t* qw, const int32_t* xq, const float* xd, float* y, int rows, int k) {
    const int nb = k / 32;
    for (int row = 0; row < rows; ++row) {
        float acc = 0.0f;
        for (int b = 0; b < nb; ++b) {
            const int32_t* blk = qw + ((size_t)(row / 8) * nb + b) * 40;
            int32_t lo = 0, hi = 0;
            for (int w = 0; w < 4; ++w) {
                const int32_t q = blk[w * 8 + row % 8];
                lo = dot4_u8s8(q & 0x0F0F0F0F, xq[(size_t)b * 8 + w], lo);
                hi = dot4_u8s8(asr(q, 4) & 0x0F0F0F0F, xq[(size_t)b * 8 + 4 + w], hi);
            }
            float sc;
            memcpy(&sc, blk + 32 + row % 8, 4);
            const int32_t dot = lo + hi - 8 * (int32_t)xd[(size_t)b * 2 + 1];
            acc += (float)dot * (sc * xd[(size_t)b * 2]);
        }
        y[row] = acc;
    }
}

/* ref:740-746 -- fp16 weights as 32-bit words (two halves), interleaved over groups of 8 rows. */
void kqo_repack_f16(const uint16_t* w, int rows, int k, int32_t* out) {
    const int kw = k / 2;
    for (int r = 0; r < rows; ++r)
        for (int j = 0; j < kw; ++j)
            out[((size_t)(r / 8) * kw + j) * 8 + r % 8] =
                (int32_t)((uint32_t)w[(size_t)r * k + 2 * j] | ((uint32_t)w[(size_t)r * k + 2 * j + 1] << 16));
}

/* ref:756-764 -- Y[c*rows + r] = sum over pairs of (w0 x0 + w1 x1), on the row-major fp16 matrix. */
void kqo_matmul_f16(const uint16_t* w, const float* x, float* y, int rows, int k, int ncols) {
    for (int c = 0; c < ncols; ++c)
        for (int r = 0; r < rows; ++r) {
            float a = 0.0f;
            for (int j = 0; j < k; j += 2)
                a += kqo_f16_to_f32(w[(size_t)r * k + j]) * x[(size_t)c * k + j] +
                     kqo_f16_to_f32(w[(size_t)r * k + j + 1]) * x[(size_t)c * k + j + 1];
            y[(size_t)c * rows + r] = a;
        }
}

/* ---- decode step ---------------------------------------------------------------- */

static int pad8(int n) { return (n + 7) / 8 * 8; }
static int imax(int a, int b) { return a > b ? a : b; }

long kqo_decode_scratch_floats(const kqo_model* m) {
    const int qd = m->heads * m->head_dim, kv = m->kv_heads * m->head_dim;
    return 3L * m->hidden + (qd + 2L * kv) + (long)m->heads * pad8(m->max_ctx) + qd + 3L * m->inter;
}
long kqo_decode_scratch_ints(const kqo_model* m) {
    return 11L * (imax(imax(m->hidden, m->inter), m->heads * m->head_dim) / 32);
}

/* Test instrumentation for the decode loop below (no counterpart in the reference).  Every time the loop quantizes an
 * activation vector -- per layer the inputs of q|k|v, wo, gate|up and down, then the lm_head's input -- its int8 words
 * (k / 4 of them) are (1) appended to the trace buffer, when one is set, and (2) when forced words are set, compared
 * with the forced words at the same offset (count of differing int8 values, of vectors holding one, largest step) and
 * then REPLACED by them.  The residual stream is traced the same way after each of the two additions of a layer (hidden
 * floats, as their bit patterns; compared by the largest difference relative to the largest magnitude).  With both
 * forced, every stage is checked on the inputs the other implementation really had, and a value that rounded the other
 * way cannot cascade into the stages after it.  Order of a step's trace: layer 0's q|k|v words, then per layer: wo
 * words, residual, gate|up words, down words, residual, the next layer's q|k|v words (after the last: the lm_head's). */
static int32_t* g_trace;
static const int32_t* g_forced;
static long g_trace_cap, g_trace_len, g_forced_len, g_diff_values, g_diff_vectors;
static int g_diff_max;
static float g_diff_x;
void kqo_decode_set_trace(int32_t* buf, long cap_words) { g_trace = buf, g_trace_cap = cap_words, g_trace_len = 0; }
long kqo_decode_trace_words(void) { return g_trace_len; }
void kqo_decode_set_forced(const int32_t* words, long n_words) { g_forced = words, g_forced_len = n_words; }
void kqo_decode_forced_stats(long* values, long* vectors, int* max_step, float* residual_rel) {
    *values = g_diff_values, *vectors = g_diff_vectors, *max_step = g_diff_max, *residual_rel = g_diff_x;
}
static void trace_q8(int32_t* xq, int k) {
    if (g_trace && g_trace_len + k / 4 <= g_trace_cap) memcpy(g_trace + g_trace_len, xq, (size_t)(k / 4) * sizeof(int32_t));
    if (g_forced && g_trace_len + k / 4 <= g_forced_len) {
        const int8_t* own = (const int8_t*)xq;
        const int8_t* other = (const int8_t*)(g_forced + g_trace_len);
        long n = 0;
        for (int i = 0; i < k; ++i) {
            const int d = abs((int)own[i] - (int)other[i]);
            n += d != 0;
            if (d > g_diff_max) g_diff_max = d;
        }
        g_diff_values += n;
        g_diff_vectors += n != 0;
        memcpy(xq, other, (size_t)k);
    }
    g_trace_len += k / 4;
}
static void trace_f32(float* x, int n) {
    if (g_trace && g_trace_len + n <= g_trace_cap) memcpy(g_trace + g_trace_len, x, (size_t)n * sizeof(float));
    if (g_forced && g_trace_len + n <= g_forced_len) {
        const float* other = (const float*)(g_forced + g_trace_len);
        float big = 0.0f, diff = 0.0f;
        for (int i = 0; i < n; ++i) {
            big = fmaxf(big, fabsf(x[i]));
            diff = fmaxf(diff, fabsf(x[i] - other[i]));
        }
        if (big > 0.0f && diff / big > g_diff_x) g_diff_x = diff / big;
        memcpy(x, other, (size_t)n * sizeof(float));
    }
    g_trace_len += n;
}

static void mv_q(const kqo_mat* w, const int32_t* xq, float* y) { /* CppBackend::matvecQuantized, llm_model.cpp:531-537 */
    const float* xd = (const float*)(xq + (w->k / 32) * 8);
    if (w->fmt == 6) kqo_matvec_q6k_q8(w->blocks, xq, xd, y, w->rows, w->k);
    else kqo_matvec_q4k_q8(w->blocks, xq, xd, y, w->rows, w->k);
}
static void mv_f(const kqo_mat* w, const float* x, int32_t* xq, float* y) { /* CppBackend::matvec, :510-516 */
    kqo_quantize_q8x4(x, xq, (float*)(xq + (w->k / 32) * 8), w->k / 32);
    trace_q8(xq, w->k);
    mv_q(w, xq, y);
}

/* llm/llm_model.cpp:287-360 for a model with quantized activations and split q/k/v, gate/up.
 * flags (extensions used by the GPU decoder's tests; 0 = the reference's loop exactly):
 *   1  K and V are rounded to fp16 as they enter the cache (the ggml path's fp16 cache: setRowsF16 ref:765-772),
 *   2  NEOX RoPE pairing (ropeGgml ref:620-635), 4  per-head RMSNorm of q and k before RoPE (rmsNorm ref:153-162
 *      on rows of head_dim, as ggml-kernelcore.cpp:757-767 runs it for Qwen3). */
void kqo_decode_token_ex(const kqo_model* m, const float* x_in, int pos, float* logits, float* sf, int32_t* xq, int flags) {
    const int hid = m->hidden, qd = m->heads * m->head_dim, kv = m->kv_heads * m->head_dim;
    const int ctx = pos + 1;
    const kqo_attn_dims ad = {m->heads, ctx, m->head_dim, kv, m->heads / m->kv_heads, pad8(ctx), pad8(m->max_ctx)};
    float* x = sf;
    float* xn = x + hid;
    float* t = xn + hid;
    float* q = t + hid;
    float* kk = q + qd;
    float* vv = kk + kv;
    float* scores = vv + kv;
    float* attn = scores + (size_t)m->heads * pad8(m->max_ctx);
    float* g = attn + qd;
    float* u = g + m->inter;
    const float lb = log2f(m->rope_base);
    const float scale = 1.0f / sqrtf((float)m->head_dim);
    const int pairs = m->head_dim / 2;

    g_trace_len = 0, g_diff_values = 0, g_diff_vectors = 0, g_diff_max = 0, g_diff_x = 0.0f;
    memcpy(x, x_in, (size_t)hid * sizeof(float));
    kqo_rms_norm(x, m->layers[0].attn_norm, xn, hid, 1, m->eps);
    for (int l = 0; l < m->n_layers; ++l) {
        const kqo_layer* L = &m->layers[l];
        if (l == 0) mv_f(&L->wq, xn, xq, q); /* later layers: the previous norm already quantized */
        else mv_q(&L->wq, xq, q);
        mv_q(&L->wk, xq, kk);
        mv_q(&L->wv, xq, vv);
        if (flags & 4) {
            kqo_rms_norm(q, L->q_norm, q, m->head_dim, m->heads, m->eps);
            kqo_rms_norm(kk, L->k_norm, kk, m->head_dim, m->kv_heads, m->eps);
        }
        if (flags & 2) {
            float* ones = (float*)malloc((size_t)pairs * sizeof(float));
            float* tmp = (float*)malloc((size_t)(qd + kv) * sizeof(float));
            for (int i = 0; i < pairs; ++i) ones[i] = 1.0f;
            const int32_t p1 = pos;
            kqo_rope_ggml(q, tmp, &p1, m->rope_ff ? m->rope_ff : ones, m->head_dim, m->heads + m->kv_heads, 1, lb, 1);
            memcpy(q, tmp, (size_t)(qd + kv) * sizeof(float));
            free(ones);
            free(tmp);
        } else if (m->rope_ff) kqo_rope_ff(q, m->rope_ff, pairs, pos, (m->heads + m->kv_heads) * pairs, lb);
        else kqo_rope(q, pairs, pos, (m->heads + m->kv_heads) * pairs, lb);
        if (flags & 1)
            for (int j = 0; j < kv; ++j) {
                kk[j] = kqo_f16_to_f32(kqo_f32_to_f16(kk[j]));
                vv[j] = kqo_f16_to_f32(kqo_f32_to_f16(vv[j]));
            }
        kqo_append_kv(kk, vv, L->k_cache, L->v_cache, kv, pad8(m->max_ctx), pos);
        kqo_attn_scores(q, L->k_cache, scores, &ad, scale);
        kqo_softmax(scores, ctx, pad8(ctx), m->heads);
        kqo_attn_values(scores, L->v_cache, attn, &ad);
        mv_f(&L->wo, attn, xq, t);
        kqo_add_sumsq(x, t, xq, hid / 32);
        if (g_forced) { /* the sums of squares belong to the replaced values */
            trace_f32(x, hid);
            memset(t, 0, (size_t)hid * sizeof(float));
            kqo_add_sumsq(x, t, xq, hid / 32);
        } else trace_f32(x, hid);
        kqo_norm_q8x4(x, L->ffn_norm, xq, hid / 32, m->eps);
        trace_q8(xq, hid);
        mv_q(&L->wg, xq, g);
        mv_q(&L->wu, xq, u);
        kqo_silu_mul_q8x4(g, u, xq, (float*)(xq + (m->inter / 32) * 8), m->inter / 32);
        trace_q8(xq, m->inter);
        mv_q(&L->wd, xq, t);
        const float* next = l + 1 < m->n_layers ? m->layers[l + 1].attn_norm : m->out_norm;
        kqo_add_sumsq(x, t, xq, hid / 32);
        if (g_forced) {
            trace_f32(x, hid);
            memset(t, 0, (size_t)hid * sizeof(float));
            kqo_add_sumsq(x, t, xq, hid / 32);
        } else trace_f32(x, hid);
        kqo_norm_q8x4(x, next, xq, hid / 32, m->eps);
        trace_q8(xq, hid);
    }
    mv_q(&m->lm_head, xq, logits);
}

void kqo_decode_token(const kqo_model* m, const float* x_in, int pos, float* logits, float* sf, int32_t* xq) {
    kqo_decode_token_ex(m, x_in, pos, logits, sf, xq, 0);
}
