/*
 * CPU oracle for mha_fwd_with_mask -- TEST INFRASTRUCTURE, not a product path.
 * Only tests, the smoke check and the benchmark's CPU-baseline legs may call it.
 *
 * Plain-C fp32 restatement of the reference semantics:
 *   - score = (q . k) * 1/sqrt(d) + mask, fp32
 *     (csrc/fa/sm89/fa_fwd_kernel.h:288-310 adds mask/scale to the raw score and
 *      scales afterwards; tests/test_mha_fwd_with_mask.py:45-48 scales q first;
 *      both are scale*s + mask)
 *   - row max clamped below so a fully masked row gives exp(-inf)=0, and a zero
 *     denominator gives an all-zero output row, never NaN
 *     (tests/test_mha_fwd_with_mask.py:49-51, csrc/fa/common/softmax.h:134-150)
 *   - optional rounding of P to the input dtype before P.V
 *     (tests/test_mha_fwd_with_mask.py:53)
 *   - GQA: kv head = h / (H / Hk)        (csrc/fa/sm89/fa_fwd_kernel.h:114,121)
 *   - mask is (B, 1, mask_sq >= Sq, mask_sk >= Sk); columns >= Sk and rows >= Sq
 *     are never read                      (csrc/fa/fa_fwd_op.cu:96-108)
 *   - lse = max + ln(sum) of the scaled masked scores, -inf for an empty row
 *     (csrc/fa/common/softmax.h:145)
 *
 * Inputs are 16-bit patterns (bf16 or IEEE fp16); output is fp32, not rounded.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

static inline float bf16_to_f32(uint16_t b) {
    uint32_t u = (uint32_t)b << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

static inline uint16_t f32_to_bf16(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return 0x7fc0;
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

static inline float fp16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu;
    uint32_t man = h & 0x3ffu;
    uint32_t u;
    if (exp == 0) {
        if (man == 0) {
            u = sign;
        } else {
            int e = -1;
            do { man <<= 1; e++; } while (!(man & 0x400u));
            man &= 0x3ffu;
            u = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        u = sign | 0x7f800000u | (man << 13);
    } else {
        u = sign | ((exp + 112u) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &u, 4);
    return f;
}

static inline uint16_t f32_to_fp16(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    uint32_t sign = (u >> 16) & 0x8000u;
    uint32_t a = u & 0x7fffffffu;
    if (a > 0x7f800000u) return (uint16_t)(sign | 0x7e00u);
    if (a >= 0x47800000u) return (uint16_t)(sign | 0x7c00u);      /* >= 65536 -> inf */
    if (a < 0x33000000u) return (uint16_t)sign;                     /* < 2^-25 -> 0 */
    int32_t e = (int32_t)(a >> 23) - 127;
    uint32_t man = (a & 0x7fffffu) | 0x800000u;
    uint32_t shift, half;
    uint16_t r;
    if (e < -14) {
        shift = (uint32_t)(13 + (-14 - e));          /* subnormal target */
        uint32_t q = man >> shift;
        uint32_t rem = man & ((1u << shift) - 1u);
        half = 1u << (shift - 1);
        if (rem > half || (rem == half && (q & 1u))) q++;
        r = (uint16_t)q;
    } else {
        uint32_t q = ((uint32_t)(e + 15) << 10) | ((man >> 13) & 0x3ffu);
        uint32_t rem = man & 0x1fffu;
        if (rem > 0x1000u || (rem == 0x1000u && (q & 1u))) q++;   /* may carry into inf */
        r = (uint16_t)q;
    }
    return (uint16_t)(sign | r);
}

static inline float widen(uint16_t x, int is_bf16) {
    return is_bf16 ? bf16_to_f32(x) : fp16_to_f32(x);
}

static inline float requant(float x, int is_bf16) {
    return is_bf16 ? bf16_to_f32(f32_to_bf16(x)) : fp16_to_f32(f32_to_fp16(x));
}

/* Conversion self-checks exposed for the tests. */
uint16_t fa_mask_oracle_f32_to_bits(float f, int is_bf16) {
    return is_bf16 ? f32_to_bf16(f) : f32_to_fp16(f);
}
float fa_mask_oracle_bits_to_f32(uint16_t b, int is_bf16) { return widen(b, is_bf16); }

int fa_mask_oracle_fwd(const uint16_t* q, const uint16_t* k, const uint16_t* v,
                       const uint16_t* mask, float* out, float* lse,
                       int B, int H, int Hk, int Sq, int Sk, int d,
                       int mask_sq, int mask_sk, int is_bf16, int quantize_p,
                       int n_threads) {
    if (B < 0 || H <= 0 || Hk <= 0 || H % Hk || Sq < 0 || Sk < 0 || d <= 0) return -1;
    if (mask_sq < Sq || mask_sk < Sk) return -2;
    const int g = H / Hk;
    const float scale = 1.0f / sqrtf((float)d);
#ifdef _OPENMP
    if (n_threads <= 0) n_threads = omp_get_max_threads();
#else
    n_threads = 1;
#endif
    int failed = 0;

    for (int b = 0; b < B; ++b) {
        for (int hk = 0; hk < Hk; ++hk) {
            /* Widen this kv head once; it serves g query heads. */
            const size_t kv_elems = (size_t)Sk * d;
            float* kf = (float*)malloc(sizeof(float) * (kv_elems ? kv_elems : 1));
            float* vf = (float*)malloc(sizeof(float) * (kv_elems ? kv_elems : 1));
            if (!kf || !vf) { free(kf); free(vf); return -3; }
            const uint16_t* kb = k + ((size_t)b * Hk + hk) * kv_elems;
            const uint16_t* vb = v + ((size_t)b * Hk + hk) * kv_elems;
            for (size_t i = 0; i < kv_elems; ++i) {
                kf[i] = widen(kb[i], is_bf16);
                vf[i] = widen(vb[i], is_bf16);
            }
            const long rows = (long)g * Sq;
#pragma omp parallel num_threads(n_threads)
            {
                float* s = (float*)malloc(sizeof(float) * (size_t)(Sk > 0 ? Sk : 1));
                float* qf = (float*)malloc(sizeof(float) * (size_t)d);
                float* acc = (float*)malloc(sizeof(float) * (size_t)d);
                if (!s || !qf || !acc) {
#pragma omp atomic write
                    failed = 1;
                }
#pragma omp for schedule(static)
                for (long r = 0; r < rows; ++r) {
                    if (!s || !qf || !acc) continue;
                    const int h = hk * g + (int)(r / Sq);
                    const int i = (int)(r % Sq);
                    const uint16_t* qrow = q + (((size_t)b * H + h) * Sq + i) * d;
                    const uint16_t* mrow = mask + ((size_t)b * mask_sq + i) * mask_sk;
                    for (int c = 0; c < d; ++c) qf[c] = widen(qrow[c], is_bf16) * scale;
                    float mx = -INFINITY;
                    for (int j = 0; j < Sk; ++j) {
                        const float* kr = kf + (size_t)j * d;
                        float dot = 0.f;
                        for (int c = 0; c < d; ++c) dot += qf[c] * kr[c];
                        const float sc = dot + widen(mrow[j], is_bf16);
                        s[j] = sc;
                        if (sc > mx) mx = sc;
                    }
                    const float mref = mx > -1e30f ? mx : -1e30f;
                    float sum = 0.f;
                    for (int j = 0; j < Sk; ++j) {
                        const float p = expf(s[j] - mref);
                        s[j] = p;
                        sum += p;
                    }
                    const float denom = sum > 1e-38f ? sum : 1e-38f;
                    for (int c = 0; c < d; ++c) acc[c] = 0.f;
                    for (int j = 0; j < Sk; ++j) {
                        float p = s[j] / denom;
                        if (quantize_p) p = requant(p, is_bf16);
                        if (p == 0.f) continue;
                        const float* vr = vf + (size_t)j * d;
                        for (int c = 0; c < d; ++c) acc[c] += p * vr[c];
                    }
                    float* orow = out + (((size_t)b * H + h) * Sq + i) * d;
                    for (int c = 0; c < d; ++c) orow[c] = acc[c];
                    if (lse)
                        lse[((size_t)b * H + h) * Sq + i] =
                            (sum > 0.f && mx > -INFINITY) ? mx + logf(sum) : -INFINITY;
                }
                free(s); free(qf); free(acc);
            }
            free(kf); free(vf);
            if (failed) return -3;
        }
    }
    return 0;
}
