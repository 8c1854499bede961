/* bpdq_oracle.c -- CPU restatement of the quantized-inference hot path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA kernels are
 * compared against; nothing in the shipped library calls it, links it or
 * falls back to it.  It may be loaded only by tests, by the smoke check and
 * by the bench's CPU-baseline leg.
 *
 * Every function restates an algorithm of the reference project
 * (heath-hunnicutt-ruach-tov/bpd-substrate) and names the reference lines it
 * follows.  The restatement is pinned by tests that compare it bit for bit
 * with the reference's own C files compiled unmodified, and with the
 * known-answer cases the reference's tests hold
 * (tests/verify_f16_fix.py, tests/check_f16_algorithm.py).
 *
 * The Q8_K activation format and the Q4_K x Q8_K dot are NOT in the
 * reference (docs/llama-kernel-audit.md:65 lists them as an unbuilt design);
 * the functions marked "builder-defined" below are this repository's own
 * definition, built from the reference's Q8_0 analogues.  For those:
 * parity unpinned.
 *
 * Build:  gcc -O2 -ffp-contract=off -shared -fPIC bpdq_oracle.c -lm
 * (-ffp-contract=off keeps "mul then add" as two roundings, which is what
 * the reference's -O2 x86-64 build does: bench/bpd_quant.c:103-105.)
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define Q4K_SB_BYTES   144   /* bench/bpd_quant.c:21-22 */
#define Q4K_SB_ELEMS   256
#define Q80_BLK_BYTES  34    /* bench/bpd_cpu.c:3886-3890 */
#define Q80_BLK_ELEMS  32
#define Q8K_BLK_BYTES  292   /* lib/gguf_emit_manifest.pl:142 (size only) */

/* ------------------------------------------------------------------ fp16 */

/* binary16 -> binary32.  Same mapping as bench/bpd_quant.c:25-38 (ldexpf
 * form) and bench/bpd_cpu.c:3928-3958 (bit-trick form) for every finite
 * input and for infinities; a NaN input gives the platform's default quiet
 * NaN with the input's sign, as bench/bpd_quant.c:33,37 does.  Written here
 * as a direct field rebuild: normal numbers re-bias the exponent, subnormals
 * are normalised by counting the leading zero of the 10-bit fraction. */
float orc_f16_to_f32(uint16_t h)
{
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t e = (h >> 10) & 0x1Fu;
    uint32_t f = h & 0x3FFu;
    uint32_t bits;
    if (e == 0x1Fu) {
        if (f) {
            float q = NAN;
            return sign ? -q : q;
        }
        bits = sign | 0x7F800000u;
    } else if (e) {
        bits = sign | ((e + 112u) << 23) | (f << 13);
    } else if (f) {
        int shift = 0;
        while (!(f & 0x400u)) { f <<= 1; shift++; }
        bits = sign | ((uint32_t)(113 - shift) << 23) | ((f & 0x3FFu) << 13);
    } else {
        bits = sign;
    }
    float out;
    memcpy(&out, &bits, 4);
    return out;
}

/* binary32 -> binary16, round to nearest even, overflow to infinity,
 * gradual underflow.  Same results as bench/bpd_cpu.c:4049-4104 (which the
 * reference states equals the F16C instruction).  Written as "add the
 * rounding increment, then shift". */
uint16_t orc_f32_to_f16(float v)
{
    uint32_t x;
    memcpy(&x, &v, 4);
    uint16_t sign = (uint16_t)((x >> 16) & 0x8000u);
    uint32_t mag = x & 0x7FFFFFFFu;
    if (mag >= 0x7F800000u) {                 /* inf / nan */
        uint32_t frac = mag & 0x7FFFFFu;
        /* bench/bpd_cpu.c:4057-4059: keep top fraction bits, force nonzero */
        return (uint16_t)(sign | 0x7C00u | (frac ? ((frac >> 13) | 1u) : 0u));
    }
    int32_t e16 = (int32_t)(mag >> 23) - 112;  /* re-biased exponent */
    uint32_t frac = mag & 0x7FFFFFu;
    if (e16 >= 31) return (uint16_t)(sign | 0x7C00u);
    if (e16 <= 0) {
        if (e16 < -10) return sign;            /* below half the least subnormal */
        uint32_t full = frac | 0x800000u;
        int sh = 14 - e16;                     /* 14..24 */
        uint32_t kept = full >> sh;
        uint32_t rem = full & ((1u << sh) - 1u);
        uint32_t half = 1u << (sh - 1);
        if (rem > half || (rem == half && (kept & 1u))) kept++;
        return (uint16_t)(sign | kept);
    }
    uint32_t kept = ((uint32_t)e16 << 10) | (frac >> 13);
    uint32_t rem = frac & 0x1FFFu;
    if (rem > 0x1000u || (rem == 0x1000u && (kept & 1u))) kept++;  /* carry may reach inf */
    return (uint16_t)(sign | kept);
}

/* ------------------------------------------------------------------ Q4_K */

/* 12 packed bytes -> eight 6-bit scales and eight 6-bit mins.
 * bench/bpd_quant.c:55-62. */
void orc_q4k_scales(const uint8_t *s, uint8_t sc[8], uint8_t mn[8])
{
    for (int j = 0; j < 4; j++) {
        sc[j]     = s[j] & 63;
        mn[j]     = s[j + 4] & 63;
        sc[j + 4] = (uint8_t)((s[j + 8] & 15) | ((s[j] >> 6) << 4));
        mn[j + 4] = (uint8_t)((s[j + 8] >> 4) | ((s[j + 4] >> 6) << 4));
    }
}

/* Nibble of element e (0..255) of a super-block.
 * layout 0 = the C-ABI layout of bench/bpd_quant.c:68-72: byte 16j+k holds
 *            element 32j+k (low) and 32j+16+k (high);
 * layout 1 = the ggml layout of bench/bench_dequant_gpu_h2h.cu:35-46: byte
 *            32c+l holds element 64c+l (low) and 64c+32+l (high). */
static inline unsigned q4k_nibble(const uint8_t *qs, int e, int layout)
{
    if (layout == 0) {
        int j = e >> 5, p = e & 31;
        uint8_t b = qs[16 * j + (p & 15)];
        return (p < 16) ? (b & 15u) : (unsigned)(b >> 4);
    } else {
        int c = e >> 6, p = e & 63;
        uint8_t b = qs[32 * c + (p & 31)];
        return (p < 32) ? (b & 15u) : (unsigned)(b >> 4);
    }
}

static void q4k_dequant_sb(const uint8_t *blk, float *out, int layout)
{
    uint16_t hd, hm;
    memcpy(&hd, blk, 2);
    memcpy(&hm, blk + 2, 2);
    float d = orc_f16_to_f32(hd), dmin = orc_f16_to_f32(hm);
    uint8_t sc[8], mn[8];
    orc_q4k_scales(blk + 4, sc, mn);
    for (int e = 0; e < Q4K_SB_ELEMS; e++) {
        int j = e >> 5;
        float scale = d * (float)sc[j];       /* bench/bpd_quant.c:64 */
        float minv = dmin * (float)mn[j];     /* bench/bpd_quant.c:65 */
        out[e] = scale * (float)q4k_nibble(blk + 16, e, layout) - minv;  /* :70-71 */
    }
}

/* bench/bpd_quant.c:77-81 (layout 0) / bench/bench_dequant_gpu_h2h.cu:27-48
 * (layout 1). */
void orc_dequant_q4k(const uint8_t *q, float *out, long n_blocks, int layout)
{
    for (long b = 0; b < n_blocks; b++)
        q4k_dequant_sb(q + b * Q4K_SB_BYTES, out + b * Q4K_SB_ELEMS, layout);
}

/* W4A32 GEMV, bench/bpd_quant.c:88-109: one fp32 accumulator per row,
 * strictly left to right over k, multiply then add (two roundings). */
void orc_qmatmul_q4k(const uint8_t *qw, const float *x, float *out,
                     int M, int K, int layout)
{
    int nb = K / Q4K_SB_ELEMS;
    float buf[Q4K_SB_ELEMS];
    for (int r = 0; r < M; r++) {
        const uint8_t *row = qw + (size_t)r * nb * Q4K_SB_BYTES;
        float acc = 0.0f;
        for (int b = 0; b < nb; b++) {
            q4k_dequant_sb(row + (size_t)b * Q4K_SB_BYTES, buf, layout);
            for (int k = 0; k < Q4K_SB_ELEMS; k++) {
                float p = buf[k] * x[b * Q4K_SB_ELEMS + k];
                acc = acc + p;
            }
        }
        out[r] = acc;
    }
}

/* Same sum carried in binary64 (products exact in double): the yardstick
 * both the reference's and the GPU's fp32 orders are measured against. */
void orc_qmatmul_q4k_f64(const uint8_t *qw, const float *x, double *out,
                         int M, int K, int layout)
{
    int nb = K / Q4K_SB_ELEMS;
    float buf[Q4K_SB_ELEMS];
    for (int r = 0; r < M; r++) {
        const uint8_t *row = qw + (size_t)r * nb * Q4K_SB_BYTES;
        double acc = 0.0;
        for (int b = 0; b < nb; b++) {
            q4k_dequant_sb(row + (size_t)b * Q4K_SB_BYTES, buf, layout);
            for (int k = 0; k < Q4K_SB_ELEMS; k++)
                acc += (double)buf[k] * (double)x[b * Q4K_SB_ELEMS + k];
        }
        out[r] = acc;
    }
}

/* W4A32 GEMM, bench/bpd_quant.c:114-137: C[row][col], B is [K][N] with N the
 * token count; each cell accumulates left to right over k. */
void orc_qmm_q4k(const uint8_t *qA, const float *B, float *C,
                 int M, int N, int K, int layout)
{
    int nb = K / Q4K_SB_ELEMS;
    float buf[Q4K_SB_ELEMS];
    for (int r = 0; r < M; r++) {
        const uint8_t *row = qA + (size_t)r * nb * Q4K_SB_BYTES;
        float *crow = C + (size_t)r * N;
        for (int c = 0; c < N; c++) crow[c] = 0.0f;
        for (int b = 0; b < nb; b++) {
            q4k_dequant_sb(row + (size_t)b * Q4K_SB_BYTES, buf, layout);
            for (int k = 0; k < Q4K_SB_ELEMS; k++) {
                const float *brow = B + (size_t)(b * Q4K_SB_ELEMS + k) * N;
                float a = buf[k];
                for (int c = 0; c < N; c++) {
                    float p = a * brow[c];
                    crow[c] = crow[c] + p;
                }
            }
        }
    }
}

/* ------------------------------------------------------------------ Q8_0 */

/* bench/bpd_cpu.c:3960-3973. */
void orc_dequant_q8_0(const uint8_t *raw, float *out, long n_blocks)
{
    for (long b = 0; b < n_blocks; b++) {
        const uint8_t *blk = raw + b * Q80_BLK_BYTES;
        float s = orc_f16_to_f32((uint16_t)(blk[0] | (blk[1] << 8)));
        const int8_t *q = (const int8_t *)(blk + 2);
        for (int i = 0; i < Q80_BLK_ELEMS; i++)
            out[b * Q80_BLK_ELEMS + i] = (float)q[i] * s;
    }
}

/* bench/bpd_cpu.c:4002-4013: gather rows by token id, dequantize. */
void orc_embed_lookup_q8_0(const uint8_t *table, const int32_t *ids, float *out,
                           int n_tokens, int embed_dim)
{
    int bpr = embed_dim / Q80_BLK_ELEMS;
    for (int t = 0; t < n_tokens; t++)
        orc_dequant_q8_0(table + (size_t)ids[t] * bpr * Q80_BLK_BYTES,
                         out + (size_t)t * embed_dim, bpr);
}

/* bench/bpd_cpu.c:4106-4136: per 32 values, stored scale = f16(amax/127),
 * multiplier = 127/amax (one IEEE division, NOT the reciprocal of the stored
 * scale), quant = round-half-even(x * multiplier). */
void orc_quant_q8_0(const float *x, uint8_t *y, long n)
{
    long nb = n / Q80_BLK_ELEMS;
    for (long b = 0; b < nb; b++) {
        const float *xb = x + b * Q80_BLK_ELEMS;
        uint8_t *yb = y + b * Q80_BLK_BYTES;
        float amax = 0.0f;
        for (int i = 0; i < Q80_BLK_ELEMS; i++) {
            float a = xb[i] < 0 ? -xb[i] : xb[i];
            if (a > amax) amax = a;
        }
        uint16_t hs = orc_f32_to_f16(amax / 127.0f);
        yb[0] = (uint8_t)(hs & 0xFF);
        yb[1] = (uint8_t)(hs >> 8);
        float mul = (amax != 0.0f) ? 127.0f / amax : 0.0f;
        for (int i = 0; i < Q80_BLK_ELEMS; i++)
            yb[2 + i] = (uint8_t)(int8_t)rintf(xb[i] * mul);
    }
}

/* Exact int32 dot of every block pair: the integer core of
 * bench/bpd_cpu.c:4270-4271, exposed so a GPU kernel's integer part can be
 * compared exactly. */
void orc_q8_0_block_dots(const uint8_t *w, const uint8_t *a, int32_t *dots,
                         long n_blocks)
{
    for (long b = 0; b < n_blocks; b++) {
        const int8_t *wq = (const int8_t *)(w + b * Q80_BLK_BYTES + 2);
        const int8_t *aq = (const int8_t *)(a + b * Q80_BLK_BYTES + 2);
        int32_t s = 0;
        for (int i = 0; i < Q80_BLK_ELEMS; i++) s += (int32_t)wq[i] * (int32_t)aq[i];
        dots[b] = s;
    }
}

/* Scalar dot, bench/bpd_cpu.c:4263-4280: sumf += (float)sumi * (wd * ad),
 * blocks left to right. */
float orc_qdot_q8_0(const uint8_t *w, const uint8_t *a, int n_blocks)
{
    float acc = 0.0f;
    for (int b = 0; b < n_blocks; b++) {
        const uint8_t *wb = w + (size_t)b * Q80_BLK_BYTES;
        const uint8_t *ab = a + (size_t)b * Q80_BLK_BYTES;
        int32_t s;
        orc_q8_0_block_dots(wb, ab, &s, 1);
        float wd = orc_f16_to_f32((uint16_t)(wb[0] | (wb[1] << 8)));
        float ad = orc_f16_to_f32((uint16_t)(ab[0] | (ab[1] << 8)));
        float scale = wd * ad;
        float term = (float)s * scale;
        acc = acc + term;
    }
    return acc;
}

/* Same dot carried in binary64. */
double orc_qdot_q8_0_f64(const uint8_t *w, const uint8_t *a, int n_blocks)
{
    double acc = 0.0;
    for (int b = 0; b < n_blocks; b++) {
        const uint8_t *wb = w + (size_t)b * Q80_BLK_BYTES;
        const uint8_t *ab = a + (size_t)b * Q80_BLK_BYTES;
        int32_t s;
        orc_q8_0_block_dots(wb, ab, &s, 1);
        double wd = orc_f16_to_f32((uint16_t)(wb[0] | (wb[1] << 8)));
        double ad = orc_f16_to_f32((uint16_t)(ab[0] | (ab[1] << 8)));
        acc += (double)s * wd * ad;
    }
    return acc;
}

/* bench/bpd_cpu.c:4295-4315: quantize each activation row, then
 * out[m*N + n] = qdot(weight row n, activation row m). */
int orc_qmatmul_q8_0(const uint8_t *W, const float *X, float *out,
                     int M, int N, int K)
{
    int bpr = K / Q80_BLK_ELEMS;
    size_t rb = (size_t)bpr * Q80_BLK_BYTES;
    uint8_t *xq = (uint8_t *)malloc((size_t)M * rb + 1);
    if (!xq) return -1;
    for (int m = 0; m < M; m++) orc_quant_q8_0(X + (size_t)m * K, xq + m * rb, K);
    for (int m = 0; m < M; m++)
        for (int n = 0; n < N; n++)
            out[(size_t)m * N + n] = orc_qdot_q8_0(W + n * rb, xq + m * rb, bpr);
    free(xq);
    return 0;
}

int orc_qmatmul_q8_0_f64(const uint8_t *W, const float *X, double *out,
                         int M, int N, int K)
{
    int bpr = K / Q80_BLK_ELEMS;
    size_t rb = (size_t)bpr * Q80_BLK_BYTES;
    uint8_t *xq = (uint8_t *)malloc((size_t)M * rb + 1);
    if (!xq) return -1;
    for (int m = 0; m < M; m++) orc_quant_q8_0(X + (size_t)m * K, xq + m * rb, K);
    for (int m = 0; m < M; m++)
        for (int n = 0; n < N; n++)
            out[(size_t)m * N + n] = orc_qdot_q8_0_f64(W + n * rb, xq + m * rb, bpr);
    free(xq);
    return 0;
}

/* The tile kernels and dispatcher of bench/bpd_gemm_q8_0_cpu.c:32-97, 159-207
 * (AVX build) on activations that are already Q8_0 rows.  Per output cell the
 * reference keeps eight fp32 lanes; lane q takes, block after block,
 *     c_q = (wd * ad) * (float)(w[4q..4q+3] . a[4q..4q+3]) + c_q
 * (a 32-bit lane of p32 is the sum of four adjacent byte products; multiply
 * and add are separate roundings), and joins the lanes at the end as
 *     s_q = c_{q+4} + c_q (q < 4);  t_0 = s_0 + s_2, t_1 = s_1 + s_3;  t_0 + t_1.
 * The tiling (which cells share a call) does not change a cell's arithmetic,
 * so this is written cell by cell.  out[j * m_weight + i]. */
void orc_qmatmul_q8_0_lanes(const uint8_t *Wq, const uint8_t *Xq, float *out,
                            int m_weight, int m_tokens, int K)
{
    int bpr = K / Q80_BLK_ELEMS;
    size_t rb = (size_t)bpr * Q80_BLK_BYTES;
    for (int j = 0; j < m_tokens; j++)
        for (int i = 0; i < m_weight; i++) {
            float c[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            for (int l = 0; l < bpr; l++) {
                const uint8_t *wb = Wq + (size_t)i * rb + (size_t)l * Q80_BLK_BYTES;
                const uint8_t *ab = Xq + (size_t)j * rb + (size_t)l * Q80_BLK_BYTES;
                float wd = orc_f16_to_f32((uint16_t)(wb[0] | (wb[1] << 8)));
                float ad = orc_f16_to_f32((uint16_t)(ab[0] | (ab[1] << 8)));
                float scale = wd * ad;
                const int8_t *wq = (const int8_t *)(wb + 2), *aq = (const int8_t *)(ab + 2);
                for (int q = 0; q < 8; q++) {
                    int32_t p = 0;
                    for (int e = 0; e < 4; e++) p += (int32_t)wq[4 * q + e] * (int32_t)aq[4 * q + e];
                    float prod = scale * (float)p;
                    c[q] = prod + c[q];
                }
            }
            float s0 = c[4] + c[0], s1 = c[5] + c[1], s2 = c[6] + c[2], s3 = c[7] + c[3];
            float t0 = s0 + s2, t1 = s1 + s3;
            out[(size_t)j * m_weight + i] = t0 + t1;
        }
}

/* ------------------------------------------- Q8_K (builder-defined format) */

/* Q8_K block, 292 bytes for 256 activations (size fact:
 * lib/gguf_emit_manifest.pl:130,142; no struct or code in the reference):
 *   bytes   0..3    float  d       = amax / 127
 *   bytes   4..259  int8   qs[256] = round-half-even(x * (127 / amax))
 *   bytes 260..291  int16  bsums[16], bsums[g] = sum of qs[16g .. 16g+15]
 * The quantizer rule is bench/bpd_cpu.c:4106-4136 lifted from 32 to 256
 * values with the scale kept in fp32.  Builder-defined: parity unpinned. */
void orc_quant_q8_K(const float *x, uint8_t *y, long n)
{
    long nb = n / Q4K_SB_ELEMS;
    for (long b = 0; b < nb; b++) {
        const float *xb = x + b * Q4K_SB_ELEMS;
        uint8_t *yb = y + b * Q8K_BLK_BYTES;
        float amax = 0.0f;
        for (int i = 0; i < Q4K_SB_ELEMS; i++) {
            float a = xb[i] < 0 ? -xb[i] : xb[i];
            if (a > amax) amax = a;
        }
        float d = amax / 127.0f;
        float mul = (amax != 0.0f) ? 127.0f / amax : 0.0f;
        memcpy(yb, &d, 4);
        int8_t *q = (int8_t *)(yb + 4);
        for (int i = 0; i < Q4K_SB_ELEMS; i++) q[i] = (int8_t)rintf(xb[i] * mul);
        for (int g = 0; g < 16; g++) {
            int16_t s = 0;
            for (int i = 0; i < 16; i++) s = (int16_t)(s + q[16 * g + i]);
            memcpy(yb + 260 + 2 * g, &s, 2);
        }
    }
}

void orc_dequant_q8_K(const uint8_t *y, float *out, long n_blocks)
{
    for (long b = 0; b < n_blocks; b++) {
        const uint8_t *yb = y + b * Q8K_BLK_BYTES;
        float d;
        memcpy(&d, yb, 4);
        const int8_t *q = (const int8_t *)(yb + 4);
        for (int i = 0; i < Q4K_SB_ELEMS; i++) out[b * Q4K_SB_ELEMS + i] = d * (float)q[i];
    }
}

/* Exact integer core of the Q4_K x Q8_K dot: for weight row r, super-block
 * b, sub-block j the int32 sum of nibble(e) * qs[e] over the sub-block's 32
 * elements.  dots is [M][K/256][8].  Builder-defined. */
void orc_q4k_q8k_subdots(const uint8_t *qw, const uint8_t *xq, int32_t *dots,
                         int M, int K, int layout)
{
    int nb = K / Q4K_SB_ELEMS;
    for (int r = 0; r < M; r++)
        for (int b = 0; b < nb; b++) {
            const uint8_t *wb = qw + ((size_t)r * nb + b) * Q4K_SB_BYTES;
            const int8_t *a = (const int8_t *)(xq + (size_t)b * Q8K_BLK_BYTES + 4);
            for (int j = 0; j < 8; j++) {
                int32_t s = 0;
                for (int p = 0; p < 32; p++) {
                    int e = 32 * j + p;
                    s += (int32_t)q4k_nibble(wb + 16, e, layout) * (int32_t)a[e];
                }
                dots[((size_t)r * nb + b) * 8 + j] = s;
            }
        }
}

/* Per super-block integer pair: isum = sum_j sc_j * dot_j,
 * msum = sum_j mn_j * (bsums[2j] + bsums[2j+1]).  Both exact in int32
 * (|isum| <= 63*60960*8, |msum| <= 63*4064*8). */
static void q4k_q8k_sb_ints(const uint8_t *wb, const uint8_t *ab, int layout,
                            int32_t *isum, int32_t *msum)
{
    uint8_t sc[8], mn[8];
    orc_q4k_scales(wb + 4, sc, mn);
    const int8_t *a = (const int8_t *)(ab + 4);
    int32_t is = 0, ms = 0;
    for (int j = 0; j < 8; j++) {
        int32_t s = 0;
        for (int p = 0; p < 32; p++) {
            int e = 32 * j + p;
            s += (int32_t)q4k_nibble(wb + 16, e, layout) * (int32_t)a[e];
        }
        int16_t b0, b1;
        memcpy(&b0, ab + 260 + 4 * j, 2);
        memcpy(&b1, ab + 262 + 4 * j, 2);
        is += (int32_t)sc[j] * s;
        ms += (int32_t)mn[j] * ((int32_t)b0 + (int32_t)b1);
    }
    *isum = is;
    *msum = ms;
}

/* Q4_K x Q8_K GEMV on pre-quantized activations (builder-defined, structure
 * of bench/bpd_cpu.c:4263-4280): per super-block
 *     term = (d * dA) * (float)isum - (dmin * dA) * (float)msum
 * accumulated left to right in fp32 (out) and in binary64 (out64, may be
 * NULL). */
void orc_qmatmul_q4k_q8k(const uint8_t *qw, const uint8_t *xq, float *out,
                         double *out64, int M, int K, int layout)
{
    int nb = K / Q4K_SB_ELEMS;
    for (int r = 0; r < M; r++) {
        float acc = 0.0f;
        double acc64 = 0.0;
        for (int b = 0; b < nb; b++) {
            const uint8_t *wb = qw + ((size_t)r * nb + b) * Q4K_SB_BYTES;
            const uint8_t *ab = xq + (size_t)b * Q8K_BLK_BYTES;
            uint16_t hd, hm;
            memcpy(&hd, wb, 2);
            memcpy(&hm, wb + 2, 2);
            float d = orc_f16_to_f32(hd), dmin = orc_f16_to_f32(hm), dA;
            memcpy(&dA, ab, 4);
            int32_t is, ms;
            q4k_q8k_sb_ints(wb, ab, layout, &is, &ms);
            float t1 = (d * dA) * (float)is;
            float t2 = (dmin * dA) * (float)ms;
            float term = t1 - t2;
            acc = acc + term;
            acc64 += (double)d * (double)dA * (double)is
                   - (double)dmin * (double)dA * (double)ms;
        }
        out[r] = acc;
        if (out64) out64[r] = acc64;
    }
}

/* Batched form: X is [T][K] fp32, quantized row by row to Q8_K, output
 * out[t*M + r] (token-major, the layout of gpu_matmul's C[M tokens][N]:
 * lib/kernel_templates_llama.pl:1104-1112). */
int orc_qmm_q4k_q8k(const uint8_t *qw, const float *X, float *out, double *out64,
                    int T, int M, int K, int layout)
{
    int nb = K / Q4K_SB_ELEMS;
    uint8_t *xq = (uint8_t *)malloc((size_t)nb * Q8K_BLK_BYTES + 1);
    if (!xq) return -1;
    for (int t = 0; t < T; t++) {
        orc_quant_q8_K(X + (size_t)t * K, xq, K);
        orc_qmatmul_q4k_q8k(qw, xq, out + (size_t)t * M,
                            out64 ? out64 + (size_t)t * M : NULL, M, K, layout);
    }
    free(xq);
    return 0;
}

/* The exact integer pair of every (token, row, super-block) of the batched
 * form: ints[((t*M + r)*nb + b)*2 + {0,1}] = (isum, msum) as defined at
 * q4k_q8k_sb_ints.  Builder-defined. */
int orc_qmm_q4k_q8k_ints(const uint8_t *qw, const float *X, int32_t *ints,
                         int T, int M, int K, int layout)
{
    int nb = K / Q4K_SB_ELEMS;
    uint8_t *xq = (uint8_t *)malloc((size_t)nb * Q8K_BLK_BYTES + 1);
    if (!xq) return -1;
    for (int t = 0; t < T; t++) {
        orc_quant_q8_K(X + (size_t)t * K, xq, K);
        for (int r = 0; r < M; r++)
            for (int b = 0; b < nb; b++) {
                int32_t *o = ints + (((size_t)t * M + r) * nb + b) * 2;
                q4k_q8k_sb_ints(qw + ((size_t)r * nb + b) * Q4K_SB_BYTES,
                                xq + (size_t)b * Q8K_BLK_BYTES, layout, o, o + 1);
            }
    }
    free(xq);
    return 0;
}

/* ----------------------------------------------- fp32 decode-dispatch ops */

/* lib/kernel_templates_llama.pl:107-145: c[col] = sum_k a[k] * b[k*n + col],
 * left to right. */
void orc_vecmat_f32(const float *a, const float *b, float *c, int k, int n)
{
    for (int col = 0; col < n; col++) {
        float acc = 0.0f;
        for (int i = 0; i < k; i++) {
            float p = a[i] * b[(size_t)i * n + col];
            acc = acc + p;
        }
        c[col] = acc;
    }
}

/* lib/kernel_templates_llama.pl:529-581: out = x * rsqrt(mean(x^2) + eps) * w,
 * carried here in binary64 and rounded once (the GPU kernel's reduction
 * order differs from any CPU loop, so the comparison is by tolerance). */
void orc_rms_norm_f64(const float *in, const float *w, float *out,
                      int rows, int cols, float eps)
{
    for (int r = 0; r < rows; r++) {
        const float *x = in + (size_t)r * cols;
        double ss = 0.0;
        for (int c = 0; c < cols; c++) ss += (double)x[c] * (double)x[c];
        double scale = 1.0 / sqrt(ss / cols + (double)eps);
        for (int c = 0; c < cols; c++)
            out[(size_t)r * cols + c] = (float)((double)x[c] * scale * (double)w[c]);
    }
}

/* ------------------------------------------------------------------------
 * Q8_0 Llama forward: restatement of bpd_llama_block_cpu / bpd_llama_forward_cpu
 * (bench/bpd_cpu.c:5608-5798) and of the steps they compose.  Own code, same
 * arithmetic; pinned against the compiled reference by tests/test_oracle_pins.py.
 * ------------------------------------------------------------------------ */

/* bench/bpd_cpu.c:4959-4988: binary64 sum of squares in index order, mean rounded
 * to fp32, scale = 1/sqrtf(mean + eps), y = (x*scale)*w. */
void orc_rmsnorm_llama(const float *in, const float *w, float *out, int rows, int cols, float eps)
{
    for (int r = 0; r < rows; r++) {
        const float *x = in + (size_t)r * cols;
        float *y = out + (size_t)r * cols;
        double acc = 0.0;
        for (int i = 0; i < cols; i++) acc += (double)x[i] * (double)x[i];
        const float mean = (float)(acc / cols);
        const float scale = 1.0f / sqrtf(mean + eps);
        for (int i = 0; i < cols; i++) y[i] = w ? x[i] * scale * w[i] : x[i] * scale;
    }
}

/* bench/bpd_cpu.c:5146-5183: pairs (2p, 2p+1) of each head rotate by theta_p / ff_p,
 * theta_0 = (float)pos, theta_{p+1} = theta_p * base^(-2/n_dims); dims past n_dims copy. */
void orc_rope_norm_freqs(const float *in, float *out, const int32_t *pos, const float *ff,
                         int n_tokens, int n_heads, int head_dim, int n_dims, float base)
{
    const float step = powf(base, -2.0f / (float)n_dims);
    for (int t = 0; t < n_tokens; t++)
        for (int h = 0; h < n_heads; h++) {
            const float *src = in + ((size_t)t * n_heads + h) * head_dim;
            float *dst = out + ((size_t)t * n_heads + h) * head_dim;
            float theta = (float)pos[t];
            for (int p = 0; 2 * p < n_dims; p++) {
                const float te = theta / (ff ? ff[p] : 1.0f);
                const float c = cosf(te), s = sinf(te);
                const float a = src[2 * p], b = src[2 * p + 1];
                dst[2 * p] = a * c - b * s;
                dst[2 * p + 1] = a * s + b * c;
                theta *= step;
            }
            for (int i = n_dims; i < head_dim; i++) dst[i] = src[i];
        }
}

/* bench/bpd_cpu.c:5204-5257: cache row pos[t] = src row t, as fp32 or rounded to f16. */
void orc_kv_cache_write(void *cache, const float *src, const int32_t *pos, int n_tokens, int row, int f16)
{
    for (int t = 0; t < n_tokens; t++)
        for (int i = 0; i < row; i++) {
            const size_t at = (size_t)pos[t] * row + i;
            if (f16) ((uint16_t *)cache)[at] = orc_f32_to_f16(src[(size_t)t * row + i]);
            else ((float *)cache)[at] = src[(size_t)t * row + i];
        }
}

/* bench/bpd_cpu.c:5370-5433: raw dots, then scale and mask (-1e38 past the query's
 * position), maximum, exp and sum, multiply by the reciprocal, weighted sum of V;
 * every one of the n_kv rows takes part. */
void orc_gqa_attn(const float *q, const float *k, const float *v, float *dst, int n_q, int n_kv,
                  int n_q_heads, int n_kv_heads, int head_dim, float scale, int kv_offset)
{
    const int group = n_q_heads / n_kv_heads;
    float *sc = (float *)malloc(sizeof(float) * (size_t)n_kv);
    for (int t = 0; t < n_q; t++)
        for (int h = 0; h < n_q_heads; h++) {
            const int kh = h / group, qpos = kv_offset + t;
            const float *pq = q + ((size_t)t * n_q_heads + h) * head_dim;
            float *pd = dst + ((size_t)t * n_q_heads + h) * head_dim;
            float mx = -1e38f;
            for (int c = 0; c < n_kv; c++) {
                const float *pk = k + ((size_t)c * n_kv_heads + kh) * head_dim;
                float s = 0.0f;
                for (int d = 0; d < head_dim; d++) s += pq[d] * pk[d];
                sc[c] = (c <= qpos) ? s * scale : -1e38f;
                if (sc[c] > mx) mx = sc[c];
            }
            float sum = 0.0f;
            for (int c = 0; c < n_kv; c++) {
                sc[c] = expf(sc[c] - mx);
                sum += sc[c];
            }
            const float inv = (sum == 0.0f) ? 0.0f : 1.0f / sum;
            for (int c = 0; c < n_kv; c++) sc[c] *= inv;
            for (int d = 0; d < head_dim; d++) pd[d] = 0.0f;
            for (int c = 0; c < n_kv; c++) {
                const float *pv = v + ((size_t)c * n_kv_heads + kh) * head_dim;
                for (int d = 0; d < head_dim; d++) pd[d] += pv[d] * sc[c];
            }
        }
    free(sc);
}

/* bench/bpd_cpu.c:4512-4529 with inner = 1: first index of the largest value. */
void orc_argmax_rows(const float *x, long *out, int rows, int n)
{
    for (int r = 0; r < rows; r++) {
        long best = 0;
        for (int kx = 1; kx < n; kx++)
            if (x[(size_t)r * n + kx] > x[(size_t)r * n + best]) best = kx;
        out[r] = best;
    }
}

typedef struct {
    int n_layers, n_heads, n_kv_heads, head_dim, embed_dim, ffn_dim, vocab_size, max_seq_len;
    float rms_eps, rope_base;
    int rope_dim, kv_cache_f16;
} orc_llama_config;            /* bench/bpd_cpu.c:5537-5553 */
typedef struct {
    const float *attn_norm_w;
    const uint8_t *w_q, *w_k, *w_v, *w_o;
    const float *ffn_norm_w;
    const uint8_t *w_gate, *w_up, *w_down;
} orc_llama_layer;             /* bench/bpd_cpu.c:5569-5579 */
typedef struct {
    const uint8_t *token_embd;
    const orc_llama_layer *layers;
    const float *output_norm_w;
    const uint8_t *output_w;
    const float *rope_freqs;
} orc_llama_weights;           /* bench/bpd_cpu.c:5582-5588 */

/* out[t*rows + r] = W row r . q8_0(X row t): the scalar product of bench/bpd_cpu.c:4295-4315,
 * which is what the reference's non-AVX build runs (bench/bpd_cpu.c:4455-4458). */
static void llama_matmul(const uint8_t *W, const float *X, float *out, int rows, int tokens, int K)
{
    orc_qmatmul_q8_0(W, X, out, tokens, rows, K);
}

/* bench/bpd_cpu.c:5608-5738 */
void orc_llama_block(float *x, const orc_llama_layer *lw, const orc_llama_config *cfg, const int32_t *pos,
                     int n_tokens, int kv_pos, void *k_cache, void *v_cache, float *s1, float *s2, float *s3,
                     const float *rope_freqs)
{
    const int E = cfg->embed_dim, H = cfg->n_heads, HKV = cfg->n_kv_heads, D = cfg->head_dim, F = cfg->ffn_dim;
    const int n_kv = cfg->max_seq_len, row = HKV * D;
    orc_rmsnorm_llama(x, lw->attn_norm_w, s1, n_tokens, E, cfg->rms_eps);
    llama_matmul(lw->w_q, s1, s2, H * D, n_tokens, E);
    llama_matmul(lw->w_k, s1, s3, row, n_tokens, E);
    orc_rope_norm_freqs(s2, s2, pos, rope_freqs, n_tokens, H, D, cfg->rope_dim, cfg->rope_base);
    orc_rope_norm_freqs(s3, s3, pos, rope_freqs, n_tokens, HKV, D, cfg->rope_dim, cfg->rope_base);
    orc_kv_cache_write(k_cache, s3, pos, n_tokens, row, cfg->kv_cache_f16);
    llama_matmul(lw->w_v, s1, s3, row, n_tokens, E);
    orc_kv_cache_write(v_cache, s3, pos, n_tokens, row, cfg->kv_cache_f16);
    const size_t n = (size_t)n_kv * row;
    float *kf = (float *)k_cache, *vf = (float *)v_cache;
    if (cfg->kv_cache_f16) {
        kf = (float *)malloc(sizeof(float) * n);
        vf = (float *)malloc(sizeof(float) * n);
        for (size_t i = 0; i < n; i++) {
            kf[i] = orc_f16_to_f32(((const uint16_t *)k_cache)[i]);
            vf[i] = orc_f16_to_f32(((const uint16_t *)v_cache)[i]);
        }
    }
    orc_gqa_attn(s2, kf, vf, s1, n_tokens, n_kv, H, HKV, D, 1.0f / sqrtf((float)D), kv_pos);
    if (cfg->kv_cache_f16) {
        free(kf);
        free(vf);
    }
    llama_matmul(lw->w_o, s1, s2, E, n_tokens, H * D);
    for (long i = 0; i < (long)n_tokens * E; i++) x[i] = x[i] + s2[i];
    orc_rmsnorm_llama(x, lw->ffn_norm_w, s1, n_tokens, E, cfg->rms_eps);
    llama_matmul(lw->w_gate, s1, s2, F, n_tokens, E);
    llama_matmul(lw->w_up, s1, s3, F, n_tokens, E);
    for (long i = 0; i < (long)n_tokens * F; i++) s2[i] = (s2[i] / (1.0f + expf(-s2[i]))) * s3[i];   /* :5504-5507 */
    llama_matmul(lw->w_down, s2, s1, E, n_tokens, F);
    for (long i = 0; i < (long)n_tokens * E; i++) x[i] = x[i] + s1[i];
}

/* bench/bpd_cpu.c:5741-5798 */
int orc_llama_forward(const int32_t *token_ids, int n_tokens, const orc_llama_weights *w, const orc_llama_config *cfg,
                      const int32_t *pos, int kv_pos, void *k_cache, void *v_cache, float *logits, long *token_out)
{
    const int E = cfg->embed_dim, F = cfg->ffn_dim, H = cfg->n_heads, D = cfg->head_dim, HKV = cfg->n_kv_heads;
    const size_t max_dim = (size_t)(E > F ? E : F), max_proj = (size_t)(H * D > F ? H * D : F);
    float *x = (float *)malloc(sizeof(float) * (size_t)n_tokens * E);
    float *s1 = (float *)malloc(sizeof(float) * (size_t)n_tokens * max_dim);
    float *s2 = (float *)malloc(sizeof(float) * (size_t)n_tokens * max_proj);
    float *s3 = (float *)malloc(sizeof(float) * (size_t)n_tokens * max_proj);
    if (!x || !s1 || !s2 || !s3) { free(x); free(s1); free(s2); free(s3); return -1; }
    orc_embed_lookup_q8_0(w->token_embd, token_ids, x, n_tokens, E);
    const size_t layer_bytes = (size_t)cfg->max_seq_len * HKV * D * (cfg->kv_cache_f16 ? 2 : 4);
    for (int l = 0; l < cfg->n_layers; l++)
        orc_llama_block(x, &w->layers[l], cfg, pos, n_tokens, kv_pos, (uint8_t *)k_cache + l * layer_bytes,
                        (uint8_t *)v_cache + l * layer_bytes, s1, s2, s3, w->rope_freqs);
    orc_rmsnorm_llama(x, w->output_norm_w, s1, n_tokens, E, cfg->rms_eps);
    llama_matmul(w->output_w, s1, logits, cfg->vocab_size, n_tokens, E);
    if (token_out) orc_argmax_rows(logits, token_out, n_tokens, cfg->vocab_size);
    free(x); free(s1); free(s2); free(s3);
    return 0;
}
