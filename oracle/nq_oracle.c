/*
 * CPU oracle for the NestQuant quantized routed-expert MoE layer.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA path is compared against and the
 * timed CPU baseline; nothing in the shipped package may link, import or call it.
 *
 * It restates, in plain C, the algorithm of the reference's CPU path:
 *   - window schedule / ring states / hash byte-sum   sm120/ref15_spec.py:43-72, sm120/moe.py:19-22,113-127
 *   - level-2 value and level-4 integer fold          sm120/ref15_spec.py:64-90,  sm120/moe.py:128-134
 *   - packed residual plane ("sub-array") layout      sm120/moe.py:36-63, sm120/nqmoe.cu:146-173
 *   - lane -> matrix index map                        sm120/ref15_spec.py:3-8,118-125, sm120/moe.py:156-166
 *   - mask mode (flagged chunks, compact P4/d4)       sm120/moe.py:146-155, sm120/nqmoe.cu:202-206
 *   - base-variant ring signs                         sm120/moe.py:141-143
 *   - one expert forward (rotations, SwiGLU, low rank, Had512)   sm120/moe.py:196-210
 *
 * Parity pin: tests/test_oracle_golden.py compares every function here with fixtures produced by
 * importing the reference's own sm120/moe.py (tests/golden/make_golden.py).
 *
 * Build: see oracle/Makefile (gcc -O2 -fopenmp -ffp-contract=off; no fast-math: the level-4
 * constants are defined by a fixed sequence of IEEE fp32 operations).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define NQO_NCODES 10
static const int KA_[NQO_NCODES] = {2, 1, 2, 2, 3, 1, 1, 2, 1, 2};
static const int MASK_[NQO_NCODES] = {0x0000, 0xEEEE, 0xAAAA, 0x8888, 0x0000, 0xAAAA, 0xFFFE, 0x9248, 0xFEFE, 0xD5AA};
#define HASH_MUL 0x83DCD12Du

static int popc16(int m) { int c = 0; for (int i = 0; i < 16; ++i) c += (m >> i) & 1; return c; }

/* bits of one lane record for window-pattern code `code` */
int nqo_rbits(int code)
{
    if (code < 0 || code >= NQO_NCODES) return -1;
    return 4 * (16 * KA_[code] + popc16(MASK_[code]));
}

/* bit offset of ring position p: step i is KA + bit (i mod 16) of MASK wide */
static int step_off(int p, int KA, int MASK)
{
    int s = (p >> 4) * (16 * KA + popc16(MASK));
    for (int i = 0; i < (p & 15); ++i) s += KA + ((MASK >> i) & 1);
    return s;
}

/* ---------------------------------------------------------------- fp16 <-> fp32/fp64, round to nearest even */
static uint16_t d2h(double v)
{
    uint16_t s = signbit(v) ? 0x8000u : 0u;
    double a = fabs(v);
    if (a != a) return 0x7E00u;
    if (a == 0.0) return s;
    if (isinf(a)) return s | 0x7C00u;
    int e; (void)frexp(a, &e);          /* a = m * 2^e, m in [0.5, 1) */
    int E = e - 1;                       /* a in [2^E, 2^(E+1)) */
    if (E < -14)
    {
        double q = nearbyint(ldexp(a, 24));   /* subnormal quantum 2^-24 */
        return s | (uint16_t)q;               /* q == 1024 lands on the smallest normal */
    }
    double q = nearbyint(ldexp(a, 10 - E));  /* in [1024, 2048] */
    if (q >= 2048.0) { q = 1024.0; ++E; }
    if (E > 15) return s | 0x7C00u;
    return s | (uint16_t)((E + 15) << 10) | (uint16_t)((int)q - 1024);
}
static float h2f(uint16_t h)
{
    const uint32_t s = (uint32_t)(h & 0x8000u) << 16, e = (h >> 10) & 31u, m = h & 1023u;
    uint32_t u; float f;
    if (e == 0) { f = (float)m * 5.9604644775390625e-8f; memcpy(&u, &f, 4); u |= s; }   /* m * 2^-24, exact */
    else if (e == 31) u = s | 0x7F800000u | (m << 13);
    else u = s | ((e + 112u) << 23) | (m << 13);
    memcpy(&f, &u, 4); return f;
}
uint16_t nqo_f2h(float f) { return d2h((double)f); }
float nqo_h2f(uint16_t h) { return h2f(h); }

/* ---------------------------------------------------------------- level-4 block constants
 * A' = fp16(1.732421875f * (1.0f/Mb)), C = fp16((N * (1.0f/Mb)) * K0 + K0 - 1024 * A'), all in fp32, this order. */
void nqo_fold_consts(int Mb, int N, uint16_t* Ah, uint16_t* Ch)
{
    volatile float rc = 1.0f / (float)Mb;
    volatile float a = 1.732421875f * rc;
    uint16_t ah = nqo_f2h(a);
    volatile float t = (float)N * rc;
    t = t * -3.453125f;
    t = t + -3.453125f;
    volatile float c = t - 1024.0f * h2f(ah);
    *Ah = ah; *Ch = nqo_f2h(c);
}
/* level-2 value from the base byte-sum; sign = +1 / -1 */
uint16_t nqo_q2(int Sb, int neg)
{
    const double A = (double)h2f(0x1eee), B = (double)h2f(0xc931);
    double sg = neg ? -1.0 : 1.0;
    return d2h((sg * A) * (1024.0 + Sb) + sg * B);
}
/* level-4 value from both byte-sums and the block word */
uint16_t nqo_q4(int Sb, int Sr, int Mb, int N, int neg)
{
    uint16_t Ah, Ch; nqo_fold_consts(Mb, N, &Ah, &Ch);
    int F = (Mb * Sb + N * Sr + 128) >> 8;
    double sg = neg ? -1.0 : 1.0;
    return d2h((sg * (double)h2f(Ah)) * (1024.0 + F) + sg * (double)h2f(Ch));
}
static int hash_sum(uint32_t state)
{
    uint32_t x = state * HASH_MUL;
    return (int)((x & 255) + ((x >> 8) & 255) + ((x >> 16) & 255) + (x >> 24));
}
int nqo_hash_sum(uint32_t state) { return hash_sum(state & 0xFFFFu); }

/* ---------------------------------------------------------------- packed plane -> record bit stream
 * A plane of `nrec` records of `bits` bits is a sequence of sub-arrays, each contiguous over all records:
 * 128-bit pieces (record-major, bits/128 per record), then a 64-, 32- and 16-bit piece when that bit of
 * bits%128 is set, then a bit-packed tail of bits%16 bits per record.  Pieces concatenate LSB-first. */
static void put_bits(uint8_t* dst, int dst_bit, const uint8_t* src, size_t src_bit, int n)
{
    for (int i = 0; i < n; ++i)
    {
        size_t sb = src_bit + (size_t)i; int b = (src[sb >> 3] >> (sb & 7)) & 1;
        int db = dst_bit + i; if (b) dst[db >> 3] |= (uint8_t)(1u << (db & 7));
    }
}
/* append record `rec` of the plane to the bit buffer `dst` at bit `dst_bit` */
static void record_bits(uint8_t* dst, int dst_bit, const uint8_t* plane, size_t rec, size_t nrec, int bits)
{
    int n4 = bits / 128, r = bits % 128, o = dst_bit;
    const uint8_t* p = plane;
    if (n4) { put_bits(dst, o, p, rec * (size_t)n4 * 128, n4 * 128); o += n4 * 128; p += nrec * 16 * (size_t)n4; }
    if (r & 64) { put_bits(dst, o, p, rec * 64, 64); o += 64; p += nrec * 8; }
    if (r & 32) { put_bits(dst, o, p, rec * 32, 32); o += 32; p += nrec * 4; }
    if (r & 16) { put_bits(dst, o, p, rec * 16, 16); o += 16; p += nrec * 2; }
    int T = bits % 16;
    if (T) put_bits(dst, o, p, rec * (size_t)T, T);
}
size_t nqo_plane_bytes(size_t nrec, int bits) { return nrec * (size_t)bits / 8 + ((bits % 16) ? 4 : 0); }

/* words of one record (for tests of the layout): out[(bits+31)/32] */
void nqo_record_words(const uint8_t* plane, size_t rec, size_t nrec, int bits, uint32_t* out)
{
    uint8_t buf[32]; memset(buf, 0, sizeof buf);
    record_bits(buf, 0, plane, rec, nrec, bits);
    for (int i = 0; i < (bits + 31) / 32; ++i) memcpy(out + i, buf + 4 * i, 4);
}

/* byte-sums S(state(p)) for the 256 positions of the ring made of records rec0..rec0+3 (tail-biting) */
static void ring_sums(const uint8_t* plane, size_t rec0, size_t nrec, int code, int* S)
{
    const int bits = nqo_rbits(code), L = 4 * bits, KA = KA_[code], MASK = MASK_[code];
    uint8_t buf[4 * 24 + 16]; memset(buf, 0, sizeof buf);
    for (int t4 = 0; t4 < 4; ++t4) record_bits(buf, t4 * bits, plane, rec0 + (size_t)t4, nrec, bits);
    for (int p = 0; p < 256; ++p)
    {
        const int off = step_off(p, KA, MASK);
        uint32_t st = 0;
        for (int i = 0; i < 16; ++i) { int b = (off + i) % L; st |= (uint32_t)((buf[b >> 3] >> (b & 7)) & 1) << i; }
        S[p] = hash_sum(st);
    }
}

/* ---------------------------------------------------------------- dense decode of one projection
 * W: fp16 bit patterns, row-major [N][K].  level 2 or 4.  flags == NULL: every chunk refined at level 4;
 * else chunk c of strip s refined iff bit c of flags[s], P4/d4 compact over the nm flagged chunks of a strip.
 * var == NULL or one byte per unit, bit g = ring g negated.  bk = base window code (0 = plain 128-bit records).
 * returns 0, or a negative code for bad arguments. */
int nqo_decode_proj(const uint8_t* base, const uint8_t* p4, const uint32_t* d4, const uint64_t* flags,
                    const uint8_t* var, int N, int K, int nm, int rk, int bk, int level, uint16_t* W)
{
    if (N % 16 || K % 128 || (level != 2 && level != 4)) return -1;
    if (rk < 0 || rk >= NQO_NCODES || bk < 0 || bk >= NQO_NCODES) return -2;
    const int S = N / 16, C = K / 128, R = flags ? nm : C;
    if (C > 64 || (flags && (nm < 0 || nm > C))) return -3;
    const size_t nrec_b = (size_t)S * C * 32, nrec_r = (size_t)S * R * 32;
    int bad = 0;
#pragma omp parallel for schedule(static) reduction(|:bad)
    for (int s = 0; s < S; ++s)
    {
        int Sb[256], Sr[256];
        for (int c = 0; c < C; ++c)
        {
            const size_t unit = (size_t)s * C + c;
            int on = level == 4; size_t ru = unit;
            if (on && flags)
            {
                const uint64_t fl = flags[s];
                on = (int)((fl >> c) & 1);
                ru = (size_t)s * nm + (size_t)__builtin_popcountll(fl & ((1ull << c) - 1ull));
                if (on && ru >= (size_t)S * nm) { bad = 1; on = 0; }
            }
            int Mb = 1, Nn = 0; uint16_t Ah = 0, Ch = 0;
            if (on) { Mb = d4[ru] & 0xFF; Nn = (d4[ru] >> 8) & 0xFF; if (Mb == 0) { bad = 1; Mb = 1; } nqo_fold_consts(Mb, Nn, &Ah, &Ch); }
            const double Ad = (double)h2f(Ah), Cd = (double)h2f(Ch);
            for (int g = 0; g < 8; ++g)
            {
                ring_sums(base, unit * 32 + (size_t)g * 4, nrec_b, bk, Sb);
                if (on) ring_sums(p4, ru * 32 + (size_t)g * 4, nrec_r, rk, Sr);
                const int neg = var ? (var[unit] >> g) & 1 : 0;
                for (int p = 0; p < 256; ++p)
                {
                    const int t4 = p >> 6, j = p & 63, pp = j >> 1, e = j & 1, t = pp >> 2, r = pp & 3;
                    const int row = 16 * s + g + 8 * (r & 1), k = 128 * c + 16 * t + 2 * t4 + 8 * (r >> 1) + e;
                    uint16_t q;
                    if (on)
                    {
                        const int F = (Mb * Sb[p] + Nn * Sr[p] + 128) >> 8;      /* integer fold, then ONE fp16 rounding */
                        q = d2h(Ad * (1024.0 + F) + Cd);
                        if (neg) q ^= 0x8000u;                                    /* ring sign: exact negation */
                    }
                    else q = nqo_q2(Sb[p], neg);
                    W[(size_t)row * K + k] = q;
                }
            }
        }
    }
    return bad ? -4 : 0;
}

/* ---------------------------------------------------------------- rotations */
/* in-place normalised Sylvester-Hadamard over consecutive blocks of `w` (power of two) fp32 values */
static void wht_blocks(float* v, int n, int w)
{
    const float sc = (float)(1.0 / sqrt((double)w));
    for (int b = 0; b < n; b += w)
    {
        float* x = v + b;
        for (int h = 1; h < w; h <<= 1)
            for (int i = 0; i < w; i += 2 * h)
                for (int j = i; j < i + h; ++j) { float a = x[j], c = x[j + h]; x[j] = a + c; x[j + h] = a - c; }
        for (int i = 0; i < w; ++i) x[i] *= sc;
    }
}
void nqo_wht(float* v, int n, int w) { wht_blocks(v, n, w); }

static void widen(const uint16_t* W, size_t n, float* F)
{
#pragma omp parallel for schedule(static)
    for (long i = 0; i < (long)n; ++i) F[i] = h2f(W[i]);
}
/* Y[t][n] = sum_k X[t][k] * W[n][k]   (fp32 accumulate) */
static void gemm_nt(const float* X, const float* W, float* Y, int T, int N, int K)
{
#pragma omp parallel for schedule(static)
    for (int n = 0; n < N; ++n)
    {
        const float* w = W + (size_t)n * K;
        for (int t = 0; t < T; ++t)
        {
            const float* x = X + (size_t)t * K;
            float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            int k = 0;
            for (; k + 8 <= K; k += 8) for (int i = 0; i < 8; ++i) acc[i] += x[k + i] * w[k + i];
            float a = ((acc[0] + acc[4]) + (acc[1] + acc[5])) + ((acc[2] + acc[6]) + (acc[3] + acc[7]));
            for (; k < K; ++k) a += x[k] * w[k];
            Y[(size_t)t * N + n] = a;
        }
    }
}

/* ---------------------------------------------------------------- one expert, T tokens
 * Wgu [2I][H], Wdn [H][I]: dense fp16 bit patterns (from nqo_decode_proj).
 * scales: fp16 [H su_g | I sv_g | I sv_u | I su_d | H sv_o | H su_u].
 * lr (may be NULL): fp16 [V_gu rg x H | U2_g rg x I | U2_u rg x I | V_dn rd x I | U2_d rd x H];
 * lr4 (used when level == 4): fp16 [U4_g rg x I | U4_u rg x I | U4_d rd x H].
 * had_dn: 128 or 512.  x: fp32 [T][H] holding fp16 values.  y: fp32 [T][H] (overwritten). */
int nqo_expert_forward(const uint16_t* Wgu, const uint16_t* Wdn, const uint16_t* scales, int H, int I, int had_dn,
                       const uint16_t* lr, const uint16_t* lr4, int rg, int rd, int level,
                       const float* x, int T, float* y)
{
    if (H % 128 || I % 128 || (had_dn != 128 && had_dn != 512) || I % had_dn) return -1;
    const uint16_t *su_g = scales, *sv_g = su_g + H, *sv_u = sv_g + I, *su_d = sv_u + I, *sv_o = su_d + I, *su_u = sv_o + H;
    float* Fgu = (float*)malloc(sizeof(float) * 2 * (size_t)I * H);
    float* Fdn = (float*)malloc(sizeof(float) * (size_t)I * H);
    float* xg = (float*)malloc(sizeof(float) * (size_t)T * H);
    float* xu = (float*)malloc(sizeof(float) * (size_t)T * H);
    float* ag = (float*)malloc(sizeof(float) * (size_t)T * I);
    float* au = (float*)malloc(sizeof(float) * (size_t)T * I);
    float* hh = (float*)malloc(sizeof(float) * (size_t)T * I);
    float* sw = (float*)malloc(sizeof(float) * (size_t)T * I);
    if (!Fgu || !Fdn || !xg || !xu || !ag || !au || !hh || !sw) return -2;
    widen(Wgu, 2 * (size_t)I * H, Fgu); widen(Wdn, (size_t)I * H, Fdn);
    for (int t = 0; t < T; ++t)
    {
        for (int k = 0; k < H; ++k)
        {
            xg[(size_t)t * H + k] = x[(size_t)t * H + k] * h2f(su_g[k]);
            xu[(size_t)t * H + k] = x[(size_t)t * H + k] * h2f(su_u[k]);
        }
        wht_blocks(xg + (size_t)t * H, H, 128); wht_blocks(xu + (size_t)t * H, H, 128);
        for (int k = 0; k < H; ++k)
        {
            xg[(size_t)t * H + k] = h2f(nqo_f2h(xg[(size_t)t * H + k]));
            xu[(size_t)t * H + k] = h2f(nqo_f2h(xu[(size_t)t * H + k]));
        }
    }
    gemm_nt(xg, Fgu, ag, T, I, H);
    gemm_nt(xu, Fgu + (size_t)I * H, au, T, I, H);
    const int use_lr = lr != NULL && (rg + rd) > 0;
    for (int t = 0; t < T; ++t)
    {
        float* g = ag + (size_t)t * I; float* u = au + (size_t)t * I;
        wht_blocks(g, I, 128); wht_blocks(u, I, 128);
        for (int i = 0; i < I; ++i) { g[i] *= h2f(sv_g[i]); u[i] *= h2f(sv_u[i]); }
        if (use_lr)
            for (int r = 0; r < rg; ++r)
            {
                float z = 0.f;
                for (int k = 0; k < H; ++k) z += x[(size_t)t * H + k] * h2f(lr[(size_t)r * H + k]);
                const uint16_t* U2g = lr + (size_t)rg * H + (size_t)r * I;
                const uint16_t* U2u = lr + (size_t)rg * H + (size_t)(rg + r) * I;
                for (int i = 0; i < I; ++i)
                {
                    g[i] += z * h2f(U2g[i]); u[i] += z * h2f(U2u[i]);
                    if (level == 4 && lr4) { g[i] += z * h2f(lr4[(size_t)r * I + i]); u[i] += z * h2f(lr4[(size_t)(rg + r) * I + i]); }
                }
            }
        float* s = sw + (size_t)t * I; float* h = hh + (size_t)t * I;
        for (int i = 0; i < I; ++i) { s[i] = g[i] / (1.0f + expf(-g[i])) * u[i]; h[i] = s[i] * h2f(su_d[i]); }
        wht_blocks(h, I, had_dn);
        for (int i = 0; i < I; ++i) h[i] = h2f(nqo_f2h(h[i]));
    }
    gemm_nt(hh, Fdn, y, T, H, I);
    for (int t = 0; t < T; ++t)
    {
        float* o = y + (size_t)t * H;
        wht_blocks(o, H, 128);
        for (int k = 0; k < H; ++k) o[k] *= h2f(sv_o[k]);
        if (use_lr)
            for (int r = 0; r < rd; ++r)
            {
                const uint16_t* Vd = lr + (size_t)rg * H + 2 * (size_t)rg * I + (size_t)r * I;
                const uint16_t* U2d = lr + (size_t)rg * H + 2 * (size_t)rg * I + (size_t)rd * I + (size_t)r * H;
                float z = 0.f;
                for (int i = 0; i < I; ++i) z += sw[(size_t)t * I + i] * h2f(Vd[i]);
                for (int k = 0; k < H; ++k)
                {
                    o[k] += z * h2f(U2d[k]);
                    if (level == 4 && lr4) o[k] += z * h2f(lr4[2 * (size_t)rg * I + (size_t)r * H + k]);
                }
            }
    }
    free(Fgu); free(Fdn); free(xg); free(xu); free(ag); free(au); free(hh); free(sw);
    return 0;
}

int nqo_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
