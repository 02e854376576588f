/*
 * CPU oracle for the ring-packed PCMM hot path of haozetao/ckks_llm.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is a plain-C restatement of the reference's
 * device arithmetic.  It is the checker the CUDA kernels are compared with and the
 * timed CPU baseline of the benchmark; nothing on the product path may call it.
 *
 * Parity status.  The reference holds no golden vectors for this path.  The
 * host-side table builders restated here (root search, psi tables, Shoup companions)
 * are pinned against the reference's own functions, compiled from the reference
 * sources into oracle/_ref/ (see oracle/build_ref.py and tests/test_oracle_vs_ref_host.py),
 * and the NTT / INTT / ModUp / PPMM / decomposition / packing restatements are pinned
 * on a GPU against the reference's own kernels compiled for sm_100a
 * (tests/test_gpu_ref_kernels.py, tests/test_gpu_ringpack.py); digests of those
 * reference-kernel outputs are committed under tests/golden/ and checked on any machine
 * (tests/test_golden.py).
 *
 * Every function cites the reference file:line it follows (paths relative to the
 * reference project root).
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <math.h>
#ifdef _OPENMP
#include <omp.h>
#endif

typedef unsigned __int128 u128;
typedef uint64_t u64;
typedef int64_t i64;

#define ORC_API __attribute__((visibility("default")))

ORC_API int orc_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

ORC_API void orc_set_threads(int n)
{
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/* ---------------------------------------------------------------------------
 * Host helpers: src/ckks/include/Utils.cuh:14-53
 * ------------------------------------------------------------------------- */
ORC_API u64 orc_mulmod(u64 a, u64 b, u64 q) { return (u64)(((u128)a * b) % q); }

ORC_API u64 orc_powmod(u64 a, u64 e, u64 q)
{
    u64 r = 1;
    while (e) {
        if (e & 1) r = orc_mulmod(r, a, q);
        a = orc_mulmod(a, a, q);
        e >>= 1;
    }
    return r;
}

/* a^-1 by Fermat, src/ckks/include/Utils.cuh:48-53 */
ORC_API u64 orc_invmod(u64 a, u64 q) { return orc_powmod(a % q, q - 2, q); }

/* floor(x * 2^64 / q), src/ckks/include/Utils.cuh:40-45 */
ORC_API u64 orc_shoup(u64 x, u64 q) { return (u64)((((u128)x) << 64) / q); }

/* floor(2^128 / q) as (hi, lo): src/ckks/include/pcmm/PCMM_Context.cuh:24-30.
 * 2^128 does not fit a 128-bit word, so divide 2^128-1 instead; the two quotients
 * differ only if q divides 2^128, which no odd q>1 does. */
ORC_API void orc_barrett_mu(u64 q, u64 *hi, u64 *lo)
{
    u128 mu = (~(u128)0) / q;
    *hi = (u64)(mu >> 64);
    *lo = (u64)mu;
}

static uint32_t bitrev32(uint32_t x, int bits)
{
    uint32_t r = 0;
    for (int i = 0; i < bits; i++) { r = (r << 1) | (x & 1); x >>= 1; }
    return r;
}

/* Factor set of `number` exactly as the reference builds it, including its loop
 * bound `i < sqrt(number)` evaluated on the shrinking cofactor and the final
 * `number > 2` insert: src/ckks/include/Utils.cuh:63-77.  Returns the count. */
static int ref_factor_set(u64 number, u64 *out, int cap)
{
    int n = 0;
    int has2 = 0;
    while (number % 2 == 0) { has2 = 1; number /= 2; }
    if (has2 && n < cap) out[n++] = 2;
    for (u64 i = 3; (double)i < sqrt((double)number); i++) {
        int hit = 0;
        while (number % i == 0) { hit = 1; number /= i; }
        if (hit && n < cap) out[n++] = i;
    }
    if (number > 2) {
        int dup = 0;
        for (int k = 0; k < n; k++) if (out[k] == number) dup = 1;
        if (!dup && n < cap) out[n++] = number;
    }
    return n;
}

/* Smallest r>=2 that is not a (phi/f)-th power residue witness for any f in the
 * factor set: src/ckks/include/Utils.cuh:79-97 */
ORC_API u64 orc_find_primitive_root(u64 modulus)
{
    u64 f[64];
    u64 phi = modulus - 1;
    int nf = ref_factor_set(phi, f, 64);
    for (u64 r = 2; r <= phi; r++) {
        int bad = 0;
        for (int k = 0; k < nf; k++) {
            if (orc_powmod(r, phi / f[k], modulus) == 1) { bad = 1; break; }
        }
        if (!bad) return r;
    }
    return (u64)-1;
}

/* src/ckks/include/Utils.cuh:99-109 */
ORC_API u64 orc_find_mth_root(u64 M, u64 q)
{
    u64 g = orc_find_primitive_root(q);
    if ((q - 1) % M != 0) return (u64)-1;
    return orc_powmod(g, (q - 1) / M, q);
}

/* psi / psi^-1 power tables in bit-reversed exponent order with n^-1 folded into
 * psiinv[1], and their Shoup companions:
 * src/ckks/include/Utils.cuh:190-210 (fillTablePsi128_special, fillTablePsi_shoup128). */
ORC_API void orc_fill_tables(u64 psi, u64 q, uint32_t n,
                             u64 *psi_tab, u64 *psiinv_tab,
                             u64 *psi_shoup, u64 *psiinv_shoup)
{
    int logn = 0;
    while ((1u << logn) < n) logn++;
    u64 psiinv = orc_invmod(psi, q);
    u64 ninv = orc_invmod(n, q);
    psi_tab[0] = psiinv_tab[0] = 1;
    for (uint32_t i = 1; i < n; i++) {
        uint32_t prev = bitrev32(i - 1, logn), next = bitrev32(i, logn);
        psi_tab[next] = orc_mulmod(psi, psi_tab[prev], q);
        psiinv_tab[next] = orc_mulmod(psiinv, psiinv_tab[prev], q);
    }
    psiinv_tab[1] = orc_mulmod(psiinv_tab[1], ninv, q);
    for (uint32_t i = 0; i < n; i++) {
        psi_shoup[i] = orc_shoup(psi_tab[i], q);
        psiinv_shoup[i] = orc_shoup(psiinv_tab[i], q);
    }
}

/* ---------------------------------------------------------------------------
 * Device primitives restated: src/ckks/include/uint128.cuh:143-212
 * ------------------------------------------------------------------------- */
static inline u64 csub_q(u64 a, u64 q)
{
    u64 t = a - q;
    return t + (t >> 63) * q;
}

/* mulMod_shoup: src/ckks/include/uint128.cuh:169-180 */
static inline u64 mulmod_shoup(u64 a, u64 b, u64 b_shoup, u64 q)
{
    u64 hi = (u64)(((u128)a * b_shoup) >> 64);
    u64 ra = a * b - hi * q;
    return csub_q(ra, q);
}

/* singleBarrett_new: src/ckks/include/uint128.cuh:183-212, instruction by instruction. */
static inline u64 barrett128(u128 a, u64 q, u64 mu_hi, u64 mu_lo)
{
    u64 alo = (u64)a, ahi = (u64)(a >> 64);
    u64 tmp = (u64)(((u128)alo * mu_lo) >> 64);
    u128 t1 = (u128)alo * mu_hi + tmp;            /* mad.lo.cc / madc.hi */
    u64 lo1 = (u64)t1, r0 = (u64)(t1 >> 64);
    u128 t2 = (u128)ahi * mu_lo + lo1;
    r0 += (u64)(t2 >> 64);
    r0 += ahi * mu_hi;
    u64 res = alo - r0 * q;
    return csub_q(res, q);
}

/* ---------------------------------------------------------------------------
 * Negacyclic NTT over one limb.
 * Forward: Cooley-Tukey, natural in -> bit-reversed out, stage m uses psi[m+i];
 * butterflies are the Harvey lazy form of src/ckks/include/ntt_60bit.cuh:293-307,
 * final reduction to [0,q) as in :669-677.
 * ------------------------------------------------------------------------- */
static void ntt_fwd_one(u64 *a, uint32_t n, u64 q, const u64 *w, const u64 *ws)
{
    u64 q2 = 2 * q;
    uint32_t t = n;
    for (uint32_t m = 1; m < n; m <<= 1) {
        t >>= 1;
        for (uint32_t i = 0; i < m; i++) {
            u64 W = w[m + i], WS = ws[m + i];
            u64 *x = a + 2 * i * t, *y = x + t;
            for (uint32_t j = 0; j < t; j++) {
                u64 A = x[j], B = y[j];
                u64 hi = (u64)(((u128)B * WS) >> 64);
                u64 twb = B * W - hi * q;
                u64 s = A - q2;
                A = s + (s >> 63) * q2;
                y[j] = A + q2 - twb;
                x[j] = A + twb;
            }
        }
    }
    for (uint32_t j = 0; j < n; j++) a[j] = csub_q(csub_q(a[j], q2), q);
}

/* Inverse: Gentleman-Sande, bit-reversed in -> natural out, n^-1 folded into
 * psiinv[1] for the odd half and applied explicitly to the even half:
 * src/ckks/include/ntt_60bit.cuh:309-318, :890-898. */
static void ntt_inv_one(u64 *a, uint32_t n, u64 q, const u64 *w, const u64 *ws,
                        u64 ninv, u64 ninv_s)
{
    u64 q2 = 2 * q;
    uint32_t t = 1;
    for (uint32_t m = n >> 1; m >= 1; m >>= 1) {
        for (uint32_t i = 0; i < m; i++) {
            u64 W = w[m + i], WS = ws[m + i];
            u64 *x = a + 2 * i * t, *y = x + t;
            for (uint32_t j = 0; j < t; j++) {
                u64 A = x[j], B = y[j];
                u64 T = A + q2 - B;
                u64 s = A + B - q2;
                u64 hi = (u64)(((u128)T * WS) >> 64);
                x[j] = s + (s >> 63) * q2;
                y[j] = T * W - hi * q;
            }
        }
        t <<= 1;
        if (m == 1) break;
    }
    uint32_t h = n >> 1;
    for (uint32_t j = 0; j < h; j++) {
        u64 e = a[j];
        u64 hi = (u64)(((u128)e * ninv_s) >> 64);
        e = e * ninv - hi * q;
        a[j] = csub_q(e, q);
        a[j + h] = csub_q(a[j + h], q);
    }
}

/* Batched transform with the addressing of Context_23::ToNTTInplace /
 * FromNTTInplace (src/ckks/include/Context_23.cuh:847-889, ntt_60bit.cuh:446-458):
 * data is [poly][poly_mod_len][n]; limb i of the call uses modulus start_mod_idx+i
 * and sits at limb offset start_limb_off+i.  Tables are [mod][n]. */
ORC_API void orc_ntt_batch(u64 *data, uint32_t n, int start_limb_off, int start_mod_idx,
                           int poly_num, int mod_num, int poly_mod_len,
                           const u64 *moduli, const u64 *tab, const u64 *tab_shoup,
                           int inverse)
{
    long total = (long)poly_num * mod_num;
#pragma omp parallel for schedule(dynamic, 1)
    for (long it = 0; it < total; it++) {
        int p = (int)(it / mod_num), i = (int)(it % mod_num);
        int mod = start_mod_idx + i;
        u64 q = moduli[mod];
        u64 *a = data + ((size_t)p * poly_mod_len + start_limb_off + i) * n;
        const u64 *w = tab + (size_t)mod * n, *ws = tab_shoup + (size_t)mod * n;
        if (!inverse) {
            ntt_fwd_one(a, n, q, w, ws);
        } else {
            u64 ninv = orc_invmod(n, q);
            ntt_inv_one(a, n, q, w, ws, ninv, orc_shoup(ninv, q));
        }
    }
}

/* Brute-force evaluation a(psi^(2*bitrev(j)+1)) for small n: independent check of
 * the ordering convention (no reference line; cross-check only). */
ORC_API void orc_ntt_bruteforce(const u64 *a, u64 *out, uint32_t n, u64 q, u64 psi)
{
    int logn = 0;
    while ((1u << logn) < n) logn++;
#pragma omp parallel for
    for (uint32_t j = 0; j < n; j++) {
        u64 x = orc_powmod(psi, 2 * (u64)bitrev32(j, logn) + 1, q);
        u64 acc = 0, pw = 1;
        for (uint32_t k = 0; k < n; k++) {
            acc = (u64)(((u128)a[k] * pw + acc) % q);
            pw = orc_mulmod(pw, x, q);
        }
        out[j] = acc;
    }
}

/* ---------------------------------------------------------------------------
 * ModUp of Q-digits to the T basis: modUpQjtoT_23_kernel,
 * src/ckks/include/BasisConv.cuh:84-159; tables src/ckks/include/Context_23.cuh:286-351.
 *   in  [batch][q_num][n]      out [batch][Qj_blockNum][t_num][n]
 * alpha = p_num limbs per digit; level l; blocks = ceil((l+1)/alpha).
 * ------------------------------------------------------------------------- */
ORC_API void orc_modup_tables(const u64 *q, int q_num, const u64 *t, int t_num, int alpha,
                              int l, u64 *hat_inv, u64 *hat_inv_shoup, u64 *hat_mod_t,
                              u64 *blk_mod_t)
{
    /* hat_inv[blk*alpha+j], hat_mod_t[(blk*t_num+k)*alpha+j], blk_mod_t[blk*t_num+k] */
    int blocks = (l + 1 + alpha - 1) / alpha;
    (void)q_num;
    for (int b = 0; b < blocks; b++) {
        for (int j = 0; j < alpha && b * alpha + j <= l; j++) {
            u64 qj = q[b * alpha + j];
            u64 prod = 1;
            for (int jj = 0; jj < alpha && b * alpha + jj <= l; jj++) {
                if (jj == j) continue;
                prod = orc_mulmod(prod, q[b * alpha + jj], qj);
            }
            u64 inv = orc_invmod(prod, qj);
            hat_inv[b * alpha + j] = inv;
            hat_inv_shoup[b * alpha + j] = orc_shoup(inv, qj);
        }
        for (int k = 0; k < t_num; k++) {
            u64 tk = t[k];
            for (int j = 0; j < alpha && b * alpha + j <= l; j++) {
                u64 prod = 1;
                for (int jj = 0; jj < alpha && b * alpha + jj <= l; jj++) {
                    if (jj == j) continue;
                    prod = orc_mulmod(prod, q[b * alpha + jj], tk);
                }
                hat_mod_t[((size_t)b * t_num + k) * alpha + j] = prod;
            }
            u64 full = 1;
            for (int j = 0; j < alpha && b * alpha + j <= l; j++)
                full = orc_mulmod(full, q[b * alpha + j], tk);
            blk_mod_t[b * t_num + k] = full;
        }
    }
}

ORC_API void orc_modup(u64 *out, const u64 *in, uint32_t n, const u64 *q, int q_num,
                       const u64 *t, int t_num, int alpha, int l, int batch)
{
    int blocks = (l + 1 + alpha - 1) / alpha;
    u64 *hat_inv = calloc((size_t)blocks * alpha, 8);
    u64 *hat_inv_s = calloc((size_t)blocks * alpha, 8);
    u64 *hat_mod_t = calloc((size_t)blocks * t_num * alpha, 8);
    u64 *blk_mod_t = calloc((size_t)blocks * t_num, 8);
    u64 *mu_hi = calloc(t_num, 8), *mu_lo = calloc(t_num, 8);
    orc_modup_tables(q, q_num, t, t_num, alpha, l, hat_inv, hat_inv_s, hat_mod_t, blk_mod_t);
    for (int k = 0; k < t_num; k++) orc_barrett_mu(t[k], &mu_hi[k], &mu_lo[k]);

    long total = (long)batch * blocks;
#pragma omp parallel for schedule(dynamic, 1)
    for (long it = 0; it < total; it++) {
        int bt = (int)(it / blocks), b = (int)(it % blocks);
        for (uint32_t x = 0; x < n; x++) {
            u64 rb[64];
            double vv = 0.0;
            int cnt = 0;
            for (int j = 0; j < alpha && j + b * alpha < l + 1; j++) {
                int idx = j + b * alpha;
                u64 qi = q[idx];
                u64 ra = in[((size_t)bt * q_num + idx) * n + x];
                rb[j] = mulmod_shoup(ra, hat_inv[idx], hat_inv_s[idx], qi);
                vv += (double)rb[j] / (double)qi;                 /* BasisConv.cuh:113-114 */
                cnt++;
            }
            int v = (int)vv;                                       /* :152 */
            for (int k = 0; k < t_num; k++) {
                u128 acc = 0;
                for (int j = 0; j < cnt; j++)
                    acc += (u128)rb[j] * hat_mod_t[((size_t)b * t_num + k) * alpha + j];
                u64 sub = (u64)(i64)v * blk_mod_t[b * t_num + k];  /* 64-bit product, :153 */
                acc -= (u128)sub;                                  /* sub_uint128_uint64 */
                out[(((size_t)bt * blocks + b) * t_num + k) * n + x] =
                    barrett128(acc, t[k], mu_hi[k], mu_lo[k]);
            }
        }
    }
    free(hat_inv); free(hat_inv_s); free(hat_mod_t); free(blk_mod_t); free(mu_hi); free(mu_lo);
}

/* ---------------------------------------------------------------------------
 * PPMM: src/ckks/include/pcmm/PPMM_kernel.cuh:12-31 (MAC and sign rule),
 * :124-250 (limb order, Barrett, rescale by the last limb, output index),
 * rescale constants src/ckks/include/Context_23.cuh:424-434.
 *   W      fp32 [M][K] row-major
 *   X[n]   pointer to ciphertext n: [limbs][C] words, C=(rank+1)*N1
 *   out    [M][limbs][C]
 * Rows [m0, m1) only are computed (so a sample of rows can be timed/checked).
 * ------------------------------------------------------------------------- */
ORC_API void orc_ppmm(const float *W, const u64 *const *X, u64 *out, int M, int K, long C,
                      int limbs, const u64 *q, double scaler, int m0, int m1)
{
    u64 *inv = calloc(limbs, 8), *inv_s = calloc(limbs, 8);
    u64 *mu_hi = calloc(limbs, 8), *mu_lo = calloc(limbs, 8);
    for (int i = 0; i < limbs; i++) {
        orc_barrett_mu(q[i], &mu_hi[i], &mu_lo[i]);
        if (i < limbs - 1) {
            inv[i] = orc_invmod(q[limbs - 1], q[i]);
            inv_s[i] = orc_shoup(inv[i], q[i]);
        }
    }
    (void)M;
    const long CT = 256;                       /* column tile kept in cache */
    long ntile = (C + CT - 1) / CT;
    long jobs = (long)(m1 - m0) * ntile;
#pragma omp parallel for schedule(dynamic, 4)
    for (long job = 0; job < jobs; job++) {
        int m = m0 + (int)(job / ntile);
        long c0 = (job % ntile) * CT, c1 = c0 + CT < C ? c0 + CT : C;
        u128 acc[256];
        u64 last[256];
        for (int i = limbs - 1; i >= 0; i--) {
            u64 qi = q[i];
            for (long c = c0; c < c1; c++) acc[c - c0] = 0;
            for (int n = 0; n < K; n++) {
                i64 w = (i64)((double)W[(size_t)m * K + n] * scaler);   /* :148 */
                u64 a = w > 0 ? (u64)w : qi + (u64)w;                  /* :23-25 */
                const u64 *xr = X[n] + (size_t)i * C;
                for (long c = c0; c < c1; c++) acc[c - c0] += (u128)a * xr[c];
            }
            u64 *orow = out + ((size_t)m * limbs + i) * C;
            if (i == limbs - 1) {
                for (long c = c0; c < c1; c++) {
                    u64 r = barrett128(acc[c - c0], qi, mu_hi[i], mu_lo[i]);
                    orow[c] = r;
                    last[c - c0] = r;
                }
            } else {
                for (long c = c0; c < c1; c++) {
                    u64 r = barrett128(acc[c - c0], qi, mu_hi[i], mu_lo[i]);
                    u64 tmp = r + qi - last[c - c0];                   /* :244, wraps mod 2^64 */
                    orow[c] = mulmod_shoup(tmp, inv[i], inv_s[i], qi);  /* :247 */
                }
            }
        }
    }
    free(inv); free(inv_s); free(mu_hi); free(mu_lo);
}

/* ---------------------------------------------------------------------------
 * Ring packing helpers for the end-to-end decrypt check.
 * ------------------------------------------------------------------------- */
static inline u64 negate_mod(u64 x, u64 q) { return x == 0 ? 0 : q - x; }

/* RLWE (coefficient domain) -> mlwe_num MLWE ciphertexts of rank k:
 * rlweCipherDecompose_kernel, src/ckks/include/pcmm/PCMM_Scheme.cuh:51-88.
 *   rlwe_a, rlwe_b : [limbs][N]     mlwe[i] : [limbs][(k+1)][N1] */
ORC_API void orc_rlwe_decompose(const u64 *rlwe_a, const u64 *rlwe_b, u64 *const *mlwe,
                                long N, int N1, int k, int mlwe_num, int limbs, const u64 *q)
{
    int gap = k / mlwe_num;
    for (int i = 0; i < mlwe_num; i++) {
        for (int l = 0; l < limbs; l++) {
            const u64 *A = rlwe_a + (size_t)l * N, *B = rlwe_b + (size_t)l * N;
            u64 *ax = mlwe[i] + (size_t)l * (k + 1) * N1;
            u64 *bx = ax + (size_t)k * N1;
            for (int g = 0; g < N1; g++) {
                long addr = (long)i * gap + (long)g * k;
                int over = addr >= N;
                ax[g] = over ? negate_mod(A[addr - N], q[l]) : A[addr];
                bx[g] = over ? negate_mod(B[addr - N], q[l]) : B[addr];
                for (int r = 1; r < k; r++) {
                    if (g == 0) {
                        addr = (long)(N1 - 1) * k + (k - r) + (long)i * gap;
                        over = addr >= N;
                        ax[g + (size_t)r * N1] = over ? A[addr - N] : negate_mod(A[addr], q[l]);
                    } else {
                        addr = (long)(g - 1) * k + (k - r) + (long)i * gap;
                        over = addr >= N;
                        ax[g + (size_t)r * N1] = over ? negate_mod(A[addr - N], q[l]) : A[addr];
                    }
                }
            }
        }
    }
}

/* MLWE secret from the RLWE secret: ringDown_kernel,
 * src/ckks/include/pcmm/ringSwitch.cuh:7-19.  s_r[j] = S[r + j*k]. */
ORC_API void orc_ring_down(const i64 *S, i64 *s_mlwe, long N, int N1, int k)
{
    for (long g = 0; g < N; g++) s_mlwe[g] = S[g / N1 + (g % N1) * k];
}

/* MLWE decryption m = b + sum_r a_r * s_r in Z_q[X]/(X^N1+1) for one limb:
 * mlweDecrypt_kernel, src/ckks/include/pcmm/PCMM_Scheme.cuh:533-555 (the reference
 * multiplies in the N1-point NTT domain; the product is the same ring element). */
ORC_API void orc_mlwe_decrypt(const u64 *ct, const i64 *s_mlwe, u64 *m, int N1, int k, u64 q)
{
#pragma omp parallel for
    for (int j = 0; j < N1; j++) {
        u128 pos = ct[(size_t)k * N1 + j];
        u128 neg = 0;
        for (int r = 0; r < k; r++) {
            const u64 *a = ct + (size_t)r * N1;
            const i64 *s = s_mlwe + (size_t)r * N1;
            for (int u = 0; u < N1; u++) {
                i64 sv;
                int sign;
                if (u <= j) { sv = s[j - u]; sign = 1; }
                else { sv = s[j - u + N1]; sign = -1; }
                if (sv == 0) continue;
                if ((sv > 0) == (sign > 0)) pos += (u128)a[u] * (u64)(sv > 0 ? sv : -sv);
                else neg += (u128)a[u] * (u64)(sv > 0 ? sv : -sv);
            }
        }
        u64 p = (u64)(pos % q), ng = (u64)(neg % q);
        m[j] = p >= ng ? p - ng : p + q - ng;
    }
}

/* Negacyclic product c = a*s in Z_q[X]/(X^N+1) with a small signed s (schoolbook;
 * used by the test-side RLWE encryption for small N only). */
ORC_API void orc_negacyclic_mul_small(const u64 *a, const i64 *s, u64 *c, long N, u64 q)
{
#pragma omp parallel for
    for (long j = 0; j < N; j++) {
        u128 pos = 0, neg = 0;
        for (long u = 0; u < N; u++) {
            i64 sv;
            int sign;
            if (u <= j) { sv = s[j - u]; sign = 1; }
            else { sv = s[j - u + N]; sign = -1; }
            if (sv == 0) continue;
            u64 mag = (u64)(sv > 0 ? sv : -sv);
            if ((sv > 0) == (sign > 0)) pos += (u128)a[u] * mag;
            else neg += (u128)a[u] * mag;
        }
        u64 p = (u64)(pos % q), ng = (u64)(neg % q);
        c[j] = p >= ng ? p - ng : p + q - ng;
    }
}

/* ---------------------------------------------------------------------------
 * MLWE -> RLWE packing, stage by stage (PCMM_Scheme::mlweCipherPacking,
 * src/ckks/include/pcmm/PCMM_Scheme.cuh:362-430).  The reference's kernels are written
 * for one special prime p and one packing limb q0 (ring-pack moduli {p | q0, q1}); the
 * same restriction holds here.  Limb order in every buffer: [p, q0].
 * ------------------------------------------------------------------------- */

/* mlweCipherEmbedding_new_kernel (:312-359) after the memset of :397.
 *   mlwe[i] : MLWE ciphertext i, limb 0 = [(k+1)][N1]
 *   E       : (k+1) polynomials (a_0..a_{k-1}, b), each [2 limbs][N]
 * coefficient g of ciphertext i lands at position g*k + i*gap; the p limb receives the
 * centred lift of the q0 residue. */
ORC_API void orc_pack_embed(const u64 *const *mlwe, u64 *E, long N, int N1, int k, int mlwe_num,
                            u64 p, u64 q0)
{
    int gap = k / mlwe_num;
    memset(E, 0, sizeof(u64) * (size_t)(k + 1) * 2 * N);
    for (int i = 0; i < mlwe_num; i++)
        for (int r = 0; r <= k; r++)
            for (int g = 0; g < N1; g++) {
                u64 v = mlwe[i][(size_t)r * N1 + g];
                long pos = (long)g * k + (long)i * gap;
                u64 *poly = E + (size_t)r * 2 * N;
                poly[N + pos] = v;
                poly[pos] = v > (q0 / 2) ? (p - (q0 - v)) % p : v;
            }
}

/* mlweCipherMultRepackingKey_kernel (:261-289): E_ntt is the first k polynomials of E in the
 * NTT domain; keys [k][2 (a,b)][2 limbs][N]; O [2 (a,b)][2 limbs][N]. */
ORC_API void orc_pack_keymac(const u64 *E_ntt, const u64 *keys, u64 *O, long N, int k, const u64 *mods)
{
    for (int m = 0; m < 2; m++) {
        u64 mu_hi, mu_lo;
        orc_barrett_mu(mods[m], &mu_hi, &mu_lo);
#pragma omp parallel for
        for (long n = 0; n < N; n++) {
            u128 acc_a = 0, acc_b = 0;
            for (int i = 0; i < k; i++) {
                u64 c = E_ntt[((size_t)i * 2 + m) * N + n];
                const u64 *key = keys + (size_t)i * 4 * N;
                acc_a += (u128)c * key[(size_t)m * N + n];
                acc_b += (u128)c * key[(size_t)(m + 2) * N + n];
            }
            O[(size_t)m * N + n] = barrett128(acc_a, mods[m], mu_hi, mu_lo);
            O[(size_t)(2 + m) * N + n] = barrett128(acc_b, mods[m], mu_hi, mu_lo);
        }
    }
}

/* ringpacking_ModDown_kernel (:291-308) on coefficient-domain O [2][2 limbs][N]:
 * out_c = (x_q + q - (x_p mod q)) * p^-1 mod q  (no centring of x_p), c in {a, b}. */
ORC_API void orc_pack_moddown(const u64 *O, u64 *out_a, u64 *out_b, long N, u64 p, u64 q0)
{
    u64 pinv = orc_invmod(p % q0, q0), pinv_s = orc_shoup(pinv, q0);
    for (int c = 0; c < 2; c++) {
        u64 *out = c ? out_b : out_a;
        for (long n = 0; n < N; n++) {
            u64 ra = O[((size_t)c * 2) * N + n] % q0;
            ra = q0 - ra + O[((size_t)c * 2 + 1) * N + n];
            out[n] = mulmod_shoup(ra, pinv, pinv_s, q0);
        }
    }
}


/* ---------------------------------------------------------------------------
 * Level changes around the PCMM: the elementwise kernels of Scheme_23::rescaleAndEqual and
 * Bootstrapper::modUpQ0toQL.  Cipher buffers are [2][stride][n]; q points at the q moduli.
 * ------------------------------------------------------------------------- */

/* mod_to_qi: src/ckks/include/Scheme_23.cuh:356-366 with barrett_reduce_uint64_uint64
 * (uint128.cuh:214-225): s = hi64(mu_hi * x), a = x - s*q, one conditional subtraction;
 * mu_hi = high word of floor(2^128/q).  The value may stay in [q, 2q) like the reference's. */
ORC_API void orc_mod_to_qi(u64 *buf, const u64 *cipher, uint32_t n, int stride, int l, const u64 *q)
{
#pragma omp parallel for collapse(2)
    for (int c = 0; c < 2; c++)
        for (int i = 0; i < l; i++) {
            u64 qi = q[i];
            u64 mu_hi = (u64)((~(u128)0 / qi) >> 64);
            for (uint32_t x = 0; x < n; x++) {
                u64 rb = cipher[((size_t)c * stride + l) * n + x];
                u64 s = (u64)(((u128)mu_hi * rb) >> 64);
                u64 a = rb - s * qi;
                buf[((size_t)c * stride + i) * n + x] = csub_q(a, qi);
            }
        }
}

/* rescaleAndEqual_new_kernel: src/ckks/include/Scheme_23.cuh:339-354.
 * qinv[i] = q_l^-1 mod q_i with its Shoup companion. */
ORC_API void orc_rescale_combine(u64 *cipher, const u64 *buf, uint32_t n, int stride, int l, const u64 *q,
                                 const u64 *qinv, const u64 *qinv_shoup)
{
#pragma omp parallel for collapse(2)
    for (int c = 0; c < 2; c++)
        for (int i = 0; i < l; i++) {
            u64 qi = q[i];
            for (uint32_t x = 0; x < n; x++) {
                size_t idx = ((size_t)c * stride + i) * n + x;
                u64 ra = cipher[idx] + 2 * qi - buf[idx];
                ra = csub_q(ra, qi);
                cipher[idx] = mulmod_shoup(ra, qinv[i], qinv_shoup[i], qi);
            }
        }
}

/* modUpQ0toQL_kernel: src/ckks/include/bootstrapping/Bootstrapping.cuh:6-23.  The C expression
 * int64_t(ra) - q0 + (qi * scale_up) mixes int64, uint64 and int operands and is therefore
 * evaluated in uint64; temp %= qi likewise. */
ORC_API void orc_modup_q0_to_ql(u64 *cipher, uint32_t n, int stride, int target_level, const u64 *q, int scale_up)
{
#pragma omp parallel for collapse(2)
    for (int c = 0; c < 2; c++)
        for (int i = 0; i < target_level; i++) {
            u64 qi = q[i + 1], q0 = q[0];
            for (uint32_t x = 0; x < n; x++) {
                u64 ra = cipher[(size_t)c * stride * n + x];
                int64_t temp;
                if (ra > q0 / 2)
                    temp = (int64_t)((u64)(int64_t)ra - q0 + (qi * (u64)(int64_t)scale_up));
                else
                    temp = (int64_t)ra;
                temp = (int64_t)((u64)temp % qi);
                cipher[((size_t)c * stride + i + 1) * n + x] = (u64)temp;
            }
        }
}

/* ---------------------------------------------------------------------------
 * Key-switch chain of the CKKS-23 evaluator (Scheme_23::mult_23, KeySwitch_23.cuh:192-236).
 * R = Ri_blockNum = ceil((p_num+q_num)/gamma); tables are passed in by the caller.
 * ------------------------------------------------------------------------- */

/* external_product_T_kernel: src/ckks/include/ExternalProduct.cuh:7-48 */
ORC_API void orc_external_product_t(u64 *out, const u64 *cipher, const u64 *swk, uint32_t n, int t_num, int R,
                                    int cipher_blocks, int blocks, int dnum, const u64 *t)
{
#pragma omp parallel for collapse(2)
    for (int blk = 0; blk < blocks; blk++)
        for (int k = 0; k < t_num; k++) {
            u64 tk = t[k], mu_hi, mu_lo;
            orc_barrett_mu(tk, &mu_hi, &mu_lo);
            for (uint32_t x = 0; x < n; x++)
                for (int h = 0; h < 2; h++) {
                    u128 acc = 0;
                    for (int i = 0; i < cipher_blocks; i++) {
                        u64 ra = cipher[((size_t)i * t_num + k) * n + x];
                        u64 rb = swk[(size_t)h * R * t_num * dnum * n +
                                     ((size_t)i * t_num * R + (size_t)blk * t_num + k) * n + x];
                        acc += (u128)ra * rb;
                    }
                    out[(size_t)h * R * t_num * n + ((size_t)blk * t_num + k) * n + x] = barrett128(acc, tk, mu_hi, mu_lo);
                }
        }
}

/* modUpTtoPQl_23_kernel: src/ckks/include/BasisConv.cuh:183-235.
 * pq = [p | q] moduli; t_hat_inv(+shoup)[t_num]; t_hat_mod_r[(p_num+q_num)][t_num]; half_t over [p | q | t];
 * t_mod_pq[p_num+q_num]. */
ORC_API void orc_modup_t_to_pql(u64 *out, const u64 *in, uint32_t n, int p_num, int q_num, int t_num, int l, int gamma,
                                int batch, const u64 *pq, const u64 *t, const u64 *t_hat_inv, const u64 *t_hat_inv_shoup,
                                const u64 *t_hat_mod_r, const u64 *half_t, const u64 *t_mod_pq)
{
    int R = (p_num + q_num + gamma - 1) / gamma;
    int blocks = (p_num + l + 1 + gamma - 1) / gamma;
#pragma omp parallel for collapse(2)
    for (int c = 0; c < batch; c++)
        for (int blk = 0; blk < blocks; blk++)
            for (uint32_t x = 0; x < n; x++) {
                u64 rb[64];
                double vv = 0;
                for (int i = 0; i < t_num; i++) {
                    u64 ra = in[(size_t)c * R * t_num * n + ((size_t)blk * t_num + i) * n + x];
                    ra = ra + half_t[p_num + q_num + i];
                    rb[i] = mulmod_shoup(ra, t_hat_inv[i], t_hat_inv_shoup[i], t[i]);
                    double rr = (double)rb[i];
                    vv += rr / (double)t[i];
                }
                int vv_floor = (int)vv;
                for (int j = 0; j < gamma && j + blk * gamma < p_num + l + 1; j++) {
                    int r = j + blk * gamma;
                    u64 ri = pq[r], mu_hi, mu_lo;
                    orc_barrett_mu(ri, &mu_hi, &mu_lo);
                    u128 acc = 0;
                    for (int i = 0; i < t_num; i++) acc += (u128)rb[i] * t_hat_mod_r[(size_t)r * t_num + i];
                    acc -= (u128)((u64)vv_floor * t_mod_pq[r]);          /* sub_uint128_uint64: wraps like the kernel */
                    u64 lo = barrett128(acc, ri, mu_hi, mu_lo);
                    lo = lo + ri - half_t[r];
                    out[(size_t)c * R * t_num * n + (size_t)r * n + x] = csub_q(lo, ri);
                }
            }
}

/* modDownPQltoQl_23_multi_kernel and _alpha1_multi_kernel: src/ckks/include/BasisConv.cuh:251-325 */
ORC_API void orc_moddown_pql_to_ql(u64 *out, const u64 *in, uint32_t n, int p_num, int q_num, int t_num, int l, int gamma,
                                   int batch, const u64 *pq, const u64 *p_hat_inv, const u64 *p_hat_inv_shoup,
                                   const u64 *p_hat_mod_q, const u64 *p_inv_mod_q, const u64 *p_inv_mod_q_shoup)
{
    int R = (p_num + q_num + gamma - 1) / gamma;
#pragma omp parallel for collapse(2)
    for (int c = 0; c < batch; c++)
        for (int i = 0; i <= l; i++) {
            u64 qi = pq[p_num + i], mu_hi, mu_lo;
            orc_barrett_mu(qi, &mu_hi, &mu_lo);
            const u64 *src = in + (size_t)c * R * t_num * n;
            for (uint32_t x = 0; x < n; x++) {
                u64 part;
                if (p_num == 1) {
                    part = src[x] % qi;
                } else {
                    u128 acc = 0;
                    for (int j = 0; j < p_num; j++) {
                        u64 rb = mulmod_shoup(src[(size_t)j * n + x], p_hat_inv[j], p_hat_inv_shoup[j], pq[j]);
                        acc += (u128)rb * p_hat_mod_q[(size_t)i * p_num + j];
                    }
                    part = barrett128(acc, qi, mu_hi, mu_lo);
                }
                u64 d = qi - part + src[(size_t)(p_num + i) * n + x];
                out[((size_t)c * q_num + i) * n + x] = mulmod_shoup(d, p_inv_mod_q[i], p_inv_mod_q_shoup[i], qi);
            }
        }
}

/* compute_c0c1c2_kernel: src/ckks/include/poly_arithmetic.cuh:787-818.  c1, c2: [2][stride][n]. */
ORC_API void orc_tensor_product(u64 *axbx, u64 *axax, u64 *bxbx, const u64 *c1, const u64 *c2, uint32_t n, int stride,
                                int limbs, const u64 *q)
{
#pragma omp parallel for
    for (int i = 0; i < limbs; i++) {
        u64 qi = q[i], mu_hi, mu_lo;
        orc_barrett_mu(qi, &mu_hi, &mu_lo);
        for (uint32_t x = 0; x < n; x++) {
            size_t a = (size_t)i * n + x, b = ((size_t)stride + i) * n + x;
            u64 ra1 = c1[a], rb1 = c1[b], ra2 = c2[a], rb2 = c2[b];
            u128 t1 = (u128)ra1 * ra2, t2 = (u128)rb1 * rb2;
            u128 t3 = (u128)(ra1 + rb1) * (ra2 + rb2);
            t3 -= t1;
            t3 -= t2;
            axax[a] = barrett128(t1, qi, mu_hi, mu_lo);
            bxbx[a] = barrett128(t2, qi, mu_hi, mu_lo);
            axbx[a] = barrett128(t3, qi, mu_hi, mu_lo);
        }
    }
}

/* cipher_add_axbx_batch_device_kernel: src/ckks/include/poly_arithmetic.cuh:155-172 */
ORC_API void orc_add_switched(u64 *cipher, const u64 *ax, const u64 *bx, uint32_t n, int stride, int limbs, const u64 *q)
{
#pragma omp parallel for
    for (int i = 0; i < limbs; i++)
        for (uint32_t x = 0; x < n; x++) {
            size_t a = (size_t)i * n + x, b = ((size_t)stride + i) * n + x;
            cipher[a] = csub_q(cipher[a] + ax[a], q[i]);
            cipher[b] = csub_q(cipher[b] + bx[a], q[i]);
        }
}
