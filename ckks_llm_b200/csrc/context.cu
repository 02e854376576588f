// Context creation: host-side table construction and upload.
#include <math.h>
#include <stdarg.h>

#include <atomic>

#include "context.cuh"

namespace ckb {

static thread_local char g_err[512] = "";
void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}
const char* get_error() { return g_err; }

std::atomic<long> g_launches{0};

static uint32_t bitrev(uint32_t x, int bits) {
    uint32_t r = 0;
    for (int i = 0; i < bits; i++) r |= ((x >> i) & 1u) << (bits - 1 - i);
    return r;
}

// The reference searches for a generator by trial: it collects the divisors it finds
// for q-1 by trial division with the bound "i < sqrt(remaining cofactor)" and adds
// the remaining cofactor when it exceeds 2 (src/ckks/include/Utils.cuh:63-97).  The
// bound is strict, so a cofactor that is the square of a prime enters the set as the
// square.  The same set is built here so the same generator, hence the same psi and
// the same NTT output order, results.
static std::vector<u64> divisor_set(u64 n) {
    std::vector<u64> s;
    if ((n & 1) == 0) {
        s.push_back(2);
        while ((n & 1) == 0) n >>= 1;
    }
    for (u64 d = 3; (double)d < sqrt((double)n); d++) {
        if (n % d) continue;
        s.push_back(d);
        do n /= d; while (n % d == 0);
    }
    if (n > 2) {
        bool seen = false;
        for (u64 v : s) seen |= (v == n);
        if (!seen) s.push_back(n);
    }
    return s;
}

u64 find_mth_root(u64 M, u64 q) {
    if ((q - 1) % M) return 0;
    const u64 phi = q - 1;
    std::vector<u64> fs = divisor_set(phi);
    for (u64 g = 2; g <= phi; g++) {
        bool generator = true;
        for (u64 f : fs)
            if (h_powmod(g, phi / f, q) == 1) { generator = false; break; }
        if (generator) return h_powmod(g, phi / M, q);
    }
    return 0;
}

// tab[bitrev(e)] = psi^e, tabinv[bitrev(e)] = psi^-e, then tabinv[1] *= n^-1
// (src/ckks/include/Utils.cuh:190-201).
void fill_psi_tables(u64 psi, u64 q, uint32_t n, std::vector<u64>& tab, std::vector<u64>& tabinv) {
    int logn = 0;
    while ((1u << logn) < n) logn++;
    tab.assign(n, 0);
    tabinv.assign(n, 0);
    const u64 psiinv = h_invmod(psi, q);
    u64 pw = 1, pwi = 1;
    for (uint32_t e = 0; e < n; e++) {
        uint32_t at = bitrev(e, logn);
        tab[at] = pw;
        tabinv[at] = pwi;
        pw = h_mulmod(pw, psi, q);
        pwi = h_mulmod(pwi, psiinv, q);
    }
    tabinv[1] = h_mulmod(tabinv[1], h_invmod(n % q, q), q);
}

int ensure_buf(u64** buf, size_t* cap, size_t words) {
    if (*cap >= words) return CKKS_B200_OK;
    if (*buf) cudaFree(*buf);
    *buf = nullptr;
    *cap = 0;
    if (cudaMalloc(buf, words * sizeof(u64)) != cudaSuccess) {
        set_error("cudaMalloc of %zu bytes failed", words * sizeof(u64));
        return CKKS_B200_ERR_NOMEM;
    }
    *cap = words;
    return CKKS_B200_OK;
}

static bool is_prime(u64 n) {
    if (n < 4) return n >= 2;
    if ((n & 1) == 0) return false;
    u64 d = n - 1;
    int r = 0;
    while ((d & 1) == 0) { d >>= 1; r++; }
    const u64 bases[] = {2, 3, 5, 7, 11, 13, 17, 19, 23, 29, 31, 37};
    for (u64 a : bases) {
        if (a % n == 0) continue;
        u64 x = h_powmod(a, d, n);
        if (x == 1 || x == n - 1) continue;
        bool comp = true;
        for (int i = 1; i < r; i++) {
            x = h_mulmod(x, x, n);
            if (x == n - 1) { comp = false; break; }
        }
        if (comp) return false;
    }
    return true;
}

}  // namespace ckb

using namespace ckb;

template <class T>
static int upload(T** dst, const std::vector<T>& src) {
    if (src.empty()) { *dst = nullptr; return CKKS_B200_OK; }
    CKB_CUDA(cudaMalloc(dst, src.size() * sizeof(T)));
    CKB_CUDA(cudaMemcpy(*dst, src.data(), src.size() * sizeof(T), cudaMemcpyHostToDevice));
    return CKKS_B200_OK;
}

extern "C" int ckks_b200_context_create(ckks_b200_context** out, int device, int logN,
                                        const uint64_t* p, int p_num, const uint64_t* q, int q_num,
                                        const uint64_t* t, int t_num) {
    CKB_REQUIRE(out != nullptr, CKKS_B200_ERR_ARG, "out is null");
    *out = nullptr;
    CKB_REQUIRE(logN >= 12 && logN <= 16, CKKS_B200_ERR_UNSUPPORTED,
                "logN=%d outside the supported range [12,16]", logN);
    CKB_REQUIRE(p_num >= 0 && q_num >= 1 && t_num >= 0, CKKS_B200_ERR_ARG, "bad modulus counts");
    CKB_REQUIRE((p_num == 0 || p) && q && (t_num == 0 || t), CKKS_B200_ERR_ARG, "null modulus list");
    CKB_REQUIRE(p_num <= 16, CKKS_B200_ERR_UNSUPPORTED, "alpha=p_num=%d exceeds 16", p_num);
    int ndev = 0;
    CKB_CUDA(cudaGetDeviceCount(&ndev));
    CKB_REQUIRE(device >= 0 && device < ndev, CKKS_B200_ERR_ARG, "device %d of %d", device, ndev);
    DeviceGuard guard(device);
    CKB_REQUIRE(guard.ok, CKKS_B200_ERR_CUDA, "cudaSetDevice(%d) failed", device);

    ckks_b200_context* c = new (std::nothrow) ckks_b200_context();
    CKB_REQUIRE(c != nullptr, CKKS_B200_ERR_NOMEM, "host allocation failed");
    c->device = device;
    c->logN = logN;
    c->N = 1u << logN;
    c->p_num = p_num; c->q_num = q_num; c->t_num = t_num;
    c->mod_num = p_num + q_num + t_num;
    c->alpha = p_num > 0 ? p_num : 1;
    c->blocks_max = (q_num + c->alpha - 1) / c->alpha;
    for (int i = 0; i < p_num; i++) c->moduli.push_back(p[i]);
    for (int i = 0; i < q_num; i++) c->moduli.push_back(q[i]);
    for (int i = 0; i < t_num; i++) c->moduli.push_back(t[i]);

    const uint32_t N = c->N;
    const u64 M = 2ull * N;
    for (int i = 0; i < c->mod_num; i++) {
        u64 m = c->moduli[i];
        if (!(m < (1ull << 62)) || !is_prime(m) || (m - 1) % M) {
            set_error("modulus %d (%llu) must be a prime = 1 mod 2N below 2^62", i, m);
            delete c;
            return CKKS_B200_ERR_ARG;
        }
    }

    std::vector<ulonglong2> fwd((size_t)c->mod_num * N), inv((size_t)c->mod_num * N), ninv(c->mod_num);
    std::vector<double> fwd_d((size_t)c->mod_num * N), inv_d((size_t)c->mod_num * N);
    c->h_psi_tab.resize(c->mod_num);
    c->h_psiinv_tab.resize(c->mod_num);
    for (int i = 0; i < c->mod_num; i++) {
        u64 m = c->moduli[i];
        u64 root = find_mth_root(M, m);
        c->psi.push_back(root);
        fill_psi_tables(root, m, N, c->h_psi_tab[i], c->h_psiinv_tab[i]);
        for (uint32_t j = 0; j < N; j++) {
            u64 w = c->h_psi_tab[i][j], wi = c->h_psiinv_tab[i][j];
            fwd[(size_t)i * N + j] = make_ulonglong2(w, h_shoup(w, m));
            inv[(size_t)i * N + j] = make_ulonglong2(wi, h_shoup(wi, m));
            // centred representatives for the FP64 back end
            fwd_d[(size_t)i * N + j] = w > m / 2 ? -(double)(m - w) : (double)w;
            inv_d[(size_t)i * N + j] = wi > m / 2 ? -(double)(m - wi) : (double)wi;
        }
        u64 ni = h_invmod(N % m, m);
        ninv[i] = make_ulonglong2(ni, h_shoup(ni, m));
    }

    // ModUp tables per level (src/ckks/include/Context_23.cuh:286-351).
    const int A = c->alpha, B = c->blocks_max, T = t_num;
    std::vector<ulonglong2> hat_inv((size_t)q_num * B * A, make_ulonglong2(0, 0));
    std::vector<u64> hat_mod_t((size_t)q_num * B * (T ? T : 1) * A, 0), blk_mod_t((size_t)q_num * B * (T ? T : 1), 0);
    std::vector<ulonglong2> t_mu(T ? T : 1);
    const u64* qv = c->moduli.data() + p_num;
    const u64* tv = c->moduli.data() + p_num + q_num;
    for (int l = 0; l < q_num && T > 0; l++) {
        int blocks = (l + 1 + A - 1) / A;
        for (int b = 0; b < blocks; b++) {
            int cnt = std::min(A, l + 1 - b * A);
            for (int j = 0; j < cnt; j++) {
                u64 qj = qv[b * A + j], prod = 1;
                for (int jj = 0; jj < cnt; jj++)
                    if (jj != j) prod = h_mulmod(prod, qv[b * A + jj] % qj, qj);
                u64 iv = h_invmod(prod, qj);
                hat_inv[((size_t)l * B + b) * A + j] = make_ulonglong2(iv, h_shoup(iv, qj));
            }
            for (int k = 0; k < T; k++) {
                u64 tk = tv[k], full = 1;
                for (int j = 0; j < cnt; j++) {
                    u64 prod = 1;
                    for (int jj = 0; jj < cnt; jj++)
                        if (jj != j) prod = h_mulmod(prod, qv[b * A + jj] % tk, tk);
                    hat_mod_t[(((size_t)l * B + b) * T + k) * A + j] = prod;
                    full = h_mulmod(full, qv[b * A + j] % tk, tk);
                }
                blk_mod_t[((size_t)l * B + b) * T + k] = full;
            }
        }
    }
    for (int k = 0; k < T; k++) {
        u64 hi, lo;
        h_barrett_mu(tv[k], &hi, &lo);
        t_mu[k] = make_ulonglong2(hi, lo);
    }

    // Byte planes of the ModUp constants for the tensor-core kernel, in the order its MMA
    // descriptors read them: per 32-deep K step a block of tc_npad rows x 32 bytes made of core
    // matrices (8 rows x 16 bytes, 128 bytes from one K half to the other, 256 bytes from one
    // 8-row group to the next).  A level qualifies when every target modulus lies in
    // [2^40, 2^62) (the kernel reduces with an FP64 quotient estimate) and when
    // sum_j rb_j*h_j (h_j = Qblk/q_j mod t_k) can never fall below v*F (F = Qblk mod t_k): the 128-bit
    // difference the reference forms would wrap there, and only the CUDA-core kernel reproduces that wrap.
    const int apad = (A + 3) / 4 * 4;
    c->tc_kpad = apad * 8;
    c->tc_npad = (T * 8 + 15) / 16 * 16;
    const size_t tile_bytes = (size_t)c->tc_kpad * c->tc_npad;
    std::vector<uint8_t> planes(T > 0 ? (size_t)q_num * B * tile_bytes : 0, 0);
    std::vector<double> t_inv(T ? T : 1, 0.0);
    c->mu_tc_ok.assign(q_num, 0);
    bool t_range_ok = T > 0 && T * 8 <= 256 && A <= 16;
    for (int k = 0; k < T; k++) {
        t_inv[k] = 1.0 / (double)tv[k];
        if (tv[k] < (1ull << 40) || tv[k] >= (1ull << 62)) t_range_ok = false;
    }
    for (int l = 0; l < q_num && T > 0; l++) {
        int blocks = (l + 1 + A - 1) / A;
        bool ok = t_range_ok;
        for (int b = 0; b < blocks; b++) {
            int cnt = std::min(A, l + 1 - b * A);
            uint8_t* tile = planes.data() + ((size_t)l * B + b) * tile_bytes;
            for (int k = 0; k < T; k++) {
                const u64 tk = tv[k];
                const u64 full = blk_mod_t[((size_t)l * B + b) * T + k];
                for (int j = 0; j < cnt; j++) {
                    u64 cst = hat_mod_t[(((size_t)l * B + b) * T + k) * A + j];
                    // v <= (sum_j rb_j/q_j)(1 + 2^-45) even after rounding, so h_j*q_j >= F(1 + 2^-40) for every j
                    // keeps sum_j rb_j*h_j >= v*F.  A one-limb digit has h = 1 and v = 0 as long as
                    // (q-1)/q rounds below 1.0, which it does for q < 2^52.
                    const u64 qj = qv[b * A + j];
                    if (cnt == 1 ? qj >= (1ull << 52) : (u128)cst * qj < (u128)full + (full >> 40) + 1) ok = false;
                    for (int bb = 0; bb < 8; bb++) {
                        const int kk = j * 8 + bb, ks = kk / 32, kc = (kk % 32) / 16, kin = kk % 16;
                        for (int a = 0; a < 8; a++) {
                            const int n = k * 8 + a;
                            tile[(size_t)ks * c->tc_npad * 32 + (size_t)(n / 8) * 256 + kc * 128 + (n % 8) * 16 + kin] =
                                (uint8_t)(cst >> (8 * a));
                        }
                        cst = h_mulmod(cst, 256 % tk, tk);
                    }
                }
            }
        }
        c->mu_tc_ok[l] = ok ? 1 : 0;
    }

    int st = CKKS_B200_OK;
    std::vector<u64> mods(c->moduli.begin(), c->moduli.end());
    if (!st) st = upload(&c->tw_fwd, fwd);
    if (!st) st = upload(&c->tw_inv, inv);
    if (!st) st = upload(&c->tw_fwd_d, fwd_d);
    if (!st) st = upload(&c->tw_inv_d, inv_d);
    if (!st) st = upload(&c->d_moduli, mods);
    if (!st) st = upload(&c->d_ninv, ninv);
    std::vector<u64> qinv64(c->mod_num);
    for (int i = 0; i < c->mod_num; i++) qinv64[i] = (u64)((((u128)1) << 64) / c->moduli[i]);
    if (!st) st = upload(&c->d_qinv64, qinv64);
    // q_l^-1 mod q_i for i < l (the reference's qiInvVecModql, Context_23.cuh:424-434)
    std::vector<ulonglong2> qlinv((size_t)q_num * q_num, make_ulonglong2(0, 0));
    for (int l = 1; l < q_num; l++)
        for (int i = 0; i < l; i++) {
            u64 inv = h_invmod(qv[l] % qv[i], qv[i]);
            qlinv[(size_t)l * q_num + i] = make_ulonglong2(inv, h_shoup(inv, qv[i]));
        }
    if (!st) st = upload(&c->d_qlinv, qlinv);

    // Key-switch chain constants (Context_23.cuh:60-192, 286-351).  T = prod t_i, P = prod p_j.
    {
        const int PQ = p_num + q_num;
        const u64* mv = c->moduli.data();
        std::vector<ulonglong2> pq_mu(PQ ? PQ : 1), t_hat_inv(T ? T : 1), p_hat_inv(p_num ? p_num : 1), p_inv_mod_q(q_num);
        std::vector<u64> t_hat_mod_r((size_t)PQ * (T ? T : 1), 0), half_t(c->mod_num, 0), t_mod_pq(PQ ? PQ : 1, 0),
            p_hat_mod_q((size_t)q_num * (p_num ? p_num : 1), 0);
        for (int i = 0; i < PQ; i++) {
            u64 hi, lo;
            h_barrett_mu(mv[i], &hi, &lo);
            pq_mu[i] = make_ulonglong2(hi, lo);
        }
        for (int i = 0; i < T; i++) {
            u64 prod = 1;
            for (int ii = 0; ii < T; ii++)
                if (ii != i) prod = h_mulmod(prod, tv[ii] % tv[i], tv[i]);
            u64 inv = h_invmod(prod, tv[i]);
            t_hat_inv[i] = make_ulonglong2(inv, h_shoup(inv, tv[i]));
        }
        for (int r = 0; r < PQ && T > 0; r++) {
            u64 full = 1;
            for (int j = 0; j < T; j++) {
                u64 prod = 1;
                for (int jj = 0; jj < T; jj++)
                    if (jj != j) prod = h_mulmod(prod, tv[jj] % mv[r], mv[r]);
                t_hat_mod_r[(size_t)r * T + j] = prod;
                full = h_mulmod(full, tv[j] % mv[r], mv[r]);
            }
            t_mod_pq[r] = full;
        }
        // floor(T/2) = (T-1)/2 for odd T; modulo m it is ((T mod 2m) - 1) / 2
        c->chain_ok = true;
        for (int i = 0; i < c->mod_num; i++) c->chain_ok = c->chain_ok && mv[i] < (1ull << 62);
        for (int i = 0; i < c->mod_num && T > 0 && c->chain_ok; i++) {
            const u128 m2 = (u128)2 * mv[i];                                  // below 2^63: products stay below 2^126
            u128 acc = 1;
            for (int j = 0; j < T; j++) acc = (acc * (tv[j] % m2)) % m2;
            half_t[i] = (u64)((acc - 1) / 2);
        }
        for (int j = 0; j < p_num; j++) {
            u64 prod = 1;
            for (int jj = 0; jj < p_num; jj++)
                if (jj != j) prod = h_mulmod(prod, mv[jj] % mv[j], mv[j]);
            u64 inv = h_invmod(prod, mv[j]);
            p_hat_inv[j] = make_ulonglong2(inv, h_shoup(inv, mv[j]));
        }
        for (int i = 0; i < q_num; i++) {
            u64 full = 1;
            for (int j = 0; j < p_num; j++) {
                u64 prod = 1;
                for (int jj = 0; jj < p_num; jj++)
                    if (jj != j) prod = h_mulmod(prod, mv[jj] % qv[i], qv[i]);
                p_hat_mod_q[(size_t)i * p_num + j] = prod;
                full = h_mulmod(full, mv[j] % qv[i], qv[i]);
            }
            u64 inv = p_num ? h_invmod(full, qv[i]) : 1;
            p_inv_mod_q[i] = make_ulonglong2(inv, h_shoup(inv, qv[i]));
        }
        if (!st) st = upload(&c->d_pq_mu, pq_mu);
        if (!st) st = upload(&c->d_t_hat_inv, t_hat_inv);
        if (!st) st = upload(&c->d_t_hat_mod_r, t_hat_mod_r);
        if (!st) st = upload(&c->d_half_t, half_t);
        if (!st) st = upload(&c->d_t_mod_pq, t_mod_pq);
        if (!st) st = upload(&c->d_p_hat_inv, p_hat_inv);
        if (!st) st = upload(&c->d_p_hat_mod_q, p_hat_mod_q);
        if (!st) st = upload(&c->d_p_inv_mod_q, p_inv_mod_q);
    }
    if (!st) st = upload(&c->mu_hat_inv, hat_inv);
    if (!st) st = upload(&c->mu_hat_mod_t, hat_mod_t);
    if (!st) st = upload(&c->mu_blk_mod_t, blk_mod_t);
    if (!st) st = upload(&c->d_t_mu, t_mu);
    if (!st) st = upload(&c->mu_planes, planes);
    {
        std::vector<u64> src_mod((size_t)q_num * B * apad, 1), tgt_mod((size_t)B * (T ? T : 1), 0);
        std::vector<ulonglong2> src_hinv((size_t)q_num * B * apad, make_ulonglong2(0, 0));
        for (int l = 0; l < q_num && T > 0; l++)
            for (int b = 0; b < (l + 1 + A - 1) / A; b++)
                for (int j = 0; j < std::min(A, l + 1 - b * A); j++) {
                    src_mod[((size_t)l * B + b) * apad + j] = qv[b * A + j];
                    src_hinv[((size_t)l * B + b) * apad + j] = hat_inv[((size_t)l * B + b) * A + j];
                }
        for (int b = 0; b < B; b++)
            for (int k = 0; k < T; k++) tgt_mod[(size_t)b * T + k] = tv[k];
        std::vector<u64> zeros((size_t)B * std::max(apad, T ? T : 1), 0);
        if (!st) st = upload(&c->mu_src_mod, src_mod);
        if (!st) st = upload(&c->mu_src_hinv, src_hinv);
        if (!st) st = upload(&c->mu_src_pre, zeros);
        if (!st) st = upload(&c->mu_tgt_mod, tgt_mod);
    }
    if (!st) st = upload(&c->d_t_inv, t_inv);
    if (!st && cudaMalloc(&c->d_flags, 16 * sizeof(int)) != cudaSuccess) st = CKKS_B200_ERR_NOMEM;
    if (!st && cudaMemset(c->d_flags, 0, 16 * sizeof(int)) != cudaSuccess) st = CKKS_B200_ERR_CUDA;
    if (!st && cudaMallocHost(&c->h_flags, 16 * sizeof(int)) != cudaSuccess) st = CKKS_B200_ERR_NOMEM;
    if (st) { ckks_b200_context_destroy(c); return st; }
    *out = c;
    return CKKS_B200_OK;
}

namespace ckb {
int build_tpq_tables(ckks_b200_context* c, int gamma) {
    if (c->tpq.count(gamma)) return CKKS_B200_OK;
    TpqTables tb;
    const int PQ = c->p_num + c->q_num, T = c->t_num;
    const u64* mv = c->moduli.data();
    const u64* tv = mv + PQ;
    const int R = (PQ + gamma - 1) / gamma, apad = (T + 3) / 4 * 4;
    tb.kpad = apad * 8;
    tb.npad = (gamma * 8 + 15) / 16 * 16;
    bool ok = c->chain_ok && T >= 2 && T <= 16 && tb.npad <= 128;
    std::vector<u64> src_mod((size_t)R * apad, 1), src_pre((size_t)R * apad, 0), tgt_mod((size_t)R * gamma, 0),
        tgt_f((size_t)R * gamma, 0), tgt_post((size_t)R * gamma, 0);
    std::vector<ulonglong2> src_hinv((size_t)R * apad, make_ulonglong2(0, 0));
    std::vector<uint8_t> planes(ok ? (size_t)R * tb.kpad * tb.npad : 0, 0);
    for (int blk = 0; blk < R && ok; blk++) {
        for (int j = 0; j < T; j++) {
            u64 prod = 1;
            for (int jj = 0; jj < T; jj++)
                if (jj != j) prod = h_mulmod(prod, tv[jj] % tv[j], tv[j]);
            const u64 inv = h_invmod(prod, tv[j]);
            src_mod[(size_t)blk * apad + j] = tv[j];
            src_hinv[(size_t)blk * apad + j] = make_ulonglong2(inv, h_shoup(inv, tv[j]));
            const u128 m2 = (u128)2 * tv[j];
            u128 acc = 1;
            for (int jj = 0; jj < T; jj++) acc = (acc * (tv[jj] % m2)) % m2;
            src_pre[(size_t)blk * apad + j] = (u64)((acc - 1) / 2);         // floor(T/2) mod t_j
        }
        uint8_t* tile = planes.data() + (size_t)blk * tb.kpad * tb.npad;
        for (int k = 0; k < gamma && blk * gamma + k < PQ; k++) {
            const u64 r = mv[blk * gamma + k];
            if (r < (1ull << 40)) ok = false;
            u64 full = 1;
            for (int j = 0; j < T; j++) full = h_mulmod(full, tv[j] % r, r);
            const u128 m2 = (u128)2 * r;
            u128 acc = 1;
            for (int j = 0; j < T; j++) acc = (acc * (tv[j] % m2)) % m2;
            tgt_mod[(size_t)blk * gamma + k] = r;
            tgt_f[(size_t)blk * gamma + k] = full;
            tgt_post[(size_t)blk * gamma + k] = (u64)((acc - 1) / 2);
            for (int j = 0; j < T; j++) {
                u64 cst = 1;
                for (int jj = 0; jj < T; jj++)
                    if (jj != j) cst = h_mulmod(cst, tv[jj] % r, r);
                // sum_j rb_j*h_j >= v*F needs h_j*t_j >= F(1 + 2^-40) for every j (see the Q -> T tables above)
                if ((u128)cst * tv[j] < (u128)full + (full >> 40) + 1) ok = false;
                for (int bb = 0; bb < 8; bb++) {
                    const int kk = j * 8 + bb, ks = kk / 32, kc = (kk % 32) / 16, kin = kk % 16;
                    for (int a = 0; a < 8; a++) {
                        const int n = k * 8 + a;
                        tile[(size_t)ks * tb.npad * 32 + (size_t)(n / 8) * 256 + kc * 128 + (n % 8) * 16 + kin] = (uint8_t)(cst >> (8 * a));
                    }
                    cst = h_mulmod(cst, 256 % r, r);
                }
            }
        }
    }
    tb.ok = ok;
    int st = CKKS_B200_OK;
    if (ok) {
        DeviceGuard guard(c->device);
        if (!st) st = upload(&tb.src_mod, src_mod);
        if (!st) st = upload(&tb.src_hinv, src_hinv);
        if (!st) st = upload(&tb.src_pre, src_pre);
        if (!st) st = upload(&tb.tgt_mod, tgt_mod);
        if (!st) st = upload(&tb.tgt_f, tgt_f);
        if (!st) st = upload(&tb.tgt_post, tgt_post);
        if (!st) st = upload(&tb.planes, planes);
    }
    c->tpq[gamma] = tb;
    return st;
}
}  // namespace ckb

extern "C" int ckks_b200_context_destroy(ckks_b200_context* c) {
    if (!c) return CKKS_B200_OK;
    DeviceGuard guard(c->device);
    for (auto& kv : c->tpq) {
        TpqTables& tb = kv.second;
        cudaFree(tb.src_mod); cudaFree(tb.src_hinv); cudaFree(tb.src_pre); cudaFree(tb.tgt_mod); cudaFree(tb.tgt_f);
        cudaFree(tb.tgt_post); cudaFree(tb.planes);
    }
    cudaFree(c->mu_src_mod); cudaFree(c->mu_src_hinv); cudaFree(c->mu_src_pre); cudaFree(c->mu_tgt_mod);
    cudaFree(c->tw_fwd); cudaFree(c->tw_inv); cudaFree(c->tw_fwd_d); cudaFree(c->tw_inv_d); cudaFree(c->d_moduli); cudaFree(c->d_ninv); cudaFree(c->d_qinv64);
    cudaFree(c->mu_hat_inv); cudaFree(c->mu_hat_mod_t); cudaFree(c->mu_blk_mod_t);
    cudaFree(c->d_pq_mu); cudaFree(c->d_t_hat_inv); cudaFree(c->d_t_hat_mod_r); cudaFree(c->d_half_t); cudaFree(c->d_t_mod_pq);
    cudaFree(c->d_p_hat_inv); cudaFree(c->d_p_hat_mod_q); cudaFree(c->d_p_inv_mod_q); cudaFree(c->ks_buf); cudaFree(c->mul_buf);
    cudaFree(c->mu_planes); cudaFree(c->d_t_inv); cudaFree(c->d_flags); cudaFree(c->d_qlinv); cudaFree(c->resc_buf);
    if (c->h_flags) cudaFreeHost(c->h_flags);
    cudaFree(c->d_t_mu); cudaFree(c->h2d_buf); cudaFree(c->h2d_buf2); cudaFree(c->ptr_buf); cudaFree(c->pack_buf);
    delete c;
    return CKKS_B200_OK;
}

extern "C" int ckks_b200_context_psi(const ckks_b200_context* c, int mod_idx, uint64_t* psi) {
    CKB_REQUIRE(c && psi, CKKS_B200_ERR_ARG, "null argument");
    CKB_REQUIRE(mod_idx >= 0 && mod_idx < c->mod_num, CKKS_B200_ERR_ARG, "mod_idx %d out of range", mod_idx);
    *psi = c->psi[mod_idx];
    return CKKS_B200_OK;
}

extern "C" int ckks_b200_context_table(const ckks_b200_context* c, int mod_idx, int inverse,
                                       uint64_t* h_table) {
    CKB_REQUIRE(c && h_table, CKKS_B200_ERR_ARG, "null argument");
    CKB_REQUIRE(mod_idx >= 0 && mod_idx < c->mod_num, CKKS_B200_ERR_ARG, "mod_idx %d out of range", mod_idx);
    const std::vector<u64>& t = inverse ? c->h_psiinv_tab[mod_idx] : c->h_psi_tab[mod_idx];
    for (uint32_t j = 0; j < c->N; j++) h_table[j] = t[j];
    return CKKS_B200_OK;
}

extern "C" int ckks_b200_version(void) { return 100; }

extern "C" const char* ckks_b200_status_string(int s) {
    switch (s) {
        case CKKS_B200_OK: return "ok";
        case CKKS_B200_ERR_ARG: return "invalid argument";
        case CKKS_B200_ERR_SHAPE: return "shape rule violated";
        case CKKS_B200_ERR_UNSUPPORTED: return "unsupported size";
        case CKKS_B200_ERR_CUDA: return "CUDA error";
        case CKKS_B200_ERR_NOMEM: return "out of memory";
        case CKKS_B200_ERR_RANGE: return "weight out of range";
        case CKKS_B200_ERR_TIMEOUT: return "device-side wait timed out";
    }
    return "unknown status";
}

extern "C" const char* ckks_b200_last_error(void) { return ckb::get_error(); }

extern "C" long ckks_b200_kernel_launches(void) { return ckb::g_launches.load(); }
