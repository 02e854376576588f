// Source-level stand-ins for the classes of the reference (haozetao/ckks_llm) that lie on the ring-packed
// plaintext x ciphertext matrix-multiply path, in the global namespace, with the reference's class names, public
// members and method signatures, forwarding to the C ABI of the B200 library (ckks_b200.h).
//
// The reference is a header-only unity build; its callers (test_rlwe_decomp.cu, src/bert/Bert.cuh) include
// "src/ckks/include/pcmm/PCMM_Scheme.cuh" and friends and call methods on objects.  The small headers beside this
// file mirror those include paths and all include this one, so a caller compiles against this tree with
// -I<this directory> (and an NTL, or the stand-in under NTL/ here) and links libckks_b200.so.
//
// What each class mirrors (paths relative to the reference root):
//   Context_23       src/ckks/include/Context_23.h:19-279     moduli, ToNTTInplace / FromNTTInplace (Context_23.cuh:847-889),
//                                                             modUpQjtoT_23 (BasisConv.cuh:161-179), key-switch steps,
//                                                             encode_coeffs / decode_coeffs (Encoder.cuh:68-160)
//   Plaintext        src/ckks/include/Plaintext.cuh:6-75
//   Ciphertext       src/ckks/include/Ciphertext.cuh:5-100
//   SecretKey        src/ckks/include/SecretKey.cuh:10-60
//   Key              src/ckks/include/Key.cuh:6-80
//   Scheme_23        src/ckks/include/Scheme_23.h              rescaleAndEqual (Scheme_23.cuh:368-385), mult_23 / conjugate_23 /
//                                                             leftRotate_23 (KeySwitch_23.cuh:192-581), encryptMsg / decryptMsg
//   SchemeAlgo       src/ckks/include/advanced/SchemeAlgo.h    constructor only (the path does not use it)
//   Bootstrapper     src/ckks/include/bootstrapping/Bootstrapper.cuh:192-209   modUpQ0toQL only
//   MLWECiphertext   src/ckks/include/pcmm/MLWECiphertext.cuh:6-78
//   MLWEPlaintext    src/ckks/include/pcmm/MLWEPlaintext.cuh
//   MLWESecretKey    src/ckks/include/pcmm/MLWESecretKey.cuh:5-58
//   PCMM_Context     src/ckks/include/pcmm/PCMM_Context.h:14-90
//   PCMM_Scheme      src/ckks/include/pcmm/PCMM_Scheme.h:12-48 (definitions PCMM_Scheme.cuh, PPMM_kernel.cuh:254-349)
//
// Differences a caller can see, all on purpose:
//   * Context_23(logN, logslots, h) takes its moduli from a short table instead of the reference's Params.cuh: for
//     logN = 16 the head of the reference's own chain (4 q, 4 p, 8 t: the ring-pack moduli {q0, q1} and the special
//     prime are the reference's), for other sizes the largest 50-bit (q), 51-bit (p) and 60-bit (t) primes that are
//     1 mod 2N.  The second constructor takes the three lists explicitly.
//   * Randomness (secret key, encryption, repacking keys) comes from std::mt19937_64 on the host with a fixed seed
//     per object, not from the reference's device generator; errors are rounded Gaussians of sigma 3.2.
//   * Scheme_23::addEncKey keeps a pointer to the secret key and encryptMsg encrypts symmetrically under it (the
//     reference builds a public encryption key): the ciphertexts have the same layout and decrypt the same way.
//   * MLWESecretKey keeps coefficients, not their N1-point transform (the reference transforms it for mlweDecrypt;
//     mlweDecrypt here multiplies in the coefficient domain on the host).
//   * PCMM_Scheme::realData_coeffShift is called by src/bert (Bert.cuh:403-412,472-490) but declared and defined
//     nowhere in the reference; it is declared here and prints that it does nothing.  coeffBitRev
//     (PCMM_Scheme.cuh:502-529) decrypts, permutes and re-encrypts with the secret key, a test shortcut that is no
//     homomorphic step: it does the same here, on the host.
//   * CUDA and library errors throw std::runtime_error instead of being ignored.
#ifndef CKKS_LLM_COMPAT_HPP
#define CKKS_LLM_COMPAT_HPP

#include <cuda_runtime.h>

#include <NTL/RR.h>

#include <cmath>
#include <cstdint>
#include <cstring>
#include <iostream>
#include <map>
#include <random>
#include <stdexcept>
#include <string>
#include <vector>

#include "../ckks_b200.h"

typedef unsigned long long uint64_tt;
typedef unsigned int uint32_tt;
typedef unsigned char uint8_tt;

namespace ckks_llm_compat {

inline void check(int status) {
    if (status != CKKS_B200_OK) throw std::runtime_error(std::string("ckks_b200: ") + ckks_b200_last_error());
}
inline void check_cuda(cudaError_t e) {
    if (e != cudaSuccess) throw std::runtime_error(std::string("CUDA: ") + cudaGetErrorString(e));
}
inline uint64_tt mulmod(uint64_tt a, uint64_tt b, uint64_tt q) { return (uint64_tt)(((unsigned __int128)a * b) % q); }
inline uint64_tt addmod(uint64_tt a, uint64_tt b, uint64_tt q) { uint64_tt s = a + b; return s >= q ? s - q : s; }
inline uint64_tt submod(uint64_tt a, uint64_tt b, uint64_tt q) { return a >= b ? a - b : a + q - b; }
inline uint64_tt from_signed(long long x, uint64_tt q) { return x >= 0 ? (uint64_tt)x % q : q - ((uint64_tt)(-x) % q == 0 ? q : (uint64_tt)(-x) % q); }
inline bool is_prime(uint64_tt n) {
    if (n < 2) return false;
    for (uint64_tt p : {2ull, 3ull, 5ull, 7ull, 11ull, 13ull, 17ull, 19ull, 23ull, 29ull, 31ull, 37ull}) if (n % p == 0) return n == p;
    uint64_tt d = n - 1; int r = 0;
    while ((d & 1) == 0) { d >>= 1; r++; }
    for (uint64_tt a : {2ull, 3ull, 5ull, 7ull, 11ull, 13ull, 17ull, 19ull, 23ull, 29ull, 31ull, 37ull}) {
        uint64_tt x = 1, b = a % n, e = d;
        for (; e; e >>= 1) { if (e & 1) x = mulmod(x, b, n); b = mulmod(b, b, n); }
        if (x == 1 || x == n - 1) continue;
        bool composite = true;
        for (int i = 0; i < r - 1; i++) { x = mulmod(x, x, n); if (x == n - 1) { composite = false; break; } }
        if (composite) return false;
    }
    return true;
}
// the `count` largest primes below 2^bits that are 1 mod two_n
inline std::vector<uint64_tt> ntt_primes(int bits, uint64_tt two_n, int count) {
    std::vector<uint64_tt> out;
    uint64_tt c = (1ull << bits) - 1;
    c -= (c - 1) % two_n;
    for (; (int)out.size() < count && c > (1ull << (bits - 1)); c -= two_n) if (is_prime(c)) out.push_back(c);
    return out;
}
template <class T>
std::vector<T> download(const T* d, size_t n) {
    std::vector<T> h(n);
    check_cuda(cudaMemcpy(h.data(), d, n * sizeof(T), cudaMemcpyDeviceToHost));
    return h;
}
template <class T>
void upload(T* d, const std::vector<T>& h) { check_cuda(cudaMemcpy(d, h.data(), h.size() * sizeof(T), cudaMemcpyHostToDevice)); }

}  // namespace ckks_llm_compat

// ---------------------------------------------------------------------------------------------------------------
class Plaintext {
public:
    uint64_tt* mx_device = nullptr;     // [L+1][N], NTT domain
    int N = 0, L = 0, l = 0, slots = 0;
    NTL::RR scale;
    Plaintext() {}
    Plaintext(int N, int L, int l, int slots, NTL::RR scale) : N(N), L(L), l(l), slots(slots), scale(scale) {
        if (l > L) std::cout << "new Plaintext error!" << std::endl;
        ckks_llm_compat::check_cuda(cudaMalloc(&mx_device, sizeof(uint64_tt) * N * (L + 1)));
    }
    Plaintext(const Plaintext&) = delete;
    Plaintext& operator=(const Plaintext&) = delete;
    virtual ~Plaintext() { if (mx_device) cudaFree(mx_device); }
};

// a limbs then b limbs, each [L+1][N], NTT domain at rest; one allocation per object, deep copies
class Ciphertext {
public:
    uint64_tt* cipher_device = nullptr;
    uint64_tt* ax_device = nullptr;
    uint64_tt* bx_device = nullptr;
    int N = 0, L = 0, l = 0, slots = 0;
    NTL::RR scale;
    Ciphertext() {}
    Ciphertext(int N, int L, int l, int slots, NTL::RR scale) : N(N), L(L), l(l), slots(slots), scale(scale) { alloc(); }
    Ciphertext(const Ciphertext& c) : N(c.N), L(c.L), l(c.l), slots(c.slots), scale(c.scale) {
        alloc();
        if (c.cipher_device) cudaMemcpy(cipher_device, c.cipher_device, bytes(), cudaMemcpyDeviceToDevice);
    }
    Ciphertext& operator=(const Ciphertext& c) {
        if (this == &c) return *this;
        if (cipher_device && bytes() != c.bytes()) { cudaFree(cipher_device); cipher_device = nullptr; }
        N = c.N; L = c.L; l = c.l; slots = c.slots; scale = c.scale;
        if (!cipher_device) alloc();
        if (c.cipher_device) cudaMemcpy(cipher_device, c.cipher_device, bytes(), cudaMemcpyDeviceToDevice);
        return *this;
    }
    virtual ~Ciphertext() { if (cipher_device) { cudaDeviceSynchronize(); cudaFree(cipher_device); } }
    size_t bytes() const { return sizeof(uint64_tt) * (size_t)N * (L + 1) * 2; }
private:
    void alloc() {
        ckks_llm_compat::check_cuda(cudaMalloc(&cipher_device, bytes()));
        ax_device = cipher_device;
        bx_device = cipher_device + (size_t)N * (L + 1);
    }
};

// ---------------------------------------------------------------------------------------------------------------
class Context_23 {
public:
    long logN, logslots, h;
    double sigma;
    int N, Nh, slots, L, K, p_num, q_num, t_num, dnum, alpha, gamma = 3;
    long precision;
    std::vector<uint64_tt> pVec, qVec, tVec;
    ckks_b200_context* b200 = nullptr;

    Context_23(long logN_, long logslots_, long h_ = 64, double sigma_ = 3.2) : logN(logN_), logslots(logslots_), h(h_), sigma(sigma_) {
        const uint64_tt two_n = 2ull << logN;
        if (logN == 16) {
            // the head of the reference's own logN = 16 chain (src/ckks/include/Params.cuh:118-150)
            qVec = {0x20000018e0001ull, 0x2000001c00001ull, 0x2000001ca0001ull, 0x2000001d20001ull};
            pVec = {0x2000002600001ull, 0x20000027e0001ull, 0x2000002800001ull, 0x20000029e0001ull};
            tVec = {0xffffffffffc0001ull, 0xfffffffff840001ull, 0xfffffffff6a0001ull, 0xfffffffff5a0001ull,
                    0xfffffffff2a0001ull, 0xfffffffff240001ull, 0xffffffffefe0001ull, 0xffffffffeca0001ull};
        } else {
            qVec = ckks_llm_compat::ntt_primes(50, two_n, 4);
            pVec = ckks_llm_compat::ntt_primes(51, two_n, 4);
            tVec = ckks_llm_compat::ntt_primes(60, two_n, 8);
        }
        precision = 1L << 49;
        init();
    }
    Context_23(long logN_, std::vector<uint64_tt> p, std::vector<uint64_tt> q, std::vector<uint64_tt> t, long precision_ = 1L << 49,
               long h_ = 192)
        : logN(logN_), logslots(logN_ - 1), h(h_), sigma(3.2), precision(precision_), pVec(std::move(p)), qVec(std::move(q)),
          tVec(std::move(t)) {
        init();
    }
    Context_23(const Context_23&) = delete;
    Context_23& operator=(const Context_23&) = delete;
    ~Context_23() { ckks_b200_context_destroy(b200); }

    void ToNTTInplace(uint64_tt* device_a, int start_poly_idx, int start_mod_idx, int poly_num, int mod_num, int poly_mod_len) {
        ckks_llm_compat::check(ckks_b200_ntt_forward(b200, (uint64_t*)device_a, start_poly_idx, start_mod_idx, poly_num, mod_num, poly_mod_len, 0));
    }
    void FromNTTInplace(uint64_tt* device_a, int start_poly_idx, int start_mod_idx, int poly_num, int mod_num, int poly_mod_len) {
        ckks_llm_compat::check(ckks_b200_ntt_inverse(b200, (uint64_t*)device_a, start_poly_idx, start_mod_idx, poly_num, mod_num, poly_mod_len, 0));
    }
    void modUpQjtoT_23(uint64_tt* output, uint64_tt* input, int l, int batch_size) {
        ckks_llm_compat::check(ckks_b200_modup_qj_to_t(b200, (uint64_t*)output, (const uint64_t*)input, l, batch_size, 0));
    }
    void external_product_T(uint64_tt* output, uint64_tt* cipher_modUp_QjtoT, uint64_tt* swk_modUp_RitoT, int l) {
        ckks_llm_compat::check(ckks_b200_external_product_t(b200, (uint64_t*)output, (const uint64_t*)cipher_modUp_QjtoT,
                                                            (const uint64_t*)swk_modUp_RitoT, l, gamma, 0));
    }
    void FromNTTInplace_for_externalProduct(uint64_tt* device_a, int l) {
        ckks_llm_compat::check(ckks_b200_ntt_inverse_ext(b200, (uint64_t*)device_a, l, gamma, 0));
    }
    void modUpTtoPQl_23(uint64_tt* modUp_TtoQj_buffer, uint64_tt* exProduct_T_temp, int l, int batch_size) {
        ckks_llm_compat::check(ckks_b200_modup_t_to_pql(b200, (uint64_t*)modUp_TtoQj_buffer, (const uint64_t*)exProduct_T_temp, l, gamma, batch_size, 0));
    }
    void modDownPQltoQl_23(uint64_tt* output, uint64_tt* modUp_TtoQj_buffer, int l, int batch_size) {
        ckks_llm_compat::check(ckks_b200_moddown_pql_to_ql(b200, (uint64_t*)output, (const uint64_t*)modUp_TtoQj_buffer, l, gamma, batch_size, 0));
    }

    // Encoder.cuh:68-95: vals is a DEVICE array of N doubles; coefficient j of limb i becomes (long)(vals[j] * scale),
    // negative values as q_i + data; then the plaintext goes to the NTT domain.
    void encode_coeffs(double* vals, Plaintext& msg) {
        std::vector<double> v = ckks_llm_compat::download(vals, (size_t)N);
        const long scale = NTL::to_long(msg.scale);
        std::vector<uint64_tt> m((size_t)N * (msg.L + 1), 0);
        for (int i = 0; i <= msg.l; i++)
            for (int j = 0; j < N; j++) {
                const long data = (long)(v[j] * scale);
                m[(size_t)i * N + j] = data >= 0 ? (uint64_tt)data : (uint64_tt)(qVec[i] + data);
            }
        ckks_llm_compat::upload(msg.mx_device, m);
        ToNTTInplace(msg.mx_device, 0, K, 1, msg.l + 1, msg.L + 1);
    }
    // Encoder.cuh:112-160, from limb 0 alone (enough while the coefficients stay below q_0 / 2 in magnitude, which
    // is the case on this path; the reference reconstructs over all limbs of the level).  vals is a DEVICE array.
    void decode_coeffs(Plaintext& msg, double* vals, bool is_bitRev = false) {
        (void)is_bitRev;
        uint64_tt* tmp;
        ckks_llm_compat::check_cuda(cudaMalloc(&tmp, sizeof(uint64_tt) * N));
        cudaMemcpy(tmp, msg.mx_device, sizeof(uint64_tt) * N, cudaMemcpyDeviceToDevice);
        FromNTTInplace(tmp, 0, K, 1, 1, 1);
        std::vector<uint64_tt> m = ckks_llm_compat::download(tmp, (size_t)N);
        cudaFree(tmp);
        const long double scale = msg.scale.v;
        std::vector<double> v(N);
        for (int j = 0; j < N; j++)
            v[j] = (double)((m[j] <= qVec[0] / 2 ? (long double)m[j] : (long double)m[j] - (long double)qVec[0]) / scale);
        ckks_llm_compat::upload(vals, v);
    }

private:
    void init() {
        N = 1 << logN; Nh = N / 2; slots = 1 << logslots;
        p_num = (int)pVec.size(); q_num = (int)qVec.size(); t_num = (int)tVec.size();
        K = p_num; L = q_num - 1; alpha = p_num; dnum = p_num ? q_num / p_num : 0;
        ckks_llm_compat::check(ckks_b200_context_create(&b200, 0, (int)logN, (const uint64_t*)pVec.data(), p_num, (const uint64_t*)qVec.data(),
                                                        q_num, (const uint64_t*)tVec.data(), t_num));
    }
};

// Ternary secret of Hamming weight context.h over [p | q], NTT domain on the device (SecretKey.cuh:18-31).
class SecretKey {
public:
    uint64_tt* sx_host = nullptr;       // the residues on the host, same layout as sx_device
    uint64_tt* sx_device = nullptr;     // [K+L+1][N], NTT domain
    std::vector<long long> s_coeffs;    // the signed coefficients (no reference counterpart; key generation reads them)
    int N, L, K;
    SecretKey(Context_23& context, cudaStream_t stream = 0) : N(context.N), L(context.L), K(context.K) {
        (void)stream;
        const int mods = K + L + 1;
        sx_host = new uint64_tt[(size_t)N * mods];
        ckks_llm_compat::check_cuda(cudaMalloc(&sx_device, sizeof(uint64_tt) * N * mods));
        std::mt19937_64 rng(0x5ec2e7);
        s_coeffs.assign(N, 0);
        for (long placed = 0; placed < context.h;) {
            const size_t pos = rng() % N;
            if (s_coeffs[pos]) continue;
            s_coeffs[pos] = (rng() & 1) ? 1 : -1;
            placed++;
        }
        std::vector<uint64_tt> res((size_t)N * mods);
        for (int i = 0; i < mods; i++) {
            const uint64_tt q = i < K ? context.pVec[i] : context.qVec[i - K];
            for (int j = 0; j < N; j++) res[(size_t)i * N + j] = ckks_llm_compat::from_signed(s_coeffs[j], q);
        }
        ckks_llm_compat::upload(sx_device, res);
        context.ToNTTInplace(sx_device, 0, 0, 1, mods, mods);
        copyToHost();
    }
    SecretKey(const SecretKey&) = delete;
    SecretKey& operator=(const SecretKey&) = delete;
    virtual ~SecretKey() { delete[] sx_host; cudaDeviceSynchronize(); cudaFree(sx_device); }
    void copyToHost() { cudaMemcpy(sx_host, sx_device, sizeof(uint64_tt) * N * (K + L + 1), cudaMemcpyDeviceToHost); }
};

// Switching-key carrier (Key.cuh:6-80): a block then b block, each [dnum][L+1+K][N].
class Key {
public:
    uint64_tt* ax_device = nullptr;
    uint64_tt* bx_device = nullptr;
    uint64_tt* cipher_device = nullptr;
    int N = 0, L = 0, K = 0, dnum = 0;
    bool owns = false;
    Key() {}
    Key(int N, int L, int K, int dnum) : N(N), L(L), K(K), dnum(dnum), owns(true) {
        ckks_llm_compat::check_cuda(cudaMalloc(&cipher_device, sizeof(uint64_tt) * N * (L + 1 + K) * dnum * 2));
        ax_device = cipher_device;
        bx_device = cipher_device + (size_t)N * (L + 1 + K) * dnum;
    }
    Key(uint64_tt* cipher, int N, int L, int K, int dnum) : N(N), L(L), K(K), dnum(dnum) {
        cipher_device = cipher;
        ax_device = cipher_device;
        bx_device = cipher_device + (size_t)N * (L + 1 + K) * dnum;
    }
    Key(const Key&) = delete;
    Key& operator=(const Key&) = delete;
    virtual ~Key() { if (owns && cipher_device) cudaFree(cipher_device); }
};

// ---------------------------------------------------------------------------------------------------------------
class Scheme_23 {
public:
    Context_23& context;
    SecretKey* enc_sk = nullptr;                 // see addEncKey
    uint64_tt* rlk_23 = nullptr;                 // relinearisation key block on the device (key generation is the caller's)
    uint64_tt* ConjKey_23 = nullptr;
    std::map<long, uint64_tt*> rotKey_vec_23;
    std::mt19937_64 host_rng{0xe4c};
    explicit Scheme_23(Context_23& context_) : context(context_) {}

    // The reference derives a public encryption key from sk; here encryptMsg encrypts symmetrically under sk.
    void addEncKey(SecretKey& sk) { enc_sk = &sk; }

    // (a, b = -a*s + m + e) per limb 0..plain.l, NTT domain; decryption is b + a*s.
    void encryptMsg(Ciphertext& cipher, Plaintext& plain) {
        if (!enc_sk) throw std::invalid_argument("addEncKey has not been called");
        const int N = context.N, L1 = cipher.L + 1, K = context.K;
        std::normal_distribution<double> gauss(0.0, context.sigma);
        std::vector<long long> e(N);
        for (int j = 0; j < N; j++) e[j] = llround(gauss(host_rng));
        std::vector<uint64_tt> em((size_t)N * L1, 0), a((size_t)N * L1, 0), b((size_t)N * L1, 0);
        for (int i = 0; i <= plain.l; i++)
            for (int j = 0; j < N; j++) em[(size_t)i * N + j] = ckks_llm_compat::from_signed(e[j], context.qVec[i]);
        uint64_tt* tmp;
        ckks_llm_compat::check_cuda(cudaMalloc(&tmp, sizeof(uint64_tt) * N * L1));
        ckks_llm_compat::upload(tmp, em);
        context.ToNTTInplace(tmp, 0, K, 1, plain.l + 1, L1);
        em = ckks_llm_compat::download(tmp, (size_t)N * L1);
        cudaFree(tmp);
        std::vector<uint64_tt> m = ckks_llm_compat::download(plain.mx_device, (size_t)N * (plain.L + 1));
        for (int i = 0; i <= plain.l; i++) {
            const uint64_tt q = context.qVec[i];
            const uint64_tt* s = enc_sk->sx_host + (size_t)(K + i) * N;
            for (int j = 0; j < N; j++) {
                const size_t x = (size_t)i * N + j;
                a[x] = host_rng() % q;
                b[x] = ckks_llm_compat::submod(ckks_llm_compat::addmod(m[x], em[x], q), ckks_llm_compat::mulmod(a[x], s[j], q), q);
            }
        }
        ckks_llm_compat::upload(cipher.ax_device, a);
        ckks_llm_compat::upload(cipher.bx_device, b);
        cipher.l = plain.l;
        cipher.scale = plain.scale;
    }
    // m = b + a*s per limb 0..cipher.l (NTT domain)
    void decryptMsg(Plaintext& plain, SecretKey& sk, Ciphertext& cipher) {
        const int N = context.N, L1 = cipher.L + 1, K = context.K;
        std::vector<uint64_tt> a = ckks_llm_compat::download(cipher.ax_device, (size_t)N * L1);
        std::vector<uint64_tt> b = ckks_llm_compat::download(cipher.bx_device, (size_t)N * L1);
        std::vector<uint64_tt> m((size_t)N * (plain.L + 1), 0);
        for (int i = 0; i <= cipher.l; i++) {
            const uint64_tt q = context.qVec[i];
            const uint64_tt* s = sk.sx_host + (size_t)(K + i) * N;
            for (int j = 0; j < N; j++) {
                const size_t x = (size_t)i * N + j;
                m[x] = ckks_llm_compat::addmod(b[x], ckks_llm_compat::mulmod(a[x], s[j], q), q);
            }
        }
        ckks_llm_compat::upload(plain.mx_device, m);
        plain.l = cipher.l;
        plain.scale = cipher.scale;
    }

    void rescaleAndEqual(Ciphertext& cipher) {
        ckks_llm_compat::check(ckks_b200_rescale(context.b200, (uint64_t*)cipher.cipher_device, cipher.L, cipher.l, 0));
        cipher.scale = cipher.scale / NTL::RR((long double)context.qVec[cipher.l]);
        cipher.l -= 1;
    }
    void mult_23(Ciphertext& cipher_res, Ciphertext& cipher1, Ciphertext& cipher2) {
        if (cipher1.l == 0 || cipher2.l == 0) throw std::invalid_argument("Ciphertexts are on level 0");
        if (rlk_23 == nullptr) throw std::invalid_argument("rotKey_23 not exists");
        const int l = cipher1.l < cipher2.l ? cipher1.l : cipher2.l;
        ckks_llm_compat::check(ckks_b200_mult(context.b200, (uint64_t*)cipher_res.cipher_device, (const uint64_t*)cipher1.cipher_device,
                                              (const uint64_t*)cipher2.cipher_device, (const uint64_t*)rlk_23, l, context.gamma, 0));
        cipher_res.l = l;
        cipher_res.scale = cipher1.scale * cipher2.scale;
    }
    void conjugate_23(Ciphertext& cipher_res, Ciphertext& cipher) {
        if (ConjKey_23 == nullptr) throw std::invalid_argument("conjKey_23 not exists");
        ckks_llm_compat::check(ckks_b200_conjugate(context.b200, (uint64_t*)cipher_res.cipher_device, (const uint64_t*)cipher.cipher_device,
                                                   (const uint64_t*)ConjKey_23, cipher.l, context.gamma, 0));
        cipher_res.l = cipher.l;
        cipher_res.scale = cipher.scale;
    }
    void conjugateAndEqual_23(Ciphertext& cipher) { conjugate_23(cipher, cipher); }
    void leftRotate_23(Ciphertext& cipher_res, Ciphertext& cipher, long rotSlots) {
        auto it = rotKey_vec_23.find(rotSlots);
        if (it == rotKey_vec_23.end() || it->second == nullptr) throw std::invalid_argument("rotKey_23 not exists");
        ckks_llm_compat::check(ckks_b200_rotate(context.b200, (uint64_t*)cipher_res.cipher_device, (const uint64_t*)cipher.cipher_device,
                                                (const uint64_t*)it->second, rotSlots, cipher.l, context.gamma, 0));
        cipher_res.l = cipher.l;
        cipher_res.scale = cipher.scale;
    }
    void leftRotateAndEqual_23(Ciphertext& cipher, long rotSlots) { leftRotate_23(cipher, cipher, rotSlots); }
};

// The path never calls into it; drivers construct one (test_rlwe_decomp.cu:43).
class SchemeAlgo {
public:
    Context_23& context;
    Scheme_23& scheme;
    SecretKey& sk;
    SchemeAlgo(Context_23& context, Scheme_23& scheme, SecretKey& sk) : context(context), scheme(scheme), sk(sk) {}
};

// Bootstrapper::modUpQ0toQL (bootstrapping/Bootstrapper.cuh:192-209); the rest of the bootstrapping is not on the path.
class Bootstrapper {
public:
    Context_23& context;
    Scheme_23& scheme;
    Bootstrapper(Context_23& context, Scheme_23& scheme) : context(context), scheme(scheme) {}
    void modUpQ0toQL(Ciphertext& cipher, int target_level) {
        if (cipher.l != 0) return;
        const int scale_up = (int)(context.qVec[0] / (uint64_tt)context.precision);     // the reference kernel's parameter is an int
        ckks_llm_compat::check(ckks_b200_modup_q0_to_ql(context.b200, (uint64_t*)cipher.cipher_device, cipher.L, target_level, scale_up, 0));
        cipher.l = target_level;
    }
};

// ---------------------------------------------------------------------------------------------------------------
// [L+1][k+1][N1] words, coefficient domain while on the path; one cudaMalloc per object, deep copies.
class MLWECiphertext {
public:
    uint64_tt* cipher_device = nullptr;
    int N1 = 0, L = 0, l = 0, k = 0;
    NTL::RR scale;
    bool owns = true;
    MLWECiphertext() {}
    MLWECiphertext(int N1, int L, int l, int k, NTL::RR scale) : N1(N1), L(L), l(l), k(k), scale(scale) {
        ckks_llm_compat::check_cuda(cudaMalloc(&cipher_device, bytes()));
    }
    MLWECiphertext(uint64_tt* cipher, int N1, int L, int l, int k, NTL::RR scale) : cipher_device(cipher), N1(N1), L(L), l(l), k(k), scale(scale), owns(false) {}
    MLWECiphertext(const MLWECiphertext& c) : N1(c.N1), L(c.L), l(c.l), k(c.k), scale(c.scale) {
        ckks_llm_compat::check_cuda(cudaMalloc(&cipher_device, bytes()));
        if (c.cipher_device) cudaMemcpy(cipher_device, c.cipher_device, bytes(), cudaMemcpyDeviceToDevice);
    }
    MLWECiphertext& operator=(MLWECiphertext& c) {
        if (this == &c) return *this;
        if (cipher_device && owns && bytes() != c.bytes()) { cudaFree(cipher_device); cipher_device = nullptr; }
        N1 = c.N1; L = c.L; l = c.l; k = c.k; scale = c.scale;
        if (!cipher_device) { ckks_llm_compat::check_cuda(cudaMalloc(&cipher_device, bytes())); owns = true; }
        if (c.cipher_device) cudaMemcpy(cipher_device, c.cipher_device, bytes(), cudaMemcpyDeviceToDevice);
        return *this;
    }
    virtual ~MLWECiphertext() {
        if (cipher_device && owns) { cudaDeviceSynchronize(); cudaFree(cipher_device); cudaDeviceSynchronize(); }
        cipher_device = nullptr;
    }
    size_t bytes() const { return sizeof(uint64_tt) * (size_t)N1 * (L + 1) * (k + 1); }
};

class MLWEPlaintext {
public:
    uint64_tt* mx_device = nullptr;     // [L+1][N1], coefficient domain
    int N1 = 0, L = 0, l = 0;
    NTL::RR scale;
    MLWEPlaintext() {}
    MLWEPlaintext(int N1, int L, int l, NTL::RR scale) : N1(N1), L(L), l(l), scale(scale) {
        ckks_llm_compat::check_cuda(cudaMalloc(&mx_device, sizeof(uint64_tt) * N1 * (L + 1)));
    }
    MLWEPlaintext(const MLWEPlaintext&) = delete;
    MLWEPlaintext& operator=(const MLWEPlaintext&) = delete;
    virtual ~MLWEPlaintext() { if (mx_device) cudaFree(mx_device); }
};

// [L+1][k][N1] words: component r of the MLWE secret modulo ring-pack modulus i (coefficients).
class MLWESecretKey {
public:
    uint64_tt* sx_device = nullptr;
    std::vector<long long> s_coeffs;    // [k][N1] signed coefficients (no reference counterpart)
    int N1 = 0, L = 0, k = 0;
    MLWESecretKey() {}
    MLWESecretKey(int N1, int L, int k) : N1(N1), L(L), k(k) {
        ckks_llm_compat::check_cuda(cudaMalloc(&sx_device, sizeof(uint64_tt) * N1 * k * (L + 1)));
    }
    MLWESecretKey(const MLWESecretKey&) = delete;
    MLWESecretKey& operator=(const MLWESecretKey&) = delete;
    virtual ~MLWESecretKey() { if (sx_device) { cudaDeviceSynchronize(); cudaFree(sx_device); } }
};

// ---------------------------------------------------------------------------------------------------------------
class PCMM_Context {
public:
    Context_23& context;
    int N1, mlwe_rank;
    int ringpack_p_count, ringpack_q_count, ringpack_pq_count;
    std::vector<uint64_tt> p_ringpack, q_ringpack, pq_ringpack;
    ckks_b200_pcmm* b200 = nullptr;

    PCMM_Context(int N1, int mlwe_rank, std::vector<uint64_tt> p_ringpack_, std::vector<uint64_tt> q_ringpack_, Context_23& context)
        : context(context), N1(N1), mlwe_rank(mlwe_rank), p_ringpack(std::move(p_ringpack_)), q_ringpack(std::move(q_ringpack_)) {
        for (auto v : p_ringpack) pq_ringpack.push_back(v);
        for (auto v : q_ringpack) pq_ringpack.push_back(v);
        ringpack_p_count = (int)p_ringpack.size();
        ringpack_q_count = (int)q_ringpack.size();
        ringpack_pq_count = (int)pq_ringpack.size();
        ckks_llm_compat::check(ckks_b200_pcmm_create(&b200, 0, N1, mlwe_rank, (const uint64_t*)q_ringpack.data(), ringpack_q_count));
    }
    PCMM_Context(const PCMM_Context&) = delete;
    PCMM_Context& operator=(const PCMM_Context&) = delete;
    ~PCMM_Context() { ckks_b200_pcmm_destroy(b200); }

    // (long)(vals[j] * scale) per coefficient and limb (PCMM_Context.cuh, encodeCoeffs / decodeCoeffs); DEVICE arrays
    void encodeCoeffs(MLWEPlaintext& plain, double* vals) {
        std::vector<double> v = ckks_llm_compat::download(vals, (size_t)N1);
        const long scale = NTL::to_long(plain.scale);
        std::vector<uint64_tt> m((size_t)N1 * (plain.L + 1), 0);
        for (int i = 0; i <= plain.l; i++)
            for (int j = 0; j < N1; j++) m[(size_t)i * N1 + j] = ckks_llm_compat::from_signed((long)(v[j] * scale), q_ringpack[i]);
        ckks_llm_compat::upload(plain.mx_device, m);
    }
    void decodeCoeffs(MLWEPlaintext& plain, double* vals) {
        std::vector<uint64_tt> m = ckks_llm_compat::download(plain.mx_device, (size_t)N1);
        const uint64_tt q = q_ringpack[0];
        std::vector<double> v(N1);
        for (int j = 0; j < N1; j++) v[j] = (double)((m[j] <= q / 2 ? (long double)m[j] : (long double)m[j] - (long double)q) / plain.scale.v);
        ckks_llm_compat::upload(vals, v);
    }
};

class PCMM_Scheme {
public:
    PCMM_Context& pcmm_context;
    Scheme_23& scheme;
    Context_23& context;
    SecretKey* sk_ptr = nullptr;

    std::vector<Key*> repackingKeys;
    uint64_tt* repacking_keys_device = nullptr;   // the keys' one block: [k][2 (a, b)][2 limbs (p, q0)][N], NTT domain
    uint64_tt* ppmm_output = nullptr;             // [rows][q_count][(k+1)*N1], grown on demand
    size_t ppmm_output_rows = 0;
    std::mt19937_64 host_rng{0x9ac4};

    PCMM_Scheme(PCMM_Context& pcmm_context, Scheme_23& scheme, SecretKey& sk)
        : pcmm_context(pcmm_context), scheme(scheme), context(scheme.context), sk_ptr(&sk) {}
    // the forms older drivers of the reference use (test_pcmm_boot.cu:50, test_bert_infer.cu:99, test_shuffle.cu:50); the
    // bootstrapper plays no part in the methods below
    template <class BootstrapperLike>
    PCMM_Scheme(PCMM_Context& pcmm_context, Scheme_23& scheme, BootstrapperLike&, SecretKey& sk)
        : pcmm_context(pcmm_context), scheme(scheme), context(scheme.context), sk_ptr(&sk) {}
    template <class BootstrapperLike>
    PCMM_Scheme(PCMM_Context& pcmm_context, Scheme_23& scheme, BootstrapperLike&)
        : pcmm_context(pcmm_context), scheme(scheme), context(scheme.context) {}
    PCMM_Scheme(const PCMM_Scheme&) = delete;
    PCMM_Scheme& operator=(const PCMM_Scheme&) = delete;
    ~PCMM_Scheme() {
        for (Key* k : repackingKeys) delete k;
        if (repacking_keys_device) cudaFree(repacking_keys_device);
        if (ppmm_output) cudaFree(ppmm_output);
    }

    // ringDown (pcmm/ringSwitch.cuh:7-19): component r of the MLWE secret takes coefficients r + j*k of the RLWE secret.
    void convertMLWESKfromRLWESK(MLWESecretKey& mlwe_sk, SecretKey& rlwe_sk) {
        const int N1 = mlwe_sk.N1, k = mlwe_sk.k;
        mlwe_sk.s_coeffs.assign((size_t)k * N1, 0);
        for (int r = 0; r < k; r++)
            for (int j = 0; j < N1; j++) mlwe_sk.s_coeffs[(size_t)r * N1 + j] = rlwe_sk.s_coeffs[r + (size_t)j * k];
        std::vector<uint64_tt> res((size_t)N1 * k * (mlwe_sk.L + 1), 0);
        for (int i = 0; i <= mlwe_sk.L && i < pcmm_context.ringpack_pq_count; i++)
            for (size_t x = 0; x < (size_t)k * N1; x++) res[(size_t)i * k * N1 + x] = ckks_llm_compat::from_signed(mlwe_sk.s_coeffs[x], pcmm_context.pq_ringpack[i]);
        ckks_llm_compat::upload(mlwe_sk.sx_device, res);
    }

    // m = b + sum_r a_r * s_r in Z_q[X]/(X^N1 + 1) per limb (PCMM_Scheme.cuh:533-555), on the host
    void mlweDecrypt(MLWECiphertext& mlwe_cipher, MLWESecretKey& mlwe_sk, MLWEPlaintext& mlwe_plain) {
        const int N1 = mlwe_cipher.N1, k = mlwe_cipher.k;
        std::vector<uint64_tt> ct = ckks_llm_compat::download(mlwe_cipher.cipher_device, (size_t)N1 * (mlwe_cipher.L + 1) * (k + 1));
        std::vector<uint64_tt> m((size_t)N1 * (mlwe_plain.L + 1), 0);
        for (int i = 0; i <= mlwe_cipher.l; i++) {
            const uint64_tt q = pcmm_context.q_ringpack[i];
            const uint64_tt* limb = ct.data() + (size_t)i * (k + 1) * N1;
            std::vector<unsigned __int128> acc(N1, 0);
            for (int r = 0; r < k; r++) {
                const long long* s = mlwe_sk.s_coeffs.data() + (size_t)r * N1;
                const uint64_tt* a = limb + (size_t)r * N1;
                for (int u = 0; u < N1; u++) {
                    if (!s[u]) continue;
                    for (int j = 0; j < N1; j++) {
                        int x = j + u;
                        bool neg = s[u] < 0;
                        if (x >= N1) { x -= N1; neg = !neg; }
                        acc[x] += neg ? (a[j] ? q - a[j] : 0) : a[j];
                    }
                }
            }
            for (int j = 0; j < N1; j++) m[(size_t)i * N1 + j] = (uint64_tt)((acc[j] + limb[(size_t)k * N1 + j]) % q);
        }
        ckks_llm_compat::upload(mlwe_plain.mx_device, m);
        mlwe_plain.l = mlwe_cipher.l;
        mlwe_plain.scale = mlwe_cipher.scale;
    }

    // PCMM_Scheme.cuh:90-125; like the reference a request for more ciphertexts than the rank prints and returns
    void rlweCipherDecompose(Ciphertext& rlwe_cipher, std::vector<MLWECiphertext*> mlwe_cipher_decomposed, uint64_tt mlwe_num, uint64_tt offset) {
        std::vector<uint64_t*> ptrs(mlwe_num ? mlwe_num : 1);
        for (uint64_tt i = 0; i < mlwe_num; i++) ptrs[i] = (uint64_t*)mlwe_cipher_decomposed[offset + i]->cipher_device;
        const int l = pcmm_context.ringpack_q_count - 1;
        const int st = ckks_b200_rlwe_decompose(context.b200, (uint64_t*)rlwe_cipher.cipher_device, rlwe_cipher.L, l, ptrs.data(), (int)mlwe_num,
                                                pcmm_context.N1, pcmm_context.mlwe_rank, 1, 0);
        if (st == CKKS_B200_ERR_SHAPE) { std::cout << ckks_b200_last_error() << std::endl; return; }
        ckks_llm_compat::check(st);
        for (uint64_tt i = 0; i < mlwe_num; i++) {
            mlwe_cipher_decomposed[offset + i]->scale = rlwe_cipher.scale;
            mlwe_cipher_decomposed[offset + i]->l = l;
        }
    }

    // PCMM_Scheme.cuh:152-223: key r is (a_r, -a_r*s + e_r + p*iota(s_r)) over {p, q0} in the NTT domain, iota placing
    // coefficient j at j*k.  Sampled on the host, transformed on the GPU.
    void addRepakcingKey(MLWESecretKey& mlwe_sk, SecretKey& rlwe_sk) {
        const int N = context.N, N1 = mlwe_sk.N1, k = mlwe_sk.k, K = context.K;
        if ((int)repackingKeys.size() == k) { std::cout << "repacking keys already generated!" << std::endl; return; }
        if (pcmm_context.ringpack_p_count != 1) { std::cout << "dnum not supported!" << std::endl; return; }
        const uint64_tt p = pcmm_context.p_ringpack[0], q0 = pcmm_context.q_ringpack[0];
        int p_idx = -1;
        for (int i = 0; i < K; i++) if (context.pVec[i] == p) p_idx = i;
        if (p_idx < 0 || context.qVec[0] != q0) throw std::invalid_argument("the ring-pack moduli must be a special prime and q0 of the context");
        const uint64_tt mods[2] = {p, q0};
        const int mod_idx[2] = {p_idx, K};
        const size_t key_words = (size_t)4 * N;                       // [a, b][p, q0][N]
        ckks_llm_compat::check_cuda(cudaMalloc(&repacking_keys_device, sizeof(uint64_tt) * key_words * k));
        std::normal_distribution<double> gauss(0.0, context.sigma);
        std::vector<uint64_tt> block(key_words * k, 0);
        for (int r = 0; r < k; r++) {
            uint64_tt* a = block.data() + key_words * r;
            uint64_tt* b = a + 2 * (size_t)N;
            std::vector<long long> e(N);
            for (int j = 0; j < N; j++) e[j] = llround(gauss(host_rng));
            for (int m = 0; m < 2; m++)
                for (int j = 0; j < N; j++) {
                    long long v = e[j];
                    unsigned __int128 emb = 0;
                    if (j % k == 0) {                                   // p * iota(s_r)
                        const long long s = mlwe_sk.s_coeffs[(size_t)r * N1 + j / k];
                        emb = s == 0 ? 0 : s > 0 ? (unsigned __int128)(p % mods[m]) : (unsigned __int128)(mods[m] - p % mods[m]) % mods[m];
                    }
                    b[(size_t)m * N + j] = (uint64_tt)((ckks_llm_compat::from_signed(v, mods[m]) + emb) % mods[m]);
                }
        }
        // e + p*iota(s_r) into the NTT domain: limb p with the p transform, limb q0 with the q0 transform
        ckks_llm_compat::upload(repacking_keys_device, block);
        for (int m = 0; m < 2; m++)
            ckks_llm_compat::check(ckks_b200_ntt_forward(context.b200, (uint64_t*)repacking_keys_device, 2 + m, mod_idx[m], k, 1, 4, 0));
        block = ckks_llm_compat::download(repacking_keys_device, key_words * k);
        for (int r = 0; r < k; r++) {
            uint64_tt* a = block.data() + key_words * r;
            uint64_tt* b = a + 2 * (size_t)N;
            for (int m = 0; m < 2; m++) {
                const uint64_tt* s = rlwe_sk.sx_host + (size_t)mod_idx[m] * N;
                for (int j = 0; j < N; j++) {
                    const size_t x = (size_t)m * N + j;
                    a[x] = host_rng() % mods[m];
                    b[x] = ckks_llm_compat::submod(b[x], ckks_llm_compat::mulmod(a[x], s[j], mods[m]), mods[m]);
                }
            }
        }
        ckks_llm_compat::upload(repacking_keys_device, block);
        for (int r = 0; r < k; r++) repackingKeys.push_back(new Key(repacking_keys_device + key_words * r, N, 0, 1, 1));
    }

    // PCMM_Scheme.cuh:362-430
    void mlweCipherPacking(Ciphertext& rlwe_cipher, std::vector<MLWECiphertext*> mlwe_cipher_decomposed, uint64_tt mlwe_num, uint64_tt offset) {
        if (!repacking_keys_device) throw std::invalid_argument("addRepakcingKey has not been called");
        std::vector<uint64_t*> ptrs(mlwe_num ? mlwe_num : 1);
        for (uint64_tt i = 0; i < mlwe_num; i++) ptrs[i] = (uint64_t*)mlwe_cipher_decomposed[offset + i]->cipher_device;
        ckks_llm_compat::check(ckks_b200_mlwe_packing(context.b200, (uint64_t*)rlwe_cipher.cipher_device, rlwe_cipher.L, ptrs.data(), (int)mlwe_num,
                                                      pcmm_context.N1, pcmm_context.mlwe_rank, (const uint64_t*)repacking_keys_device, 0));
        rlwe_cipher.l = pcmm_context.ringpack_q_count - 1 - 1;          // :418-420
        rlwe_cipher.scale = mlwe_cipher_decomposed[offset]->scale;
    }

    // pcmm/PPMM_kernel.cuh:254-349: shape violations print the reference's message and return; the first limb of
    // result row i replaces ciphertext i for i < mlwe_num and the scales are updated (:345-348)
    void PPMM(float* plain_mat, std::vector<MLWECiphertext*> mlwe_cipher_decomposed, int mat_M, int mat_N, int mat_K, int mlwe_num) {
        if (mat_K != pcmm_context.N1) { std::cout << "matrix K should be equal to N1!" << std::endl; return; }
        if (mat_N != mlwe_num) { std::cout << "matrix N should be equal to mlwe number!" << std::endl; return; }
        const long C = (long)(pcmm_context.mlwe_rank + 1) * pcmm_context.N1;
        if (ppmm_output_rows < (size_t)mat_M) {
            if (ppmm_output) cudaFree(ppmm_output);
            ckks_llm_compat::check_cuda(cudaMalloc(&ppmm_output, sizeof(uint64_tt) * C * pcmm_context.ringpack_q_count * mat_M));
            ppmm_output_rows = mat_M;
        }
        std::vector<const uint64_t*> ptrs(mlwe_num);
        std::vector<uint64_t*> wptrs(mlwe_num);
        for (int i = 0; i < mlwe_num; i++) {
            ptrs[i] = (const uint64_t*)mlwe_cipher_decomposed[i]->cipher_device;
            wptrs[i] = (uint64_t*)mlwe_cipher_decomposed[i]->cipher_device;
        }
        // scaler = (long)(q_last * 2^49 / scale): :283-284 writes q_ringpack[1], the last of the reference's two moduli
        // and the one its kernel rescales by
        const NTL::RR q_div((long double)pcmm_context.q_ringpack[pcmm_context.ringpack_q_count - 1]);
        const long scaler = NTL::to_long(q_div * NTL::RR((long double)(1LL << 49)) / mlwe_cipher_decomposed[0]->scale);
        ckks_llm_compat::check(ckks_b200_pcmm_ppmm(pcmm_context.b200, plain_mat, ptrs.data(), (uint64_t*)ppmm_output, mat_M, mat_N, mat_K, mlwe_num,
                                                   (double)scaler, 0, C, CKKS_B200_PCMM_AUTO, 0));
        const int rows_back = mlwe_num < mat_M ? mlwe_num : mat_M;
        ckks_llm_compat::check(ckks_b200_pcmm_copy_back(pcmm_context.b200, (const uint64_t*)ppmm_output, wptrs.data(), rows_back, 1, 0));
        for (int i = 0; i < mlwe_num; i++)
            mlwe_cipher_decomposed[i]->scale = mlwe_cipher_decomposed[i]->scale * NTL::RR((long double)scaler) / q_div;
    }

    // Called by src/bert (Bert.cuh:403-412,472-490) and declared nowhere in the reference: there is no behaviour to
    // reproduce.  Declared so that such callers compile; does nothing and says so once.
    void realData_coeffShift(Ciphertext& rlwe_cipher, int direction) {
        (void)rlwe_cipher; (void)direction;
        static bool said = false;
        if (!said) { std::cout << "realData_coeffShift: not defined by the reference, nothing done" << std::endl; said = true; }
    }

    // PCMM_Scheme.cuh:502-529: decrypt, bit-reverse the plaintext coefficients within the slots, encrypt again.
    void coeffBitRev(Ciphertext& rlwe_cipher) {
        if (!sk_ptr) throw std::invalid_argument("coeffBitRev needs the secret key");
        Plaintext plain(context.N, rlwe_cipher.L, rlwe_cipher.l, rlwe_cipher.slots, rlwe_cipher.scale);
        scheme.decryptMsg(plain, *sk_ptr, rlwe_cipher);
        context.FromNTTInplace(plain.mx_device, 0, context.K, 1, rlwe_cipher.l + 1, rlwe_cipher.L + 1);
        std::vector<uint64_tt> m = ckks_llm_compat::download(plain.mx_device, (size_t)context.N * (rlwe_cipher.L + 1));
        const int logn = (int)context.logN;
        for (int i = 0; i <= rlwe_cipher.l; i++) {
            uint64_tt* limb = m.data() + (size_t)i * context.N;
            for (uint32_t x = 0; x < (uint32_t)context.N; x++) {
                uint32_t y = 0;
                for (int b = 0; b < logn; b++) y |= ((x >> b) & 1u) << (logn - 1 - b);
                if (x < y) std::swap(limb[x], limb[y]);
            }
        }
        ckks_llm_compat::upload(plain.mx_device, m);
        context.ToNTTInplace(plain.mx_device, 0, context.K, 1, rlwe_cipher.l + 1, rlwe_cipher.L + 1);
        SecretKey* keep = scheme.enc_sk;
        scheme.enc_sk = sk_ptr;
        scheme.encryptMsg(rlwe_cipher, plain);
        scheme.enc_sk = keep;
    }
};

// ---------------------------------------------------------------------------------------------------------------
// Small utilities the reference's drivers use around the path (TimeUtils.cuh:10-35, Utils.cuh:135-164,447-470,
// precision.cuh:9-60,179-230).
class CUDATimer {
public:
    cudaEvent_t start_event, stop_event;
    explicit CUDATimer() { cudaEventCreate(&start_event); cudaEventCreate(&stop_event); }
    ~CUDATimer() { cudaEventDestroy(start_event); cudaEventDestroy(stop_event); }
    inline void start() const { cudaEventRecord(start_event); }
    inline float stop() {
        cudaEventRecord(stop_event);
        cudaEventSynchronize(stop_event);
        float milliseconds = 0;
        cudaEventElapsedTime(&milliseconds, start_event, stop_event);
        return milliseconds;
    }
};

static std::mt19937_64 rng(20260101);          // the drivers' global generator (Utils.cuh:135; seeded here, not from a device)
inline void randomDoubleArray(double* doubleArray, long num, double bound = 1.0) {
    std::uniform_real_distribution<double> randnum(-bound, bound);
    for (long i = 0; i < num; ++i) doubleArray[i] = randnum(rng);
}
inline void print_device_array(double* data, int num, const char* vname) {
    std::vector<double> h = ckks_llm_compat::download(data, (size_t)(num < 8 ? num : 8));
    printf("%s = [", vname);
    for (double v : h) printf("%.8f, ", v);
    printf("...]\n");
}
// residues: the first words of each of mod_num limbs of N words (Utils.cuh:362-380)
inline void print_device_array(uint64_tt* data, int N, int mod_num, const char* vname) {
    const int show = N < 16 ? N : 16;
    printf("%s = [", vname);
    for (int i = 0; i < mod_num; i++) {
        std::vector<uint64_tt> h = ckks_llm_compat::download(data + (size_t)i * N, (size_t)show);
        printf("[");
        for (uint64_tt v : h) printf("%llu, ", v);
        printf("],\n");
    }
}
struct PrecisionStats {
    double min_log2 = 0, avg_log2 = 0, max_err = 0;
    std::string String() const {
        char buf[200];
        snprintf(buf, sizeof(buf), "precision (log2): min %.2f  avg %.2f   max abs error %.3e\n", min_log2, avg_log2, max_err);
        return buf;
    }
};
inline PrecisionStats GetPrecisionStats(const std::vector<double>& valuesTest, const std::vector<double>& valuesWant) {
    PrecisionStats st;
    st.min_log2 = 1e9;
    for (size_t i = 0; i < valuesWant.size(); i++) {
        const double e = std::fabs(valuesTest[i] - valuesWant[i]);
        const double p = e > 0 ? -std::log2(e) : 64.0;
        st.min_log2 = p < st.min_log2 ? p : st.min_log2;
        st.avg_log2 += p / valuesWant.size();
        st.max_err = e > st.max_err ? e : st.max_err;
    }
    return st;
}

#endif  // CKKS_LLM_COMPAT_HPP
