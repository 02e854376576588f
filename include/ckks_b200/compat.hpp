// C++ classes with the reference's names and signatures for the hot path, forwarding to
// the C ABI (ckks_b200.h).  For callers that want Context_23 / MLWECiphertext /
// PCMM_Context / PCMM_Scheme without the rest of the reference tree.
//
// Mirrors (paths relative to the reference root):
//   Context_23::ToNTTInplace / FromNTTInplace   src/ckks/include/Context_23.cuh:847-889
//   Context_23::modUpQjtoT_23                   src/ckks/include/BasisConv.cuh:161-179
//   MLWECiphertext                              src/ckks/include/pcmm/MLWECiphertext.cuh:6-78
//   PCMM_Context                                src/ckks/include/pcmm/PCMM_Context.h:14-90
//   PCMM_Scheme::PPMM                           src/ckks/include/pcmm/PPMM_kernel.cuh:254-349
// Differences: `NTL::RR scale` is `long double`; constructors take the modulus lists
// explicitly (the reference hard-codes them per logN in Params.cuh); CUDA errors surface as
// std::runtime_error instead of being ignored; shape violations print the reference's
// message and return, as the reference does.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>
#include <iostream>
#include <stdexcept>
#include <string>
#include <map>
#include <vector>

#include "../ckks_b200.h"

namespace ckks_b200 {

typedef unsigned long long uint64_tt;

inline void check(int status) {
    if (status != CKKS_B200_OK) throw std::runtime_error(std::string("ckks_b200: ") + ckks_b200_last_error());
}

class Context_23 {
public:
    int logN;
    long N;
    int L, K, p_num, q_num, t_num;
    std::vector<uint64_tt> pVec, qVec, tVec;
    ckks_b200_context* b200 = nullptr;

    Context_23(int logN_, std::vector<uint64_tt> p, std::vector<uint64_tt> q, std::vector<uint64_tt> t, int device = 0)
        : logN(logN_), N(1L << logN_), pVec(std::move(p)), qVec(std::move(q)), tVec(std::move(t)) {
        p_num = (int)pVec.size(); q_num = (int)qVec.size(); t_num = (int)tVec.size();
        K = p_num; L = q_num - 1;
        check(ckks_b200_context_create(&b200, device, logN, (const uint64_t*)pVec.data(), p_num,
                                       (const uint64_t*)qVec.data(), q_num, (const uint64_t*)tVec.data(), t_num));
    }
    Context_23(const Context_23&) = delete;
    Context_23& operator=(const Context_23&) = delete;
    ~Context_23() { ckks_b200_context_destroy(b200); }

    void ToNTTInplace(uint64_tt* device_a, int start_poly_idx, int start_mod_idx, int poly_num, int mod_num,
                      int poly_mod_len, cudaStream_t stream = 0) {
        check(ckks_b200_ntt_forward(b200, (uint64_t*)device_a, start_poly_idx, start_mod_idx, poly_num, mod_num,
                                    poly_mod_len, stream));
    }
    void FromNTTInplace(uint64_tt* device_a, int start_poly_idx, int start_mod_idx, int poly_num, int mod_num,
                        int poly_mod_len, cudaStream_t stream = 0) {
        check(ckks_b200_ntt_inverse(b200, (uint64_t*)device_a, start_poly_idx, start_mod_idx, poly_num, mod_num,
                                    poly_mod_len, stream));
    }
    void modUpQjtoT_23(uint64_tt* output, uint64_tt* input, int l, int batch_size, cudaStream_t stream = 0) {
        check(ckks_b200_modup_qj_to_t(b200, (uint64_t*)output, (const uint64_t*)input, l, batch_size, stream));
    }

    // Key-switch chain of Scheme_23::mult_23 (KeySwitch_23.cuh:219-232); gamma as in Params.cuh:28.
    int gamma = 3;
    void external_product_T(uint64_tt* output, uint64_tt* cipher_modUp_QjtoT, uint64_tt* swk_modUp_RitoT, int l,
                            cudaStream_t stream = 0) {
        check(ckks_b200_external_product_t(b200, (uint64_t*)output, (const uint64_t*)cipher_modUp_QjtoT,
                                           (const uint64_t*)swk_modUp_RitoT, l, gamma, stream));
    }
    void FromNTTInplace_for_externalProduct(uint64_tt* device_a, int l, cudaStream_t stream = 0) {
        check(ckks_b200_ntt_inverse_ext(b200, (uint64_t*)device_a, l, gamma, stream));
    }
    void modUpTtoPQl_23(uint64_tt* modUp_TtoQj_buffer, uint64_tt* exProduct_T_temp, int l, int batch_size,
                        cudaStream_t stream = 0) {
        check(ckks_b200_modup_t_to_pql(b200, (uint64_t*)modUp_TtoQj_buffer, (const uint64_t*)exProduct_T_temp, l, gamma,
                                       batch_size, stream));
    }
    void modDownPQltoQl_23(uint64_tt* output, uint64_tt* modUp_TtoQj_buffer, int l, int batch_size, cudaStream_t stream = 0) {
        check(ckks_b200_moddown_pql_to_ql(b200, (uint64_t*)output, (const uint64_t*)modUp_TtoQj_buffer, l, gamma, batch_size,
                                          stream));
    }
};

// RLWE ciphertext carrier with the members the path reads (Ciphertext.cuh:5-100): cipher_device holds the a
// limbs then the b limbs, each [L+1][N], and is owned by the caller.
struct Ciphertext {
    uint64_tt* cipher_device = nullptr;
    long N = 0;
    int L = 0, l = 0, slots = 0;
    long double scale = 1.0L;
};

// Scheme_23::rescaleAndEqual(Ciphertext&) (Scheme_23.cuh:368-385).
class Scheme_23 {
public:
    Context_23& context;
    explicit Scheme_23(Context_23& context_) : context(context_) {}
    // Scheme_23::mult_23 (KeySwitch_23.cuh:192-236); rlk_23 is the relinearisation key block on the device.
    uint64_tt* rlk_23 = nullptr;
    void mult_23(Ciphertext& cipher_res, Ciphertext& cipher1, Ciphertext& cipher2, cudaStream_t stream = 0) {
        if (cipher1.l == 0 || cipher2.l == 0) throw std::invalid_argument("Ciphertexts are on level 0");
        if (rlk_23 == nullptr) throw std::invalid_argument("rotKey_23 not exists");
        const int l = cipher1.l < cipher2.l ? cipher1.l : cipher2.l;
        check(ckks_b200_mult(context.b200, (uint64_t*)cipher_res.cipher_device, (const uint64_t*)cipher1.cipher_device,
                             (const uint64_t*)cipher2.cipher_device, (const uint64_t*)rlk_23, l, context.gamma, stream));
        cipher_res.l = l;
        cipher_res.scale = cipher1.scale * cipher2.scale;
    }
    // Scheme_23::conjugate_23 / conjugateAndEqual_23 (KeySwitch_23.cuh:433-507); ConjKey_23 is the key block on the device.
    uint64_tt* ConjKey_23 = nullptr;
    void conjugate_23(Ciphertext& cipher_res, Ciphertext& cipher, cudaStream_t stream = 0) {
        if (ConjKey_23 == nullptr) throw std::invalid_argument("conjKey_23 not exists");
        check(ckks_b200_conjugate(context.b200, (uint64_t*)cipher_res.cipher_device, (const uint64_t*)cipher.cipher_device,
                                  (const uint64_t*)ConjKey_23, cipher.l, context.gamma, stream));
        cipher_res.l = cipher.l;
        cipher_res.scale = cipher.scale;
    }
    void conjugateAndEqual_23(Ciphertext& cipher, cudaStream_t stream = 0) { conjugate_23(cipher, cipher, stream); }
    // Scheme_23::leftRotate_23 / leftRotateAndEqual_23 (KeySwitch_23.cuh:509-581); rotKey_vec_23[rotSlots] is the key
    // block of that rotation on the device (the reference's addLeftRotKey_23 fills it).
    std::map<long, uint64_tt*> rotKey_vec_23;
    void leftRotate_23(Ciphertext& cipher_res, Ciphertext& cipher, long rotSlots, cudaStream_t stream = 0) {
        auto it = rotKey_vec_23.find(rotSlots);
        if (it == rotKey_vec_23.end() || it->second == nullptr) throw std::invalid_argument("rotKey_23 not exists");
        check(ckks_b200_rotate(context.b200, (uint64_t*)cipher_res.cipher_device, (const uint64_t*)cipher.cipher_device,
                               (const uint64_t*)it->second, rotSlots, cipher.l, context.gamma, stream));
        cipher_res.l = cipher.l;
        cipher_res.scale = cipher.scale;
    }
    void leftRotateAndEqual_23(Ciphertext& cipher, long rotSlots, cudaStream_t stream = 0) {
        leftRotate_23(cipher, cipher, rotSlots, stream);
    }
    void rescaleAndEqual(Ciphertext& cipher, cudaStream_t stream = 0) {
        check(ckks_b200_rescale(context.b200, (uint64_t*)cipher.cipher_device, cipher.L, cipher.l, stream));
        cipher.scale = cipher.scale / (long double)context.qVec[cipher.l];
        cipher.l -= 1;
    }
};

// Bootstrapper::modUpQ0toQL(Ciphertext&, int) (bootstrapping/Bootstrapper.cuh:192-209).
class Bootstrapper {
public:
    Context_23& context;
    uint64_tt precision;
    Bootstrapper(Context_23& context_, uint64_tt precision_) : context(context_), precision(precision_) {}
    void modUpQ0toQL(Ciphertext& cipher, int target_level, cudaStream_t stream = 0) {
        if (cipher.l != 0) return;
        const int scale_up = (int)(context.qVec[0] / precision);       // the reference kernel's parameter is an int
        check(ckks_b200_modup_q0_to_ql(context.b200, (uint64_t*)cipher.cipher_device, cipher.L, target_level, scale_up, stream));
        cipher.l = target_level;
    }
};

// One cudaMalloc per object, freed in the destructor, deep copy on copy: the reference's
// ownership rules (MLWECiphertext.cuh:26-77).
class MLWECiphertext {
public:
    uint64_tt* cipher_device = nullptr;
    int N1 = 0, L = 0, l = 0, k = 0;
    long double scale = 0;

    MLWECiphertext() {}
    MLWECiphertext(int N1_, int L_, int l_, int k_, long double scale_) : N1(N1_), L(L_), l(l_), k(k_), scale(scale_) {
        if (cudaMalloc(&cipher_device, bytes()) != cudaSuccess) throw std::runtime_error("cudaMalloc failed");
    }
    MLWECiphertext(const MLWECiphertext& c) : N1(c.N1), L(c.L), l(c.l), k(c.k), scale(c.scale) {
        if (cudaMalloc(&cipher_device, bytes()) != cudaSuccess) throw std::runtime_error("cudaMalloc failed");
        if (c.cipher_device) cudaMemcpy(cipher_device, c.cipher_device, bytes(), cudaMemcpyDeviceToDevice);
    }
    MLWECiphertext& operator=(const MLWECiphertext& c) {
        if (this == &c) return *this;
        if (cipher_device && bytes() != c.bytes()) { cudaFree(cipher_device); cipher_device = nullptr; }
        N1 = c.N1; L = c.L; l = c.l; k = c.k; scale = c.scale;
        if (!cipher_device && cudaMalloc(&cipher_device, bytes()) != cudaSuccess) throw std::runtime_error("cudaMalloc failed");
        if (c.cipher_device) cudaMemcpy(cipher_device, c.cipher_device, bytes(), cudaMemcpyDeviceToDevice);
        return *this;
    }
    virtual ~MLWECiphertext() {
        if (cipher_device) { cudaFree(cipher_device); cipher_device = nullptr; }
    }
    size_t bytes() const { return sizeof(uint64_tt) * (size_t)N1 * (L + 1) * (k + 1); }
};

class PCMM_Context {
public:
    int N1, mlwe_rank;
    int ringpack_p_count, ringpack_q_count, ringpack_pq_count;
    std::vector<uint64_tt> p_ringpack, q_ringpack, pq_ringpack;
    ckks_b200_pcmm* b200 = nullptr;

    PCMM_Context(int N1_, int mlwe_rank_, std::vector<uint64_tt> p, std::vector<uint64_tt> q, int device = 0)
        : N1(N1_), mlwe_rank(mlwe_rank_), p_ringpack(std::move(p)), q_ringpack(std::move(q)) {
        for (auto v : p_ringpack) pq_ringpack.push_back(v);
        for (auto v : q_ringpack) pq_ringpack.push_back(v);
        ringpack_p_count = (int)p_ringpack.size();
        ringpack_q_count = (int)q_ringpack.size();
        ringpack_pq_count = (int)pq_ringpack.size();
        check(ckks_b200_pcmm_create(&b200, device, N1, mlwe_rank, (const uint64_t*)q_ringpack.data(), ringpack_q_count));
    }
    PCMM_Context(const PCMM_Context&) = delete;
    PCMM_Context& operator=(const PCMM_Context&) = delete;
    ~PCMM_Context() { ckks_b200_pcmm_destroy(b200); }
};

// scaler = (long)(q_last * target / scale) and the scale PPMM leaves, scale * scaler / q_last
// (PPMM_kernel.cuh:283-284,346 write q_ringpack[1], the last of the reference's two moduli and the one its kernel
// rescales by; with more limbs that is the last one).
inline long ppmm_scaler(const std::vector<uint64_tt>& q_ringpack, long double scale, long double target = (long double)(1LL << 49)) {
    return (long)((long double)q_ringpack.back() * target / scale);
}
inline long double ppmm_scale_after(const std::vector<uint64_tt>& q_ringpack, long double scale, long scaler) {
    return scale * scaler / (long double)q_ringpack.back();
}

class PCMM_Scheme {
public:
    PCMM_Context& pcmm_context;
    uint64_tt* ppmm_output = nullptr;     // [rows][q_count][(k+1)*N1], grown on demand
    size_t ppmm_output_rows = 0;
    int algo = CKKS_B200_PCMM_AUTO;

    explicit PCMM_Scheme(PCMM_Context& ctx) : pcmm_context(ctx) {}
    ~PCMM_Scheme() { if (ppmm_output) cudaFree(ppmm_output); }

    void PPMM(float* plain_mat, std::vector<MLWECiphertext*> mlwe_cipher_decomposed, int mat_M, int mat_N, int mat_K,
              int mlwe_num, cudaStream_t stream = 0) {
        if (mat_K != pcmm_context.N1) { std::cout << "matrix K should be equal to N1!" << std::endl; return; }
        if (mat_N != mlwe_num) { std::cout << "matrix N should be equal to mlwe number!" << std::endl; return; }
        const long C = (long)(pcmm_context.mlwe_rank + 1) * pcmm_context.N1;
        if (ppmm_output_rows < (size_t)mat_M) {
            if (ppmm_output) cudaFree(ppmm_output);
            if (cudaMalloc(&ppmm_output, sizeof(uint64_tt) * C * pcmm_context.ringpack_q_count * mat_M) != cudaSuccess)
                throw std::runtime_error("cudaMalloc failed");
            ppmm_output_rows = mat_M;
        }
        std::vector<const uint64_t*> ptrs(mlwe_num);
        std::vector<uint64_t*> wptrs(mlwe_num);
        for (int i = 0; i < mlwe_num; i++) {
            ptrs[i] = (const uint64_t*)mlwe_cipher_decomposed[i]->cipher_device;
            wptrs[i] = (uint64_t*)mlwe_cipher_decomposed[i]->cipher_device;
        }
        const long scaler = ppmm_scaler(pcmm_context.q_ringpack, mlwe_cipher_decomposed[0]->scale);
        check(ckks_b200_pcmm_ppmm(pcmm_context.b200, plain_mat, ptrs.data(), (uint64_t*)ppmm_output, mat_M, mat_N, mat_K,
                                  mlwe_num, (double)scaler, 0, C, algo, stream));
        const int rows_back = mlwe_num < mat_M ? mlwe_num : mat_M;
        check(ckks_b200_pcmm_copy_back(pcmm_context.b200, (const uint64_t*)ppmm_output, wptrs.data(), rows_back, 1, stream));
        for (int i = 0; i < mlwe_num; i++)
            mlwe_cipher_decomposed[i]->scale = ppmm_scale_after(pcmm_context.q_ringpack, mlwe_cipher_decomposed[i]->scale, scaler);
    }

    // rlweCipherDecompose of every source (PCMM_Scheme.cuh:90-125) feeding PPMM, as the one call that never
    // writes the decomposed ciphertexts.  The sources are in the coefficient domain (the state between the
    // decomposition's inverse and forward transforms); `scale` is theirs.  mlwe_cipher_decomposed only
    // receives what PPMM leaves in it: the first limb of result row i in ciphertext i, and the new scale.
    void decomposeAndPPMM(float* plain_mat, const std::vector<ckks_b200_rlwe_source>& sources, double scale,
                          std::vector<MLWECiphertext*> mlwe_cipher_decomposed, int mat_M, int mat_N, int mat_K,
                          int mlwe_num, cudaStream_t stream = 0) {
        if (mat_K != pcmm_context.N1) { std::cout << "matrix K should be equal to N1!" << std::endl; return; }
        if (mat_N != mlwe_num) { std::cout << "matrix N should be equal to mlwe number!" << std::endl; return; }
        const long C = (long)(pcmm_context.mlwe_rank + 1) * pcmm_context.N1;
        if (ppmm_output_rows < (size_t)mat_M) {
            if (ppmm_output) cudaFree(ppmm_output);
            if (cudaMalloc(&ppmm_output, sizeof(uint64_tt) * C * pcmm_context.ringpack_q_count * mat_M) != cudaSuccess)
                throw std::runtime_error("cudaMalloc failed");
            ppmm_output_rows = mat_M;
        }
        const long scaler = ppmm_scaler(pcmm_context.q_ringpack, scale);
        check(ckks_b200_pcmm_ppmm_rlwe(pcmm_context.b200, plain_mat, sources.data(), (int)sources.size(),
                                       (uint64_t*)ppmm_output, mat_M, mat_N, mat_K, mlwe_num, (double)scaler, 0, C, stream));
        std::vector<uint64_t*> wptrs(mlwe_num);
        for (int i = 0; i < mlwe_num; i++) wptrs[i] = (uint64_t*)mlwe_cipher_decomposed[i]->cipher_device;
        const int rows_back = mlwe_num < mat_M ? mlwe_num : mat_M;
        check(ckks_b200_pcmm_copy_back(pcmm_context.b200, (const uint64_t*)ppmm_output, wptrs.data(), rows_back, 1, stream));
        for (int i = 0; i < mlwe_num; i++) mlwe_cipher_decomposed[i]->scale = ppmm_scale_after(pcmm_context.q_ringpack, scale, scaler);
    }
};

}  // namespace ckks_b200
