// Thin driver around the REAL reference (haozetao/ckks_llm), compiled from the reference
// sources where they lie (never copied into this repository) into oracle/_ref/.
//
// TEST INFRASTRUCTURE ONLY.  It exposes, through a few extern "C" entry points,
//   * the reference's own host table builders (findMthRootOfUnity,
//     fillTablePsi128_special, fillTablePsi_shoup128: src/ckks/include/Utils.cuh), and
//   * the reference's own CUDA kernels for the hot path, launched by the reference's own
//     host launchers where those need no big-number state:
//     Context_23::ToNTTInplace / FromNTTInplace (src/ckks/include/Context_23.cuh:847-889),
//     Context_23::modUpQjtoT_23 (src/ckks/include/BasisConv.cuh:161-179), and
//     pcmm_cuda_core_kernel<mat_N> with the launch shape of PCMM_Scheme::PPMM
//     (src/ckks/include/pcmm/PPMM_kernel.cuh:294-329).
// The reference's constructors need the NTL big-number library, which is absent; the
// driver therefore fills the handful of plain-integer members those launchers read on a
// zero-initialised Context_23 object and uploads tables passed in by the caller.  NTL
// itself is replaced by the do-nothing stand-in under oracle/ref_shim/.
#include <iostream>
#include <string>
#include <sstream>
#include <vector>
#include <cmath>
using namespace std;

#include "Context_23.cuh"
#include "Scheme_23.cuh"
#include "TimeUtils.cuh"
#include "pcmm/PCMM_Context.cuh"
#include "pcmm/PCMM_Scheme.cuh"
#include "bootstrapping/Bootstrapping.cuh"

#define RD_CUDA(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { fprintf(stderr, "ref_driver: %s -> %s\n", #x, cudaGetErrorString(e_)); return 100 + (int)e_; } } while (0)

extern "C" unsigned long long ref_find_mth_root(unsigned long long M, unsigned long long q) {
    return findMthRootOfUnity(M, q);
}

extern "C" void ref_fill_tables(unsigned long long psi, unsigned long long q, unsigned n,
                                unsigned long long* psi_tab, unsigned long long* psiinv_tab,
                                unsigned long long* psi_shoup, unsigned long long* psiinv_shoup) {
    uint64_tt psiinv = modinv128(psi, q);
    uint64_tt ninv = modinv128(n, q);
    fillTablePsi128_special(psi, q, psiinv, psi_tab, psiinv_tab, n, ninv);
    fillTablePsi_shoup128(psi_tab, q, psiinv_tab, psi_shoup, psiinv_shoup, n);
}

static Context_23* fake_context() {
    // No constructor runs: only plain-integer and pointer members are used below.
    return (Context_23*)calloc(1, sizeof(Context_23));
}

static int upload_pqt(const unsigned long long* pqt, int n_mod) {
    std::vector<uint64_tt> m(pqt, pqt + n_mod), m2(n_mod), mh(n_mod), ml(n_mod);
    for (int i = 0; i < n_mod; i++) {
        m2[i] = m[i] * 2;
        unsigned __int128 mu = (~(unsigned __int128)0) / m[i];
        mh[i] = (uint64_tt)(mu >> 64);
        ml[i] = (uint64_tt)mu;
    }
    RD_CUDA(cudaMemcpyToSymbol(pqt_cons, m.data(), 8 * n_mod));
    RD_CUDA(cudaMemcpyToSymbol(pqt2_cons, m2.data(), 8 * n_mod));
    RD_CUDA(cudaMemcpyToSymbol(pqt_mu_cons_high, mh.data(), 8 * n_mod));
    RD_CUDA(cudaMemcpyToSymbol(pqt_mu_cons_low, ml.data(), 8 * n_mod));
    return 0;
}

// Forward / inverse NTT of h_data [poly_num][poly_mod_len][N] with the reference kernels.
extern "C" int ref_ntt(unsigned long long* h_data, int logN, const unsigned long long* pqt, int n_mod,
                       int start_poly_idx, int start_mod_idx, int poly_num, int mod_num,
                       int poly_mod_len, int inverse) {
    if (n_mod > max_pqt_num) return 1;
    const long N = 1L << logN;
    int rc = upload_pqt(pqt, n_mod);
    if (rc) return rc;
    std::vector<uint64_tt> psi((size_t)n_mod * N), psiinv((size_t)n_mod * N), psis((size_t)n_mod * N),
        psiinvs((size_t)n_mod * N), ninv(n_mod), ninvs(n_mod);
    for (int i = 0; i < n_mod; i++) {
        uint64_tt root = findMthRootOfUnity(2 * N, pqt[i]);
        ref_fill_tables(root, pqt[i], (unsigned)N, (unsigned long long*)&psi[(size_t)i * N],
                        (unsigned long long*)&psiinv[(size_t)i * N], (unsigned long long*)&psis[(size_t)i * N],
                        (unsigned long long*)&psiinvs[(size_t)i * N]);
        ninv[i] = modinv128(N, pqt[i]);
        ninvs[i] = x_Shoup(ninv[i], pqt[i]);
    }
    Context_23* c = fake_context();
    c->N = N;
    c->logN = logN;
    size_t tb = sizeof(uint64_tt) * n_mod * N;
    RD_CUDA(cudaMalloc(&c->psi_table_device, tb));
    RD_CUDA(cudaMalloc(&c->psiinv_table_device, tb));
    RD_CUDA(cudaMalloc(&c->psi_shoup_table_device, tb));
    RD_CUDA(cudaMalloc(&c->psiinv_shoup_table_device, tb));
    RD_CUDA(cudaMalloc(&c->n_inv_device, 8 * n_mod));
    RD_CUDA(cudaMalloc(&c->n_inv_shoup_device, 8 * n_mod));
    RD_CUDA(cudaMemcpy(c->psi_table_device, psi.data(), tb, cudaMemcpyHostToDevice));
    RD_CUDA(cudaMemcpy(c->psiinv_table_device, psiinv.data(), tb, cudaMemcpyHostToDevice));
    RD_CUDA(cudaMemcpy(c->psi_shoup_table_device, psis.data(), tb, cudaMemcpyHostToDevice));
    RD_CUDA(cudaMemcpy(c->psiinv_shoup_table_device, psiinvs.data(), tb, cudaMemcpyHostToDevice));
    RD_CUDA(cudaMemcpy(c->n_inv_device, ninv.data(), 8 * n_mod, cudaMemcpyHostToDevice));
    RD_CUDA(cudaMemcpy(c->n_inv_shoup_device, ninvs.data(), 8 * n_mod, cudaMemcpyHostToDevice));
    uint64_tt* d = nullptr;
    size_t db = sizeof(uint64_tt) * (size_t)poly_num * poly_mod_len * N;
    RD_CUDA(cudaMalloc(&d, db));
    RD_CUDA(cudaMemcpy(d, h_data, db, cudaMemcpyHostToDevice));
    if (inverse) c->FromNTTInplace(d, start_poly_idx, start_mod_idx, poly_num, mod_num, poly_mod_len);
    else c->ToNTTInplace(d, start_poly_idx, start_mod_idx, poly_num, mod_num, poly_mod_len);
    RD_CUDA(cudaGetLastError());
    RD_CUDA(cudaDeviceSynchronize());
    RD_CUDA(cudaMemcpy(h_data, d, db, cudaMemcpyDeviceToHost));
    cudaFree(d);
    cudaFree(c->psi_table_device); cudaFree(c->psiinv_table_device);
    cudaFree(c->psi_shoup_table_device); cudaFree(c->psiinv_shoup_table_device);
    cudaFree(c->n_inv_device); cudaFree(c->n_inv_shoup_device);
    free(c);
    return 0;
}

// modUpQjtoT_23 at level l.  Tables are for level l only, in the reference's layout:
// hat_inv[blk*p_num+j], hat_mod_t[(blk*t_num+k)*p_num+j], blk_mod_t[blk*t_num+k].
extern "C" int ref_modup(unsigned long long* h_out, const unsigned long long* h_in, int logN,
                         const unsigned long long* pqt, int p_num, int q_num, int t_num, int l, int batch,
                         const unsigned long long* hat_inv, const unsigned long long* hat_inv_shoup,
                         const unsigned long long* hat_mod_t, const unsigned long long* blk_mod_t) {
    const int n_mod = p_num + q_num + t_num;
    if (n_mod > max_pqt_num || p_num > max_p_num || t_num > max_tnum) return 1;
    const long N = 1L << logN;
    int rc = upload_pqt(pqt, n_mod);
    if (rc) return rc;
    Context_23* c = fake_context();
    c->N = N;
    c->p_num = p_num; c->q_num = q_num; c->t_num = t_num;
    c->gamma = 0;
    c->Qj_blockNum = (q_num + p_num - 1) / p_num;
    const int B = c->Qj_blockNum;
    const int blocks = (l + 1 + p_num - 1) / p_num;
    // the launcher offsets each table by l * (size of one level); allocate so that offset
    // lands on the level passed in
    size_t s_inv = (size_t)B * p_num, s_hat = (size_t)B * t_num * p_num, s_blk = (size_t)B * t_num;
    RD_CUDA(cudaMalloc(&c->QjHatInvVecModQj_23_device, 8 * s_inv * (l + 1)));
    RD_CUDA(cudaMalloc(&c->QjHatInvVecModQj_23_shoup_device, 8 * s_inv * (l + 1)));
    RD_CUDA(cudaMalloc(&c->QjHatVecModT_23_device, 8 * s_hat * (l + 1)));
    RD_CUDA(cudaMalloc(&c->Qjmodti_device, 8 * s_blk * (l + 1)));
    RD_CUDA(cudaMemcpy(c->QjHatInvVecModQj_23_device + s_inv * l, hat_inv, 8 * (size_t)blocks * p_num, cudaMemcpyHostToDevice));
    RD_CUDA(cudaMemcpy(c->QjHatInvVecModQj_23_shoup_device + s_inv * l, hat_inv_shoup, 8 * (size_t)blocks * p_num, cudaMemcpyHostToDevice));
    RD_CUDA(cudaMemcpy(c->QjHatVecModT_23_device + s_hat * l, hat_mod_t, 8 * (size_t)blocks * t_num * p_num, cudaMemcpyHostToDevice));
    RD_CUDA(cudaMemcpy(c->Qjmodti_device + s_blk * l, blk_mod_t, 8 * (size_t)blocks * t_num, cudaMemcpyHostToDevice));
    uint64_tt *din = nullptr, *dout = nullptr;
    size_t ib = 8 * (size_t)batch * q_num * N, ob = 8 * (size_t)batch * blocks * t_num * N;
    RD_CUDA(cudaMalloc(&din, ib));
    RD_CUDA(cudaMalloc(&dout, ob));
    RD_CUDA(cudaMemcpy(din, h_in, ib, cudaMemcpyHostToDevice));
    c->modUpQjtoT_23(dout, din, l, batch);
    RD_CUDA(cudaGetLastError());
    RD_CUDA(cudaDeviceSynchronize());
    RD_CUDA(cudaMemcpy(h_out, dout, ob, cudaMemcpyDeviceToHost));
    cudaFree(din); cudaFree(dout);
    cudaFree(c->QjHatInvVecModQj_23_device); cudaFree(c->QjHatInvVecModQj_23_shoup_device);
    cudaFree(c->QjHatVecModT_23_device); cudaFree(c->Qjmodti_device);
    free(c);
    return 0;
}

// pcmm_cuda_core_kernel<mat_N> with the grid/block of PCMM_Scheme::PPMM.
// h_X is [mat_N][limbs][C] contiguous, h_out [mat_M][limbs][C]; qinv[i] = q_last^-1 mod q_i.
extern "C" int ref_ppmm(const float* h_W, const unsigned long long* h_X, unsigned long long* h_out, int mat_M,
                        int mat_N, int N1, int mlwe_rank, int limbs, const unsigned long long* q, double scaler,
                        const unsigned long long* qinv, const unsigned long long* qinv_shoup) {
    if (limbs > 4 || mat_M % 32 || ((long)N1 * (mlwe_rank + 1)) % 32) return 1;
    std::vector<uint64_tt> mh(limbs), ml(limbs), qq(q, q + limbs);
    for (int i = 0; i < limbs; i++) {
        unsigned __int128 mu = (~(unsigned __int128)0) / q[i];
        mh[i] = (uint64_tt)(mu >> 64);
        ml[i] = (uint64_tt)mu;
    }
    RD_CUDA(cudaMemcpyToSymbol(ringpack_pq_cons, qq.data(), 8 * limbs));
    RD_CUDA(cudaMemcpyToSymbol(ringpack_pq_mu_high_cons, mh.data(), 8 * limbs));
    RD_CUDA(cudaMemcpyToSymbol(ringpack_pq_mu_low_cons, ml.data(), 8 * limbs));
    const size_t C = (size_t)N1 * (mlwe_rank + 1);
    float* dW = nullptr;
    uint64_tt *dX = nullptr, *dout = nullptr, *dinv = nullptr, *dinvs = nullptr;
    uint64_tt** dptr = nullptr;
    RD_CUDA(cudaMalloc(&dW, sizeof(float) * mat_M * mat_N));
    RD_CUDA(cudaMalloc(&dX, 8 * C * limbs * mat_N));
    RD_CUDA(cudaMalloc(&dout, 8 * C * limbs * mat_M));
    RD_CUDA(cudaMalloc(&dinv, 8 * limbs));
    RD_CUDA(cudaMalloc(&dinvs, 8 * limbs));
    RD_CUDA(cudaMalloc(&dptr, sizeof(uint64_tt*) * mat_N));
    std::vector<uint64_tt*> ptrs(mat_N);
    for (int n = 0; n < mat_N; n++) ptrs[n] = dX + C * limbs * n;
    RD_CUDA(cudaMemcpy(dW, h_W, sizeof(float) * mat_M * mat_N, cudaMemcpyHostToDevice));
    RD_CUDA(cudaMemcpy(dX, h_X, 8 * C * limbs * mat_N, cudaMemcpyHostToDevice));
    RD_CUDA(cudaMemcpy(dptr, ptrs.data(), sizeof(uint64_tt*) * mat_N, cudaMemcpyHostToDevice));
    RD_CUDA(cudaMemcpy(dinv, qinv, 8 * limbs, cudaMemcpyHostToDevice));
    RD_CUDA(cudaMemcpy(dinvs, qinv_shoup, 8 * limbs, cudaMemcpyHostToDevice));
    RD_CUDA(cudaMemset(dout, 0, 8 * C * limbs * mat_M));
    dim3 ppmm_block(mat_M / TILE_WIDTH_M, N1 * (mlwe_rank + 1) / TILE_WIDTH_K);
    dim3 ppmm_thread(32, (TILE_WIDTH_M * TILE_WIDTH_K) / (16 * 16));
    int SMem_size = (TILE_WIDTH_M * TILE_WIDTH_N * (sizeof(int64_tt)) + TILE_WIDTH_N * TILE_WIDTH_K * sizeof(uint64_tt)) * 2;
#define RD_LAUNCH(NN)                                                                                         \
    cudaFuncSetAttribute(&pcmm_cuda_core_kernel<NN>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMem_size); \
    pcmm_cuda_core_kernel<NN><<<ppmm_block, ppmm_thread, SMem_size>>>(dW, dptr, dout, N1, mlwe_rank, limbs, 0, scaler, dinv, dinvs)
    if (mat_N == 128) { RD_LAUNCH(128); }
    else if (mat_N == 256) { RD_LAUNCH(256); }
    else if (mat_N == 512) { RD_LAUNCH(512); }
    else if (mat_N == 768) { RD_LAUNCH(768); }
    else if (mat_N == 3072) { RD_LAUNCH(3072); }
    else return 2;
    RD_CUDA(cudaGetLastError());
    RD_CUDA(cudaDeviceSynchronize());
    RD_CUDA(cudaMemcpy(h_out, dout, 8 * C * limbs * mat_M, cudaMemcpyDeviceToHost));
    cudaFree(dW); cudaFree(dX); cudaFree(dout); cudaFree(dinv); cudaFree(dinvs); cudaFree(dptr);
    return 0;
}

// rlweCipherDecompose_kernel<mlwe_rank> with the launch shape of PCMM_Scheme::rlweCipherDecompose
// (src/ckks/include/pcmm/PCMM_Scheme.cuh:51-125), on coefficient-domain input.
// h_rlwe is [2][L+1][N]; h_mlwe receives mlwe_num ciphertexts of [l+1][(rank+1)*N1] back to back.
extern "C" int ref_decompose(const unsigned long long* h_rlwe, unsigned long long* h_mlwe, int logN, int N1,
                             int mlwe_rank, int mlwe_num, int L, int l, const unsigned long long* q) {
    if (mlwe_rank != 256 && mlwe_rank != 512) return 1;
    if (N1 % ringSwitch_block) return 2;
    const long N = 1L << logN;
    int rc = upload_pqt(q, L + 1);          // p_num = 0: modulus index = limb index
    if (rc) return rc;
    const size_t ct_words = (size_t)(l + 1) * (mlwe_rank + 1) * N1;
    uint64_tt *d_rlwe = nullptr, *d_mlwe = nullptr;
    uint64_tt** d_ptr = nullptr;
    RD_CUDA(cudaMalloc(&d_rlwe, 8 * 2 * (size_t)(L + 1) * N));
    RD_CUDA(cudaMalloc(&d_mlwe, 8 * ct_words * mlwe_num));
    RD_CUDA(cudaMalloc(&d_ptr, sizeof(uint64_tt*) * mlwe_num));
    RD_CUDA(cudaMemcpy(d_rlwe, h_rlwe, 8 * 2 * (size_t)(L + 1) * N, cudaMemcpyHostToDevice));
    RD_CUDA(cudaMemset(d_mlwe, 0xff, 8 * ct_words * mlwe_num));
    std::vector<uint64_tt*> ptrs(mlwe_num);
    for (int i = 0; i < mlwe_num; i++) ptrs[i] = d_mlwe + ct_words * i;
    RD_CUDA(cudaMemcpy(d_ptr, ptrs.data(), sizeof(uint64_tt*) * mlwe_num, cudaMemcpyHostToDevice));
    dim3 grid(N1 / ringSwitch_block, l + 1, mlwe_num);
    if (mlwe_rank == 256)
        rlweCipherDecompose_kernel<256><<<grid, ringSwitch_block>>>(d_rlwe, d_ptr, (int)N, N1, mlwe_num, l, L, 0);
    else
        rlweCipherDecompose_kernel<512><<<grid, ringSwitch_block>>>(d_rlwe, d_ptr, (int)N, N1, mlwe_num, l, L, 0);
    RD_CUDA(cudaGetLastError());
    RD_CUDA(cudaDeviceSynchronize());
    RD_CUDA(cudaMemcpy(h_mlwe, d_mlwe, 8 * ct_words * mlwe_num, cudaMemcpyDeviceToHost));
    cudaFree(d_rlwe); cudaFree(d_mlwe); cudaFree(d_ptr);
    return 0;
}

// The three kernels of PCMM_Scheme::mlweCipherPacking (src/ckks/include/pcmm/PCMM_Scheme.cuh:261-359),
// each on its own so that every stage of the oracle can be pinned.  Ring-pack moduli [p | q0, q1].
static int upload_ringpack(unsigned long long p, unsigned long long q0) {
    uint64_tt m[2] = {p, q0}, mh[2], ml[2];
    for (int i = 0; i < 2; i++) {
        unsigned __int128 mu = (~(unsigned __int128)0) / m[i];
        mh[i] = (uint64_tt)(mu >> 64);
        ml[i] = (uint64_tt)mu;
    }
    RD_CUDA(cudaMemcpyToSymbol(ringpack_pq_cons, m, 16));
    RD_CUDA(cudaMemcpyToSymbol(ringpack_pq_mu_high_cons, mh, 16));
    RD_CUDA(cudaMemcpyToSymbol(ringpack_pq_mu_low_cons, ml, 16));
    return 0;
}

// h_mlwe: mlwe_num ciphertexts, limb 0 only, [(rank+1)*N1] each; h_E: (rank+1) polynomials of [2][N].
extern "C" int ref_pack_embed(const unsigned long long* h_mlwe, unsigned long long* h_E, int logN, int N1, int mlwe_rank,
                              int mlwe_num, unsigned long long p, unsigned long long q0) {
    if (N1 % ringSwitch_block) return 2;
    const long N = 1L << logN;
    int rc = upload_ringpack(p, q0);
    if (rc) return rc;
    const size_t ct = (size_t)(mlwe_rank + 1) * N1, eb = 8 * (size_t)(mlwe_rank + 1) * 2 * N;
    uint64_tt *d_mlwe = nullptr, *d_E = nullptr;
    uint64_tt** d_ptr = nullptr;
    RD_CUDA(cudaMalloc(&d_mlwe, 8 * ct * mlwe_num));
    RD_CUDA(cudaMalloc(&d_E, eb));
    RD_CUDA(cudaMalloc(&d_ptr, sizeof(uint64_tt*) * mlwe_num));
    RD_CUDA(cudaMemcpy(d_mlwe, h_mlwe, 8 * ct * mlwe_num, cudaMemcpyHostToDevice));
    std::vector<uint64_tt*> ptrs(mlwe_num);
    for (int i = 0; i < mlwe_num; i++) ptrs[i] = d_mlwe + ct * i;
    RD_CUDA(cudaMemcpy(d_ptr, ptrs.data(), sizeof(uint64_tt*) * mlwe_num, cudaMemcpyHostToDevice));
    RD_CUDA(cudaMemset(d_E, 0, eb));                                                   // :397
    dim3 grid(N1 / ringSwitch_block, 1, mlwe_num);
    mlweCipherEmbedding_new_kernel<<<grid, ringSwitch_block>>>(d_E, d_ptr, N1, (int)N, mlwe_rank, mlwe_num, 1, 2);
    RD_CUDA(cudaGetLastError());
    RD_CUDA(cudaDeviceSynchronize());
    RD_CUDA(cudaMemcpy(h_E, d_E, eb, cudaMemcpyDeviceToHost));
    cudaFree(d_mlwe); cudaFree(d_E); cudaFree(d_ptr);
    return 0;
}

// h_E: rank polynomials of [2][N] in the NTT domain; h_keys [rank][2][2][N]; h_O [2][2][N].
extern "C" int ref_pack_keymac(const unsigned long long* h_E, const unsigned long long* h_keys, unsigned long long* h_O,
                               int logN, int N1, int mlwe_rank, unsigned long long p, unsigned long long q0) {
    if (mlwe_rank != 256 && mlwe_rank != 512) return 1;
    const long N = 1L << logN;
    int rc = upload_ringpack(p, q0);
    if (rc) return rc;
    uint64_tt *d_E = nullptr, *d_K = nullptr, *d_O = nullptr;
    RD_CUDA(cudaMalloc(&d_E, 8 * (size_t)mlwe_rank * 2 * N));
    RD_CUDA(cudaMalloc(&d_K, 8 * (size_t)mlwe_rank * 4 * N));
    RD_CUDA(cudaMalloc(&d_O, 8 * 4 * N));
    RD_CUDA(cudaMemcpy(d_E, h_E, 8 * (size_t)mlwe_rank * 2 * N, cudaMemcpyHostToDevice));
    RD_CUDA(cudaMemcpy(d_K, h_keys, 8 * (size_t)mlwe_rank * 4 * N, cudaMemcpyHostToDevice));
    dim3 grid(N / ringSwitch_block, 2);
    if (mlwe_rank == 256) mlweCipherMultRepackingKey_kernel<256><<<grid, ringSwitch_block>>>(d_O, d_E, d_K, N1, (int)N, 2);
    else mlweCipherMultRepackingKey_kernel<512><<<grid, ringSwitch_block>>>(d_O, d_E, d_K, N1, (int)N, 2);
    RD_CUDA(cudaGetLastError());
    RD_CUDA(cudaDeviceSynchronize());
    RD_CUDA(cudaMemcpy(h_O, d_O, 8 * 4 * N, cudaMemcpyDeviceToHost));
    cudaFree(d_E); cudaFree(d_K); cudaFree(d_O);
    return 0;
}

// h_O [2][2][N] coefficient domain -> h_out [2][N] (a, b) mod q0.
extern "C" int ref_pack_moddown(const unsigned long long* h_O, unsigned long long* h_out, int logN, unsigned long long p,
                                unsigned long long q0) {
    const long N = 1L << logN;
    int rc = upload_ringpack(p, q0);
    if (rc) return rc;
    uint64_tt pinv = modinv128(p, q0), pinv_s = x_Shoup(pinv, q0);
    uint64_tt *d_O = nullptr, *d_out = nullptr, *d_pinv = nullptr, *d_pinvs = nullptr;
    RD_CUDA(cudaMalloc(&d_O, 8 * 4 * N));
    RD_CUDA(cudaMalloc(&d_out, 8 * 2 * N));
    RD_CUDA(cudaMalloc(&d_pinv, 8));
    RD_CUDA(cudaMalloc(&d_pinvs, 8));
    RD_CUDA(cudaMemcpy(d_O, h_O, 8 * 4 * N, cudaMemcpyHostToDevice));
    RD_CUDA(cudaMemcpy(d_pinv, &pinv, 8, cudaMemcpyHostToDevice));
    RD_CUDA(cudaMemcpy(d_pinvs, &pinv_s, 8, cudaMemcpyHostToDevice));
    dim3 grid(N / ringSwitch_block, 1, 2);
    ringpacking_ModDown_kernel<<<grid, ringSwitch_block>>>(d_out, d_O, (int)N, 1, 2, 1, d_pinv, d_pinvs);
    RD_CUDA(cudaGetLastError());
    RD_CUDA(cudaDeviceSynchronize());
    RD_CUDA(cudaMemcpy(h_out, d_out, 8 * 2 * N, cudaMemcpyDeviceToHost));
    cudaFree(d_O); cudaFree(d_out); cudaFree(d_pinv); cudaFree(d_pinvs);
    return 0;
}

// The elementwise kernels of Scheme_23::rescaleAndEqual (Scheme_23.cuh:339-385) on a cipher buffer
// [2][q_stride][N]: stage 0 = mod_to_qi (h_cipher -> h_buf), stage 1 = rescaleAndEqual_new_kernel
// (h_cipher, h_buf -> h_cipher).  The transforms between them are ref_ntt's.  pqt = [p | q].
extern "C" int ref_rescale_stage(unsigned long long* h_cipher, unsigned long long* h_buf, int logN,
                                 const unsigned long long* pqt, int p_num, int q_stride, int l, int stage,
                                 const unsigned long long* qinv, const unsigned long long* qinv_shoup) {
    const int n_mod = p_num + q_stride;
    if (n_mod > max_pqt_num || l < 1) return 1;
    const long N = 1L << logN;
    int rc = upload_pqt(pqt, n_mod);
    if (rc) return rc;
    const size_t bytes = 8 * (size_t)2 * q_stride * N;
    uint64_tt *dc = nullptr, *db = nullptr, *dq = nullptr, *dqs = nullptr;
    RD_CUDA(cudaMalloc(&dc, bytes));
    RD_CUDA(cudaMalloc(&db, bytes));
    RD_CUDA(cudaMalloc(&dq, 8 * l));
    RD_CUDA(cudaMalloc(&dqs, 8 * l));
    RD_CUDA(cudaMemcpy(dc, h_cipher, bytes, cudaMemcpyHostToDevice));
    RD_CUDA(cudaMemcpy(db, h_buf, bytes, cudaMemcpyHostToDevice));
    RD_CUDA(cudaMemcpy(dq, qinv, 8 * l, cudaMemcpyHostToDevice));
    RD_CUDA(cudaMemcpy(dqs, qinv_shoup, 8 * l, cudaMemcpyHostToDevice));
    dim3 resc_dim(N / rescale_block, l, 2);
    if (stage == 0) mod_to_qi<<<resc_dim, rescale_block>>>(db, dc, N, p_num, q_stride, l);
    else rescaleAndEqual_new_kernel<<<resc_dim, rescale_block>>>(dc, db, N, p_num, q_stride, l, dq, dqs);
    RD_CUDA(cudaGetLastError());
    RD_CUDA(cudaDeviceSynchronize());
    RD_CUDA(cudaMemcpy(h_cipher, dc, bytes, cudaMemcpyDeviceToHost));
    RD_CUDA(cudaMemcpy(h_buf, db, bytes, cudaMemcpyDeviceToHost));
    cudaFree(dc); cudaFree(db); cudaFree(dq); cudaFree(dqs);
    return 0;
}

// modUpQ0toQL_kernel (bootstrapping/Bootstrapping.cuh:6-23) on a cipher buffer [2][q_stride][N]
// whose limb 0 holds coefficients; fills limbs 1..target_level.
extern "C" int ref_modup_q0_to_ql(unsigned long long* h_cipher, int logN, const unsigned long long* pqt, int p_num,
                                  int q_stride, int target_level, int scale_up) {
    const int n_mod = p_num + q_stride;
    if (n_mod > max_pqt_num || target_level < 1 || target_level >= q_stride) return 1;
    const long N = 1L << logN;
    if (N < modUpQ0toQL_block) return 1;
    int rc = upload_pqt(pqt, n_mod);
    if (rc) return rc;
    const size_t bytes = 8 * (size_t)2 * q_stride * N;
    uint64_tt* dc = nullptr;
    RD_CUDA(cudaMalloc(&dc, bytes));
    RD_CUDA(cudaMemcpy(dc, h_cipher, bytes, cudaMemcpyHostToDevice));
    dim3 dim(N / modUpQ0toQL_block, target_level, 2);
    modUpQ0toQL_kernel<<<dim, modUpQ0toQL_block>>>(dc, N, p_num, q_stride, scale_up);
    RD_CUDA(cudaGetLastError());
    RD_CUDA(cudaDeviceSynchronize());
    RD_CUDA(cudaMemcpy(h_cipher, dc, bytes, cudaMemcpyDeviceToHost));
    cudaFree(dc);
    return 0;
}

// The three kernels of the key-switch chain through the reference's own launchers
// (Context_23::external_product_T, modUpTtoPQl_23, modDownPQltoQl_23) on a zero-initialised context
// whose integer members and table pointers are filled here.  pqt = [p | q | t]; tables come from the
// caller in the reference's layouts.  stage 0: external product (h_in = digits over T, h_aux = key);
// stage 1: T -> [p | q]; stage 2: ModDown.  Buffers are [2][R*t_num][N] except the ModDown output [2][q_num][N].
extern "C" int ref_keyswitch_stage(unsigned long long* h_out, const unsigned long long* h_in, const unsigned long long* h_aux,
                                   int logN, const unsigned long long* pqt, int p_num, int q_num, int t_num, int l, int gamma,
                                   int stage, const unsigned long long* t_hat_inv, const unsigned long long* t_hat_inv_shoup,
                                   const unsigned long long* t_hat_mod_r, const unsigned long long* half_t,
                                   const unsigned long long* t_mod_pq, const unsigned long long* p_hat_inv,
                                   const unsigned long long* p_hat_inv_shoup, const unsigned long long* p_hat_mod_q,
                                   const unsigned long long* p_inv_mod_q, const unsigned long long* p_inv_mod_q_shoup) {
    const int n_mod = p_num + q_num + t_num;
    if (n_mod > max_pqt_num || p_num > max_p_num || t_num > max_tnum) return 1;
    const long N = 1L << logN;
    int rc = upload_pqt(pqt, n_mod);
    if (rc) return rc;
    RD_CUDA(cudaMemcpyToSymbol(halfTmodpqti_cons, half_t, 8 * n_mod));
    RD_CUDA(cudaMemcpyToSymbol(Tmodpqi_cons, t_mod_pq, 8 * (p_num + q_num)));
    RD_CUDA(cudaMemcpyToSymbol(Pinvmodqi_cons, p_inv_mod_q, 8 * q_num));
    RD_CUDA(cudaMemcpyToSymbol(Pinvmodqi_shoup_cons, p_inv_mod_q_shoup, 8 * q_num));
    RD_CUDA(cudaMemcpyToSymbol(pHatInvVecModp_cons, p_hat_inv, 8 * p_num));
    RD_CUDA(cudaMemcpyToSymbol(pHatInvVecModp_shoup_cons, p_hat_inv_shoup, 8 * p_num));
    Context_23* c = fake_context();
    c->N = N;
    c->logN = logN;
    c->p_num = p_num; c->q_num = q_num; c->t_num = t_num;
    c->K = p_num; c->L = q_num - 1;
    c->gamma = gamma;
    c->dnum = q_num / p_num;
    c->Ri_blockNum = (p_num + q_num + gamma - 1) / gamma;
    const int R = c->Ri_blockNum;
    if (R > max_Riblock_num) { free(c); return 1; }
    const size_t tb = (size_t)2 * R * t_num * N;
    RD_CUDA(cudaMalloc(&c->THatInvVecModti_23_device, 8 * t_num));
    RD_CUDA(cudaMalloc(&c->THatInvVecModti_23_shoup_device, 8 * t_num));
    RD_CUDA(cudaMalloc(&c->THatVecModRi_23_device, 8 * (size_t)(p_num + q_num) * t_num));
    RD_CUDA(cudaMalloc(&c->pHatVecModq_23_device, 8 * (size_t)q_num * p_num));
    RD_CUDA(cudaMemcpy(c->THatInvVecModti_23_device, t_hat_inv, 8 * t_num, cudaMemcpyHostToDevice));
    RD_CUDA(cudaMemcpy(c->THatInvVecModti_23_shoup_device, t_hat_inv_shoup, 8 * t_num, cudaMemcpyHostToDevice));
    RD_CUDA(cudaMemcpy(c->THatVecModRi_23_device, t_hat_mod_r, 8 * (size_t)(p_num + q_num) * t_num, cudaMemcpyHostToDevice));
    RD_CUDA(cudaMemcpy(c->pHatVecModq_23_device, p_hat_mod_q, 8 * (size_t)q_num * p_num, cudaMemcpyHostToDevice));
    uint64_tt *din = nullptr, *daux = nullptr, *dout = nullptr;
    const int cipher_blocks = (l + 1 + p_num - 1) / p_num;
    const size_t in_words = stage == 0 ? (size_t)cipher_blocks * t_num * N : tb;
    const size_t aux_words = stage == 0 ? (size_t)2 * c->dnum * R * t_num * N : 1;
    const size_t out_words = stage == 2 ? (size_t)2 * q_num * N : tb;
    RD_CUDA(cudaMalloc(&din, 8 * in_words));
    RD_CUDA(cudaMalloc(&daux, 8 * aux_words));
    RD_CUDA(cudaMalloc(&dout, 8 * out_words));
    RD_CUDA(cudaMemcpy(din, h_in, 8 * in_words, cudaMemcpyHostToDevice));
    if (stage == 0) RD_CUDA(cudaMemcpy(daux, h_aux, 8 * aux_words, cudaMemcpyHostToDevice));
    RD_CUDA(cudaMemcpy(dout, h_out, 8 * out_words, cudaMemcpyHostToDevice));
    if (stage == 0) c->external_product_T(dout, din, daux, l);
    else if (stage == 1) c->modUpTtoPQl_23(dout, din, l, 2);
    else c->modDownPQltoQl_23(dout, din, l, 2);
    RD_CUDA(cudaGetLastError());
    RD_CUDA(cudaDeviceSynchronize());
    RD_CUDA(cudaMemcpy(h_out, dout, 8 * out_words, cudaMemcpyDeviceToHost));
    cudaFree(din); cudaFree(daux); cudaFree(dout);
    cudaFree(c->THatInvVecModti_23_device); cudaFree(c->THatInvVecModti_23_shoup_device);
    cudaFree(c->THatVecModRi_23_device); cudaFree(c->pHatVecModq_23_device);
    free(c);
    return 0;
}

// compute_c0c1c2 and cipher_add_axbx_batch_device (poly_arithmetic.cuh:787-824, :155-172, :416-420) as
// Scheme_23::mult_23 calls them, on Ciphertext buffers [2][q_num][N]; pq = [p | q].  mode 0: h_out = the three
// products [3][q_num][N] (a1b2+a2b1, a1a2, b1b2) of h_c1 and h_c2; mode 1: h_c1 += (h_c2 viewed as [ax | bx]).
extern "C" int ref_tensor_product(unsigned long long* h_out, unsigned long long* h_c1, const unsigned long long* h_c2,
                                  int logN, const unsigned long long* pq, int p_num, int q_num, int l, int mode) {
    const int n_mod = p_num + q_num;
    if (n_mod > max_pqt_num) return 1;
    const long N = 1L << logN;
    int rc = upload_pqt(pq, n_mod);
    if (rc) return rc;
    const size_t half = (size_t)q_num * N, bytes = 8 * 2 * half;
    uint64_tt *d1 = nullptr, *d2 = nullptr, *d3 = nullptr;
    RD_CUDA(cudaMalloc(&d1, bytes));
    RD_CUDA(cudaMalloc(&d2, bytes));
    RD_CUDA(cudaMalloc(&d3, 8 * 3 * half));
    RD_CUDA(cudaMemcpy(d1, h_c1, bytes, cudaMemcpyHostToDevice));
    RD_CUDA(cudaMemcpy(d2, h_c2, bytes, cudaMemcpyHostToDevice));
    RD_CUDA(cudaMemset(d3, 0, 8 * 3 * half));
    if (mode == 0) {
        compute_c0c1c2(d3, d3 + half, d3 + 2 * half, d1, d2, d1 + half, d2 + half, N, 0, p_num, l + 1);
    } else {
        cipher_add_axbx_batch_device(d1, d2, d2 + half, N, p_num, l + 1, q_num);
    }
    RD_CUDA(cudaGetLastError());
    RD_CUDA(cudaDeviceSynchronize());
    if (mode == 0) RD_CUDA(cudaMemcpy(h_out, d3, 8 * 3 * half, cudaMemcpyDeviceToHost));
    else RD_CUDA(cudaMemcpy(h_c1, d1, bytes, cudaMemcpyDeviceToHost));
    cudaFree(d1); cudaFree(d2); cudaFree(d3);
    return 0;
}

// The three small steps Scheme_23::conjugate_23 and leftRotate_23 add around the key-switch chain
// (KeySwitch_23.cuh:452-453, :469, :577-580), on Ciphertext buffers [2][q_num][N]; pq = [p | q].
//   mode 0: sk_and_poly_conjugate on limbs 0..l of both halves of h_in -> h_out          (poly_arithmetic.cuh:666-680)
//   mode 1: sk_and_poly_LeftRot_ntt_double of h_in by rot_slots -> h_out, with rotGroups built as
//           Context_23.cuh:650-656 builds them                                            (poly_arithmetic.cuh:581-603)
//   mode 2: poly_add_batch_device: b half of h_out (preloaded) += b half of h_in        (poly_arithmetic.cuh:111-121, :395-399)
extern "C" int ref_galois(unsigned long long* h_out, const unsigned long long* h_in, int logN,
                          const unsigned long long* pq, int p_num, int q_num, int l, long rot_slots, int mode) {
    const int n_mod = p_num + q_num;
    if (n_mod > max_pqt_num) return 1;
    const long N = 1L << logN, Nh = N / 2, M = 2 * N;
    int rc = upload_pqt(pq, n_mod);
    if (rc) return rc;
    const size_t half = (size_t)q_num * N, bytes = 8 * 2 * half;
    uint64_tt *din = nullptr, *dout = nullptr, *drot = nullptr;
    RD_CUDA(cudaMalloc(&din, bytes));
    RD_CUDA(cudaMalloc(&dout, bytes));
    RD_CUDA(cudaMemcpy(din, h_in, bytes, cudaMemcpyHostToDevice));
    RD_CUDA(cudaMemcpy(dout, h_out, bytes, cudaMemcpyHostToDevice));
    if (mode == 0) {
        sk_and_poly_conjugate(dout, din, N, q_num, 0, 0, l + 1);
        sk_and_poly_conjugate(dout + half, din + half, N, q_num, 0, 0, l + 1);
    } else if (mode == 1) {
        std::vector<uint64_tt> rot(Nh);
        long five = 1;
        for (long i = 0; i < Nh; ++i) { rot[i] = five; five = five * 5 % M; }
        RD_CUDA(cudaMalloc(&drot, 8 * Nh));
        RD_CUDA(cudaMemcpy(drot, rot.data(), 8 * Nh, cudaMemcpyHostToDevice));
        sk_and_poly_LeftRot_ntt_double(dout, din, drot, N, p_num, q_num, rot_slots, 0, 0, l + 1);
    } else {
        poly_add_batch_device(dout + half, din + half, N, 0, 0, p_num, l + 1);
    }
    RD_CUDA(cudaGetLastError());
    RD_CUDA(cudaDeviceSynchronize());
    RD_CUDA(cudaMemcpy(h_out, dout, bytes, cudaMemcpyDeviceToHost));
    cudaFree(din); cudaFree(dout);
    if (drot) cudaFree(drot);
    return 0;
}
