// Context handle: moduli, NTT twiddle tables and ModUp tables resident in HBM.
#pragma once
#include <map>
#include <vector>

#include "common.cuh"

// Tables of the tensor-core T -> [p | q] conversion for one gamma (modup_umma.cu), all on the device:
// per block of gamma targets the source columns (the t moduli, the same for every block), the targets and
// the byte planes of ((T/t_j) * 2^(8b)) mod r.
struct TpqTables {
    bool ok = false;              // every target in [2^40, 2^62), the reference's 128-bit difference cannot wrap
    int kpad = 0, npad = 0;
    u64* src_mod = nullptr;       // [R][apad]
    ulonglong2* src_hinv = nullptr;
    u64* src_pre = nullptr;       // floor(T/2) mod t_j
    u64* tgt_mod = nullptr;       // [R][gamma]
    u64* tgt_f = nullptr;         // T mod r
    u64* tgt_post = nullptr;      // floor(T/2) mod r
    uint8_t* planes = nullptr;    // [R][kpad/32][npad][32]
};

struct ckks_b200_context {
    int device = 0;
    int logN = 0;
    uint32_t N = 0;
    int p_num = 0, q_num = 0, t_num = 0, mod_num = 0;
    int alpha = 0;          // limbs per digit (= p_num)
    int blocks_max = 0;     // ceil(q_num / alpha)

    std::vector<u64> moduli;                 // [p | q | t]
    std::vector<u64> psi;                    // 2N-th root per modulus
    std::vector<std::vector<u64>> h_psi_tab, h_psiinv_tab;   // kept for ckks_b200_context_table

    // Device tables.  Twiddles are interleaved {w, floor(w*2^64/q)} pairs so one
    // 128-bit load fetches both: tw_fwd/tw_inv are [mod_num][N] ulonglong2.
    ulonglong2* tw_fwd = nullptr;
    ulonglong2* tw_inv = nullptr;
    double* tw_fwd_d = nullptr;              // [mod_num][N] the same twiddles as centred doubles (FP64 back end)
    double* tw_inv_d = nullptr;
    u64* d_moduli = nullptr;                 // [mod_num]
    ulonglong2* d_ninv = nullptr;            // [mod_num] {N^-1, shoup}
    u64* d_qinv64 = nullptr;                 // [mod_num] floor(2^64 / q)
    ulonglong2* d_qlinv = nullptr;           // [q_num][q_num] row l, entry i < l: {q_l^-1 mod q_i, shoup} (rescale)

    // ModUp tables, one group per level l in [0, q_num):
    //   hat_inv   [l][blocks_max*alpha]           {inv, shoup} of (Qblk/q_j)^-1 mod q_j
    //   hat_mod_t [l][blocks_max][t_num][alpha]   (Qblk/q_j) mod t_k
    //   blk_mod_t [l][blocks_max][t_num]          Qblk mod t_k
    ulonglong2* mu_hat_inv = nullptr;
    u64* mu_hat_mod_t = nullptr;
    u64* mu_blk_mod_t = nullptr;
    ulonglong2* d_t_mu = nullptr;            // [t_num] Barrett mu {hi, lo}

    // Tensor-core ModUp (modup_umma.cu).  The contraction runs over the bytes of the rb_j:
    // K index j*8+b stands for byte b of rb_j, and the constant it meets is
    // ((Qblk/q_j) * 2^(8b)) mod t_k, itself cut into eight bytes (row k*8+a = byte a for target k).
    //   mu_planes [l][blocks_max][tc_kpad/32][tc_npad rows][32 bytes]  in MMA core-matrix order
    //   mu_tc_ok  [l]  1 when level l may take the tensor-core kernel
    //   d_t_inv   [t_num] 1.0 / t_k
    uint8_t* mu_planes = nullptr;
    std::vector<uint8_t> mu_tc_ok;
    double* d_t_inv = nullptr;
    int tc_kpad = 0, tc_npad = 0;
    // the same conversion's per-block tables in the generic form the kernel reads:
    u64* mu_src_mod = nullptr;               // [l][blocks_max][tc_kpad/8]  q_j of the digit (1 beyond it)
    ulonglong2* mu_src_hinv = nullptr;       // [l][blocks_max][tc_kpad/8]
    u64* mu_src_pre = nullptr;               // zeros (nothing is pre-added or post-subtracted in this conversion)
    u64* mu_tgt_mod = nullptr;               // [blocks_max][t_num]  the t moduli for every block
    std::map<int, TpqTables> tpq;            // tables of the T -> [p | q] conversion, by gamma, built on first use
    int modup_algo = 0;                      // CKKS_B200_MODUP_AUTO / _TENSOR / _SIMT
    int* d_flags = nullptr;                  // [16] [1] = site of a device-side wait that ran out
    long long wait_budget = 0;               // clock cycles a device-side wait may take (0: the library's default)
    int exact_count = 0;                     // test switch of ckks_b200_context_test_exact_count
    int withhold_commit = 0;                 // test switch of ckks_b200_context_test_withhold_commit, consumed by one launch
    int* h_flags = nullptr;                  // pinned mirror

    // Key-switch chain (keyswitch.cu), the reference's tables of Context_23.cuh:60-192 and :286-351:
    ulonglong2* d_pq_mu = nullptr;           // [p_num+q_num] Barrett mu {hi, lo} of [p | q]
    ulonglong2* d_t_hat_inv = nullptr;       // [t_num] {(T/t_i)^-1 mod t_i, shoup}
    u64* d_t_hat_mod_r = nullptr;            // [p_num+q_num][t_num] (T/t_i) mod r, r over [p | q]
    u64* d_half_t = nullptr;                 // [mod_num] floor(T/2) mod each of [p | q | t]
    u64* d_t_mod_pq = nullptr;               // [p_num+q_num] T mod r
    ulonglong2* d_p_hat_inv = nullptr;       // [p_num] {(P/p_j)^-1 mod p_j, shoup}
    u64* d_p_hat_mod_q = nullptr;            // [q_num][p_num] (P/p_j) mod q_i
    ulonglong2* d_p_inv_mod_q = nullptr;     // [q_num] {P^-1 mod q_i, shoup}
    bool chain_ok = false;                   // every modulus below 2^62 (the tables above are built only then)
    u64* ks_buf = nullptr;                   // workspace of ckks_b200_keyswitch
    size_t ks_cap = 0;
    u64* mul_buf = nullptr;                  // the three products and the switched pair of ckks_b200_mult
    size_t mul_cap = 0;

    // Scratch for the *_host entry points, grown on demand.
    u64* h2d_buf = nullptr;
    size_t h2d_cap = 0;
    u64* h2d_buf2 = nullptr;
    size_t h2d_cap2 = 0;
    u64* ptr_buf = nullptr;                  // device copy of a caller's pointer table
    size_t ptr_cap = 0;
    u64* pack_buf = nullptr;                 // embedded MLWE polynomials and key products of the packing
    size_t pack_cap = 0;
    u64* resc_buf = nullptr;                 // the last limb spread over the lower limbs (rescale)
    size_t resc_cap = 0;
};

namespace ckb {
// Smallest r >= 2 with r^((q-1)/f) != 1 for every f in the factor set the reference
// derives for q-1, raised to (q-1)/M: the same root the reference would pick.
u64 find_mth_root(u64 M, u64 q);
void fill_psi_tables(u64 psi, u64 q, uint32_t n, std::vector<u64>& tab, std::vector<u64>& tabinv);
int ensure_buf(u64** buf, size_t* cap, size_t words);
// Builds (once per gamma) the tables of the tensor-core T -> [p | q] conversion.
int build_tpq_tables(ckks_b200_context* c, int gamma);
bool modup_t_tensor_ok(const ckks_b200_context* c, int gamma);
int modup_t_tensor(ckks_b200_context* c, u64* d_out, const u64* d_in, int l, int gamma, int batch, cudaStream_t st);
// Tensor-core ModUp (modup_umma.cu): whether level l qualifies, and the launch.
bool modup_tensor_ok(const ckks_b200_context* c, int l);
int modup_tensor(ckks_b200_context* c, u64* d_out, const u64* d_in, int l, int batch, cudaStream_t st);
}  // namespace ckb
