/*
 * ckks_b200.h -- C ABI of the B200-native CKKS hot path: batched negacyclic RNS
 * NTT/INTT, Q-digit -> T basis conversion (ModUp) and the ring-packed
 * plaintext x ciphertext matrix multiply (PPMM/PCMM).
 *
 * The reference (haozetao/ckks_llm) is a header-only CUDA/C++ unity build with no
 * C interface; each entry point below names the reference C++ member it stands in
 * for (file:line relative to the reference root).  All functions return 0 on
 * success or a CKKS_B200_ERR_* code, never throw and never print; a description of
 * the last failure on the calling thread is available from ckks_b200_last_error().
 * Pointers named d_* are device pointers on the handle's device, h_* are host
 * pointers.  `stream` is a cudaStream_t passed as void* (NULL = default stream).
 * No entry point falls back to a CPU implementation: without a CUDA device every
 * compute call fails with CKKS_B200_ERR_CUDA.
 */
#ifndef CKKS_B200_H
#define CKKS_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CKKS_B200_OK 0
#define CKKS_B200_ERR_ARG 1         /* null pointer, negative count, bad index */
#define CKKS_B200_ERR_SHAPE 2       /* shape rule of the reference violated */
#define CKKS_B200_ERR_UNSUPPORTED 3 /* size outside what the kernels were built for */
#define CKKS_B200_ERR_CUDA 4        /* a CUDA runtime call failed */
#define CKKS_B200_ERR_NOMEM 5       /* device or host allocation failed */
#define CKKS_B200_ERR_RANGE 6       /* scaled weight does not fit the byte planes */
#define CKKS_B200_ERR_TIMEOUT 7     /* a bounded device-side wait ran out */

typedef struct ckks_b200_context ckks_b200_context;
typedef struct ckks_b200_pcmm ckks_b200_pcmm;

int ckks_b200_version(void);
const char* ckks_b200_status_string(int status);
const char* ckks_b200_last_error(void);

/* ---- context ---------------------------------------------------------------
 * Tables the path needs from Context_23: moduli in the order [p | q | t]
 * (src/ckks/include/Context_23.cuh:56-113), 2N-th roots and psi / psi^-1 power
 * tables with Shoup companions (Utils.cuh:99-109,190-210; upload
 * Context_23.cuh:481-521), N^-1 (Context_23.cuh:140-157) and the Q-digit -> T
 * conversion tables for every level (Context_23.cuh:286-351).  alpha (limbs per
 * digit) equals p_num as in the reference (Context_23.cuh:31-32).
 * logN in [12,16]; every modulus is an odd prime = 1 mod 2N below 2^62. */
int ckks_b200_context_create(ckks_b200_context** out, int device, int logN,
                             const uint64_t* p, int p_num,
                             const uint64_t* q, int q_num,
                             const uint64_t* t, int t_num);
int ckks_b200_context_destroy(ckks_b200_context* ctx);
/* 2N-th root of unity chosen for modulus index mod_idx (index into [p|q|t]). */
int ckks_b200_context_psi(const ckks_b200_context* ctx, int mod_idx, uint64_t* psi);
/* Copy of the psi (inverse=0) or psi^-1 (inverse=1) table of one modulus, N words,
 * bit-reversed exponent order, n^-1 folded into psiinv[1] (Utils.cuh:190-201). */
int ckks_b200_context_table(const ckks_b200_context* ctx, int mod_idx, int inverse,
                            uint64_t* h_table);

/* ---- NTT / INTT ------------------------------------------------------------
 * Context_23::ToNTTInplace / FromNTTInplace (Context_23.cuh:847-889): in place on
 * [poly_num][poly_mod_len][N] words; limb i of the call (i < mod_num) lives at limb
 * offset start_limb_off+i and uses modulus index start_mod_idx+i.  Forward takes
 * natural order to bit-reversed order, inverse the opposite and includes N^-1;
 * outputs are canonical residues in [0,q). */
int ckks_b200_ntt_forward(ckks_b200_context* ctx, uint64_t* d_data, int start_limb_off,
                          int start_mod_idx, int poly_num, int mod_num, int poly_mod_len,
                          void* stream);
int ckks_b200_ntt_inverse(ckks_b200_context* ctx, uint64_t* d_data, int start_limb_off,
                          int start_mod_idx, int poly_num, int mod_num, int poly_mod_len,
                          void* stream);
/* Same transforms on a host buffer: copy in, transform, copy out, synchronise. */
int ckks_b200_ntt_forward_host(ckks_b200_context* ctx, uint64_t* h_data, int start_limb_off,
                               int start_mod_idx, int poly_num, int mod_num, int poly_mod_len);
int ckks_b200_ntt_inverse_host(ckks_b200_context* ctx, uint64_t* h_data, int start_limb_off,
                               int start_mod_idx, int poly_num, int mod_num, int poly_mod_len);

/* ---- ModUp -----------------------------------------------------------------
 * Context_23::modUpQjtoT_23 (BasisConv.cuh:84-179): for level l, every digit of
 * alpha consecutive Q-limbs of in[batch][q_num][N] (coefficient domain) is extended
 * to the t_num limbs of T: out[batch][ceil((l+1)/alpha)][t_num][N]. */
int ckks_b200_modup_qj_to_t(ckks_b200_context* ctx, uint64_t* d_out, const uint64_t* d_in,
                            int l, int batch, void* stream);
int ckks_b200_modup_qj_to_t_host(ckks_b200_context* ctx, uint64_t* h_out, const uint64_t* h_in,
                                 int l, int batch);
/* Kernel choice for ModUp on this context (no counterpart in the reference, which has one
 * kernel).  AUTO takes the tensor-core kernel (the alpha x t_num table product as an 8-bit
 * tcgen05 matrix product) on every level whose tables qualify and the 64-bit CUDA-core kernel
 * elsewhere; TENSOR insists and returns CKKS_B200_ERR_UNSUPPORTED on a level that does not
 * qualify; SIMT always takes the CUDA-core kernel.  Both give the reference's residues. */
#define CKKS_B200_MODUP_AUTO 0
#define CKKS_B200_MODUP_TENSOR 1
#define CKKS_B200_MODUP_SIMT 2
int ckks_b200_modup_set_algo(ckks_b200_context* ctx, int algo);
/* Synchronises `stream` and returns CKKS_B200_ERR_TIMEOUT when a bounded device-side wait
 * of a tensor-core ModUp on this context ran out since the last check (the *_host entry
 * point checks by itself). */
int ckks_b200_context_check(ckks_b200_context* ctx, void* stream);
/* Clock cycles a device-side wait of the tensor-core ModUp may take before it gives up (0 = the library's default,
 * about two seconds).  No reference counterpart: the reference has no bounded waits. */
int ckks_b200_context_set_wait_budget(ckks_b200_context* ctx, long long cycles);
/* Test support for the time-out path (no reference counterpart).  With on != 0 the next tensor-core ModUp on this
 * context leaves out the completion signal of one tile, so the threads that wait for it run into the wait budget:
 * they raise the flag and leave, the kernel frees its tensor memory and returns normally, and the next
 * ckks_b200_context_check returns CKKS_B200_ERR_TIMEOUT (the output of that launch is then incomplete).  Nothing
 * faults or hangs; set a short budget first.  The switch arms one launch. */
int ckks_b200_context_test_withhold_commit(ckks_b200_context* ctx, int on);
/* Test support for the overflow count of the tensor-core conversions (no reference counterpart).  The kernel takes
 * the count from a sum of products with reciprocals and repeats it with the reference's IEEE divisions
 * (BasisConv.cuh:121-131) only where that sum lies within 2^-40 of an integer, which random inputs practically never
 * reach.  With on != 0 every coefficient takes the division path, so a parity test covers it.  Stays set until
 * cleared. */
int ckks_b200_context_test_exact_count(ckks_b200_context* ctx, int on);

/* ---- level changes around the PCMM ------------------------------------------
 * d_cipher is the reference's Ciphertext buffer, a limbs then b limbs, each [L+1][N], NTT
 * domain, limb i modulo q_i of the context.
 *
 * Scheme_23::rescaleAndEqual (Scheme_23.cuh:339-385): divides a level-l ciphertext by q_l:
 * limbs i < l become (x_i - NTT_i(INTT_l(x_l) mod q_i)) * q_l^-1 mod q_i.  As in the reference
 * limb l is left holding its coefficients; the caller lowers the level and divides the scale by
 * q_l (:380-381).  1 <= l <= L. */
int ckks_b200_rescale(ckks_b200_context* ctx, uint64_t* d_cipher, int L, int l, void* stream);
/* Bootstrapper::modUpQ0toQL (bootstrapping/Bootstrapper.cuh:192-209, kernel Bootstrapping.cuh:6-23):
 * raises a level-0 ciphertext to target_level: the coefficients of limb 0 are lifted centred
 * (values above q_0/2 become x - q_0 + q_i*scale_up, in 64-bit unsigned arithmetic like the
 * reference) and reduced modulo q_1..q_target, then limbs 0..target_level go back to the NTT
 * domain.  scale_up is the reference's qVec[0] / precision (:203). */
int ckks_b200_modup_q0_to_ql(ckks_b200_context* ctx, uint64_t* d_cipher, int L, int target_level,
                             long long scale_up, void* stream);
/* The same two steps on `count` ciphertexts stored one after another, [count][2][L+1][N], all at the same
 * level: every transform and elementwise kernel runs once over all of them.  A single ciphertext leaves most
 * of the GPU idle (its inverse transform is two limb-polynomials); callers that keep their ciphertexts in one
 * pool get several times the rate from these forms.  Results are those of `count` single calls. */
int ckks_b200_rescale_batch(ckks_b200_context* ctx, uint64_t* d_ciphers, int count, int L, int l, void* stream);
int ckks_b200_modup_q0_to_ql_batch(ckks_b200_context* ctx, uint64_t* d_ciphers, int count, int L, int target_level,
                                   long long scale_up, void* stream);

/* ---- key-switch chain -------------------------------------------------------
 * The steps of Scheme_23::mult_23 / rotate / conjugate between the tensor product and the final
 * addition (KeySwitch_23.cuh:192-236), after modUpQjtoT_23 and the NTT over T.  gamma is the
 * reference's Context_23::gamma (moduli of [p | q] per output block); R = ceil((p_num+q_num)/gamma)
 * is its Ri_blockNum and dnum = q_num / p_num.  Every modulus must be below 2^62.
 *
 * Context_23::external_product_T (ExternalProduct.cuh:7-97): d_cipher_t [ceil((l+1)/p_num)][t_num][N]
 * (digits over T, NTT domain); d_swk the key, [2][dnum][R][t_num][N]; d_out [2][R][t_num][N], of which
 * blocks 0..ceil((p_num+l+1)/gamma)-1 are written. */
int ckks_b200_external_product_t(ckks_b200_context* ctx, uint64_t* d_out, const uint64_t* d_cipher_t,
                                 const uint64_t* d_swk, int l, int gamma, void* stream);
/* Context_23::FromNTTInplace_for_externalProduct (Context_23.cuh:909-930) as the chain calls it: the
 * inverse transform over T of the written blocks of both halves of a [2][R][t_num][N] buffer. */
int ckks_b200_ntt_inverse_ext(ckks_b200_context* ctx, uint64_t* d_data, int l, int gamma, void* stream);
/* Context_23::modUpTtoPQl_23 (BasisConv.cuh:183-248): d_in [batch][R][t_num][N] (coefficients over T)
 * -> d_out, same half stride R*t_num*N, limb i of [p | q_0..q_l] at offset i*N of its half. */
int ckks_b200_modup_t_to_pql(ckks_b200_context* ctx, uint64_t* d_out, const uint64_t* d_in, int l, int gamma,
                             int batch, void* stream);
/* Context_23::modDownPQltoQl_23 (BasisConv.cuh:251-347): d_in as written by ckks_b200_modup_t_to_pql ->
 * d_out [batch][q_num][N], limbs 0..l (coefficients). */
int ckks_b200_moddown_pql_to_ql(ckks_b200_context* ctx, uint64_t* d_out, const uint64_t* d_in, int l, int gamma,
                                int batch, void* stream);
/* The whole chain for one polynomial, as mult_23 runs it (KeySwitch_23.cuh:219-232): d_in [l+1][N]
 * (NTT domain) -> INTT -> modUpQjtoT_23 -> NTT over T -> external product with d_swk -> INTT -> modUp to
 * [p | q] -> modDown -> NTT; d_out [2][q_num][N], limbs 0..l.  Workspaces belong to the context. */
int ckks_b200_keyswitch(ckks_b200_context* ctx, uint64_t* d_out, const uint64_t* d_in, const uint64_t* d_swk,
                        int l, int gamma, void* stream);
/* Scheme_23::mult_23 (KeySwitch_23.cuh:192-236): ciphertext times ciphertext with relinearisation: the three
 * products per limb (compute_c0c1c2, poly_arithmetic.cuh:787-824), the key-switch chain on a1*a2 with the
 * relinearisation key d_rlk, and the final addition (cipher_add_axbx_batch_device, poly_arithmetic.cuh:155-172,
 * :416-420).  d_res, d_c1, d_c2: Ciphertext buffers [2][q_num][N], NTT domain, both operands at level l >= 1;
 * d_res may be one of the operands.  The caller multiplies the scales and sets the level (:211-212). */
int ckks_b200_mult(ckks_b200_context* ctx, uint64_t* d_res, const uint64_t* d_c1, const uint64_t* d_c2,
                   const uint64_t* d_rlk, int l, int gamma, void* stream);
/* Scheme_23::conjugate_23 and conjugateAndEqual_23 (KeySwitch_23.cuh:433-507): both polynomials reversed in the NTT
 * domain (sk_and_poly_conjugate_kernel, poly_arithmetic.cuh:666-674), the key-switch chain on the reversed a with
 * the conjugation key d_conj_key (laid out like every switching key above), the reversed b added to the b half.
 * d_res and d_cipher: Ciphertext buffers [2][q_num][N], NTT domain, level l; d_res may be d_cipher. */
int ckks_b200_conjugate(ckks_b200_context* ctx, uint64_t* d_res, const uint64_t* d_cipher, const uint64_t* d_conj_key,
                        int l, int gamma, void* stream);
/* Scheme_23::leftRotate_23 and leftRotateAndEqual_23 (KeySwitch_23.cuh:509-581): the chain on a with the key of
 * this rotation, b added to the b half, both halves permuted in the NTT domain by the Galois element
 * 5^(N/2 - rot_slots) mod 2N (sk_and_poly_LeftRot_ntt_kernel, poly_arithmetic.cuh:581-596; rotGroups,
 * Context_23.cuh:650-656).  1 <= rot_slots <= N/2.  d_res may be d_cipher. */
int ckks_b200_rotate(ckks_b200_context* ctx, uint64_t* d_res, const uint64_t* d_cipher, const uint64_t* d_rot_key,
                     long rot_slots, int l, int gamma, void* stream);

/* ---- ring packing, RLWE -> MLWE ---------------------------------------------
 * PCMM_Scheme::rlweCipherDecompose (pcmm/PCMM_Scheme.cuh:51-125): d_rlwe is the
 * reference's Ciphertext buffer, a limbs then b limbs, each [L+1][N]; limbs 0..l are
 * used with q moduli 0..l of the context.  MLWE ciphertext i is written to
 * h_mlwe_ptrs[i] (HOST array of device pointers) as [l+1][(k+1)*N1] with k = mlwe_rank =
 * N/N1 and gap = k/mlwe_num between extracted combs.  With ntt_domain != 0 the RLWE
 * ciphertext is taken out of and put back into the NTT domain around the gather, as the
 * reference does (:107,:124); with 0 it is read as coefficients and left untouched.
 * mlwe_num > mlwe_rank is the reference's error case (:103-106) -> CKKS_B200_ERR_SHAPE. */
int ckks_b200_rlwe_decompose(ckks_b200_context* ctx, uint64_t* d_rlwe, int L, int l,
                             uint64_t* const* h_mlwe_ptrs, int mlwe_num, int N1, int mlwe_rank,
                             int ntt_domain, void* stream);

/* ---- ring packing, MLWE -> RLWE ---------------------------------------------
 * PCMM_Scheme::mlweCipherPacking (pcmm/PCMM_Scheme.cuh:362-430) with its kernels
 * (:261-359): limb 0 of the mlwe_num MLWE ciphertexts in h_mlwe_ptrs (HOST array of
 * device pointers, each [..][(k+1)*N1]) is embedded into degree N with the centred lift
 * q0 -> p*q0, the k a-polynomials go through the NTT, are multiplied with the repacking
 * keys and summed, and the result comes back through INTT, ModDown by p, + b and NTT into
 * limb 0 of d_rlwe (a limbs then b limbs, each [L+1][N]; the caller sets l = 0 and the scale
 * as at :418-420).  As in the reference the ring-pack moduli are one special prime p (the
 * LAST p of the context) and one packing limb q0 (the FIRST q), with p > q0.
 * d_keys: the reference's contiguous key block, [k][2 (a,b)][2 limbs (p,q0)][N], NTT
 * domain (Key.cuh:20-25 with addRepakcingKey's sizes, PCMM_Scheme.cuh:170-186). */
int ckks_b200_mlwe_packing(ckks_b200_context* ctx, uint64_t* d_rlwe, int L,
                           uint64_t* const* h_mlwe_ptrs, int mlwe_num, int N1, int mlwe_rank,
                           const uint64_t* d_keys, void* stream);

/* ---- PCMM ------------------------------------------------------------------
 * Parameter carrier of PCMM_Context for the multiply (pcmm/PCMM_Context.cuh:7-57):
 * MLWE degree N1, rank k, and the ring-pack q moduli the product runs over
 * (any odd q < 2^62; the reference uses {q0,q1}). */
int ckks_b200_pcmm_create(ckks_b200_pcmm** out, int device, int N1, int mlwe_rank,
                          const uint64_t* q_ringpack, int q_count);
int ckks_b200_pcmm_destroy(ckks_b200_pcmm* pc);

#define CKKS_B200_PCMM_AUTO 0   /* tensor-core path (tcgen05) */
#define CKKS_B200_PCMM_TENSOR 1 /* same, explicit */
#define CKKS_B200_PCMM_SIMT 2   /* 64-bit CUDA-core path, the reference's formulation */

/* Scales a weight matrix (w = (int64)((double)W*scaler), PPMM_kernel.cuh:148) and cuts its byte planes once, and
 * keeps both on the handle: multiplies on this handle that pass d_W = NULL with the same mat_M, mat_N and scaler use
 * them, skip the per-call weight pre-pass and with it the one host wait a multiply otherwise contains (the read-back
 * of the weight range), so that such a call only enqueues work.  The reference re-converts the weights in every block
 * of every call (:148); layer weights are static, so a caller prepares each matrix once.  Preparing again, or any
 * multiply on the handle that passes its own d_W, replaces the kept weights.  Synchronises `stream` once. */
int ckks_b200_pcmm_prepare_weights(ckks_b200_pcmm* pc, const float* d_W, int mat_M, int mat_N, double scaler,
                                   void* stream);

/* PCMM_Scheme::PPMM (pcmm/PPMM_kernel.cuh:254-349) and its kernel (:93-252):
 *   out[m][i][c] = rescale_i( sum_n a(m,n,i) * X[n][i][c] mod q_i )
 * with w = (int64)((double)W[m][n]*scaler) truncated toward zero, a = w>0 ? w : q_i+w,
 * limbs processed last to first and every limb but the last rescaled by the last
 * (:213-249).  d_W is fp32 [mat_M][mat_N] row-major; h_X_ptrs is a HOST array of
 * mlwe_num device pointers, ciphertext n laid out [q_count][(k+1)*N1]
 * (pcmm/MLWECiphertext.cuh:8-10); d_out is [mat_M][q_count][(k+1)*N1], the
 * reference's ppmm_output.  Shape rules of the reference are kept: mat_K == N1 and
 * mat_N == mlwe_num, else CKKS_B200_ERR_SHAPE (:256-263).  Only columns
 * [col_begin, col_end) of every row are computed (multiples of 32, or the full
 * width); pass 0 and (k+1)*N1 for the whole product.  The call is asynchronous on
 * `stream` once the weights are known: with d_W given it waits for the stream once, to
 * read the range of the scaled weights back; with d_W = NULL it uses the weights kept by
 * ckks_b200_pcmm_prepare_weights and does not wait.
 * Ranges: the tensor-core path computes the exact signed sum and needs bits(q) + bits(w) +
 * ceil(log2 mat_N) <= 110 (a contraction too deep for one pass of 32-bit accumulators is cut
 * into several, summed in 128 bits).  The CUDA-core path accumulates a*x in 128 bits without
 * a range check, as the reference kernel does (:28,:106); it is refused
 * (CKKS_B200_ERR_RANGE / CKKS_B200_ERR_UNSUPPORTED) when |w| is not below the moduli or
 * ceil(log2 mat_N) + 2*bits(q) > 128, where the reference's sum could wrap. */
int ckks_b200_pcmm_ppmm(ckks_b200_pcmm* pc, const float* d_W, const uint64_t* const* h_X_ptrs,
                        uint64_t* d_out, int mat_M, int mat_N, int mat_K, int mlwe_num,
                        double scaler, long col_begin, long col_end, int algo, void* stream);
/* Decompose and multiply in one call: PCMM_Scheme::rlweCipherDecompose
 * (pcmm/PCMM_Scheme.cuh:51-125) feeding PCMM_Scheme::PPMM (pcmm/PPMM_kernel.cuh:254-349)
 * without the MLWE ciphertexts in between.  Source s stands for the call
 * rlweCipherDecompose(cipher_s, buffer, mlwe_num_s, offset_s): d_rlwe is that ciphertext,
 * [2][L+1][N] words in the COEFFICIENT domain (the state between the decomposition's
 * inverse and forward transforms; run ckks_b200_ntt_inverse first on a ciphertext in the
 * NTT domain), limb i reduced modulo ring-pack modulus i.  Every MLWE index in
 * [0, mlwe_num) must be filled by exactly one source.  The result is word for word that
 * of ckks_b200_rlwe_decompose on every source followed by ckks_b200_pcmm_ppmm (tensor-core
 * path).  Asynchronous on `stream`. */
typedef struct {
    const uint64_t* d_rlwe;
    int L;        /* the ciphertext holds L+1 limbs per polynomial */
    int mlwe_num; /* ciphertexts taken from it (gap = rank / mlwe_num) */
    int offset;   /* index of its first ciphertext among the multiply's inputs */
} ckks_b200_rlwe_source;
int ckks_b200_pcmm_ppmm_rlwe(ckks_b200_pcmm* pc, const float* d_W, const ckks_b200_rlwe_source* sources,
                             int n_sources, uint64_t* d_out, int mat_M, int mat_N, int mat_K, int mlwe_num,
                             double scaler, long col_begin, long col_end, void* stream);
/* Host-buffer form: h_W fp32 [M][N], h_X contiguous [mlwe_num][q_count][(k+1)*N1],
 * h_out [M][q_count][(k+1)*N1]; copies in, multiplies, copies out, synchronises.
 * The columns are cut into chunks that move through copy-in, multiply and copy-out
 * streams as a pipeline; ckks_b200_pcmm_set_host_chunks fixes their number (0 = chosen
 * from the size of the call). */
int ckks_b200_pcmm_set_host_chunks(ckks_b200_pcmm* pc, int chunks);
int ckks_b200_pcmm_ppmm_host(ckks_b200_pcmm* pc, const float* h_W, const uint64_t* h_X,
                             uint64_t* h_out, int mat_M, int mat_N, int mat_K, int mlwe_num,
                             double scaler, int algo);
/* Host-buffer form of ckks_b200_pcmm_ppmm_rlwe: the d_rlwe members of h_sources are HOST pointers here.  The RLWE
 * ciphertexts (2*(L+1)*N words each) are what crosses the bus on the way in, mlwe_num times less than the MLWE
 * ciphertexts cut from them; h_out as in ckks_b200_pcmm_ppmm_host.  Copies in, multiplies in column chunks
 * overlapped with the copy-out, synchronises. */
int ckks_b200_pcmm_ppmm_rlwe_host(ckks_b200_pcmm* pc, const float* h_W, const ckks_b200_rlwe_source* h_sources,
                                  int n_sources, uint64_t* h_out, int mat_M, int mat_N, int mat_K, int mlwe_num,
                                  double scaler);
/* The copy-back PPMM ends with (:345-348): row i of d_out, first `limbs` limbs, is
 * copied over ciphertext i for i < mlwe_num (the reference hard-codes limbs = 2). */
int ckks_b200_pcmm_copy_back(ckks_b200_pcmm* pc, const uint64_t* d_out,
                             uint64_t* const* h_X_ptrs, int mlwe_num, int limbs, void* stream);
/* Waits for `stream` and reports CKKS_B200_ERR_TIMEOUT if a bounded device-side wait
 * of a tensor-core multiply on this handle gave up since the last check, however many
 * multiplies ran in between: the record survives later launches and is cleared by the check
 * that reports it (no reference counterpart: the reference never checks a CUDA status). */
int ckks_b200_pcmm_check(ckks_b200_pcmm* pc, void* stream);
/* Clock cycles a device-side wait of the tensor-core multiply may take before it gives up (0 = the library's
 * default, about two seconds).  No reference counterpart. */
int ckks_b200_pcmm_set_wait_budget(ckks_b200_pcmm* pc, long long cycles);
/* Test support for the time-out path (no reference counterpart).  In the next tensor-core multiply on this handle the
 * thread that feeds operand tiles to every CTA stops before its tile number `stage` (counted from 0 per CTA) and
 * signals nothing, so the wait for that tile runs into the wait budget: the kernel raises the flag, waits for its
 * copies and instructions in flight, frees its tensor memory and returns normally; ckks_b200_pcmm_check then returns
 * CKKS_B200_ERR_TIMEOUT and the output of that launch is incomplete.  Nothing faults or hangs; set a short budget
 * first.  -1 switches it off; the switch arms one launch. */
int ckks_b200_pcmm_test_withhold_stage(ckks_b200_pcmm* pc, int stage);
/* No counterpart in the reference (which runs on one GPU).  For a multiply split by column range over several
 * GPUs whose consumer wants the whole output on every GPU: d_peer_out holds up to 7 device pointers, valid on
 * this GPU, to the OTHER GPUs' output buffers (same [M][limbs][C] layout; peer mappings, e.g. opened CUDA IPC
 * handles).  From the next tensor-core multiply on, every word the kernel stores to d_out it also stores, at the
 * same offset, into each of them (plain peer stores over NVLink from the epilogue), so the gather costs no
 * separate pass.  The words are in place on the peers once this GPU's stream has been synchronised; the ranks
 * then meet on the host.  count = 0 switches it off.  The CUDA-core algorithm does not support it. */
int ckks_b200_pcmm_set_peer_outputs(ckks_b200_pcmm* pc, uint64_t* const* d_peer_out, int count);
/* No counterpart in the reference.  The other way to bring a column-sharded multiply together: every output ROW (one
 * MLWE ciphertext, the unit PCMM_Scheme::mlweCipherPacking consumes, pcmm/PCMM_Scheme.cuh:362-430) has one owner
 * among `world` <= 8 GPUs, and the multiply stores each word it computes into its row's owner only (its own buffer or
 * one plain peer store over NVLink), instead of into everybody.  After every rank's launch and a stream
 * synchronisation each rank holds ALL columns of ITS rows; a rank sends (world-1)/world of what it computes and
 * receives as much, against (world-1) times its output for the broadcast above.  Rows are dealt out in equal
 * contiguous runs of ceil(mat_M/world) rounded up to a multiple of 32 (ckks_b200_pcmm_row_owner_range gives a rank's
 * run).  d_out_by_rank[r] is rank r's output buffer as addressable from this GPU (same [M][limbs][C] layout; the
 * entry of self_rank is ignored: the call's d_out is used).  world = 0 switches it off; it replaces
 * ckks_b200_pcmm_set_peer_outputs while on.  The CUDA-core algorithm does not support it. */
int ckks_b200_pcmm_set_row_owners(ckks_b200_pcmm* pc, uint64_t* const* d_out_by_rank, int world, int self_rank);
int ckks_b200_pcmm_row_owner_range(int mat_M, int world, int rank, int* row_begin, int* row_end);
/* Helpers for the pointers above when the other GPUs belong to other processes: ckks_b200_ipc_open maps the
 * allocation behind a 64-byte CUDA IPC memory handle (cudaIpcGetMemHandle in the owning process) for use by
 * kernels on `device` (cudaIpcOpenMemHandle with lazy peer access, `device` current) and returns its base
 * address; ckks_b200_ipc_close unmaps it. */
int ckks_b200_ipc_open(int device, const void* handle, void** d_base);
int ckks_b200_ipc_close(int device, void* d_base);
/* Device time in milliseconds of the latest tensor-core multiply on this handle, split
 * into its slicing pre-pass and its main kernel; waits for them.  Stands in for the
 * CUDATimer the reference wraps around its kernel (PPMM_kernel.cuh:301-343). */
int ckks_b200_pcmm_last_timing(ckks_b200_pcmm* pc, float* prepass_ms, float* main_ms);
/* No counterpart in the reference.  PPMM for callers that are not allowed to allocate
 * device memory (a serving process whose pool owns the GPU, a real-time loop, a sandboxed
 * plug-in): the same product as ckks_b200_pcmm_ppmm on the CUDA-core kernel, with no
 * handle and with all working memory (flags, ciphertext pointer table, scaled weights)
 * in one fixed array inside the library image, about 8 MB on every GPU the entry point
 * has been called on.  Runs on the CURRENT device.  Limits: mat_N <= 4096, mat_M*mat_N <= 2^20,
 * q_count <= 24; larger sizes return CKKS_B200_ERR_UNSUPPORTED.  It calls no allocator.
 * The array is shared by all calls: calls whose work overlaps on one GPU race and must be
 * serialised by the caller.  Every call waits for the stream once (it reads the weight range
 * back), so none may be issued while the stream is being captured into a CUDA graph; the
 * first call on each device also looks up the array's address.  The CUDA runtime loads device
 * code lazily by default: the 8 MB are claimed on a GPU at that first call, not when the
 * library is opened, so make one small warm-up call per device before a memory pool takes
 * the whole GPU (or set CUDA_MODULE_LOADING=EAGER).  Weight and K ranges as for the CUDA-core
 * algorithm of ckks_b200_pcmm_ppmm. */
int ckks_b200_pcmm_ppmm_static(const float* d_W, const uint64_t* const* h_X_ptrs, uint64_t* d_out,
                               int mat_M, int mat_N, int mat_K, int mlwe_num, int N1, int mlwe_rank,
                               const uint64_t* q_ringpack, int q_count, double scaler, void* stream);
/* Number of kernels this library has launched on the calling process so far. */
long ckks_b200_kernel_launches(void);

#ifdef __cplusplus
}
#endif
#endif /* CKKS_B200_H */
