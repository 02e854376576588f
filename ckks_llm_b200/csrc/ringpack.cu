// Ring packing, RLWE -> MLWE direction: PCMM_Scheme::rlweCipherDecompose of the reference
// (src/ckks/include/pcmm/PCMM_Scheme.cuh:51-125).  One RLWE ciphertext (a, b) of degree N
// becomes mlwe_num MLWE ciphertexts of rank k = N/N1 and degree N1:
//   b_i[g]     =  B[i*gap + g*k]
//   a_i,0[g]   =  A[i*gap + g*k]
//   a_i,r[g]   =  A[(g-1)*k + (k-r) + i*gap]                 g >= 1, r = 1..k-1
//   a_i,r[0]   = -A[(N1-1)*k + (k-r) + i*gap]                (an index >= N wraps and flips the sign)
// with gap = k / mlwe_num, in the coefficient domain; the reference runs an inverse NTT on
// the RLWE ciphertext first and a forward NTT afterwards, and so does this entry point.
//
// One thread writes one output word; consecutive threads write consecutive words of an
// MLWE polynomial (coalesced), and read the RLWE limb with stride k.  The limb (512 KiB at
// N = 2^16) is read k times over and stays in L2, so HBM sees the output stream only:
// (k+1)*N1 words per MLWE ciphertext per limb.
#include "context.cuh"

using namespace ckb;

namespace {

__global__ void __launch_bounds__(256) rlwe_decompose_kernel(const u64* __restrict__ rlwe, u64* const* __restrict__ mlwe,
                                                             const u64* __restrict__ q_moduli, long N, int N1, int k,
                                                             int mlwe_num, int L) {
    const long C = (long)(k + 1) * N1;
    const long w = (long)blockIdx.x * blockDim.x + threadIdx.x;     // word inside one limb of one MLWE ciphertext
    if (w >= C) return;
    const int limb = blockIdx.y, i = blockIdx.z;
    const u64 q = q_moduli[limb];
    const int gap = k / mlwe_num;
    const int r = (int)(w / N1), g = (int)(w % N1);
    const u64* A = rlwe + N * limb;
    const u64* B = rlwe + N * (L + 1 + limb);
    long addr;
    bool negate;
    const u64* src;
    if (r == k) {                 // b polynomial
        addr = (long)i * gap + (long)g * k;
        src = B;
        negate = false;
    } else if (r == 0) {
        addr = (long)i * gap + (long)g * k;
        src = A;
        negate = false;
    } else if (g == 0) {
        addr = (long)(N1 - 1) * k + (k - r) + (long)i * gap;
        src = A;
        negate = true;
    } else {
        addr = (long)(g - 1) * k + (k - r) + (long)i * gap;
        src = A;
        negate = false;
    }
    if (addr >= N) { addr -= N; negate = !negate; }
    u64 v = src[addr];
    if (negate) v = v == 0 ? 0 : q - v;
    mlwe[i][(size_t)limb * C + w] = v;
}

}  // namespace

extern "C" int ckks_b200_rlwe_decompose(ckks_b200_context* c, uint64_t* d_rlwe, int L, int l,
                                        uint64_t* const* h_mlwe_ptrs, int mlwe_num, int N1, int mlwe_rank,
                                        int ntt_domain, void* stream) {
    CKB_REQUIRE(c && d_rlwe && h_mlwe_ptrs, CKKS_B200_ERR_ARG, "null argument");
    CKB_REQUIRE(N1 >= 1 && mlwe_rank >= 1 && (long)N1 * mlwe_rank == (long)c->N, CKKS_B200_ERR_SHAPE,
                "N1 * rank must equal N (%d * %d vs %u)", N1, mlwe_rank, c->N);
    CKB_REQUIRE(l >= 0 && l <= L && L < c->q_num, CKKS_B200_ERR_ARG, "levels l=%d L=%d outside the %d q moduli", l, L, c->q_num);
    // the reference's check (PCMM_Scheme.cuh:103-106)
    CKB_REQUIRE(mlwe_num >= 1 && mlwe_num <= mlwe_rank, CKKS_B200_ERR_SHAPE,
                "rlweCipherDecompose extract number muse <= mlwe_rank");
    CKB_REQUIRE(mlwe_num <= 65535, CKKS_B200_ERR_UNSUPPORTED, "more than 65535 MLWE ciphertexts in one call");
    for (int i = 0; i < mlwe_num; i++)
        CKB_REQUIRE(h_mlwe_ptrs[i] != nullptr, CKKS_B200_ERR_ARG, "MLWE pointer %d is null", i);
    DeviceGuard guard(c->device);
    CKB_REQUIRE(guard.ok, CKKS_B200_ERR_CUDA, "cudaSetDevice(%d) failed", c->device);
    cudaStream_t st = (cudaStream_t)stream;
    int rc = ensure_buf(&c->ptr_buf, &c->ptr_cap, (size_t)mlwe_num);
    if (rc) return rc;
    CKB_CUDA(cudaMemcpyAsync(c->ptr_buf, h_mlwe_ptrs, sizeof(u64*) * mlwe_num, cudaMemcpyHostToDevice, st));
    if (ntt_domain) {
        rc = ckks_b200_ntt_inverse(c, d_rlwe, 0, c->p_num, 2, l + 1, L + 1, stream);     // :107
        if (rc) return rc;
    }
    const long C = (long)(mlwe_rank + 1) * N1;
    dim3 grid((unsigned)((C + 255) / 256), l + 1, mlwe_num);
    rlwe_decompose_kernel<<<grid, 256, 0, st>>>((const u64*)d_rlwe, (u64* const*)c->ptr_buf, c->d_moduli + c->p_num,
                                                (long)c->N, N1, mlwe_rank, mlwe_num, L);
    count_launch();
    CKB_CUDA(cudaGetLastError());
    if (ntt_domain) {
        rc = ckks_b200_ntt_forward(c, d_rlwe, 0, c->p_num, 2, l + 1, L + 1, stream);      // :124
        if (rc) return rc;
    }
    return CKKS_B200_OK;
}
