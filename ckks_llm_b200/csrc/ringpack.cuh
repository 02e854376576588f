// The RLWE -> MLWE index map of PCMM_Scheme::rlweCipherDecompose
// (src/ckks/include/pcmm/PCMM_Scheme.cuh:51-88), shared by the decompose kernel and by the
// ciphertext slicing pre-pass of the PCMM that reads the RLWE ciphertext directly:
//   b_i[g]     =  B[i*gap + g*k]
//   a_i,0[g]   =  A[i*gap + g*k]
//   a_i,r[g]   =  A[(g-1)*k + (k-r) + i*gap]                 g >= 1, r = 1..k-1
//   a_i,r[0]   = -A[(N1-1)*k + (k-r) + i*gap]                (an index >= N wraps and flips the sign)
#pragma once
#include "common.cuh"

namespace ckb {

// word g of polynomial r of MLWE ciphertext i, one limb (the index maps at the top of the file)
__device__ __forceinline__ u64 decompose_word(const u64* __restrict__ A, const u64* __restrict__ B, u64 q, long N, int N1, int k,
                                              int gap, int i, int r, int g) {
    long addr;
    bool negate = false;
    const u64* src = A;
    if (r == k) {                 // b polynomial
        addr = (long)i * gap + (long)g * k;
        src = B;
    } else if (r == 0) {
        addr = (long)i * gap + (long)g * k;
    } else if (g == 0) {
        addr = (long)(N1 - 1) * k + (k - r) + (long)i * gap;
        negate = true;
    } else {
        addr = (long)(g - 1) * k + (k - r) + (long)i * gap;
    }
    if (addr >= N) { addr -= N; negate = !negate; }
    const u64 v = src[addr];
    return negate ? (v == 0 ? 0 : q - v) : v;
}

}  // namespace ckb
