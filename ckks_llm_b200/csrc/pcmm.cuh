// PCMM handle: ring-pack moduli, per-limb constants and device workspaces.
#pragma once
#include <vector>

#include "common.cuh"

// Per-limb constants, one entry per ring-pack q modulus.
struct PcmmLimb {
    u64 q;
    u64 mu_hi, mu_lo;      // floor(2^128 / q)
    u64 inv, inv_shoup;    // q_last^-1 mod q and its Shoup companion (unused for the last limb)
    u64 off_hi, off_lo;    // a multiple of q that exceeds 2^110, added before reducing signed sums
    u64 pad;
};

// Where MLWE ciphertext n of a multiply comes from when the PCMM reads RLWE ciphertexts directly:
// ciphertext i of the decomposition of `rlwe` ([2][L+1][N] words, coefficient domain) with the given gap.
struct RlweSlot {
    const u64* rlwe;
    int L, i, gap, pad;
};

struct ckks_b200_pcmm {
    int device = 0;
    int N1 = 0, rank = 0, q_count = 0;
    long C = 0;                       // (rank+1)*N1 words per ciphertext per limb
    std::vector<u64> q;
    PcmmLimb* d_limbs = nullptr;

    long long* d_w = nullptr;         // scaled weights [M][K] (int64)
    size_t w_cap = 0;
    const u64** d_xptrs = nullptr;    // device copy of the ciphertext pointer table
    size_t xptrs_cap = 0;
    RlweSlot* d_slots = nullptr;      // per-ciphertext sources of the multiply that decomposes on the fly
    size_t slots_cap = 0;
    u64* peer_out[7] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};   // see ckks_b200_pcmm_set_peer_outputs
    int n_peers = 0;
    int* d_flags = nullptr;           // [0] max |w| bits seen, [1] device-side wait timeout, ...
    int* h_flags = nullptr;           // pinned mirror

    // tensor-core path workspaces
    uint8_t* d_wplanes = nullptr;     // weight byte planes in MMA tile order
    size_t wplanes_cap = 0;
    uint8_t* d_xplanes = nullptr;     // ciphertext byte planes in MMA tile order
    size_t xplanes_cap = 0;

    // events around the pre-pass and the main kernel of the latest tensor-core multiply
    cudaEvent_t ev[3] = {nullptr, nullptr, nullptr};
    bool ev_valid = false;

    // streams and events of the pipelined *_host entry point
    cudaStream_t hs[3] = {nullptr, nullptr, nullptr};
    std::vector<cudaEvent_t> hev;
    int host_chunks = 0;   // column chunks of the host-buffer call; 0 = chosen from the size

    // staging for the *_host entry point
    float* d_W_host = nullptr;
    size_t W_host_cap = 0;
    u64* d_X_host = nullptr;
    size_t X_host_cap = 0;
    u64* d_out_host = nullptr;
    size_t out_host_cap = 0;
};

namespace ckb {
template <class T>
int ensure_dev(T** buf, size_t* cap, size_t count) {
    if (*cap >= count) return CKKS_B200_OK;
    if (*buf) cudaFree((void*)*buf);
    *buf = nullptr;
    *cap = 0;
    if (cudaMalloc((void**)buf, count * sizeof(T)) != cudaSuccess) {
        cudaGetLastError();
        set_error("cudaMalloc of %zu bytes failed", count * sizeof(T));
        return CKKS_B200_ERR_NOMEM;
    }
    *cap = count;
    return CKKS_B200_OK;
}

// Tensor-core path (pcmm_umma.cu).  w_bits = bit length of the largest |w|.  The ciphertext words come from
// the pointer table d_xptrs, or, when d_slots is given, straight from RLWE ciphertexts through the
// decomposition's index map.
// slots_regular: N1 is a multiple of 32, every aligned run of 16 ciphertexts lies in one source with consecutive
// indices and no gap exceeds pcmm_slots_max_gap(), which lets the pre-pass share RLWE words between polynomials.
int pcmm_tensor(ckks_b200_pcmm* pc, const long long* d_w, const u64* const* d_xptrs, const RlweSlot* d_slots,
                bool slots_regular, u64* d_out, int M, int K, long col_begin, long col_end, int w_bits, cudaStream_t st);
int pcmm_slots_max_gap();
int pcmm_reserve_planes(ckks_b200_pcmm* pc, int M, int K, long ncols);
}  // namespace ckb
