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
    // see ckks_b200_pcmm_set_row_owners: output buffer of every rank (nullptr = the call's d_out), rows per owner
    u64* owner_out[8] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
    int n_owners = 0, self_rank = 0;
    // [0] max |w| bits seen, [2] a scaled weight out of range: both cleared by every weight scaling;
    // [1] site of a device-side wait that ran out: set by kernels, cleared only by ckks_b200_pcmm_check
    int* d_flags = nullptr;
    int* h_flags = nullptr;           // pinned mirror
    long long wait_budget = 0;        // clock cycles a device-side wait may take (0: the library's default)
    int withhold_stage = -1;          // see ckks_b200_pcmm_test_withhold_stage; consumed by the next tensor-core launch

    // weights kept by ckks_b200_pcmm_prepare_weights: d_w and d_wplanes hold them, multiplies that pass a null
    // weight pointer use them
    bool prep_valid = false;
    int prep_M = 0, prep_K = 0, prep_w_bits = 0;
    int prep_sw = 0, prep_sc = 0;     // plane configuration d_wplanes was cut for (0: not cut yet)
    double prep_scaler = 0.0;

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
// Where the ciphertext words of a multiply come from: a device table of pointers, or (table == nullptr) ciphertext n
// at base + n * stride words, or RLWE ciphertexts through the decomposition's index map (slots != nullptr).
struct PcmmSource {
    const u64* const* table = nullptr;
    const u64* base = nullptr;
    size_t stride = 0;
    const RlweSlot* slots = nullptr;
    bool slots_regular = false;
};
// weights_ready: d_wplanes already holds the planes of these weights (prepared weights), skip their slicing.
int pcmm_tensor(ckks_b200_pcmm* pc, const long long* d_w, const PcmmSource& src, u64* d_out, int M, int K,
                long col_begin, long col_end, int w_bits, bool weights_ready, cudaStream_t st);
// Plane configuration (SW, SC) and K blocks per accumulation pass the tensor-core path takes for these weights.
int pcmm_tensor_plan(const ckks_b200_pcmm* pc, int K, int w_bits, int* sw_out, int* sc_out, int* kpass_out);
int pcmm_slots_max_gap();
int pcmm_reserve_planes(ckks_b200_pcmm* pc, int M, int K, long ncols);
}  // namespace ckb
