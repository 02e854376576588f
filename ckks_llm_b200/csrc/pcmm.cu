// PCMM entry points: handle management, weight scaling pre-pass, the 64-bit CUDA-core
// multiply, and the host-buffer wrapper.  The tensor-core multiply lives in
// pcmm_umma.cu.  Semantics follow PCMM_Scheme::PPMM and pcmm_cuda_core_kernel of the
// reference (src/ckks/include/pcmm/PPMM_kernel.cuh:93-349).
#include <cstring>

#include "pcmm.cuh"
#include "pcmm_simt.cuh"

using namespace ckb;

namespace {

// w[m][n] = (int64) trunc((double)W[m][n] * scaler)   (PPMM_kernel.cuh:148)
// flags[0] collects the largest bit length of |w|; flags[2] is set when the product is
// not representable in int64 (NaN/inf or |.| >= 2^62).
__global__ void scale_weights_kernel(const float* W, long long* w, size_t count, double scaler, int* flags) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    int bits = 0;
    if (i < count) {
        double v = (double)W[i] * scaler;
        long long iv = 0;
        if (!(fabs(v) < 4611686018427387904.0)) {
            atomicOr(&flags[2], 1);
        } else {
            iv = (long long)v;
            unsigned long long mag = iv < 0 ? (unsigned long long)(-iv) : (unsigned long long)iv;
            bits = 64 - __clzll(mag);
        }
        w[i] = iv;
    }
    bits = __reduce_max_sync(0xffffffffu, bits);
    if ((threadIdx.x & 31) == 0 && bits > 0) atomicMax(&flags[0], bits);
}

// Scales the weights into pc->d_w (one kernel, one read-back of the flags: the stream is synchronised) and
// returns the bit length of the largest |w|.
int scale_weights(ckks_b200_pcmm* pc, const float* d_W, int M, int K, double scaler, cudaStream_t st, int* w_bits) {
    int rc = ensure_dev(&pc->d_w, &pc->w_cap, (size_t)M * K);
    if (rc) return rc;
    pc->prep_valid = false;                                        // d_w is about to change
    // words 0 and 2 belong to this pre-pass; word 1 (a wait that ran out) is only cleared by the check that reports it
    CKB_CUDA(cudaMemsetAsync(pc->d_flags, 0, sizeof(int), st));
    CKB_CUDA(cudaMemsetAsync(pc->d_flags + 2, 0, sizeof(int), st));
    size_t count = (size_t)M * K;
    scale_weights_kernel<<<(unsigned)((count + 255) / 256), 256, 0, st>>>(d_W, pc->d_w, count, scaler, pc->d_flags);
    count_launch();
    CKB_CUDA(cudaGetLastError());
    CKB_CUDA(cudaMemcpyAsync(pc->h_flags, pc->d_flags, 16 * sizeof(int), cudaMemcpyDeviceToHost, st));
    CKB_CUDA(cudaStreamSynchronize(st));
    CKB_REQUIRE(pc->h_flags[2] == 0, CKKS_B200_ERR_RANGE,
                "a scaled weight is not finite or exceeds 2^62 in magnitude");
    *w_bits = pc->h_flags[0];
    return CKKS_B200_OK;
}

// The 64-bit kernel accumulates a * x in 128 bits without a range check, like the reference kernel
// (PPMM_kernel.cuh:28,106).  Inside this bound the sum cannot wrap and q + w cannot either, so the CUDA-core and the
// tensor-core paths agree; beyond it the call is refused instead of returning the reference's wrapped words.
int simt_range_check(const ckks_b200_pcmm* pc, int K, int w_bits) {
    int q_bits = 0;
    for (u64 q : pc->q) {
        int b = 64 - __builtin_clzll(q);
        q_bits = b > q_bits ? b : q_bits;
    }
    int klog = 0;
    while ((1 << klog) < K) klog++;
    CKB_REQUIRE(w_bits < q_bits, CKKS_B200_ERR_RANGE, "a scaled weight of %d bits is not below the %d-bit moduli", w_bits, q_bits);
    CKB_REQUIRE(klog + 2 * q_bits <= 128, CKKS_B200_ERR_UNSUPPORTED,
                "K=%d products of two %d-bit factors do not fit the 128-bit accumulator of the CUDA-core kernel", K, q_bits);
    return CKKS_B200_OK;
}

// Uploads the pointer table unless the ciphertexts sit at one stride from one another (then base + n * stride
// addresses them and nothing is copied).
int make_source(ckks_b200_pcmm* pc, const u64* const* h_X_ptrs, int K, cudaStream_t st, PcmmSource* src) {
    bool strided = K >= 2 && h_X_ptrs[1] > h_X_ptrs[0];
    const size_t stride = strided ? (size_t)(h_X_ptrs[1] - h_X_ptrs[0]) : 0;
    for (int n = 2; n < K && strided; n++) strided = h_X_ptrs[n] == h_X_ptrs[0] + (size_t)n * stride;
    if (strided) {
        src->base = h_X_ptrs[0];
        src->stride = stride;
        return CKKS_B200_OK;
    }
    int rc = ensure_dev(&pc->d_xptrs, &pc->xptrs_cap, (size_t)K);
    if (rc) return rc;
    CKB_CUDA(cudaMemcpyAsync((void*)pc->d_xptrs, h_X_ptrs, sizeof(u64*) * K, cudaMemcpyHostToDevice, st));
    src->table = pc->d_xptrs;
    return CKKS_B200_OK;
}

int check_shape(const ckks_b200_pcmm* pc, int mat_M, int mat_N, int mat_K, int mlwe_num, long col_begin, long col_end) {
    // the reference's two shape rules (PPMM_kernel.cuh:256-263)
    CKB_REQUIRE(mat_K == pc->N1, CKKS_B200_ERR_SHAPE, "matrix K should be equal to N1!");
    CKB_REQUIRE(mat_N == mlwe_num, CKKS_B200_ERR_SHAPE, "matrix N should be equal to mlwe number!");
    CKB_REQUIRE(mat_M >= 1 && mat_N >= 1, CKKS_B200_ERR_ARG, "M and N must be positive");
    CKB_REQUIRE(mat_N <= (1 << 20), CKKS_B200_ERR_UNSUPPORTED, "contraction length above 2^20");
    CKB_REQUIRE(col_begin >= 0 && col_begin < col_end && col_end <= pc->C, CKKS_B200_ERR_ARG,
                "column range [%ld,%ld) outside [0,%ld)", col_begin, col_end, pc->C);
    CKB_REQUIRE(col_begin % 32 == 0 && (col_end % 32 == 0 || col_end == pc->C), CKKS_B200_ERR_ARG,
                "column range must start and end on multiples of 32");
    return CKKS_B200_OK;
}

// Weights of a multiply: scaled now from d_W, or, with d_W null, the ones ckks_b200_pcmm_prepare_weights left.
int resolve_weights(ckks_b200_pcmm* pc, const float* d_W, int mat_M, int mat_N, double scaler, cudaStream_t st, int* w_bits,
                    bool* ready) {
    if (d_W == nullptr) {
        CKB_REQUIRE(pc->prep_valid, CKKS_B200_ERR_ARG, "null weight pointer and no prepared weights on this handle");
        CKB_REQUIRE(pc->prep_M == mat_M && pc->prep_K == mat_N && pc->prep_scaler == scaler, CKKS_B200_ERR_ARG,
                    "the prepared weights are %dx%d at scaler %g, the call asks for %dx%d at %g", pc->prep_M, pc->prep_K,
                    pc->prep_scaler, mat_M, mat_N, scaler);
        *w_bits = pc->prep_w_bits;
        *ready = true;
        return CKKS_B200_OK;
    }
    *ready = false;
    return scale_weights(pc, d_W, mat_M, mat_N, scaler, st, w_bits);
}

int run_simt(ckks_b200_pcmm* pc, const PcmmSource& src, u64* d_out, int mat_M, int mat_N, long col_begin, long col_end,
             int w_bits, cudaStream_t st) {
    CKB_REQUIRE(pc->n_peers == 0 && pc->n_owners == 0, CKKS_B200_ERR_UNSUPPORTED,
                "outputs on other GPUs are written by the tensor-core kernel only");
    int rc = simt_range_check(pc, mat_N, w_bits);
    if (rc) return rc;
    dim3 grid((unsigned)((col_end - col_begin + TS - 1) / TS), (mat_M + TS - 1) / TS);
    SimtOperands ops{pc->d_w, src.table, src.base, src.stride};
    pcmm_simt_kernel<SimtLimbsPtr><<<grid, 256, 0, st>>>(ops, (u64*)d_out, SimtLimbsPtr{pc->d_limbs}, mat_M, mat_N, pc->C,
                                                         pc->q_count, col_begin, col_end);
    count_launch();
    CKB_CUDA(cudaGetLastError());
    return CKKS_B200_OK;
}

}  // namespace

extern "C" int ckks_b200_pcmm_create(ckks_b200_pcmm** out, int device, int N1, int mlwe_rank,
                                     const uint64_t* q_ringpack, int q_count) {
    CKB_REQUIRE(out != nullptr, CKKS_B200_ERR_ARG, "out is null");
    *out = nullptr;
    CKB_REQUIRE(q_ringpack && q_count >= 1 && q_count <= 64, CKKS_B200_ERR_ARG, "q_count %d outside [1,64]", q_count);
    CKB_REQUIRE(N1 >= 1 && mlwe_rank >= 1, CKKS_B200_ERR_ARG, "N1 and rank must be positive");
    int ndev = 0;
    CKB_CUDA(cudaGetDeviceCount(&ndev));
    CKB_REQUIRE(device >= 0 && device < ndev, CKKS_B200_ERR_ARG, "device %d of %d", device, ndev);
    DeviceGuard guard(device);
    CKB_REQUIRE(guard.ok, CKKS_B200_ERR_CUDA, "cudaSetDevice(%d) failed", device);
    std::vector<PcmmLimb> L(q_count);
    for (int i = 0; i < q_count; i++) {
        u64 q = q_ringpack[i];
        CKB_REQUIRE((q & 1) && q > 2 && q < (1ull << 62), CKKS_B200_ERR_ARG,
                    "ring-pack modulus %d (%llu) must be odd and below 2^62", i, q);
        L[i].q = q;
        h_barrett_mu(q, &L[i].mu_hi, &L[i].mu_lo);
        L[i].inv = L[i].inv_shoup = 0;
        // smallest multiple of q that is >= 2^112
        u128 k = (((u128)1 << 112) + q - 1) / q;
        u128 off = k * q;
        L[i].off_hi = (u64)(off >> 64);
        L[i].off_lo = (u64)off;
        L[i].pad = 0;
    }
    const u64 ql = q_ringpack[q_count - 1];
    for (int i = 0; i + 1 < q_count; i++) {
        u64 q = L[i].q;
        CKB_REQUIRE(ql % q != 0, CKKS_B200_ERR_ARG, "moduli %d and %d are not coprime", i, q_count - 1);
        // extended Euclid: the moduli need not be prime for the multiply
        __int128 a = ql % q, b = q, x0 = 1, x1 = 0;
        while (b) { __int128 t = a / b; __int128 r = a - t * b; a = b; b = r; __int128 xn = x0 - t * x1; x0 = x1; x1 = xn; }
        CKB_REQUIRE(a == 1, CKKS_B200_ERR_ARG, "moduli %d and %d are not coprime", i, q_count - 1);
        __int128 inv = x0 % (__int128)q;
        if (inv < 0) inv += q;
        L[i].inv = (u64)inv;
        L[i].inv_shoup = h_shoup(L[i].inv, q);
    }
    ckks_b200_pcmm* pc = new (std::nothrow) ckks_b200_pcmm();
    CKB_REQUIRE(pc != nullptr, CKKS_B200_ERR_NOMEM, "host allocation failed");
    pc->device = device;
    pc->N1 = N1;
    pc->rank = mlwe_rank;
    pc->q_count = q_count;
    pc->C = (long)(mlwe_rank + 1) * N1;
    pc->q.assign(q_ringpack, q_ringpack + q_count);
    cudaError_t e = cudaMalloc(&pc->d_limbs, sizeof(PcmmLimb) * q_count);
    if (e == cudaSuccess) e = cudaMemcpy(pc->d_limbs, L.data(), sizeof(PcmmLimb) * q_count, cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMalloc(&pc->d_flags, 16 * sizeof(int));
    if (e == cudaSuccess) e = cudaMallocHost(&pc->h_flags, 16 * sizeof(int));
    for (int i = 0; i < 3 && e == cudaSuccess; i++) e = cudaEventCreate(&pc->ev[i]);
    if (e != cudaSuccess) {
        set_error("allocating the PCMM handle failed: %s", cudaGetErrorString(e));
        ckks_b200_pcmm_destroy(pc);
        return CKKS_B200_ERR_CUDA;
    }
    *out = pc;
    return CKKS_B200_OK;
}

extern "C" int ckks_b200_pcmm_destroy(ckks_b200_pcmm* pc) {
    if (!pc) return CKKS_B200_OK;
    DeviceGuard guard(pc->device);
    cudaFree(pc->d_limbs); cudaFree(pc->d_w); cudaFree((void*)pc->d_xptrs); cudaFree(pc->d_slots); cudaFree(pc->d_flags);
    if (pc->h_flags) cudaFreeHost(pc->h_flags);
    cudaFree(pc->d_wplanes); cudaFree(pc->d_xplanes);
    for (int i = 0; i < 3; i++) if (pc->ev[i]) cudaEventDestroy(pc->ev[i]);
    for (int i = 0; i < 3; i++) if (pc->hs[i]) cudaStreamDestroy(pc->hs[i]);
    for (cudaEvent_t e : pc->hev) cudaEventDestroy(e);
    cudaFree(pc->d_W_host); cudaFree(pc->d_X_host); cudaFree(pc->d_out_host);
    delete pc;
    return CKKS_B200_OK;
}

// Opens a CUDA IPC memory handle exported by another process (another rank's cudaIpcGetMemHandle) for use from
// `device`: the mapping is made with that device current and with lazy peer access, which is what lets kernels
// running on it store into the other GPU's memory.
extern "C" int ckks_b200_ipc_open(int device, const void* handle, void** d_base) {
    CKB_REQUIRE(handle != nullptr && d_base != nullptr, CKKS_B200_ERR_ARG, "null argument");
    DeviceGuard guard(device);
    CKB_REQUIRE(guard.ok, CKKS_B200_ERR_CUDA, "cudaSetDevice(%d) failed", device);
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    CKB_CUDA(cudaIpcOpenMemHandle(d_base, h, cudaIpcMemLazyEnablePeerAccess));
    return CKKS_B200_OK;
}

extern "C" int ckks_b200_ipc_close(int device, void* d_base) {
    CKB_REQUIRE(d_base != nullptr, CKKS_B200_ERR_ARG, "null argument");
    DeviceGuard guard(device);
    CKB_REQUIRE(guard.ok, CKKS_B200_ERR_CUDA, "cudaSetDevice(%d) failed", device);
    CKB_CUDA(cudaIpcCloseMemHandle(d_base));
    return CKKS_B200_OK;
}

extern "C" int ckks_b200_pcmm_set_peer_outputs(ckks_b200_pcmm* pc, uint64_t* const* d_peer_out, int count) {
    CKB_REQUIRE(pc != nullptr && count >= 0 && count <= 7, CKKS_B200_ERR_ARG, "null handle or peer count outside [0,7]");
    CKB_REQUIRE(count == 0 || d_peer_out != nullptr, CKKS_B200_ERR_ARG, "null pointer table");
    for (int i = 0; i < count; i++) CKB_REQUIRE(d_peer_out[i] != nullptr, CKKS_B200_ERR_ARG, "peer pointer %d is null", i);
    for (int i = 0; i < 7; i++) pc->peer_out[i] = i < count ? (u64*)d_peer_out[i] : nullptr;
    pc->n_peers = count;
    if (count > 0) pc->n_owners = 0;            // one scheme at a time
    return CKKS_B200_OK;
}

extern "C" int ckks_b200_pcmm_set_row_owners(ckks_b200_pcmm* pc, uint64_t* const* d_out_by_rank, int world, int self_rank) {
    CKB_REQUIRE(pc != nullptr && world >= 0 && world <= 8, CKKS_B200_ERR_ARG, "null handle or world size outside [0,8]");
    CKB_REQUIRE(world == 0 || (d_out_by_rank != nullptr && self_rank >= 0 && self_rank < world), CKKS_B200_ERR_ARG,
                "null pointer table or rank %d outside [0,%d)", self_rank, world);
    for (int i = 0; i < world; i++)
        CKB_REQUIRE(i == self_rank || d_out_by_rank[i] != nullptr, CKKS_B200_ERR_ARG, "output pointer of rank %d is null", i);
    for (int i = 0; i < 8; i++) pc->owner_out[i] = (i < world && i != self_rank) ? (u64*)d_out_by_rank[i] : nullptr;
    pc->n_owners = world;
    pc->self_rank = world > 0 ? self_rank : 0;
    if (world > 0) pc->n_peers = 0;
    return CKKS_B200_OK;
}

extern "C" int ckks_b200_pcmm_row_owner_range(int mat_M, int world, int rank, int* row_begin, int* row_end) {
    CKB_REQUIRE(mat_M >= 1 && world >= 1 && rank >= 0 && rank < world && row_begin && row_end, CKKS_B200_ERR_ARG,
                "bad argument");
    const int per = ((mat_M + world - 1) / world + 31) / 32 * 32;
    const long b = (long)per * rank, e = b + per;
    *row_begin = (int)(b < mat_M ? b : mat_M);
    *row_end = (int)(e < mat_M ? e : mat_M);
    return CKKS_B200_OK;
}

extern "C" int ckks_b200_pcmm_set_wait_budget(ckks_b200_pcmm* pc, long long cycles) {
    CKB_REQUIRE(pc != nullptr && cycles >= 0, CKKS_B200_ERR_ARG, "null handle or negative budget");
    pc->wait_budget = cycles;
    return CKKS_B200_OK;
}

extern "C" int ckks_b200_pcmm_test_withhold_stage(ckks_b200_pcmm* pc, int stage) {
    CKB_REQUIRE(pc != nullptr && stage >= -1, CKKS_B200_ERR_ARG, "null handle or stage below -1");
    pc->withhold_stage = stage;
    return CKKS_B200_OK;
}

extern "C" int ckks_b200_pcmm_prepare_weights(ckks_b200_pcmm* pc, const float* d_W, int mat_M, int mat_N, double scaler,
                                              void* stream) {
    CKB_REQUIRE(pc && d_W, CKKS_B200_ERR_ARG, "null argument");
    CKB_REQUIRE(mat_M >= 1 && mat_N >= 1 && mat_N <= (1 << 20), CKKS_B200_ERR_ARG, "M and N must be positive, N at most 2^20");
    DeviceGuard guard(pc->device);
    CKB_REQUIRE(guard.ok, CKKS_B200_ERR_CUDA, "cudaSetDevice(%d) failed", pc->device);
    cudaStream_t st = (cudaStream_t)stream;
    int w_bits = 0;
    int rc = scale_weights(pc, d_W, mat_M, mat_N, scaler, st, &w_bits);
    if (rc) return rc;
    // cut the byte planes now; a handle whose moduli or weights the tensor-core path cannot take keeps the scaled
    // weights for the CUDA-core kernel
    int sw = 0, sc = 0, kpass = 0;
    if (pcmm_tensor_plan(pc, mat_N, w_bits, &sw, &sc, &kpass) == CKKS_B200_OK) {
        rc = pcmm_tensor(pc, pc->d_w, PcmmSource{}, nullptr, mat_M, mat_N, 0, 0, w_bits, false, st);
        if (rc) return rc;
    }
    pc->prep_valid = true;
    pc->prep_M = mat_M;
    pc->prep_K = mat_N;
    pc->prep_w_bits = w_bits;
    pc->prep_scaler = scaler;
    return CKKS_B200_OK;
}

extern "C" int ckks_b200_pcmm_ppmm(ckks_b200_pcmm* pc, const float* d_W,
                                   const uint64_t* const* h_X_ptrs, uint64_t* d_out, int mat_M,
                                   int mat_N, int mat_K, int mlwe_num, double scaler,
                                   long col_begin, long col_end, int algo, void* stream) {
    CKB_REQUIRE(pc && h_X_ptrs && d_out, CKKS_B200_ERR_ARG, "null argument");
    int rc = check_shape(pc, mat_M, mat_N, mat_K, mlwe_num, col_begin, col_end);
    if (rc) return rc;
    CKB_REQUIRE(algo >= 0 && algo <= 2, CKKS_B200_ERR_ARG, "unknown algorithm %d", algo);
    for (int n = 0; n < mlwe_num; n++)
        CKB_REQUIRE(h_X_ptrs[n] != nullptr, CKKS_B200_ERR_ARG, "ciphertext pointer %d is null", n);
    DeviceGuard guard(pc->device);
    CKB_REQUIRE(guard.ok, CKKS_B200_ERR_CUDA, "cudaSetDevice(%d) failed", pc->device);
    cudaStream_t st = (cudaStream_t)stream;
    int w_bits = 0;
    bool ready = false;
    rc = resolve_weights(pc, d_W, mat_M, mat_N, scaler, st, &w_bits, &ready);
    if (rc) return rc;
    PcmmSource src;
    rc = make_source(pc, (const u64* const*)h_X_ptrs, mat_N, st, &src);
    if (rc) return rc;
    if (algo == CKKS_B200_PCMM_SIMT) return run_simt(pc, src, (u64*)d_out, mat_M, mat_N, col_begin, col_end, w_bits, st);
    return pcmm_tensor(pc, pc->d_w, src, (u64*)d_out, mat_M, mat_N, col_begin, col_end, w_bits, ready && pc->prep_sw != 0, st);
}

namespace {

// Checks the sources of a decompose-and-multiply call and fills one slot per MLWE ciphertext; `regular` says whether
// the pre-pass that shares RLWE words between polynomials applies.
int build_slots(const ckks_b200_pcmm* pc, const ckks_b200_rlwe_source* sources, int n_sources, int mlwe_num,
                std::vector<RlweSlot>* slots_out, bool* regular_out) {
    CKB_REQUIRE(n_sources >= 1, CKKS_B200_ERR_ARG, "no source ciphertext");
    std::vector<RlweSlot>& slots = *slots_out;
    slots.assign(mlwe_num, RlweSlot{nullptr, 0, 0, 0, 0});
    for (int s = 0; s < n_sources; s++) {
        const ckks_b200_rlwe_source& S = sources[s];
        CKB_REQUIRE(S.d_rlwe != nullptr, CKKS_B200_ERR_ARG, "source %d is null", s);
        CKB_REQUIRE(S.L + 1 >= pc->q_count, CKKS_B200_ERR_ARG, "source %d holds %d limbs, the multiply runs %d", s, S.L + 1,
                    pc->q_count);
        // the reference's check (PCMM_Scheme.cuh:103-106)
        CKB_REQUIRE(S.mlwe_num >= 1 && S.mlwe_num <= pc->rank, CKKS_B200_ERR_SHAPE,
                    "rlweCipherDecompose extract number muse <= mlwe_rank");
        CKB_REQUIRE(S.offset >= 0 && S.offset + S.mlwe_num <= mlwe_num, CKKS_B200_ERR_ARG,
                    "source %d fills ciphertexts [%d,%d) of %d", s, S.offset, S.offset + S.mlwe_num, mlwe_num);
        for (int i = 0; i < S.mlwe_num; i++) {
            RlweSlot& d = slots[S.offset + i];
            CKB_REQUIRE(d.rlwe == nullptr, CKKS_B200_ERR_ARG, "ciphertext %d is filled by two sources", S.offset + i);
            d.rlwe = (const u64*)S.d_rlwe;
            d.L = S.L;
            d.i = i;
            d.gap = pc->rank / S.mlwe_num;
        }
    }
    for (int n = 0; n < mlwe_num; n++)
        CKB_REQUIRE(slots[n].rlwe != nullptr, CKKS_B200_ERR_ARG, "ciphertext %d is filled by no source", n);
    // the pre-pass that shares RLWE words between polynomials wants every aligned run of 16 ciphertexts from one source
    bool regular = pc->N1 % 32 == 0 && (long)pc->rank * pc->N1 >= 256;     // its index arithmetic wraps at most once
    for (int n0 = 0; n0 < mlwe_num && regular; n0 += 16) {
        const RlweSlot& f = slots[n0];
        if (f.gap > pcmm_slots_max_gap()) regular = false;
        for (int n = n0 + 1; n < mlwe_num && n < n0 + 16 && regular; n++)
            regular = slots[n].rlwe == f.rlwe && slots[n].L == f.L && slots[n].gap == f.gap && slots[n].i == f.i + (n - n0);
    }
    *regular_out = regular;
    return CKKS_B200_OK;
}

}  // namespace

// PCMM_Scheme::rlweCipherDecompose (PCMM_Scheme.cuh:51-125) followed by PCMM_Scheme::PPMM
// (PPMM_kernel.cuh:254-349) as one call: the multiply's slicing pre-pass reads the RLWE
// ciphertexts through the decomposition's index map, so the K MLWE ciphertexts (K times the
// size of what they are made from) are never written to or read from HBM.
extern "C" int ckks_b200_pcmm_ppmm_rlwe(ckks_b200_pcmm* pc, const float* d_W, const ckks_b200_rlwe_source* sources,
                                        int n_sources, uint64_t* d_out, int mat_M, int mat_N, int mat_K,
                                        int mlwe_num, double scaler, long col_begin, long col_end, void* stream) {
    CKB_REQUIRE(pc && sources && d_out, CKKS_B200_ERR_ARG, "null argument");
    int rc = check_shape(pc, mat_M, mat_N, mat_K, mlwe_num, col_begin, col_end);
    if (rc) return rc;
    std::vector<RlweSlot> slots;
    bool regular = false;
    rc = build_slots(pc, sources, n_sources, mlwe_num, &slots, &regular);
    if (rc) return rc;
    DeviceGuard guard(pc->device);
    CKB_REQUIRE(guard.ok, CKKS_B200_ERR_CUDA, "cudaSetDevice(%d) failed", pc->device);
    cudaStream_t st = (cudaStream_t)stream;
    rc = ensure_dev(&pc->d_slots, &pc->slots_cap, (size_t)mlwe_num);
    if (rc) return rc;
    // from pageable memory: the runtime has taken its copy of `slots` when this call returns
    CKB_CUDA(cudaMemcpyAsync(pc->d_slots, slots.data(), sizeof(RlweSlot) * mlwe_num, cudaMemcpyHostToDevice, st));
    int w_bits = 0;
    bool ready = false;
    rc = resolve_weights(pc, d_W, mat_M, mat_N, scaler, st, &w_bits, &ready);
    if (rc) return rc;
    PcmmSource src;
    src.slots = pc->d_slots;
    src.slots_regular = regular;
    return pcmm_tensor(pc, pc->d_w, src, (u64*)d_out, mat_M, mat_N, col_begin, col_end, w_bits, ready && pc->prep_sw != 0, st);
}

extern "C" int ckks_b200_pcmm_set_host_chunks(ckks_b200_pcmm* pc, int chunks) {
    CKB_REQUIRE(pc, CKKS_B200_ERR_ARG, "null handle");
    CKB_REQUIRE(chunks >= 0 && chunks <= 256, CKKS_B200_ERR_ARG, "chunk count %d outside [0,256]", chunks);
    pc->host_chunks = chunks;
    return CKKS_B200_OK;
}

namespace {

// Shared body of the two host-buffer entry points.  The weights are scaled (and their planes cut) once, then the
// columns are cut into chunks that move through three streams as a pipeline: while chunk i is multiplied, chunk i+1
// is on its way in (only when the ciphertexts themselves come from the host) and chunk i-1 on its way out.  Nothing
// in the chunk loop waits on the host, and the flags are read once at the end.
int host_pipeline(ckks_b200_pcmm* pc, const float* h_W, const uint64_t* h_X, const std::vector<RlweSlot>* slots,
                  bool slots_regular, uint64_t* h_out, int mat_M, int mat_N, double scaler, int algo) {
    const size_t ct_words = (size_t)pc->q_count * pc->C;
    int rc = ensure_dev(&pc->d_W_host, &pc->W_host_cap, (size_t)mat_M * mat_N);
    if (!rc && h_X) rc = ensure_dev(&pc->d_X_host, &pc->X_host_cap, ct_words * mat_N);
    if (!rc) rc = ensure_dev(&pc->d_out_host, &pc->out_host_cap, ct_words * mat_M);
    if (rc) return rc;
    for (int i = 0; i < 3; i++)
        if (!pc->hs[i]) CKB_CUDA(cudaStreamCreateWithFlags(&pc->hs[i], cudaStreamNonBlocking));
    cudaStream_t s_in = pc->hs[0], s_mm = pc->hs[1], s_out = pc->hs[2];
    const long tiles = (pc->C + 31) / 32;
    const size_t total_bytes = 8 * ct_words * ((size_t)(h_X ? mat_N : 0) + mat_M);
    // Equal chunks of 32-column tiles.  Sixteen is the measured optimum at the BERT shape (8.07 GB each way): fewer
    // leave the link idle while the first chunk comes in and the last goes out, more make the rows of the strided
    // host copies short (8 chunks 204 ms, 16 chunks 195 ms, 64 chunks 264 ms; small chunks at the two ends only,
    // 220 ms).
    std::vector<long> widths;
    {
        long n = pc->host_chunks > 0 ? pc->host_chunks : total_bytes > ((size_t)256 << 20) ? 16 : 1;
        if (n > tiles) n = tiles;
        for (long i = 0; i < n; i++) widths.push_back(tiles / n + (i < tiles % n ? 1 : 0));
    }
    const int nchunk = (int)widths.size();
    long widest = 0;
    for (long w : widths) widest = w > widest ? w : widest;
    if (algo != CKKS_B200_PCMM_SIMT) {
        rc = pcmm_reserve_planes(pc, mat_M, mat_N, widest * 32);
        if (rc) return rc;
    }
    while ((int)pc->hev.size() < 2 * nchunk + 1) {
        cudaEvent_t e;
        CKB_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
        pc->hev.push_back(e);
    }
    CKB_CUDA(cudaMemcpyAsync(pc->d_W_host, h_W, sizeof(float) * mat_M * mat_N, cudaMemcpyHostToDevice, s_mm));
    if (slots) {
        rc = ensure_dev(&pc->d_slots, &pc->slots_cap, (size_t)mat_N);
        if (rc) return rc;
        CKB_CUDA(cudaMemcpyAsync(pc->d_slots, slots->data(), sizeof(RlweSlot) * mat_N, cudaMemcpyHostToDevice, s_mm));
    }
    int w_bits = 0;
    rc = scale_weights(pc, pc->d_W_host, mat_M, mat_N, scaler, s_mm, &w_bits);       // the one host wait before the loop
    if (rc) return rc;
    if (algo == CKKS_B200_PCMM_SIMT) {
        CKB_REQUIRE(slots == nullptr, CKKS_B200_ERR_UNSUPPORTED, "the CUDA-core kernel reads stored MLWE ciphertexts only");
        rc = simt_range_check(pc, mat_N, w_bits);
    } else {
        rc = pcmm_tensor(pc, pc->d_w, PcmmSource{}, nullptr, mat_M, mat_N, 0, 0, w_bits, false, s_mm);     // weight planes
    }
    if (rc) return rc;
    PcmmSource src;
    if (slots) {
        src.slots = pc->d_slots;
        src.slots_regular = slots_regular;
    } else {
        src.base = pc->d_X_host;
        src.stride = ct_words;
    }
    const size_t pitch = (size_t)pc->C * 8;
    long t0 = 0;
    for (int i = 0; i < nchunk; i++) {
        const long t1 = t0 + widths[i];
        const long c0 = t0 * 32;
        long c1 = t1 * 32;
        t0 = t1;
        if (c1 > pc->C) c1 = pc->C;
        if (h_X) {
            CKB_CUDA(cudaMemcpy2DAsync(pc->d_X_host + c0, pitch, h_X + c0, pitch, (size_t)(c1 - c0) * 8,
                                       (size_t)mat_N * pc->q_count, cudaMemcpyHostToDevice, s_in));
            CKB_CUDA(cudaEventRecord(pc->hev[2 * i], s_in));
            CKB_CUDA(cudaStreamWaitEvent(s_mm, pc->hev[2 * i], 0));
        }
        if (algo == CKKS_B200_PCMM_SIMT) rc = run_simt(pc, src, pc->d_out_host, mat_M, mat_N, c0, c1, w_bits, s_mm);
        else rc = pcmm_tensor(pc, pc->d_w, src, pc->d_out_host, mat_M, mat_N, c0, c1, w_bits, true, s_mm);
        if (rc) return rc;
        CKB_CUDA(cudaEventRecord(pc->hev[2 * i + 1], s_mm));
        CKB_CUDA(cudaStreamWaitEvent(s_out, pc->hev[2 * i + 1], 0));
        CKB_CUDA(cudaMemcpy2DAsync(h_out + c0, pitch, pc->d_out_host + c0, pitch, (size_t)(c1 - c0) * 8,
                                   (size_t)mat_M * pc->q_count, cudaMemcpyDeviceToHost, s_out));
    }
    CKB_CUDA(cudaStreamSynchronize(s_out));
    if (algo != CKKS_B200_PCMM_SIMT) {
        rc = ckks_b200_pcmm_check(pc, s_mm);
        if (rc) return rc;
    }
    return CKKS_B200_OK;
}

}  // namespace

extern "C" int ckks_b200_pcmm_ppmm_host(ckks_b200_pcmm* pc, const float* h_W, const uint64_t* h_X,
                                        uint64_t* h_out, int mat_M, int mat_N, int mat_K,
                                        int mlwe_num, double scaler, int algo) {
    CKB_REQUIRE(pc && h_W && h_X && h_out, CKKS_B200_ERR_ARG, "null argument");
    int rc = check_shape(pc, mat_M, mat_N, mat_K, mlwe_num, 0, pc->C);
    if (rc) return rc;
    CKB_REQUIRE(algo >= 0 && algo <= 2, CKKS_B200_ERR_ARG, "unknown algorithm %d", algo);
    DeviceGuard guard(pc->device);
    CKB_REQUIRE(guard.ok, CKKS_B200_ERR_CUDA, "cudaSetDevice(%d) failed", pc->device);
    return host_pipeline(pc, h_W, h_X, nullptr, false, h_out, mat_M, mat_N, scaler, algo);
}

// Host-buffer form of ckks_b200_pcmm_ppmm_rlwe: the RLWE ciphertexts (2*(L+1)*N words each, K times smaller than the
// MLWE ciphertexts cut from them) are what crosses the bus on the way in.
extern "C" int ckks_b200_pcmm_ppmm_rlwe_host(ckks_b200_pcmm* pc, const float* h_W, const ckks_b200_rlwe_source* h_sources,
                                             int n_sources, uint64_t* h_out, int mat_M, int mat_N, int mat_K, int mlwe_num,
                                             double scaler) {
    CKB_REQUIRE(pc && h_W && h_sources && h_out, CKKS_B200_ERR_ARG, "null argument");
    int rc = check_shape(pc, mat_M, mat_N, mat_K, mlwe_num, 0, pc->C);
    if (rc) return rc;
    CKB_REQUIRE(n_sources >= 1 && n_sources <= 64, CKKS_B200_ERR_ARG, "source count %d outside [1,64]", n_sources);
    DeviceGuard guard(pc->device);
    CKB_REQUIRE(guard.ok, CKKS_B200_ERR_CUDA, "cudaSetDevice(%d) failed", pc->device);
    // device copies of the sources, one after another in the staging buffer of the ciphertexts
    const size_t N = (size_t)pc->rank * pc->N1;
    size_t words = 0;
    for (int s = 0; s < n_sources; s++) {
        CKB_REQUIRE(h_sources[s].d_rlwe != nullptr && h_sources[s].L >= 0, CKKS_B200_ERR_ARG, "source %d is null", s);
        words += 2 * (size_t)(h_sources[s].L + 1) * N;
    }
    rc = ensure_dev(&pc->d_X_host, &pc->X_host_cap, words);
    if (rc) return rc;
    for (int i = 0; i < 3; i++)
        if (!pc->hs[i]) CKB_CUDA(cudaStreamCreateWithFlags(&pc->hs[i], cudaStreamNonBlocking));
    std::vector<ckks_b200_rlwe_source> dev(h_sources, h_sources + n_sources);
    size_t off = 0;
    for (int s = 0; s < n_sources; s++) {
        const size_t w = 2 * (size_t)(h_sources[s].L + 1) * N;
        CKB_CUDA(cudaMemcpyAsync(pc->d_X_host + off, h_sources[s].d_rlwe, w * 8, cudaMemcpyHostToDevice, pc->hs[1]));
        dev[s].d_rlwe = (const uint64_t*)(pc->d_X_host + off);
        off += w;
    }
    std::vector<RlweSlot> slots;
    bool regular = false;
    rc = build_slots(pc, dev.data(), n_sources, mlwe_num, &slots, &regular);
    if (rc) return rc;
    return host_pipeline(pc, h_W, nullptr, &slots, regular, h_out, mat_M, mat_N, scaler, CKKS_B200_PCMM_TENSOR);
}

// The reference copies the first limb of row i of ppmm_output back over ciphertext i,
// reading rows at a stride of two limbs because it always runs two
// (PPMM_kernel.cuh:345-348).  Here the row stride is the real q_count and the caller
// chooses how many leading limbs to copy; limbs = 1 on a two-limb handle reproduces the
// reference.
extern "C" int ckks_b200_pcmm_copy_back(ckks_b200_pcmm* pc, const uint64_t* d_out,
                                        uint64_t* const* h_X_ptrs, int mlwe_num, int limbs,
                                        void* stream) {
    CKB_REQUIRE(pc && d_out && h_X_ptrs, CKKS_B200_ERR_ARG, "null argument");
    CKB_REQUIRE(limbs >= 1 && limbs <= pc->q_count && mlwe_num >= 0, CKKS_B200_ERR_ARG, "bad limb or ciphertext count");
    DeviceGuard guard(pc->device);
    CKB_REQUIRE(guard.ok, CKKS_B200_ERR_CUDA, "cudaSetDevice(%d) failed", pc->device);
    const size_t row = (size_t)pc->q_count * pc->C;
    for (int i = 0; i < mlwe_num; i++) {
        CKB_REQUIRE(h_X_ptrs[i] != nullptr, CKKS_B200_ERR_ARG, "ciphertext pointer %d is null", i);
        CKB_CUDA(cudaMemcpyAsync(h_X_ptrs[i], d_out + row * i, 8 * (size_t)limbs * pc->C,
                                 cudaMemcpyDeviceToDevice, (cudaStream_t)stream));
    }
    return CKKS_B200_OK;
}
