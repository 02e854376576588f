// PCMM entry points: handle management, weight scaling pre-pass, the 64-bit CUDA-core
// multiply, and the host-buffer wrapper.  The tensor-core multiply lives in
// pcmm_umma.cu.  Semantics follow PCMM_Scheme::PPMM and pcmm_cuda_core_kernel of the
// reference (src/ckks/include/pcmm/PPMM_kernel.cuh:93-349).
#include <cstring>

#include "pcmm.cuh"

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

// ---------------------------------------------------------------------------
// CUDA-core multiply: 64x64 output tile per CTA, 4x4 outputs per thread, 128-bit
// accumulators, limbs last to first with the rescale fused (PPMM_kernel.cuh:213-249).
// ---------------------------------------------------------------------------
constexpr int TS = 64, TK = 16;

__global__ void __launch_bounds__(256) pcmm_simt_kernel(const long long* __restrict__ w,
                                                        const u64* const* __restrict__ X,
                                                        u64* __restrict__ out, const PcmmLimb* limbs,
                                                        int M, int K, long C, int limb_num,
                                                        long col_begin, long col_end) {
    __shared__ u64 As[TK][TS + 1];
    __shared__ u64 Xs[TK][TS];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const long c0 = col_begin + (long)blockIdx.x * TS;
    const int m0 = blockIdx.y * TS;
    u64 last[4][4];

    for (int i = limb_num - 1; i >= 0; i--) {
        const PcmmLimb L = limbs[i];
        u64 lo[4][4], hi[4][4];
#pragma unroll
        for (int r = 0; r < 4; r++)
#pragma unroll
            for (int s = 0; s < 4; s++) lo[r][s] = hi[r][s] = 0;

        for (int k0 = 0; k0 < K; k0 += TK) {
            __syncthreads();
            for (int e = threadIdx.x; e < TS * TK; e += 256) {
                int kk = e % TK, mm = e / TK;
                long long wv = (m0 + mm < M && k0 + kk < K) ? w[(size_t)(m0 + mm) * K + k0 + kk] : 0;
                // a = w > 0 ? w : q + w   (PPMM_kernel.cuh:23-25); padding contributes q*0
                As[kk][mm] = wv > 0 ? (u64)wv : L.q + (u64)wv;
            }
            for (int e = threadIdx.x; e < TS * TK; e += 256) {
                int cc = e % TS, kk = e / TS;
                u64 xv = 0;
                if (k0 + kk < K && c0 + cc < col_end) xv = X[k0 + kk][(size_t)i * C + c0 + cc];
                Xs[kk][cc] = xv;
            }
            __syncthreads();
#pragma unroll 4
            for (int kk = 0; kk < TK; kk++) {
                u64 a[4], x[4];
#pragma unroll
                for (int r = 0; r < 4; r++) a[r] = As[kk][ty + 16 * r];
#pragma unroll
                for (int s = 0; s < 4; s++) x[s] = Xs[kk][tx + 16 * s];
#pragma unroll
                for (int r = 0; r < 4; r++)
#pragma unroll
                    for (int s = 0; s < 4; s++) mac128(lo[r][s], hi[r][s], a[r], x[s]);
            }
        }
#pragma unroll
        for (int r = 0; r < 4; r++) {
            const int m = m0 + ty + 16 * r;
#pragma unroll
            for (int s = 0; s < 4; s++) {
                const long c = c0 + tx + 16 * s;
                u64 res = barrett128(lo[r][s], hi[r][s], L.q, L.mu_hi, L.mu_lo);
                if (i == limb_num - 1) {
                    last[r][s] = res;
                } else {
                    u64 tmp = res + L.q - last[r][s];            // wraps mod 2^64 as in :244
                    res = shoup_mul(tmp, L.inv, L.inv_shoup, L.q);
                }
                if (m < M && c < col_end) out[((size_t)m * limb_num + i) * C + c] = res;
            }
        }
    }
}

int prepare(ckks_b200_pcmm* pc, const float* d_W, const u64* const* h_X_ptrs, int M, int K,
            double scaler, cudaStream_t st, int* w_bits) {
    int rc = ensure_dev(&pc->d_w, &pc->w_cap, (size_t)M * K);
    if (rc) return rc;
    if (h_X_ptrs) {
        rc = ensure_dev(&pc->d_xptrs, &pc->xptrs_cap, (size_t)K);
        if (rc) return rc;
        CKB_CUDA(cudaMemcpyAsync((void*)pc->d_xptrs, h_X_ptrs, sizeof(u64*) * K, cudaMemcpyHostToDevice, st));
    }
    CKB_CUDA(cudaMemsetAsync(pc->d_flags, 0, 16 * sizeof(int), st));
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
    return CKKS_B200_OK;
}

extern "C" int ckks_b200_pcmm_ppmm(ckks_b200_pcmm* pc, const float* d_W,
                                   const uint64_t* const* h_X_ptrs, uint64_t* d_out, int mat_M,
                                   int mat_N, int mat_K, int mlwe_num, double scaler,
                                   long col_begin, long col_end, int algo, void* stream) {
    CKB_REQUIRE(pc && d_W && h_X_ptrs && d_out, CKKS_B200_ERR_ARG, "null argument");
    // the reference's two shape rules (PPMM_kernel.cuh:256-263)
    CKB_REQUIRE(mat_K == pc->N1, CKKS_B200_ERR_SHAPE, "matrix K should be equal to N1!");
    CKB_REQUIRE(mat_N == mlwe_num, CKKS_B200_ERR_SHAPE, "matrix N should be equal to mlwe number!");
    CKB_REQUIRE(mat_M >= 1 && mat_N >= 1, CKKS_B200_ERR_ARG, "M and N must be positive");
    CKB_REQUIRE(mat_N <= (1 << 20), CKKS_B200_ERR_UNSUPPORTED, "contraction length above 2^20");
    CKB_REQUIRE(col_begin >= 0 && col_begin < col_end && col_end <= pc->C, CKKS_B200_ERR_ARG,
                "column range [%ld,%ld) outside [0,%ld)", col_begin, col_end, pc->C);
    CKB_REQUIRE(col_begin % 32 == 0 && (col_end % 32 == 0 || col_end == pc->C), CKKS_B200_ERR_ARG,
                "column range must start and end on multiples of 32");
    CKB_REQUIRE(algo >= 0 && algo <= 2, CKKS_B200_ERR_ARG, "unknown algorithm %d", algo);
    for (int n = 0; n < mlwe_num; n++)
        CKB_REQUIRE(h_X_ptrs[n] != nullptr, CKKS_B200_ERR_ARG, "ciphertext pointer %d is null", n);
    DeviceGuard guard(pc->device);
    CKB_REQUIRE(guard.ok, CKKS_B200_ERR_CUDA, "cudaSetDevice(%d) failed", pc->device);
    cudaStream_t st = (cudaStream_t)stream;
    int w_bits = 0;
    int rc = prepare(pc, d_W, (const u64* const*)h_X_ptrs, mat_M, mat_N, scaler, st, &w_bits);
    if (rc) return rc;
    if (algo == CKKS_B200_PCMM_SIMT) {
        CKB_REQUIRE(pc->n_peers == 0, CKKS_B200_ERR_UNSUPPORTED, "peer outputs are written by the tensor-core kernel only");
        dim3 grid((unsigned)((col_end - col_begin + TS - 1) / TS), (mat_M + TS - 1) / TS);
        pcmm_simt_kernel<<<grid, 256, 0, st>>>(pc->d_w, pc->d_xptrs, (u64*)d_out, pc->d_limbs, mat_M,
                                               mat_N, pc->C, pc->q_count, col_begin, col_end);
        count_launch();
        CKB_CUDA(cudaGetLastError());
        return CKKS_B200_OK;
    }
    return pcmm_tensor(pc, pc->d_w, pc->d_xptrs, nullptr, false, (u64*)d_out, mat_M, mat_N, col_begin, col_end,
                       w_bits, st);
}

// PCMM_Scheme::rlweCipherDecompose (PCMM_Scheme.cuh:51-125) followed by PCMM_Scheme::PPMM
// (PPMM_kernel.cuh:254-349) as one call: the multiply's slicing pre-pass reads the RLWE
// ciphertexts through the decomposition's index map, so the K MLWE ciphertexts (K times the
// size of what they are made from) are never written to or read from HBM.
extern "C" int ckks_b200_pcmm_ppmm_rlwe(ckks_b200_pcmm* pc, const float* d_W, const ckks_b200_rlwe_source* sources,
                                        int n_sources, uint64_t* d_out, int mat_M, int mat_N, int mat_K,
                                        int mlwe_num, double scaler, long col_begin, long col_end, void* stream) {
    CKB_REQUIRE(pc && d_W && sources && d_out, CKKS_B200_ERR_ARG, "null argument");
    CKB_REQUIRE(mat_K == pc->N1, CKKS_B200_ERR_SHAPE, "matrix K should be equal to N1!");
    CKB_REQUIRE(mat_N == mlwe_num, CKKS_B200_ERR_SHAPE, "matrix N should be equal to mlwe number!");
    CKB_REQUIRE(mat_M >= 1 && mat_N >= 1, CKKS_B200_ERR_ARG, "M and N must be positive");
    CKB_REQUIRE(mat_N <= (1 << 20), CKKS_B200_ERR_UNSUPPORTED, "contraction length above 2^20");
    CKB_REQUIRE(col_begin >= 0 && col_begin < col_end && col_end <= pc->C, CKKS_B200_ERR_ARG,
                "column range [%ld,%ld) outside [0,%ld)", col_begin, col_end, pc->C);
    CKB_REQUIRE(col_begin % 32 == 0 && (col_end % 32 == 0 || col_end == pc->C), CKKS_B200_ERR_ARG,
                "column range must start and end on multiples of 32");
    CKB_REQUIRE(n_sources >= 1, CKKS_B200_ERR_ARG, "no source ciphertext");
    // every MLWE index must be produced by exactly one source
    std::vector<RlweSlot> slots(mlwe_num, RlweSlot{nullptr, 0, 0, 0, 0});
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
    DeviceGuard guard(pc->device);
    CKB_REQUIRE(guard.ok, CKKS_B200_ERR_CUDA, "cudaSetDevice(%d) failed", pc->device);
    cudaStream_t st = (cudaStream_t)stream;
    int rc = ensure_dev(&pc->d_slots, &pc->slots_cap, (size_t)mlwe_num);
    if (rc) return rc;
    CKB_CUDA(cudaMemcpyAsync(pc->d_slots, slots.data(), sizeof(RlweSlot) * mlwe_num, cudaMemcpyHostToDevice, st));
    int w_bits = 0;
    rc = prepare(pc, d_W, nullptr, mat_M, mat_N, scaler, st, &w_bits);      // synchronises: `slots` may go out of scope
    if (rc) return rc;
    // the pre-pass that shares RLWE words between polynomials wants every aligned run of 16 ciphertexts from one source
    bool regular = pc->N1 % 32 == 0 && (long)pc->rank * pc->N1 >= 256;     // its index arithmetic wraps at most once
    for (int n0 = 0; n0 < mlwe_num && regular; n0 += 16) {
        const RlweSlot& f = slots[n0];
        if (f.gap > pcmm_slots_max_gap()) regular = false;
        for (int n = n0 + 1; n < mlwe_num && n < n0 + 16 && regular; n++)
            regular = slots[n].rlwe == f.rlwe && slots[n].L == f.L && slots[n].gap == f.gap && slots[n].i == f.i + (n - n0);
    }
    return pcmm_tensor(pc, pc->d_w, nullptr, pc->d_slots, regular, (u64*)d_out, mat_M, mat_N, col_begin, col_end, w_bits,
                       st);
}

extern "C" int ckks_b200_pcmm_set_host_chunks(ckks_b200_pcmm* pc, int chunks) {
    CKB_REQUIRE(pc, CKKS_B200_ERR_ARG, "null handle");
    CKB_REQUIRE(chunks >= 0 && chunks <= 256, CKKS_B200_ERR_ARG, "chunk count %d outside [0,256]", chunks);
    pc->host_chunks = chunks;
    return CKKS_B200_OK;
}

extern "C" int ckks_b200_pcmm_ppmm_host(ckks_b200_pcmm* pc, const float* h_W, const uint64_t* h_X,
                                        uint64_t* h_out, int mat_M, int mat_N, int mat_K,
                                        int mlwe_num, double scaler, int algo) {
    CKB_REQUIRE(pc && h_W && h_X && h_out, CKKS_B200_ERR_ARG, "null argument");
    CKB_REQUIRE(mat_K == pc->N1, CKKS_B200_ERR_SHAPE, "matrix K should be equal to N1!");
    CKB_REQUIRE(mat_N == mlwe_num, CKKS_B200_ERR_SHAPE, "matrix N should be equal to mlwe number!");
    CKB_REQUIRE(mat_M >= 1 && mat_N >= 1, CKKS_B200_ERR_ARG, "M and N must be positive");
    DeviceGuard guard(pc->device);
    CKB_REQUIRE(guard.ok, CKKS_B200_ERR_CUDA, "cudaSetDevice(%d) failed", pc->device);
    const size_t ct_words = (size_t)pc->q_count * pc->C;
    int rc = ensure_dev(&pc->d_W_host, &pc->W_host_cap, (size_t)mat_M * mat_N);
    if (!rc) rc = ensure_dev(&pc->d_X_host, &pc->X_host_cap, ct_words * mlwe_num);
    if (!rc) rc = ensure_dev(&pc->d_out_host, &pc->out_host_cap, ct_words * mat_M);
    if (rc) return rc;
    // Column chunks are pipelined over three streams: while chunk i is multiplied, chunk i+1
    // is on its way in and chunk i-1 on its way out (columns are independent of one another).
    for (int i = 0; i < 3; i++)
        if (!pc->hs[i]) CKB_CUDA(cudaStreamCreateWithFlags(&pc->hs[i], cudaStreamNonBlocking));
    cudaStream_t s_in = pc->hs[0], s_mm = pc->hs[1], s_out = pc->hs[2];
    const long tiles = (pc->C + 31) / 32;
    const size_t total_bytes = 8 * ct_words * ((size_t)mlwe_num + mat_M);
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
    rc = pcmm_reserve_planes(pc, mat_M, mat_N, widest * 32);
    if (rc) return rc;
    while ((int)pc->hev.size() < 2 * nchunk) {
        cudaEvent_t e;
        CKB_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
        pc->hev.push_back(e);
    }
    CKB_CUDA(cudaMemcpyAsync(pc->d_W_host, h_W, sizeof(float) * mat_M * mat_N, cudaMemcpyHostToDevice, s_in));
    std::vector<const uint64_t*> ptrs(mlwe_num);
    for (int n = 0; n < mlwe_num; n++) ptrs[n] = (const uint64_t*)(pc->d_X_host + ct_words * n);
    const size_t pitch = (size_t)pc->C * 8;
    long t0 = 0;
    for (int i = 0; i < nchunk; i++) {
        const long t1 = t0 + widths[i];
        const long c0 = t0 * 32;
        long c1 = t1 * 32;
        t0 = t1;
        if (c1 > pc->C) c1 = pc->C;
        CKB_CUDA(cudaMemcpy2DAsync(pc->d_X_host + c0, pitch, h_X + c0, pitch, (size_t)(c1 - c0) * 8,
                                   (size_t)mlwe_num * pc->q_count, cudaMemcpyHostToDevice, s_in));
        CKB_CUDA(cudaEventRecord(pc->hev[2 * i], s_in));
        CKB_CUDA(cudaStreamWaitEvent(s_mm, pc->hev[2 * i], 0));
        rc = ckks_b200_pcmm_ppmm(pc, pc->d_W_host, ptrs.data(), (uint64_t*)pc->d_out_host, mat_M, mat_N, mat_K,
                                 mlwe_num, scaler, c0, c1, algo, s_mm);
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
