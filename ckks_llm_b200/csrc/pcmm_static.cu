// PPMM for callers that must not allocate.
//
// Some hosts of this library run where device allocation is off limits once the
// process is up: an inference server whose memory pool owns the whole GPU and treats any
// later cudaMalloc as a leak or an out-of-memory risk, a real-time loop that cannot
// afford the implicit device synchronisation an allocation or a free brings, or a
// sandboxed plug-in whose allocator hooks forbid raw CUDA allocations.  The regular
// entry point (ckks_b200_pcmm_ppmm) needs a handle and grows workspaces with
// cudaMalloc on first use, so it is closed to such callers.
//
// ckks_b200_pcmm_ppmm_static is the same multiply on the 64-bit CUDA-core kernel with
// every byte of working memory taken from one array that is part of the library image:
// a file-scope __device__ array.  It takes no handle; the per-limb constants are computed
// on the host and travel as kernel arguments.  The array holds, in this order, 256 bytes of
// flags, the table of ciphertext pointers (kMaxK entries) and the scaled weights
// (kMaxWeights int64).
//
// When the array comes to exist: the CUDA runtime loads a library's device code lazily by
// default, so the 8 MB are claimed on a GPU when this file's code is first touched there,
// which is the first call of the entry point on that GPU (its address look-up), not the
// moment the shared library is opened.  A host whose memory pool is about to take all of
// the GPU should therefore make one small warm-up call per device before the pool is
// created (or run with CUDA_MODULE_LOADING=EAGER); from then on the array stays until the
// process exits.
//
// Rules that follow from sharing one array:
//   * sizes above the stated maxima are refused with CKKS_B200_ERR_UNSUPPORTED;
//   * the array keeps whatever the previous call left; the flags are cleared at the start
//     of every call and everything else is overwritten before it is read;
//   * two calls whose work overlaps on the same GPU (different streams or threads) race
//     on the array: callers serialise them;
//   * every call copies its flags back to the host and waits for the stream once, so no
//     call may be issued while the stream is being captured into a CUDA graph; the first
//     call on each device additionally looks up the array's device address.
#include <mutex>

#include "pcmm_simt.cuh"

using namespace ckb;

namespace {

constexpr int kMaxK = 4096;                        // ciphertexts (= mat_N) per call
constexpr size_t kMaxWeights = (size_t)1 << 20;    // mat_M * mat_N per call
constexpr int kMaxLimbs = kSimtMaxLimbsByValue;    // ring-pack q moduli per call (24): their constants travel by value
constexpr int kMaxDevices = 64;
constexpr size_t kFlagsBytes = 256;
constexpr size_t kPtrBytes = (size_t)kMaxK * sizeof(u64*);
constexpr size_t kWeightsOffset = kFlagsBytes + kPtrBytes;          // 33024, a multiple of 256
constexpr size_t kScratchBytes = kWeightsOffset + kMaxWeights * sizeof(long long);

// About 8.03 MB per GPU.  In host code this name is only a handle for the runtime's
// symbol look-up, never a pointer a kernel could use.
static __device__ __align__(256) unsigned char g_static_scratch[kScratchBytes];

std::mutex g_setup_mutex;
unsigned char* g_scratch_addr[kMaxDevices] = {};

// Device address of the scratch array on the CURRENT device, looked up once per device.
int scratch_on_current_device(unsigned char** out) {
    int dev = -1;
    CKB_CUDA(cudaGetDevice(&dev));
    CKB_REQUIRE(dev >= 0 && dev < kMaxDevices, CKKS_B200_ERR_UNSUPPORTED, "device index %d above %d", dev, kMaxDevices - 1);
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (g_scratch_addr[dev] == nullptr) {
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess || p == nullptr) {
            set_error("cudaGetSymbolAddress of the static scratch failed on device %d: %s", dev, cudaGetErrorString(e));
            return CKKS_B200_ERR_CUDA;
        }
        g_scratch_addr[dev] = (unsigned char*)p;
    }
    *out = g_scratch_addr[dev];
    return CKKS_B200_OK;
}

// w = (int64) trunc((double)W * scaler) into the scratch; flags[0] collects the bit length of the
// largest |w|, flags[2] marks a value that does not fit (src/ckks/include/pcmm/PPMM_kernel.cuh:148
// for the conversion).
__global__ void static_scale_kernel(const float* W, unsigned char* scratch, size_t count, double scaler) {
    long long* w = reinterpret_cast<long long*>(scratch + kWeightsOffset);
    int* flags = reinterpret_cast<int*>(scratch);
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= count) return;
    double v = (double)W[i] * scaler;
    long long iv = 0;
    if (!(fabs(v) < 4611686018427387904.0)) atomicOr(&flags[2], 1);
    else iv = (long long)v;
    w[i] = iv;
    const unsigned long long mag = iv < 0 ? (unsigned long long)(-iv) : (unsigned long long)iv;
    if (mag) atomicMax(&flags[0], 64 - __clzll(mag));       // bit length of the largest |w|
}

}  // namespace

extern "C" int ckks_b200_pcmm_ppmm_static(const float* d_W, const uint64_t* const* h_X_ptrs, uint64_t* d_out,
                                          int mat_M, int mat_N, int mat_K, int mlwe_num, int N1, int mlwe_rank,
                                          const uint64_t* q_ringpack, int q_count, double scaler, void* stream) {
    CKB_REQUIRE(d_W && h_X_ptrs && d_out && q_ringpack, CKKS_B200_ERR_ARG, "null argument");
    CKB_REQUIRE(N1 >= 1 && mlwe_rank >= 1, CKKS_B200_ERR_ARG, "N1 and rank must be positive");
    CKB_REQUIRE(mat_K == N1, CKKS_B200_ERR_SHAPE, "matrix K should be equal to N1!");
    CKB_REQUIRE(mat_N == mlwe_num, CKKS_B200_ERR_SHAPE, "matrix N should be equal to mlwe number!");
    CKB_REQUIRE(mat_M >= 1 && mat_N >= 1, CKKS_B200_ERR_ARG, "M and N must be positive");
    CKB_REQUIRE(q_count >= 1 && q_count <= kMaxLimbs, CKKS_B200_ERR_UNSUPPORTED,
                "q_count %d exceeds the static limit of %d limbs", q_count, kMaxLimbs);
    CKB_REQUIRE(mat_N <= kMaxK, CKKS_B200_ERR_UNSUPPORTED,
                "mat_N %d exceeds the static scratch limit of %d ciphertexts", mat_N, kMaxK);
    CKB_REQUIRE((size_t)mat_M * (size_t)mat_N <= kMaxWeights, CKKS_B200_ERR_UNSUPPORTED,
                "mat_M*mat_N = %zu exceeds the static scratch limit of %zu weights",
                (size_t)mat_M * (size_t)mat_N, kMaxWeights);
    for (int n = 0; n < mlwe_num; n++)
        CKB_REQUIRE(h_X_ptrs[n] != nullptr, CKKS_B200_ERR_ARG, "ciphertext pointer %d is null", n);

    SimtLimbsVal limbs = {};
    for (int i = 0; i < q_count; i++) {
        const u64 q = q_ringpack[i];
        CKB_REQUIRE((q & 1) && q > 2 && q < (1ull << 62), CKKS_B200_ERR_ARG,
                    "ring-pack modulus %d (%llu) must be odd and below 2^62", i, q);
        limbs.l[i].q = q;
        h_barrett_mu(q, &limbs.l[i].mu_hi, &limbs.l[i].mu_lo);
    }
    const u64 ql = q_ringpack[q_count - 1];
    for (int i = 0; i + 1 < q_count; i++) {
        const u64 q = limbs.l[i].q;
        __int128 a = ql % q, b = q, x0 = 1, x1 = 0;
        while (b) {
            __int128 t = a / b, r = a - t * b;
            a = b; b = r;
            __int128 xn = x0 - t * x1;
            x0 = x1; x1 = xn;
        }
        CKB_REQUIRE(a == 1, CKKS_B200_ERR_ARG, "moduli %d and %d are not coprime", i, q_count - 1);
        __int128 inv = x0 % (__int128)q;
        if (inv < 0) inv += q;
        limbs.l[i].inv = (u64)inv;
        limbs.l[i].inv_shoup = h_shoup((u64)inv, q);
    }

    unsigned char* scratch = nullptr;
    int rc = scratch_on_current_device(&scratch);
    if (rc) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    const long C = (long)(mlwe_rank + 1) * N1;
    const size_t count = (size_t)mat_M * mat_N;

    CKB_CUDA(cudaMemsetAsync(scratch, 0, kFlagsBytes, st));                  // flags start at zero
    CKB_CUDA(cudaMemcpyAsync(scratch + kFlagsBytes, h_X_ptrs, sizeof(u64*) * mat_N, cudaMemcpyHostToDevice, st));
    static_scale_kernel<<<(unsigned)((count + 255) / 256), 256, 0, st>>>(d_W, scratch, count, scaler);
    count_launch();
    CKB_CUDA(cudaGetLastError());
    int flags[4] = {0, 0, 0, 0};
    CKB_CUDA(cudaMemcpyAsync(flags, scratch, sizeof(flags), cudaMemcpyDeviceToHost, st));
    CKB_CUDA(cudaStreamSynchronize(st));
    CKB_REQUIRE(flags[2] == 0, CKKS_B200_ERR_RANGE, "a scaled weight is not finite or exceeds 2^62 in magnitude");
    // The 128-bit accumulator of the kernel has no range check (neither has the reference's, PPMM_kernel.cuh:28,106):
    // refuse what could wrap it instead of returning wrapped words.
    int w_bits = flags[0], q_bits = 0, klog = 0;
    for (int i = 0; i < q_count; i++) {
        const int b = 64 - __builtin_clzll(q_ringpack[i]);
        q_bits = b > q_bits ? b : q_bits;
    }
    while ((1 << klog) < mat_N) klog++;
    CKB_REQUIRE(w_bits < q_bits, CKKS_B200_ERR_RANGE, "a scaled weight of %d bits is not below the %d-bit moduli", w_bits, q_bits);
    CKB_REQUIRE(klog + 2 * q_bits <= 128, CKKS_B200_ERR_UNSUPPORTED,
                "K=%d products of two %d-bit factors do not fit the 128-bit accumulator of the CUDA-core kernel", mat_N, q_bits);
    dim3 grid((unsigned)((C + TS - 1) / TS), (mat_M + TS - 1) / TS);
    SimtOperands ops{reinterpret_cast<const long long*>(scratch + kWeightsOffset),
                     reinterpret_cast<const u64* const*>(scratch + kFlagsBytes), nullptr, 0};
    pcmm_simt_kernel<SimtLimbsVal><<<grid, 256, 0, st>>>(ops, (u64*)d_out, limbs, mat_M, mat_N, C, q_count, 0, C);
    count_launch();
    CKB_CUDA(cudaGetLastError());
    return CKKS_B200_OK;
}
