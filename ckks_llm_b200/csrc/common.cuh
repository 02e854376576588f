// Shared declarations of the B200 CKKS hot-path library: status codes, error
// reporting, and the 64/128-bit modular primitives every kernel uses.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <atomic>
#include <string>

#include "../../include/ckks_b200.h"

typedef unsigned long long u64;   // same width as uint64_t; the type CUDA intrinsics take
typedef unsigned __int128 u128;

namespace ckb {

// Thread-local message describing the last non-OK status returned on this thread.
void set_error(const char* fmt, ...);
const char* get_error();

#define CKB_CUDA(call)                                                              \
    do {                                                                            \
        cudaError_t e__ = (call);                                                   \
        if (e__ != cudaSuccess) {                                                   \
            ckb::set_error("%s failed: %s (%s:%d)", #call, cudaGetErrorString(e__), \
                           __FILE__, __LINE__);                                     \
            return CKKS_B200_ERR_CUDA;                                              \
        }                                                                           \
    } while (0)

#define CKB_REQUIRE(cond, code, ...)   \
    do {                               \
        if (!(cond)) {                 \
            ckb::set_error(__VA_ARGS__); \
            return (code);             \
        }                              \
    } while (0)

// Count of kernels launched by this library in this process.
extern std::atomic<long> g_launches;
inline void count_launch(long n = 1) { g_launches += n; }

// ---------------------------------------------------------------------------
// Programmatic dependent launch, for the chains of short kernels (transforms, level changes, key switching): a
// kernel launched with launch_after() may be scheduled while the kernel before it in the stream is still running.
// It sets up what does not depend on that kernel (indices, constant tables, tensor memory) and calls
// wait_for_previous_kernel() before it touches anything else in global memory; the wait returns once the previous
// kernel has completed and its writes are visible.  The previous kernel opens the door with let_next_kernel_start()
// (without it the dependent is scheduled when the previous kernel ends, as usual); launched the ordinary way, both
// calls pass straight through.  Only kernels that wait may be launched with launch_after().
// ---------------------------------------------------------------------------
#ifdef __CUDACC__
__device__ __forceinline__ void wait_for_previous_kernel() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void let_next_kernel_start() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <class... Params, class... Args>
inline cudaError_t launch_after(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, args...);
}
#endif

// RAII guard: make `device` current for the duration of a call, then restore.
struct DeviceGuard {
    int prev = -1;
    bool ok = true;
    explicit DeviceGuard(int device) {
        if (cudaGetDevice(&prev) != cudaSuccess) { ok = false; return; }
        if (prev != device && cudaSetDevice(device) != cudaSuccess) ok = false;
    }
    ~DeviceGuard() {
        if (prev >= 0) cudaSetDevice(prev);
    }
};

// ---------------------------------------------------------------------------
// Host-side integer helpers (exact, via 128-bit words).
// ---------------------------------------------------------------------------
inline u64 h_mulmod(u64 a, u64 b, u64 q) { return (u64)(((u128)a * b) % q); }
inline u64 h_powmod(u64 a, u64 e, u64 q) {
    u64 r = 1;
    a %= q;
    for (; e; e >>= 1) {
        if (e & 1) r = h_mulmod(r, a, q);
        a = h_mulmod(a, a, q);
    }
    return r;
}
inline u64 h_invmod(u64 a, u64 q) { return h_powmod(a, q - 2, q); }   // q prime
inline u64 h_shoup(u64 x, u64 q) { return (u64)((((u128)x) << 64) / q); }
inline void h_barrett_mu(u64 q, u64* hi, u64* lo) {
    u128 mu = (~(u128)0) / q;   // == floor(2^128/q) for every odd q > 1
    *hi = (u64)(mu >> 64);
    *lo = (u64)mu;
}

// ---------------------------------------------------------------------------
// Device primitives.
// ---------------------------------------------------------------------------
#ifdef __CUDACC__
// x in [0, 2q) -> [0, q)
__device__ __forceinline__ u64 csub(u64 x, u64 q) { return x >= q ? x - q : x; }

// a*w mod q, lazy: result in [0, 2q) for any 64-bit a when ws = floor(w*2^64/q).
__device__ __forceinline__ u64 shoup_lazy(u64 a, u64 w, u64 ws, u64 q) {
    return a * w - __umul64hi(a, ws) * q;
}
// Cheaper lazy product: the quotient estimate keeps three of the four 32x32 partial
// products of a*ws and drops their carries, so it is the exact estimate or up to two less;
// the result lies in [0, 4q) for any 64-bit a.
__device__ __forceinline__ u64 shoup_lazy4(u64 a, u64 w, u64 ws, u64 q) {
    const uint32_t al = (uint32_t)a, ah = (uint32_t)(a >> 32);
    const uint32_t wl = (uint32_t)ws, wh = (uint32_t)(ws >> 32);
    const u64 x = (u64)ah * wl, y = (u64)al * wh;
    const u64 est = (u64)ah * wh + (x >> 32) + (y >> 32);
    return a * w - est * q;
}
__device__ __forceinline__ u64 shoup_mul(u64 a, u64 w, u64 ws, u64 q) {
    return csub(shoup_lazy(a, w, ws, q), q);
}

// (hi:lo) mod q for any 128-bit value, mu = floor(2^128/q) as (mu_hi, mu_lo), q < 2^63.
// Quotient estimate is floor(a*mu/2^128) (low 64 bits), which is the true quotient or
// one less, so a single conditional subtraction finishes.
__device__ __forceinline__ u64 barrett128(u64 lo, u64 hi, u64 q, u64 mu_hi, u64 mu_lo) {
    u64 t0 = __umul64hi(lo, mu_lo);
    u64 m1 = lo * mu_hi, c1 = __umul64hi(lo, mu_hi);
    u64 m2 = hi * mu_lo, c2 = __umul64hi(hi, mu_lo);
    u64 s = t0 + m1;
    u64 carry = s < t0;
    u64 s2 = s + m2;
    carry += s2 < s;
    u64 qhat = c1 + c2 + carry + hi * mu_hi;
    return csub(lo - qhat * q, q);
}

// (hi:lo) += a * b, one carry chain
__device__ __forceinline__ void mac128(u64& lo, u64& hi, u64 a, u64 b) {
    asm("{\n\t"
        "mad.lo.cc.u64 %0, %2, %3, %0;\n\t"
        "madc.hi.u64 %1, %2, %3, %1;\n\t"
        "}"
        : "+l"(lo), "+l"(hi)
        : "l"(a), "l"(b));
}
#endif

}  // namespace ckb
