// The 64-bit CUDA-core multiply of the PCMM, shared by the handle-based entry point (pcmm.cu) and the
// allocation-free one (pcmm_static.cu): 64x64 output tile per CTA, 4x4 outputs per thread, 128-bit accumulators,
// limbs last to first with the rescale by the last limb fused, as pcmm_cuda_core_kernel of the reference does it
// (src/ckks/include/pcmm/PPMM_kernel.cuh:12-31 for the product and its sign rule, :213-249 for the limb order, the
// Barrett reduction and the rescale).
#pragma once
#include "pcmm.cuh"

namespace ckb {

constexpr int TS = 64, TK = 16;

// Operands: scaled weights [M][K]; ciphertext n through a table of pointers, or at base + n * stride words.
struct SimtOperands {
    const long long* w;
    const u64* const* table;
    const u64* base;
    size_t stride;
};

struct SimtLimb {
    u64 q, mu_hi, mu_lo, inv, inv_shoup;
};
// Per-limb constants read from the handle's table in global memory ...
struct SimtLimbsPtr {
    const PcmmLimb* p;
    __device__ __forceinline__ SimtLimb get(int i) const {
        const PcmmLimb L = p[i];
        return SimtLimb{L.q, L.mu_hi, L.mu_lo, L.inv, L.inv_shoup};
    }
};
// ... or travelling by value as a kernel argument (no device memory needed for them).
constexpr int kSimtMaxLimbsByValue = 24;
struct SimtLimbsVal {
    SimtLimb l[kSimtMaxLimbsByValue];
    __device__ __forceinline__ SimtLimb get(int i) const { return l[i]; }
};

template <class LIMBS>
__global__ void __launch_bounds__(256) pcmm_simt_kernel(SimtOperands ops, u64* __restrict__ out, LIMBS limbs, int M, int K,
                                                        long C, int limb_num, long col_begin, long col_end) {
    __shared__ u64 As[TK][TS + 1];
    __shared__ u64 Xs[TK][TS];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const long c0 = col_begin + (long)blockIdx.x * TS;
    const int m0 = blockIdx.y * TS;
    u64 last[4][4];

    for (int i = limb_num - 1; i >= 0; i--) {
        const SimtLimb L = limbs.get(i);
        u64 lo[4][4], hi[4][4];
#pragma unroll
        for (int r = 0; r < 4; r++)
#pragma unroll
            for (int s = 0; s < 4; s++) lo[r][s] = hi[r][s] = 0;

        for (int k0 = 0; k0 < K; k0 += TK) {
            __syncthreads();
            for (int e = threadIdx.x; e < TS * TK; e += 256) {
                int kk = e % TK, mm = e / TK;
                long long wv = (m0 + mm < M && k0 + kk < K) ? ops.w[(size_t)(m0 + mm) * K + k0 + kk] : 0;
                // a = w > 0 ? w : q + w   (PPMM_kernel.cuh:23-25); padding contributes q*0
                As[kk][mm] = wv > 0 ? (u64)wv : L.q + (u64)wv;
            }
            for (int e = threadIdx.x; e < TS * TK; e += 256) {
                int cc = e % TS, kk = e / TS;
                u64 xv = 0;
                if (k0 + kk < K && c0 + cc < col_end) {
                    const u64* ct = ops.table ? ops.table[k0 + kk] : ops.base + (size_t)(k0 + kk) * ops.stride;
                    xv = ct[(size_t)i * C + c0 + cc];
                }
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

}  // namespace ckb
