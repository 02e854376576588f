// The two level-changing steps either side of the PCMM in the reference's BERT pipeline, both
// small INTT -> elementwise -> NTT sandwiches over a Ciphertext buffer [2 polys][L+1 limbs][N]:
//
//   Scheme_23::rescaleAndEqual (src/ckks/include/Scheme_23.cuh:339-385): divide by the last limb.
//     INTT of limb l; c_i = (x_l mod q_i) for i < l; NTT of the c_i; x_i <- (x_i - c_i) * q_l^-1 mod q_i.
//   Bootstrapper::modUpQ0toQL (bootstrapping/Bootstrapper.cuh:192-209, Bootstrapping.cuh:6-23): raise a
//     level-0 ciphertext to target_level.  INTT of limb 0; limb i+1 <- centred lift of x_0 (with the
//     reference's + q_i * scale_up) reduced modulo q_{i+1}; NTT of limbs 0..target_level.
//
// The elementwise kernels process both polynomials and every target limb of one coefficient slice
// per thread block, so the source limb is read from HBM once and served from L1/L2 afterwards.
#include "context.cuh"

using namespace ckb;

namespace {

constexpr int kThreads = 256;

// x mod q for any 64-bit x: quotient estimate with floor(2^64/q), at most two corrections.
__device__ __forceinline__ u64 reduce64(u64 x, u64 q, u64 qinv64) {
    u64 r = x - __umul64hi(x, qinv64) * q;
    r = csub(r, q);
    return csub(r, q);
}

// buf[c][i][x] = cipher[c][l][x] mod q_i, i < l   (mod_to_qi, Scheme_23.cuh:356-366).  The reference
// subtracts q at most once after its estimate and may leave a value in [q, 2q); what it then feeds to
// the NTT is that value's residue, so the canonical residue written here gives the same transform.
__global__ void __launch_bounds__(kThreads) rescale_spread_kernel(u64* __restrict__ buf, const u64* __restrict__ cipher,
                                                                  uint32_t N, int stride, int l, const u64* __restrict__ q,
                                                                  const u64* __restrict__ qinv64) {
    const uint32_t x = blockIdx.x * kThreads + threadIdx.x;
    const int c = blockIdx.y;
    let_next_kernel_start();
    if (x >= N) return;
    wait_for_previous_kernel();
    const u64 v = cipher[((size_t)c * stride + l) * N + x];
    for (int i = 0; i < l; i++) buf[((size_t)c * stride + i) * N + x] = reduce64(v, q[i], qinv64[i]);
}

// cipher[c][i][x] = (cipher[c][i][x] - buf[c][i][x]) * q_l^-1 mod q_i   (rescaleAndEqual_new_kernel, :339-354)
__global__ void __launch_bounds__(kThreads) rescale_combine_kernel(u64* __restrict__ cipher, const u64* __restrict__ buf,
                                                                   uint32_t N, int stride, int l, const u64* __restrict__ q,
                                                                   const ulonglong2* __restrict__ qlinv) {
    const uint32_t x = blockIdx.x * kThreads + threadIdx.x;
    const int i = blockIdx.y, c = blockIdx.z;
    let_next_kernel_start();
    if (x >= N) return;
    wait_for_previous_kernel();
    const size_t idx = ((size_t)c * stride + i) * N + x;
    const u64 qi = q[i];
    const u64 d = csub(cipher[idx] + qi - buf[idx], qi);          // both operands are canonical
    const ulonglong2 w = qlinv[i];
    cipher[idx] = shoup_mul(d, w.x, w.y, qi);
}

// limb i+1 of both polynomials from the coefficients in limb 0   (modUpQ0toQL_kernel, Bootstrapping.cuh:6-23).
// The reference's mixed signed/unsigned expression is 64-bit unsigned arithmetic throughout: for
// x > q0/2 the value is x - q0 + q_i*scale_up modulo 2^64, then modulo q_i.
__global__ void __launch_bounds__(kThreads) modup_q0_kernel(u64* __restrict__ cipher, uint32_t N, int stride, int target_level,
                                                            const u64* __restrict__ q, const u64* __restrict__ qinv64,
                                                            u64 scale_up) {
    const uint32_t x = blockIdx.x * kThreads + threadIdx.x;
    const int c = blockIdx.y;
    let_next_kernel_start();
    if (x >= N) return;
    wait_for_previous_kernel();
    const u64 q0 = q[0];
    const u64 v = cipher[(size_t)c * stride * N + x];
    for (int i = 0; i < target_level; i++) {
        const u64 qi = q[i + 1];
        const u64 t = v > q0 / 2 ? v - q0 + qi * scale_up : v;
        cipher[((size_t)c * stride + i + 1) * N + x] = reduce64(t, qi, qinv64[i + 1]);
    }
}

}  // namespace

// `count` ciphertexts laid out one after another ([count][2][L+1][N]) go through every stage together: the
// transforms see 2*count polynomials, the elementwise kernels 2*count slices.  One ciphertext alone leaves most
// of the GPU idle (its inverse transform is two limb-polynomials), so callers that keep their ciphertexts in one
// pool should use the batched forms.
extern "C" int ckks_b200_rescale_batch(ckks_b200_context* c, uint64_t* d_ciphers, int count, int L, int l, void* stream) {
    CKB_REQUIRE(c && d_ciphers, CKKS_B200_ERR_ARG, "null argument");
    CKB_REQUIRE(count >= 1 && count <= 16384, CKKS_B200_ERR_ARG, "ciphertext count %d outside [1,16384]", count);
    CKB_REQUIRE(L >= 1 && L + 1 <= c->q_num, CKKS_B200_ERR_ARG, "L=%d needs %d q moduli, the context has %d", L, L + 1,
                c->q_num);
    CKB_REQUIRE(l >= 1 && l <= L, CKKS_B200_ERR_ARG, "level %d outside [1,%d]: nothing to rescale by", l, L);
    DeviceGuard guard(c->device);
    CKB_REQUIRE(guard.ok, CKKS_B200_ERR_CUDA, "cudaSetDevice(%d) failed", c->device);
    cudaStream_t st = (cudaStream_t)stream;
    const int K = c->p_num, stride = L + 1, polys = 2 * count;
    int rc = ensure_buf(&c->resc_buf, &c->resc_cap, (size_t)polys * stride * c->N);
    if (rc) return rc;
    rc = ckks_b200_ntt_inverse(c, d_ciphers, l, K + l, polys, 1, stride, stream);
    if (rc) return rc;
    const u64* q = c->d_moduli + K;
    dim3 g1((c->N + kThreads - 1) / kThreads, polys);
    CKB_CUDA(launch_after(rescale_spread_kernel, g1, dim3(kThreads), 0, st, c->resc_buf, (const u64*)d_ciphers, (uint32_t)c->N, stride, l, q,
                          (const u64*)(c->d_qinv64 + K)));
    count_launch();
    CKB_CUDA(cudaGetLastError());
    rc = ckks_b200_ntt_forward(c, (uint64_t*)c->resc_buf, 0, K, polys, l, stride, stream);
    if (rc) return rc;
    dim3 g2((c->N + kThreads - 1) / kThreads, l, polys);
    CKB_CUDA(launch_after(rescale_combine_kernel, g2, dim3(kThreads), 0, st, (u64*)d_ciphers, c->resc_buf, c->N, stride, l, q,
                          c->d_qlinv + (size_t)l * c->q_num));
    count_launch();
    CKB_CUDA(cudaGetLastError());
    return CKKS_B200_OK;
}

extern "C" int ckks_b200_rescale(ckks_b200_context* c, uint64_t* d_cipher, int L, int l, void* stream) {
    return ckks_b200_rescale_batch(c, d_cipher, 1, L, l, stream);
}

extern "C" int ckks_b200_modup_q0_to_ql_batch(ckks_b200_context* c, uint64_t* d_ciphers, int count, int L, int target_level,
                                              long long scale_up, void* stream) {
    CKB_REQUIRE(c && d_ciphers, CKKS_B200_ERR_ARG, "null argument");
    CKB_REQUIRE(count >= 1 && count <= 16384, CKKS_B200_ERR_ARG, "ciphertext count %d outside [1,16384]", count);
    CKB_REQUIRE(L >= 1 && L + 1 <= c->q_num, CKKS_B200_ERR_ARG, "L=%d needs %d q moduli, the context has %d", L, L + 1,
                c->q_num);
    CKB_REQUIRE(target_level >= 1 && target_level <= L, CKKS_B200_ERR_ARG, "target level %d outside [1,%d]", target_level, L);
    DeviceGuard guard(c->device);
    CKB_REQUIRE(guard.ok, CKKS_B200_ERR_CUDA, "cudaSetDevice(%d) failed", c->device);
    cudaStream_t st = (cudaStream_t)stream;
    const int K = c->p_num, stride = L + 1, polys = 2 * count;
    int rc = ckks_b200_ntt_inverse(c, d_ciphers, 0, K, polys, 1, stride, stream);
    if (rc) return rc;
    dim3 g((c->N + kThreads - 1) / kThreads, polys);
    CKB_CUDA(launch_after(modup_q0_kernel, g, dim3(kThreads), 0, st, (u64*)d_ciphers, c->N, stride, target_level, c->d_moduli + K,
                          c->d_qinv64 + K, (u64)scale_up));
    count_launch();
    CKB_CUDA(cudaGetLastError());
    return ckks_b200_ntt_forward(c, d_ciphers, 0, K, polys, target_level + 1, stride, stream);
}

extern "C" int ckks_b200_modup_q0_to_ql(ckks_b200_context* c, uint64_t* d_cipher, int L, int target_level,
                                        long long scale_up, void* stream) {
    return ckks_b200_modup_q0_to_ql_batch(c, d_cipher, 1, L, target_level, scale_up, stream);
}
