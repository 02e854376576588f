// The key-switch chain of the reference's CKKS-23 evaluator after modUpQjtoT_23 and the NTT
// over T (Scheme_23::mult_23, src/ckks/include/KeySwitch_23.cuh:192-236):
//
//   external_product_T   (ExternalProduct.cuh:7-97)   digits x key blocks, summed modulo t_k
//   INTT over T          (Context_23.cuh:909-930)     the same transform as everywhere else
//   modUpTtoPQl_23       (BasisConv.cuh:183-248)      T -> [p | q_0..q_l], gamma moduli per block,
//                                                     centred by T/2, IEEE-double overflow count
//   modDownPQltoQl_23    (BasisConv.cuh:251-347)      [p | q] -> q: subtract the p part, times P^-1
//
// Buffer layouts are the reference's.  With R = ceil((p_num+q_num)/gamma) (Ri_blockNum) a "T buffer"
// holds 2 halves (the a and b parts of the key) of R blocks of t_num limbs; the "PQ buffer" re-uses the
// same half stride R*t_num*N and holds limb i of [p | q] at offset i*N inside its half.
#include "context.cuh"

using namespace ckb;

namespace {

constexpr int kThreads = 256;

// out[h][blk][k][x] = sum_i cipher[i][k][x] * swk[h][i][blk][k][x] mod t_k      (external_product_T_kernel)
__global__ void __launch_bounds__(kThreads) external_product_kernel(u64* __restrict__ out, const u64* __restrict__ cipher,
                                                                    const u64* __restrict__ swk, uint32_t N, int t_num, int R,
                                                                    int cipher_blocks, int dnum, const u64* __restrict__ t,
                                                                    const ulonglong2* __restrict__ t_mu) {
    const uint32_t x = blockIdx.x * kThreads + threadIdx.x;
    const int k = blockIdx.y, blk = blockIdx.z;
    let_next_kernel_start();
    if (x >= N) return;
    wait_for_previous_kernel();
    const size_t half_swk = (size_t)R * t_num * dnum * N, half_out = (size_t)R * t_num * N;
    u64 lo0 = 0, hi0 = 0, lo1 = 0, hi1 = 0;
    for (int i = 0; i < cipher_blocks; i++) {
        const u64 ra = cipher[((size_t)i * t_num + k) * N + x];
        const size_t s = ((size_t)i * t_num * R + (size_t)blk * t_num + k) * N + x;
        mac128(lo0, hi0, ra, swk[s]);
        mac128(lo1, hi1, ra, swk[half_swk + s]);
    }
    const ulonglong2 mu = t_mu[k];
    const size_t o = ((size_t)blk * t_num + k) * N + x;
    out[o] = barrett128(lo0, hi0, t[k], mu.x, mu.y);
    out[half_out + o] = barrett128(lo1, hi1, t[k], mu.x, mu.y);
}

struct ModUpTArgs {
    u64* out;
    const u64* in;
    const u64* pq;                 // [p | q] moduli
    const ulonglong2* pq_mu;       // Barrett mu {hi, lo} of [p | q]
    const u64* t;                  // t moduli
    const ulonglong2* t_hat_inv;   // [t_num] {(T/t_i)^-1 mod t_i, shoup}
    const u64* t_hat_mod_r;        // [p_num+q_num][t_num] (T/t_i) mod r
    const u64* half_t;             // [p_num+q_num+t_num] floor(T/2) mod each modulus
    const u64* t_mod_pq;           // [p_num+q_num] T mod r
    uint32_t N;
    int p_num, q_num, t_num, l, gamma, R;
};

// modUpTtoPQl_23_kernel: one thread per (half, block, coefficient); the block's gamma outputs share the rb_i.
template <int TMAX>
__global__ void __launch_bounds__(kThreads) modup_t_kernel(ModUpTArgs P) {
    const uint32_t x = blockIdx.x * kThreads + threadIdx.x;
    const int blk = blockIdx.y, c = blockIdx.z;
    let_next_kernel_start();
    if (x >= P.N) return;
    wait_for_previous_kernel();
    const size_t half = (size_t)P.R * P.t_num * P.N;
    const u64* src = P.in + c * half + (size_t)blk * P.t_num * P.N + x;
    u64 rb[TMAX];
    double vv = 0.0;
#pragma unroll
    for (int i = 0; i < TMAX; i++) {
        rb[i] = 0;
        if (i < P.t_num) {
            const u64 ti = P.t[i];
            const u64 ra = src[(size_t)i * P.N] + P.half_t[P.p_num + P.q_num + i];
            const ulonglong2 w = P.t_hat_inv[i];
            rb[i] = shoup_mul(ra, w.x, w.y, ti);
            vv += __ddiv_rn((double)rb[i], (double)ti);
        }
    }
    const u64 v = (u64)(long long)(int)vv;
    for (int j = 0; j < P.gamma; j++) {
        const int r = j + blk * P.gamma;
        if (r >= P.p_num + P.l + 1) break;
        const u64 ri = P.pq[r];
        u64 lo = 0, hi = 0;
#pragma unroll
        for (int i = 0; i < TMAX; i++)
            if (i < P.t_num) mac128(lo, hi, rb[i], P.t_hat_mod_r[(size_t)r * P.t_num + i]);
        const u64 sub = v * P.t_mod_pq[r];
        hi -= (lo < sub);
        lo -= sub;
        const ulonglong2 mu = P.pq_mu[r];
        u64 res = barrett128(lo, hi, ri, mu.x, mu.y);
        res = csub(res + ri - P.half_t[r], ri);
        P.out[c * half + (size_t)r * P.N + x] = res;
    }
}

struct ModDownArgs {
    u64* out;
    const u64* in;
    const u64* pq;
    const ulonglong2* pq_mu;
    const u64* qinv64;             // floor(2^64/m) of [p | q]
    const ulonglong2* p_hat_inv;   // [p_num] {(P/p_j)^-1 mod p_j, shoup}
    const u64* p_hat_mod_q;        // [q_num][p_num] (P/p_j) mod q_i
    const ulonglong2* p_inv_mod_q; // [q_num] {P^-1 mod q_i, shoup}
    uint32_t N;
    int p_num, q_num, t_num, R;
};

// modDownPQltoQl_23_multi_kernel / _alpha1_multi_kernel: out[c][i][x] = (x_{q_i} - [x_P]_{q_i}) * P^-1 mod q_i,
// where [x_P]_{q_i} is the fast-basis-conversion value of the p part (no overflow correction, as in the reference).
// One thread per coefficient: the p_num products rb_j are formed once and serve every output limb.
template <int PMAX>
__global__ void __launch_bounds__(kThreads) moddown_kernel(ModDownArgs P, int l) {
    const uint32_t x = blockIdx.x * kThreads + threadIdx.x;
    const int c = blockIdx.y;
    let_next_kernel_start();
    if (x >= P.N) return;
    wait_for_previous_kernel();
    const u64* src = P.in + (size_t)c * P.R * P.t_num * P.N + x;
    u64 rb[PMAX];
#pragma unroll
    for (int j = 0; j < PMAX; j++) {
        rb[j] = 0;
        if (j < P.p_num) {
            if (P.p_num == 1) {
                rb[j] = src[0];
            } else {
                const ulonglong2 w = P.p_hat_inv[j];
                rb[j] = shoup_mul(src[(size_t)j * P.N], w.x, w.y, P.pq[j]);
            }
        }
    }
    for (int i = 0; i <= l; i++) {
        const u64 qi = P.pq[P.p_num + i];
        u64 part;
        if (P.p_num == 1) {
            u64 r = rb[0] - __umul64hi(rb[0], P.qinv64[P.p_num + i]) * qi;      // x_p % q_i
            r = csub(r, qi);
            part = csub(r, qi);
        } else {
            u64 lo = 0, hi = 0;
#pragma unroll
            for (int j = 0; j < PMAX; j++)
                if (j < P.p_num) mac128(lo, hi, rb[j], P.p_hat_mod_q[(size_t)i * P.p_num + j]);
            const ulonglong2 mu = P.pq_mu[P.p_num + i];
            part = barrett128(lo, hi, qi, mu.x, mu.y);
        }
        const u64 d = qi - part + src[(size_t)(P.p_num + i) * P.N];       // in (0, 2q)
        const ulonglong2 w = P.p_inv_mod_q[i];
        P.out[((size_t)c * P.q_num + i) * P.N + x] = shoup_mul(d, w.x, w.y, qi);
    }
}

// compute_c0c1c2_kernel (src/ckks/include/poly_arithmetic.cuh:787-818): the three products of a ciphertext
// multiplication per limb, a1*a2, b1*b2 and a1*b2 + a2*b1 (as (a1+b1)(a2+b2) minus the other two), modulo q_i.
__global__ void __launch_bounds__(kThreads) tensor_product_kernel(u64* __restrict__ axbx, u64* __restrict__ axax,
                                                                  u64* __restrict__ bxbx, const u64* __restrict__ c1,
                                                                  const u64* __restrict__ c2, uint32_t N, int stride,
                                                                  const u64* __restrict__ q, const ulonglong2* __restrict__ mu) {
    const uint32_t x = blockIdx.x * kThreads + threadIdx.x;
    const int i = blockIdx.y;
    if (x >= N) return;
    const size_t a = (size_t)i * N + x, b = ((size_t)stride + i) * N + x;
    const u64 a1 = c1[a], b1 = c1[b], a2 = c2[a], b2 = c2[b];
    const u64 qi = q[i];
    const ulonglong2 m = mu[i];
    u64 l1 = 0, h1 = 0, l2 = 0, h2 = 0, l3 = 0, h3 = 0;
    mac128(l1, h1, a1, a2);
    mac128(l2, h2, b1, b2);
    mac128(l3, h3, a1 + b1, a2 + b2);
    h3 -= h1 + (l3 < l1);
    l3 -= l1;
    h3 -= h2 + (l3 < l2);
    l3 -= l2;
    axax[a] = barrett128(l1, h1, qi, m.x, m.y);
    bxbx[a] = barrett128(l2, h2, qi, m.x, m.y);
    axbx[a] = barrett128(l3, h3, qi, m.x, m.y);
}

// cipher_add_axbx_batch_device_kernel (poly_arithmetic.cuh:155-172): a += ax, b += bx per limb.
__global__ void __launch_bounds__(kThreads) add_switched_kernel(u64* __restrict__ cipher, const u64* __restrict__ ax,
                                                                const u64* __restrict__ bx, uint32_t N, int stride,
                                                                const u64* __restrict__ q) {
    const uint32_t x = blockIdx.x * kThreads + threadIdx.x;
    const int i = blockIdx.y;
    if (x >= N) return;
    const size_t a = (size_t)i * N + x, b = ((size_t)stride + i) * N + x;
    const u64 qi = q[i];
    cipher[a] = csub(cipher[a] + ax[a], qi);
    cipher[b] = csub(cipher[b] + bx[a], qi);
}

// sk_and_poly_conjugate_kernel (poly_arithmetic.cuh:666-674): conjugation reverses a polynomial's words in the NTT domain.
__global__ void __launch_bounds__(kThreads) reverse_kernel(u64* __restrict__ out, const u64* __restrict__ in, uint32_t N) {
    const uint32_t x = blockIdx.x * kThreads + threadIdx.x;
    const int i = blockIdx.y;
    if (x >= N) return;
    out[(size_t)i * N + x] = in[(size_t)i * N + (N - 1 - x)];
}

// b half of the switched pair += reversed b of the input (conjugate_23's closing poly_add_batch_device, KeySwitch_23.cuh:469)
__global__ void __launch_bounds__(kThreads) add_reversed_b_kernel(u64* __restrict__ sw, const u64* __restrict__ cipher, uint32_t N,
                                                                  int stride, const u64* __restrict__ q) {
    const uint32_t x = blockIdx.x * kThreads + threadIdx.x;
    const int i = blockIdx.y;
    if (x >= N) return;
    const size_t b = ((size_t)stride + i) * N;
    sw[b + x] = csub(sw[b + x] + cipher[b + (N - 1 - x)], q[i]);
}

// leftRotate_23's last two steps in one pass (KeySwitch_23.cuh:577-580): b added to the switched b half
// (poly_add_batch_device), then both halves permuted in the NTT domain (sk_and_poly_LeftRot_ntt_kernel,
// poly_arithmetic.cuh:581-596): word x holds the value at the odd power 2*bitrev(x)+1 and goes to the position of
// the power pow*(2*bitrev(x)+1) mod 2N.
__global__ void __launch_bounds__(kThreads) rotate_add_kernel(u64* __restrict__ out, const u64* __restrict__ sw,
                                                              const u64* __restrict__ cipher, uint32_t N, int logN, int stride,
                                                              const u64* __restrict__ q, u64 pow) {
    const uint32_t x = blockIdx.x * kThreads + threadIdx.x;
    const int i = blockIdx.y, half = blockIdx.z;
    if (x >= N) return;
    const size_t base = ((size_t)half * stride + i) * N;
    u64 v = sw[base + x];
    if (half == 1) v = csub(v + cipher[base + x], q[i]);
    const u64 odd = 2 * (u64)(__brev(x) >> (32 - logN)) + 1;
    const uint32_t t = (uint32_t)(((pow * odd) & (2 * (u64)N - 1)) - 1) >> 1;
    out[base + (__brev(t) >> (32 - logN))] = v;
}

int check_chain(ckks_b200_context* c, int l, int gamma) {
    CKB_REQUIRE(c != nullptr, CKKS_B200_ERR_ARG, "null argument");
    CKB_REQUIRE(c->t_num > 0 && c->p_num > 0, CKKS_B200_ERR_ARG, "the context has no T basis or no special primes");
    CKB_REQUIRE(l >= 0 && l < c->q_num, CKKS_B200_ERR_ARG, "level %d outside [0,%d)", l, c->q_num);
    CKB_REQUIRE(gamma >= 1, CKKS_B200_ERR_ARG, "gamma must be positive");
    CKB_REQUIRE(c->chain_ok, CKKS_B200_ERR_UNSUPPORTED, "the key-switch chain needs every modulus below 2^62");
    return CKKS_B200_OK;
}

}  // namespace

extern "C" int ckks_b200_external_product_t(ckks_b200_context* c, uint64_t* d_out, const uint64_t* d_cipher_t,
                                            const uint64_t* d_swk, int l, int gamma, void* stream) {
    int rc = check_chain(c, l, gamma);
    if (rc) return rc;
    CKB_REQUIRE(d_out && d_cipher_t && d_swk, CKKS_B200_ERR_ARG, "null argument");
    DeviceGuard guard(c->device);
    CKB_REQUIRE(guard.ok, CKKS_B200_ERR_CUDA, "cudaSetDevice(%d) failed", c->device);
    const int R = (c->p_num + c->q_num + gamma - 1) / gamma;
    const int cipher_blocks = (l + 1 + c->p_num - 1) / c->p_num;
    const int blocks = (c->p_num + l + 1 + gamma - 1) / gamma;
    const int dnum = c->q_num / c->p_num;
    dim3 grid((c->N + kThreads - 1) / kThreads, c->t_num, blocks);
    CKB_CUDA(launch_after(external_product_kernel, grid, dim3(kThreads), 0, (cudaStream_t)stream, (u64*)d_out, (const u64*)d_cipher_t,
                          (const u64*)d_swk, c->N, c->t_num, R, cipher_blocks, dnum, c->d_moduli + c->p_num + c->q_num, c->d_t_mu));
    count_launch();
    CKB_CUDA(cudaGetLastError());
    return CKKS_B200_OK;
}

extern "C" int ckks_b200_ntt_inverse_ext(ckks_b200_context* c, uint64_t* d_data, int l, int gamma, void* stream) {
    int rc = check_chain(c, l, gamma);
    if (rc) return rc;
    const int R = (c->p_num + c->q_num + gamma - 1) / gamma;
    const int blocks = (c->p_num + l + 1 + gamma - 1) / gamma;
    for (int h = 0; h < 2 && !rc; h++)
        rc = ckks_b200_ntt_inverse(c, d_data + (size_t)h * R * c->t_num * c->N, 0, c->p_num + c->q_num, blocks, c->t_num,
                                   c->t_num, stream);
    return rc;
}

extern "C" int ckks_b200_modup_t_to_pql(ckks_b200_context* c, uint64_t* d_out, const uint64_t* d_in, int l, int gamma,
                                        int batch, void* stream) {
    int rc = check_chain(c, l, gamma);
    if (rc) return rc;
    CKB_REQUIRE(d_out && d_in && batch >= 0 && batch <= 65535, CKKS_B200_ERR_ARG, "null argument or bad batch");
    CKB_REQUIRE(c->t_num <= 16, CKKS_B200_ERR_UNSUPPORTED, "t_num=%d exceeds 16", c->t_num);
    if (batch == 0) return CKKS_B200_OK;
    DeviceGuard guard(c->device);
    CKB_REQUIRE(guard.ok, CKKS_B200_ERR_CUDA, "cudaSetDevice(%d) failed", c->device);
    // the tensor-core contraction where this gamma's tables qualify (the kernel choice follows ModUp's), else CUDA cores
    rc = build_tpq_tables(c, gamma);
    if (rc) return rc;
    CKB_REQUIRE(c->modup_algo != CKKS_B200_MODUP_TENSOR || modup_t_tensor_ok(c, gamma), CKKS_B200_ERR_UNSUPPORTED,
                "the T -> [p | q] tables of gamma=%d do not qualify for the tensor-core conversion", gamma);
    if (c->modup_algo != CKKS_B200_MODUP_SIMT && modup_t_tensor_ok(c, gamma))
        return modup_t_tensor(c, (u64*)d_out, (const u64*)d_in, l, gamma, batch, (cudaStream_t)stream);
    ModUpTArgs P;
    P.out = (u64*)d_out;
    P.in = (const u64*)d_in;
    P.pq = c->d_moduli;
    P.pq_mu = c->d_pq_mu;
    P.t = c->d_moduli + c->p_num + c->q_num;
    P.t_hat_inv = c->d_t_hat_inv;
    P.t_hat_mod_r = c->d_t_hat_mod_r;
    P.half_t = c->d_half_t;
    P.t_mod_pq = c->d_t_mod_pq;
    P.N = c->N;
    P.p_num = c->p_num;
    P.q_num = c->q_num;
    P.t_num = c->t_num;
    P.l = l;
    P.gamma = gamma;
    P.R = (c->p_num + c->q_num + gamma - 1) / gamma;
    const int blocks = (c->p_num + l + 1 + gamma - 1) / gamma;
    dim3 grid((c->N + kThreads - 1) / kThreads, blocks, batch);
    if (c->t_num <= 4) CKB_CUDA(launch_after(modup_t_kernel<4>, grid, dim3(kThreads), 0, (cudaStream_t)stream, P));
    else if (c->t_num <= 8) CKB_CUDA(launch_after(modup_t_kernel<8>, grid, dim3(kThreads), 0, (cudaStream_t)stream, P));
    else CKB_CUDA(launch_after(modup_t_kernel<16>, grid, dim3(kThreads), 0, (cudaStream_t)stream, P));
    count_launch();
    CKB_CUDA(cudaGetLastError());
    return CKKS_B200_OK;
}

extern "C" int ckks_b200_moddown_pql_to_ql(ckks_b200_context* c, uint64_t* d_out, const uint64_t* d_in, int l, int gamma,
                                           int batch, void* stream) {
    int rc = check_chain(c, l, gamma);
    if (rc) return rc;
    CKB_REQUIRE(d_out && d_in && batch >= 0 && batch <= 65535, CKKS_B200_ERR_ARG, "null argument or bad batch");
    if (batch == 0) return CKKS_B200_OK;
    DeviceGuard guard(c->device);
    CKB_REQUIRE(guard.ok, CKKS_B200_ERR_CUDA, "cudaSetDevice(%d) failed", c->device);
    ModDownArgs P;
    P.out = (u64*)d_out;
    P.in = (const u64*)d_in;
    P.pq = c->d_moduli;
    P.pq_mu = c->d_pq_mu;
    P.qinv64 = c->d_qinv64;
    P.p_hat_inv = c->d_p_hat_inv;
    P.p_hat_mod_q = c->d_p_hat_mod_q;
    P.p_inv_mod_q = c->d_p_inv_mod_q;
    P.N = c->N;
    P.p_num = c->p_num;
    P.q_num = c->q_num;
    P.t_num = c->t_num;
    P.R = (c->p_num + c->q_num + gamma - 1) / gamma;
    dim3 grid((c->N + kThreads - 1) / kThreads, batch);
    if (c->p_num <= 4) CKB_CUDA(launch_after(moddown_kernel<4>, grid, dim3(kThreads), 0, (cudaStream_t)stream, P, l));
    else if (c->p_num <= 8) CKB_CUDA(launch_after(moddown_kernel<8>, grid, dim3(kThreads), 0, (cudaStream_t)stream, P, l));
    else CKB_CUDA(launch_after(moddown_kernel<16>, grid, dim3(kThreads), 0, (cudaStream_t)stream, P, l));
    count_launch();
    CKB_CUDA(cudaGetLastError());
    return CKKS_B200_OK;
}

// The whole chain on one polynomial: d_in holds limbs 0..l (NTT domain, stride L+1 limbs is not needed: [l+1][N]
// contiguous from limb 0); d_out receives the two switched polynomials, [2][q_num][N], NTT domain, limbs 0..l.
extern "C" int ckks_b200_keyswitch(ckks_b200_context* c, uint64_t* d_out, const uint64_t* d_in, const uint64_t* d_swk,
                                   int l, int gamma, void* stream) {
    int rc = check_chain(c, l, gamma);
    if (rc) return rc;
    CKB_REQUIRE(d_out && d_in && d_swk, CKKS_B200_ERR_ARG, "null argument");
    DeviceGuard guard(c->device);
    CKB_REQUIRE(guard.ok, CKKS_B200_ERR_CUDA, "cudaSetDevice(%d) failed", c->device);
    cudaStream_t st = (cudaStream_t)stream;
    const int K = c->p_num, T = c->t_num;
    const int R = (K + c->q_num + gamma - 1) / gamma;
    const int cipher_blocks = (l + 1 + K - 1) / K;
    const size_t n = c->N;
    // workspace: coefficients of the input [q_num][N] | its T digits [blocks_max][T][N] | T buffer | PQ buffer
    const size_t w_in = (size_t)c->q_num * n, w_dig = (size_t)c->blocks_max * T * n, w_t = (size_t)2 * R * T * n;
    rc = ensure_buf(&c->ks_buf, &c->ks_cap, w_in + w_dig + 2 * w_t);
    if (rc) return rc;
    u64* coef = c->ks_buf;
    u64* dig = coef + w_in;
    u64* tbuf = dig + w_dig;
    u64* pqbuf = tbuf + w_t;
    CKB_CUDA(cudaMemcpyAsync(coef, d_in, (size_t)(l + 1) * n * 8, cudaMemcpyDeviceToDevice, st));
    rc = ckks_b200_ntt_inverse(c, (uint64_t*)coef, 0, K, 1, l + 1, c->q_num, stream);
    if (!rc) rc = ckks_b200_modup_qj_to_t(c, (uint64_t*)dig, (const uint64_t*)coef, l, 1, stream);
    if (!rc) rc = ckks_b200_ntt_forward(c, (uint64_t*)dig, 0, K + c->q_num, cipher_blocks, T, T, stream);
    if (!rc) rc = ckks_b200_external_product_t(c, (uint64_t*)tbuf, (const uint64_t*)dig, d_swk, l, gamma, stream);
    if (!rc) rc = ckks_b200_ntt_inverse_ext(c, (uint64_t*)tbuf, l, gamma, stream);
    if (!rc) rc = ckks_b200_modup_t_to_pql(c, (uint64_t*)pqbuf, (const uint64_t*)tbuf, l, gamma, 2, stream);
    if (!rc) rc = ckks_b200_moddown_pql_to_ql(c, d_out, (const uint64_t*)pqbuf, l, gamma, 2, stream);
    if (!rc) rc = ckks_b200_ntt_forward(c, d_out, 0, K, 2, l + 1, c->q_num, stream);
    return rc;
}

// Scheme_23::mult_23 (src/ckks/include/KeySwitch_23.cuh:192-236): d_res = d_c1 * d_c2 relinearised with the key
// d_rlk.  All three are Ciphertext buffers, a limbs then b limbs, each [q_num][N], NTT domain, level l >= 1 as in the
// reference (its level-0 and missing-key cases are the caller's, :194-201).  d_res may be one of the operands.
extern "C" int ckks_b200_mult(ckks_b200_context* c, uint64_t* d_res, const uint64_t* d_c1, const uint64_t* d_c2,
                              const uint64_t* d_rlk, int l, int gamma, void* stream) {
    int rc = check_chain(c, l, gamma);
    if (rc) return rc;
    CKB_REQUIRE(d_res && d_c1 && d_c2 && d_rlk, CKKS_B200_ERR_ARG, "null argument");
    DeviceGuard guard(c->device);
    CKB_REQUIRE(guard.ok, CKKS_B200_ERR_CUDA, "cudaSetDevice(%d) failed", c->device);
    cudaStream_t st = (cudaStream_t)stream;
    const size_t n = c->N, limb_words = (size_t)c->q_num * n;
    rc = ensure_buf(&c->mul_buf, &c->mul_cap, 5 * limb_words);
    if (rc) return rc;
    u64 *axbx = c->mul_buf, *axax = axbx + limb_words, *bxbx = axax + limb_words, *sw = bxbx + limb_words;
    const u64* q = c->d_moduli + c->p_num;
    dim3 grid((c->N + kThreads - 1) / kThreads, l + 1);
    tensor_product_kernel<<<grid, kThreads, 0, st>>>(axbx, axax, bxbx, (const u64*)d_c1, (const u64*)d_c2, c->N, c->q_num, q,
                                                     c->d_pq_mu + c->p_num);
    count_launch();
    CKB_CUDA(cudaGetLastError());
    rc = ckks_b200_keyswitch(c, (uint64_t*)sw, (const uint64_t*)axax, d_rlk, l, gamma, stream);
    if (rc) return rc;
    add_switched_kernel<<<grid, kThreads, 0, st>>>(sw, axbx, bxbx, c->N, c->q_num, q);
    count_launch();
    CKB_CUDA(cudaGetLastError());
    // the switched pair lives in the workspace so that d_res may alias an operand; only limbs 0..l are copied
    CKB_CUDA(cudaMemcpy2DAsync(d_res, limb_words * 8, sw, limb_words * 8, (size_t)(l + 1) * n * 8, 2, cudaMemcpyDeviceToDevice, st));
    return CKKS_B200_OK;
}

// Scheme_23::conjugate_23 / conjugateAndEqual_23 (KeySwitch_23.cuh:433-507): a and b reversed in the NTT domain, the
// chain on the reversed a with the conjugation key, the reversed b added to the b half.  d_res may be d_cipher.
extern "C" int ckks_b200_conjugate(ckks_b200_context* c, uint64_t* d_res, const uint64_t* d_cipher, const uint64_t* d_conj_key,
                                   int l, int gamma, void* stream) {
    int rc = check_chain(c, l, gamma);
    if (rc) return rc;
    CKB_REQUIRE(d_res && d_cipher && d_conj_key, CKKS_B200_ERR_ARG, "null argument");
    DeviceGuard guard(c->device);
    CKB_REQUIRE(guard.ok, CKKS_B200_ERR_CUDA, "cudaSetDevice(%d) failed", c->device);
    cudaStream_t st = (cudaStream_t)stream;
    const size_t n = c->N, limb_words = (size_t)c->q_num * n;
    rc = ensure_buf(&c->mul_buf, &c->mul_cap, 5 * limb_words);
    if (rc) return rc;
    u64 *arev = c->mul_buf, *sw = c->mul_buf + 3 * limb_words;
    const u64* q = c->d_moduli + c->p_num;
    dim3 grid((c->N + kThreads - 1) / kThreads, l + 1);
    reverse_kernel<<<grid, kThreads, 0, st>>>(arev, (const u64*)d_cipher, c->N);
    count_launch();
    CKB_CUDA(cudaGetLastError());
    rc = ckks_b200_keyswitch(c, (uint64_t*)sw, (const uint64_t*)arev, d_conj_key, l, gamma, stream);
    if (rc) return rc;
    add_reversed_b_kernel<<<grid, kThreads, 0, st>>>(sw, (const u64*)d_cipher, c->N, c->q_num, q);
    count_launch();
    CKB_CUDA(cudaGetLastError());
    CKB_CUDA(cudaMemcpy2DAsync(d_res, limb_words * 8, sw, limb_words * 8, (size_t)(l + 1) * n * 8, 2, cudaMemcpyDeviceToDevice, st));
    return CKKS_B200_OK;
}

// Scheme_23::leftRotate_23 / leftRotateAndEqual_23 (KeySwitch_23.cuh:509-581): the chain on a with the key of this
// rotation, b added, both halves permuted by the Galois element 5^(N/2 - rot_slots) mod 2N.  d_res may be d_cipher.
extern "C" int ckks_b200_rotate(ckks_b200_context* c, uint64_t* d_res, const uint64_t* d_cipher, const uint64_t* d_rot_key,
                                long rot_slots, int l, int gamma, void* stream) {
    int rc = check_chain(c, l, gamma);
    if (rc) return rc;
    CKB_REQUIRE(d_res && d_cipher && d_rot_key, CKKS_B200_ERR_ARG, "null argument");
    // the reference indexes rotGroups[N/2 - rot_slots], an array of N/2 entries (Context_23.cuh:650-656)
    CKB_REQUIRE(rot_slots >= 1 && rot_slots <= (long)(c->N / 2), CKKS_B200_ERR_ARG, "rotation by %ld slots outside [1,%u]",
                rot_slots, c->N / 2);
    DeviceGuard guard(c->device);
    CKB_REQUIRE(guard.ok, CKKS_B200_ERR_CUDA, "cudaSetDevice(%d) failed", c->device);
    cudaStream_t st = (cudaStream_t)stream;
    const size_t n = c->N, limb_words = (size_t)c->q_num * n;
    rc = ensure_buf(&c->mul_buf, &c->mul_cap, 5 * limb_words);
    if (rc) return rc;
    u64 *out = c->mul_buf, *sw = c->mul_buf + 3 * limb_words;
    u64 pow = 1;
    for (long e = 0; e < (long)(c->N / 2) - rot_slots; e++) pow = pow * 5 % (2 * (u64)c->N);
    rc = ckks_b200_keyswitch(c, (uint64_t*)sw, d_cipher, d_rot_key, l, gamma, stream);
    if (rc) return rc;
    int logN = 0;
    while ((1u << logN) < c->N) logN++;
    dim3 grid((c->N + kThreads - 1) / kThreads, l + 1, 2);
    rotate_add_kernel<<<grid, kThreads, 0, st>>>(out, sw, (const u64*)d_cipher, c->N, logN, c->q_num, c->d_moduli + c->p_num, pow);
    count_launch();
    CKB_CUDA(cudaGetLastError());
    CKB_CUDA(cudaMemcpy2DAsync(d_res, limb_words * 8, out, limb_words * 8, (size_t)(l + 1) * n * 8, 2, cudaMemcpyDeviceToDevice, st));
    return CKKS_B200_OK;
}
