// ModUp of Q-digits to the auxiliary basis T (fast basis conversion with the
// floating-point overflow count), the operation of Context_23::modUpQjtoT_23 in the
// reference (src/ckks/include/BasisConv.cuh:84-179).
//
// This file holds the CUDA-core kernel and the dispatch; levels whose tables qualify go to the
// tensor-core kernel in modup_umma.cu.  In the CUDA-core kernel
// one thread converts one coefficient of one digit: it reads the alpha residues of the
// digit (coalesced across the warp, one limb at a time), forms rb_j = x_j * (Qblk/q_j)^-1
// mod q_j and the overflow count v = trunc(sum_j rb_j / q_j) in IEEE double precision in
// limb order, and for every target modulus t_k accumulates sum_j rb_j * (Qblk/q_j mod t_k)
// in 128 bits, subtracts v * (Qblk mod t_k) and reduces.  Tables sit in shared memory.
// The kernel is a pure stream over HBM: (alpha + t_num) words per thread.
#include "context.cuh"

using namespace ckb;

namespace {

constexpr int kMaxAlpha = 16;
constexpr int kThreads = 128;

struct ModUpArgs {
    u64* out;
    const u64* in;
    const u64* q;                 // q moduli [q_num]
    const u64* t;                 // t moduli [t_num]
    const ulonglong2* t_mu;       // [t_num] {hi, lo}
    const ulonglong2* hat_inv;    // [blocks_max*alpha] for this level
    const u64* hat_mod_t;         // [blocks_max][t_num][alpha] for this level
    const u64* blk_mod_t;         // [blocks_max][t_num] for this level
    uint32_t N;
    int q_num, t_num, alpha, l, blocks;
};

template <int ALPHA>
__global__ void __launch_bounds__(kThreads) modup_kernel(ModUpArgs P) {
    extern __shared__ u64 sm[];
    const int blk = blockIdx.y, bt = blockIdx.z;
    const int cnt = min(P.alpha, P.l + 1 - blk * P.alpha);
    u64* s_hat = sm;                          // [t_num][alpha]
    u64* s_blk = sm + P.t_num * P.alpha;      // [t_num]
    for (int i = threadIdx.x; i < P.t_num * P.alpha; i += kThreads)
        s_hat[i] = P.hat_mod_t[(size_t)blk * P.t_num * P.alpha + i];
    for (int i = threadIdx.x; i < P.t_num; i += kThreads) s_blk[i] = P.blk_mod_t[blk * P.t_num + i];
    __syncthreads();

    const uint32_t x = blockIdx.x * kThreads + threadIdx.x;
    if (x >= P.N) return;
    const u64* src = P.in + ((size_t)bt * P.q_num + (size_t)blk * P.alpha) * P.N + x;
    u64 rb[ALPHA];
    double vv = 0.0;
#pragma unroll
    for (int j = 0; j < ALPHA; j++) {
        rb[j] = 0;
        if (j < cnt) {
            const u64 qj = P.q[blk * P.alpha + j];
            const ulonglong2 hi = P.hat_inv[blk * P.alpha + j];
            rb[j] = shoup_mul(src[(size_t)j * P.N], hi.x, hi.y, qj);
            vv += __ddiv_rn((double)rb[j], (double)qj);
        }
    }
    const u64 v = (u64)(long long)(int)vv;
    u64* dst = P.out + (((size_t)bt * P.blocks + blk) * P.t_num) * P.N + x;
    for (int k = 0; k < P.t_num; k++) {
        u64 lo = 0, hi = 0;
#pragma unroll
        for (int j = 0; j < ALPHA; j++)
            if (j < cnt) mac128(lo, hi, rb[j], s_hat[k * P.alpha + j]);
        const u64 sub = v * s_blk[k];
        hi -= (lo < sub);
        lo -= sub;
        const ulonglong2 mu = P.t_mu[k];
        dst[(size_t)k * P.N] = barrett128(lo, hi, P.t[k], mu.x, mu.y);
    }
}

int run_modup(ckks_b200_context* c, u64* d_out, const u64* d_in, int l, int batch, cudaStream_t st) {
    CKB_REQUIRE(c && d_out && d_in, CKKS_B200_ERR_ARG, "null argument");
    CKB_REQUIRE(c->t_num > 0 && c->p_num > 0, CKKS_B200_ERR_ARG,
                "the context has no T basis or no digit size (p_num)");
    CKB_REQUIRE(l >= 0 && l < c->q_num, CKKS_B200_ERR_ARG, "level %d outside [0,%d)", l, c->q_num);
    CKB_REQUIRE(batch >= 0 && batch <= 65535, CKKS_B200_ERR_ARG, "batch %d outside [0,65535]", batch);
    if (batch == 0) return CKKS_B200_OK;
    DeviceGuard guard(c->device);
    CKB_REQUIRE(guard.ok, CKKS_B200_ERR_CUDA, "cudaSetDevice(%d) failed", c->device);
    CKB_REQUIRE(c->modup_algo != CKKS_B200_MODUP_TENSOR || modup_tensor_ok(c, l), CKKS_B200_ERR_UNSUPPORTED,
                "level %d does not qualify for the tensor-core ModUp (moduli outside [2^40,2^62), more than 16 of them, "
                "or tables on which the reference's 128-bit difference could wrap)", l);
    if (c->modup_algo != CKKS_B200_MODUP_SIMT && modup_tensor_ok(c, l)) return modup_tensor(c, d_out, d_in, l, batch, st);
    const int A = c->alpha, B = c->blocks_max, T = c->t_num;
    ModUpArgs P;
    P.out = d_out;
    P.in = d_in;
    P.q = c->d_moduli + c->p_num;
    P.t = c->d_moduli + c->p_num + c->q_num;
    P.t_mu = c->d_t_mu;
    P.hat_inv = c->mu_hat_inv + (size_t)l * B * A;
    P.hat_mod_t = c->mu_hat_mod_t + (size_t)l * B * T * A;
    P.blk_mod_t = c->mu_blk_mod_t + (size_t)l * B * T;
    P.N = c->N;
    P.q_num = c->q_num;
    P.t_num = T;
    P.alpha = A;
    P.l = l;
    P.blocks = (l + 1 + A - 1) / A;
    dim3 grid(c->N / kThreads, P.blocks, batch);
    size_t smem = (size_t)(T * A + T) * sizeof(u64);
    if (A <= 4) modup_kernel<4><<<grid, kThreads, smem, st>>>(P);
    else if (A <= 8) modup_kernel<8><<<grid, kThreads, smem, st>>>(P);
    else modup_kernel<kMaxAlpha><<<grid, kThreads, smem, st>>>(P);
    count_launch();
    CKB_CUDA(cudaGetLastError());
    return CKKS_B200_OK;
}

}  // namespace

extern "C" int ckks_b200_modup_set_algo(ckks_b200_context* c, int algo) {
    CKB_REQUIRE(c != nullptr, CKKS_B200_ERR_ARG, "null argument");
    CKB_REQUIRE(algo >= 0 && algo <= 2, CKKS_B200_ERR_ARG, "unknown algorithm %d", algo);
    c->modup_algo = algo;
    return CKKS_B200_OK;
}

extern "C" int ckks_b200_context_set_wait_budget(ckks_b200_context* c, long long cycles) {
    CKB_REQUIRE(c != nullptr && cycles >= 0, CKKS_B200_ERR_ARG, "null handle or negative budget");
    c->wait_budget = cycles;
    return CKKS_B200_OK;
}

extern "C" int ckks_b200_context_test_withhold_commit(ckks_b200_context* c, int on) {
    CKB_REQUIRE(c != nullptr, CKKS_B200_ERR_ARG, "null handle");
    c->withhold_commit = on ? 1 : 0;
    return CKKS_B200_OK;
}

extern "C" int ckks_b200_context_test_exact_count(ckks_b200_context* c, int on) {
    CKB_REQUIRE(c != nullptr, CKKS_B200_ERR_ARG, "null handle");
    c->exact_count = on ? 1 : 0;
    return CKKS_B200_OK;
}

// Synchronise `stream` and report whether a bounded device-side wait of a tensor-core
// ModUp on this context ran out since the last check.
extern "C" int ckks_b200_context_check(ckks_b200_context* c, void* stream) {
    CKB_REQUIRE(c != nullptr, CKKS_B200_ERR_ARG, "null argument");
    DeviceGuard guard(c->device);
    CKB_REQUIRE(guard.ok, CKKS_B200_ERR_CUDA, "cudaSetDevice(%d) failed", c->device);
    cudaStream_t st = (cudaStream_t)stream;
    CKB_CUDA(cudaMemcpyAsync(c->h_flags, c->d_flags, 16 * sizeof(int), cudaMemcpyDeviceToHost, st));
    CKB_CUDA(cudaMemsetAsync(c->d_flags, 0, 16 * sizeof(int), st));
    CKB_CUDA(cudaStreamSynchronize(st));
    CKB_REQUIRE(c->h_flags[1] == 0, CKKS_B200_ERR_TIMEOUT,
                "a device-side wait ran out of its clock budget (site %d)", c->h_flags[1]);
    return CKKS_B200_OK;
}

extern "C" int ckks_b200_modup_qj_to_t(ckks_b200_context* c, uint64_t* d_out, const uint64_t* d_in,
                                       int l, int batch, void* stream) {
    return run_modup(c, (u64*)d_out, (const u64*)d_in, l, batch, (cudaStream_t)stream);
}

extern "C" int ckks_b200_modup_qj_to_t_host(ckks_b200_context* c, uint64_t* h_out,
                                            const uint64_t* h_in, int l, int batch) {
    CKB_REQUIRE(c && h_out && h_in, CKKS_B200_ERR_ARG, "null argument");
    CKB_REQUIRE(l >= 0 && l < c->q_num && batch >= 0, CKKS_B200_ERR_ARG, "bad level or batch");
    if (batch == 0) return CKKS_B200_OK;
    DeviceGuard guard(c->device);
    CKB_REQUIRE(guard.ok, CKKS_B200_ERR_CUDA, "cudaSetDevice(%d) failed", c->device);
    const int blocks = (l + 1 + c->alpha - 1) / c->alpha;
    size_t in_words = (size_t)batch * c->q_num * c->N;
    size_t out_words = (size_t)batch * blocks * c->t_num * c->N;
    int st = ensure_buf(&c->h2d_buf, &c->h2d_cap, in_words);
    if (st) return st;
    st = ensure_buf(&c->h2d_buf2, &c->h2d_cap2, out_words);
    if (st) return st;
    CKB_CUDA(cudaMemcpyAsync(c->h2d_buf, h_in, in_words * 8, cudaMemcpyHostToDevice, 0));
    st = run_modup(c, c->h2d_buf2, c->h2d_buf, l, batch, 0);
    if (st) return st;
    CKB_CUDA(cudaMemcpyAsync(h_out, c->h2d_buf2, out_words * 8, cudaMemcpyDeviceToHost, 0));
    return ckks_b200_context_check(c, 0);
}
