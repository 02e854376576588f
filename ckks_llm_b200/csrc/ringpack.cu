// Ring packing, RLWE -> MLWE direction: PCMM_Scheme::rlweCipherDecompose of the reference
// (src/ckks/include/pcmm/PCMM_Scheme.cuh:51-125).  One RLWE ciphertext (a, b) of degree N
// becomes mlwe_num MLWE ciphertexts of rank k = N/N1 and degree N1:
//   b_i[g]     =  B[i*gap + g*k]
//   a_i,0[g]   =  A[i*gap + g*k]
//   a_i,r[g]   =  A[(g-1)*k + (k-r) + i*gap]                 g >= 1, r = 1..k-1
//   a_i,r[0]   = -A[(N1-1)*k + (k-r) + i*gap]                (an index >= N wraps and flips the sign)
// with gap = k / mlwe_num, in the coefficient domain; the reference runs an inverse NTT on
// the RLWE ciphertext first and a forward NTT afterwards, and so does this entry point.
//
// For 1 <= r < k the source index falls by one as r rises by one, while the output is contiguous in g.
// A thread block therefore moves a 32 x 32 tile of (r, g) through shared memory: it reads with lanes
// along r (consecutive RLWE words) and writes with lanes along g (consecutive MLWE words), so both
// sides are coalesced.  HBM sees the output stream, (k+1)*N1 words per MLWE ciphertext per limb; the
// RLWE limb (512 KiB at N = 2^16) is re-read from L2.
#include "context.cuh"
#include "ringpack.cuh"

using namespace ckb;

namespace {

__global__ void __launch_bounds__(256) rlwe_decompose_kernel(const u64* __restrict__ rlwe, u64* const* __restrict__ mlwe,
                                                             const u64* __restrict__ q_moduli, long N, int N1, int k,
                                                             int mlwe_num, int L, int g_tiles) {
    __shared__ u64 tile[32][33];
    const int tx = threadIdx.x, ty = threadIdx.y;               // 32 x 8
    const int r0 = (blockIdx.x / g_tiles) * 32, g0 = (blockIdx.x % g_tiles) * 32;
    const int limb = blockIdx.y, i = blockIdx.z;
    const u64 q = q_moduli[limb];
    const int gap = k / mlwe_num;
    const u64* A = rlwe + N * limb;
    const u64* B = rlwe + N * (L + 1 + limb);
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const int g = g0 + ty + 8 * j, r = r0 + tx;             // lanes along r
        if (g < N1 && r <= k) tile[ty + 8 * j][tx] = decompose_word(A, B, q, N, N1, k, gap, i, r, g);
    }
    __syncthreads();
    const long C = (long)(k + 1) * N1;
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const int r = r0 + ty + 8 * j, g = g0 + tx;             // lanes along g
        if (g < N1 && r <= k) mlwe[i][(size_t)limb * C + (size_t)r * N1 + g] = tile[tx][ty + 8 * j];
    }
}

// The same decomposition for the usual case (N1 a multiple of 32, gap of at most 2), using its structure: with the
// negacyclic convention A[x +- N] = -A[x], word g of polynomial r < k of ciphertext i is
//   a_i,r[g] = A[g*k + i*gap - r]          (b_i[g] = B[g*k + i*gap])
// so ciphertexts and polynomials see the same RLWE words shifted against one another.  A block takes 32 values of g,
// 64 ciphertexts (four runs of 16) and DRB polynomials, loads per run and g the 15*gap + DRB words those share into
// shared memory, and writes their 64 x DRB row segments of 256 bytes from there: 256 KB of output per block against
// 8 KB for the tile transposes above, and an eighth of their reads.  The last "row block" is the b polynomial alone.
constexpr int DRB = 16;
constexpr int DSEG = 15 * 2 + DRB + 1;       // odd row length: lanes along g read distinct banks

__global__ void __launch_bounds__(256) rlwe_decompose_rows_kernel(const u64* __restrict__ rlwe, u64* const* __restrict__ mlwe,
                                                                  const u64* __restrict__ q_moduli, long N, int N1, int k,
                                                                  int mlwe_num, int L) {
    __shared__ u64 seg[4][32][DSEG];
    const int g_tiles = N1 / 32, rbn = (k + DRB - 1) / DRB;
    const int gt = blockIdx.x % g_tiles, rb = blockIdx.x / g_tiles;
    const int limb = blockIdx.z;
    const bool bpoly = rb == rbn;
    const int r0 = bpoly ? 0 : rb * DRB;                     // first polynomial, as it enters the index
    const int rows = bpoly ? 1 : (k - r0 < DRB ? k - r0 : DRB);
    const int crow0 = bpoly ? k : r0;                        // its row among the k+1 polynomials of a ciphertext
    const int g0 = gt * 32, n0 = blockIdx.y * 64;
    const int gap = k / mlwe_num;
    const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
    const u64 q = q_moduli[limb];
    const u64* src = rlwe + N * ((bpoly ? L + 1 : 0) + limb);
    {
        const int run = warp & 3, i0 = n0 + run * 16;
        if (i0 < mlwe_num) {
            const int span = 15 * gap + DRB;
            // four values of g per step, so that four loads are in flight before the first is used
            for (int x = lane; x < span; x += 32) {
                for (int gq = warp >> 2; gq < 32; gq += 8) {
                    u64 v[4];
                    bool neg[4];
#pragma unroll
                    for (int u = 0; u < 4; u++) {
                        long idx = (long)(g0 + gq + 2 * u) * k + (long)i0 * gap - (r0 + DRB - 1) + x;
                        neg[u] = false;
                        if (idx < 0) { idx += N; neg[u] = true; }
                        else if (idx >= N) { idx -= N; neg[u] = true; }
                        v[u] = src[idx];
                    }
#pragma unroll
                    for (int u = 0; u < 4; u++) seg[run][gq + 2 * u][x] = neg[u] ? (v[u] == 0 ? 0 : q - v[u]) : v[u];
                }
            }
        }
    }
    __syncthreads();
    const int cc = t & 31, run = (t >> 5) & 3, half = t >> 7;
    const int i0 = n0 + run * 16 + half * 8;                 // this thread writes ciphertexts i0 .. i0+7
    const long C = (long)(k + 1) * N1;
    u64* out[8];
#pragma unroll
    for (int e = 0; e < 8; e++) out[e] = i0 + e < mlwe_num ? mlwe[i0 + e] + (size_t)limb * C + g0 + cc : nullptr;
    const u64* row = seg[run][cc];
    for (int rr = 0; rr < rows; rr++) {
        const size_t off = (size_t)(crow0 + rr) * N1;
        int x = half * 8 * gap + (DRB - 1) - rr;
#pragma unroll
        for (int e = 0; e < 8; e++, x += gap)
            if (out[e]) out[e][off] = row[x];
    }
}

// ---------------------------------------------------------------------------
// MLWE -> RLWE packing (PCMM_Scheme::mlweCipherPacking, PCMM_Scheme.cuh:362-430), for the
// reference's ring-pack shape: one special prime p and one packing limb q0.  Buffers hold
// the limbs in the order [p, q0].
// ---------------------------------------------------------------------------

// mlweCipherEmbedding_new_kernel (:312-359): coefficient g of polynomial r of ciphertext i
// goes to position g*k + i*gap of embedded polynomial r; the p limb gets the centred lift.
// E: (k+1) polynomials of [2][N], zeroed beforehand.
// The source is contiguous in g, the destination in i: a 32 x 32 tile of (i, g) goes through shared memory so that
// both the reads (lanes along g) and the writes (lanes along i) are coalesced.
__global__ void __launch_bounds__(256) pack_embed_kernel(const u64* const* __restrict__ mlwe, u64* __restrict__ E, long N,
                                                         int N1, int k, int mlwe_num, u64 p, u64 q0, int g_tiles) {
    __shared__ u64 tile[32][33];
    const int tx = threadIdx.x, ty = threadIdx.y;               // 32 x 8
    const int i0 = (blockIdx.x / g_tiles) * 32, g0 = (blockIdx.x % g_tiles) * 32;
    const int r = blockIdx.y;
    const int gap = k / mlwe_num;
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const int i = i0 + ty + 8 * j, g = g0 + tx;             // lanes along g
        if (i < mlwe_num && g < N1) tile[ty + 8 * j][tx] = mlwe[i][(size_t)r * N1 + g];      // limb 0 of ciphertext i
    }
    __syncthreads();
    u64* poly = E + (size_t)r * 2 * N;
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const int g = g0 + ty + 8 * j, i = i0 + tx;             // lanes along i
        if (i < mlwe_num && g < N1) {
            const u64 v = tile[tx][ty + 8 * j];
            const long pos = (long)g * k + (long)i * gap;
            poly[N + pos] = v;
            poly[pos] = v > (q0 >> 1) ? (p - (q0 - v)) % p : v;
        }
    }
}

// mlweCipherMultRepackingKey_kernel (:261-289): (A, B) = sum_i E_i * key_i in the NTT domain.
// keys: [k][2 (a,b)][2 limbs][N]; O: [2 (a,b)][2 limbs][N].
__global__ void __launch_bounds__(128) pack_keymac_kernel(const u64* __restrict__ E, const u64* __restrict__ keys,
                                                          u64* __restrict__ O, long N, int k, u64 m0, u64 m0_mu_hi,
                                                          u64 m0_mu_lo, u64 m1, u64 m1_mu_hi, u64 m1_mu_lo) {
    const long n = (long)blockIdx.x * blockDim.x + threadIdx.x;
    const int m = blockIdx.y;
    if (n >= N) return;
    u64 alo = 0, ahi = 0, blo = 0, bhi = 0;
#pragma unroll 4
    for (int i = 0; i < k; i++) {
        const u64 c = E[((size_t)i * 2 + m) * N + n];
        const u64* key = keys + (size_t)i * 4 * N;
        mac128(alo, ahi, c, __ldg(key + (size_t)m * N + n));
        mac128(blo, bhi, c, __ldg(key + (size_t)(m + 2) * N + n));
    }
    const u64 mod = m ? m1 : m0, mh = m ? m1_mu_hi : m0_mu_hi, ml = m ? m1_mu_lo : m0_mu_lo;
    O[(size_t)m * N + n] = barrett128(alo, ahi, mod, mh, ml);
    O[(size_t)(2 + m) * N + n] = barrett128(blo, bhi, mod, mh, ml);
}

// ringpacking_ModDown_kernel (:291-308) followed by the addition of the embedded b
// (:426): out_c = (x_q + q - (x_p mod q)) * p^-1 mod q; b additionally + b_embedded mod q.
__global__ void __launch_bounds__(256) pack_moddown_kernel(const u64* __restrict__ O, const u64* __restrict__ b_embedded,
                                                           u64* __restrict__ out_a, u64* __restrict__ out_b, long N,
                                                           u64 q0, u64 pinv, u64 pinv_shoup) {
    const long n = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (n >= N) return;
    const int c = blockIdx.y;
    u64 ra = O[((size_t)c * 2) * N + n] % q0;
    ra = q0 - ra + O[((size_t)c * 2 + 1) * N + n];
    u64 r = shoup_mul(ra, pinv, pinv_shoup, q0);
    if (c == 0) {
        out_a[n] = r;
    } else {
        r += b_embedded[n];
        out_b[n] = csub(r, q0);
    }
}

}  // namespace

extern "C" int ckks_b200_mlwe_packing(ckks_b200_context* c, uint64_t* d_rlwe, int L, uint64_t* const* h_mlwe_ptrs,
                                      int mlwe_num, int N1, int mlwe_rank, const uint64_t* d_keys, void* stream) {
    CKB_REQUIRE(c && d_rlwe && h_mlwe_ptrs && d_keys, CKKS_B200_ERR_ARG, "null argument");
    CKB_REQUIRE(c->p_num >= 1, CKKS_B200_ERR_ARG, "packing needs a special prime p in the context");
    CKB_REQUIRE(N1 >= 1 && mlwe_rank >= 1 && (long)N1 * mlwe_rank == (long)c->N, CKKS_B200_ERR_SHAPE,
                "N1 * rank must equal N (%d * %d vs %u)", N1, mlwe_rank, c->N);
    CKB_REQUIRE(mlwe_num >= 1 && mlwe_num <= mlwe_rank && mlwe_num <= 65535, CKKS_B200_ERR_SHAPE,
                "mlwe_num %d outside [1, rank]", mlwe_num);
    CKB_REQUIRE(L >= 0 && L < c->q_num, CKKS_B200_ERR_ARG, "L=%d outside the %d q moduli", L, c->q_num);
    for (int i = 0; i < mlwe_num; i++)
        CKB_REQUIRE(h_mlwe_ptrs[i] != nullptr, CKKS_B200_ERR_ARG, "MLWE pointer %d is null", i);
    DeviceGuard guard(c->device);
    CKB_REQUIRE(guard.ok, CKKS_B200_ERR_CUDA, "cudaSetDevice(%d) failed", c->device);
    cudaStream_t st = (cudaStream_t)stream;
    const long N = c->N;
    const int k = mlwe_rank;
    const u64 p = c->moduli[c->p_num - 1], q0 = c->moduli[c->p_num];
    CKB_REQUIRE(p > q0, CKKS_B200_ERR_ARG, "the special prime must exceed q0 (centred lift, PCMM_Scheme.cuh:334)");
    int rc = ensure_buf(&c->ptr_buf, &c->ptr_cap, (size_t)mlwe_num);
    if (!rc) rc = ensure_buf(&c->pack_buf, &c->pack_cap, (size_t)(k + 1) * 2 * N + 4 * N);
    if (rc) return rc;
    u64* E = c->pack_buf;
    u64* O = E + (size_t)(k + 1) * 2 * N;
    CKB_CUDA(cudaMemcpyAsync(c->ptr_buf, h_mlwe_ptrs, sizeof(u64*) * mlwe_num, cudaMemcpyHostToDevice, st));
    // the reference clears the buffer (:397); with as many ciphertexts as the rank every position is written below
    if (mlwe_num != k) CKB_CUDA(cudaMemsetAsync(E, 0, sizeof(u64) * (size_t)(k + 1) * 2 * N, st));
    const int g_tiles = (N1 + 31) / 32;
    pack_embed_kernel<<<dim3((unsigned)(((mlwe_num + 31) / 32) * g_tiles), k + 1), dim3(32, 8), 0, st>>>(
        (const u64* const*)c->ptr_buf, E, N, N1, k, mlwe_num, p, q0, g_tiles);
    count_launch();
    CKB_CUDA(cudaGetLastError());
    // the k a-polynomials to the NTT domain over [p, q0] (:401)
    rc = ckks_b200_ntt_forward(c, (uint64_t*)E, 0, c->p_num - 1, k, 2, 2, stream);
    if (rc) return rc;
    u64 mu[4];
    h_barrett_mu(p, &mu[0], &mu[1]);
    h_barrett_mu(q0, &mu[2], &mu[3]);
    pack_keymac_kernel<<<dim3((unsigned)((N + 127) / 128), 2), 128, 0, st>>>(E, (const u64*)d_keys, O, N, k, p, mu[0], mu[1],
                                                                            q0, mu[2], mu[3]);
    count_launch();
    CKB_CUDA(cudaGetLastError());
    rc = ckks_b200_ntt_inverse(c, (uint64_t*)O, 0, c->p_num - 1, 2, 2, 2, stream);                                   // :416
    if (rc) return rc;
    const u64 pinv = h_invmod(p % q0, q0);
    u64* out_a = (u64*)d_rlwe;
    u64* out_b = (u64*)d_rlwe + (size_t)N * (L + 1);
    pack_moddown_kernel<<<dim3((unsigned)((N + 255) / 256), 2), 256, 0, st>>>(O, E + (size_t)k * 2 * N + N, out_a, out_b, N, q0,
                                                                             pinv, h_shoup(pinv, q0));
    count_launch();
    CKB_CUDA(cudaGetLastError());
    return ckks_b200_ntt_forward(c, d_rlwe, 0, c->p_num, 2, 1, L + 1, stream);                            // :428
}

extern "C" int ckks_b200_rlwe_decompose(ckks_b200_context* c, uint64_t* d_rlwe, int L, int l,
                                        uint64_t* const* h_mlwe_ptrs, int mlwe_num, int N1, int mlwe_rank,
                                        int ntt_domain, void* stream) {
    CKB_REQUIRE(c && d_rlwe && h_mlwe_ptrs, CKKS_B200_ERR_ARG, "null argument");
    CKB_REQUIRE(N1 >= 1 && mlwe_rank >= 1 && (long)N1 * mlwe_rank == (long)c->N, CKKS_B200_ERR_SHAPE,
                "N1 * rank must equal N (%d * %d vs %u)", N1, mlwe_rank, c->N);
    CKB_REQUIRE(l >= 0 && l <= L && L < c->q_num, CKKS_B200_ERR_ARG, "levels l=%d L=%d outside the %d q moduli", l, L, c->q_num);
    // the reference's check (PCMM_Scheme.cuh:103-106)
    CKB_REQUIRE(mlwe_num >= 1 && mlwe_num <= mlwe_rank, CKKS_B200_ERR_SHAPE,
                "rlweCipherDecompose extract number muse <= mlwe_rank");
    CKB_REQUIRE(mlwe_num <= 65535, CKKS_B200_ERR_UNSUPPORTED, "more than 65535 MLWE ciphertexts in one call");
    for (int i = 0; i < mlwe_num; i++)
        CKB_REQUIRE(h_mlwe_ptrs[i] != nullptr, CKKS_B200_ERR_ARG, "MLWE pointer %d is null", i);
    DeviceGuard guard(c->device);
    CKB_REQUIRE(guard.ok, CKKS_B200_ERR_CUDA, "cudaSetDevice(%d) failed", c->device);
    cudaStream_t st = (cudaStream_t)stream;
    int rc = ensure_buf(&c->ptr_buf, &c->ptr_cap, (size_t)mlwe_num);
    if (rc) return rc;
    CKB_CUDA(cudaMemcpyAsync(c->ptr_buf, h_mlwe_ptrs, sizeof(u64*) * mlwe_num, cudaMemcpyHostToDevice, st));
    if (ntt_domain) {
        rc = ckks_b200_ntt_inverse(c, d_rlwe, 0, c->p_num, 2, l + 1, L + 1, stream);     // :107
        if (rc) return rc;
    }
    if (N1 % 32 == 0 && mlwe_rank / mlwe_num <= 2 && c->N >= 256) {
        dim3 grid((unsigned)((N1 / 32) * ((mlwe_rank + DRB - 1) / DRB + 1)), (mlwe_num + 63) / 64, l + 1);
        rlwe_decompose_rows_kernel<<<grid, 256, 0, st>>>((const u64*)d_rlwe, (u64* const*)c->ptr_buf, c->d_moduli + c->p_num,
                                                         (long)c->N, N1, mlwe_rank, mlwe_num, L);
    } else {
        const int g_tiles = (N1 + 31) / 32;
        dim3 grid((unsigned)((mlwe_rank / 32 + 1) * g_tiles), l + 1, mlwe_num);
        rlwe_decompose_kernel<<<grid, dim3(32, 8), 0, st>>>((const u64*)d_rlwe, (u64* const*)c->ptr_buf, c->d_moduli + c->p_num,
                                                            (long)c->N, N1, mlwe_rank, mlwe_num, L, g_tiles);
    }
    count_launch();
    CKB_CUDA(cudaGetLastError());
    if (ntt_domain) {
        rc = ckks_b200_ntt_forward(c, d_rlwe, 0, c->p_num, 2, l + 1, L + 1, stream);      // :124
        if (rc) return rc;
    }
    return CKKS_B200_OK;
}
