// Batched negacyclic NTT / INTT over RNS limbs for N = 2^12 .. 2^16.
//
// A transform is split into a strided phase (the first logN-8 Cooley-Tukey stages,
// which couple elements 256 apart or more) and a contiguous phase (the last 8 stages
// on 256-point chunks); the inverse runs the two phases in the opposite order with
// Gentleman-Sande butterflies.  In both kernels a thread owns 8 values at a time and
// runs up to three butterfly stages on them in registers ("window" of three index
// bits); between windows the values are exchanged through shared memory.  The first
// window of a kernel loads straight from global memory and the last one stores
// straight back, so a value crosses shared memory twice per kernel at most.
//
// Stage s (m = 2^s groups) uses twiddle psi_table[m + group]; with x the position of
// an element in the polynomial and b the index bit the stage pairs on, that index is
// (N + x) >> (b + 1).  Outputs are canonical.  Semantics follow
// Context_23::ToNTTInplace / FromNTTInplace of the reference
// (src/ckks/include/Context_23.cuh:847-889, butterflies ntt_60bit.cuh:293-318).
#include "context.cuh"

using namespace ckb;

namespace {

struct NttArgs {
    u64* data;
    const ulonglong2* tw;     // [mod][N] {w, w_shoup}
    const u64* moduli;        // [mod]
    const ulonglong2* ninv;   // [mod] {N^-1, shoup}
    const u64* qinv64;        // [mod] floor(2^64 / q)
    int logN;
    int start_limb_off, start_mod_idx, poly_mod_len;
};

__device__ __forceinline__ ulonglong2 ldtw(const ulonglong2* p) { return __ldg(p); }

// Harvey butterflies.  Forward keeps values in [0, 4q), inverse in [0, 2q).
// With LAZY the forward butterfly skips the conditional subtraction: values then grow by
// at most 2q per stage, (2*logN+1)*q < 2^64 after all stages when q < 2^58, and the Shoup
// product is exact for any 64-bit input; one reduction at the very end restores [0, q).
template <bool LAZY>
__device__ __forceinline__ void ct_bfly(u64& a, u64& b, ulonglong2 w, u64 q, u64 q2) {
    u64 t = shoup_lazy(b, w.x, w.y, q);       // [0, 2q)
    u64 s = a;
    if (!LAZY) s = a >= q2 ? a - q2 : a;      // [0, 2q)
    a = s + t;
    b = s + q2 - t;
}
__device__ __forceinline__ void gs_bfly(u64& a, u64& b, ulonglong2 w, u64 q, u64 q2) {
    u64 t = a + q2 - b;
    u64 s = a + b;
    a = s >= q2 ? s - q2 : s;
    b = shoup_lazy(t, w.x, w.y, q);
}

// Three forward stages on a[0..7]; a[j] sits at index base | (j << fb).  S0..S1 select
// which of the three (stage 0 pairs on the top bit of the window).  widx is the
// twiddle index of stage 0 for this thread's group.
template <int S0, int S1, bool LAZY>
__device__ __forceinline__ void fwd8(u64 (&a)[8], const ulonglong2* tw, uint32_t widx, u64 q, u64 q2) {
    if (S0 <= 0 && 0 < S1) {
        ulonglong2 w = ldtw(tw + widx);
#pragma unroll
        for (int j = 0; j < 4; j++) ct_bfly<LAZY>(a[j], a[j + 4], w, q, q2);
    }
    if (S0 <= 1 && 1 < S1) {
#pragma unroll
        for (int h = 0; h < 2; h++) {
            ulonglong2 w = ldtw(tw + 2 * widx + h);
            ct_bfly<LAZY>(a[4 * h], a[4 * h + 2], w, q, q2);
            ct_bfly<LAZY>(a[4 * h + 1], a[4 * h + 3], w, q, q2);
        }
    }
    if (S0 <= 2 && 2 < S1) {
#pragma unroll
        for (int i = 0; i < 4; i++) {
            ulonglong2 w = ldtw(tw + 4 * widx + i);
            ct_bfly<LAZY>(a[2 * i], a[2 * i + 1], w, q, q2);
        }
    }
}

// The same three stages undone, bottom bit first.
template <int S0, int S1>
__device__ __forceinline__ void inv8(u64 (&a)[8], const ulonglong2* tw, uint32_t widx, u64 q, u64 q2) {
    if (S0 <= 2 && 2 < S1) {
#pragma unroll
        for (int i = 0; i < 4; i++) {
            ulonglong2 w = ldtw(tw + 4 * widx + i);
            gs_bfly(a[2 * i], a[2 * i + 1], w, q, q2);
        }
    }
    if (S0 <= 1 && 1 < S1) {
#pragma unroll
        for (int h = 0; h < 2; h++) {
            ulonglong2 w = ldtw(tw + 2 * widx + h);
            gs_bfly(a[4 * h], a[4 * h + 2], w, q, q2);
            gs_bfly(a[4 * h + 1], a[4 * h + 3], w, q, q2);
        }
    }
    if (S0 <= 0 && 0 < S1) {
        ulonglong2 w = ldtw(tw + widx);
#pragma unroll
        for (int j = 0; j < 4; j++) gs_bfly(a[j], a[j + 4], w, q, q2);
    }
}

template <int NST, bool LAZY>
__device__ __forceinline__ void fwd_n(u64 (&a)[8], const ulonglong2* tw, uint32_t widx, u64 q, u64 q2) {
    if (NST == 3) fwd8<0, 3, LAZY>(a, tw, widx, q, q2);
    else if (NST == 2) fwd8<0, 2, LAZY>(a, tw, widx, q, q2);
    else fwd8<0, 1, LAZY>(a, tw, widx, q, q2);
}
template <int NST>
__device__ __forceinline__ void inv_n(u64 (&a)[8], const ulonglong2* tw, uint32_t widx, u64 q, u64 q2) {
    if (NST == 3) inv8<0, 3>(a, tw, widx, q, q2);
    else if (NST == 2) inv8<0, 2>(a, tw, widx, q, q2);
    else inv8<0, 1>(a, tw, widx, q, q2);
}

// ---------------------------------------------------------------------------
// Contiguous phase: 16 chunks of 256 points per CTA, one warp per chunk.
// Shared-memory position of point p of a chunk: the low four bits are XOR-ed with
// bits 4..6 so that all three windows are bank-conflict free for 64-bit accesses.
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t swz(uint32_t p) {
    return p ^ ((p >> 4) & 7u) ^ (((p >> 5) & 1u) << 3);
}

constexpr int kChunk = 256;
constexpr int kChunksPerCta = 16;
constexpr int kThreadsB = 32 * kChunksPerCta;

// Moduli below this bound take the lazy forward butterflies (see ct_bfly).
constexpr u64 kLazyBound = 1ull << 58;

template <bool LAZY>
__device__ __forceinline__ void ntt_fwd_contig_body(const NttArgs& P, u64* S) {
    const int lane = threadIdx.x & 31, v = threadIdx.x >> 5;
    const int limb = blockIdx.y, poly = blockIdx.z;
    const int mod = P.start_mod_idx + limb;
    const u64 q = P.moduli[mod], q2 = 2 * q;
    const uint32_t N = 1u << P.logN;
    const ulonglong2* tw = P.tw + ((size_t)mod << P.logN);
    const uint32_t x0 = (blockIdx.x * kChunksPerCta + v) * kChunk;   // position of the chunk
    u64* g = P.data + (((size_t)poly * P.poly_mod_len + P.start_limb_off + limb) << P.logN) + x0;
    u64* s = S + v * kChunk;
    u64 a[8];

    // window bits 7..5: p = j*32 + lane
#pragma unroll
    for (int j = 0; j < 8; j++) a[j] = g[j * 32 + lane];
    fwd8<0, 3, LAZY>(a, tw, (N + x0) >> 8, q, q2);
#pragma unroll
    for (int j = 0; j < 8; j++) s[swz(j * 32 + lane)] = a[j];
    __syncwarp();

    // window bits 4..2: p = hi*32 + j*4 + lo, lane = hi*4 + lo
    {
        const uint32_t lo = lane & 3, hi = lane >> 2;
#pragma unroll
        for (int j = 0; j < 8; j++) a[j] = s[swz(hi * 32 + j * 4 + lo)];
        fwd8<0, 3, LAZY>(a, tw, ((N + x0) >> 5) + hi, q, q2);
#pragma unroll
        for (int j = 0; j < 8; j++) s[swz(hi * 32 + j * 4 + lo)] = a[j];
    }
    __syncwarp();

    // window bits 2..0, stages on bits 1 and 0 only: p = lane*8 + j
#pragma unroll
    for (int j = 0; j < 8; j++) a[j] = s[swz(lane * 8 + j)];
    fwd8<1, 3, LAZY>(a, tw, ((N + x0) >> 3) + lane, q, q2);
    if (LAZY) {
        // values are below (2*logN+1)*q: one Barrett-style step with floor(2^64/q) brings them to [0, 2q)
        const u64 qinv64 = P.qinv64[mod];
#pragma unroll
        for (int j = 0; j < 8; j++) a[j] = csub(a[j] - __umul64hi(a[j], qinv64) * q, q);
    } else {
#pragma unroll
        for (int j = 0; j < 8; j++) a[j] = csub(csub(a[j], q2), q);
    }
    ulonglong2* go = reinterpret_cast<ulonglong2*>(g + lane * 8);
#pragma unroll
    for (int j = 0; j < 4; j++) go[j] = make_ulonglong2(a[2 * j], a[2 * j + 1]);
}

__global__ void __launch_bounds__(kThreadsB, 2) ntt_fwd_contig(NttArgs P) {
    __shared__ u64 S[kChunk * kChunksPerCta];
    const u64 q = P.moduli[P.start_mod_idx + blockIdx.y];
    if (q < kLazyBound) ntt_fwd_contig_body<true>(P, S);
    else ntt_fwd_contig_body<false>(P, S);
}

__global__ void __launch_bounds__(kThreadsB, 2) ntt_inv_contig(NttArgs P) {
    __shared__ u64 S[kChunk * kChunksPerCta];
    const int lane = threadIdx.x & 31, v = threadIdx.x >> 5;
    const int limb = blockIdx.y, poly = blockIdx.z;
    const int mod = P.start_mod_idx + limb;
    const u64 q = P.moduli[mod], q2 = 2 * q;
    const uint32_t N = 1u << P.logN;
    const ulonglong2* tw = P.tw + ((size_t)mod << P.logN);
    const uint32_t x0 = (blockIdx.x * kChunksPerCta + v) * kChunk;
    u64* g = P.data + (((size_t)poly * P.poly_mod_len + P.start_limb_off + limb) << P.logN) + x0;
    u64* s = S + v * kChunk;
    u64 a[8];

    const ulonglong2* gi = reinterpret_cast<const ulonglong2*>(g + lane * 8);
#pragma unroll
    for (int j = 0; j < 4; j++) {
        ulonglong2 t = gi[j];
        a[2 * j] = t.x;
        a[2 * j + 1] = t.y;
    }
    inv8<1, 3>(a, tw, ((N + x0) >> 3) + lane, q, q2);
#pragma unroll
    for (int j = 0; j < 8; j++) s[swz(lane * 8 + j)] = a[j];
    __syncwarp();
    {
        const uint32_t lo = lane & 3, hi = lane >> 2;
#pragma unroll
        for (int j = 0; j < 8; j++) a[j] = s[swz(hi * 32 + j * 4 + lo)];
        inv8<0, 3>(a, tw, ((N + x0) >> 5) + hi, q, q2);
#pragma unroll
        for (int j = 0; j < 8; j++) s[swz(hi * 32 + j * 4 + lo)] = a[j];
    }
    __syncwarp();
#pragma unroll
    for (int j = 0; j < 8; j++) a[j] = s[swz(j * 32 + lane)];
    inv8<0, 3>(a, tw, (N + x0) >> 8, q, q2);
    // values stay in [0, 2q); the strided phase finishes the transform
#pragma unroll
    for (int j = 0; j < 8; j++) g[j * 32 + lane] = a[j];
}

// ---------------------------------------------------------------------------
// Strided phase: SA = logN-8 stages on vectors of R = 2^SA points with stride 256.
// A CTA owns a tile of R rows x CW consecutive columns (CW = min(256, 4096/R)),
// indexed idx = row*CW + col; the stage bits are the top SA bits of idx.
// Window w covers idx bits [T-3(w+1), T-3w) and runs min(3, SA-3w) stages.
// ---------------------------------------------------------------------------
template <int SA>
struct StridedCfg {
    static constexpr int R = 1 << SA;
    static constexpr int CW = (4096 / R) < 256 ? (4096 / R) : 256;
    static constexpr int LOGCW = CW == 256 ? 8 : CW == 128 ? 7 : CW == 64 ? 6 : CW == 32 ? 5 : 4;
    static constexpr int T = SA + LOGCW;
    static constexpr int THREADS = (1 << T) / 8;
    static constexpr int NWIN = (SA + 2) / 3;
};

template <int SA, int WIN>
__device__ __forceinline__ uint32_t strided_base(uint32_t tid) {
    constexpr int fb = StridedCfg<SA>::T - 3 * (WIN + 1);
    return ((tid >> fb) << (fb + 3)) | (tid & ((1u << fb) - 1));
}

template <int SA, int WIN, bool INV, bool LAZY = false>
__device__ __forceinline__ void strided_window(u64 (&a)[8], const ulonglong2* tw, uint32_t base, u64 q, u64 q2) {
    using C = StridedCfg<SA>;
    constexpr int fb = C::T - 3 * (WIN + 1);
    constexpr int nst = (SA - 3 * WIN) < 3 ? (SA - 3 * WIN) : 3;
    const uint32_t widx = ((1u << C::T) + base) >> (fb + 3);
    if (INV) inv_n<nst>(a, tw, widx, q, q2);
    else fwd_n<nst, LAZY>(a, tw, widx, q, q2);
}

template <int SA>
__device__ __forceinline__ u64* strided_gptr(u64* g, uint32_t idx) {
    using C = StridedCfg<SA>;
    return g + ((size_t)(idx >> C::LOGCW) << 8) + (idx & (C::CW - 1));
}

template <int SA, int WIN>
__device__ __forceinline__ void strided_ld_smem(u64 (&a)[8], const u64* S, uint32_t base) {
    constexpr int fb = StridedCfg<SA>::T - 3 * (WIN + 1);
#pragma unroll
    for (int j = 0; j < 8; j++) a[j] = S[base | (j << fb)];
}
template <int SA, int WIN>
__device__ __forceinline__ void strided_st_smem(const u64 (&a)[8], u64* S, uint32_t base) {
    constexpr int fb = StridedCfg<SA>::T - 3 * (WIN + 1);
#pragma unroll
    for (int j = 0; j < 8; j++) S[base | (j << fb)] = a[j];
}
template <int SA, int WIN>
__device__ __forceinline__ void strided_ld_gmem(u64 (&a)[8], u64* g, uint32_t base) {
    constexpr int fb = StridedCfg<SA>::T - 3 * (WIN + 1);
#pragma unroll
    for (int j = 0; j < 8; j++) a[j] = *strided_gptr<SA>(g, base | (j << fb));
}
template <int SA, int WIN>
__device__ __forceinline__ void strided_st_gmem(const u64 (&a)[8], u64* g, uint32_t base) {
    constexpr int fb = StridedCfg<SA>::T - 3 * (WIN + 1);
#pragma unroll
    for (int j = 0; j < 8; j++) *strided_gptr<SA>(g, base | (j << fb)) = a[j];
}

template <int SA, bool LAZY>
__device__ __forceinline__ void ntt_fwd_strided_body(const NttArgs& P, u64* S) {
    using C = StridedCfg<SA>;
    const uint32_t tid = threadIdx.x;
    const int limb = blockIdx.y, poly = blockIdx.z;
    const int mod = P.start_mod_idx + limb;
    const u64 q = P.moduli[mod], q2 = 2 * q;
    const ulonglong2* tw = P.tw + ((size_t)mod << P.logN);
    u64* g = P.data + (((size_t)poly * P.poly_mod_len + P.start_limb_off + limb) << P.logN) +
             (size_t)blockIdx.x * C::CW;
    u64 a[8];
    uint32_t base = strided_base<SA, 0>(tid);
    strided_ld_gmem<SA, 0>(a, g, base);
    strided_window<SA, 0, false, LAZY>(a, tw, base, q, q2);
    if (C::NWIN == 1) { strided_st_gmem<SA, 0>(a, g, base); return; }
    strided_st_smem<SA, 0>(a, S, base);
    __syncthreads();
    base = strided_base<SA, 1>(tid);
    strided_ld_smem<SA, 1>(a, S, base);
    strided_window<SA, 1, false, LAZY>(a, tw, base, q, q2);
    if (C::NWIN == 2) { strided_st_gmem<SA, 1>(a, g, base); return; }
    strided_st_smem<SA, 1>(a, S, base);
    __syncthreads();
    base = strided_base<SA, 2>(tid);
    strided_ld_smem<SA, 2>(a, S, base);
    strided_window<SA, 2, false, LAZY>(a, tw, base, q, q2);
    strided_st_gmem<SA, 2>(a, g, base);
}

template <int SA>
__global__ void __launch_bounds__(StridedCfg<SA>::THREADS, 2) ntt_fwd_strided(NttArgs P) {
    using C = StridedCfg<SA>;
    __shared__ u64 S[C::NWIN > 1 ? (1 << C::T) : 1];
    const u64 q = P.moduli[P.start_mod_idx + blockIdx.y];
    if (q < kLazyBound) ntt_fwd_strided_body<SA, true>(P, S);
    else ntt_fwd_strided_body<SA, false>(P, S);
}

// Final scaling of the inverse transform: the last stage's twiddle psiinv[1] already
// carries N^-1 for the upper half (a[4..7] of the top window); the lower half is
// multiplied by N^-1 here (src/ckks/include/ntt_60bit.cuh:890-898).
__device__ __forceinline__ void inv_finish(u64 (&a)[8], ulonglong2 ninv, u64 q) {
#pragma unroll
    for (int j = 0; j < 4; j++) {
        a[j] = shoup_mul(a[j], ninv.x, ninv.y, q);
        a[j + 4] = csub(a[j + 4], q);
    }
}

template <int SA>
__global__ void __launch_bounds__(StridedCfg<SA>::THREADS, 2) ntt_inv_strided(NttArgs P) {
    using C = StridedCfg<SA>;
    __shared__ u64 S[C::NWIN > 1 ? (1 << C::T) : 1];
    const uint32_t tid = threadIdx.x;
    const int limb = blockIdx.y, poly = blockIdx.z;
    const int mod = P.start_mod_idx + limb;
    const u64 q = P.moduli[mod], q2 = 2 * q;
    const ulonglong2* tw = P.tw + ((size_t)mod << P.logN);
    const ulonglong2 ninv = P.ninv[mod];
    u64* g = P.data + (((size_t)poly * P.poly_mod_len + P.start_limb_off + limb) << P.logN) +
             (size_t)blockIdx.x * C::CW;
    u64 a[8];
    uint32_t base;
    if (C::NWIN == 3) {
        base = strided_base<SA, 2>(tid);
        strided_ld_gmem<SA, 2>(a, g, base);
        strided_window<SA, 2, true>(a, tw, base, q, q2);
        strided_st_smem<SA, 2>(a, S, base);
        __syncthreads();
    }
    if (C::NWIN >= 2) {
        base = strided_base<SA, 1>(tid);
        if (C::NWIN == 2) strided_ld_gmem<SA, 1>(a, g, base);
        else strided_ld_smem<SA, 1>(a, S, base);
        strided_window<SA, 1, true>(a, tw, base, q, q2);
        strided_st_smem<SA, 1>(a, S, base);
        __syncthreads();
    }
    base = strided_base<SA, 0>(tid);
    if (C::NWIN == 1) strided_ld_gmem<SA, 0>(a, g, base);
    else strided_ld_smem<SA, 0>(a, S, base);
    strided_window<SA, 0, true>(a, tw, base, q, q2);
    inv_finish(a, ninv, q);
    strided_st_gmem<SA, 0>(a, g, base);
}

template <int SA>
void launch_strided(bool inverse, dim3 grid_lp, const NttArgs& P, cudaStream_t st) {
    using C = StridedCfg<SA>;
    dim3 grid(256 / C::CW, grid_lp.y, grid_lp.z);
    if (inverse) ntt_inv_strided<SA><<<grid, C::THREADS, 0, st>>>(P);
    else ntt_fwd_strided<SA><<<grid, C::THREADS, 0, st>>>(P);
}

int run_ntt(ckks_b200_context* c, u64* d_data, int start_limb_off, int start_mod_idx, int poly_num,
            int mod_num, int poly_mod_len, bool inverse, cudaStream_t st) {
    CKB_REQUIRE(c && d_data, CKKS_B200_ERR_ARG, "null argument");
    CKB_REQUIRE(poly_num >= 0 && mod_num >= 0 && poly_mod_len >= 0 && start_limb_off >= 0 &&
                    start_mod_idx >= 0, CKKS_B200_ERR_ARG, "negative count or offset");
    CKB_REQUIRE(start_mod_idx + mod_num <= c->mod_num, CKKS_B200_ERR_ARG,
                "moduli [%d,%d) exceed the %d of the context", start_mod_idx,
                start_mod_idx + mod_num, c->mod_num);
    CKB_REQUIRE(start_limb_off + mod_num <= poly_mod_len, CKKS_B200_ERR_ARG,
                "limbs [%d,%d) exceed poly_mod_len=%d", start_limb_off, start_limb_off + mod_num,
                poly_mod_len);
    CKB_REQUIRE(mod_num <= 65535 && poly_num <= 65535, CKKS_B200_ERR_UNSUPPORTED,
                "more than 65535 limbs or polynomials in one call");
    if (poly_num == 0 || mod_num == 0) return CKKS_B200_OK;
    DeviceGuard guard(c->device);
    CKB_REQUIRE(guard.ok, CKKS_B200_ERR_CUDA, "cudaSetDevice(%d) failed", c->device);

    NttArgs P;
    P.data = d_data;
    P.tw = inverse ? c->tw_inv : c->tw_fwd;
    P.moduli = c->d_moduli;
    P.ninv = c->d_ninv;
    P.qinv64 = c->d_qinv64;
    P.logN = c->logN;
    P.start_limb_off = start_limb_off;
    P.start_mod_idx = start_mod_idx;
    P.poly_mod_len = poly_mod_len;

    dim3 grid_c(c->N / (kChunk * kChunksPerCta), mod_num, poly_num);
    auto strided = [&]() {
        switch (c->logN - 8) {
            case 4: launch_strided<4>(inverse, grid_c, P, st); break;
            case 5: launch_strided<5>(inverse, grid_c, P, st); break;
            case 6: launch_strided<6>(inverse, grid_c, P, st); break;
            case 7: launch_strided<7>(inverse, grid_c, P, st); break;
            case 8: launch_strided<8>(inverse, grid_c, P, st); break;
        }
    };
    if (!inverse) {
        strided();
        ntt_fwd_contig<<<grid_c, kThreadsB, 0, st>>>(P);
    } else {
        ntt_inv_contig<<<grid_c, kThreadsB, 0, st>>>(P);
        strided();
    }
    count_launch(2);
    CKB_CUDA(cudaGetLastError());
    return CKKS_B200_OK;
}

int run_ntt_host(ckks_b200_context* c, u64* h_data, int start_limb_off, int start_mod_idx,
                 int poly_num, int mod_num, int poly_mod_len, bool inverse) {
    CKB_REQUIRE(c && h_data, CKKS_B200_ERR_ARG, "null argument");
    CKB_REQUIRE(poly_num >= 0 && poly_mod_len >= 0, CKKS_B200_ERR_ARG, "negative count");
    DeviceGuard guard(c->device);
    CKB_REQUIRE(guard.ok, CKKS_B200_ERR_CUDA, "cudaSetDevice(%d) failed", c->device);
    size_t words = (size_t)poly_num * poly_mod_len * c->N;
    if (words == 0) return CKKS_B200_OK;
    int st = ensure_buf(&c->h2d_buf, &c->h2d_cap, words);
    if (st) return st;
    CKB_CUDA(cudaMemcpyAsync(c->h2d_buf, h_data, words * 8, cudaMemcpyHostToDevice, 0));
    st = run_ntt(c, c->h2d_buf, start_limb_off, start_mod_idx, poly_num, mod_num, poly_mod_len,
                 inverse, 0);
    if (st) return st;
    CKB_CUDA(cudaMemcpyAsync(h_data, c->h2d_buf, words * 8, cudaMemcpyDeviceToHost, 0));
    CKB_CUDA(cudaStreamSynchronize(0));
    return CKKS_B200_OK;
}

}  // namespace

extern "C" int ckks_b200_ntt_forward(ckks_b200_context* c, uint64_t* d, int lo, int mi, int pn,
                                     int mn, int pml, void* stream) {
    return run_ntt(c, (u64*)d, lo, mi, pn, mn, pml, false, (cudaStream_t)stream);
}
extern "C" int ckks_b200_ntt_inverse(ckks_b200_context* c, uint64_t* d, int lo, int mi, int pn,
                                     int mn, int pml, void* stream) {
    return run_ntt(c, (u64*)d, lo, mi, pn, mn, pml, true, (cudaStream_t)stream);
}
extern "C" int ckks_b200_ntt_forward_host(ckks_b200_context* c, uint64_t* h, int lo, int mi, int pn,
                                          int mn, int pml) {
    return run_ntt_host(c, (u64*)h, lo, mi, pn, mn, pml, false);
}
extern "C" int ckks_b200_ntt_inverse_host(ckks_b200_context* c, uint64_t* h, int lo, int mi, int pn,
                                          int mn, int pml) {
    return run_ntt_host(c, (u64*)h, lo, mi, pn, mn, pml, true);
}
