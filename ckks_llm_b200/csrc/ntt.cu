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
//
// Three arithmetic back ends compute the same residues and are chosen per limb from the
// size of its modulus:
//   F64   (q < 2^50)  values are exact integers held in doubles; a product with a twiddle
//                     is one error-free multiplication (mul + fma), a quotient estimate
//                     rounded to an integer with the 1.5*2^52 trick, and an exact fma
//                     remainder: six FP64 operations, against one 64-bit high product
//                     and two 64-bit low products on the integer pipes, which on this GPU
//                     issue at a fraction of the FP64 rate (measured: 61 dfma vs 6.8
//                     umul64hi lane-operations per clock per SM).
//   LAZY  (q < 2^57)  64-bit Harvey butterflies without per-stage corrections and with a
//                     three-partial-product quotient estimate.
//   EXACT (otherwise) 64-bit Harvey butterflies, values in [0,4q) / [0,2q).
// Between the two kernels of a transform the in-place buffer holds the back end's lazy
// representation (for F64 the bit pattern of the double); the last kernel restores
// canonical residues.
#include <cuda_pipeline_primitives.h>

#include "context.cuh"

using namespace ckb;

namespace {

struct NttArgs {
    u64* data;
    const ulonglong2* tw;     // [mod][N] {w, w_shoup}
    const double* tw_d;       // [mod][N] w as double (exact below 2^53)
    const u64* moduli;        // [mod]
    const ulonglong2* ninv;   // [mod] {N^-1, shoup}
    const u64* qinv64;        // [mod] floor(2^64 / q)
    int logN;
    int start_limb_off, start_mod_idx, poly_mod_len;
};

constexpr u64 kF64Bound = 1ull << 50;
constexpr u64 kLazyBound = 1ull << 57;

// ---------------------------------------------------------------------------
// Arithmetic back ends.  V is the in-flight value type (64 bits wide), TW the twiddle.
// ct<R>: forward butterfly; gs<R>: inverse butterfly.  R asks the F64 back end for its
// extra range reduction on that stage; the integer back ends ignore it.
// ---------------------------------------------------------------------------
template <bool LAZY>
struct IntArith {
    typedef u64 V;
    typedef ulonglong2 TW;
    u64 q, q2, qinv64;
    ulonglong2 ninv;
    const ulonglong2* tw;
    __device__ __forceinline__ void init(const NttArgs& P, int mod) {
        q = P.moduli[mod];
        q2 = 2 * q;
        qinv64 = P.qinv64[mod];
        ninv = P.ninv[mod];
        tw = P.tw + ((size_t)mod << P.logN);
    }
    __device__ __forceinline__ TW twiddle(uint32_t i) const { return __ldg(tw + i); }
    __device__ __forceinline__ V from_word(u64 x) const { return x; }
    __device__ __forceinline__ u64 to_word(V x) const { return x; }
    __device__ __forceinline__ V from_canonical(u64 x) const { return x; }
    template <bool R>
    __device__ __forceinline__ void ct(V& a, V& b, TW w) const {
        if (LAZY) {
            // no correction: values grow by at most 4q per stage, (4*logN+1)*q < 2^64
            u64 t = shoup_lazy4(b, w.x, w.y, q);
            b = a + 2 * q2 - t;
            a = a + t;
        } else {
            u64 t = shoup_lazy(b, w.x, w.y, q);      // [0, 2q)
            u64 s = a >= q2 ? a - q2 : a;            // [0, 2q)
            a = s + t;
            b = s + q2 - t;                          // both in [0, 4q)
        }
    }
    template <bool R>
    __device__ __forceinline__ void gs(V& a, V& b, TW w) const {
        if (LAZY) {                                  // values in [0, 4q)
            const u64 q4 = 2 * q2;
            u64 t = a + q4 - b, s = a + b;
            a = s >= q4 ? s - q4 : s;
            b = shoup_lazy4(t, w.x, w.y, q);
        } else {                                     // values in [0, 2q)
            u64 t = a + q2 - b, s = a + b;
            a = s >= q2 ? s - q2 : s;
            b = shoup_lazy(t, w.x, w.y, q);
        }
    }
    // any lazy forward value -> [0, q)
    __device__ __forceinline__ u64 canonical_fwd(V x) const {
        if (LAZY) return csub(x - __umul64hi(x, qinv64) * q, q);
        return csub(csub(x, q2), q);
    }
    // last inverse stage: the lower half still needs N^-1, the upper half got it with psiinv[1]
    __device__ __forceinline__ u64 canonical_inv_lo(V x) const { return shoup_mul(x, ninv.x, ninv.y, q); }
    __device__ __forceinline__ u64 canonical_inv_hi(V x) const {
        if (LAZY) x = csub(x, q2);
        return csub(x, q);
    }
};

struct F64Arith {
    typedef double V;
    typedef double TW;
    double q, u, ninv;
    const double* tw;
    __device__ __forceinline__ void init(const NttArgs& P, int mod) {
        const u64 qi = P.moduli[mod];
        q = (double)qi;
        u = __drcp_rn(q);
        const u64 ni = P.ninv[mod].x;
        ninv = ni > qi / 2 ? -(double)(qi - ni) : (double)ni;
        tw = P.tw_d + ((size_t)mod << P.logN);
    }
    __device__ __forceinline__ TW twiddle(uint32_t i) const { return __ldg(tw + i); }
    __device__ __forceinline__ V from_word(u64 x) const { return __longlong_as_double((long long)x); }
    __device__ __forceinline__ u64 to_word(V x) const { return (u64)__double_as_longlong(x); }
    // exact for x < 2^52
    __device__ __forceinline__ V from_canonical(u64 x) const {
        return __dadd_rn(__longlong_as_double((long long)(x | 0x4330000000000000ull)), -4503599627370496.0);
    }
    // x - rint(x/q)*q, exact; |result| <= q/2 + tiny for |x| < 2^52.  1.5*2^52 rounds to an integer.
    __device__ __forceinline__ V reduce(V x) const {
        double c = __dadd_rn(__fma_rn(x, u, 6755399441055744.0), -6755399441055744.0);
        return __fma_rn(-c, q, x);
    }
    // b*w - c*q for an integer c near b*w/q, computed without error: h + l = b*w exactly,
    // h - c*q is exact because it is a small integer, and adding l stays below 2^53.
    // Twiddles are stored centred, |w| <= q/2 < 2^49, which halves both error terms:
    // |b| < 2^52  ->  |result| <= q/2 + 3|b|/16 for q up to 2^50.
    __device__ __forceinline__ V mulmod(V b, V w) const {
        double h = __dmul_rn(b, w);
        double l = __fma_rn(b, w, -h);
        double c = __dadd_rn(__fma_rn(h, u, 6755399441055744.0), -6755399441055744.0);
        double d = __fma_rn(-c, q, h);
        return __dadd_rn(d, l);
    }
    // Forward: a is reduced on one stage in three (R); with bound B on the inputs a stage
    // yields B + T(B) without and 0.51q + T(B) with the reduction, T(B) = q/2 + 3B/16, so
    // the cycle (R, -, -) keeps every value below 3.5q < 2^52.
    template <bool R>
    __device__ __forceinline__ void ct(V& a, V& b, TW w) const {
        double t = mulmod(b, w);
        double s = R ? reduce(a) : a;
        a = __dadd_rn(s, t);
        b = __dadd_rn(s, -t);
    }
    // Inverse: the sum is reduced on every stage; products then stay below 0.8q and
    // differences below 1.6q.
    template <bool R>
    __device__ __forceinline__ void gs(V& a, V& b, TW w) const {
        double s = __dadd_rn(a, b), d = __dadd_rn(a, -b);
        a = reduce(s);
        b = mulmod(d, w);
    }
    __device__ __forceinline__ u64 canonical(V x) const {
        x = reduce(x);
        if (x < 0.0) x = __dadd_rn(x, q);
        return (u64)__double_as_longlong(__dadd_rn(x, 4503599627370496.0)) & 0x000FFFFFFFFFFFFFull;
    }
    __device__ __forceinline__ u64 canonical_fwd(V x) const { return canonical(x); }
    __device__ __forceinline__ u64 canonical_inv_lo(V x) const { return canonical(mulmod(x, ninv)); }
    __device__ __forceinline__ u64 canonical_inv_hi(V x) const { return canonical(x); }
};

// ---------------------------------------------------------------------------
// Three stages on v[0..7]; v[j] sits at index base | (j << fb).  Stage s of the window
// pairs on window bit 2-s; S0..S1 selects which stages run.  widx is the twiddle index
// of stage 0 for this thread's group.
// ---------------------------------------------------------------------------
// RM: bit s set = stage s applies the back end's range reduction.
template <int S0, int S1, int RM, class A>
__device__ __forceinline__ void fwd8(const A& ar, typename A::V (&v)[8], uint32_t widx) {
    if (S0 <= 0 && 0 < S1) {
        typename A::TW w = ar.twiddle(widx);
#pragma unroll
        for (int j = 0; j < 4; j++) ar.template ct<(RM & 1) != 0>(v[j], v[j + 4], w);
    }
    if (S0 <= 1 && 1 < S1) {
#pragma unroll
        for (int h = 0; h < 2; h++) {
            typename A::TW w = ar.twiddle(2 * widx + h);
            ar.template ct<(RM & 2) != 0>(v[4 * h], v[4 * h + 2], w);
            ar.template ct<(RM & 2) != 0>(v[4 * h + 1], v[4 * h + 3], w);
        }
    }
    if (S0 <= 2 && 2 < S1) {
#pragma unroll
        for (int i = 0; i < 4; i++) {
            typename A::TW w = ar.twiddle(4 * widx + i);
            ar.template ct<(RM & 4) != 0>(v[2 * i], v[2 * i + 1], w);
        }
    }
}

// The same stages undone, bottom bit first.  K is the number, within its kernel, of the
// first stage this call executes; odd-numbered stages set R.
template <int S0, int S1, int K, class A>
__device__ __forceinline__ void inv8(const A& ar, typename A::V (&v)[8], uint32_t widx) {
    constexpr int first = S1 - 1;       // window stage executed first
    if (S0 <= 2 && 2 < S1) {
#pragma unroll
        for (int i = 0; i < 4; i++) {
            typename A::TW w = ar.twiddle(4 * widx + i);
            ar.template gs<((K + first - 2) & 1) == 1>(v[2 * i], v[2 * i + 1], w);
        }
    }
    if (S0 <= 1 && 1 < S1) {
#pragma unroll
        for (int h = 0; h < 2; h++) {
            typename A::TW w = ar.twiddle(2 * widx + h);
            ar.template gs<((K + first - 1) & 1) == 1>(v[4 * h], v[4 * h + 2], w);
            ar.template gs<((K + first - 1) & 1) == 1>(v[4 * h + 1], v[4 * h + 3], w);
        }
    }
    if (S0 <= 0 && 0 < S1) {
        typename A::TW w = ar.twiddle(widx);
#pragma unroll
        for (int j = 0; j < 4; j++) ar.template gs<((K + first - 0) & 1) == 1>(v[j], v[j + 4], w);
    }
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

// A CTA walks over `tiles` consecutive tiles of 16 chunks; warp v owns chunk v of every tile.
// While a chunk is in the butterflies the next one is already on its way into the warp's
// other shared-memory buffer (asynchronous 8-byte copies straight to the swizzled positions),
// so loads stay in flight through the compute phases.
__device__ __forceinline__ void prefetch_chunk(u64* sbuf, const u64* g, int lane) {
#pragma unroll
    for (int j = 0; j < 8; j++) {
        const uint32_t p = j * 32 + lane;
        __pipeline_memcpy_async(sbuf + swz(p), g + p, 8);
    }
    __pipeline_commit();
}

template <class A>
__device__ __forceinline__ void fwd_contig_body(const NttArgs& P, u64* S, int tiles) {
    typedef typename A::V V;
    const int lane = threadIdx.x & 31, vv = threadIdx.x >> 5;
    const int limb = blockIdx.y, poly = blockIdx.z;
    A ar;
    ar.init(P, P.start_mod_idx + limb);
    const uint32_t N = 1u << P.logN;
    u64* gl = P.data + (((size_t)poly * P.poly_mod_len + P.start_limb_off + limb) << P.logN);
    const uint32_t xfirst = (blockIdx.x * tiles * kChunksPerCta + vv) * kChunk;
    u64* sbuf = S + vv * 2 * kChunk;            // two buffers per warp
    V a[8];
    prefetch_chunk(sbuf, gl + xfirst, lane);
    for (int t = 0; t < tiles; t++) {
        const uint32_t x0 = xfirst + t * kChunksPerCta * kChunk;      // position of the chunk
        u64* s = sbuf + (t & 1) * kChunk;
        __syncwarp();                            // every lane is done with the other buffer
        if (t + 1 < tiles) {
            prefetch_chunk(sbuf + ((t + 1) & 1) * kChunk, gl + x0 + kChunksPerCta * kChunk, lane);
            __pipeline_wait_prior(1);
        } else {
            __pipeline_wait_prior(0);
        }
        __syncwarp();

        // window bits 7..5: p = j*32 + lane
#pragma unroll
        for (int j = 0; j < 8; j++) a[j] = ar.from_word(s[swz(j * 32 + lane)]);
        fwd8<0, 3, 1>(ar, a, (N + x0) >> 8);             // kernel stages 0 (reducing), 1, 2
#pragma unroll
        for (int j = 0; j < 8; j++) s[swz(j * 32 + lane)] = ar.to_word(a[j]);
        __syncwarp();

        // window bits 4..2: p = hi*32 + j*4 + lo, lane = hi*4 + lo
        {
            const uint32_t lo = lane & 3, hi = lane >> 2;
#pragma unroll
            for (int j = 0; j < 8; j++) a[j] = ar.from_word(s[swz(hi * 32 + j * 4 + lo)]);
            fwd8<0, 3, 1>(ar, a, ((N + x0) >> 5) + hi);  // stages 3 (reducing), 4, 5
#pragma unroll
            for (int j = 0; j < 8; j++) s[swz(hi * 32 + j * 4 + lo)] = ar.to_word(a[j]);
        }
        __syncwarp();

        // window bits 2..0, stages on bits 1 and 0 only: p = lane*8 + j
#pragma unroll
        for (int j = 0; j < 8; j++) a[j] = ar.from_word(s[swz(lane * 8 + j)]);
        fwd8<1, 3, 2>(ar, a, ((N + x0) >> 3) + lane);    // stages 6 (reducing), 7
        ulonglong2* go = reinterpret_cast<ulonglong2*>(gl + x0 + lane * 8);
#pragma unroll
        for (int j = 0; j < 4; j++) go[j] = make_ulonglong2(ar.canonical_fwd(a[2 * j]), ar.canonical_fwd(a[2 * j + 1]));
    }
}

template <class A>
__device__ __forceinline__ void inv_contig_body(const NttArgs& P, u64* S, int tiles) {
    typedef typename A::V V;
    const int lane = threadIdx.x & 31, vv = threadIdx.x >> 5;
    const int limb = blockIdx.y, poly = blockIdx.z;
    A ar;
    ar.init(P, P.start_mod_idx + limb);
    const uint32_t N = 1u << P.logN;
    u64* gl = P.data + (((size_t)poly * P.poly_mod_len + P.start_limb_off + limb) << P.logN);
    const uint32_t xfirst = (blockIdx.x * tiles * kChunksPerCta + vv) * kChunk;
    u64* sbuf = S + vv * 2 * kChunk;
    V a[8];
    prefetch_chunk(sbuf, gl + xfirst, lane);
    for (int t = 0; t < tiles; t++) {
        const uint32_t x0 = xfirst + t * kChunksPerCta * kChunk;
        u64* s = sbuf + (t & 1) * kChunk;
        __syncwarp();
        if (t + 1 < tiles) {
            prefetch_chunk(sbuf + ((t + 1) & 1) * kChunk, gl + x0 + kChunksPerCta * kChunk, lane);
            __pipeline_wait_prior(1);
        } else {
            __pipeline_wait_prior(0);
        }
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 8; j++) a[j] = ar.from_canonical(s[swz(lane * 8 + j)]);
        inv8<1, 3, 0>(ar, a, ((N + x0) >> 3) + lane);            // stages 0, 1 of this kernel
#pragma unroll
        for (int j = 0; j < 8; j++) s[swz(lane * 8 + j)] = ar.to_word(a[j]);
        __syncwarp();
        {
            const uint32_t lo = lane & 3, hi = lane >> 2;
#pragma unroll
            for (int j = 0; j < 8; j++) a[j] = ar.from_word(s[swz(hi * 32 + j * 4 + lo)]);
            inv8<0, 3, 2>(ar, a, ((N + x0) >> 5) + hi);          // stages 2, 3, 4
#pragma unroll
            for (int j = 0; j < 8; j++) s[swz(hi * 32 + j * 4 + lo)] = ar.to_word(a[j]);
        }
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 8; j++) a[j] = ar.from_word(s[swz(j * 32 + lane)]);
        inv8<0, 3, 5>(ar, a, (N + x0) >> 8);                      // stages 5, 6, 7
        // values stay lazy; the strided phase finishes the transform
#pragma unroll
        for (int j = 0; j < 8; j++) gl[x0 + j * 32 + lane] = ar.to_word(a[j]);
    }
}

template <bool INV>
__global__ void __launch_bounds__(kThreadsB, 2) ntt_contig(NttArgs P, int tiles) {
    extern __shared__ __align__(16) u64 S[];       // 2 buffers x 16 chunks x 256 words
    const u64 q = P.moduli[P.start_mod_idx + blockIdx.y];
    if (q < kF64Bound) {
        if (INV) inv_contig_body<F64Arith>(P, S, tiles); else fwd_contig_body<F64Arith>(P, S, tiles);
    } else if (q < kLazyBound) {
        if (INV) inv_contig_body<IntArith<true>>(P, S, tiles); else fwd_contig_body<IntArith<true>>(P, S, tiles);
    } else {
        if (INV) inv_contig_body<IntArith<false>>(P, S, tiles); else fwd_contig_body<IntArith<false>>(P, S, tiles);
    }
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
struct Win {
    typedef StridedCfg<SA> C;
    static constexpr int fb = C::T - 3 * (WIN + 1);
    static constexpr int nst_raw = SA - 3 * WIN;
    static constexpr int nst = nst_raw < 1 ? 1 : (nst_raw < 3 ? nst_raw : 3);
    // stages executed before this window in the inverse kernel (windows run high to low)
    static constexpr int inv_before = (SA - 3 * (WIN + 1)) > 0 ? (SA - 3 * (WIN + 1)) : 0;
    __device__ static __forceinline__ uint32_t base(uint32_t tid) {
        return ((tid >> fb) << (fb + 3)) | (tid & ((1u << fb) - 1));
    }
    __device__ static __forceinline__ uint32_t widx(uint32_t b) { return ((1u << C::T) + b) >> (fb + 3); }
    __device__ static __forceinline__ u64* gptr(u64* g, uint32_t idx) {
        return g + ((size_t)(idx >> C::LOGCW) << 8) + (idx & (C::CW - 1));
    }
};

template <int SA, class A>
__device__ __forceinline__ void fwd_strided_body(const NttArgs& P, u64* S) {
    typedef StridedCfg<SA> C;
    typedef typename A::V V;
    const uint32_t tid = threadIdx.x;
    const int limb = blockIdx.y, poly = blockIdx.z;
    A ar;
    ar.init(P, P.start_mod_idx + limb);
    u64* g = P.data + (((size_t)poly * P.poly_mod_len + P.start_limb_off + limb) << P.logN) +
             (size_t)blockIdx.x * C::CW;
    V a[8];
    uint32_t b = Win<SA, 0>::base(tid);
#pragma unroll
    for (int j = 0; j < 8; j++) a[j] = ar.from_canonical(*Win<SA, 0>::gptr(g, b | (j << Win<SA, 0>::fb)));
    fwd8<0, Win<SA, 0>::nst, 4>(ar, a, Win<SA, 0>::widx(b));      // the third stage of a window reduces
    if (C::NWIN >= 2) {
#pragma unroll
        for (int j = 0; j < 8; j++) S[b | (j << Win<SA, 0>::fb)] = ar.to_word(a[j]);
        __syncthreads();
        b = Win<SA, 1>::base(tid);
#pragma unroll
        for (int j = 0; j < 8; j++) a[j] = ar.from_word(S[b | (j << Win<SA, 1>::fb)]);
        fwd8<0, Win<SA, 1>::nst, 4>(ar, a, Win<SA, 1>::widx(b));
    }
    if (C::NWIN >= 3) {
#pragma unroll
        for (int j = 0; j < 8; j++) S[b | (j << Win<SA, 1>::fb)] = ar.to_word(a[j]);
        __syncthreads();
        b = Win<SA, 2>::base(tid);
#pragma unroll
        for (int j = 0; j < 8; j++) a[j] = ar.from_word(S[b | (j << Win<SA, 2>::fb)]);
        fwd8<0, Win<SA, 2>::nst, 4>(ar, a, Win<SA, 2>::widx(b));
    }
    constexpr int LW = C::NWIN - 1;
#pragma unroll
    for (int j = 0; j < 8; j++) *Win<SA, LW>::gptr(g, b | (j << Win<SA, LW>::fb)) = ar.to_word(a[j]);
}

template <int SA, class A>
__device__ __forceinline__ void inv_strided_body(const NttArgs& P, u64* S) {
    typedef StridedCfg<SA> C;
    typedef typename A::V V;
    const uint32_t tid = threadIdx.x;
    const int limb = blockIdx.y, poly = blockIdx.z;
    A ar;
    ar.init(P, P.start_mod_idx + limb);
    u64* g = P.data + (((size_t)poly * P.poly_mod_len + P.start_limb_off + limb) << P.logN) +
             (size_t)blockIdx.x * C::CW;
    V a[8];
    constexpr int LW = C::NWIN - 1;
    uint32_t b = Win<SA, LW>::base(tid);
#pragma unroll
    for (int j = 0; j < 8; j++) a[j] = ar.from_word(*Win<SA, LW>::gptr(g, b | (j << Win<SA, LW>::fb)));
    if (C::NWIN == 3) {
        inv8<0, Win<SA, 2>::nst, Win<SA, 2>::inv_before>(ar, a, Win<SA, 2>::widx(b));
#pragma unroll
        for (int j = 0; j < 8; j++) S[b | (j << Win<SA, 2>::fb)] = ar.to_word(a[j]);
        __syncthreads();
        b = Win<SA, 1>::base(tid);
#pragma unroll
        for (int j = 0; j < 8; j++) a[j] = ar.from_word(S[b | (j << Win<SA, 1>::fb)]);
    }
    if (C::NWIN >= 2) {
        inv8<0, Win<SA, 1>::nst, Win<SA, 1>::inv_before>(ar, a, Win<SA, 1>::widx(b));
#pragma unroll
        for (int j = 0; j < 8; j++) S[b | (j << Win<SA, 1>::fb)] = ar.to_word(a[j]);
        __syncthreads();
        b = Win<SA, 0>::base(tid);
#pragma unroll
        for (int j = 0; j < 8; j++) a[j] = ar.from_word(S[b | (j << Win<SA, 0>::fb)]);
    }
    inv8<0, Win<SA, 0>::nst, Win<SA, 0>::inv_before>(ar, a, Win<SA, 0>::widx(b));
    // Final scaling: the last stage's twiddle psiinv[1] already carries N^-1 for the upper
    // half (a[4..7] of the top window); the lower half is multiplied by N^-1 here
    // (src/ckks/include/ntt_60bit.cuh:890-898).
#pragma unroll
    for (int j = 0; j < 8; j++) {
        const u64 r = j < 4 ? ar.canonical_inv_lo(a[j]) : ar.canonical_inv_hi(a[j]);
        *Win<SA, 0>::gptr(g, b | (j << Win<SA, 0>::fb)) = r;
    }
}

template <int SA, bool INV>
__global__ void __launch_bounds__(StridedCfg<SA>::THREADS, 2) ntt_strided(NttArgs P) {
    typedef StridedCfg<SA> C;
    __shared__ u64 S[C::NWIN > 1 ? (1 << C::T) : 1];
    const u64 q = P.moduli[P.start_mod_idx + blockIdx.y];
    if (q < kF64Bound) {
        if (INV) inv_strided_body<SA, F64Arith>(P, S); else fwd_strided_body<SA, F64Arith>(P, S);
    } else if (q < kLazyBound) {
        if (INV) inv_strided_body<SA, IntArith<true>>(P, S); else fwd_strided_body<SA, IntArith<true>>(P, S);
    } else {
        if (INV) inv_strided_body<SA, IntArith<false>>(P, S); else fwd_strided_body<SA, IntArith<false>>(P, S);
    }
}

template <int SA>
void launch_strided(bool inverse, dim3 grid_lp, const NttArgs& P, cudaStream_t st) {
    typedef StridedCfg<SA> C;
    dim3 grid(256 / C::CW, grid_lp.y, grid_lp.z);
    if (inverse) ntt_strided<SA, true><<<grid, C::THREADS, 0, st>>>(P);
    else ntt_strided<SA, false><<<grid, C::THREADS, 0, st>>>(P);
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
    P.tw_d = inverse ? c->tw_inv_d : c->tw_fwd_d;
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
    // the contiguous kernel walks over several tiles per CTA so that its prefetch has something to run ahead of
    const int ntile = c->N / (kChunk * kChunksPerCta);
    // ... unless the call is so small that walking would leave SMs without a CTA: then more, shorter CTAs
    int tiles = ntile >= 4 ? 4 : ntile;
    {
        static int sms = 0;
        if (sms == 0 && cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, c->device) != cudaSuccess) sms = 148;
        const long transforms = (long)mod_num * poly_num;
        while (tiles > 1 && transforms * (ntile / tiles) < 2L * sms) tiles >>= 1;
    }
    const size_t smem_c = 2 * kChunk * kChunksPerCta * sizeof(u64);
    dim3 grid_k(ntile / tiles, mod_num, poly_num);
    if (!inverse) {
        strided();
        CKB_CUDA(cudaFuncSetAttribute(ntt_contig<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_c));
        ntt_contig<false><<<grid_k, kThreadsB, smem_c, st>>>(P, tiles);
    } else {
        CKB_CUDA(cudaFuncSetAttribute(ntt_contig<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_c));
        ntt_contig<true><<<grid_k, kThreadsB, smem_c, st>>>(P, tiles);
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
