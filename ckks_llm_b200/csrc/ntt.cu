// Batched negacyclic NTT / INTT over RNS limbs for N = 2^12 .. 2^16.
//
// A transform is split into a strided phase (the first logN-8 Cooley-Tukey stages, which
// couple elements 256 apart or more) and a contiguous phase (the last 8 stages on 256-point
// chunks); the inverse runs the two phases in the opposite order with Gentleman-Sande
// butterflies.  Each phase is one kernel that reads and writes the data once.
//
// Both kernels work on tiles of 4096 words with 256 threads.  A thread owns 16 values at a time
// and runs up to four butterfly stages on them in registers (a "window" of four index bits), so
// a phase of up to eight stages is two windows with ONE exchange through shared memory in
// between.  A CTA walks over several tiles; while one is in the butterflies the next is on its
// way from global memory into the other half of a double buffer (16-byte asynchronous copies),
// and the first window reads its values from that buffer.  Every global access of a warp covers
// whole 128-byte lines (the load/store path of an SM takes one line per cycle, and with 16
// words per thread that, not HBM, is the first limit these kernels meet): results a lane holds as
// 16 consecutive words leave through shared memory, and the contiguous phase, which uses each of
// its 4080 twiddles per tile in one butterfly only, copies them into shared memory in order and
// walks over the polynomials of the call at a fixed tile position so that they are fetched once.
//
// Stage s (m = 2^s groups) uses twiddle psi_table[m + group]; with x the position of an element
// in the polynomial and b the index bit the stage pairs on, that index is (N + x) >> (b + 1).
// Outputs are canonical.  Semantics follow Context_23::ToNTTInplace / FromNTTInplace of the
// reference (src/ckks/include/Context_23.cuh:847-889, butterflies ntt_60bit.cuh:293-318).
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
    // last inverse stage: the same butterfly; N^-1 follows in canonical_inv_lo
    __device__ __forceinline__ void gs_last(V& a, V& b, TW w) const { gs<true>(a, b, w); }
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
    double q, u, ninv, to_pos;
    long long qi;
    const double* tw;
    __device__ __forceinline__ void init(const NttArgs& P, int mod) {
        qi = (long long)P.moduli[mod];
        q = (double)qi;
        to_pos = 4503599627370496.0 + 2.0 * q;                   // 2^52 + 2q, an integer below 2^53
        u = __drcp_rn(q);
        const long long ni = (long long)P.ninv[mod].x;
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
    // the cycle (-, -, R) starting from canonical inputs keeps every value below 3.5q < 2^52,
    // and a transform whose last stage reduces ends below 1.7q.
    template <bool R>
    __device__ __forceinline__ void ct(V& a, V& b, TW w) const {
        double t = mulmod(b, w);
        double s = R ? reduce(a) : a;
        a = __dadd_rn(s, t);
        b = __dadd_rn(s, -t);
    }
    // Inverse: the difference goes through the product (below q/2 + 3|d|/16), the sum is reduced on two stages in
    // three (R).  With S the bound on the inputs, |d| <= 2S must stay below 2^52 = 4q: the cycle (R, R, -) from
    // canonical inputs keeps S below 1.93q.
    template <bool R>
    __device__ __forceinline__ void gs(V& a, V& b, TW w) const {
        double s = __dadd_rn(a, b), d = __dadd_rn(a, -b);
        a = R ? reduce(s) : s;
        b = mulmod(d, w);
    }
    // Last inverse stage: N^-1 is due on both outputs.  The table's psiinv[1] carries it for the difference
    // (src/ckks/include/Utils.cuh:190-201); the sum gets it as its own product, which also reduces it.
    __device__ __forceinline__ void gs_last(V& a, V& b, TW w) const {
        double s = __dadd_rn(a, b), d = __dadd_rn(a, -b);
        a = mulmod(s, ninv);
        b = mulmod(d, w);
    }
    // |x| < 2q -> [0, q).  x + 2q lies in (0, 4q), below 2^52, so adding 2^52 + 2q leaves it in the mantissa as an
    // integer; the two conditional subtractions run on the integer pipe (the FP64 pipe is what these kernels wait for).
    __device__ __forceinline__ u64 canonical(V x) const {
        u64 v = (u64)__double_as_longlong(__dadd_rn(x, to_pos)) & 0x000FFFFFFFFFFFFFull;
        v = v >= 2 * (u64)qi ? v - 2 * (u64)qi : v;
        return v >= (u64)qi ? v - (u64)qi : v;
    }
    __device__ __forceinline__ u64 canonical_fwd(V x) const { return canonical(x); }
    __device__ __forceinline__ u64 canonical_inv_lo(V x) const { return canonical(x); }      // gs_last applied N^-1
    __device__ __forceinline__ u64 canonical_inv_hi(V x) const { return canonical(x); }
};

// ---------------------------------------------------------------------------
// Twiddles of a four-stage window: stage s takes 2^s of them, get<s>(w) fetches those.
// ---------------------------------------------------------------------------
// From the table in global memory: stage s uses psi[(widx << s) + h], widx the index of stage 0.
template <class A>
struct TwGlobal {
    const A& ar;
    uint32_t widx;
    template <int s>
    __device__ __forceinline__ void get(typename A::TW (&w)[1 << s]) const {
#pragma unroll
        for (int h = 0; h < (1 << s); h++) w[h] = ar.twiddle((widx << s) + h);
    }
};

// The twiddles of one tile of the contiguous phase (16 chunks), staged in shared memory as eight runs that are
// contiguous in the table: for window A (chunk bits 7..4) stage s has 2^s per chunk, for window B (bits 3..0)
// 2^s per 16 points.  Offsets in words; the runs of B's last two stages are stored with their 16-byte units
// permuted so that the lanes of a quarter-warp, each reading its own 32 or 64 bytes, hit different banks.
__host__ __device__ constexpr int tw_a(int s) { return s == 0 ? 0 : s == 1 ? 16 : s == 2 ? 48 : 112; }
__host__ __device__ constexpr int tw_b(int s) { return s == 0 ? 240 : s == 1 ? 496 : s == 2 ? 1008 : 2032; }
constexpr int kTwWords = 4080;

struct TwSharedA {
    const double* base;
    int c;                                   // chunk inside the tile
    template <int s>
    __device__ __forceinline__ void get(double (&w)[1 << s]) const {
        const double* p = base + tw_a(s) + (c << s);
#pragma unroll
        for (int h = 0; h < (1 << s); h++) w[h] = p[h];
    }
};
struct TwSharedB {
    const double* base;
    int lp;                                  // 16-point group inside the tile (chunk * 16 + lane of the chunk)
    template <int s>
    __device__ __forceinline__ void get(double (&w)[1 << s]) const {
        if (s == 0) {
            w[0] = base[tw_b(0) + lp];
        } else {
            constexpr int units = (1 << s) / 2;                             // 16-byte units per lane
            const int perm = s == 3 ? ((lp >> 1) & 3) : s == 2 ? ((lp >> 2) & 1) : 0;
            const double2* p = reinterpret_cast<const double2*>(base + tw_b(s)) + lp * units;
#pragma unroll
            for (int k = 0; k < units; k++) {
                const double2 t = p[k ^ perm];
                w[2 * k] = t.x;
                w[2 * k + 1] = t.y;
            }
        }
    }
};

// The strided phase takes its twiddles from the first 256 entries of the limb's table whatever the tile (stage s of
// window 0 uses entries 2^s .. 2^(s+1)-1, window 1 those from 16 on): they sit in shared memory, copied once per CTA.
constexpr int kTwStrided = 256;
template <class TW>
struct TwSharedS {                           // 16-byte twiddles of the integer back ends: one load each
    const TW* base;
    uint32_t widx;
    template <int s>
    __device__ __forceinline__ void get(TW (&w)[1 << s]) const {
#pragma unroll
        for (int h = 0; h < (1 << s); h++) w[h] = base[(widx << s) + h];
    }
};
template <>
struct TwSharedS<double> {                   // doubles: two per load
    const double* base;
    uint32_t widx;
    template <int s>
    __device__ __forceinline__ void get(double (&w)[1 << s]) const {
        const double* p = base + (widx << s);
        if (s == 0) {
            w[0] = p[0];
        } else {
            const double2* p2 = reinterpret_cast<const double2*>(p);
#pragma unroll
            for (int k = 0; k < (1 << s) / 2; k++) {
                const double2 t = p2[k];
                w[2 * k] = t.x;
                w[2 * k + 1] = t.y;
            }
        }
    }
};

// Copies the twiddle runs of the tile at position xt into shared memory (all threads of the CTA, 16 bytes per copy).
__device__ __forceinline__ void stage_twiddles(double* dst, const double* table, uint32_t N, uint32_t xt, int tid, int nthreads) {
    for (int U = tid; U < kTwWords / 2; U += nthreads) {
        // which run this unit belongs to
        int s, first, win_b;
        if (U < 120) { win_b = 0; s = U < 8 ? 0 : U < 24 ? 1 : U < 56 ? 2 : 3; first = tw_a(s) / 2; }
        else { win_b = 1; s = U < 248 ? 0 : U < 504 ? 1 : U < 1016 ? 2 : 3; first = tw_b(s) / 2; }
        const int u = U - first;
        const uint32_t start = (N + xt) >> ((win_b ? 4 : 8) - s);            // first table index of the run
        const int pu = (win_b && s == 3) ? (u ^ ((u >> 3) & 3)) : (win_b && s == 2) ? (u ^ ((u >> 3) & 1)) : u;
        __pipeline_memcpy_async(dst + 2 * (first + pu), table + start + 2 * u, 16);
    }
}

// ---------------------------------------------------------------------------
// Four stages on v[0..15]; v[j] sits at index base | (j << fb).  Stage s of the window pairs on
// window bit 3-s; stages S0..S1-1 run.  RM: bit s set = stage s applies the back end's range reduction.
// ---------------------------------------------------------------------------
template <int S0, int S1, int RM, class A, class TWS>
__device__ __forceinline__ void fwd16(const A& ar, typename A::V (&v)[16], const TWS& tws) {
    if (S0 <= 0 && 0 < S1) {
        typename A::TW w[1];
        tws.template get<0>(w);
#pragma unroll
        for (int j = 0; j < 8; j++) ar.template ct<(RM & 1) != 0>(v[j], v[j + 8], w[0]);
    }
    if (S0 <= 1 && 1 < S1) {
        typename A::TW w[2];
        tws.template get<1>(w);
#pragma unroll
        for (int h = 0; h < 2; h++)
#pragma unroll
            for (int j = 0; j < 4; j++) ar.template ct<(RM & 2) != 0>(v[8 * h + j], v[8 * h + j + 4], w[h]);
    }
    if (S0 <= 2 && 2 < S1) {
        typename A::TW w[4];
        tws.template get<2>(w);
#pragma unroll
        for (int h = 0; h < 4; h++)
#pragma unroll
            for (int j = 0; j < 2; j++) ar.template ct<(RM & 4) != 0>(v[4 * h + j], v[4 * h + j + 2], w[h]);
    }
    if (S0 <= 3 && 3 < S1) {
        typename A::TW w[8];
        tws.template get<3>(w);
#pragma unroll
        for (int h = 0; h < 8; h++) ar.template ct<(RM & 8) != 0>(v[2 * h], v[2 * h + 1], w[h]);
    }
}

// The same stages undone, bottom bit first.  RM as above (the inverse reduces its sums on the marked stages);
// LAST: stage 0 of this window is the last stage of the transform and applies N^-1.
template <int S0, int S1, int RM, bool LAST, class A, class TWS>
__device__ __forceinline__ void inv16(const A& ar, typename A::V (&v)[16], const TWS& tws) {
    if (S0 <= 3 && 3 < S1) {
        typename A::TW w[8];
        tws.template get<3>(w);
#pragma unroll
        for (int h = 0; h < 8; h++) ar.template gs<(RM & 8) != 0>(v[2 * h], v[2 * h + 1], w[h]);
    }
    if (S0 <= 2 && 2 < S1) {
        typename A::TW w[4];
        tws.template get<2>(w);
#pragma unroll
        for (int h = 0; h < 4; h++)
#pragma unroll
            for (int j = 0; j < 2; j++) ar.template gs<(RM & 4) != 0>(v[4 * h + j], v[4 * h + j + 2], w[h]);
    }
    if (S0 <= 1 && 1 < S1) {
        typename A::TW w[2];
        tws.template get<1>(w);
#pragma unroll
        for (int h = 0; h < 2; h++)
#pragma unroll
            for (int j = 0; j < 4; j++) ar.template gs<(RM & 2) != 0>(v[8 * h + j], v[8 * h + j + 4], w[h]);
    }
    if (S0 <= 0 && 0 < S1) {
        typename A::TW w[1];
        tws.template get<0>(w);
#pragma unroll
        for (int j = 0; j < 8; j++) {
            if (LAST) ar.gs_last(v[j], v[j + 8], w[0]);
            else ar.template gs<(RM & 1) != 0>(v[j], v[j + 8], w[0]);
        }
    }
}

// Reduction masks.  Forward: a stage reduces when the number of stages after it is a multiple of three, so the last
// stage does (the results end below 1.7q) and at most three stages in a row do not (3.5q from canonical inputs or
// from the 1.7q a reducing stage leaves); the very first stage has nothing to reduce.  REM = stages of the transform
// after stage 0 of the window.  Inverse: the stage executed as number e of the transform (0 = first) reduces unless
// e % 3 == 2.
__host__ __device__ constexpr int fwd_mask(int REM, bool first_window) {
    return ((REM % 3 == 0 && !first_window) ? 1 : 0) | (((REM - 1) % 3 == 0) ? 2 : 0) | (((REM - 2) % 3 == 0) ? 4 : 0) |
           (((REM - 3) % 3 == 0) ? 8 : 0);
}
// a window whose stages 3, 2, 1, 0 are executed as numbers E3, E3+1, E3+2, E3+3
__host__ __device__ constexpr int inv_mask(int E3) {
    return ((E3 % 3 != 2) ? 8 : 0) | (((E3 + 1) % 3 != 2) ? 4 : 0) | (((E3 + 2) % 3 != 2) ? 2 : 0) | (((E3 + 3) % 3 != 2) ? 1 : 0);
}

constexpr int kTile = 4096;            // words per tile
constexpr int kThreads = 256;          // 16 values per thread
constexpr int kChunk = 256;            // points per chunk of the contiguous phase

// ---------------------------------------------------------------------------
// Contiguous phase.  A tile is 16 chunks of 256 consecutive points; a half-warp owns one chunk.
// Window A pairs on chunk bits 7..4: lane l of the chunk holds points j*16 + l.  Window B pairs on
// bits 3..0: lane l holds the 16 consecutive points l*16 + j.  Shared-memory position of point p of
// a chunk: bits 1..3 are XOR-ed with bits 4..6, which keeps pairs of points together (16-byte
// copies and 128-bit accesses stay aligned) and makes both windows bank-conflict free.
// A CTA stays at one tile position of one limb and walks over polynomials, so the tile's twiddles
// are staged once (back ends whose twiddle is one double; the integer back ends read the table).
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t swz(uint32_t p) { return p ^ (((p >> 4) & 7u) << 1); }

// This warp's two chunks of a tile, global -> shared, 16 bytes per copy, 8 copies per lane.
__device__ __forceinline__ void prefetch_chunks(u64* swarp, const u64* gwarp, int lane) {
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const uint32_t p = 2 * (i * 32 + lane);                 // word inside the warp's 512
        __pipeline_memcpy_async(swarp + (p & 256) + swz(p & 255), gwarp + p, 16);
    }
}

template <class A>
struct StagesTwiddles { static constexpr bool value = false; };
template <>
struct StagesTwiddles<F64Arith> { static constexpr bool value = true; };

template <bool INV, class A>
__device__ __forceinline__ void contig_body(const NttArgs& P, u64* S, int poly0, int npoly) {
    typedef typename A::V V;
    constexpr bool STAGED = StagesTwiddles<A>::value;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, l = lane & 15;
    const int limb = blockIdx.y;
    A ar;
    ar.init(P, P.start_mod_idx + limb);
    const uint32_t N = 1u << P.logN;
    const uint32_t xt = (uint32_t)blockIdx.x * kTile;                           // the tile's position in its polynomial
    const uint32_t xwarp = xt + warp * 512;                                     // this warp's two chunks
    const uint32_t coff = (lane >> 4) * kChunk;                                 // this half-warp's chunk
    const uint32_t x0 = xwarp + coff;
    u64* sbuf = S + warp * 1024;                                                // two buffers of 512 words per warp
    const double* stw = reinterpret_cast<const double*>(S + 2 * kTile);         // the staged twiddles
    auto gpoly = [&](int t) { return P.data + (((size_t)(poly0 + t) * P.poly_mod_len + P.start_limb_off + limb) << P.logN); };
    V a[16];
    if (STAGED) stage_twiddles(const_cast<double*>(stw), P.tw_d + ((size_t)(P.start_mod_idx + limb) << P.logN), N, xt, tid, kThreads);
    wait_for_previous_kernel();
    prefetch_chunks(sbuf, gpoly(0) + xwarp, lane);
    __pipeline_commit();
    for (int t = 0; t < npoly; t++) {
        u64* gl = gpoly(t);
        u64* s = sbuf + (t & 1) * 512 + coff;
        __syncwarp();                                             // every lane is done with the other buffer
        if (t + 1 < npoly) prefetch_chunks(sbuf + ((t + 1) & 1) * 512, gpoly(t + 1) + xwarp, lane);
        __pipeline_commit();
        __pipeline_wait_prior(1);
        if (STAGED && t == 0) __syncthreads();                    // the twiddles came in through every thread's copies
        else __syncwarp();

        const int c = warp * 2 + (lane >> 4);                     // chunk inside the tile
        if (!INV) {
            // window A, chunk bits 7..4: p = j*16 + l
#pragma unroll
            for (int j = 0; j < 16; j++) a[j] = ar.from_word(s[j * 16 + (l ^ ((j & 7) << 1))]);
            // the last eight stages of the transform: seven follow the first of them
            if constexpr (STAGED) fwd16<0, 4, fwd_mask(7, false), A>(ar, a, TwSharedA{stw, c});
            else fwd16<0, 4, fwd_mask(7, false), A>(ar, a, TwGlobal<A>{ar, (N + x0) >> 8});
#pragma unroll
            for (int j = 0; j < 16; j++) s[j * 16 + (l ^ ((j & 7) << 1))] = ar.to_word(a[j]);
            __syncwarp();
            // window B, chunk bits 3..0: p = l*16 + j, read as pairs
            ulonglong2* s2 = reinterpret_cast<ulonglong2*>(s + l * 16);
#pragma unroll
            for (int m = 0; m < 8; m++) {
                const ulonglong2 w = s2[m ^ (l & 7)];
                a[2 * m] = ar.from_word(w.x);
                a[2 * m + 1] = ar.from_word(w.y);
            }
            if constexpr (STAGED) fwd16<0, 4, fwd_mask(3, false), A>(ar, a, TwSharedB{stw, c * 16 + l});
            else fwd16<0, 4, fwd_mask(3, false), A>(ar, a, TwGlobal<A>{ar, ((N + x0) >> 4) + l});
            // A lane holds 16 consecutive words; storing them from here would touch 32 different 128-byte lines
            // per instruction.  They go back through the chunk's buffer and leave with 16 lanes per line.
#pragma unroll
            for (int m = 0; m < 8; m++) s2[m ^ (l & 7)] = make_ulonglong2(ar.canonical_fwd(a[2 * m]), ar.canonical_fwd(a[2 * m + 1]));
            __syncwarp();
#pragma unroll
            for (int j = 0; j < 16; j++) gl[x0 + j * 16 + l] = s[j * 16 + (l ^ ((j & 7) << 1))];
        } else {
            // window B first: p = l*16 + j
            ulonglong2* s2 = reinterpret_cast<ulonglong2*>(s + l * 16);
#pragma unroll
            for (int m = 0; m < 8; m++) {
                const ulonglong2 w = s2[m ^ (l & 7)];
                a[2 * m] = ar.from_canonical(w.x);
                a[2 * m + 1] = ar.from_canonical(w.y);
            }
            // executed as stages 0..3 of the inverse
            if constexpr (STAGED) inv16<0, 4, inv_mask(0), false, A>(ar, a, TwSharedB{stw, c * 16 + l});
            else inv16<0, 4, inv_mask(0), false, A>(ar, a, TwGlobal<A>{ar, ((N + x0) >> 4) + l});
#pragma unroll
            for (int m = 0; m < 8; m++) s2[m ^ (l & 7)] = make_ulonglong2(ar.to_word(a[2 * m]), ar.to_word(a[2 * m + 1]));
            __syncwarp();
            // window A: p = j*16 + l
#pragma unroll
            for (int j = 0; j < 16; j++) a[j] = ar.from_word(s[j * 16 + (l ^ ((j & 7) << 1))]);
            // stages 4..7
            if constexpr (STAGED) inv16<0, 4, inv_mask(4), false, A>(ar, a, TwSharedA{stw, c});
            else inv16<0, 4, inv_mask(4), false, A>(ar, a, TwGlobal<A>{ar, (N + x0) >> 8});
            // values stay lazy; the strided phase finishes the transform
#pragma unroll
            for (int j = 0; j < 16; j++) gl[x0 + j * 16 + l] = ar.to_word(a[j]);
        }
    }
}

// grid: (tile position, limb, group of `walk` polynomials)
template <bool INV>
__global__ void __launch_bounds__(kThreads, 2) ntt_contig(NttArgs P, int poly_num, int walk) {
    extern __shared__ __align__(16) u64 S[];       // 2 buffers x 4096 words, then the tile's twiddles
    let_next_kernel_start();
    const int poly0 = blockIdx.z * walk;
    const int npoly = poly_num - poly0 < walk ? poly_num - poly0 : walk;
    const u64 q = P.moduli[P.start_mod_idx + blockIdx.y];
    if (q < kF64Bound) contig_body<INV, F64Arith>(P, S, poly0, npoly);
    else if (q < kLazyBound) contig_body<INV, IntArith<true>>(P, S, poly0, npoly);
    else contig_body<INV, IntArith<false>>(P, S, poly0, npoly);
}

// ---------------------------------------------------------------------------
// Strided phase: SA = logN-8 stages on vectors of R = 2^SA points with stride 256.
// A tile is R rows x CW consecutive columns, CW = 4096/R, indexed idx = row*CW + col (12 bits); the
// stage bits are the top SA bits of idx.  Window 0 covers idx bits 8..11 (four stages), window 1
// bits 4..7 (the remaining SA-4 stages, none for logN = 12).  Shared memory holds the tile at its
// idx, which both windows read and write without bank conflicts.  The phase has 2^SA - 1 twiddles
// per limb in all, so they are read from the table (they stay in L1).
// ---------------------------------------------------------------------------
template <int SA>
struct StridedCfg {
    static constexpr int R = 1 << SA;
    static constexpr int CW = 4096 / R;
    static constexpr int LOGCW = 12 - SA;
    static constexpr int NST1 = SA - 4;            // stages of window 1
    __device__ static __forceinline__ size_t goff(uint32_t idx) {      // offset of tile element idx from the tile's origin
        return ((size_t)(idx >> LOGCW) << 8) + (idx & (CW - 1));
    }
};

template <int SA>
__device__ __forceinline__ void prefetch_tile(u64* sbuf, const u64* gtile, uint32_t tid) {
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const uint32_t p = 2 * (i * kThreads + tid);
        __pipeline_memcpy_async(sbuf + p, gtile + StridedCfg<SA>::goff(p), 16);
    }
}

template <int SA, bool INV, class A>
__device__ __forceinline__ void strided_body(const NttArgs& P, u64* S, int tiles) {
    typedef StridedCfg<SA> C;
    typedef typename A::V V;
    const uint32_t tid = threadIdx.x;
    const int limb = blockIdx.y, poly = blockIdx.z;
    A ar;
    ar.init(P, P.start_mod_idx + limb);
    u64* g = P.data + (((size_t)poly * P.poly_mod_len + P.start_limb_off + limb) << P.logN) +
             (size_t)blockIdx.x * tiles * C::CW;
    const uint32_t b1 = ((tid >> 4) << 8) | (tid & 15);          // window 1: v[j] at b1 | j << 4
    typedef typename A::TW TW;
    TW* stw = reinterpret_cast<TW*>(S + 2 * kTile);
    if (tid < kTwStrided) stw[tid] = ar.twiddle(tid);            // visible after the first barrier of the tile loop
    const TwSharedS<TW> sw0{stw, 1u}, sw1{stw, 16u + (tid >> 4)};
    V a[16];
    wait_for_previous_kernel();
    prefetch_tile<SA>(S, g, tid);
    __pipeline_commit();
    for (int t = 0; t < tiles; t++) {
        u64* s = S + (t & 1) * kTile;
        u64* gt = g + (size_t)t * C::CW;
        __pipeline_wait_prior(0);                                 // this thread's copies of tile t have landed
        __syncthreads();                                          // ... and everybody's; everybody is also done with tile t-1,
        if (t + 1 < tiles) prefetch_tile<SA>(S + ((t + 1) & 1) * kTile, gt + C::CW, tid);   // whose buffer takes tile t+1
        __pipeline_commit();
        if (!INV) {
            // window 0: v[j] at idx j*256 + tid; one twiddle set for the whole grid
#pragma unroll
            for (int j = 0; j < 16; j++) a[j] = ar.from_canonical(s[j * 256 + tid]);
            fwd16<0, 4, fwd_mask(8 + SA - 1, true), A>(ar, a, sw0);
            if (C::NST1 > 0) {
#pragma unroll
                for (int j = 0; j < 16; j++) s[j * 256 + tid] = ar.to_word(a[j]);
                __syncthreads();
#pragma unroll
                for (int j = 0; j < 16; j++) a[j] = ar.from_word(s[b1 | (j << 4)]);
                fwd16<0, C::NST1, fwd_mask(8 + SA - 5, false), A>(ar, a, sw1);
#pragma unroll
                for (int j = 0; j < 16; j++) gt[C::goff(b1 | (j << 4))] = ar.to_word(a[j]);
            } else {
#pragma unroll
                for (int j = 0; j < 16; j++) gt[C::goff(j * 256 + tid)] = ar.to_word(a[j]);
            }
        } else {
            if (C::NST1 > 0) {
#pragma unroll
                for (int j = 0; j < 16; j++) a[j] = ar.from_word(s[b1 | (j << 4)]);
                // window 1 runs its NST1 stages as numbers 8.. of the inverse: its stage NST1-1 first
                inv16<0, C::NST1, inv_mask(8 + C::NST1 - 4), false, A>(ar, a, sw1);
#pragma unroll
                for (int j = 0; j < 16; j++) s[b1 | (j << 4)] = ar.to_word(a[j]);
                __syncthreads();
            }
#pragma unroll
            for (int j = 0; j < 16; j++) a[j] = ar.from_word(s[j * 256 + tid]);
            inv16<0, 4, inv_mask(8 + C::NST1), true, A>(ar, a, sw0);
            // Final scaling: the last stage's twiddle psiinv[1] already carries N^-1 for the upper half (a[8..15]);
            // the lower half still needs it (src/ckks/include/ntt_60bit.cuh:890-898): the integer back ends multiply
            // here, the FP64 back end did in its last butterfly.
#pragma unroll
            for (int j = 0; j < 16; j++) {
                const u64 r = j < 8 ? ar.canonical_inv_lo(a[j]) : ar.canonical_inv_hi(a[j]);
                gt[C::goff(j * 256 + tid)] = r;
            }
        }
    }
}

// grid: (group of `tiles` tiles, limb, polynomial).  Three CTAs per SM (80 registers, no spills): the CTA-wide
// barriers of this phase leave the FP64 pipe idle unless other CTAs fill in.
template <int SA, bool INV>
__global__ void __launch_bounds__(kThreads, 3) ntt_strided(NttArgs P, int tiles) {
    extern __shared__ __align__(16) u64 S[];       // 2 buffers x 4096 words, then 256 twiddles of up to 16 bytes
    let_next_kernel_start();
    const u64 q = P.moduli[P.start_mod_idx + blockIdx.y];
    if (q < kF64Bound) strided_body<SA, INV, F64Arith>(P, S, tiles);
    else if (q < kLazyBound) strided_body<SA, INV, IntArith<true>>(P, S, tiles);
    else strided_body<SA, INV, IntArith<false>>(P, S, tiles);
}

constexpr size_t kSmemStrided = (2 * kTile + 2 * kTwStrided) * sizeof(u64);
constexpr size_t kSmemContig = 3 * kTile * sizeof(u64);

// Both kernels of a transform are launched as programmatic dependents of whatever kernel precedes them in the
// stream: they wait for it (wait_for_previous_kernel) after their set-up, before the first access to the data.
template <class... Params, class... Args>
int launch_kernel(void (*kernel)(Params...), dim3 grid, size_t smem, cudaStream_t st, Args... args) {
    CKB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    CKB_CUDA(launch_after(kernel, grid, dim3(kThreads), smem, st, args...));
    return CKKS_B200_OK;
}

template <int SA>
int launch_strided(bool inverse, int ntile, int tiles, int mod_num, int poly_num, const NttArgs& P, cudaStream_t st) {
    dim3 grid(ntile / tiles, mod_num, poly_num);
    return inverse ? launch_kernel(ntt_strided<SA, true>, grid, kSmemStrided, st, P, tiles)
                   : launch_kernel(ntt_strided<SA, false>, grid, kSmemStrided, st, P, tiles);
}

int launch_contig(bool inverse, int ntile, int walk, int mod_num, int poly_num, const NttArgs& P, cudaStream_t st) {
    dim3 grid(ntile, mod_num, (poly_num + walk - 1) / walk);
    return inverse ? launch_kernel(ntt_contig<true>, grid, kSmemContig, st, P, poly_num, walk)
                   : launch_kernel(ntt_contig<false>, grid, kSmemContig, st, P, poly_num, walk);
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

    // A CTA walks over several tiles (strided phase) or polynomials (contiguous phase) so that its prefetch has
    // something to run ahead of, unless the call is so small that walking would leave SMs without a CTA: then more,
    // shorter CTAs.
    static int sms = 0;
    if (sms == 0 && cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, c->device) != cudaSuccess) sms = 148;
    const int ntile = c->N / kTile;
    const long transforms = (long)mod_num * poly_num;
    int tiles = ntile >= 4 ? 4 : ntile;
    while (tiles > 1 && transforms * (ntile / tiles) < 2L * sms) tiles >>= 1;
    int walk = poly_num >= 8 ? 8 : poly_num;
    while (walk > 1 && (long)ntile * mod_num * ((poly_num + walk - 1) / walk) < 4L * sms) walk = (walk + 1) / 2;
    auto strided = [&]() -> int {
        switch (c->logN - 8) {
            case 4: return launch_strided<4>(inverse, ntile, tiles, mod_num, poly_num, P, st);
            case 5: return launch_strided<5>(inverse, ntile, tiles, mod_num, poly_num, P, st);
            case 6: return launch_strided<6>(inverse, ntile, tiles, mod_num, poly_num, P, st);
            case 7: return launch_strided<7>(inverse, ntile, tiles, mod_num, poly_num, P, st);
            default: return launch_strided<8>(inverse, ntile, tiles, mod_num, poly_num, P, st);
        }
    };
    int rc = inverse ? launch_contig(true, ntile, walk, mod_num, poly_num, P, st) : strided();
    if (rc) return rc;
    rc = inverse ? strided() : launch_contig(false, ntile, walk, mod_num, poly_num, P, st);
    if (rc) return rc;
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
