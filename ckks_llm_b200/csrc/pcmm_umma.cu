// PCMM on the 5th-generation tensor cores (tcgen05, sm_100a).
//
// out[m][i][c] = (sum_n w[m][n] * X[n][i][c]) mod q_i is an exact integer GEMM per limb.
// Both operands are cut into 8-bit planes: w (int64, two's complement) into SW planes of
// which the top one is signed, X (residues below 2^(8*SC)) into SC unsigned planes.  The
// product of weight plane a and ciphertext plane b carries weight 2^(8(a+b)), so all
// plane pairs with the same d = a+b may share one s32 accumulator ("diagonal").
//
// Mapping onto one UMMA (M=128, K=32, kind::i8): operand A is a 128-row tile of weight
// plane a; operand B is the 32-column ciphertext tile of all SC planes stacked
// (N = 32*SC rows); the destination is placed at TMEM column 32*a, so plane pair (a,b)
// lands in columns [32(a+b), 32(a+b)+32) and equal diagonals accumulate in place.
// A tile therefore costs SW instructions per 32-deep K step and (SW+SC-1)*32 TMEM
// columns.  The epilogue reads the diagonals back, recombines them into a 128-bit
// signed integer, adds a multiple of q to make it positive, Barrett-reduces, applies the
// reference's rescale by the last limb, and stores.
//
// Operands reach shared memory by bulk asynchronous copies (the TMA engine) of
// contiguous blobs that two pre-pass kernels have laid out in exactly the core-matrix
// order the MMA descriptors expect (K-major, no swizzle: 8 rows x 16 bytes per core
// matrix, 128 B between the two K halves, 256 B between 8-row groups).
//
// Roles inside a CTA (persistent, one per SM): warp 0 issues the copies, warp 1 owns
// TMEM and issues the MMAs, warps 2..9 are the epilogue.  Every wait on an mbarrier is
// bounded by a clock budget; a wait that runs out raises a flag the host turns into
// CKKS_B200_ERR_TIMEOUT, and the CTA drains and exits.
#include "pcmm.cuh"
#include "ringpack.cuh"
#include "umma.cuh"

using namespace ckb;
using namespace ckb::umma;

namespace {

constexpr int TC = 32;             // ciphertext columns per tile
constexpr int KB = 64;             // contraction depth per pipeline stage
constexpr int KS = KB / 32;        // UMMA K steps per stage
constexpr int A_PLANE_STEP = TM * 32;   // bytes of one weight plane, one K step
constexpr int B_PLANE_STEP = TC * 32;   // bytes of one ciphertext plane, one K step
constexpr int NUM_EPI_WARPS = 8;
constexpr int NUM_THREADS = 32 * (2 + NUM_EPI_WARPS);
// Per-warp staging tile of the epilogue: 32 rows x 16 words, rows padded to 144 bytes so
// that both the row-per-lane writes and the row-contiguous reads are bank-conflict free.
constexpr int STG_ROW = 144;
constexpr int STG_WARP = 32 * STG_ROW;
constexpr int STG_BYTES = NUM_EPI_WARPS * STG_WARP;

// Where the epilogue stores a word besides (or instead of) the call's own output buffer.
constexpr int DEST_LOCAL = 0;      // the call's output buffer only
constexpr int DEST_BROADCAST = 1;  // also, at the same offset, into every buffer of dests[0..n_dests)
constexpr int DEST_OWNERS = 2;     // row m goes, at the same offset, into dests[m / rows_per_owner] only

struct UmmaArgs {
    const uint8_t* wplanes;    // [mt][kb][a][ks][4096]
    const uint8_t* xplanes;    // [limb][ct][kb][ks][b][1024]
    u64* out;                  // [M][limbs][C]
    u64* dests[8];             // output buffers of the same shape, most of them on other GPUs (see DEST_*)
    int n_dests;
    int rows_per_owner;
    const PcmmLimb* limbs;
    int* flags;
    int M, limbs_n;
    long C;
    long col_begin, col_end;   // columns covered by xplanes: ct 0 starts at col_begin
    int MT, CT, KBN;           // tiles in M, tiles in columns, pipeline stages per tile
    int num_stages;
    int kpass;                 // K blocks accumulated in tensor memory before the epilogue takes the partial sums over
    long long wait_budget;     // clock cycles a wait on an mbarrier may take
    int withhold;              // test switch: the producer stops before its copy number `withhold` (-1: off)
};

template <int SW, int SC>
struct Cfg {
    static constexpr int ND = SW + SC - 1;
    static constexpr int A_STAGE = SW * KS * A_PLANE_STEP;
    static constexpr int B_STAGE = SC * KS * B_PLANE_STEP;
    static constexpr int STAGE = A_STAGE + B_STAGE;
    static constexpr int TMEM_COLS = ND * TC <= 128 ? 128 : ND * TC <= 256 ? 256 : 512;
    static constexpr int SMEM_BUDGET = 227 * 1024 - 2048 - STG_BYTES;
    static constexpr int MAX_STAGES = SMEM_BUDGET / STAGE < 8 ? SMEM_BUDGET / STAGE : 8;
};

// ---------------------------------------------------------------------------
// Pre-pass 1: weight planes.  One thread per (row, 16-wide K chunk) writes 16 bytes per
// plane.  Rows and K beyond the matrix are zero.
// ---------------------------------------------------------------------------
__global__ void slice_weights_kernel(const long long* __restrict__ w, uint8_t* __restrict__ planes, int M,
                                     int K, int MT, int KBN, int SW) {
    const long chunks_per_row = (long)KBN * (KB / 16);
    const long total = (long)MT * TM * chunks_per_row;
    long id = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (id >= total) return;
    const int row = (int)(id % (MT * TM));      // rows fastest: consecutive threads fill one core matrix column
    const long ch = id / (MT * TM);
    const int kb = (int)(ch / (KB / 16)), k16 = (int)(ch % (KB / 16));
    const int ks = k16 / 2, kc = k16 % 2;
    const int mt = row / TM, r = row % TM;
    long long v[16];
#pragma unroll
    for (int e = 0; e < 16; e++) {
        int n = kb * KB + k16 * 16 + e;
        v[e] = (row < M && n < K) ? w[(size_t)row * K + n] : 0;
    }
    for (int a = 0; a < SW; a++) {
        uint32_t pk[4];
#pragma unroll
        for (int wd = 0; wd < 4; wd++) {
            uint32_t x = 0;
#pragma unroll
            for (int e = 0; e < 4; e++) x |= (uint32_t)((v[wd * 4 + e] >> (8 * a)) & 0xff) << (8 * e);
            pk[wd] = x;
        }
        size_t off = ((((size_t)mt * KBN + kb) * SW + a) * KS + ks) * A_PLANE_STEP + (size_t)(r / 8) * 256 +
                     kc * 128 + (r % 8) * 16;
        *reinterpret_cast<uint4*>(planes + off) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
    }
}

// Pre-pass 2: ciphertext planes for columns [col_begin, col_begin + CT*32).  One thread
// per (limb, column, 16-wide K chunk); lanes run over columns so every ciphertext read is
// coalesced.
__global__ void slice_cipher_kernel(const u64* const* __restrict__ X, const u64* __restrict__ xbase, size_t xstride,
                                    uint8_t* __restrict__ planes, int K, long C, int limbs_n, long col_begin, long col_end,
                                    int CT, int KBN, int SC) {
    const long ncol = (long)CT * TC;
    const long col = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (col >= ncol) return;
    const int k16g = blockIdx.y;                 // global 16-chunk index along K
    const int limb = blockIdx.z;
    const int kb = k16g / (KB / 16), k16 = k16g % (KB / 16);
    const int ks = k16 / 2, kc = k16 % 2;
    const long c = col_begin + col;
    u64 v[16];
#pragma unroll
    for (int e = 0; e < 16; e++) {
        int n = k16g * 16 + e;
        // ciphertext n: entry n of the pointer table, or base + n * stride when there is no table
        v[e] = (n < K && c < col_end) ? (X ? X[n] : xbase + (size_t)n * xstride)[(size_t)limb * C + c] : 0;
    }
    const int ct = (int)(col / TC), cc = (int)(col % TC);
    for (int b = 0; b < SC; b++) {
        uint32_t pk[4];
#pragma unroll
        for (int wd = 0; wd < 4; wd++) {
            uint32_t x = 0;
#pragma unroll
            for (int e = 0; e < 4; e++) x |= (uint32_t)((v[wd * 4 + e] >> (8 * b)) & 0xff) << (8 * e);
            pk[wd] = x;
        }
        size_t off = (((((size_t)limb * CT + ct) * KBN + kb) * KS + ks) * SC + b) * B_PLANE_STEP +
                     (size_t)(cc / 8) * 256 + kc * 128 + (cc % 8) * 16;
        *reinterpret_cast<uint4*>(planes + off) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
    }
}

// Pre-pass 2 when the multiply reads RLWE ciphertexts directly: the same planes, with word
// (n, limb, c) taken through the decomposition's index map instead of from a stored MLWE
// ciphertext, so the MLWE ciphertexts never exist in HBM (the RLWE ciphertexts stay in L2:
// 16*N bytes per limb against (rank+1)*N1*8 bytes per limb for EACH of the K ciphertexts made
// from them).  One block per (column tile, K block, limb): the source is contiguous in n (for a
// gap of one), the plane blob wants 16 n per 16-byte store, so a 32-column x 64-n tile goes
// through shared memory, read with lanes along n and sliced with lanes along the columns.
__global__ void __launch_bounds__(256) slice_rlwe_kernel(const RlweSlot* __restrict__ slots, uint8_t* __restrict__ planes,
                                                         const PcmmLimb* __restrict__ limbs, int K, long N, int N1,
                                                         int rank, long col_begin, long col_end, int CT, int KBN, int SC) {
    static_assert(KB == 64 && TC == 32, "the thread mapping below is written for 64 x 32 tiles");
    __shared__ u64 tile[TC][KB + 1];
    const int ct = blockIdx.x, kb = blockIdx.y, limb = blockIdx.z;
    const int t = threadIdx.x;
    const u64 q = limbs[limb].q;
    {
        const int nl = t & (KB - 1), n = kb * KB + nl;
        RlweSlot s = {nullptr, 0, 0, 0, 0};
        if (n < K) s = slots[n];
        const u64* A = s.rlwe + N * limb;
        const u64* B = s.rlwe + N * (s.L + 1 + limb);
        // column c = r*N1 + g: one division for the tile's first column, steps from there
        const long c0 = col_begin + (long)ct * TC;
        const int r0 = (int)(c0 / N1), g0 = (int)(c0 - (long)r0 * N1);
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const int cl = (t >> 6) + 4 * j;
            int r = r0, g = g0 + cl;
            while (g >= N1) { g -= N1; r++; }
            u64 v = 0;
            if (n < K && c0 + cl < col_end) v = decompose_word(A, B, q, N, N1, rank, s.gap, s.i, r, g);
            tile[cl][nl] = v;
        }
    }
    __syncthreads();
    const int cc = t & 31, k16 = (t >> 5) & 3, half = t >> 7;
    const int ks = k16 / 2, kc = k16 % 2;
    u64 v[16];
#pragma unroll
    for (int e = 0; e < 16; e++) v[e] = tile[cc][k16 * 16 + e];
    for (int b = half; b < SC; b += 2) {
        uint32_t pk[4];
#pragma unroll
        for (int wd = 0; wd < 4; wd++) {
            uint32_t x = 0;
#pragma unroll
            for (int e = 0; e < 4; e++) x |= (uint32_t)((v[wd * 4 + e] >> (8 * b)) & 0xff) << (8 * e);
            pk[wd] = x;
        }
        size_t off = (((((size_t)limb * CT + ct) * KBN + kb) * KS + ks) * SC + b) * B_PLANE_STEP +
                     (size_t)(cc / 8) * 256 + kc * 128 + (cc % 8) * 16;
        *reinterpret_cast<uint4*>(planes + off) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
    }
}

// The same pre-pass for the usual case (N1 a multiple of 32, every aligned run of 16
// ciphertexts inside one source, gaps of at most 2), using the structure of the
// decomposition: with the negacyclic convention A[x +- N] = -A[x], word g of polynomial
// r < k of ciphertext i is
//   a_i,r[g] = A[g*k + i*gap - r]          (b_i[g] = B[g*k + i*gap])
// so ciphertexts i and polynomials r see the same RLWE words shifted against one another.
// A block takes 32 values of g, one K block of 64 ciphertexts (four runs of 16, each from
// its own source) and RB polynomials: per run and g it loads the 15*gap + RB words those
// share (12 % of the words it emits, at a gap of one) into shared memory and cuts the
// planes of its RB column tiles from them.  The last "row block" is the b polynomial alone.
constexpr int RB = 16;
constexpr int SEG_MAX_GAP = 2;
constexpr int SEG = 15 * SEG_MAX_GAP + RB + 1;     // odd: lanes along g fall into distinct banks (32-bit words)

__global__ void __launch_bounds__(256) slice_rlwe_rows_kernel(const RlweSlot* __restrict__ slots, uint8_t* __restrict__ planes,
                                                              const PcmmLimb* __restrict__ limbs, int K, long N, int N1,
                                                              int rank, long col_begin, long col_end, int CT, int KBN,
                                                              int SC) {
    static_assert(KB == 64 && TC == 32, "the thread mapping below is written for 64 x 32 tiles");
    // low and high words apart: a thread cuts either planes 0-3 or planes 4-7 and reads only the words it needs
    __shared__ uint32_t seg[2][4][TC][SEG];
    const int g_tiles = N1 / TC, rbn = (rank + RB - 1) / RB;
    const int gt = blockIdx.x % g_tiles, rb = blockIdx.x / g_tiles;
    const int kb = blockIdx.y, limb = blockIdx.z;
    const bool bpoly = rb == rbn;
    const int r0 = bpoly ? 0 : rb * RB;                                   // first polynomial, as it enters the index
    const int rows = bpoly ? 1 : (rank - r0 < RB ? rank - r0 : RB);
    const int crow0 = bpoly ? rank : r0;                                  // its row among the (k+1) rows of columns
    const int g0 = gt * TC;
    {
        const long c_first = (long)crow0 * N1 + g0, c_last = (long)(crow0 + rows - 1) * N1 + g0;
        if (c_last < col_begin || c_first >= col_end) return;             // block-uniform
    }
    const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
    const int n0 = kb * KB;
    const u64 q = limbs[limb].q;
    {
        // warp w loads run w & 3 for every other g: seg[.][run][g][x] = A[(g0+g)*k + i0*gap - (r0 + RB - 1) + x], signed
        const int run = warp & 3, nr = n0 + run * 16;
        if (nr < K) {
            const RlweSlot s = slots[nr];
            const int span = 15 * s.gap + RB;
            const u64* src = s.rlwe + N * ((bpoly ? s.L + 1 : 0) + limb);
            // four values of g per step, so that four loads are in flight before the first is used
            for (int x = lane; x < span; x += 32) {
                for (int gq = warp >> 2; gq < TC; gq += 8) {
                    u64 v[4];
                    bool neg[4];
#pragma unroll
                    for (int u = 0; u < 4; u++) {
                        long idx = (long)(g0 + gq + 2 * u) * rank + (long)s.i * s.gap - (r0 + RB - 1) + x;
                        neg[u] = false;
                        if (idx < 0) { idx += N; neg[u] = true; }
                        else if (idx >= N) { idx -= N; neg[u] = true; }
                        v[u] = src[idx];
                    }
#pragma unroll
                    for (int u = 0; u < 4; u++) {
                        const u64 w = neg[u] ? (v[u] == 0 ? 0 : q - v[u]) : v[u];
                        seg[0][run][gq + 2 * u][x] = (uint32_t)w;
                        seg[1][run][gq + 2 * u][x] = (uint32_t)(w >> 32);
                    }
                }
            }
        }
    }
    __syncthreads();
    const int cc = t & 31, k16 = (t >> 5) & 3, half = t >> 7;
    const int ks = k16 / 2, kc = k16 % 2;
    const uint32_t* row = seg[half][k16][cc];
    const int valid = K - n0 - k16 * 16;                                   // ciphertexts of this run that exist
    const int gap = valid > 0 ? slots[n0 + k16 * 16].gap : 1;
    // planes of one column tile from the 16 words of this thread's (column, run of 16 ciphertexts)
    auto emit = [&](const uint32_t (&w)[16], int ct) {
        uint8_t* dst = planes + ((((size_t)limb * CT + ct) * KBN + kb) * KS + ks) * SC * B_PLANE_STEP +
                       (size_t)(cc / 8) * 256 + kc * 128 + (cc % 8) * 16;
#pragma unroll
        for (int bb = 0; bb < 4; bb++) {
            const int b = half * 4 + bb;
            if (b < SC) {
                uint32_t pk[4];
#pragma unroll
                for (int wd = 0; wd < 4; wd++) {
                    const uint32_t lo = __byte_perm(w[wd * 4 + 0], w[wd * 4 + 1], bb | ((4 + bb) << 4));
                    const uint32_t hi = __byte_perm(w[wd * 4 + 2], w[wd * 4 + 3], bb | ((4 + bb) << 4));
                    pk[wd] = __byte_perm(lo, hi, 0x5410);
                }
                *reinterpret_cast<uint4*>(dst + (size_t)b * B_PLANE_STEP) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
            }
        }
    };
    if (gap == 1 && rows == RB && valid >= 16) {
        // Gap one, a whole row block, a whole run: polynomial r0 + rr needs words 15 - rr .. 30 - rr of the run, so
        // the 31 words are read once and every polynomial takes its window of them from registers.
        uint32_t win[RB + 15];
#pragma unroll
        for (int j = 0; j < RB + 15; j++) win[j] = row[j];
#pragma unroll
        for (int rr = 0; rr < RB; rr++) {
            const long c = (long)(crow0 + rr) * N1 + g0;
            if (c < col_begin || c >= col_end) continue;                   // block-uniform
            uint32_t w[16];
#pragma unroll
            for (int e = 0; e < 16; e++) w[e] = win[(RB - 1) - rr + e];
            emit(w, (int)((c - col_begin) / TC));
        }
        return;
    }
    for (int rr = 0; rr < rows; rr++) {
        const long c = (long)(crow0 + rr) * N1 + g0;
        if (c < col_begin || c >= col_end) continue;                       // block-uniform
        uint32_t w[16];
        int x = (RB - 1) - rr;
#pragma unroll
        for (int e = 0; e < 16; e++, x += gap) w[e] = e < valid ? row[x] : 0u;
        emit(w, (int)((c - col_begin) / TC));
    }
}

// Reads the ND diagonal accumulators of 16 output columns (this thread's row) out of tensor memory and recombines
// them, sum_d v_d * 2^(8d), into signed 128-bit sums; ADD accumulates onto acc instead of overwriting it.
// The caller tells the MMA issuer that tensor memory is free only after the recombination: signalling as soon as the
// second half of the columns sits in registers (nothing is left to read then) measured 2 to 3 % SLOWER in a same-box
// comparison, because the next tile's instructions then issue while the epilogue warps that share the issuer's
// scheduler are still in their arithmetic.
template <int ND, bool ADD>
__device__ __forceinline__ void drain_accumulators(uint32_t taddr, unsigned __int128 (&acc)[16]) {
#pragma unroll
    for (int g = 0; g < 2; g++) {
        int32_t v[ND][8];
#pragma unroll
        for (int d = 0; d < ND; d++) tmem_ld8(taddr + d * TC + g * 8, v[d]);
        tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 8; e++) {
            // groups of four diagonals fit a signed 64-bit word (|v_d| < 2^31, top shift 24), and the groups sit
            // 32 bits apart
            long long grp[(ND + 3) / 4];
#pragma unroll
            for (int gi = 0; gi < (ND + 3) / 4; gi++) {
                long long t = 0;
#pragma unroll
                for (int k = 3; k >= 0; k--)
                    if (gi * 4 + k < ND) t = t * 256 + (long long)v[gi * 4 + k][e];
                grp[gi] = t;
            }
            __int128 s = 0;
#pragma unroll
            for (int gi = (ND + 3) / 4 - 1; gi >= 0; gi--) s = s * ((__int128)1 << 32) + grp[gi];
            if (ADD) acc[g * 8 + e] += (unsigned __int128)s;
            else acc[g * 8 + e] = (unsigned __int128)s;
        }
    }
}

// ---------------------------------------------------------------------------
// Main kernel
// ---------------------------------------------------------------------------
// DEST: one of DEST_LOCAL / DEST_BROADCAST / DEST_OWNERS.  KSPLIT: the contraction is accumulated in passes of P.kpass
// K blocks (a K too deep for one pass of s32 accumulators); without it one pass takes all P.KBN blocks.
template <int SW, int SC, int DEST, bool KSPLIT>
__global__ void __launch_bounds__(NUM_THREADS, 1) pcmm_umma_kernel(UmmaArgs P) {
    using C_ = Cfg<SW, SC>;
    constexpr bool PEERS = DEST != DEST_LOCAL;
    extern __shared__ __align__(1024) uint8_t smem[];
    __shared__ uint64_t bars[2 * 8 + 3];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag, never_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int NS = P.num_stages;
    const uint32_t smem_base = smem_u32(smem);
    const uint32_t full_bar = smem_u32(&bars[0]);          // [NS]
    const uint32_t empty_bar = smem_u32(&bars[8]);         // [NS]
    const uint32_t tmem_full_bar = smem_u32(&bars[16]);
    const uint32_t tmem_empty_bar = smem_u32(&bars[17]);
    const uint32_t mma_done_bar = smem_u32(&bars[18]);     // used on the way out of a launch that gave up
    const long long budget = P.wait_budget;

    if (threadIdx.x == 0) {
        for (int s = 0; s < NS; s++) {
            mbar_init(full_bar + 8 * s, 1);
            mbar_init(empty_bar + 8 * s, 1);
        }
        mbar_init(tmem_full_bar, 1);
        mbar_init(tmem_empty_bar, NUM_EPI_WARPS);
        mbar_init(mma_done_bar, 1);
        abort_flag = 0;
        never_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&tmem_base_slot), C_::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;

    const long num_items = (long)P.MT * P.CT;
    const int limbs_n = P.limbs_n;

    if (warp == 0) {
        // ---------------- producer ----------------
        if (lane == 0) {
            uint32_t s = 0, ph = 0, issued = 0;    // ring position, its phase parity, stages issued so far
            bool ok = true, withheld = false;
            const int krot = (int)((blockIdx.x / P.MT) % P.KBN);
            for (long item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
                const int mt = (int)(item % P.MT);
                const long ct = item / P.MT;
                const uint8_t* const asrc0 = P.wplanes + (size_t)mt * P.KBN * C_::A_STAGE;
                for (int limb = limbs_n - 1; limb >= 0 && ok; limb--) {
                    const uint8_t* const bsrc0 = P.xplanes + ((size_t)limb * P.CT + ct) * P.KBN * C_::B_STAGE;
                    // The sum over K is exact, so its order is free: every CTA starts at another
                    // K block, which keeps the CTAs from asking L2 for the same weight block at once.
                    int kbr = krot;
                    for (int kb = 0; kb < P.KBN; kb++) {
                        // Test switch: stop producing in front of this stage and say nothing, so that the wait of
                        // the MMA issuer on this stage's barrier runs into its clock budget.
                        if ((int)issued == P.withhold) { withheld = true; ok = false; break; }
                        if (issued >= (uint32_t)NS && !mbar_wait(empty_bar + 8 * s, ph ^ 1, P.flags, 1, &abort_flag, budget)) { ok = false; break; }
                        const uint32_t dst = smem_base + s * C_::STAGE;
                        mbar_arrive_expect_tx(full_bar + 8 * s, C_::STAGE);
                        bulk_g2s(dst, asrc0 + (size_t)kbr * C_::A_STAGE, C_::A_STAGE, full_bar + 8 * s);
                        bulk_g2s(dst + C_::A_STAGE, bsrc0 + (size_t)kbr * C_::B_STAGE, C_::B_STAGE, full_bar + 8 * s);
                        if (++kbr == P.KBN) kbr = 0;
                        issued++;
                        if (++s == (uint32_t)NS) { s = 0; ph ^= 1; }
                    }
                }
            }
            if (!ok && !withheld) atomicExch(&abort_flag, 1);
            // Drain: every copy this thread issued must have landed before the CTA exits.  The last
            // min(issued, NS) copies sit in the ring positions before s, going backwards.
            uint32_t n = issued < (uint32_t)NS ? issued : (uint32_t)NS;
            uint32_t ds = s, dph = ph;
            for (uint32_t j = 0; j < n; j++) {
                if (ds == 0) { ds = NS; dph ^= 1; }
                ds--;
                mbar_wait(full_bar + 8 * ds, dph, P.flags, 2, &never_flag, budget);
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            uint32_t s = 0, ph = 0, tile = 0;
            bool ok = true;
            constexpr uint32_t idesc_full_u = instr_desc(TC * SC, false);
            constexpr uint32_t idesc_full_s = instr_desc(TC * SC, true);
            constexpr uint32_t idesc_head_u = instr_desc(TC * (SC - 1), false);
            constexpr uint32_t idesc_head_s = instr_desc(TC * (SC - 1), true);
            constexpr uint32_t idesc_tail_u = instr_desc(TC, false);
            constexpr uint32_t idesc_tail_s = instr_desc(TC, true);
            const uint32_t base16 = smem_base >> 4;
            // A "tile" of the tensor-memory handshake is one accumulation pass: all K blocks of an (item, limb)
            // pair, or P.kpass of them at a time when the whole K would overflow the s32 accumulators.
            for (long item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
                for (int limb = limbs_n - 1; limb >= 0 && ok; limb--) {
                  const int kstep = KSPLIT ? P.kpass : P.KBN;
                  for (int kb0 = 0; kb0 < P.KBN && ok; kb0 += kstep, tile++) {
                    if (tile > 0 && !mbar_wait(tmem_empty_bar, (tile - 1) & 1, P.flags, 3, &abort_flag, budget)) { ok = false; break; }
                    tc_fence_after();
                    const int kb1 = (KSPLIT && kb0 + kstep < P.KBN) ? kb0 + kstep : P.KBN;
                    for (int kb = kb0; kb < kb1; kb++) {
                        if (!mbar_wait(full_bar + 8 * s, ph, P.flags, 4, &abort_flag, budget)) { ok = false; break; }
                        tc_fence_after();
                        const uint32_t a16 = base16 + s * (C_::STAGE >> 4);
                        const uint32_t b16 = a16 + (C_::A_STAGE >> 4);
                        if (kb == kb0) {
                            // First K step of the tile: plane 0 overwrites its columns; every later plane
                            // accumulates into the columns it shares with earlier planes and overwrites
                            // the new top diagonal (ciphertext plane SC-1) with a second instruction.
#pragma unroll
                            for (int a = 0; a < SW; a++) {
                                const uint64_t adesc = smem_desc(a16 + ((a * KS) * A_PLANE_STEP >> 4));
                                const bool sgn = (a == SW - 1);
                                const uint32_t d = tmem_base + a * TC;
                                if (a == 0) {
                                    umma_i8(d, adesc, smem_desc(b16), idesc_full_u, 0);
                                } else {
                                    umma_i8(d, adesc, smem_desc(b16), sgn ? idesc_head_s : idesc_head_u, 1);
                                    umma_i8(d + (SC - 1) * TC, adesc, smem_desc(b16 + ((SC - 1) * B_PLANE_STEP >> 4)),
                                            sgn ? idesc_tail_s : idesc_tail_u, 0);
                                }
                            }
                        }
#pragma unroll
                        for (int ks = 0; ks < KS; ks++) {
                            if (ks == 0 && kb == kb0) continue;
                            const uint64_t bdesc = smem_desc(b16 + (ks * SC * B_PLANE_STEP >> 4));
#pragma unroll
                            for (int a = 0; a < SW; a++)
                                umma_i8(tmem_base + a * TC, smem_desc(a16 + ((a * KS + ks) * A_PLANE_STEP >> 4)), bdesc,
                                        a == SW - 1 ? idesc_full_s : idesc_full_u, 1);
                        }
                        umma_commit(empty_bar + 8 * s);
                        if (++s == (uint32_t)NS) { s = 0; ph ^= 1; }
                    }
                    if (ok) umma_commit(tmem_full_bar);
                  }
                }
            }
            if (!ok) {
                atomicExch(&abort_flag, 1);
                // the instructions already issued still read shared memory and write tensor memory: see them out
                umma_commit(mma_done_bar);
                mbar_wait(mma_done_bar, 0, P.flags, 6, &never_flag, budget);
            }
        }
    } else {
        // ---------------- epilogue ----------------
        const int ew = warp - 2;
        const int quarter = warp & 3;          // TMEM lanes this warp may read
        const int half = ew >> 2;              // which 16 of the 32 columns
        uint8_t* stg = smem + (size_t)NS * C_::STAGE + (size_t)ew * STG_WARP;
        u64 last[16];
        bool vec_ok = (P.C & 1) == 0 && (reinterpret_cast<uintptr_t>(P.out) & 15) == 0;   // 16-byte stores stay aligned
        if (PEERS)
            for (int dest = 0; dest < P.n_dests; dest++) vec_ok = vec_ok && (reinterpret_cast<uintptr_t>(P.dests[dest]) & 15) == 0;
        uint32_t tile = 0;
        bool ok = true;
        for (long item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
            const int mt = (int)(item % P.MT);
            const long ct = item / P.MT;
            const long c0 = P.col_begin + ct * TC + half * 16;
            for (int limb = limbs_n - 1; limb >= 0 && ok; limb--) {
                unsigned __int128 acc[16];
                const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + half * 16;
                if (!KSPLIT) {
                    // the usual case: the whole contraction sits in tensor memory
                    if (!mbar_wait(tmem_full_bar, tile & 1, P.flags, 5, &abort_flag, budget)) { ok = false; break; }
                    tc_fence_after();
                    drain_accumulators<C_::ND, false>(taddr, acc);
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(tmem_empty_bar);
                    tile++;
                } else {
                    // one round per accumulation pass of the MMA issuer; the partial sums add up in 128 bits
#pragma unroll
                    for (int e = 0; e < 16; e++) acc[e] = 0;
                    for (int kb0 = 0; kb0 < P.KBN; kb0 += P.kpass, tile++) {
                        if (!mbar_wait(tmem_full_bar, tile & 1, P.flags, 5, &abort_flag, budget)) { ok = false; break; }
                        tc_fence_after();
                        drain_accumulators<C_::ND, true>(taddr, acc);
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(tmem_empty_bar);
                    }
                }
                if (!ok) break;

                const PcmmLimb L = P.limbs[limb];
                const unsigned __int128 off = ((unsigned __int128)L.off_hi << 64) | L.off_lo;
                u64 res[16];
#pragma unroll
                for (int e = 0; e < 16; e++) {
                    unsigned __int128 t = acc[e] + off;
                    u64 r = barrett128((u64)t, (u64)(t >> 64), L.q, L.mu_hi, L.mu_lo);
                    if (limb == limbs_n - 1) {
                        last[e] = r;                              // kept in registers for the other limbs
                    } else {
                        u64 tmp = r + L.q - last[e];              // wraps mod 2^64 like the reference
                        r = shoup_mul(tmp, L.inv, L.inv_shoup, L.q);
                    }
                    res[e] = r;
                }
                // Transpose through the warp's staging tile so that every store instruction
                // writes whole 128-byte lines: lane = row while writing the tile, lanes run
                // along a row while reading it back.
                if (PEERS) bulk_wait_read();              // the copy engine is done reading this lane's row of the tile
                __syncwarp();
#pragma unroll
                for (int e = 0; e < 8; e++)
                    *reinterpret_cast<ulonglong2*>(stg + lane * STG_ROW + e * 16) = make_ulonglong2(res[2 * e], res[2 * e + 1]);
                if (PEERS) {
                    // A lane's row of the tile is 128 contiguous bytes of the output: one bulk copy per destination
                    // (the local buffer and every peer's, over NVLink) straight from the staging tile.  The copies
                    // run on the copy engine, so the warp does not issue 8 x 8 sixteen-byte stores per row and
                    // goes back to the next tile while they drain.
                    const bool whole = vec_ok && c0 + 16 <= P.col_end && mt * TM + quarter * 32 + 32 <= P.M;    // warp-uniform
                    if (whole) {
                        fence_proxy_async_smem();
                        const int row = mt * TM + quarter * 32 + lane;
                        const size_t off = ((size_t)row * limbs_n + limb) * P.C + c0;
                        const uint32_t src = smem_u32(stg + lane * STG_ROW);
                        if (DEST == DEST_OWNERS) {
                            bulk_s2g(P.dests[row / P.rows_per_owner] + off, src, 128);      // this row's owner, nobody else
                        } else {
                            bulk_s2g(P.out + off, src, 128);
                            for (int dest = 0; dest < P.n_dests; dest++) bulk_s2g(P.dests[dest] + off, src, 128);
                        }
                        bulk_commit();
                        continue;
                    }
                }
                __syncwarp();
                const int sub_r = lane >> 3, pair = lane & 7;
                const long c = c0 + pair * 2;
#pragma unroll
                for (int it = 0; it < 8; it++) {
                    const int r = it * 4 + sub_r;
                    const int mm = mt * TM + quarter * 32 + r;
                    const ulonglong2 v = *reinterpret_cast<const ulonglong2*>(stg + r * STG_ROW + pair * 16);
                    if (mm < P.M) {
                        const size_t off = ((size_t)mm * limbs_n + limb) * P.C + c;
                        // the local output, then the same words into every peer's output buffer (plain
                        // peer stores over NVLink): the gather of a column-sharded multiply rides on the epilogue
                        for (int dest = -1; dest < (DEST == DEST_BROADCAST ? P.n_dests : 0); dest++) {
                            u64* dst = (DEST == DEST_OWNERS ? P.dests[mm / P.rows_per_owner] : dest < 0 ? P.out : P.dests[dest]) + off;
                            if (vec_ok && c + 1 < P.col_end) {
                                *reinterpret_cast<ulonglong2*>(dst) = v;
                            } else {
                                if (c < P.col_end) dst[0] = v.x;
                                if (c + 1 < P.col_end) dst[1] = v.y;
                            }
                        }
                    }
                }
            }
        }
        if (PEERS) bulk_wait_all();                       // every destination is written before the CTA retires
        if (!ok) atomicExch(&abort_flag, 1);
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, C_::TMEM_COLS);
    }
}

template <int SW, int SC>
int launch(ckks_b200_pcmm* pc, const long long* d_w, const PcmmSource& src, u64* d_out, int M, int K, long col_begin,
           long col_end, int kpass, bool weights_ready, cudaStream_t st) {
    using C_ = Cfg<SW, SC>;
    const int MT = (M + TM - 1) / TM;
    const long ncol = col_end - col_begin;
    const int CT = (int)((ncol + TC - 1) / TC);
    const int KBN = (K + KB - 1) / KB;
    const size_t wbytes = (size_t)MT * KBN * C_::A_STAGE;
    const size_t xbytes = (size_t)pc->q_count * CT * KBN * C_::B_STAGE;
    if (weights_ready) {
        CKB_REQUIRE(pc->wplanes_cap >= wbytes && pc->prep_sw == SW && pc->prep_sc == SC, CKKS_B200_ERR_ARG,
                    "the prepared weight planes do not belong to this multiply");
    } else {
        int rc = ensure_dev(&pc->d_wplanes, &pc->wplanes_cap, wbytes);
        if (rc) return rc;
    }
    int rc = ensure_dev(&pc->d_xplanes, &pc->xplanes_cap, xbytes);
    if (rc) return rc;

    CKB_CUDA(cudaEventRecord(pc->ev[0], st));
    {
        if (!weights_ready) {
            long total = (long)MT * TM * KBN * (KB / 16);
            slice_weights_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(d_w, pc->d_wplanes, M, K, MT, KBN, SW);
            count_launch();
        }
        if (d_out == nullptr) {                 // weight preparation only
            CKB_CUDA(cudaGetLastError());
            return CKKS_B200_OK;
        }
        if (src.slots && src.slots_regular) {
            dim3 grid((unsigned)((pc->N1 / TC) * ((pc->rank + RB - 1) / RB + 1)), KBN, pc->q_count);
            slice_rlwe_rows_kernel<<<grid, 256, 0, st>>>(src.slots, pc->d_xplanes, pc->d_limbs, K, (long)pc->rank * pc->N1,
                                                         pc->N1, pc->rank, col_begin, col_end, CT, KBN, SC);
        } else if (src.slots) {
            dim3 grid((unsigned)CT, KBN, pc->q_count);
            slice_rlwe_kernel<<<grid, 256, 0, st>>>(src.slots, pc->d_xplanes, pc->d_limbs, K, (long)pc->rank * pc->N1, pc->N1,
                                                    pc->rank, col_begin, col_end, CT, KBN, SC);
        } else {
            dim3 grid((unsigned)(((long)CT * TC + 127) / 128), KBN * (KB / 16), pc->q_count);
            slice_cipher_kernel<<<grid, 128, 0, st>>>(src.table, src.base, src.stride, pc->d_xplanes, K, pc->C, pc->q_count,
                                                      col_begin, col_end, CT, KBN, SC);
        }
        count_launch();
        CKB_CUDA(cudaGetLastError());
    }

    int sms = 0;
    CKB_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, pc->device));
    UmmaArgs P;
    P.wplanes = pc->d_wplanes;
    P.xplanes = pc->d_xplanes;
    P.out = d_out;
    int dest = DEST_LOCAL;
    P.n_dests = 0;
    P.rows_per_owner = 1;
    for (int i = 0; i < 8; i++) P.dests[i] = nullptr;
    if (pc->n_owners > 0) {
        // rows are dealt out in equal runs, a whole number of 32-row groups each, so that one warp's rows share an owner
        dest = DEST_OWNERS;
        P.n_dests = pc->n_owners;
        P.rows_per_owner = ((M + pc->n_owners - 1) / pc->n_owners + 31) / 32 * 32;
        for (int i = 0; i < pc->n_owners; i++) P.dests[i] = (i == pc->self_rank || !pc->owner_out[i]) ? d_out : pc->owner_out[i];
    } else if (pc->n_peers > 0) {
        dest = DEST_BROADCAST;
        P.n_dests = pc->n_peers;
        for (int i = 0; i < pc->n_peers; i++) P.dests[i] = pc->peer_out[i];
    }
    P.limbs = pc->d_limbs;
    P.flags = pc->d_flags;
    P.M = M;
    P.limbs_n = pc->q_count;
    P.C = pc->C;
    P.col_begin = col_begin;
    P.col_end = col_end;
    P.MT = MT;
    P.CT = CT;
    P.KBN = KBN;
    P.num_stages = C_::MAX_STAGES;
    P.kpass = kpass;
    P.wait_budget = pc->wait_budget > 0 ? pc->wait_budget : WAIT_BUDGET;
    P.withhold = pc->withhold_stage;
    pc->withhold_stage = -1;                    // the test switch arms one launch
    const size_t smem = (size_t)C_::MAX_STAGES * C_::STAGE + STG_BYTES;
    long items = (long)MT * CT;
    int grid = (int)(items < sms ? items : sms);
    CKB_CUDA(cudaEventRecord(pc->ev[1], st));
    const bool ksplit = kpass < KBN;
    void (*kernel)(UmmaArgs) =
        dest == DEST_OWNERS      ? (ksplit ? pcmm_umma_kernel<SW, SC, DEST_OWNERS, true> : pcmm_umma_kernel<SW, SC, DEST_OWNERS, false>)
        : dest == DEST_BROADCAST ? (ksplit ? pcmm_umma_kernel<SW, SC, DEST_BROADCAST, true> : pcmm_umma_kernel<SW, SC, DEST_BROADCAST, false>)
                                 : (ksplit ? pcmm_umma_kernel<SW, SC, DEST_LOCAL, true> : pcmm_umma_kernel<SW, SC, DEST_LOCAL, false>);
    CKB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kernel<<<grid, NUM_THREADS, smem, st>>>(P);
    count_launch();
    CKB_CUDA(cudaGetLastError());
    CKB_CUDA(cudaEventRecord(pc->ev[2], st));
    pc->ev_valid = true;
    return CKKS_B200_OK;
}

}  // namespace

namespace ckb {

int pcmm_slots_max_gap() { return SEG_MAX_GAP; }

// Grows the plane workspaces to what any plane configuration needs for ncols columns, so that a pipeline of
// multiplies over column chunks of different widths never reallocates (and synchronises) in mid-flight.
int pcmm_reserve_planes(ckks_b200_pcmm* pc, int M, int K, long ncols) {
    const int MT = (M + TM - 1) / TM, KBN = (K + KB - 1) / KB;
    const long CT = (ncols + TC - 1) / TC;
    int rc = ensure_dev(&pc->d_wplanes, &pc->wplanes_cap, (size_t)MT * KBN * Cfg<8, 8>::A_STAGE);
    if (!rc) rc = ensure_dev(&pc->d_xplanes, &pc->xplanes_cap, (size_t)pc->q_count * CT * KBN * Cfg<8, 8>::B_STAGE);
    return rc;
}

// The plane configuration and the number of K blocks per accumulation pass for weights of w_bits bits: the
// narrowest configuration that holds the planes, with the contraction cut into passes short enough for
// min(SW,SC) * (blocks * KB) * 255 * 255 to stay below 2^31 in every s32 accumulator.
int pcmm_tensor_plan(const ckks_b200_pcmm* pc, int K, int w_bits, int* sw_out, int* sc_out, int* kpass_out) {
    int q_bits = 0;
    for (u64 q : pc->q) {
        int b = 64 - __builtin_clzll(q);
        q_bits = b > q_bits ? b : q_bits;
    }
    const int sc = (q_bits + 7) / 8;
    const int sw = (w_bits + 1 + 7) / 8 > 0 ? (w_bits + 1 + 7) / 8 : 1;
    int klog = 0;
    while ((1 << klog) < K) klog++;
    CKB_REQUIRE(q_bits + w_bits + klog <= 110, CKKS_B200_ERR_UNSUPPORTED,
                "sum of %d-bit weights times %d-bit residues over K=%d exceeds the 110-bit accumulator budget",
                w_bits, q_bits, K);
    struct Inst { int sw, sc; };
    const Inst insts[] = {{4, 5}, {5, 7}, {6, 7}, {8, 8}};
    for (const Inst& in : insts) {
        if (sw > in.sw || sc > in.sc) continue;
        const int pairs = in.sw < in.sc ? in.sw : in.sc;
        const long long blocks = ((1ll << 31) - 1) / ((long long)pairs * 65025ll * KB);      // K blocks one pass may hold
        const int KBN = (K + KB - 1) / KB;
        *sw_out = in.sw;
        *sc_out = in.sc;
        *kpass_out = blocks >= KBN ? KBN : (int)blocks;
        return CKKS_B200_OK;
    }
    set_error("no tensor-core configuration holds %d weight planes and %d residue planes", sw, sc);
    return CKKS_B200_ERR_UNSUPPORTED;
}

int pcmm_tensor(ckks_b200_pcmm* pc, const long long* d_w, const PcmmSource& src, u64* d_out, int M, int K,
                long col_begin, long col_end, int w_bits, bool weights_ready, cudaStream_t st) {
    int sw = 0, sc = 0, kpass = 0;
    int rc = pcmm_tensor_plan(pc, K, w_bits, &sw, &sc, &kpass);
    if (rc) return rc;
    if (!weights_ready) pc->prep_sw = pc->prep_sc = 0;       // the planes are about to be overwritten
    if (sw == 4) rc = launch<4, 5>(pc, d_w, src, d_out, M, K, col_begin, col_end, kpass, weights_ready, st);
    else if (sw == 5) rc = launch<5, 7>(pc, d_w, src, d_out, M, K, col_begin, col_end, kpass, weights_ready, st);
    else if (sw == 6) rc = launch<6, 7>(pc, d_w, src, d_out, M, K, col_begin, col_end, kpass, weights_ready, st);
    else rc = launch<8, 8>(pc, d_w, src, d_out, M, K, col_begin, col_end, kpass, weights_ready, st);
    if (!rc && !weights_ready) { pc->prep_sw = sw; pc->prep_sc = sc; }
    return rc;
}

}  // namespace ckb

// Synchronise `stream` and report whether any bounded device-side wait of a tensor-core
// launch on this handle ran out since the last check.
extern "C" int ckks_b200_pcmm_check(ckks_b200_pcmm* pc, void* stream) {
    CKB_REQUIRE(pc != nullptr, CKKS_B200_ERR_ARG, "null argument");
    DeviceGuard guard(pc->device);
    CKB_REQUIRE(guard.ok, CKKS_B200_ERR_CUDA, "cudaSetDevice(%d) failed", pc->device);
    cudaStream_t st = (cudaStream_t)stream;
    CKB_CUDA(cudaMemcpyAsync(pc->h_flags, pc->d_flags, 16 * sizeof(int), cudaMemcpyDeviceToHost, st));
    CKB_CUDA(cudaMemsetAsync(pc->d_flags + 1, 0, sizeof(int), st));      // reported once: cleared by the check that reads it
    CKB_CUDA(cudaStreamSynchronize(st));
    CKB_REQUIRE(pc->h_flags[1] == 0, CKKS_B200_ERR_TIMEOUT,
                "a device-side wait ran out of its clock budget (site %d)", pc->h_flags[1]);
    return CKKS_B200_OK;
}

// Device time of the latest tensor-core multiply on this handle: the two slicing
// pre-pass kernels and the main kernel, in milliseconds (waits for them to finish).
extern "C" int ckks_b200_pcmm_last_timing(ckks_b200_pcmm* pc, float* prepass_ms, float* main_ms) {
    CKB_REQUIRE(pc && prepass_ms && main_ms, CKKS_B200_ERR_ARG, "null argument");
    CKB_REQUIRE(pc->ev_valid, CKKS_B200_ERR_ARG, "no tensor-core multiply has run on this handle");
    DeviceGuard guard(pc->device);
    CKB_REQUIRE(guard.ok, CKKS_B200_ERR_CUDA, "cudaSetDevice(%d) failed", pc->device);
    CKB_CUDA(cudaEventSynchronize(pc->ev[2]));
    CKB_CUDA(cudaEventElapsedTime(prepass_ms, pc->ev[0], pc->ev[1]));
    CKB_CUDA(cudaEventElapsedTime(main_ms, pc->ev[1], pc->ev[2]));
    return CKKS_B200_OK;
}
