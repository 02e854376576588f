// ModUp on the 5th-generation tensor cores (tcgen05, sm_100a): the operation of
// Context_23::modUpQjtoT_23 in the reference (src/ckks/include/BasisConv.cuh:84-179) with the
// alpha x t_num table product moved off the 64-bit integer multiplier.
//
// For one coefficient of one digit the conversion is
//     out_k = ( sum_j rb_j * (Qblk/q_j mod t_k)  -  v * (Qblk mod t_k) )  mod t_k ,
//     rb_j = x_j * (Qblk/q_j)^-1 mod q_j ,   v = trunc( sum_j rb_j / q_j )  in IEEE doubles.
// Write rb_j in bytes, rb_j = sum_b rb_{j,b} 2^(8b).  Modulo t_k the sum equals
//     sum_{j,b} rb_{j,b} * c_{k,j,b} ,   c_{k,j,b} = ((Qblk/q_j) * 2^(8b)) mod t_k ,
// and with c_{k,j,b} cut into bytes too this is an unsigned 8-bit matrix product:
//     D[x][k*8+a] = sum_{(j,b)} rb_{j,b}[x] * byte_a(c_{k,j,b}) ,   K = 8*alpha,  N = 8*t_num .
// One UMMA (M = 128 coefficients) per 32 bytes of K does it; the s32 results stay below 2^23.
// Each thread then recombines its row, sum_a D_a 2^(8a) < 2^80, adds the negated overflow term from a
// small table, reduces the sum modulo t_k with one FP64 quotient estimate (t_k in [2^40, 2^62)) and
// stores.
//
// With source moduli below 2^50 rb_j comes off the FP64 pipe as a value in (-0.7 q_j, 0.7 q_j); q_j is
// added to every one of them instead of to the negative ones only, and the overflow count rises by the
// number of limbs so treated: rb_j + q_j contributes one more Qblk to the sum, which the table entry for
// the larger count takes away again.  The residues are those of the canonical rb_j.
//
// The result is the exact residue.  The reference (and the CUDA-core kernel in modup.cu) forms
// the difference in 128 bits, which equals the exact residue unless the sum falls below
// v*(Qblk mod t_k); context creation checks the tables for that and sends such levels to the
// CUDA-core kernel.
//
// The same kernel serves the second conversion of the key-switch chain, Context_23::modUpTtoPQl_23
// (BasisConv.cuh:183-248): there the sources are the t moduli (60-bit, so rb_j is a Shoup product of
// x_j + floor(T/2)), the targets of a block are gamma moduli of [p | q], and floor(T/2) mod r is
// subtracted at the end, which the overflow table absorbs.  Everything that differs between the two
// conversions sits in per-block tables: source moduli, inverse hat constants and pre-added constants;
// target moduli, the multiple subtracted per unit of the overflow count and the constant subtracted
// at the end; the byte planes; and four strides.
//
// A CTA runs NG independent groups of 128 threads: five when the 8*t_num accumulator columns of a group
// fit 96 tensor-memory columns (t_num <= 12), four with 128 columns each otherwise.  A group owns one
// operand tile in shared memory and its columns of tensor memory and walks over tiles of 128 coefficients: every
// thread prepares its coefficient's row, one thread issues the instructions, all wait on the
// group's mbarrier (bounded; a wait that runs out raises a flag and the group leaves), then
// every thread finishes its own row.  The next tile's residues are loaded before that wait.
#include "context.cuh"
#include "umma.cuh"

using namespace ckb;
using namespace ckb::umma;

namespace {

constexpr int TMEM_COLS = 512;           // the whole tensor memory of the SM, split evenly over the groups

struct BconvArgs {
    u64* out;
    const u64* in;
    const u64* src_mod;           // [blocks][APAD]  modulus of source limb j of block blk (1: no such limb)
    const ulonglong2* src_hinv;   // [blocks][APAD]  {hat_j^-1 mod m_j, shoup}
    const u64* src_pre;           // [blocks][APAD]  added to the residue before the product
    const u64* tgt_mod;           // [blocks][tg]    target moduli
    const u64* tgt_f;             // [blocks][tg]    (product of the block's source moduli) mod r
    const u64* tgt_post;          // [blocks][tg]    subtracted at the end, below r
    const uint8_t* planes;        // [blocks][kpad/32][npad][32]
    int* flags;
    uint32_t N;
    int blocks, batch, tg, npad;
    int tgt_limit;                // target k of block blk exists iff blk*tg + k < tgt_limit
    int xshift;                   // log2 of the tiles per limb, N / 128
    bool fast;                    // the conditions of the kernel's FAST form hold
    double near;                  // the count is redone with divisions when the estimate is this close to an integer
    long long wait_budget;        // clock cycles a wait on a group's mbarrier may take
    int withhold;                 // test switch: group 0 of CTA 0 leaves out the commit of its first tile
    size_t in_batch, in_blk, out_batch, out_blk;      // strides in words; limb j / target k sits j*N / k*N further
};

__device__ __forceinline__ void group_sync(int id) { asm volatile("bar.sync %0, 128;" ::"r"(id) : "memory"); }
// AND of a predicate over the 128 threads of a group (also a barrier).
__device__ __forceinline__ bool group_all(bool p, int id) {
    uint32_t r;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.b32 p, %1, 0;\n\t"
        "bar.red.and.pred q, %2, 128, p;\n\t"
        "selp.u32 %0, 1, 0, q;\n\t}"
        : "=r"(r)
        : "r"((uint32_t)p), "r"(id)
        : "memory");
    return r != 0;
}

// u64 below 2^52 -> double, exactly: plant the value in the mantissa of 2^52 and subtract the offset.
__device__ __forceinline__ double small_to_double(u64 x) {
    return __hiloint2double(0x43300000 + (int)(x >> 32), (int)(uint32_t)x) - 4503599627370496.0;
}
__device__ __forceinline__ u64 mad_wide(uint32_t a, uint32_t b, u64 c) {
    u64 d;
    asm("mad.wide.u32 %0, %1, %2, %3;" : "=l"(d) : "r"(a), "r"(b), "l"(c));
    return d;
}

// F64Q: every source modulus is below 2^50 and nothing is pre-added, and rb_j = x_j * w_j mod m_j is then formed on the FP64 pipe
// (exact: h + l = x*w with h = fl(x*w), l the FMA remainder; h - c*q is a small integer for
// c = rint(h/q); w is kept centred, |w| <= q/2, so the result stays within (-0.7q, 0.7q)).
// Otherwise rb_j is a 64-bit Shoup product.
// FAST: every block has all tg targets, tg is a multiple of four and every target modulus is at least 2^49, so
// the quotient of the 81-bit sum fits 32 bits and nothing in the epilogue is conditional.
template <int APAD, bool F64Q, int NG, bool FAST>
__global__ void __launch_bounds__(128 * NG, 1) bconv_umma_kernel(BconvArgs P) {
    constexpr int GROUPS = NG, THREADS = 128 * NG, GROUP_COLS = NG == 5 ? 96 : 128;
    constexpr int KSTEPS = APAD * 8 / 32;
    constexpr int A_TILE = KSTEPS * TM * 32;
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ uint64_t bars[GROUPS];
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;

    const int tid = threadIdx.x, warp = tid >> 5;
    const int g = tid >> 7, r = tid & 127;
    const int T = P.tg;
    let_next_kernel_start();          // its set-up may overlap this kernel; its own wait keeps it off the data
    const int b_tile = KSTEPS * P.npad * 32;
    uint8_t* sA = smem + g * A_TILE;
    uint8_t* sB = smem + GROUPS * A_TILE;                                   // [blocks][KSTEPS][npad*32]
    const int BA = P.blocks * APAD, NV = 2 * APAD + 1;
    double2* s_f = reinterpret_cast<double2*>(sB + P.blocks * b_tile);     // [blocks][APAD][2]  {m_j, 1/m_j}, {w_j, 2^52 + m_j}
    ulonglong2* s_hinv = reinterpret_cast<ulonglong2*>(s_f + 2 * BA);      // [blocks][APAD]  {hat_j^-1 mod m_j, shoup}
    ulonglong2* s_tk = s_hinv + BA;                                        // [blocks][T]  {t_k (0: none), bits of 2^32 / t_k}
    u64* s_q = reinterpret_cast<u64*>(s_tk + P.blocks * T);                // [blocks][APAD]  source moduli (1: none)
    u64* s_pre = s_q + BA;                                                 // [blocks][APAD]
    u64* s_nv = s_pre + BA;                                                // [blocks][NV][T]  -(v*F + post) mod t_k
    int* s_nlive = reinterpret_cast<int*>(s_nv + P.blocks * NV * T);       // [blocks]  limbs of the digit (they come first)

    for (int i = tid; i < P.blocks * b_tile / 16; i += THREADS)
        reinterpret_cast<uint4*>(sB)[i] = reinterpret_cast<const uint4*>(P.planes)[i];
    for (int i = tid; i < BA; i += THREADS) {
        const u64 mj = P.src_mod[i];
        const bool live = mj != 1;
        s_q[i] = mj;
        s_hinv[i] = live ? P.src_hinv[i] : make_ulonglong2(0, 0);
        s_pre[i] = live ? P.src_pre[i] : 0;
        const u64 w = live ? P.src_hinv[i].x : 0;
        // without a limb: w = 0 and 1/m = 0 make rb = 0 and leave the count alone
        s_f[2 * i] = make_double2((double)mj, live ? 1.0 / (double)mj : 0.0);
        s_f[2 * i + 1] = make_double2(w > mj / 2 ? -(double)(mj - w) : (double)w,
                                      4503599627370496.0 + (live && F64Q ? (double)mj : 0.0));
    }
    for (int i = tid; i < P.blocks; i += THREADS) {
        int n = 0;
        for (int j = 0; j < APAD; j++) n += P.src_mod[i * APAD + j] != 1;
        s_nlive[i] = n;
    }
    for (int i = tid; i < P.blocks * T; i += THREADS) {
        const int blk = i / T, k = i % T;
        const bool live = blk * T + k < P.tgt_limit && P.tgt_mod[i] != 0;
        const u64 rk = live ? P.tgt_mod[i] : 0;
        s_tk[i] = make_ulonglong2(rk, (u64)__double_as_longlong(live ? 4294967296.0 / (double)rk : 0.0));
        u64 acc = live ? P.tgt_post[i] : 0;
        const u64 f = live ? P.tgt_f[i] : 0;
        for (int v = 0; v < NV; v++) {
            s_nv[(blk * NV + v) * T + k] = acc ? rk - acc : 0;
            acc += f;                        // f, acc < r < 2^62: no overflow
            if (acc >= rk) acc -= rk;
        }
    }
    if (tid == 0) {
        for (int i = 0; i < GROUPS; i++) mbar_init(smem_u32(&bars[i]), 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        tmem_alloc(smem_u32(&tmem_slot), TMEM_COLS);
        tmem_relinquish();
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // the constant tiles, for the MMA's reads
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_g = tmem_slot + g * GROUP_COLS;
    const uint32_t bar = smem_u32(&bars[g]);
    const uint32_t a16 = smem_u32(sA) >> 4, b16 = smem_u32(sB) >> 4;
    const uint32_t idesc = instr_desc(P.npad, false);

    const uint32_t total = (uint32_t)P.batch * P.blocks << P.xshift;
    const uint32_t stride = gridDim.x * GROUPS;
    uint32_t tile = blockIdx.x * GROUPS + g;

    const uint32_t limb_bytes = P.N * 8;
    // where a tile's coefficient r sits: its digit, its first source limb, its first target
    auto locate = [&](uint32_t tl, int& blk, const u64*& src, u64*& dst) {
        const uint32_t xt = tl & ((1u << P.xshift) - 1), rest = tl >> P.xshift;
        const uint32_t bt = rest / (uint32_t)P.blocks;
        blk = (int)(rest - bt * P.blocks);
        src = P.in + (size_t)bt * P.in_batch + (size_t)blk * P.in_blk + xt * TM + r;
        dst = P.out + (size_t)bt * P.out_batch + (size_t)blk * P.out_blk + xt * TM + r;
    };
    // residues of that coefficient, one per limb of its digit (zero beyond the digit)
    auto load_tile = [&](const u64* src, int blk, u64 (&x)[APAD]) {
        const int nl = s_nlive[blk];
#pragma unroll
        for (int j = 0; j < APAD; j++)
            x[j] = j < nl ? *reinterpret_cast<const u64*>(mad_wide((uint32_t)j, limb_bytes, (u64)src)) : 0;
    };

    u64 cur[APAD];
    int blk = 0, blk_next = 0;
    const u64 *src = nullptr;
    u64 *dst = nullptr, *dst_next = nullptr;
    wait_for_previous_kernel();       // the tables above are constants of the context; the residues are not
    if (tile < total) {
        locate(tile, blk, src, dst);
        load_tile(src, blk, cur);
    }
    uint32_t phase = 0;
    bool ok = true;
    // byte offset of this thread's row inside a K step: 8-row group, row in the group
    const uint32_t row_off = (uint32_t)(r >> 3) * 256 + (uint32_t)(r & 7) * 16;
    while (tile < total && ok) {
        // ---- rb_j, the overflow count, and this coefficient's row of the byte matrix ----
        // The reference's count is v = trunc(sum_j rb_j / q_j) with IEEE divisions added in limb
        // order.  est = sum_j rb_j * (1/q_j) differs from that sum by less than 2^-46, so both
        // truncate alike unless est sits within 2^-40 of an integer; only then are the divisions made.
        // On the FP64 path rb_j is kept signed in the sum and q_j added to every limb of the digit, so the
        // count starts at the number of limbs.
        double est = F64Q ? (double)s_nlive[blk] : 0.0;
#pragma unroll
        for (int j = 0; j < APAD; j++) {
            u64 rb;
            const double2 f0 = s_f[2 * (blk * APAD + j)];              // {q, 1/q}
            if (F64Q) {
                const double2 f1 = s_f[2 * (blk * APAD + j) + 1];      // {w, 2^52 + q}
                const double x = small_to_double(cur[j]);
                const double h = __dmul_rn(x, f1.x);
                const double l = __fma_rn(x, f1.x, -h);
                const double c = __dadd_rn(__fma_rn(h, f0.y, 6755399441055744.0), -6755399441055744.0);
                const double rbd = __dadd_rn(__fma_rn(-c, f0.x, h), l);          // in (-0.7q, 0.7q)
                est = __fma_rn(rbd, f0.y, est);
                rb = (u64)__double_as_longlong(__dadd_rn(rbd, f1.y)) & 0x000FFFFFFFFFFFFFull;   // rbd + q, below 2^51
            } else {
                const ulonglong2 hi = s_hinv[blk * APAD + j];
                rb = shoup_mul(cur[j] + s_pre[blk * APAD + j], hi.x, hi.y, s_q[blk * APAD + j]);   // exact for any 64-bit operand
                est = __fma_rn((double)rb, f0.y, est);
            }
            // K index j*8+b: step j/4, K half (j%4)/2, byte offset (j%2)*8 inside the 16-byte row
            *reinterpret_cast<u64*>(sA + (j / 4) * (TM * 32) + ((j % 4) / 2) * 128 + row_off + (j % 2) * 8) = rb;
        }
        int v = (int)est;
        {
            const double frac = est - (double)v;
            if (frac < P.near || frac > 1.0 - P.near) {
                double vv = 0.0;
                int added = 0;
                for (int j = 0; j < APAD; j++) {
                    u64 rb = *reinterpret_cast<const u64*>(sA + (j / 4) * (TM * 32) + ((j % 4) / 2) * 128 + row_off + (j % 2) * 8);
                    const u64 q = s_q[blk * APAD + j];
                    if (F64Q && rb >= q) {                                   // the stored value is the canonical one or q more
                        rb -= q;
                        added++;
                    }
                    vv += __ddiv_rn((double)rb, (double)q);                  // rb = 0 beyond the digit: adds 0.0
                }
                v = (int)vv + added;
            }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        const uint32_t next = tile + stride;
        if (next < total) {
            locate(next, blk_next, src, dst_next);
            load_tile(src, blk_next, cur);
        }
        group_sync(1 + g);
        if (r == 0) {
            tc_fence_after();
#pragma unroll
            for (int ks = 0; ks < KSTEPS; ks++)
                umma_i8(tmem_g, smem_desc(a16 + (ks * TM * 32 >> 4)),
                        smem_desc(b16 + ((blk * b_tile + ks * P.npad * 32) >> 4)), idesc, ks > 0);
            // Test switch: without the commit nothing ever arrives on the group's barrier, and the wait below runs
            // into its clock budget.
            if (!(P.withhold && blockIdx.x == 0 && g == 0 && phase == 0)) umma_commit(bar);
        }
        bool mine = mbar_wait(bar, phase, P.flags, 10 + g, &abort_flag, P.wait_budget);
        phase ^= 1;
        ok = group_all(mine, 1 + g);
        if (!ok) break;
        tc_fence_after();

        // ---- this coefficient's row: recombine, add the negated overflow term, reduce, store ----
        const uint32_t taddr = tmem_g + ((uint32_t)((warp & 3) * 32) << 16);
        const u64* nv = s_nv + (blk * NV + v) * T;
        const ulonglong2* tk2 = s_tk + blk * T;
        for (int k0 = 0; k0 < T; k0 += 4) {
            int32_t D[4][8];
#pragma unroll
            for (int u = 0; u < 4; u++) tmem_ld8(taddr + (k0 + u) * 8, D[u]);
            tmem_ld_wait();
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const int k = k0 + u;
                if (!FAST && k >= T) break;
                // sum_a D_a 2^(8a) in two halves of four (each below 2^48)
                const u64 g0 = mad_wide((uint32_t)D[u][3], 1u << 24, mad_wide((uint32_t)D[u][2], 1u << 16,
                               mad_wide((uint32_t)D[u][1], 1u << 8, (u64)(uint32_t)D[u][0])));
                const u64 g1 = mad_wide((uint32_t)D[u][7], 1u << 24, mad_wide((uint32_t)D[u][6], 1u << 16,
                               mad_wide((uint32_t)D[u][5], 1u << 8, (u64)(uint32_t)D[u][4])));
                const ulonglong2 tt = tk2[k];                // {t_k, 2^32 / t_k}
                const u64 s0 = g0 + nv[k];                   // below 2^63
                const u64 lo = s0 + (g1 << 32);              // the sum modulo 2^64
                const u64 top = g1 + (s0 >> 32);             // the sum / 2^32, below 2^49
                // nearest integer to top * 2^32 / t_k: within 1/2 + 2^-7 of the quotient of the sum
                const double qd = __fma_rn(small_to_double(top), __longlong_as_double((long long)tt.y), 4503599627370496.0);
                u64 res;                                     // in (-0.51 t, 0.51 t) modulo 2^64
                if (FAST) {
                    const uint32_t qh = (uint32_t)__double2loint(qd);
                    res = lo - (mad_wide(qh, (uint32_t)tt.x, 0) + ((u64)(qh * (uint32_t)(tt.x >> 32)) << 32));
                } else {
                    const u64 qh = (u64)__double_as_longlong(qd) & 0xFFFFFFFFFFFFFull;
                    res = lo - qh * tt.x;
                }
                if ((long long)res < 0) res += tt.x;
                if (FAST || tt.x != 0)                       // no such target in this block otherwise
                    *reinterpret_cast<u64*>(mad_wide((uint32_t)k, limb_bytes, (u64)dst)) = res;
            }
        }
        tc_fence_before();
        tile = next;
        blk = blk_next;
        dst = dst_next;
    }
    if (!ok && r == 0) atomicExch(&abort_flag, 1);

    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        tmem_dealloc(tmem_slot, TMEM_COLS);
    }
}

template <int APAD, bool F64Q, int NG, bool FAST>
int launch_groups(ckks_b200_context* c, const BconvArgs& P, cudaStream_t st) {
    constexpr int GROUPS = NG, THREADS = 128 * NG;
    constexpr int KSTEPS = APAD * 8 / 32;
    // operand tiles, byte planes, then the tables in the kernel's order: 32 + 16 + 8 + 8 bytes per source limb,
    // 16 per target, the negated overflow terms and the limb counts
    const size_t smem = (size_t)GROUPS * KSTEPS * TM * 32 + (size_t)P.blocks * KSTEPS * P.npad * 32 +
                        (size_t)P.blocks * APAD * 64 + (size_t)P.blocks * P.tg * 16 +
                        (size_t)P.blocks * (2 * APAD + 1) * P.tg * 8 + (size_t)P.blocks * 4;
    CKB_REQUIRE(smem <= 200 * 1024, CKKS_B200_ERR_UNSUPPORTED, "ModUp tables of %zu bytes do not fit shared memory", smem);
    CKB_CUDA(cudaFuncSetAttribute(bconv_umma_kernel<APAD, F64Q, NG, FAST>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    int sms = 0;
    CKB_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, c->device));
    const long total = (long)P.batch * P.blocks * (P.N / TM);
    CKB_REQUIRE(total < (1l << 31) && (P.N & (P.N - 1)) == 0, CKKS_B200_ERR_UNSUPPORTED,
                "ModUp of %ld tiles (N = %u) is beyond the kernel's 32-bit tile index", total, P.N);
    const long want = (total + GROUPS - 1) / GROUPS;
    const int grid = (int)(want < sms ? want : sms);
    BconvArgs Q = P;
    Q.xshift = 0;
    while ((TM << Q.xshift) < (int)P.N) Q.xshift++;
    Q.wait_budget = c->wait_budget > 0 ? c->wait_budget : WAIT_BUDGET;
    Q.withhold = c->withhold_commit;
    Q.near = c->exact_count ? 0.75 : 0x1p-40;               // 0.75: every estimate counts as close
    c->withhold_commit = 0;                                 // the test switch arms one launch
    CKB_CUDA(launch_after(bconv_umma_kernel<APAD, F64Q, NG, FAST>, dim3(grid), dim3(THREADS), smem, st, Q));
    count_launch();
    CKB_CUDA(cudaGetLastError());
    return CKKS_B200_OK;
}

template <int APAD, bool F64Q>
int launch(ckks_b200_context* c, const BconvArgs& P, cudaStream_t st) {
    // the accumulator loads run in groups of four targets, so five groups need 8*ceil4(t_num) <= 96
    const bool five = (P.tg + 3) / 4 * 32 <= 96;
    if (P.fast) return five ? launch_groups<APAD, F64Q, 5, true>(c, P, st) : launch_groups<APAD, F64Q, 4, true>(c, P, st);
    return five ? launch_groups<APAD, F64Q, 5, false>(c, P, st) : launch_groups<APAD, F64Q, 4, false>(c, P, st);
}

template <bool F64Q>
int launch_apad(ckks_b200_context* c, const BconvArgs& P, int kpad, cudaStream_t st) {
    if (kpad == 32) return launch<4, F64Q>(c, P, st);
    if (kpad == 64) return launch<8, F64Q>(c, P, st);
    if (kpad == 96) return launch<12, F64Q>(c, P, st);
    return launch<16, F64Q>(c, P, st);
}

}  // namespace

namespace ckb {

bool modup_tensor_ok(const ckks_b200_context* c, int l) {
    return c->mu_planes != nullptr && l >= 0 && l < (int)c->mu_tc_ok.size() && c->mu_tc_ok[l] != 0 &&
           c->N % TM == 0 && c->tc_npad <= 128;
}

int modup_tensor(ckks_b200_context* c, u64* d_out, const u64* d_in, int l, int batch, cudaStream_t st) {
    const int A = c->alpha, B = c->blocks_max, T = c->t_num, AP = c->tc_kpad / 8;
    BconvArgs P;
    P.out = d_out;
    P.in = d_in;
    P.src_mod = c->mu_src_mod + (size_t)l * B * AP;
    P.src_hinv = c->mu_src_hinv + (size_t)l * B * AP;
    P.src_pre = c->mu_src_pre;                          // zeros
    P.tgt_mod = c->mu_tgt_mod;                          // the t moduli for every block
    P.tgt_f = c->mu_blk_mod_t + (size_t)l * B * T;
    P.tgt_post = c->mu_src_pre;                         // zeros
    P.planes = c->mu_planes + (size_t)l * B * c->tc_kpad * c->tc_npad;
    P.flags = c->d_flags;
    P.N = c->N;
    P.blocks = (l + 1 + A - 1) / A;
    P.batch = batch;
    P.tg = T;
    P.npad = c->tc_npad;
    P.tgt_limit = 1 << 30;
    P.in_batch = (size_t)c->q_num * c->N;
    P.in_blk = (size_t)A * c->N;
    P.out_batch = (size_t)P.blocks * T * c->N;
    P.out_blk = (size_t)T * c->N;
    bool q_small = true;
    for (int i = 0; i < c->q_num; i++) q_small = q_small && c->moduli[c->p_num + i] < (1ull << 50);
    P.fast = T % 4 == 0;                                // every digit is converted to all t moduli
    for (int k = 0; k < T; k++) P.fast = P.fast && c->moduli[c->p_num + c->q_num + k] >= (1ull << 49);
    return q_small ? launch_apad<true>(c, P, c->tc_kpad, st) : launch_apad<false>(c, P, c->tc_kpad, st);
}

bool modup_t_tensor_ok(const ckks_b200_context* c, int gamma) {
    auto it = c->tpq.find(gamma);
    return it != c->tpq.end() && it->second.ok && c->N % TM == 0;
}

// Context_23::modUpTtoPQl_23 on the tensor cores; the tables of this gamma were built by the caller (keyswitch.cu).
int modup_t_tensor(ckks_b200_context* c, u64* d_out, const u64* d_in, int l, int gamma, int batch, cudaStream_t st) {
    const TpqTables& tb = c->tpq.at(gamma);
    const int R = (c->p_num + c->q_num + gamma - 1) / gamma;
    BconvArgs P;
    P.out = d_out;
    P.in = d_in;
    P.src_mod = tb.src_mod;
    P.src_hinv = tb.src_hinv;
    P.src_pre = tb.src_pre;
    P.tgt_mod = tb.tgt_mod;
    P.tgt_f = tb.tgt_f;
    P.tgt_post = tb.tgt_post;
    P.planes = tb.planes;
    P.flags = c->d_flags;
    P.N = c->N;
    P.blocks = (c->p_num + l + 1 + gamma - 1) / gamma;
    P.batch = batch;
    P.tg = gamma;
    P.npad = tb.npad;
    P.tgt_limit = c->p_num + l + 1;
    P.in_batch = (size_t)R * c->t_num * c->N;
    P.in_blk = (size_t)c->t_num * c->N;
    P.out_batch = P.in_batch;
    P.out_blk = (size_t)gamma * c->N;
    P.fast = false;                                     // the last block may have fewer than gamma targets
    return launch_apad<false>(c, P, tb.kpad, st);
}

}  // namespace ckb
