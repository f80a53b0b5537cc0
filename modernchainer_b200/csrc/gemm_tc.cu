// bf16 tensor-core GEMM for sm_100a: tcgen05.mma with the accumulator in TMEM, operands
// staged in shared memory by per-CTA TMA loads, persistent warp-specialised CTAs.
//
//   D[M,N] (+)= A * B (+ bias) -> act,  f32 accumulate, D stored as bf16 or f32.
//
// Operand storage (both bf16):
//   K-major  : [rows, K] with K contiguous  -> TMA box {64 k, rows} -> 128-byte swizzled rows
//   MN-major : [K, rows] with rows contiguous -> TMA boxes {64 rows, 64 k}
// so fprop (x W^T), dgrad (g W) and wgrad (g^T x) all read the tensors where they lie; no
// transposed copy is ever made.
//
// CTA layout (352 threads): warp 0 issues the TMA copies of A and warp 6 those of B, warp 1
// issues MMA and owns the TMEM allocation, warps 2..5 drain the accumulator (one TMEM lane
// quarter each) and hand D to TMA in 128-byte-row boxes; warps 7..10 are a second such group
// that takes every other 64-column chunk where shared memory has room for its boxes (short-K
// tiles are bound by the epilogue).  Two accumulators (2 x BN columns of
// TMEM) let the epilogue of tile i overlap the MMAs of tile i+1.  A 4..8-deep smem ring
// decouples TMA from MMA.  Each of the single-thread roles is latency-bound on its own
// instruction stream (a runtime division in the MMA loop alone cost 20% of the tensor rate),
// so their loops carry ring counters instead of dividing and the copies are split over two
// threads.  Optionally two CTAs of a cluster pair up on one 256-row tile (cta_group::2).
//
// Every wait on an mbarrier is bounded by wall time; on expiry the CTA raises the device
// error word, stops issuing work, and still frees its TMEM before returning.
#include <cuda.h>

#include <cstdlib>

#include "common.cuh"
#include "internal.h"

namespace {

constexpr int BM = 128;
constexpr int BK = 64; // 64 bf16 = one 128-byte swizzle row
constexpr int kThreads = 352; // 11 warps: A producer, MMA issuer, epilogue group 0 (warps 2-5), B producer, epilogue group 1 (warps 7-10)
constexpr unsigned long long kWaitLimitNs = 2000000000ull; // 2 s

struct TcArgs {
    void *d;
    void *d_pre;
    const float *bias;
    long long m, n, k, ldd;
    int out_bf16, accumulate, act, split_k, vec_red; // out_bf16: the output is a 16-bit type (bf16, or f16 when `f16` is set)
    int f16;                                          // operands and 16-bit outputs are IEEE f16 instead of bf16
    int tma_out;  // 1: the epilogue stages output boxes in shared memory and TMA writes (or adds) them
    int bias_vec; // bias base is 16-byte aligned
    int a_mn, b_mn;
    unsigned idesc;
    int m_tiles, n_tiles, kb_total, kb_per_split;
    int n_fast; // tile order: 0 = row blocks fastest, 1 = column blocks fastest (see tile_coords)
    int stages; // depth of the operand ring actually used (tuning knob; at most the compiled depth)
    int ring;   // output boxes per epilogue warp: 2, or 4 when one operand stage is given up for them
    int epi_groups; // epilogue groups of four warps in use: 1 or 2
    // Split tail (sk_splits > 1): the sk_rem tiles that would form a mostly empty last wave (tile indices from sk_full
    // on) are each cut into sk_splits slices of sk_kb k-blocks; the slices are the first work items, the sk_full whole
    // tiles follow.  An accumulating output takes the
    // slices' f32 partial sums directly (TMA reduce-add through map_pre = the output).  Any other output is finished
    // inside the kernel: slices 1 .. S-1 leave their partial sums in fix_ws, slice 0 adds them to its own accumulator in
    // slice order and runs the normal epilogue (bias, activation, rounding, second output).
    int sk_full, sk_rem, sk_splits, sk_kb;
    // [sk_rem][2 (pair half)][sk_splits - 1][4 lane quarters][BN / 32 column blocks][8][32 lanes] float4: the 32 x 32 block a warp
    // reads from TMEM at once, laid out so that one warp-wide store or load covers 512 contiguous bytes; nullptr unless
    // slices are finished in the kernel
    float *fix_ws;
    unsigned *fix_cnt; // [sk_rem][2][8 epilogue warps]: slices that have left their partial sums; zero between launches
    uint4 *zero_ptr;   // side job of the epilogue warps before their first tile: zero_n16 16-byte pieces of zeros from here
    long long zero_n16;
    unsigned int *err;
};

constexpr int kFixTiles = 148;        // split-tail tiles a launch may finish in the kernel (size of mcb_ctx::tc_fix_cnt)
// planner's charge for leaving and collecting the partial sums of a split tail.  Measured on 8192-row problems with 768
// output columns (96 tiles of 256 x 256 on 74 CTA pairs): K = 3072 gains 2 us over 128 x 192 tiles, K = 2304 loses 2 us,
// K = 768 loses 8 us; 7000 cycles puts the line between the first two.
constexpr double kFixCycles = 7000.0;

struct WorkItem {
    unsigned t;   // tile index (tn-major: t = tn * m_tiles + tm)
    int kb0, kb1; // k-block range
    int split;    // index of the slice along K (0 for whole tiles)
    bool partial; // slice of a split-tail tile: f32 partial sum into the workspace
};
__device__ __forceinline__ WorkItem decode_work(const TcArgs &args, unsigned w, unsigned tiles_mn, bool one_split) {
    WorkItem it;
    if (args.sk_splits > 1) {
        // the slices come FIRST: what follows them in a worker's list (whole tiles) hides the time their partial sums
        // take to meet, and the last item of every worker ends with a plain epilogue
        const unsigned n_slices = (unsigned)args.sk_rem * (unsigned)args.sk_splits;
        if (w >= n_slices) {
            it.t = w - n_slices;
            it.kb0 = 0;
            it.kb1 = args.kb_total;
            it.split = 0;
            it.partial = false;
        } else {
            const unsigned idx = w, q = idx / (unsigned)args.sk_splits;
            it.split = (int)(idx - q * (unsigned)args.sk_splits);
            it.t = (unsigned)args.sk_full + q;
            it.kb0 = it.split * args.sk_kb;
            it.kb1 = min(it.kb0 + args.sk_kb, args.kb_total);
            it.partial = true;
        }
        return it;
    }
    it.split = one_split ? 0 : (int)(w / tiles_mn);
    it.t = w - (unsigned)it.split * tiles_mn;
    it.kb0 = it.split * args.kb_per_split;
    it.kb1 = min(it.kb0 + args.kb_per_split, args.kb_total);
    it.partial = false;
    return it;
}

// Tile index -> (column block, row block).  Consecutive indices run at the same time, so the order decides which operand
// they share in L2: rows fastest (the default) shares the B block of one column block; columns fastest (n_fast) makes
// the few column blocks of one row block run together and read that row block's A slab once -- the order for a huge A
// against a small B (the lm_head gradients: a 524 MB logit-gradient matrix against 768 columns).
__device__ __forceinline__ void tile_coords(const TcArgs &args, unsigned t, unsigned m_tiles, unsigned &tn, unsigned &tm) {
    if (args.n_fast) {
        tm = t / (unsigned)args.n_tiles;
        tn = t - tm * (unsigned)args.n_tiles;
    } else {
        tn = t / m_tiles;
        tm = t - tn * m_tiles;
    }
}

// ------------------------------------------------------------------ PTX wrappers
__device__ __forceinline__ unsigned smem_u32(const void *p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(unsigned long long *bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(unsigned long long *bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned long long *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_test(unsigned long long *bar, unsigned parity) {
    unsigned ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok)
                 : "r"(smem_u32(bar)), "r"(parity)
                 : "memory");
    return ok != 0;
}
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
// bounded wait; returns false after the time limit or once another role aborted
__device__ __forceinline__ bool mbar_wait(unsigned long long *bar, unsigned parity, volatile int *abort_flag,
                                          unsigned int *err, unsigned sleep_ns = 0) {
    if (mbar_test(bar, parity)) return true;
    unsigned long long t0 = global_ns();
    unsigned spins = 0;
    for (;;) {
        if (mbar_test(bar, parity)) return true;
        if (sleep_ns) __nanosleep(sleep_ns); // waits a whole tile long: leave the issue slots to the MMA warp
        if ((++spins & 63u) == 0) {
            if (*abort_flag) return false;
            if (global_ns() - t0 > kWaitLimitNs) {
                *abort_flag = 1;
                atomicOr(err, MCB_DEVERR_TIMEOUT);
                return false;
            }
        }
    }
}

// Bounded wait until the counter at `flag` (written by other CTAs of this launch) has reached `want`.
__device__ __forceinline__ bool flag_wait(const unsigned *flag, unsigned want, volatile int *abort_flag, unsigned int *err) {
    unsigned long long t0 = global_ns();
    unsigned spins = 0;
    for (;;) {
        unsigned v;
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
        if (v >= want) return true;
        __nanosleep(64);
        if ((++spins & 63u) == 0) {
            if (*abort_flag) return false;
            if (global_ns() - t0 > kWaitLimitNs) {
                *abort_flag = 1;
                atomicOr(err, MCB_DEVERR_TIMEOUT);
                return false;
            }
        }
    }
}

__device__ __forceinline__ void tma_load_2d(void *smem_dst, const CUtensorMap *map, unsigned long long *bar, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 :
                 : "r"(smem_u32(smem_dst)), "l"((unsigned long long)map), "r"(smem_u32(bar)), "r"(x), "r"(y)
                 : "memory");
}

__device__ __forceinline__ void tmem_alloc(unsigned *smem_dst, unsigned ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc(unsigned taddr, unsigned ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(unsigned long long *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_mma(unsigned tmem_d, unsigned long long adesc, unsigned long long bdesc, unsigned idesc,
                                       unsigned accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 :
                 : "r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
                 : "memory");
}
// ---- CTA-pair (cta_group::2) forms: two CTAs of one cluster act as one 256-row MMA.  Barriers
// sit at the same shared-memory offset in both CTAs; `mapa` turns a local barrier address into
// the cluster address of the same barrier in the pair's leader (cluster rank 0).
__device__ __forceinline__ unsigned leader_addr(const void *p) {
    unsigned r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, 0;" : "=r"(r) : "r"(smem_u32(p)));
    return r;
}
__device__ __forceinline__ unsigned cluster_rank() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// arrive on a barrier of the leader CTA from either CTA of the pair
__device__ __forceinline__ void mbar_arrive_leader(unsigned long long *bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(leader_addr(bar)) : "memory");
}
// per-CTA TMA load whose completion bytes are counted on the LEADER's barrier (no multicast: the
// data lands only in the issuing CTA's shared memory)
__device__ __forceinline__ void tma_load_2d_pair(void *smem_dst, const CUtensorMap *map, unsigned long long *bar, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 :
                 : "r"(smem_u32(smem_dst)), "l"((unsigned long long)map), "r"(leader_addr(bar)), "r"(x), "r"(y)
                 : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(unsigned *smem_dst, unsigned ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc_pair(unsigned taddr, unsigned ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// completion of the pair's MMAs arrives on the barrier at this offset in BOTH CTAs (mask 0b11)
__device__ __forceinline__ void tc_commit_pair(unsigned long long *bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(smem_u32(bar)),
                 "h"((unsigned short)3)
                 : "memory");
}
__device__ __forceinline__ void tc_mma_pair(unsigned tmem_d, unsigned long long adesc, unsigned long long bdesc, unsigned idesc,
                                            unsigned accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 :
                 : "r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
                 : "memory");
}
// forms for the MMA issue loop: descriptors as (low, high) words, barriers as shared-space addresses
template <bool PAIR>
__device__ __forceinline__ void tc_mma_words(unsigned tmem_d, unsigned a_lo, unsigned a_hi, unsigned b_lo, unsigned b_hi, unsigned idesc,
                                             unsigned accumulate) {
    if (PAIR)
        asm volatile("{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tsetp.ne.b32 p, %6, 0;\n\tmov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %4};\n\t"
                     "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %5, p;\n\t}"
                     :
                     : "r"(tmem_d), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
                     : "memory");
    else
        asm volatile("{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tsetp.ne.b32 p, %6, 0;\n\tmov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %4};\n\t"
                     "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t}"
                     :
                     : "r"(tmem_d), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
                     : "memory");
}
template <bool PAIR> __device__ __forceinline__ void tc_commit_addr(unsigned bar_addr) {
    if (PAIR)
        asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar_addr),
                     "h"((unsigned short)3)
                     : "memory");
    else
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_addr) : "memory");
}
__device__ __forceinline__ bool mbar_test_addr(unsigned bar_addr, unsigned parity) {
    unsigned ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok)
                 : "r"(bar_addr), "r"(parity)
                 : "memory");
    return ok != 0;
}
__device__ __forceinline__ void tmem_ld32(unsigned taddr, unsigned (&r)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr)
                 : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ---- output path: a warp stages a [32 rows x 128 bytes] box in shared memory (128-byte swizzle)
// and one lane hands it to TMA, which writes whole rows and clips at the matrix edge.  Compared
// with per-lane row-strided global stores this removes 32 separate L2 transactions per
// instruction from the load/store unit.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap *map, const void *smem_src, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                 :
                 : "l"((unsigned long long)map), "r"(smem_u32(smem_src)), "r"(x), "r"(y)
                 : "memory");
}
// same box, added to the f32 matrix in global memory (split-K and gradient accumulation)
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap *map, const void *smem_src, int x, int y) {
    asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];"
                 :
                 : "l"((unsigned long long)map), "r"(smem_u32(smem_src)), "r"(x), "r"(y)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// all but the newest group have finished READING their shared-memory source
__device__ __forceinline__ void bulk_wait_read1() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// two f32 values rounded to nearest even and packed as bf16 (F16 = false) or f16 (F16 = true)
template <bool F16> __device__ __forceinline__ unsigned pack16(float a, float b) {
    if (F16) {
        __half2 p = __floats2half2_rn(a, b);
        return *(unsigned *)&p;
    }
    __nv_bfloat162 p = __floats2bfloat162_rn(a, b);
    return *(unsigned *)&p;
}
template <bool F16, int N> __device__ __forceinline__ void pack_row(const float (&v)[N], unsigned (&w)[N / 2]) {
#pragma unroll
    for (int j = 0; j < N / 2; ++j) w[j] = pack16<F16>(v[2 * j], v[2 * j + 1]);
}
// the branch on the format is taken once per row chunk, outside the conversion loop
template <int N> __device__ __forceinline__ void pack_row_any(const float (&v)[N], unsigned (&w)[N / 2], int f16) {
    if (f16) pack_row<true, N>(v, w);
    else pack_row<false, N>(v, w);
}

// Per-warp staging ring of two (or four) 4 KB boxes.  `issued` counts the boxes handed to TMA so far.
struct StageRing {
    unsigned char *base;
    unsigned issued;
};
// Wait until the box about to be overwritten has been read, and return it.
__device__ __forceinline__ unsigned char *ring_acquire(StageRing &rg, int lane, int ring) {
    if (lane == 0) {
        if (ring == 4) asm volatile("cp.async.bulk.wait_group.read 3;" ::: "memory");
        else bulk_wait_read1();
    }
    __syncwarp();
    return rg.base + (rg.issued & (unsigned)(ring - 1)) * 4096u;
}
// 16-byte piece `j` (0..7) of this lane's 128-byte row, at its swizzled position
__device__ __forceinline__ void ring_put(unsigned char *box, int lane, int j, uint4 piece) {
    *(uint4 *)(box + lane * 128 + ((j ^ (lane & 7)) << 4)) = piece;
}
__device__ __forceinline__ void ring_submit(StageRing &rg, unsigned char *box, const CUtensorMap *map, int x, int y, bool reduce, int lane) {
    fence_async_smem();
    __syncwarp();
    if (lane == 0) {
        if (reduce) tma_reduce_add_2d(map, box, x, y);
        else tma_store_2d(map, box, x, y);
        bulk_commit();
    }
    ++rg.issued;
}

// Shared-memory matrix descriptor (sm_100 format): start address >> 4 in bits [0,14),
// leading byte offset >> 4 in [16,30), stride byte offset >> 4 in [32,46), version 1 in
// [46,48), layout type 2 (128-byte swizzle) in [61,64).
__device__ __forceinline__ unsigned long long make_desc(unsigned smem_addr, unsigned lbo_bytes, unsigned sbo_bytes) {
    unsigned long long d = 0;
    d |= (unsigned long long)((smem_addr & 0x3FFFFu) >> 4);
    d |= (unsigned long long)((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= (unsigned long long)((sbo_bytes >> 4) & 0x3FFFu) << 32;
    d |= 1ull << 46;
    d |= 2ull << 61;
    return d;
}

// GELU for the bf16 epilogue: the hardware tanh approximation (relative error ~2^-11) is below
// bf16 resolution and keeps the epilogue shorter than the MMA time of the next tile
__device__ __forceinline__ float gelu_f(float v) {
    float v3 = v * v * v;
    float t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.7978845608028654f * (v + 0.044715f * v3)));
    return 0.5f * v * (1.0f + t);
}

// PAIR = two CTAs of a cluster share one 256 x BN tile: each loads its own 128 rows of A and half
// of the BN columns of B, so a CTA's shared-memory traffic per MMA flop is half that of the
// single-CTA form (which is bound by shared-memory bandwidth, not by the tensor pipe).
template <int BN, bool PAIR> struct Cfg {
    static constexpr int kBRows = PAIR ? BN / 2 : BN; // B rows (output columns) staged per CTA
    static constexpr int kStageBytes = (BM + kBRows) * BK * 2;
    static constexpr int kStages = PAIR ? (BN == 128 ? 8 : 6) : (BN == 128 ? 6 : 4);
    // Output boxes: 4 KB each, `ring` per epilogue warp.  One epilogue group (four warps, one per TMEM lane quarter) needs
    // 32 KB with two boxes each.  Tiles whose main loop is short (K of a few hundred) are bound by the epilogue, so where
    // shared memory allows a second group of four warps takes every other 64-column chunk: 128 x 192 tiles have the room
    // beside their four stages, 256-wide pair tiles give up one of six stages for it (chosen per launch).
    static constexpr int kMaxGroups = ((BN == 192 && !PAIR) || (BN == 256 && PAIR)) ? 2 : 1;
    static constexpr int kOutStageBytes = 4 * 2 * 4096;
    static constexpr int kTileAndOutBytes = (BN == 256 && PAIR) ? (kStages * kStageBytes + kOutStageBytes) /* = 5 stages + 64 KB */
                                                                : (kStages * kStageBytes + kMaxGroups * kOutStageBytes);
    static constexpr int kSmemBytes = kTileAndOutBytes + 1024 /*align*/ + 256 /*barriers*/;
    static_assert(kSmemBytes <= 227 * 1024, "shared memory budget of one CTA");
};

template <int BN, bool PAIR>
__global__ void __launch_bounds__(kThreads, 1)
tc_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const __grid_constant__ CUtensorMap map_d, const __grid_constant__ CUtensorMap map_pre, TcArgs args) {
    using C = Cfg<BN, PAIR>;
    constexpr int kStages = C::kStages;
    constexpr int kABytes = BM * BK * 2, kBBytes = C::kBRows * BK * 2;
    extern __shared__ unsigned char smem_raw[];
    // operand tiles need 1024-byte alignment for the 128-byte swizzle pattern
    unsigned char *tiles = (unsigned char *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    // the output boxes follow the operand stages in use: a launch may run one stage less and give that room to a
    // deeper ring of output boxes (args.ring = 4); the barriers sit behind the compiled maximum of both
    unsigned char *out_stage = tiles + (unsigned)args.stages * C::kStageBytes; // 1024-aligned: stage sizes are multiples of 8 KB
    unsigned long long *bars = (unsigned long long *)(tiles + C::kTileAndOutBytes);
    unsigned long long *full_bar = bars, *empty_bar = bars + kStages;
    unsigned long long *acc_full = bars + 2 * kStages, *acc_empty = acc_full + 2;
    unsigned *tmem_slot = (unsigned *)(acc_empty + 2);
    volatile int *abort_flag = (volatile int *)(tmem_slot + 1);

    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // rank inside the pair (0 = leader: arms the full barriers and issues the MMAs) and the
    // persistent work stride: one work item per CTA, or per pair
    const unsigned crank = PAIR ? cluster_rank() : 0u;
    // 32-bit work indices (the host checks the item count): a 64-bit division per tile in a
    // single-thread role is hundreds of cycles of pipeline bubble
    const unsigned w_first = PAIR ? (blockIdx.x >> 1) : blockIdx.x;
    const unsigned w_stride = PAIR ? (gridDim.x >> 1) : gridDim.x;
    constexpr int kTileM = PAIR ? 2 * BM : BM;
    const unsigned nst = (unsigned)args.stages; // ring depth in use, <= kStages
    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&full_bar[s], 2); // one arming arrival per operand producer
            mbar_init(&empty_bar[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&acc_full[a], 1);
            mbar_init(&acc_empty[a], (PAIR ? 8u : 4u) * (unsigned)args.epi_groups); // the leader also collects the peer's epilogue warps
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        if (PAIR) {
            tmem_alloc_pair(tmem_slot, 512);
            tmem_relinquish_pair();
        } else {
            tmem_alloc(tmem_slot, 512);
            tmem_relinquish();
        }
    }
    tc_fence_before();
    __syncthreads();
    if (PAIR) cluster_sync_all(); // the peer's barriers exist before anything signals them
    tc_fence_after();
    unsigned tmem_base = *tmem_slot;
    // everything above touched only shared and tensor memory, so it may run while the previous kernel of the
    // stream drains; from here on global memory is read and written
    dep_wait();
    dep_trigger();

    const unsigned tiles_mn = (unsigned)args.m_tiles * (unsigned)args.n_tiles;
    const unsigned work_total =
        args.sk_splits > 1 ? (unsigned)args.sk_full + (unsigned)args.sk_rem * (unsigned)args.sk_splits : tiles_mn * (unsigned)args.split_k;
    const unsigned m_tiles = (unsigned)args.m_tiles;
    const bool one_split = args.split_k == 1;

    if (warp == 0 || warp == 6) {
        // ---------------------------------------------------------------- TMA producers
        // Two single-thread producers, one per operand (warp 0: A, warp 6: B), so that the serial
        // cost of waiting, arming and issuing copies is split over two instruction streams; each
        // arms the full barrier with its own operand's bytes.
        if (lane == 0) {
            const bool is_a = (warp == 0);
            const CUtensorMap *map = is_a ? &map_a : &map_b;
            const bool mn = is_a ? (args.a_mn != 0) : (args.b_mn != 0);
            const int rows = is_a ? BM : C::kBRows;            // operand rows staged per CTA
            const unsigned bytes = (unsigned)rows * BK * 2u;
            const unsigned tile_off = is_a ? 0u : (unsigned)kABytes;
            unsigned it = 0;
            int s = 0;
            unsigned ph = 0;
            bool ok = true;
            for (unsigned w = w_first; w < work_total && ok; w += w_stride) {
                const WorkItem wi = decode_work(args, w, tiles_mn, one_split);
                const unsigned t = wi.t;
                unsigned tn, tm;
                tile_coords(args, t, m_tiles, tn, tm);
                int r0 = is_a ? (int)tm * kTileM + (int)crank * BM : (int)tn * BN + (int)crank * (PAIR ? BN / 2 : 0);
                const int kb0 = wi.kb0, kb1 = wi.kb1;
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    ok = mbar_wait(&empty_bar[s], ph ^ 1u, abort_flag, args.err);
                    if (!ok) break;
                    unsigned char *dst = tiles + s * C::kStageBytes + tile_off;
                    unsigned long long *fb = &full_bar[s];
                    int k0 = kb * BK;
                    if (PAIR) {
                        // the leader's barrier counts the bytes of both CTAs' copies of this operand
                        if (crank == 0) mbar_expect_tx(fb, 2u * bytes);
                        if (!mn) {
                            tma_load_2d_pair(dst, map, fb, k0, r0);
                        } else {
                            for (int b = 0; b < rows / 64; ++b) tma_load_2d_pair(dst + b * 8192, map, fb, r0 + b * 64, k0);
                        }
                    } else {
                        mbar_expect_tx(fb, bytes);
                        if (!mn) {
                            tma_load_2d(dst, map, fb, k0, r0);
                        } else {
                            for (int b = 0; b < rows / 64; ++b) tma_load_2d(dst + b * 8192, map, fb, r0 + b * 64, k0);
                        }
                    }
                    if (++s == (int)nst) {
                        s = 0;
                        ph ^= 1u;
                    }
                }
            }
            // drain: wait until every copy that was issued has been consumed (bounded), so none
            // is still writing this CTA's shared memory when it exits
            for (int d = 0; d < (int)nst; ++d) {
                unsigned filled = (it > (unsigned)d) ? ((it - 1 - d) / nst + 1) : 0; // times stage d was filled
                if (filled == 0) continue;
                if (!mbar_wait(&empty_bar[d], (filled - 1) & 1u, abort_flag, args.err)) break;
            }
            if (*abort_flag) {
                // gave up: let copies that are still in flight land before this CTA can exit
                unsigned long long t0 = global_ns();
                while (global_ns() - t0 < 200000ull) {
                }
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer (the leader, in a pair)
        if (lane == 0 && crank == 0) {
            // This thread's instruction stream is the critical path: every instruction between two
            // MMAs costs a few cycles of tensor-pipe idle time.  So the loop carries ready-made
            // descriptor words and barrier addresses and only adds small offsets to them.
            unsigned tile_it = 0;
            unsigned a_lbo = args.a_mn ? 8192u : 16u, a_kinc = (args.a_mn ? 2048u : 32u) >> 4;
            unsigned b_lbo = args.b_mn ? 8192u : 16u, b_kinc = (args.b_mn ? 2048u : 32u) >> 4;
            const unsigned long long a_desc0 = make_desc(smem_u32(tiles), a_lbo, 1024u);
            const unsigned long long b_desc0 = make_desc(smem_u32(tiles) + kABytes, b_lbo, 1024u);
            // only the 14-bit start-address field changes (operands sit below 256 KB, so no carry)
            const unsigned a_hi = (unsigned)(a_desc0 >> 32), b_hi = (unsigned)(b_desc0 >> 32);
            const unsigned a_lo0 = (unsigned)a_desc0, b_lo0 = (unsigned)b_desc0;
            constexpr unsigned kStageInc = (unsigned)C::kStageBytes >> 4;
            const unsigned full0 = smem_u32(full_bar), empty0 = smem_u32(empty_bar);
            const unsigned idesc = args.idesc;
            unsigned s = 0, soff = 0, ph = 0;
            bool ok = true;
            for (unsigned w = w_first; w < work_total && ok; w += w_stride, ++tile_it) {
                const WorkItem wi = decode_work(args, w, tiles_mn, one_split);
                const int nkb = wi.kb1 - wi.kb0;
                int acc = tile_it & 1;
                unsigned acc_ph = (tile_it >> 1) & 1u;
                if (!mbar_wait(&acc_empty[acc], acc_ph ^ 1u, abort_flag, args.err)) break;
                tc_fence_after();
                const unsigned tmem_d = tmem_base + (unsigned)(acc * BN);
                unsigned accum = 0; // the first MMA of a tile overwrites the accumulator
                for (int i = 0; i < nkb; ++i) {
                    if (!mbar_test_addr(full0 + s * 8u, ph)) {
                        ok = mbar_wait(&full_bar[s], ph, abort_flag, args.err);
                        if (!ok) break;
                    }
                    const unsigned al = a_lo0 + soff, bl = b_lo0 + soff;
#pragma unroll
                    for (int j = 0; j < BK / 16; ++j) {
                        if (PAIR) tc_mma_words<true>(tmem_d, al + j * a_kinc, a_hi, bl + j * b_kinc, b_hi, idesc, j == 0 ? accum : 1u);
                        else tc_mma_words<false>(tmem_d, al + j * a_kinc, a_hi, bl + j * b_kinc, b_hi, idesc, j == 0 ? accum : 1u);
                    }
                    accum = 1u;
                    // frees the smem stage (in both CTAs of a pair) once these MMAs have read it
                    tc_commit_addr<PAIR>(empty0 + s * 8u);
                    if (++s == nst) {
                        s = 0;
                        soff = 0;
                        ph ^= 1u;
                    } else {
                        soff += kStageInc;
                    }
                }
                if (!ok) break;
                // accumulator complete
                tc_commit_addr<PAIR>(smem_u32(&acc_full[acc]));
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue (warps 2..5)
        int q = warp & 3; // TMEM lane quarter this warp may access
        const int ew = warp < 6 ? warp - 2 : warp - 3; // epilogue warp 0..7; group 0 = warps 2-5, group 1 = warps 7-10
        const int grp = ew >> 2, groups = args.epi_groups; // a group takes every groups-th chunk of a tile
        unsigned tile_it = 0;
        StageRing rg;
        rg.base = out_stage + ew * (args.ring * 4096);
        rg.issued = 0;
        if (args.zero_n16 > 0 && grp < groups) {
            // nothing to drain until the first accumulator is complete: clear the buffer the caller named (the output of the
            // accumulating GEMM that comes next in the stream), every epilogue thread of the grid its share
            const long long per_cta = 128ll * groups, me = (long long)blockIdx.x * per_cta + (long long)ew * 32 + lane;
            const long long all = (long long)gridDim.x * per_cta;
            const uint4 z = make_uint4(0u, 0u, 0u, 0u);
            for (long long i = me; i < args.zero_n16; i += all) args.zero_ptr[i] = z;
        }
        for (unsigned w = w_first; w < work_total && grp < groups; w += w_stride, ++tile_it) {
            const WorkItem wi = decode_work(args, w, tiles_mn, one_split);
            const int split = wi.split;
            const unsigned t = wi.t;
            const bool part = wi.partial; // slice of a split-tail tile: plain f32 partial sum, added into the workspace
            bool has_k = wi.kb0 < args.kb_total;
            // a pair's CTA holds its own 128 rows of the 256-row tile in its TMEM lanes, all BN columns
            unsigned tn, tm;
            tile_coords(args, t, m_tiles, tn, tm);
            long long m0 = (long long)tm * kTileM + (long long)crank * BM, n0 = (long long)tn * BN;
            int acc = tile_it & 1;
            unsigned acc_ph = (tile_it >> 1) & 1u;
            if (!mbar_wait(&acc_full[acc], acc_ph, abort_flag, args.err, 100u)) break;
            tc_fence_after();
            long long row = m0 + q * 32 + lane;
            // ---- slice of a split-tail tile whose output is finished in the kernel.  Each epilogue warp settles its own
            // elements with the warps of the same index in the other slices.  Slices 1 .. S-1 leave their partial sums
            // (slot = slice - 1) and count themselves done; slice 0 waits (bounded) for that count, adds the partial
            // sums to its accumulator in slice order -- so the result does not depend on who finished first -- and runs
            // the normal epilogue.  All slices of a launch are first items of distinct workers, so the ones slice 0
            // waits for are running at the same time and depend on nothing.
            int others = 0;
            const float *pbase = nullptr;
            if (part && args.fix_ws) {
                const unsigned ridx = t - (unsigned)args.sk_full;
                unsigned *cnt = args.fix_cnt + ((ridx * 2u + crank) * 8u + (unsigned)ew);
                const int n_other = args.sk_splits - 1;
                float *mine = args.fix_ws + (size_t)(ridx * 2u + crank) * (size_t)n_other * (size_t)(BM * BN) + (size_t)(q * 32) * BN + lane * 4;
                if (split > 0) {
                    float *dst = mine + (size_t)(split - 1) * (size_t)(BM * BN);
                    const int cw = args.out_bf16 ? 64 : 32; // the chunks this warp owns in the finishing pass of this launch
#pragma unroll 1
                    for (int c0 = grp * cw; c0 < BN; c0 += cw * groups) {
#pragma unroll 1
                        for (int h = 0; h < cw; h += 32) {
                            unsigned r[32];
                            tmem_ld32(tmem_base + ((unsigned)(q * 32) << 16) + (unsigned)(acc * BN + c0 + h), r);
                            tmem_ld_wait();
#pragma unroll
                            for (int j = 0; j < 8; ++j) *(uint4 *)(dst + (c0 + h) * 32 + j * 128) = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
                        }
                    }
                    __threadfence();
                    __syncwarp();
                    if (lane == 0) atomicAdd(cnt, 1u);
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) {
                        if (PAIR) mbar_arrive_leader(&acc_empty[acc]);
                        else mbar_arrive(&acc_empty[acc]);
                    }
                    continue;
                }
                int okw = 1;
                if (lane == 0) {
                    okw = flag_wait(cnt, (unsigned)n_other, abort_flag, args.err) ? 1 : 0;
                    *cnt = 0; // every other slice has counted itself: ready for the next launch
                }
                okw = __shfl_sync(0xffffffffu, okw, 0);
                __threadfence();
                if (!okw) break;
                others = n_other;
                pbase = mine;
            }
            const bool fin = others > 0;         // finishes a split tile: behaves as a whole tile from here on
            const bool part_out = part && !fin;  // partial sums go straight into an accumulating output
            bool add_bias = args.bias != nullptr && ((split == 0 && !part) || fin);
            if (args.tma_out) {
                // ---- staged output: rows of this warp's 32-row slab go out as 128-byte swizzled boxes
                const int y0 = (int)(m0 + q * 32);
                const bool live = has_k && (long long)y0 < args.m;
                if (args.out_bf16 && !part_out) {
#pragma unroll 1
                    for (int c0 = grp * 64; c0 < BN; c0 += 64 * groups) {
                        unsigned r0[32], r1[32];
                        unsigned taddr = tmem_base + ((unsigned)(q * 32) << 16) + (unsigned)(acc * BN + c0);
                        tmem_ld32(taddr, r0);
                        tmem_ld32(taddr + 32u, r1);
                        tmem_ld_wait();
                        long long col0 = n0 + c0;
                        if (!live || col0 >= args.n) continue;
                        float v[64];
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            v[j] = __uint_as_float(r0[j]);
                            v[32 + j] = __uint_as_float(r1[j]);
                        }
                        for (int s = 0; s < others; ++s) {
                            const float4 *pp = (const float4 *)(pbase + (size_t)s * (size_t)(BM * BN) + c0 * 32);
                            float4 p4[16];
#pragma unroll
                            for (int j = 0; j < 16; ++j) p4[j] = __ldcg(pp + j * 32); // 32-column block c0 (j < 8), then block c0 + 32
#pragma unroll
                            for (int j = 0; j < 16; ++j) {
                                v[4 * j] += p4[j].x; v[4 * j + 1] += p4[j].y; v[4 * j + 2] += p4[j].z; v[4 * j + 3] += p4[j].w;
                            }
                        }
                        if (add_bias) {
                            if (args.bias_vec && col0 + 64 <= args.n) {
                                const float4 *bp = (const float4 *)(args.bias + col0); // col0 is a multiple of 64
#pragma unroll
                                for (int j = 0; j < 16; ++j) {
                                    float4 b4 = __ldg(bp + j);
                                    v[4 * j] += b4.x; v[4 * j + 1] += b4.y; v[4 * j + 2] += b4.z; v[4 * j + 3] += b4.w;
                                }
                            } else {
#pragma unroll
                                for (int j = 0; j < 64; ++j)
                                    if (col0 + j < args.n) v[j] += args.bias[col0 + j];
                            }
                        }
                        if (args.d_pre) {
                            unsigned char *box = ring_acquire(rg, lane, args.ring);
                            unsigned w[32];
                            pack_row_any<64>(v, w, args.f16);
#pragma unroll
                            for (int j = 0; j < 8; ++j) ring_put(box, lane, j, make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]));
                            ring_submit(rg, box, &map_pre, (int)col0, y0, false, lane);
                        }
                        if (args.act == MCB_ACT_GELU) {
#pragma unroll
                            for (int j = 0; j < 64; ++j) v[j] = gelu_f(v[j]);
                        } else if (args.act == MCB_ACT_RELU) {
#pragma unroll
                            for (int j = 0; j < 64; ++j) v[j] = v[j] > 0.0f ? v[j] : 0.0f;
                        }
                        unsigned char *box = ring_acquire(rg, lane, args.ring);
                        {
                            unsigned w[32];
                            pack_row_any<64>(v, w, args.f16);
#pragma unroll
                            for (int j = 0; j < 8; ++j) ring_put(box, lane, j, make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]));
                        }
                        ring_submit(rg, box, &map_d, (int)col0, y0, false, lane);
                    }
                } else {
#pragma unroll 1
                    for (int c0 = grp * 32; c0 < BN; c0 += 32 * groups) {
                        unsigned r[32];
                        unsigned taddr = tmem_base + ((unsigned)(q * 32) << 16) + (unsigned)(acc * BN + c0);
                        tmem_ld32(taddr, r);
                        tmem_ld_wait();
                        long long col0 = n0 + c0;
                        if (!live || col0 >= args.n) continue;
                        float v[32];
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
                        for (int s = 0; s < others; ++s) {
                            const float4 *pp = (const float4 *)(pbase + (size_t)s * (size_t)(BM * BN) + c0 * 32);
                            float4 p4[8];
#pragma unroll
                            for (int j = 0; j < 8; ++j) p4[j] = __ldcg(pp + j * 32);
#pragma unroll
                            for (int j = 0; j < 8; ++j) {
                                v[4 * j] += p4[j].x; v[4 * j + 1] += p4[j].y; v[4 * j + 2] += p4[j].z; v[4 * j + 3] += p4[j].w;
                            }
                        }
                        if (add_bias) {
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                if (col0 + j < args.n) v[j] += args.bias[col0 + j];
                        }
                        if (!args.accumulate && !part_out) {
                            if (args.act == MCB_ACT_GELU) {
#pragma unroll
                                for (int j = 0; j < 32; ++j) v[j] = gelu_f(v[j]);
                            } else if (args.act == MCB_ACT_RELU) {
#pragma unroll
                                for (int j = 0; j < 32; ++j) v[j] = v[j] > 0.0f ? v[j] : 0.0f;
                            }
                        }
                        unsigned char *box = ring_acquire(rg, lane, args.ring);
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            ring_put(box, lane, j,
                                     make_uint4(__float_as_uint(v[4 * j]), __float_as_uint(v[4 * j + 1]), __float_as_uint(v[4 * j + 2]),
                                                __float_as_uint(v[4 * j + 3])));
                        ring_submit(rg, box, part_out ? &map_pre : &map_d, (int)col0, y0, args.accumulate != 0 || part_out, lane);
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    if (PAIR) mbar_arrive_leader(&acc_empty[acc]);
                    else mbar_arrive(&acc_empty[acc]);
                }
                continue;
            }
#pragma unroll 1
            for (int c0 = grp * 32; c0 < BN; c0 += 32 * groups) {
                unsigned r[32];
                unsigned taddr = tmem_base + ((unsigned)(q * 32) << 16) + (unsigned)(acc * BN + c0);
                tmem_ld32(taddr, r);
                tmem_ld_wait();
                long long col0 = n0 + c0;
                if (row < args.m && col0 < args.n && has_k) {
                    float v[32];
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
                    if (add_bias) {
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (col0 + j < args.n) v[j] += args.bias[col0 + j];
                    }
                    bool full = (col0 + 32 <= args.n);
                    if (args.accumulate) {
                        float *dst = (float *)args.d + row * args.ldd + col0;
                        if (full && args.vec_red) {
                            // 128-bit reductions: a quarter of the L2 atomic operations of the scalar form
#pragma unroll
                            for (int j = 0; j < 32; j += 4)
                                asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + j), "f"(v[j]), "f"(v[j + 1]),
                                             "f"(v[j + 2]), "f"(v[j + 3])
                                             : "memory");
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                if (full || col0 + j < args.n) atomicAdd(dst + j, v[j]);
                        }
                    } else if (args.out_bf16) {
                        __nv_bfloat16 *dst = (__nv_bfloat16 *)args.d + row * args.ldd + col0;
                        __nv_bfloat16 *pre = args.d_pre ? (__nv_bfloat16 *)args.d_pre + row * args.ldd + col0 : nullptr;
                        if (pre) {
                            unsigned w[16];
                            pack_row_any<32>(v, w, args.f16);
                            if (full) {
#pragma unroll
                                for (int j = 0; j < 4; ++j) *(uint4 *)(pre + 8 * j) = make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
                            } else {
                                for (int j = 0; j < 32; ++j)
                                    if (col0 + j < args.n) ((unsigned short *)pre)[j] = (unsigned short)(w[j >> 1] >> ((j & 1) * 16));
                            }
                        }
                        if (args.act == MCB_ACT_GELU) {
#pragma unroll
                            for (int j = 0; j < 32; ++j) v[j] = gelu_f(v[j]);
                        } else if (args.act == MCB_ACT_RELU) {
#pragma unroll
                            for (int j = 0; j < 32; ++j) v[j] = v[j] > 0.0f ? v[j] : 0.0f;
                        }
                        unsigned w[16];
                        pack_row_any<32>(v, w, args.f16);
                        if (full) {
#pragma unroll
                            for (int j = 0; j < 4; ++j) *(uint4 *)(dst + 8 * j) = make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
                        } else {
                            for (int j = 0; j < 32; ++j)
                                if (col0 + j < args.n) ((unsigned short *)dst)[j] = (unsigned short)(w[j >> 1] >> ((j & 1) * 16));
                        }
                    } else {
                        float *dst = (float *)args.d + row * args.ldd + col0;
                        if (args.act == MCB_ACT_GELU) {
#pragma unroll
                            for (int j = 0; j < 32; ++j) v[j] = gelu_f(v[j]);
                        } else if (args.act == MCB_ACT_RELU) {
#pragma unroll
                            for (int j = 0; j < 32; ++j) v[j] = v[j] > 0.0f ? v[j] : 0.0f;
                        }
                        if (full) {
#pragma unroll
                            for (int j = 0; j < 32; j += 4) *(float4 *)(dst + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                        } else {
                            for (int j = 0; j < 32; ++j)
                                if (col0 + j < args.n) dst[j] = v[j];
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (PAIR) mbar_arrive_leader(&acc_empty[acc]);
                else mbar_arrive(&acc_empty[acc]);
            }
        }
        // output boxes still being read from this CTA's shared memory must be done before it exits
        if (lane == 0) bulk_wait_all();
    }
    tc_fence_before();
    __syncthreads();
    if (PAIR) {
        // neither CTA may exit (or free the shared TMEM allocation) while its peer can still signal
        // its barriers or while the leader's MMAs can still read its operand tiles
        cluster_sync_all();
        if (warp == 1) tmem_dealloc_pair(tmem_base, 512);
    } else if (warp == 1) {
        tmem_dealloc(tmem_base, 512);
    }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void *p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

// 2-D bf16 tensor map: inner (contiguous) extent `inner`, outer extent `outer`, row pitch `ld` elements
mcb_status make_map(mcb_ctx *ctx, CUtensorMap *map, const void *base, long long inner, long long outer, long long ld,
                    int box_inner, int box_outer, bool f16 = false) {
    EncodeTiledFn enc = get_encode();
    if (!enc) return mcb_fail(ctx, MCB_BACKEND, "cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)box_inner, (cuuint32_t)box_outer};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return mcb_fail(ctx, MCB_BACKEND, "cuTensorMapEncodeTiled failed with %d", (int)r);
    return MCB_OK;
}

// output matrix [m, n] with row pitch ldd, written in boxes of {128 bytes, 32 rows}
mcb_status make_out_map(mcb_ctx *ctx, CUtensorMap *map, const void *base, bool bf16, long long n, long long m, long long ldd, bool f16 = false) {
    EncodeTiledFn enc = get_encode();
    if (!enc) return mcb_fail(ctx, MCB_BACKEND, "cuTensorMapEncodeTiled is not available from the driver");
    const int es = bf16 ? 2 : 4;
    cuuint64_t dims[2] = {(cuuint64_t)n, (cuuint64_t)m};
    cuuint64_t strides[1] = {(cuuint64_t)ldd * es};
    cuuint32_t box[2] = {(cuuint32_t)(128 / es), 32u};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, bf16 ? (f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16) : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void *>(base), dims,
                     strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return mcb_fail(ctx, MCB_BACKEND, "cuTensorMapEncodeTiled (output) failed with %d", (int)r);
    return MCB_OK;
}

template <int BN, bool PAIR> mcb_status launch(mcb_ctx *ctx, const TcGemmParams &p) {
    using C = Cfg<BN, PAIR>;
    constexpr int kTileM = PAIR ? 2 * BM : BM;
    CUtensorMap map_a, map_b;
    const bool f16 = p.in_dt == MCB_F16;
    if (!p.a_mn_major) MCB_TRY(make_map(ctx, &map_a, p.a, p.k, p.m, p.lda, BK, BM, f16));
    else MCB_TRY(make_map(ctx, &map_a, p.a, p.m, p.k, p.lda, 64, BK, f16));
    if (!p.b_mn_major) MCB_TRY(make_map(ctx, &map_b, p.b, p.k, p.n, p.ldb, BK, C::kBRows, f16));
    else MCB_TRY(make_map(ctx, &map_b, p.b, p.n, p.k, p.ldb, 64, BK, f16));
    TcArgs a;
    a.d = p.d;
    a.d_pre = p.d_pre;
    a.bias = p.bias;
    a.m = p.m; a.n = p.n; a.k = p.k; a.ldd = p.ldd;
    a.out_bf16 = mcb_is_lp(p.out_dt);
    a.f16 = f16;
    a.accumulate = p.accumulate;
    a.vec_red = (p.ldd % 4 == 0) && mcb_aligned16(p.d);
    a.act = p.act;
    a.a_mn = p.a_mn_major;
    a.b_mn = p.b_mn_major;
    // kind::f16 instruction descriptor: f32 accumulator (bit 4); operand formats in bits 7-9 (A) and 10-12 (B): 0 = f16, 1 = bf16
    a.idesc = (1u << 4) | (f16 ? 0u : ((1u << 7) | (1u << 10))) | ((unsigned)(p.a_mn_major ? 1 : 0) << 15) |
              ((unsigned)(p.b_mn_major ? 1 : 0) << 16) | ((unsigned)(BN >> 3) << 17) | ((unsigned)(kTileM >> 4) << 24);
    a.m_tiles = (int)((p.m + kTileM - 1) / kTileM);
    a.n_tiles = (int)((p.n + BN - 1) / BN);
    a.kb_total = (int)((p.k + BK - 1) / BK);
    // A that cannot stay in L2 (126 MB) beside a B that can: walk the column blocks of a row block together
    a.n_fast = ((double)p.m * (double)p.k * 2.0 > 96.0e6 && (double)p.n * (double)p.k * 2.0 < 64.0e6 && a.n_tiles > 1) ? 1 : 0;
    int split = p.split_k < 1 ? 1 : p.split_k;
    if (split > a.kb_total) split = a.kb_total > 0 ? a.kb_total : 1;
    a.kb_per_split = (a.kb_total + split - 1) / split;
    split = a.kb_total > 0 ? (a.kb_total + a.kb_per_split - 1) / a.kb_per_split : 1;
    a.split_k = split;
    a.err = ctx->d_err;
    if ((long long)a.m_tiles * a.n_tiles * split >= (1ll << 31) || p.m >= (1ll << 31) || p.n >= (1ll << 31) || p.k >= (1ll << 31))
        return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "tensor-core GEMM: dimensions beyond 2^31 are not supported");
    a.bias_vec = p.bias && mcb_aligned16(p.bias);
    a.stages = C::kStages;
    a.ring = 2;
    // Short reductions on 256-wide pair tiles are bound by the latency of the output stores (eight 4 KB boxes per
    // tile and warp, sixteen with a second output), not by the operand ring: one stage less, four boxes in flight.
    // (8192x3072x768: 34.8 -> 32.6 us; with K = 8192 or more the sixth stage is worth more: 323 -> 347 us.)
    // The room of that stage goes either to four boxes per warp or to a second group of four epilogue warps (two boxes
    // each) that takes every other chunk; MCB_TC_EPI=1 keeps the single group (tuning knob).
    const bool one_group = knob_val(ctx, K_TC_EPI, 0) == 1;
    a.epi_groups = 1;
    const int short_kb = knob_val(ctx, K_TC_EPI_KB, 16); // tuning knob: k-blocks per item up to which the stage is traded
    if (PAIR && BN == 256 && a.kb_per_split <= short_kb && C::kStageBytes * 1 >= 4 * 2 * 4096 && !knob_on(ctx, K_TC_STAGES)) {
        a.stages = C::kStages - 1;
        if (one_group) a.ring = 4;
        else a.epi_groups = 2;
    }
    if (BN == 192 && !PAIR && !one_group) a.epi_groups = 2; // 128 x 192 tiles: room for both groups beside the four stages
    if (knob_on(ctx, K_TC_STAGES)) {
        int v = knob_val(ctx, K_TC_STAGES, 0);
        if (v >= 2 && v < C::kStages) a.stages = v;
    }
    // TMA output needs a 16-byte aligned base and row pitch; only an accumulating f32 output may lack them
    a.tma_out = mcb_aligned16(p.d) && (p.ldd * (a.out_bf16 ? 2 : 4)) % 16 == 0 && (!p.d_pre || mcb_aligned16(p.d_pre));
    const bool no_tma_out = knob_on(ctx, K_TC_DIRECT_OUT); // tuning knob: per-lane global stores
    if (no_tma_out) a.tma_out = 0;
    CUtensorMap map_d, map_pre;
    memset(&map_d, 0, sizeof(map_d));
    memset(&map_pre, 0, sizeof(map_pre));
    if (a.tma_out) {
        MCB_TRY(make_out_map(ctx, &map_d, p.d, a.out_bf16, p.n, p.m, p.ldd, f16));
        if (p.d_pre) MCB_TRY(make_out_map(ctx, &map_pre, p.d_pre, a.out_bf16, p.n, p.m, p.ldd, f16));
    }
    long long work = (long long)a.m_tiles * a.n_tiles * split;
    static bool attr_set = false;
    static int max_pairs = 0;
    if (!attr_set) {
        MCB_CUDA(ctx, cudaFuncSetAttribute(tc_gemm_kernel<BN, PAIR>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes));
        if (PAIR) {
            // how many 2-CTA clusters can be resident at once (GPCs with an odd SM count leave one SM idle)
            cudaLaunchConfig_t qc = {};
            qc.gridDim = dim3(ctx->sm_count & ~1);
            qc.blockDim = dim3(kThreads);
            qc.dynamicSmemBytes = C::kSmemBytes;
            cudaLaunchAttribute qa[1];
            qa[0].id = cudaLaunchAttributeClusterDimension;
            qa[0].val.clusterDim.x = 2;
            qa[0].val.clusterDim.y = 1;
            qa[0].val.clusterDim.z = 1;
            qc.attrs = qa;
            qc.numAttrs = 1;
            int nc = 0;
            MCB_CUDA(ctx, cudaOccupancyMaxActiveClusters(&nc, tc_gemm_kernel<BN, PAIR>, &qc));
            max_pairs = nc > 0 ? nc : 1;
            if (max_pairs > ctx->sm_count / 2) max_pairs = ctx->sm_count / 2;
        }
        attr_set = true;
    }
    // Split tail: when the tiles do not fill the last wave, the tiles of that wave are cut along K so that every
    // worker gets one slice.  An accumulating output takes the slices directly; any other output is finished inside
    // the kernel by slice 0 of each tile (TcArgs::fix_ws).
    void *ws = nullptr;
    a.sk_full = a.sk_rem = a.sk_kb = 0;
    a.sk_splits = 1;
    a.fix_ws = nullptr;
    a.fix_cnt = nullptr;
    a.zero_ptr = (uint4 *)p.zero_ptr;
    a.zero_n16 = p.zero_ptr ? (long long)(p.zero_bytes / 16) : 0;
    const int workers = PAIR ? max_pairs : ctx->sm_count;
    const long long tiles = (long long)a.m_tiles * a.n_tiles;
    const bool direct = p.accumulate && !p.bias; // slices add straight into the f32 output
    if (p.split_tail && a.tma_out && split == 1 && tiles > workers && (direct || !p.accumulate)) {
        const long long rem = tiles % workers, full = tiles - rem;
        int s = rem > 0 ? (int)(workers / rem) : 1;
        if (s > 8) s = 8;
        if (s > a.kb_total / 4) s = a.kb_total / 4;
        if (s >= 2) {
            const int kb = (a.kb_total + s - 1) / s;
            s = (a.kb_total + kb - 1) / kb;
            const size_t ws_bytes = direct ? 0 : sizeof(float) * (size_t)rem * 2 * (size_t)(s - 1) * BM * BN;
            if (s >= 2 && ws_bytes <= ((size_t)96 << 20) && rem <= kFixTiles) {
                if (direct) {
                    map_pre = map_d;
                } else {
                    MCB_TRY(mcb_alloc(ctx, ws_bytes, &ws));
                    a.fix_ws = (float *)ws;
                    a.fix_cnt = ctx->tc_fix_cnt;
                }
                a.sk_full = (int)full;
                a.sk_rem = (int)rem;
                a.sk_splits = s;
                a.sk_kb = kb;
                work = full + rem * s;
            }
        }
    }
    cudaError_t le;
    if (!PAIR) {
        int grid = (int)(work < ctx->sm_count ? work : ctx->sm_count);
        le = mcb_launch_dep(ctx, tc_gemm_kernel<BN, false>, dim3(grid), dim3(kThreads), C::kSmemBytes, map_a, map_b, map_d, map_pre, a);
    } else {
        int pairs = (int)(work < max_pairs ? work : max_pairs);
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2 * pairs);
        cfg.blockDim = dim3(kThreads);
        cfg.dynamicSmemBytes = C::kSmemBytes;
        cfg.stream = ctx->stream;
        cudaLaunchAttribute at[2];
        at[0].id = cudaLaunchAttributeClusterDimension;
        at[0].val.clusterDim.x = 2;
        at[0].val.clusterDim.y = 1;
        at[0].val.clusterDim.z = 1;
        at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization; // see dep_wait() in the kernel
        at[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = at;
        cfg.numAttrs = ctx->dep_launch ? 2 : 1;
        le = cudaLaunchKernelEx(&cfg, tc_gemm_kernel<BN, true>, map_a, map_b, map_d, map_pre, a);
    }
    if (ws) mcb_free(ctx, ws); // stream-ordered reuse: whoever gets the block next is enqueued behind this kernel
    MCB_CUDA(ctx, le);
    MCB_LAUNCHED(ctx);
    return MCB_OK;
}

} // namespace

mcb_status mcb_tc_gemm(mcb_ctx *ctx, const TcGemmParams &p) {
    if (p.zero_ptr && (p.m == 0 || p.n == 0 || p.k == 0)) MCB_TRY(mcb_memset(ctx, p.zero_ptr, 0, p.zero_bytes)); // no kernel will run: clear it here
    if (p.m == 0 || p.n == 0) return MCB_OK;
    ProfScope prof(ctx, MCB_PROF_GEMM_TC, 2.0 * (double)p.m * (double)p.n * (double)p.k,
                   2.0 * ((double)p.m * p.k + (double)p.n * p.k) + (double)p.m * p.n * (mcb_is_lp(p.out_dt) ? 2.0 : 4.0));
    if (p.k == 0) {
        if (p.accumulate) return MCB_OK;
        return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "tensor-core GEMM needs k > 0");
    }
    if ((p.lda % 8) || (p.ldb % 8) || !mcb_aligned16(p.a) || !mcb_aligned16(p.b))
        return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "tensor-core GEMM operands need 16-byte aligned bases and row pitches that are multiples of 8 elements");
    if (!mcb_is_lp(p.in_dt)) return mcb_fail(ctx, MCB_UNSUPPORTED_DTYPE, "tensor-core GEMM operands must be bf16 or f16");
    if (p.out_dt != p.in_dt && p.out_dt != MCB_F32) return mcb_fail(ctx, MCB_UNSUPPORTED_DTYPE, "GEMM output must be f32 or the operands' 16-bit type");
    if (p.accumulate && p.out_dt != MCB_F32) return mcb_fail(ctx, MCB_UNSUPPORTED_DTYPE, "accumulating GEMM output must be f32");
    if (p.zero_ptr && (!mcb_aligned16(p.zero_ptr) || p.zero_bytes % 16))
        return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "the buffer a GEMM clears on the side must be 16-byte aligned and a multiple of 16 bytes long");
    if (p.split_k > 1 && !p.accumulate) return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "split-K needs the accumulating epilogue");
    // vector stores in the epilogue need ldd and d aligned; otherwise the scalar tail path is used per row
    if ((mcb_is_lp(p.out_dt) && ((p.ldd % 8) || !mcb_aligned16(p.d))) || (p.out_dt == MCB_F32 && !p.accumulate && ((p.ldd % 4) || !mcb_aligned16(p.d))))
        return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "GEMM output needs a 16-byte aligned base and row pitch");
    int bn = p.bn, split = p.split_k < 1 ? 1 : p.split_k;
    // reproducible runs: slices of one reduction reach the output in arrival order, so there are none
    const bool fixed_order = knob_on(ctx, K_DETERMINISTIC);
    if (fixed_order) split = 1;
    bn = knob_val(ctx, K_TC_BN, bn); // tuning knob: force the tile width
    if (bn != 128 && bn != 192 && bn != 256) {
        int s2 = split;
        mcb_tc_plan(ctx, p.m, p.n, p.k, false, p.accumulate, split, &bn, &s2);
    }
    TcGemmParams q = p;
    q.split_k = split;
    int pair = p.pair;
    pair = knob_val(ctx, K_TC_PAIR, pair); // tuning knob: 0 single CTA, 1 CTA pair
    if (pair < 0) pair = (bn != 192 && p.m > 128) ? 1 : 0;
    if (bn == 192) pair = 0; // half of 192 columns is not a whole number of 64-column boxes
    // Split tail on 256 x 256 pair tiles against the planned form, by the same cycle estimate as mcb_tc_plan
    // plus kFixCycles for leaving and collecting the partial sums of the slices
    int tail = p.split_tail;
    tail = knob_val(ctx, K_TC_SPLIT_TAIL, tail); // tuning knob: 0 never, 1 whenever it applies
    if (fixed_order && p.accumulate) tail = 0; // (a tail finished in the kernel adds in slice order: reproducible as it is)
    const bool tail_ok = (p.accumulate ? (p.bias == nullptr) : (split == 1)) && p.m > 128 && !knob_on(ctx, K_TC_BN);
    if (tail < 0 && tail_ok) {
        const long long kb = (p.k + BK - 1) / BK, workers = ctx->sm_count / 2;
        const long long tiles = ((p.m + 255) / 256) * ((p.n + 255) / 256), rem = tiles % workers;
        long long s = rem > 0 ? workers / rem : 1;
        if (s > 8) s = 8;
        if (s > kb / 4) s = kb / 4;
        tail = 0;
        if (tiles > workers && s >= 2) {
            const double per_tail = 4.0 * 128.0 + 60.0;
            // an accumulating output takes the slices directly; otherwise workspace memset + finishing kernel
            const double cost_tail = (double)((tiles / workers) * kb + (kb + s - 1) / s) * per_tail + 12.0 * 256 + (p.accumulate ? 1000.0 : kFixCycles);
            // the planned form: `split` slices of every tile
            const long long w_now = pair ? ctx->sm_count / 2 : ctx->sm_count;
            const long long t_now = ((p.m + (pair ? 255 : 127)) / (pair ? 256 : 128)) * ((p.n + bn - 1) / bn);
            const long long kb_item = (kb + split - 1) / split, items = t_now * ((kb + kb_item - 1) / kb_item);
            const double mma = bn / 2.0 > 125.0 ? bn / 2.0 : 125.0;
            const double cost_now = (double)((items + w_now - 1) / w_now) * (double)kb_item * (4.0 * mma + 60.0) + (p.accumulate ? 12.0 : 5.0) * bn +
                                    (split > 1 ? 300.0 * split + (double)(split - 1) * (double)p.m * (double)p.n * 1.0e-3 : 0.0);
            if (cost_tail < 0.9 * cost_now) tail = 1;
        }
    }
    if (!tail_ok || tail < 0) tail = 0;
    q.split_tail = tail;
    if (tail) {
        bn = 256;
        pair = 1;
        q.split_k = 1; // the tail is the only part that is cut along K
    }
    if (pair) {
        if (bn == 256) return launch<256, true>(ctx, q);
        return launch<128, true>(ctx, q);
    }
    if (bn == 256) return launch<256, false>(ctx, q);
    if (bn == 192) return launch<192, false>(ctx, q);
    return launch<128, false>(ctx, q);
}

// Picks the tile width (and, when the caller can zero the output and accept atomic accumulation,
// the split of the reduction dimension) that minimises a cycle estimate for one CTA:
//   waves * k_blocks_per_item * (4 * max(BN/2, 125) + 60)  +  exposed epilogue
// where the first term is the time of the four K=16 MMAs of one 64-deep block at M=128.
void mcb_tc_plan(mcb_ctx *ctx, int64_t m, int64_t n, int64_t k, bool allow_split, bool atomic_out, int fixed_split, int *bn_out,
                 int *split_out) {
    const int cands[3] = {256, 192, 128};
    long long m_tiles = (m + BM - 1) / BM, kb_total = (k + BK - 1) / BK;
    double best = 1e300;
    int best_bn = 256, best_split = 1;
    int max_split = allow_split ? 16 : 1;
    for (int i = 0; i < 3; ++i) {
        int bn = cands[i];
        long long tiles = m_tiles * ((n + bn - 1) / bn);
        for (int s = 1; s <= max_split; ++s) {
            int sp = allow_split ? s : (fixed_split < 1 ? 1 : fixed_split);
            if (sp > 1 && kb_total / sp < 4) break;
            long long kb = (kb_total + sp - 1) / sp;
            long long items = tiles * ((kb_total + kb - 1) / kb);
            long long waves = (items + ctx->sm_count - 1) / ctx->sm_count;
            bool atomics = atomic_out || sp > 1;
            double epi = (atomics ? 12.0 : 5.0) * bn;
            // with several waves the epilogue of all but the last tile hides behind the next tile's MMAs
            // one K=16 MMA at M=128 takes bn/2 cycles but never less than ~125 (the A operand's 4 KB
            // leave shared memory at 32 B/clk), so narrow tiles run the tensor pipe below its rate
            double mma = bn / 2.0 > 125.0 ? bn / 2.0 : 125.0;
            // every additional slice adds the whole f32 output once more into L2 (measured: 13 us per slice on a
            // 32000 x 768 output, i.e. about 1e-3 cycles per output element and slice)
            double cost = (double)waves * (double)kb * (4.0 * mma + 60.0) + epi +
                          (sp > 1 ? 300.0 * sp + (double)(sp - 1) * (double)m * (double)n * 1.0e-3 : 0.0);
            if (bn == 256 && sp == 1 && m > 128) {
                // unsplit 256-wide tiles may run with a split tail (see mcb_tc_gemm): same estimate as there
                const long long workers = ctx->sm_count / 2, t256 = ((m + 255) / 256) * ((n + 255) / 256), rem = t256 % workers;
                long long st = rem > 0 ? workers / rem : 1;
                if (st > 8) st = 8;
                if (st > kb_total / 4) st = kb_total / 4;
                if (t256 > workers && st >= 2) {
                    const double tail = (double)((t256 / workers) * kb_total + (kb_total + st - 1) / st) * (4.0 * 128.0 + 60.0) + 12.0 * 256 +
                                        (atomic_out ? 1000.0 : kFixCycles);
                    if (tail < 0.9 * cost) cost = tail;
                }
            }
            if (cost < best - 1e-9) {
                best = cost;
                best_bn = bn;
                best_split = sp;
            }
        }
    }
    *bn_out = best_bn;
    *split_out = best_split;
}

extern "C" mcb_status mcb_gemm_bf16(mcb_ctx *ctx, const void *a, int32_t a_mn_major, const void *b, int32_t b_mn_major,
                                    void *d, int32_t out_dt, const float *bias, int64_t m, int64_t n, int64_t k,
                                    int32_t accumulate, int32_t split_k) {
    return mcb_gemm_lowp(ctx, MCB_BF16, a, a_mn_major, b, b_mn_major, d, out_dt, bias, m, n, k, accumulate, split_k);
}

extern "C" mcb_status mcb_gemm_lowp(mcb_ctx *ctx, int32_t in_dt, const void *a, int32_t a_mn_major, const void *b, int32_t b_mn_major,
                                    void *d, int32_t out_dt, const float *bias, int64_t m, int64_t n, int64_t k,
                                    int32_t accumulate, int32_t split_k) {
    MCB_CHECK_CTX(ctx);
    TcGemmParams p;
    p.in_dt = in_dt;
    p.a = a; p.b = b; p.d = d; p.bias = bias;
    p.a_mn_major = a_mn_major; p.b_mn_major = b_mn_major;
    p.out_dt = out_dt;
    p.m = m; p.n = n; p.k = k;
    p.lda = a_mn_major ? m : k;
    p.ldb = b_mn_major ? n : k;
    p.ldd = n;
    p.accumulate = accumulate;
    p.split_k = split_k;
    if (split_k <= 0) { // let the library choose; splitting is only possible with the accumulating epilogue
        int bn = 0, sp = 1;
        mcb_tc_plan(ctx, m, n, k, accumulate != 0, accumulate != 0, 1, &bn, &sp);
        p.bn = bn;
        p.split_k = sp;
    }
    return mcb_tc_gemm(ctx, p);
}
