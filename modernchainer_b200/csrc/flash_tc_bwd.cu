// Fused attention backward on the tcgen05 tensor cores (bf16 / f16, head_dim 64): two kernels from one template and a third:
//   MODE 0 (dK, dV): one CTA per 128-key tile; K_j, V_j stay in shared memory, the query tiles stream through.
//   MODE 1 (dQ)    : one CTA per 128-query tile; Q_i, dO_i stay, the key tiles stream through (recomputes S, dP, dS).
//   flash_tc_dq_kernel: dQ += dS K from the dS tiles that MODE 0 leaves in a scratch buffer as it goes (32 KB per pair,
//                    the bytes of its shared-memory tile), so dQ costs 8 MMAs per pair and no exponentials instead of 16
//                    MMAs and a second evaluation of P and dS.  The default; MODE 1 stays for sequences whose dS would
//                    not fit the scratch limit and as a cross-check (knob MCB_FLASH_DQ_RECOMPUTE).
// Per (query tile, key tile) pair, with rows = queries (TMEM lanes) and columns = keys:
//   S  = Q K^T, dP = dO V^T         tcgen05.mma M=128 N=128 K=64 each, both into TMEM
//   P  = exp2(S * scale*log2e - lse*log2e),  dS = P * (dP - delta)     (masked pairs give 0)
//        eight warps, two per TMEM lane quarter, each thread takes 64 keys of its query row: one TMEM round
//        trip for S and dP, independent arithmetic per element, results packed to bf16 into shared memory as
//        [key block][query block][64 queries][64 keys] atoms of 8 KB with the 128-byte swizzle.  That one
//        layout serves as the K-major operand dS (for dQ) and as the MN-major operands P^T, dS^T (for dV, dK).
//   MODE 0: dV += P^T dO, dK += dS^T Q   M=128 (keys) N=64 K=128 (queries), accumulators in TMEM for the whole walk
//   MODE 1: dQ += dS K                   M=128 (queries) N=64 K=128 (keys)
// The next pair's S / dP are issued as soon as the rows have read the current ones, so they run under the
// exponentials; the 1/sqrt(hd) factor is applied once, to dK and dQ, in the epilogue.
// delta = rowsum(O * dO) and the log-sum-exp come from the forward pass / a small pre-kernel.
// Roles (320 threads): warp 0 TMA, warp 1 MMA + TMEM, warps 2..9 the pair arithmetic and the epilogue.
// Every mbarrier wait is bounded; on expiry the CTA raises the device error word and drains.
#include "internal.h"
#include "tc_ptx.cuh"

using namespace tcptx;

namespace {

constexpr int HD = 64;
constexpr int BT = 128;  // tile edge: queries and keys per tile
constexpr int kThreads = 320;
constexpr int kTileBytes = BT * HD * 2;  // 16 KB
// shared memory: X0 X1 (resident pair) | Y0 Y1 x 2 stages (streamed pair) | P | dS | barriers
constexpr int kSmemX = 0, kSmemY = 2 * kTileBytes, kSmemP = kSmemY + 4 * kTileBytes, kSmemDS = kSmemP + 2 * kTileBytes,
              kSmemBar = kSmemDS + 2 * kTileBytes;
constexpr int kSmemBytes = kSmemBar + 128 + 1024;
constexpr unsigned kTmemCols = 512;
constexpr unsigned kColS = 0, kColDP = 128, kColAcc0 = 256, kColAcc1 = 320;
constexpr unsigned kColDSt = 320; // MODE 1: dS as packed bf16 pairs (64 columns), the A operand of dQ += dS K, read from TMEM
constexpr unsigned kColAccAlt1 = 448; // MODE 1: dQ accumulator of odd jobs (even jobs: kColAcc0); MODE 0 alternates kColAcc0 / +64 and 384 / 448

struct BwdArgs {
    const float *lse, *delta;  // [n, heads, seq]
    int seq, heads, causal;
    int tiles, nh_total, jobs; // tiles per sequence, samples * heads, tiles * nh_total
    float scale, scale_log2;
    unsigned int *err;
    // optional by-product: column sums of the bf16 values each epilogue warp writes (the q / k / v bias gradients before
    // their final reduction): row (sample * tiles + tile) * 4 + lane quarter of [.., bias_ld], columns which * dim + head * 64
    float *bias_partial;
    int bias_ld, dim;
    // MODE 0 only, optional: where to leave dS of every pair for flash_tc_dq_kernel, [sample * heads + head][query tile][key tile]
    // blocks of kDsBytes (the shared-memory tile as it is)
    unsigned char *ds_out;
};
constexpr int kDsBytes = 2 * kTileBytes;

// One job = one (owned tile, sample, head).  Jobs are numbered heaviest first (job / nh_total is the weight rank: under a
// causal mask the owned tile that walks the most streamed tiles) and dealt to the persistent CTAs in boustrophedon order
// (first pass: CTA c takes job c, second pass: job 2G-1-c, ...), which balances the step counts as well as longest-first list
// scheduling does (24 against an average of 23.4 steps on 148 CTAs for 8 x 12 heads of 8 tiles).
struct Job {
    int n, h, nh, own, t_first, nt, o0;
};
template <int MODE> __device__ __forceinline__ bool job_at(const BwdArgs &args, int it, Job &j) {
    const int G = (int)gridDim.x, c = (int)blockIdx.x;
    const int idx = it * G + ((it & 1) ? G - 1 - c : c);
    if (idx >= args.jobs) return false;
    const int rank = idx / args.nh_total;
    j.nh = idx - rank * args.nh_total;
    j.n = j.nh / args.heads;
    j.h = j.nh % args.heads;
    // MODE 0: the CTA owns key tile `own`; query tiles own..tiles-1 (causal) or all stream through.
    // MODE 1: the CTA owns query tile `own` (late tiles first when causal); key tiles 0..own (causal) or all stream through.
    j.own = (MODE == 1 && args.causal) ? args.tiles - 1 - rank : rank;
    j.t_first = (MODE == 0 && args.causal) ? j.own : 0;
    j.nt = (MODE == 0) ? args.tiles - j.t_first : (args.causal ? j.own + 1 : args.tiles);
    j.o0 = j.own * BT;
    return true;
}

// Persistent: one CTA per SM walks its jobs.  All barriers count steps (pairs of tiles) globally across the jobs of a CTA,
// so the next job's resident tiles are loaded as soon as the last S / dP of the current job has read the old ones, its
// first S / dP are issued behind the current job's last accumulating MMAs, and its first pair's arithmetic follows the
// current job's epilogue directly.  The accumulators alternate between two sets of TMEM columns from job to job.
template <int MODE, bool F16>
__global__ void __launch_bounds__(kThreads, 1)
flash_tc_bwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                    const __grid_constant__ CUtensorMap map_do, const __grid_constant__ CUtensorMap map_out0,
                    const __grid_constant__ CUtensorMap map_out1, BwdArgs args) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char *smem = (unsigned char *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char *sX0 = smem + kSmemX, *sX1 = sX0 + kTileBytes, *sP = smem + kSmemP, *sDS = smem + kSmemDS;
    unsigned long long *bars = (unsigned long long *)(smem + kSmemBar);
    unsigned long long *x_full = bars, *y_full = bars + 1, *y_empty = bars + 3, *sd_full = bars + 5, *sd_free = bars + 6, *pds_full = bars + 7,
                       *mma_done = bars + 8, *x_empty = bars + 9, *epi_done = bars + 10;
    unsigned *tmem_slot = (unsigned *)(bars + 11);
    volatile int *abort_flag = (volatile int *)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles = args.tiles;

    if (threadIdx.x == 0) {
        prefetch_map(&map_q);
        prefetch_map(&map_k);
        prefetch_map(&map_v);
        prefetch_map(&map_do);
        prefetch_map(&map_out0);
        prefetch_map(&map_out1);
        mbar_init(x_full, 1);
        mbar_init(x_empty, 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(&y_full[s], 1);
            mbar_init(&y_empty[s], 1);
        }
        mbar_init(sd_full, 1);
        mbar_init(sd_free, 8);
        mbar_init(pds_full, 8);
        mbar_init(mma_done, 1);
        mbar_init(epi_done, 8);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem_base = *tmem_slot;
    // Only shared and tensor memory so far: this much may overlap the previous kernel of the stream.  The dK/dV
    // kernel (MODE 0) waits here for everything before it.  The recomputing dQ kernel (MODE 1) is launched right behind
    // it, reads the same inputs and writes other bytes, so it needs nothing from MODE 0: it starts on the SMs that MODE 0's
    // tail leaves idle (MODE 0 raised its trigger after its own wait, so all earlier kernels are complete by then) and
    // waits for MODE 0 only before it exits, which keeps the stream in order for whatever follows.
    if (MODE == 0) dep_wait();
    dep_trigger();

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            bool ok = true;
            unsigned g = 0; // steps issued so far, over all jobs of this CTA
            Job jb;
            for (int it = 0; ok && job_at<MODE>(args, it, jb); ++it) {
                // the resident pair: free again once the last S / dP of the previous job has read it
                if (it > 0) ok = mbar_wait(x_empty, (unsigned)(it - 1) & 1u, abort_flag, args.err);
                if (!ok) break;
                mbar_expect_tx(x_full, 2 * kTileBytes);
                if (MODE == 0) {
                    tma_load_3d(sX0, &map_k, x_full, jb.h * HD, jb.o0, jb.n);
                    tma_load_3d(sX1, &map_v, x_full, jb.h * HD, jb.o0, jb.n);
                } else {
                    tma_load_3d(sX0, &map_q, x_full, jb.h * HD, jb.o0, jb.n);
                    tma_load_3d(sX1, &map_do, x_full, jb.h * HD, jb.o0, jb.n);
                }
                for (int t = 0; t < jb.nt && ok; ++t, ++g) {
                    const unsigned st = g & 1u;
                    ok = mbar_wait(&y_empty[st], ((g >> 1) & 1u) ^ 1u, abort_flag, args.err);
                    if (!ok) break;
                    unsigned char *y0 = smem + kSmemY + st * 2 * kTileBytes, *y1 = y0 + kTileBytes;
                    const int r0 = (jb.t_first + t) * BT;
                    mbar_expect_tx(&y_full[st], 2 * kTileBytes);
                    if (MODE == 0) {
                        tma_load_3d(y0, &map_q, &y_full[st], jb.h * HD, r0, jb.n);
                        tma_load_3d(y1, &map_do, &y_full[st], jb.h * HD, r0, jb.n);
                    } else {
                        tma_load_3d(y0, &map_k, &y_full[st], jb.h * HD, r0, jb.n);
                        tma_load_3d(y1, &map_v, &y_full[st], jb.h * HD, r0, jb.n);
                    }
                }
            }
            for (unsigned st = 0; st < 2 && ok; ++st) { // drain: every stage that was filled has been consumed
                const unsigned fills = (g > st) ? ((g - 1 - st) / 2 + 1) : 0;
                if (fills) ok = mbar_wait(&y_empty[st], (fills - 1) & 1u, abort_flag, args.err);
            }
            if (*abort_flag) {
                unsigned long long t0 = global_ns();
                while (global_ns() - t0 < 200000ull) {
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr unsigned idesc_sd = make_idesc(BT, BT, 0, 0, F16);                       // S, dP: both operands K-major
            constexpr unsigned idesc_acc = make_idesc(BT, HD, MODE == 0 ? 1 : 0, 1, F16);      // MODE 0: A = P^T / dS^T (MN-major); MODE 1: A = dS (K-major)
            const unsigned x0 = smem_u32(sX0), x1 = smem_u32(sX1), p_addr = smem_u32(sP), ds_addr = smem_u32(sDS);
            auto issue_sd = [&](unsigned gg) {
                const unsigned y0 = smem_u32(smem + kSmemY + (gg & 1u) * 2 * kTileBytes), y1 = y0 + kTileBytes;
                // S = Q K^T and dP = dO V^T: MODE 0 streams (Q, dO) against resident (K, V); MODE 1 the other way round
                const unsigned a_s = MODE == 0 ? y0 : x0, b_s = MODE == 0 ? x0 : y0, a_p = MODE == 0 ? y1 : x1, b_p = MODE == 0 ? x1 : y1;
#pragma unroll
                for (int ks = 0; ks < HD / 16; ++ks)
                    tc_mma(tmem_base + kColS, make_desc(a_s + ks * 32, 16, 1024), make_desc(b_s + ks * 32, 16, 1024), idesc_sd, ks > 0 ? 1u : 0u);
#pragma unroll
                for (int ks = 0; ks < HD / 16; ++ks)
                    tc_mma(tmem_base + kColDP, make_desc(a_p + ks * 32, 16, 1024), make_desc(b_p + ks * 32, 16, 1024), idesc_sd, ks > 0 ? 1u : 0u);
                tc_commit(sd_full);
            };
            Job jb, nx;
            bool have = job_at<MODE>(args, 0, jb);
            bool ok = true;
            unsigned g = 0; // global step counter
            if (have) {
                ok = mbar_wait(x_full, 0, abort_flag, args.err);
                if (ok) ok = mbar_wait(&y_full[0], 0, abort_flag, args.err);
                if (ok) {
                    tc_fence_after();
                    issue_sd(0);
                    if (jb.nt == 1) tc_commit(x_empty); // the job's last S / dP has been issued: the resident pair is free once it has run
                }
            }
            for (int it = 0; ok && have; ++it) {
                const bool have_next = job_at<MODE>(args, it + 1, nx);
                // accumulators of this job: MODE 0 dV | dK, MODE 1 dQ; two sets of TMEM columns, alternating from job to job
                const unsigned acc_a = MODE == 0 ? kColAcc0 + (unsigned)(it & 1) * 128u : ((it & 1) ? kColAccAlt1 : kColAcc0);
                const unsigned acc_b = acc_a + 64u;
                for (int t = 0; t < jb.nt && ok; ++t, ++g) {
                    const unsigned st = g & 1u;
                    if (t + 1 < jb.nt) {
                        // next scores of this job as soon as their streamed pair is here and the rows have read the current ones
                        ok = mbar_wait(&y_full[(g + 1) & 1u], ((g + 1) >> 1) & 1u, abort_flag, args.err);
                        if (ok) ok = mbar_wait(sd_free, g & 1u, abort_flag, args.err);
                        if (!ok) break;
                        tc_fence_after();
                        issue_sd(g + 1);
                        if (t + 2 == jb.nt) tc_commit(x_empty);
                    }
                    ok = mbar_wait(pds_full, g & 1u, abort_flag, args.err);
                    if (!ok) break;
                    tc_fence_after();
                    const unsigned y0 = smem_u32(smem + kSmemY + st * 2 * kTileBytes), y1 = y0 + kTileBytes;
                    const unsigned acc = (t > 0) ? 1u : 0u;
                    const bool spill = MODE == 0 && args.ds_out != nullptr;
                    if (spill) { // dS of this pair to the scratch of the dQ kernel, while the MMAs below read the same tile
                        const size_t slot = ((size_t)jb.nh * tiles + (size_t)(jb.t_first + t)) * tiles + (size_t)jb.own;
                        bulk_store(args.ds_out + slot * kDsBytes, sDS, kDsBytes);
                        bulk_commit();
                    }
                    if (MODE == 0) {
                        // dV += P^T dO, dK += dS^T Q: A is MN-major over [key block (16 KB)][query block (8 KB)] atoms,
                        // 16 queries per step = 2048 bytes inside a query block; B = dO / Q as loaded ([queries, hd]: MN-major)
#pragma unroll
                        for (int ks = 0; ks < BT / 16; ++ks) {
                            const unsigned a_off = (ks >> 2) * 8192 + (ks & 3) * 2048;
                            tc_mma(tmem_base + acc_a, make_desc(p_addr + a_off, 16384, 1024), make_desc(y1 + ks * 2048, 8192, 1024), idesc_acc,
                                   (ks > 0) ? 1u : acc);
                        }
#pragma unroll
                        for (int ks = 0; ks < BT / 16; ++ks) {
                            const unsigned a_off = (ks >> 2) * 8192 + (ks & 3) * 2048;
                            tc_mma(tmem_base + acc_b, make_desc(ds_addr + a_off, 16384, 1024), make_desc(y0 + ks * 2048, 8192, 1024), idesc_acc,
                                   (ks > 0) ? 1u : acc);
                        }
                    } else {
                        // dQ += dS K: A = dS straight from TMEM (16 keys = 8 columns of packed pairs per step);
                        // B = K as loaded ([keys, hd]: MN-major), 16 keys = 2048 bytes
#pragma unroll
                        for (int ks = 0; ks < BT / 16; ++ks)
                            tc_mma_ta(tmem_base + acc_a, tmem_base + kColDSt + ks * 8, make_desc(y0 + ks * 2048, 8192, 1024), idesc_acc,
                                      (ks > 0) ? 1u : acc);
                    }
                    if (spill) bulk_wait_read0(); // mma_done also tells the rows that dS may be overwritten
                    tc_commit(mma_done);
                    tc_commit(&y_empty[st]);
                    if (t + 1 == jb.nt && have_next) {
                        // first scores of the NEXT job, queued behind this job's last accumulating MMAs: they run while the
                        // rows write this job's results out
                        ok = mbar_wait(x_full, (unsigned)(it + 1) & 1u, abort_flag, args.err);
                        if (ok) ok = mbar_wait(&y_full[(g + 1) & 1u], ((g + 1) >> 1) & 1u, abort_flag, args.err);
                        if (ok) ok = mbar_wait(sd_free, g & 1u, abort_flag, args.err);
                        if (!ok) break;
                        tc_fence_after();
                        issue_sd(g + 1);
                        if (nx.nt == 1) tc_commit(x_empty);
                    }
                }
                jb = nx;
                have = have_next;
            }
            if (MODE == 0 && args.ds_out) bulk_wait_all();
        }
    } else {
        // ------------------------------------------------------------ pair arithmetic and epilogue (warps 2..9)
        const int wq = warp & 3;                 // TMEM lane quarter
        const int hh = (warp - 2) >> 2;          // which 64 keys of the row this thread takes
        const int row_local = wq * 32 + lane;    // query inside the tile = TMEM lane
        const unsigned lane_addr = ((unsigned)(wq * 32) << 16);
        bool ok = true;
        unsigned g = 0; // global step counter
        Job jb;
        for (int it = 0; ok && job_at<MODE>(args, it, jb); ++it) {
            const int n = jb.n, h = jb.h, own = jb.own, o0 = jb.o0, nt = jb.nt;
            const long long stat_base = ((long long)n * args.heads + h) * args.seq;
            float lse2 = INFINITY, dl = 0.0f;
            if (MODE == 1) {
                const int qrow = o0 + row_local;
                if (qrow < args.seq) {
                    lse2 = args.lse[stat_base + qrow] * 1.4426950408889634f;
                    dl = args.delta[stat_base + qrow];
                }
            }
            for (int t = 0; t < nt && ok; ++t, ++g) {
                const int q0 = (MODE == 0) ? (jb.t_first + t) * BT : o0;  // first query of this pair
                const int k0 = (MODE == 0) ? o0 : t * BT;                 // first key of this pair
                const int qrow = q0 + row_local;
                if (MODE == 0) {
                    lse2 = INFINITY;
                    dl = 0.0f;
                    if (qrow < args.seq) {
                        lse2 = args.lse[stat_base + qrow] * 1.4426950408889634f;
                        dl = args.delta[stat_base + qrow];
                    }
                }
                ok = mbar_wait(sd_full, g & 1u, abort_flag, args.err);
                if (!ok) break;
                tc_fence_after();
                unsigned s[64], d[64];
                tmem_ld32(tmem_base + lane_addr + kColS + hh * 64, *reinterpret_cast<unsigned(*)[32]>(&s[0]));
                tmem_ld32(tmem_base + lane_addr + kColS + hh * 64 + 32, *reinterpret_cast<unsigned(*)[32]>(&s[32]));
                tmem_ld32(tmem_base + lane_addr + kColDP + hh * 64, *reinterpret_cast<unsigned(*)[32]>(&d[0]));
                tmem_ld32(tmem_base + lane_addr + kColDP + hh * 64 + 32, *reinterpret_cast<unsigned(*)[32]>(&d[32]));
                tmem_ld_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(sd_free);
                const bool masked = (args.causal && (k0 + BT - 1 > q0)) || (k0 + BT > args.seq);
                if (masked) {
#pragma unroll
                    for (int e = 0; e < 64; ++e) {
                        int col = k0 + hh * 64 + e;
                        if (col >= args.seq || (args.causal && col > qrow)) s[e] = 0xff800000u; // exp2(-inf) = 0
                    }
                }
                const float neg_l = -lse2; // +inf for rows past the end: p = 0 there
#pragma unroll
                for (int e = 0; e < 64; e += 2) {
                    float p0 = fast_exp2(fmaf(__uint_as_float(s[e]), args.scale_log2, neg_l));
                    float p1 = fast_exp2(fmaf(__uint_as_float(s[e + 1]), args.scale_log2, neg_l));
                    float g0 = p0 * (__uint_as_float(d[e]) - dl), g1 = p1 * (__uint_as_float(d[e + 1]) - dl);
                    s[e >> 1] = pack16<F16>(p0, p1);   // packed pairs fill the front of the same registers
                    d[e >> 1] = pack16<F16>(g0, g1);
                }
                if (g > 0) { // the previous pair's MMAs (of this job or the one before) may still be reading P / dS
                    ok = mbar_wait(mma_done, (g - 1) & 1u, abort_flag, args.err);
                    if (!ok) break;
                    tc_fence_after();
                }
                if (MODE == 1) {
                    // dS into TMEM: this row's lane, columns of this thread's 64 keys
                    tmem_st32(tmem_base + lane_addr + kColDSt + hh * 32, *reinterpret_cast<unsigned(*)[32]>(&d[0]));
                    tmem_st_wait();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(pds_full);
                    continue;
                }
                // atom [key block hh][query block row>>6]: row (row & 63) of 128 bytes, 16-byte chunk c at (c ^ (row & 7))
                const unsigned atom = (unsigned)hh * 16384u + (unsigned)(row_local >> 6) * 8192u + (unsigned)(row_local & 63) * 128u;
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    const unsigned off = atom + (unsigned)((c ^ (row_local & 7)) << 4);
                    if (MODE == 0) *(uint4 *)(sP + off) = make_uint4(s[c * 4], s[c * 4 + 1], s[c * 4 + 2], s[c * 4 + 3]);
                    *(uint4 *)(sDS + off) = make_uint4(d[c * 4], d[c * 4 + 1], d[c * 4 + 2], d[c * 4 + 3]);
                }
                fence_async_smem();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(pds_full);
            }
            if (!ok) break;
            // ---- epilogue of the job: accumulators as bf16 through shared memory and TMA
            ok = mbar_wait(mma_done, (g - 1) & 1u, abort_flag, args.err);
            if (!ok) break;
            if (MODE == 0 || hh == 0) {
                tc_fence_after();
                // MODE 0: warps with hh = 0 write dV (first accumulator), hh = 1 write dK (second, times 1/sqrt(hd)); MODE 1: dQ (scaled)
                const unsigned acc_a = MODE == 0 ? kColAcc0 + (unsigned)(it & 1) * 128u : ((it & 1) ? kColAccAlt1 : kColAcc0);
                const unsigned col = (MODE == 0 && hh == 1) ? acc_a + 64u : acc_a;
                const float f = (MODE == 0 && hh == 0) ? 1.0f : args.scale;
                const CUtensorMap *om = (MODE == 0 && hh == 1) ? &map_out1 : &map_out0;
                unsigned char *stage = sP + (warp - 2) * 4096; // this warp's [32 rows x 128 bytes] box (P is no longer read)
#pragma unroll 1
                for (int c = 0; c < HD / 32; ++c) {
                    unsigned o[32];
                    tmem_ld32(tmem_base + lane_addr + col + c * 32, o);
                    tmem_ld_wait();
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        uint4 piece;
                        piece.x = pack16<F16>(__uint_as_float(o[q * 8]) * f, __uint_as_float(o[q * 8 + 1]) * f);
                        piece.y = pack16<F16>(__uint_as_float(o[q * 8 + 2]) * f, __uint_as_float(o[q * 8 + 3]) * f);
                        piece.z = pack16<F16>(__uint_as_float(o[q * 8 + 4]) * f, __uint_as_float(o[q * 8 + 5]) * f);
                        piece.w = pack16<F16>(__uint_as_float(o[q * 8 + 6]) * f, __uint_as_float(o[q * 8 + 7]) * f);
                        int chunk = c * 4 + q;
                        *(uint4 *)(stage + lane * 128 + ((chunk ^ (lane & 7)) << 4)) = piece;
                    }
                }
                fence_async_smem();
                __syncwarp();
                if (args.bias_partial) {
                    // lane l sums columns 2l, 2l+1 of this warp's 32 staged rows (the rounded values; rows past the sequence end excluded)
                    float c0 = 0.0f, c1 = 0.0f;
                    const int rows_live = min(32, args.seq - (o0 + wq * 32));
                    for (int rr = 0; rr < rows_live; ++rr) {
                        const unsigned w2 = *(const unsigned *)(stage + rr * 128 + (((lane >> 2) ^ (rr & 7)) << 4) + (lane & 3) * 4);
                        if (F16) {
                            const float2 pr = __half22float2(*reinterpret_cast<const __half2 *>(&w2));
                            c0 += pr.x;
                            c1 += pr.y;
                        } else {
                            c0 += __uint_as_float(w2 << 16);
                            c1 += __uint_as_float(w2 & 0xFFFF0000u);
                        }
                    }
                    const int which = MODE == 1 ? 0 : (hh == 1 ? 1 : 2); // dq, dk, dv column block of the packed gradient
                    float *dst = args.bias_partial + ((size_t)(n * tiles + own) * 4 + wq) * args.bias_ld + which * args.dim + h * HD + 2 * lane;
                    *(float2 *)dst = make_float2(c0, c1);
                }
                if (lane == 0 && o0 + wq * 32 < args.seq) {
                    tma_store_3d(om, stage, h * HD, o0 + wq * 32, n);
                    bulk_commit();
                    bulk_wait_read0(); // the staging tile has been read; the write itself completes before the grid does
                }
                __syncwarp();
            }
            // the staging boxes lie in the P tile: no row may write the next job's P before every warp's box has been read
            __syncwarp();
            if (lane == 0) mbar_arrive(epi_done);
            ok = mbar_wait(epi_done, (unsigned)it & 1u, abort_flag, args.err);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
    if (MODE == 1) dep_wait();
}

// ------------------------------------------------------------------ dQ from the dS tiles of the dK/dV kernel
// One CTA per (128-query tile, sample, head), two per SM.  Per key tile: one 32 KB bulk copy of dS (two [128 queries x 64
// keys] K-major tiles with the 128-byte swizzle, exactly as the dK/dV kernel's rows wrote them) and the K tile, then
// dQ += dS K as eight M=128 N=64 K=16 MMAs into 64 TMEM columns.  Roles (192 threads): warp 0 copies, warp 1 MMAs,
// warps 2..5 the epilogue (scale, round, TMA store, column sums for the q bias gradient).  Every wait is bounded.
constexpr int kDqThreads = 192;
constexpr int kDqStages = 2;
constexpr int kDqStageBytes = kDsBytes + kTileBytes; // 48 KB
constexpr int kDqSmemOut = kDqStages * kDqStageBytes, kDqSmemBar = kDqSmemOut + 4 * 4096;
constexpr int kDqSmemBytes = kDqSmemBar + 128 + 768;
static_assert(2 * (kDqSmemBytes + 1024) <= 228 * 1024, "two CTAs per SM");

struct DqArgs {
    const unsigned char *ds;
    int seq, heads, causal;
    float scale;
    unsigned int *err;
    float *bias_partial;
    int bias_ld, dim;
};

template <bool F16>
__global__ void __launch_bounds__(kDqThreads, 2)
flash_tc_dq_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_dq, DqArgs args) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char *smem = (unsigned char *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned long long *bars = (unsigned long long *)(smem + kDqSmemBar);
    unsigned long long *full = bars, *empty = bars + kDqStages, *acc_done = bars + 2 * kDqStages;
    unsigned *tmem_slot = (unsigned *)(acc_done + 1);
    volatile int *abort_flag = (volatile int *)(tmem_slot + 1);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int lin = (int)(blockIdx.y * gridDim.x + blockIdx.x), rank = lin / (int)gridDim.y, nh = lin - rank * (int)gridDim.y;
    const int n = nh / args.heads, h = nh % args.heads;
    const int tiles = (args.seq + BT - 1) / BT;
    const int own = args.causal ? (int)gridDim.x - 1 - rank : rank; // late query tiles walk the most key tiles: first
    const int nt = args.causal ? own + 1 : tiles;
    const int o0 = own * BT;
    if ((uintptr_t)(smem + kDqSmemBar + 128) > (uintptr_t)smem_raw + kDqSmemBytes) { // the dynamic segment started less aligned than assumed
        if (threadIdx.x == 0) atomicOr(args.err, MCB_DEVERR_TIMEOUT);
        return;
    }
    if (threadIdx.x == 0) {
        prefetch_map(&map_k);
        prefetch_map(&map_dq);
        for (int s = 0; s < kDqStages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        mbar_init(acc_done, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, 64);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem_base = *tmem_slot;
    dep_wait(); // the dS tiles come from the kernel before this one
    dep_trigger();

    if (warp == 0) {
        if (lane == 0) {
            const unsigned char *src = args.ds + ((size_t)nh * tiles + (size_t)own) * tiles * kDsBytes;
            bool ok = true;
            for (int t = 0; t < nt && ok; ++t) {
                const int st = t % kDqStages;
                ok = mbar_wait(&empty[st], ((unsigned)(t / kDqStages) & 1u) ^ 1u, abort_flag, args.err);
                if (!ok) break;
                unsigned char *sd = smem + st * kDqStageBytes;
                mbar_expect_tx(&full[st], kDqStageBytes);
                bulk_load(sd, src + (size_t)t * kDsBytes, kDsBytes, &full[st]);
                tma_load_3d(sd + kDsBytes, &map_k, &full[st], h * HD, t * BT, n);
            }
            for (int st = 0; st < kDqStages && ok; ++st) { // drain: nothing is still landing in shared memory at exit
                const int fills = (nt > st) ? ((nt - 1 - st) / kDqStages + 1) : 0;
                if (fills) ok = mbar_wait(&empty[st], (unsigned)(fills - 1) & 1u, abort_flag, args.err);
            }
            if (*abort_flag) {
                unsigned long long t0 = global_ns();
                while (global_ns() - t0 < 200000ull) {
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr unsigned idesc = make_idesc(BT, HD, 0, 1, F16); // A = dS (K-major), B = K as loaded ([keys, hd]: MN-major)
            bool ok = true;
            for (int t = 0; t < nt && ok; ++t) {
                const int st = t % kDqStages;
                ok = mbar_wait(&full[st], (unsigned)(t / kDqStages) & 1u, abort_flag, args.err);
                if (!ok) break;
                tc_fence_after();
                const unsigned ds_addr = smem_u32(smem + st * kDqStageBytes), k_addr = ds_addr + kDsBytes;
#pragma unroll
                for (int ks = 0; ks < BT / 16; ++ks) // 16 keys per step: 32 bytes inside a 64-key block of 16 KB
                    tc_mma(tmem_base, make_desc(ds_addr + (ks >> 2) * 16384 + (ks & 3) * 32, 16, 1024), make_desc(k_addr + ks * 2048, 8192, 1024), idesc,
                           (t > 0 || ks > 0) ? 1u : 0u);
                tc_commit(&empty[st]);
            }
            if (ok) tc_commit(acc_done);
        }
    } else {
        const int wq = warp & 3;
        const unsigned lane_addr = ((unsigned)(wq * 32) << 16);
        bool ok = nt > 0 ? mbar_wait(acc_done, 0, abort_flag, args.err) : true;
        if (ok) {
            tc_fence_after();
            unsigned char *stage = smem + kDqSmemOut + wq * 4096; // this warp's [32 rows x 128 bytes] box
#pragma unroll 1
            for (int c = 0; c < HD / 32; ++c) {
                unsigned o[32];
                if (nt > 0) {
                    tmem_ld32(tmem_base + lane_addr + c * 32, o);
                    tmem_ld_wait();
                } else {
#pragma unroll
                    for (int e = 0; e < 32; ++e) o[e] = 0u;
                }
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    uint4 piece;
                    piece.x = pack16<F16>(__uint_as_float(o[q * 8]) * args.scale, __uint_as_float(o[q * 8 + 1]) * args.scale);
                    piece.y = pack16<F16>(__uint_as_float(o[q * 8 + 2]) * args.scale, __uint_as_float(o[q * 8 + 3]) * args.scale);
                    piece.z = pack16<F16>(__uint_as_float(o[q * 8 + 4]) * args.scale, __uint_as_float(o[q * 8 + 5]) * args.scale);
                    piece.w = pack16<F16>(__uint_as_float(o[q * 8 + 6]) * args.scale, __uint_as_float(o[q * 8 + 7]) * args.scale);
                    const int chunk = c * 4 + q;
                    *(uint4 *)(stage + lane * 128 + ((chunk ^ (lane & 7)) << 4)) = piece;
                }
            }
            fence_async_smem();
            __syncwarp();
            if (args.bias_partial) { // lane l sums columns 2l, 2l+1 of this warp's 32 staged rows (the rounded values)
                float c0 = 0.0f, c1 = 0.0f;
                const int rows_live = min(32, args.seq - (o0 + wq * 32));
                for (int rr = 0; rr < rows_live; ++rr) {
                    const unsigned w2 = *(const unsigned *)(stage + rr * 128 + (((lane >> 2) ^ (rr & 7)) << 4) + (lane & 3) * 4);
                    if (F16) {
                        const float2 pr = __half22float2(*reinterpret_cast<const __half2 *>(&w2));
                        c0 += pr.x;
                        c1 += pr.y;
                    } else {
                        c0 += __uint_as_float(w2 << 16);
                        c1 += __uint_as_float(w2 & 0xFFFF0000u);
                    }
                }
                float *dst = args.bias_partial + ((size_t)(n * tiles + own) * 4 + wq) * args.bias_ld + h * HD + 2 * lane;
                *(float2 *)dst = make_float2(c0, c1);
            }
            if (lane == 0 && o0 + wq * 32 < args.seq) {
                tma_store_3d(&map_dq, stage, h * HD, o0 + wq * 32, n);
                bulk_commit();
                bulk_wait_read0();
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, 64);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);
EncodeTiledFn get_encode() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void *p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess && qres == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

// [n][seq][cols] bf16 view with row pitch `ld` elements; boxes of {64 columns, box_rows rows, 1 sample}
mcb_status make_map3(mcb_ctx *ctx, CUtensorMap *map, const void *base, long long cols, long long seq, long long n, long long ld, int box_rows, bool f16) {
    EncodeTiledFn enc = get_encode();
    if (!enc) return mcb_fail(ctx, MCB_BACKEND, "cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)seq, (cuuint64_t)n};
    cuuint64_t strides[2] = {(cuuint64_t)ld * 2, (cuuint64_t)ld * 2 * (cuuint64_t)seq};
    cuuint32_t box[3] = {64u, (cuuint32_t)box_rows, 1u};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = enc(map, f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return mcb_fail(ctx, MCB_BACKEND, "cuTensorMapEncodeTiled (attention backward) failed with %d", (int)r);
    return MCB_OK;
}

} // namespace

// dq, dk, dv from q, k, v, dO and the forward's log-sum-exp; `delta` = rowsum(O * dO) per (sample, head, row).
// MCB_UNSUPPORTED (nothing launched) outside the kernel's range.
mcb_status mcb_flash_tc_backward(mcb_ctx *ctx, const void *q, const void *k, const void *v, const void *gout, const float *lse, const float *delta,
                                 void *dq, void *dk, void *dv, int64_t n, int64_t seq, int64_t dim, int64_t heads, int32_t causal, int64_t ldi,
                                 int64_t ldo, int64_t ldg, float *bias_partial, int64_t bias_ld, int32_t dt) {
    if (!mcb_is_lp(dt)) return MCB_UNSUPPORTED;
    const bool f16 = dt == MCB_F16;
    if (heads <= 0 || dim != heads * HD || ldi % 8 || ldo % 8 || ldg % 8 || n * heads > 65535) return MCB_UNSUPPORTED;
    if (!mcb_aligned16(q) || !mcb_aligned16(k) || !mcb_aligned16(v) || !mcb_aligned16(gout) || !mcb_aligned16(dq) || !mcb_aligned16(dk) ||
        !mcb_aligned16(dv))
        return MCB_UNSUPPORTED;
    if (n == 0 || seq == 0) return MCB_OK;
    CUtensorMap mq, mk, mv, mdo, mdq, mdk, mdv;
    MCB_TRY(make_map3(ctx, &mq, q, dim, seq, n, ldi, BT, f16));
    MCB_TRY(make_map3(ctx, &mk, k, dim, seq, n, ldi, BT, f16));
    MCB_TRY(make_map3(ctx, &mv, v, dim, seq, n, ldi, BT, f16));
    MCB_TRY(make_map3(ctx, &mdo, gout, dim, seq, n, ldo, BT, f16));
    MCB_TRY(make_map3(ctx, &mdq, dq, dim, seq, n, ldg, 32, f16));
    MCB_TRY(make_map3(ctx, &mdk, dk, dim, seq, n, ldg, 32, f16));
    MCB_TRY(make_map3(ctx, &mdv, dv, dim, seq, n, ldg, 32, f16));
    BwdArgs a;
    a.lse = lse;
    a.delta = delta;
    a.seq = (int)seq;
    a.heads = (int)heads;
    a.causal = causal;
    a.tiles = (int)((seq + BT - 1) / BT);
    a.nh_total = (int)(n * heads);
    a.jobs = a.tiles * a.nh_total;
    a.scale = 1.0f / sqrtf((float)HD);
    a.scale_log2 = a.scale * 1.4426950408889634f;
    a.err = ctx->d_err;
    a.bias_partial = bias_partial;
    a.bias_ld = (int)bias_ld;
    a.dim = (int)dim;
    a.ds_out = nullptr;
    // dQ from the dS tiles the dK/dV kernel leaves (32 KB per pair of tiles), unless that scratch would pass 1 GiB
    const long long tiles = (seq + BT - 1) / BT;
    const size_t ds_bytes = (size_t)n * heads * tiles * tiles * kDsBytes;
    void *ds = nullptr;
    if (!knob_on(ctx, K_FLASH_DQ_RECOMPUTE) && ds_bytes <= ((size_t)1 << 30)) {
        MCB_TRY(mcb_alloc(ctx, ds_bytes, &ds));
        a.ds_out = (unsigned char *)ds;
    }
    static bool attr_set = false;
    if (!attr_set) {
        MCB_CUDA(ctx, cudaFuncSetAttribute(flash_tc_bwd_kernel<0, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
        MCB_CUDA(ctx, cudaFuncSetAttribute(flash_tc_bwd_kernel<1, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
        MCB_CUDA(ctx, cudaFuncSetAttribute(flash_tc_bwd_kernel<0, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
        MCB_CUDA(ctx, cudaFuncSetAttribute(flash_tc_bwd_kernel<1, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
        MCB_CUDA(ctx, cudaFuncSetAttribute(flash_tc_dq_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kDqSmemBytes));
        MCB_CUDA(ctx, cudaFuncSetAttribute(flash_tc_dq_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kDqSmemBytes));
        attr_set = true;
    }
    const dim3 grid((unsigned)tiles, (unsigned)(n * heads));              // one CTA per job (the dQ-from-dS kernel)
    // persistent CTAs for the tile-pair kernels; MCB_FLASH_BWD_ONE_JOB (test knob) gives every job a CTA of its own
    const dim3 pgrid((unsigned)((a.jobs < ctx->sm_count || knob_on(ctx, K_FLASH_BWD_ONE_JOB)) ? a.jobs : ctx->sm_count));
    cudaError_t e;
    if (f16) e = mcb_launch_dep(ctx, flash_tc_bwd_kernel<0, true>, pgrid, dim3(kThreads), kSmemBytes, mq, mk, mv, mdo, mdv, mdk, a);
    else e = mcb_launch_dep(ctx, flash_tc_bwd_kernel<0, false>, pgrid, dim3(kThreads), kSmemBytes, mq, mk, mv, mdo, mdv, mdk, a);
    if (e == cudaSuccess) {
        ctx->launches++;
        if (ds) {
            DqArgs d;
            d.ds = (const unsigned char *)ds;
            d.seq = (int)seq;
            d.heads = (int)heads;
            d.causal = causal;
            d.scale = a.scale;
            d.err = ctx->d_err;
            d.bias_partial = bias_partial;
            d.bias_ld = (int)bias_ld;
            d.dim = (int)dim;
            if (f16) e = mcb_launch_dep(ctx, flash_tc_dq_kernel<true>, grid, dim3(kDqThreads), kDqSmemBytes, mk, mdq, d);
            else e = mcb_launch_dep(ctx, flash_tc_dq_kernel<false>, grid, dim3(kDqThreads), kDqSmemBytes, mk, mdq, d);
        } else {
            if (f16) e = mcb_launch_dep(ctx, flash_tc_bwd_kernel<1, true>, pgrid, dim3(kThreads), kSmemBytes, mq, mk, mv, mdo, mdq, mdq, a);
            else e = mcb_launch_dep(ctx, flash_tc_bwd_kernel<1, false>, pgrid, dim3(kThreads), kSmemBytes, mq, mk, mv, mdo, mdq, mdq, a);
        }
    }
    if (ds) mcb_free(ctx, ds); // stream-ordered reuse: whoever gets the block next is enqueued behind the dQ kernel
    MCB_CUDA(ctx, e);
    MCB_LAUNCHED(ctx);
    return MCB_OK;
}

int64_t mcb_flash_bias_rows(int64_t n, int64_t seq) { return n * ((seq + BT - 1) / BT) * 4; }
