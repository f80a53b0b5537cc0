// Fused attention forward on the tcgen05 tensor cores (bf16, head_dim 64).
//
// One CTA per (128-query tile, sample, head); it walks the key/value tiles of 128 keys that the
// tile may see (all of them, or up to the diagonal when causal):
//   S = Q K^T      tcgen05.mma  M=128 N=128 K=64, A = Q tile, B = K tile (both K-major in smem), D in TMEM
//   P = softmax    one thread per query row reads its row of S from TMEM (tcgen05.ld), keeps a
//                  running maximum m and sum l in the log2 domain, writes P as packed bf16 back into
//                  TMEM (tcgen05.st)
//   O += P V       tcgen05.mma  M=128 N=64 K=128, A = P from TMEM, B = V tile as loaded ([keys, 64]: MN-major)
// O stays in TMEM for the whole walk.  When a row's maximum grows it is NOT followed at once: the
// reference maximum is only moved (and O, l rescaled) when it lags by more than 8 in the log2 domain,
// so the probabilities stay below 2^8 and the rescale of O, a TMEM round trip, is rare.
// Roles (192 threads): warp 0 issues the TMA copies (Q once, K/V through a two-stage ring), warp 1
// allocates TMEM and issues the MMAs, warps 2..5 are the softmax rows and the epilogue (O / l as
// bf16 through shared memory and TMA, log-sum-exp per row for the backward pass).  The next S = Q K^T
// is issued as soon as the softmax rows have read the previous S, so it overlaps the exponentials.
// Two CTAs fit on an SM (about 97 KB of shared memory and 256 TMEM columns each).
// Every mbarrier wait is bounded; on expiry the CTA raises the device error word and drains.
#include "internal.h"
#include "tc_ptx.cuh"

using namespace tcptx;

namespace {

constexpr int HD = 64;    // head dimension
constexpr int BM = 128;   // queries per CTA
constexpr int BN = 128;   // keys per tile
constexpr int kThreads = 192;
constexpr int kTileBytes = 128 * 64 * 2; // a [128 x 64] bf16 tile: 16 KB
constexpr int kStages = 2;
// shared memory: Q | K0 V0 | K1 V1 | output staging (16 KB) | barriers.  P never touches shared memory: it goes from
// the softmax registers into TMEM and is the A operand of P V from there.
constexpr int kSmemQ = 0, kSmemKV = kTileBytes, kSmemP = kSmemKV + kStages * 2 * kTileBytes, kSmemBar = kSmemP + kTileBytes;
// Two CTAs must fit in the SM's 228 KB (each also pays 1 KB of system reservation): 115,712 bytes at most.
// The alignment slack is therefore 768 bytes, not 1024; the kernel checks that the aligned carve-up fits.
constexpr int kSmemBytes = kSmemBar + 128 + 768;
static_assert(2 * (kSmemBytes + 1024) <= 228 * 1024, "two CTAs per SM");
constexpr unsigned kTmemCols = 256; // S: columns [0,128), O: [128,192), P as packed bf16 pairs: [192,256)
constexpr unsigned kColS = 0, kColO = 128, kColP = 192;

struct FwdArgs {
    float *lse;        // [n, heads, seq]
    int seq, heads, causal;
    float scale_log2;  // 1/sqrt(hd) * log2(e)
    unsigned int *err;
};

template <bool F16>
__global__ void __launch_bounds__(kThreads, 2)
flash_tc_fwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                    const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_o, FwdArgs args) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char *smem = (unsigned char *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char *sQ = smem + kSmemQ, *sP = smem + kSmemP;
    unsigned long long *bars = (unsigned long long *)(smem + kSmemBar);
    // K and V have separate rings: a K tile is free again as soon as its Q K^T has run, long before the
    // P V of the same step, so the next K tile is on its way while the softmax of the current one runs
    unsigned long long *q_full = bars, *k_full = bars + 1, *k_empty = bars + 3, *v_full = bars + 5, *v_empty = bars + 7, *s_full = bars + 9,
                       *s_free = bars + 10, *p_full = bars + 11, *pv_done = bars + 12;
    unsigned *tmem_slot = (unsigned *)(bars + 13);
    volatile int *abort_flag = (volatile int *)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // causal: late query tiles walk the most key tiles, so they are scheduled first
    // (CTAs are dispatched in the order of their linear index, read here as (weight rank, sample*head): all the longest
    // jobs of the grid start first and the shortest fill the tail)
    const int lin = (int)(blockIdx.y * gridDim.x + blockIdx.x), rank = lin / (int)gridDim.y, nh = lin - rank * (int)gridDim.y;
    const int qt = args.causal ? (int)gridDim.x - 1 - rank : rank;
    const int n = nh / args.heads, h = nh % args.heads;
    const int q0 = qt * BM;
    const int kt_all = (args.seq + BN - 1) / BN;
    const int nt = args.causal ? min(qt + 1, kt_all) : kt_all;

    if ((uintptr_t)(smem + kSmemBar + 128) > (uintptr_t)smem_raw + kSmemBytes) { // the dynamic segment started less aligned than assumed
        if (threadIdx.x == 0) atomicOr(args.err, MCB_DEVERR_TIMEOUT);
        return;
    }
    if (threadIdx.x == 0) {
        prefetch_map(&map_q);
        prefetch_map(&map_k);
        prefetch_map(&map_v);
        prefetch_map(&map_o);
        mbar_init(q_full, 1);
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&k_full[s], 1);
            mbar_init(&k_empty[s], 1);
            mbar_init(&v_full[s], 1);
            mbar_init(&v_empty[s], 1);
        }
        mbar_init(s_full, 1);
        mbar_init(s_free, 4);
        mbar_init(p_full, 4);
        mbar_init(pv_done, 1);
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
    // only shared and tensor memory so far: this much may overlap the previous kernel of the stream
    dep_wait();
    dep_trigger();

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            mbar_expect_tx(q_full, kTileBytes);
            tma_load_3d(sQ, &map_q, q_full, h * HD, q0, n);
            bool ok = true;
            for (int j = 0; j < nt && ok; ++j) {
                const int st = j & 1;
                const unsigned ph = ((j >> 1) & 1) ^ 1u;
                unsigned char *sk = smem + kSmemKV + st * 2 * kTileBytes, *sv = sk + kTileBytes;
                ok = mbar_wait(&k_empty[st], ph, abort_flag, args.err);
                if (!ok) break;
                mbar_expect_tx(&k_full[st], kTileBytes);
                tma_load_3d(sk, &map_k, &k_full[st], h * HD, j * BN, n);
                ok = mbar_wait(&v_empty[st], ph, abort_flag, args.err);
                if (!ok) break;
                mbar_expect_tx(&v_full[st], kTileBytes);
                tma_load_3d(sv, &map_v, &v_full[st], h * HD, j * BN, n);
            }
            // drain: every stage that was filled has been consumed before this CTA can exit
            for (int st = 0; st < kStages && ok; ++st) {
                int fills = (nt > st) ? ((nt - 1 - st) / kStages + 1) : 0;
                if (fills) ok = mbar_wait(&k_empty[st], (unsigned)(fills - 1) & 1u, abort_flag, args.err);
                if (fills && ok) ok = mbar_wait(&v_empty[st], (unsigned)(fills - 1) & 1u, abort_flag, args.err);
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
            constexpr unsigned idesc_s = make_idesc(BM, BN, 0, 0, F16);   // S = Q K^T: both operands K-major
            constexpr unsigned idesc_o = make_idesc(BM, HD, 0, 1, F16);   // O += P V: V is [keys, hd] = MN-major B
            const unsigned tmem_s = tmem_base + kColS, tmem_o = tmem_base + kColO;
            const unsigned a_q = smem_u32(sQ);
            bool ok = mbar_wait(q_full, 0, abort_flag, args.err);
            auto issue_s = [&](int j) {
                const unsigned b_k = smem_u32(smem + kSmemKV + (j & 1) * 2 * kTileBytes);
#pragma unroll
                for (int ks = 0; ks < HD / 16; ++ks)
                    tc_mma(tmem_s, make_desc(a_q + ks * 32, 16, 1024), make_desc(b_k + ks * 32, 16, 1024), idesc_s, ks > 0 ? 1u : 0u);
                tc_commit(s_full);
                tc_commit(&k_empty[j & 1]);
            };
            if (ok) ok = mbar_wait(&k_full[0], 0, abort_flag, args.err);
            if (ok) {
                tc_fence_after();
                issue_s(0);
            }
            for (int j = 0; j < nt && ok; ++j) {
                const int st = j & 1;
                if (j + 1 < nt) {
                    // next scores as soon as their K tile is here and the rows have read the current S
                    ok = mbar_wait(&k_full[(j + 1) & 1], ((j + 1) >> 1) & 1u, abort_flag, args.err);
                    if (ok) ok = mbar_wait(s_free, (unsigned)j & 1u, abort_flag, args.err);
                    if (!ok) break;
                    tc_fence_after();
                    issue_s(j + 1);
                }
                ok = mbar_wait(&v_full[st], (unsigned)(j >> 1) & 1u, abort_flag, args.err);
                if (ok) ok = mbar_wait(p_full, (unsigned)j & 1u, abort_flag, args.err);
                if (!ok) break;
                tc_fence_after();
                const unsigned b_v = smem_u32(smem + kSmemKV + st * 2 * kTileBytes + kTileBytes);
#pragma unroll
                for (int ks = 0; ks < BN / 16; ++ks) {
                    // P from TMEM: 16 keys = 8 columns of packed pairs per step; V: 16 keys = 2048 bytes per step
                    unsigned long long bd = make_desc(b_v + ks * 2048, 8192, 1024);
                    tc_mma_ta(tmem_o, tmem_base + kColP + ks * 8, bd, idesc_o, (j > 0 || ks > 0) ? 1u : 0u);
                }
                tc_commit(pv_done);
                tc_commit(&v_empty[st]);
            }
        }
    } else {
        // ------------------------------------------------------------ softmax rows and epilogue (warps 2..5)
        const int wq = warp & 3;               // TMEM lane quarter of this warp
        const int row_local = wq * 32 + lane;  // query row inside the tile = TMEM lane
        const int row = q0 + row_local;
        const unsigned lane_addr = ((unsigned)(wq * 32) << 16);
        float m_ref = -INFINITY, l = 0.0f;
        bool ok = true;
        for (int j = 0; j < nt && ok; ++j) {
            ok = mbar_wait(s_full, (unsigned)j & 1u, abort_flag, args.err);
            if (!ok) break;
            tc_fence_after();
            const int k0 = j * BN;
            const bool masked = (args.causal && (k0 + BN - 1 > q0)) || (k0 + BN > args.seq); // diagonal tile or keys past the end
            // the whole row of S in registers with ONE wait: a TMEM round trip per 32 columns (and a second
            // pass over TMEM for the exponentials) cost more than all the arithmetic of the tile
            unsigned r[BN];
#pragma unroll
            for (int c = 0; c < BN / 32; ++c) tmem_ld32(tmem_base + lane_addr + kColS + c * 32, *reinterpret_cast<unsigned(*)[32]>(&r[c * 32]));
            tmem_ld_wait();
            // S has been read: the next Q K^T may overwrite it
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(s_free);
            if (masked) { // diagonal tile or keys past the end: masked scores become -inf (the scale is positive)
#pragma unroll
                for (int e = 0; e < BN; ++e) {
                    int col = k0 + e;
                    if (col >= args.seq || (args.causal && col > row)) r[e] = 0xff800000u;
                }
            }
            // row maximum of the raw scores, four independent chains (one chain of 128 dependent max
            // operations costs more than the exponentials); the positive scale commutes with max
            float mq[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int e = 0; e < BN; e += 4) {
                mq[0] = fmaxf(mq[0], __uint_as_float(r[e]));
                mq[1] = fmaxf(mq[1], __uint_as_float(r[e + 1]));
                mq[2] = fmaxf(mq[2], __uint_as_float(r[e + 2]));
                mq[3] = fmaxf(mq[3], __uint_as_float(r[e + 3]));
            }
            const float mx = fmaxf(fmaxf(mq[0], mq[1]), fmaxf(mq[2], mq[3])) * args.scale_log2;
            // move the reference maximum only when it lags by more than 8 (or is still -inf)
            float alpha = 1.0f;
            const bool move = mx > m_ref + 8.0f;
            if (move) {
                alpha = (m_ref == -INFINITY) ? 0.0f : fast_exp2(m_ref - mx);
                m_ref = mx;
                l *= alpha;
            }
            const bool any_move = __any_sync(0xffffffffu, move) && j > 0;
            const float neg_m = (m_ref == -INFINITY) ? 0.0f : -m_ref; // a fully masked row keeps p = 0
            float sq[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int e = 0; e < BN; e += 8) {
                float p[8];
#pragma unroll
                for (int t = 0; t < 8; ++t) p[t] = fast_exp2(fmaf(__uint_as_float(r[e + t]), args.scale_log2, neg_m));
                sq[0] += p[0] + p[1];
                sq[1] += p[2] + p[3];
                sq[2] += p[4] + p[5];
                sq[3] += p[6] + p[7];
#pragma unroll
                for (int t = 0; t < 4; ++t) r[(e >> 1) + t] = pack16<F16>(p[2 * t], p[2 * t + 1]); // packed pairs fill the front of the same registers
            }
            const float sum = (sq[0] + sq[1]) + (sq[2] + sq[3]);
            l += sum;
            // P's buffer and O are busy until the previous P V has finished
            if (j > 0) {
                ok = mbar_wait(pv_done, (unsigned)(j - 1) & 1u, abort_flag, args.err);
                if (!ok) break;
                tc_fence_after();
            }
            if (any_move) { // warp-uniform: rows whose maximum did not move multiply by exactly 1
#pragma unroll 1
                for (int c = 0; c < HD / 32; ++c) {
                    unsigned o[32];
                    tmem_ld32(tmem_base + lane_addr + kColO + c * 32, o);
                    tmem_ld_wait();
#pragma unroll
                    for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * alpha);
                    tmem_st32(tmem_base + lane_addr + kColO + c * 32, o);
                }
                tmem_st_wait();
            }
            // P into TMEM (this row's lane, 64 columns of packed bf16 pairs): the A operand of P V
            tmem_st32(tmem_base + lane_addr + kColP, *reinterpret_cast<unsigned(*)[32]>(&r[0]));
            tmem_st32(tmem_base + lane_addr + kColP + 32, *reinterpret_cast<unsigned(*)[32]>(&r[32]));
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full);
        }
        // ---- epilogue: O / l as bf16 through shared memory and TMA; log-sum-exp for the backward pass
        if (ok && nt > 0) ok = mbar_wait(pv_done, (unsigned)(nt - 1) & 1u, abort_flag, args.err);
        if (ok) {
            tc_fence_after();
            const float inv = l > 0.0f ? 1.0f / l : 0.0f;
            unsigned char *stage = sP + wq * 4096; // this warp's [32 rows x 128 bytes] box
#pragma unroll 1
            for (int c = 0; c < HD / 32; ++c) {
                unsigned o[32];
                tmem_ld32(tmem_base + lane_addr + kColO + c * 32, o);
                tmem_ld_wait();
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    uint4 piece;
                    piece.x = pack16<F16>(__uint_as_float(o[q * 8]) * inv, __uint_as_float(o[q * 8 + 1]) * inv);
                    piece.y = pack16<F16>(__uint_as_float(o[q * 8 + 2]) * inv, __uint_as_float(o[q * 8 + 3]) * inv);
                    piece.z = pack16<F16>(__uint_as_float(o[q * 8 + 4]) * inv, __uint_as_float(o[q * 8 + 5]) * inv);
                    piece.w = pack16<F16>(__uint_as_float(o[q * 8 + 6]) * inv, __uint_as_float(o[q * 8 + 7]) * inv);
                    int chunk = c * 4 + q;
                    *(uint4 *)(stage + lane * 128 + ((chunk ^ (lane & 7)) << 4)) = piece;
                }
            }
            fence_async_smem();
            __syncwarp();
            if (lane == 0 && q0 + wq * 32 < args.seq) {
                tma_store_3d(&map_o, stage, h * HD, q0 + wq * 32, n);
                bulk_commit();
                bulk_wait_read0(); // the staging tile has been read; the write itself completes before the grid does
            }
            if (row < args.seq)
                args.lse[((long long)n * args.heads + h) * args.seq + row] = (l > 0.0f) ? m_ref * 0.6931471805599453f + logf(l) : -INFINITY;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
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

// [n][seq][cols] bf16 view with row pitch `ld` elements; boxes of {64 columns, box_rows rows, 1 sample}.
// Rows past the end of a sample are zero-filled on load and dropped on store.
mcb_status make_map3(mcb_ctx *ctx, CUtensorMap *map, const void *base, long long cols, long long seq, long long n, long long ld, int box_rows, bool f16) {
    EncodeTiledFn enc = get_encode();
    if (!enc) return mcb_fail(ctx, MCB_BACKEND, "cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)seq, (cuuint64_t)n};
    cuuint64_t strides[2] = {(cuuint64_t)ld * 2, (cuuint64_t)ld * 2 * (cuuint64_t)seq};
    cuuint32_t box[3] = {64u, (cuuint32_t)box_rows, 1u};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = enc(map, f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return mcb_fail(ctx, MCB_BACKEND, "cuTensorMapEncodeTiled (attention) failed with %d", (int)r);
    return MCB_OK;
}

} // namespace

bool mcb_flash_tc_supported(int64_t dim, int64_t heads, int64_t ldi, int64_t ldo, const void *q, const void *k, const void *v, const void *out) {
    return heads > 0 && dim == heads * HD && ldi % 8 == 0 && ldo % 8 == 0 && mcb_aligned16(q) && mcb_aligned16(k) && mcb_aligned16(v) &&
           mcb_aligned16(out);
}

mcb_status mcb_flash_tc_forward(mcb_ctx *ctx, const void *q, const void *k, const void *v, void *out, float *lse, int64_t n, int64_t seq,
                                int64_t dim, int64_t heads, int32_t causal, int64_t ldi, int64_t ldo, int32_t dt) {
    if (!mcb_is_lp(dt)) return MCB_UNSUPPORTED;
    const bool f16 = dt == MCB_F16;
    if (!mcb_flash_tc_supported(dim, heads, ldi, ldo, q, k, v, out)) return MCB_UNSUPPORTED;
    if (n * heads > 65535) return MCB_UNSUPPORTED;
    if (n == 0 || seq == 0) return MCB_OK;
    CUtensorMap mq, mk, mv, mo;
    MCB_TRY(make_map3(ctx, &mq, q, dim, seq, n, ldi, BM, f16));
    MCB_TRY(make_map3(ctx, &mk, k, dim, seq, n, ldi, BN, f16));
    MCB_TRY(make_map3(ctx, &mv, v, dim, seq, n, ldi, BN, f16));
    MCB_TRY(make_map3(ctx, &mo, out, dim, seq, n, ldo, 32, f16));
    FwdArgs a;
    a.lse = lse;
    a.seq = (int)seq;
    a.heads = (int)heads;
    a.causal = causal;
    a.scale_log2 = (1.0f / sqrtf((float)HD)) * 1.4426950408889634f;
    a.err = ctx->d_err;
    static bool attr_set = false;
    if (!attr_set) {
        MCB_CUDA(ctx, cudaFuncSetAttribute(flash_tc_fwd_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
        MCB_CUDA(ctx, cudaFuncSetAttribute(flash_tc_fwd_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
        attr_set = true;
    }
    dim3 grid((unsigned)((seq + BM - 1) / BM), (unsigned)(n * heads));
    if (f16) MCB_CUDA(ctx, mcb_launch_dep(ctx, flash_tc_fwd_kernel<true>, grid, dim3(kThreads), kSmemBytes, mq, mk, mv, mo, a));
    else MCB_CUDA(ctx, mcb_launch_dep(ctx, flash_tc_fwd_kernel<false>, grid, dim3(kThreads), kSmemBytes, mq, mk, mv, mo, a));
    MCB_LAUNCHED(ctx);
    return MCB_OK;
}
