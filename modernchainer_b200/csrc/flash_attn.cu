// Fused bf16 attention for head_dim 64: forward and backward without materialising the
// [seq, seq] probability matrix.  Online softmax in f32, products on the warp-level tensor
// path (mma.sync m16n8k16 bf16 -> f32), operands staged in 128-byte-swizzled shared memory
// with cp.async double buffering.
//
// q, k, v, o, grads: [n, seq, dim] bf16 with head h in columns h*64 .. h*64+63.  Row pitches are
// separate arguments (ldi for q/k/v, ldo for o/do, ldg for dq/dk/dv), so q, k, v may be the three
// column blocks of one packed [n*seq, 3*dim] projection output and the gradients of one packed buffer.
// lse: [n, heads, seq] f32, natural-log row log-sum-exp of the scaled scores.
//
// Backward is three kernels: delta = rowsum(dO * O); dK/dV per key tile (loop over query
// tiles); dQ per query tile (loop over key tiles).  Both recompute P from q, k and lse, so no
// float atomics are needed and the result does not depend on scheduling.
#include "common.cuh"
#include "internal.h"

namespace {

typedef __nv_bfloat16 bf16;
constexpr int HD = 64;        // head dim
constexpr int TILE = 64;      // rows per tile (queries or keys)
constexpr int TILE_BYTES = TILE * HD * 2;
constexpr int kThreads = 128; // 4 warps x 16 rows

__device__ __forceinline__ unsigned smem_addr(const void *p) { return (unsigned)__cvta_generic_to_shared(p); }
// byte offset of 16-byte chunk `chunk` of row `row` inside a [64][64] bf16 tile (XOR swizzle)
__device__ __forceinline__ int swz(int row, int chunk) { return row * 128 + ((chunk ^ (row & 7)) << 4); }

__device__ __forceinline__ void cp_async16(void *smem, const void *gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr(smem)), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldsm4(unsigned (&r)[4], const unsigned char *p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(smem_addr(p)));
}
__device__ __forceinline__ void ldsm4_t(unsigned (&r)[4], const unsigned char *p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(smem_addr(p)));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack2(float x, float y) {
    __nv_bfloat162 v = __floats2bfloat162_rn(x, y);
    return *reinterpret_cast<unsigned *>(&v);
}

// loads rows [0, 64) of a head slice (row pitch `ld` elements) into a swizzled tile; rows at or
// beyond `valid` are zero-filled
__device__ __forceinline__ void load_tile(unsigned char *tile, const bf16 *g, long long ld, int valid) {
#pragma unroll
    for (int i = 0; i < (TILE * 8) / kThreads; ++i) {
        int c = threadIdx.x + i * kThreads;
        int row = c >> 3, chunk = c & 7;
        unsigned char *dst = tile + swz(row, chunk);
        if (row < valid) cp_async16(dst, g + (long long)row * ld + chunk * 8);
        else *reinterpret_cast<uint4 *>(dst) = make_uint4(0, 0, 0, 0);
    }
}

// A-operand fragments (16 rows of this warp x 64 k) from a [rows][k] tile
__device__ __forceinline__ void load_a_frags(unsigned (&f)[4][4], const unsigned char *tile, int warp, int lane) {
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) ldsm4(f[ks], tile + swz(warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1), ks * 2 + (lane >> 4)));
}

// acc[16 x 64] += A[16 x 64(k)] * B^T where the tile stores B as [n = 64][k = 64] (k contiguous)
__device__ __forceinline__ void gemm_nk(float (&acc)[8][4], const unsigned (&a)[4][4], const unsigned char *tile, int lane) {
#pragma unroll
    for (int ks = 0; ks < 4; ++ks)
#pragma unroll
        for (int np = 0; np < 4; ++np) {
            unsigned b[4];
            ldsm4(b, tile + swz(np * 16 + (lane & 7) + 8 * (lane >> 4), ks * 2 + ((lane >> 3) & 1)));
            mma16816(acc[2 * np], a[ks], b[0], b[1]);
            mma16816(acc[2 * np + 1], a[ks], b[2], b[3]);
        }
}

// acc[16 x 64(n)] += P[16 x 64(k)] * B where the tile stores B as [k = 64][n = 64] (n contiguous);
// P comes from accumulator registers p[8][4] (f32) converted on the fly
__device__ __forceinline__ void gemm_kn(float (&acc)[8][4], const float (&p)[8][4], const unsigned char *tile, int lane) {
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
        unsigned a[4];
        a[0] = pack2(p[2 * ks][0], p[2 * ks][1]);
        a[1] = pack2(p[2 * ks][2], p[2 * ks][3]);
        a[2] = pack2(p[2 * ks + 1][0], p[2 * ks + 1][1]);
        a[3] = pack2(p[2 * ks + 1][2], p[2 * ks + 1][3]);
#pragma unroll
        for (int np = 0; np < 4; ++np) {
            unsigned b[4];
            ldsm4_t(b, tile + swz(ks * 16 + (lane & 7) + 8 * ((lane >> 3) & 1), np * 2 + (lane >> 4)));
            mma16816(acc[2 * np], a, b[0], b[1]);
            mma16816(acc[2 * np + 1], a, b[2], b[3]);
        }
    }
}

__device__ __forceinline__ void zero_acc(float (&a)[8][4]) {
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) a[i][j] = 0.0f;
}

// stores a 16 x 64 f32 accumulator block of this warp as bf16 rows of a head slice
__device__ __forceinline__ void store_rows(bf16 *g, long long ld, int row0, int valid, const float (&acc)[8][4], float mul0, float mul1,
                                           int lane) {
    int gq = lane >> 2, tig = lane & 3;
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
        int col = nt * 8 + 2 * tig;
        int r0 = row0 + gq, r1 = r0 + 8;
        if (r0 < valid) *reinterpret_cast<unsigned *>(g + (long long)r0 * ld + col) = pack2(acc[nt][0] * mul0, acc[nt][1] * mul0);
        if (r1 < valid) *reinterpret_cast<unsigned *>(g + (long long)r1 * ld + col) = pack2(acc[nt][2] * mul1, acc[nt][3] * mul1);
    }
}

// 2^x on the special-function unit (about 2 ulp; the probabilities are rounded to bf16 right after)
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// ------------------------------------------------------------------ forward
template <bool CAUSAL>
__global__ void __launch_bounds__(kThreads) flash_fwd_kernel(const bf16 *__restrict__ Q, const bf16 *__restrict__ K, const bf16 *__restrict__ V,
                                                             bf16 *__restrict__ O, float *__restrict__ LSE, int S, int D, int DO, int DG, int H,
                                                             float scale_log2) {
    __shared__ __align__(128) unsigned char smem[TILE_BYTES * 5];
    unsigned char *sQ = smem, *sK[2] = {smem + TILE_BYTES, smem + 3 * TILE_BYTES}, *sV[2] = {smem + 2 * TILE_BYTES, smem + 4 * TILE_BYTES};
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gq = lane >> 2, tig = lane & 3;
    // causal: late query tiles visit the most key tiles, so they are scheduled first
    int qt = CAUSAL ? (int)(gridDim.x - 1 - blockIdx.x) : (int)blockIdx.x, n = blockIdx.y / H, h = blockIdx.y % H;
    long long base = (long long)n * S * D + (long long)h * HD;      // q, k, v (row pitch D)
    long long base_o = (long long)n * S * DO + (long long)h * HD;   // o, do (row pitch DO)
    long long base_g = (long long)n * S * DG + (long long)h * HD;   // dq, dk, dv (row pitch DG)
    (void)base_o;
    (void)base_g;
    int q0 = qt * TILE;
    int ntiles = CAUSAL ? qt + 1 : (S + TILE - 1) / TILE;
    load_tile(sQ, Q + base + (long long)q0 * D, D, S - q0);
    load_tile(sK[0], K + base, D, S);
    load_tile(sV[0], V + base, D, S);
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();
    unsigned qf[4][4];
    load_a_frags(qf, sQ, warp, lane);
    float o[8][4];
    zero_acc(o);
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};
    int row0 = q0 + warp * 16 + gq;
    for (int j = 0; j < ntiles; ++j) {
        int st = j & 1;
        if (j + 1 < ntiles) {
            int k1 = (j + 1) * TILE;
            load_tile(sK[st ^ 1], K + base + (long long)k1 * D, D, S - k1);
            load_tile(sV[st ^ 1], V + base + (long long)k1 * D, D, S - k1);
            cp_async_commit();
        }
        float s[8][4];
        zero_acc(s);
        gemm_nk(s, qf, sK[st], lane);
        bool need_mask = (CAUSAL && j == ntiles - 1) || (j + 1) * TILE > S;
#pragma unroll
        for (int nt = 0; nt < 8; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float v = s[nt][e] * scale_log2;
                if (need_mask) {
                    int col = j * TILE + nt * 8 + 2 * tig + (e & 1);
                    int row = row0 + 8 * (e >> 1);
                    if (col >= S || (CAUSAL && col > row)) v = -INFINITY;
                }
                s[nt][e] = v;
            }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            float mx = -INFINITY;
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) mx = fmaxf(mx, fmaxf(s[nt][2 * r], s[nt][2 * r + 1]));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            float mnew = fmaxf(m[r], mx);
            float msafe = (mnew == -INFINITY) ? 0.0f : mnew;
            float corr = fast_exp2(m[r] - msafe);
            float sum = 0.0f;
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
                float p0 = fast_exp2(s[nt][2 * r] - msafe), p1 = fast_exp2(s[nt][2 * r + 1] - msafe);
                s[nt][2 * r] = p0;
                s[nt][2 * r + 1] = p1;
                sum += p0 + p1;
                o[nt][2 * r] *= corr;
                o[nt][2 * r + 1] *= corr;
            }
            l[r] = l[r] * corr + sum;
            m[r] = mnew;
        }
        gemm_kn(o, s, sV[st], lane);
        if (j + 1 < ntiles) cp_async_wait<0>();
        __syncthreads();
    }
    float inv[2], lse[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        float t = l[r];
        t += __shfl_xor_sync(0xffffffffu, t, 1);
        t += __shfl_xor_sync(0xffffffffu, t, 2);
        inv[r] = t > 0.0f ? 1.0f / t : 0.0f;
        lse[r] = (t > 0.0f) ? m[r] * 0.6931471805599453f + logf(t) : -INFINITY;
    }
    store_rows(O + base_o, DO, q0 + warp * 16, S, o, inv[0], inv[1], lane);
    if (tig == 0) {
        long long lb = ((long long)n * H + h) * S;
        if (row0 < S) LSE[lb + row0] = lse[0];
        if (row0 + 8 < S) LSE[lb + row0 + 8] = lse[1];
    }
}

// ------------------------------------------------------------------ backward: delta
template <typename T>
__global__ void flash_delta_kernel(const T *__restrict__ O, const T *__restrict__ dO, float *__restrict__ delta, int S, int DO, int DG, int H,
                                   long long total_chunks) {
    // eight lanes per (sample, row, head): 16 bytes of O and of dO each, so a warp reads 512 contiguous bytes of a row
    dep_wait();
    dep_trigger();
    long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const bool live = t < total_chunks;
    if (!live) t = total_chunks - 1;
    const int per_row = H * (HD / 8);
    const long long srow = t / per_row; // n * S + row
    const int chunk = (int)(t - srow * per_row);
    const int h = chunk >> 3;
    const uint4 a = *reinterpret_cast<const uint4 *>(O + srow * DO + chunk * 8);
    const uint4 b = *reinterpret_cast<const uint4 *>(dO + srow * DG + chunk * 8);
    const uint32_t *pa = reinterpret_cast<const uint32_t *>(&a), *pb = reinterpret_cast<const uint32_t *>(&b);
    float v = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 x = Lp<T>::unpack2(pa[i]), y = Lp<T>::unpack2(pb[i]);
        v = fmaf(x.x, y.x, fmaf(x.y, y.y, v));
    }
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    v += __shfl_xor_sync(0xffffffffu, v, 2);
    v += __shfl_xor_sync(0xffffffffu, v, 4);
    if (live && (threadIdx.x & 7) == 0) {
        const long long n = srow / S, row = srow - n * S;
        delta[(n * H + h) * S + row] = v;
    }
}

// ------------------------------------------------------------------ backward: dQ
template <bool CAUSAL>
__global__ void __launch_bounds__(kThreads) flash_dq_kernel(const bf16 *__restrict__ Q, const bf16 *__restrict__ K, const bf16 *__restrict__ V,
                                                            const bf16 *__restrict__ dO, const float *__restrict__ LSE,
                                                            const float *__restrict__ DELTA, bf16 *__restrict__ dQ, int S, int D, int DO, int DG, int H,
                                                            float scale, float scale_log2) {
    __shared__ __align__(128) unsigned char smem[TILE_BYTES * 6];
    unsigned char *sQ = smem, *sdO = smem + TILE_BYTES;
    unsigned char *sK[2] = {smem + 2 * TILE_BYTES, smem + 4 * TILE_BYTES}, *sV[2] = {smem + 3 * TILE_BYTES, smem + 5 * TILE_BYTES};
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gq = lane >> 2, tig = lane & 3;
    // causal: late query tiles visit the most key tiles, so they are scheduled first
    int qt = CAUSAL ? (int)(gridDim.x - 1 - blockIdx.x) : (int)blockIdx.x, n = blockIdx.y / H, h = blockIdx.y % H;
    long long base = (long long)n * S * D + (long long)h * HD;      // q, k, v (row pitch D)
    long long base_o = (long long)n * S * DO + (long long)h * HD;   // o, do (row pitch DO)
    long long base_g = (long long)n * S * DG + (long long)h * HD;   // dq, dk, dv (row pitch DG)
    (void)base_o;
    (void)base_g;
    long long lb = ((long long)n * H + h) * S;
    int q0 = qt * TILE;
    int ntiles = CAUSAL ? qt + 1 : (S + TILE - 1) / TILE;
    load_tile(sQ, Q + base + (long long)q0 * D, D, S - q0);
    load_tile(sdO, dO + base_o + (long long)q0 * DO, DO, S - q0);
    load_tile(sK[0], K + base, D, S);
    load_tile(sV[0], V + base, D, S);
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();
    unsigned qf[4][4], dof[4][4];
    load_a_frags(qf, sQ, warp, lane);
    load_a_frags(dof, sdO, warp, lane);
    int row0 = q0 + warp * 16 + gq;
    float lse2[2], dl[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        int row = row0 + 8 * r;
        lse2[r] = row < S ? LSE[lb + row] * 1.4426950408889634f : 0.0f;
        dl[r] = row < S ? DELTA[lb + row] : 0.0f;
    }
    float dq[8][4];
    zero_acc(dq);
    for (int j = 0; j < ntiles; ++j) {
        int st = j & 1;
        if (j + 1 < ntiles) {
            int k1 = (j + 1) * TILE;
            load_tile(sK[st ^ 1], K + base + (long long)k1 * D, D, S - k1);
            load_tile(sV[st ^ 1], V + base + (long long)k1 * D, D, S - k1);
            cp_async_commit();
        }
        float s[8][4], dp[8][4];
        zero_acc(s);
        zero_acc(dp);
        gemm_nk(s, qf, sK[st], lane);
        gemm_nk(dp, dof, sV[st], lane);
        bool need_mask = (CAUSAL && j == ntiles - 1) || (j + 1) * TILE > S;
#pragma unroll
        for (int nt = 0; nt < 8; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                int r = e >> 1;
                float p = fast_exp2(s[nt][e] * scale_log2 - lse2[r]);
                if (need_mask) {
                    int col = j * TILE + nt * 8 + 2 * tig + (e & 1);
                    int row = row0 + 8 * r;
                    if (col >= S || row >= S || (CAUSAL && col > row)) p = 0.0f;
                }
                s[nt][e] = p * (dp[nt][e] - dl[r]); // dS (without the 1/sqrt(hd) factor)
            }
        gemm_kn(dq, s, sK[st], lane);
        if (j + 1 < ntiles) cp_async_wait<0>();
        __syncthreads();
    }
    store_rows(dQ + base_g, DG, q0 + warp * 16, S, dq, scale, scale, lane);
}

// ------------------------------------------------------------------ backward: dK, dV
template <bool CAUSAL>
__global__ void __launch_bounds__(kThreads) flash_dkv_kernel(const bf16 *__restrict__ Q, const bf16 *__restrict__ K, const bf16 *__restrict__ V,
                                                             const bf16 *__restrict__ dO, const float *__restrict__ LSE,
                                                             const float *__restrict__ DELTA, bf16 *__restrict__ dK, bf16 *__restrict__ dV,
                                                             int S, int D, int DO, int DG, int H, float scale, float scale_log2) {
    __shared__ __align__(128) unsigned char smem[TILE_BYTES * 4];
    __shared__ float sLse[2][TILE], sDelta[2][TILE];
    unsigned char *sQ[2] = {smem, smem + 2 * TILE_BYTES}, *sdO[2] = {smem + TILE_BYTES, smem + 3 * TILE_BYTES};
    // K and V are only read once, into registers: they borrow the second pipeline stage
    unsigned char *sK = sQ[1], *sV = sdO[1];
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gq = lane >> 2, tig = lane & 3;
    int kt = blockIdx.x, n = blockIdx.y / H, h = blockIdx.y % H;
    long long base = (long long)n * S * D + (long long)h * HD;      // q, k, v (row pitch D)
    long long base_o = (long long)n * S * DO + (long long)h * HD;   // o, do (row pitch DO)
    long long base_g = (long long)n * S * DG + (long long)h * HD;   // dq, dk, dv (row pitch DG)
    (void)base_o;
    (void)base_g;
    long long lb = ((long long)n * H + h) * S;
    int k0 = kt * TILE;
    int qtiles = (S + TILE - 1) / TILE;
    int i0 = CAUSAL ? kt : 0;
    auto load_q = [&](int i, int st) {
        int q1 = i * TILE;
        load_tile(sQ[st], Q + base + (long long)q1 * D, D, S - q1);
        load_tile(sdO[st], dO + base_o + (long long)q1 * DO, DO, S - q1);
        if (threadIdx.x < TILE) {
            int row = q1 + threadIdx.x;
            sLse[st][threadIdx.x] = row < S ? LSE[lb + row] * 1.4426950408889634f : 0.0f;
            sDelta[st][threadIdx.x] = row < S ? DELTA[lb + row] : 0.0f;
        }
    };
    load_tile(sK, K + base + (long long)k0 * D, D, S - k0);
    load_tile(sV, V + base + (long long)k0 * D, D, S - k0);
    load_q(i0, 0);
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();
    unsigned kf[4][4], vf[4][4];
    load_a_frags(kf, sK, warp, lane);
    load_a_frags(vf, sV, warp, lane);
    __syncthreads(); // stage 1 may now be overwritten by the first prefetch
    int krow0 = k0 + warp * 16 + gq;
    float dk[8][4], dv[8][4];
    zero_acc(dk);
    zero_acc(dv);
    for (int i = i0; i < qtiles; ++i) {
        int st = (i - i0) & 1;
        if (i + 1 < qtiles) {
            load_q(i + 1, st ^ 1);
            cp_async_commit();
        }
        float s[8][4], dp[8][4];
        zero_acc(s);
        zero_acc(dp);
        gemm_nk(s, kf, sQ[st], lane);   // S^T[key, query]
        gemm_nk(dp, vf, sdO[st], lane); // dP^T[key, query]
        bool need_mask = (CAUSAL && i == kt) || (i + 1) * TILE > S || k0 + TILE > S;
#pragma unroll
        for (int nt = 0; nt < 8; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                int qc = nt * 8 + 2 * tig + (e & 1);
                float p = fast_exp2(s[nt][e] * scale_log2 - sLse[st][qc]);
                if (need_mask) {
                    int qrow = i * TILE + qc;
                    int krow = krow0 + 8 * (e >> 1);
                    if (qrow >= S || krow >= S || (CAUSAL && krow > qrow)) p = 0.0f;
                }
                s[nt][e] = p;                                  // P^T
                dp[nt][e] = p * (dp[nt][e] - sDelta[st][qc]);  // dS^T
            }
        gemm_kn(dv, s, sdO[st], lane);
        gemm_kn(dk, dp, sQ[st], lane);
        if (i + 1 < qtiles) cp_async_wait<0>();
        __syncthreads();
    }
    store_rows(dK + base_g, DG, k0 + warp * 16, S, dk, scale, scale, lane);
    store_rows(dV + base_g, DG, k0 + warp * 16, S, dv, 1.0f, 1.0f, lane);
}

} // namespace

bool mcb_flash_supported(int64_t dim, int64_t heads, int32_t dt) { return mcb_is_lp(dt) && heads > 0 && dim == heads * HD; }

mcb_status mcb_flash_forward(mcb_ctx *ctx, const void *q, const void *k, const void *v, void *out, float *lse, int64_t n, int64_t seq,
                             int64_t dim, int64_t heads, int32_t causal, int64_t ldi, int64_t ldo, int32_t dt) {
    if (ldi % 8 || ldo % 8) return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "fused attention needs row pitches that are multiples of 8");
    if (!mcb_aligned16(q) || !mcb_aligned16(k) || !mcb_aligned16(v) || !mcb_aligned16(out) || (dim % 8))
        return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "fused attention needs 16-byte aligned tensors");
    if (n * heads > 65535) return mcb_fail(ctx, MCB_UNSUPPORTED, "fused attention: n * heads > 65535");
    // the tcgen05 / TMEM forward first; MCB_FLASH_LEGACY (test knob) keeps the mma.sync kernel
    if (!knob_on(ctx, K_FLASH_LEGACY) || dt == MCB_F16) {
        mcb_status tc = mcb_flash_tc_forward(ctx, q, k, v, out, lse, n, seq, dim, heads, causal, ldi, ldo, dt);
        if (tc != MCB_UNSUPPORTED) return tc;
    }
    if (dt != MCB_BF16) return mcb_fail(ctx, MCB_UNSUPPORTED, "fused f16 attention: shape outside the tensor-core kernel's range");
    float scale_log2 = (1.0f / sqrtf((float)HD)) * 1.4426950408889634f;
    dim3 grid((unsigned)((seq + TILE - 1) / TILE), (unsigned)(n * heads));
    if (causal)
        flash_fwd_kernel<true><<<grid, kThreads, 0, ctx->stream>>>((const bf16 *)q, (const bf16 *)k, (const bf16 *)v, (bf16 *)out, lse, (int)seq, (int)ldi, (int)ldo, (int)ldo, (int)heads, scale_log2);
    else
        flash_fwd_kernel<false><<<grid, kThreads, 0, ctx->stream>>>((const bf16 *)q, (const bf16 *)k, (const bf16 *)v, (bf16 *)out, lse, (int)seq, (int)ldi, (int)ldo, (int)ldo, (int)heads, scale_log2);
    MCB_LAUNCHED(ctx);
    return MCB_OK;
}

mcb_status mcb_flash_backward(mcb_ctx *ctx, const void *q, const void *k, const void *v, const void *out, const void *gout, const float *lse,
                              void *dq, void *dk, void *dv, int64_t n, int64_t seq, int64_t dim, int64_t heads, int32_t causal,
                              int64_t ldi, int64_t ldo, int64_t ldg, float *bias_partial, int64_t bias_ld, int *bias_done, int32_t dt) {
    (void)dim;
    if (bias_done) *bias_done = 0;
    if (ldi % 8 || ldo % 8 || ldg % 8) return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "fused attention needs row pitches that are multiples of 8");
    if (n * heads > 65535) return mcb_fail(ctx, MCB_UNSUPPORTED, "fused attention: n * heads > 65535");
    if ((((uintptr_t)out) | ((uintptr_t)gout) | ((uintptr_t)q) | ((uintptr_t)k) | ((uintptr_t)v) | ((uintptr_t)dq) | ((uintptr_t)dk) | ((uintptr_t)dv)) & 15)
        return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "fused attention needs 16-byte aligned tensors");
    float scale = 1.0f / sqrtf((float)HD), scale_log2 = scale * 1.4426950408889634f;
    long long rows = n * heads * seq;
    void *delta = nullptr;
    MCB_TRY(mcb_alloc(ctx, sizeof(float) * rows, &delta));
    {
        const long long chunks = rows * (HD / 8);
        // gout has the pitch of out; ldg is the pitch of dq / dk / dv
        if (dt == MCB_F16)
            MCB_CUDA(ctx, mcb_launch_dep(ctx, flash_delta_kernel<__half>, dim3((unsigned)((chunks + 255) / 256)), dim3(256), 0, (const __half *)out, (const __half *)gout, (float *)delta, (int)seq, (int)ldo, (int)ldo, (int)heads, chunks));
        else
            MCB_CUDA(ctx, mcb_launch_dep(ctx, flash_delta_kernel<bf16>, dim3((unsigned)((chunks + 255) / 256)), dim3(256), 0, (const bf16 *)out, (const bf16 *)gout, (float *)delta, (int)seq, (int)ldo, (int)ldo, (int)heads, chunks));
    }
    ctx->launches++;
    // the tcgen05 / TMEM kernels first; MCB_FLASH_LEGACY (test knob) keeps the mma.sync pair
    if ((!knob_on(ctx, K_FLASH_LEGACY) && !knob_on(ctx, K_FLASH_LEGACY_BWD)) || dt == MCB_F16) {
        mcb_status tc = mcb_flash_tc_backward(ctx, q, k, v, gout, lse, (const float *)delta, dq, dk, dv, n, seq, dim, heads, causal, ldi, ldo, ldg,
                                              bias_partial, bias_ld, dt);
        if (tc != MCB_UNSUPPORTED) {
            if (bias_done && bias_partial && tc == MCB_OK) *bias_done = 1;
            mcb_free(ctx, delta); // stream-ordered reuse
            return tc;
        }
    }
    if (dt != MCB_BF16) {
        mcb_free(ctx, delta);
        return mcb_fail(ctx, MCB_UNSUPPORTED, "fused f16 attention backward: shape outside the tensor-core kernel's range");
    }
    dim3 grid((unsigned)((seq + TILE - 1) / TILE), (unsigned)(n * heads));
    if (causal) {
        flash_dkv_kernel<true><<<grid, kThreads, 0, ctx->stream>>>((const bf16 *)q, (const bf16 *)k, (const bf16 *)v, (const bf16 *)gout, lse, (const float *)delta, (bf16 *)dk, (bf16 *)dv, (int)seq, (int)ldi, (int)ldo, (int)ldg, (int)heads, scale, scale_log2);
        flash_dq_kernel<true><<<grid, kThreads, 0, ctx->stream>>>((const bf16 *)q, (const bf16 *)k, (const bf16 *)v, (const bf16 *)gout, lse, (const float *)delta, (bf16 *)dq, (int)seq, (int)ldi, (int)ldo, (int)ldg, (int)heads, scale, scale_log2);
    } else {
        flash_dkv_kernel<false><<<grid, kThreads, 0, ctx->stream>>>((const bf16 *)q, (const bf16 *)k, (const bf16 *)v, (const bf16 *)gout, lse, (const float *)delta, (bf16 *)dk, (bf16 *)dv, (int)seq, (int)ldi, (int)ldo, (int)ldg, (int)heads, scale, scale_log2);
        flash_dq_kernel<false><<<grid, kThreads, 0, ctx->stream>>>((const bf16 *)q, (const bf16 *)k, (const bf16 *)v, (const bf16 *)gout, lse, (const float *)delta, (bf16 *)dq, (int)seq, (int)ldi, (int)ldo, (int)ldg, (int)heads, scale, scale_log2);
    }
    ctx->launches += 2;
    cudaError_t e = cudaGetLastError();
    mcb_free(ctx, delta); // stream-ordered reuse: later users of the block are enqueued after these kernels
    if (e != cudaSuccess) return mcb_cuda_check(ctx, e, "fused attention backward launch");
    return MCB_OK;
}
