// f32 contractions on the tcgen05 tensor cores at f32 accuracy, and the convolution built on them.
//
// An f32 operand X is cut into two IEEE f16 pieces after scaling by a power of two s (exact):
//     hi = f16(X s),  lo = f16(X s - hi)        =>  X s = hi + lo up to 2^-22 |X s|
// and a product A B becomes three tensor-core GEMMs with exact f16 x f16 products and f32 accumulation,
//     (A sa)(B sb) ~= Ah Bh + Ah Bl + Al Bh     (the dropped Al Bl is 2^-22 of the result)
// accumulated into one f32 output and divided by sa sb (a power of two) afterwards.  s is chosen per operand
// from its largest magnitude (read on the device: no host round trip), so f16's narrow range is never left.
// The pieces reproduce an f32 product to about 2^-21; what limits the accuracy is the tensor core's own accumulation
// (see split_gemm), kept near 2e-6 by slicing long reductions: inside the 1e-5 bar for f32 parity.
//
// Convolution (Conv2dOp, crates/modern-chainer-autograd/src/host_ops.rs:57-180; a single-threaded host loop in
// the reference) is lowered to those GEMMs through an explicit column matrix:
//   forward   col[M, K] (M = n oh ow rows, K = c kh kw) x W[O, K]^T -> [M, O], then to NCHW with the bias
//   dgrad     g[M, O] x W[O, K] -> dcol[M, K], gathered back into dx (each input pixel sums the <= kh kw
//             column entries that read it)
//   wgrad     g^T[O, M] x col[M, K] -> dW[O, K]
// The column matrix is written as its two f16 pieces (K padded to a multiple of 8 for the 16-byte row pitch the TMA
// tensor maps need).  Backward writes it again (one more HBM-bound pass) instead of keeping 2 x M x K8 f16 values
// alive from forward to backward.
#include "internal.h"

namespace {

constexpr int kThreads = 256;

struct ConvDims {
    int n, c, h, w, o, kh, kw, stride, pad, oh, ow;
    int k, k8; // c kh kw and its multiple-of-8 padding
    long long m; // n oh ow
};

// ---- largest magnitude of an f32 array, as the bits of a non-negative float (monotone as unsigned)
__global__ void amax_kernel(const float *__restrict__ x, long long n, unsigned *__restrict__ out) {
    float m = 0.0f;
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x, stride = (long long)gridDim.x * blockDim.x;
    for (; i < n; i += stride) {
        float v = fabsf(x[i]);
        m = (v > m && v < INFINITY) ? v : m; // inf / nan do not set the scale; they propagate through the pieces
    }
    m = warp_max(m);
    if ((threadIdx.x & 31) == 0 && m > 0.0f) atomicMax(out, __float_as_uint(m));
}

// power-of-two scale that brings `amax` into [2^12, 2^13): products of two such operands stay below 2^26 and a sum of
// 2^30 of them is still finite in f32; f16 (max 65504) holds every scaled element
__device__ __forceinline__ float scale_of(unsigned amax_bits) {
    float amax = __uint_as_float(amax_bits);
    if (!(amax > 0.0f)) return 1.0f;
    int e;
    frexpf(amax, &e); // amax = f 2^e, f in [0.5, 1)
    return ldexpf(1.0f, 13 - e);
}

__device__ __forceinline__ void split1(float v, float s, __half &hi, __half &lo) {
    float t = v * s;
    hi = __float2half_rn(t);
    lo = __float2half_rn(t - __half2float(hi));
}

// Layout of the pieces: three [rows, cols8] f16 matrices, piece p at `out + p * piece_stride` with row pitch `ld`:
//   side by side (ld = 3 cols8, piece_stride = cols8): one K-major operand whose reduction index runs through the three pieces
//   stacked      (ld = cols8, piece_stride = rows cols8): the same for an MN-major operand (the reduction index counts rows)
// The A-side operand of a product carries (hi, hi, lo), the B-side (hi, lo, hi): the reduction over the concatenated
// index then yields Ah Bh + Ah Bl + Al Bh in ONE GEMM launch, with no accumulating passes over the output.
__device__ __forceinline__ void put3(__half *out, long long at, long long piece_stride, __half h, __half l, int b_side) {
    out[at] = h;
    out[at + piece_stride] = b_side ? l : h;
    out[at + 2 * piece_stride] = b_side ? h : l;
}

// generic [rows, cols] f32 -> pieces (columns cols..cols8-1 zero)
__global__ void split_rows_kernel(const float *__restrict__ x, long long rows, int cols, int cols8, const unsigned *__restrict__ amax,
                                  __half *__restrict__ out, long long ld, long long piece_stride, int b_side) {
    const float s = scale_of(*amax);
    long long total = rows * cols8;
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x, stride = (long long)gridDim.x * blockDim.x;
    for (; i < total; i += stride) {
        long long r = i / cols8;
        int c = (int)(i - r * cols8);
        __half h = __float2half_rn(0.0f), l = h;
        if (c < cols) split1(x[r * cols + c], s, h, l);
        put3(out, r * ld + c, piece_stride, h, l, b_side);
    }
}

// g NCHW [n, o, oh, ow] -> A-side pieces [M = n oh ow, O] side by side (row pitch 3 O).  Tiles of 32 positions x 32
// channels go through shared memory, so the NCHW reads run along positions and the writes along channels.
__global__ void __launch_bounds__(256) split_nchw_to_rows_kernel(const float *__restrict__ g, ConvDims d, const unsigned *__restrict__ amax,
                                                                 __half *__restrict__ out) {
    __shared__ float tile[32][33];
    const float s = scale_of(*amax);
    const int plane = d.oh * d.ow;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const long long ni = blockIdx.z;
    const int r0 = blockIdx.x * 32, o0 = blockIdx.y * 32;
#pragma unroll
    for (int j = 0; j < 4; ++j) { // tile[channel][position]
        const int o = o0 + ty + 8 * j, r = r0 + tx;
        tile[ty + 8 * j][tx] = (o < d.o && r < plane) ? g[(ni * d.o + o) * plane + r] : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int r = r0 + ty + 8 * j, o = o0 + tx;
        if (r < plane && o < d.o) {
            __half h, l;
            split1(tile[tx][ty + 8 * j], s, h, l);
            put3(out, (ni * plane + r) * (3ll * d.o) + o, d.o, h, l, 0);
        }
    }
}

// x NCHW -> A-side column-matrix pieces [M, K8] side by side (row pitch 3 K8); column k = (ci kh + ky) kw + kx, zero outside
// the image and in the padding
// One thread per (row, group of 8 columns): the row's position is decoded once, the column's (ci, ky, kx) advances by
// counting, and each piece receives one 16-byte store.
__global__ void im2col_split_kernel(const float *__restrict__ x, ConvDims d, const unsigned *__restrict__ amax, __half *__restrict__ out) {
    const float s = scale_of(*amax);
    const int groups = d.k8 >> 3;
    const long long total = d.m * groups;
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x, stride = (long long)gridDim.x * blockDim.x;
    for (; i < total; i += stride) {
        const long long m = i / groups;
        int k = (int)(i - m * groups) << 3;
        const int mm = (int)(m % ((long long)d.ow * d.oh));
        const long long ni = m / ((long long)d.ow * d.oh);
        const int xo = mm % d.ow, yo = mm / d.ow;
        int kx = k % d.kw, ky = (k / d.kw) % d.kh, ci = k / (d.kw * d.kh);
        __align__(16) __half h[8], l[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            float v = 0.0f;
            if (k + j < d.k) {
                const int iy = yo * d.stride + ky - d.pad, ix = xo * d.stride + kx - d.pad;
                if (iy >= 0 && iy < d.h && ix >= 0 && ix < d.w) v = x[((ni * d.c + ci) * d.h + iy) * d.w + ix];
            }
            split1(v, s, h[j], l[j]);
            if (++kx == d.kw) {
                kx = 0;
                if (++ky == d.kh) {
                    ky = 0;
                    ++ci;
                }
            }
        }
        __half *dst = out + m * (3ll * d.k8) + k; // 16-byte aligned: k8 and k are multiples of 8
        *reinterpret_cast<uint4 *>(dst) = *reinterpret_cast<const uint4 *>(h);
        *reinterpret_cast<uint4 *>(dst + d.k8) = *reinterpret_cast<const uint4 *>(h);
        *reinterpret_cast<uint4 *>(dst + 2 * d.k8) = *reinterpret_cast<const uint4 *>(l);
    }
}

// [M, O] f32 product (of scaled operands) -> NCHW output with the scale undone and the bias added (tiles through shared memory)
__global__ void __launch_bounds__(256) rows_to_nchw_kernel(const float *__restrict__ acc, ConvDims d, const unsigned *__restrict__ amax_a,
                                                           const unsigned *__restrict__ amax_b, const float *__restrict__ bias, float *__restrict__ out) {
    __shared__ float tile[32][33];
    const float inv = 1.0f / (scale_of(*amax_a) * scale_of(*amax_b)); // a power of two: exact
    const int plane = d.oh * d.ow;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const long long ni = blockIdx.z;
    const int r0 = blockIdx.x * 32, o0 = blockIdx.y * 32;
#pragma unroll
    for (int j = 0; j < 4; ++j) { // tile[position][channel]
        const int r = r0 + ty + 8 * j, o = o0 + tx;
        tile[ty + 8 * j][tx] = (r < plane && o < d.o) ? acc[(ni * plane + r) * d.o + o] : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int o = o0 + ty + 8 * j, r = r0 + tx;
        if (o < d.o && r < plane) {
            const float v = tile[tx][ty + 8 * j] * inv;
            out[(ni * d.o + o) * plane + r] = bias ? v + bias[o] : v;
        }
    }
}

// dcol [M, K8] -> dx NCHW: every input pixel gathers the column entries that read it.  A block takes 32 pixels of one
// image row and 32 channels: the gathers run along the channel index (neighbouring columns of dcol), the stores along x.
__global__ void __launch_bounds__(256) col2im_kernel(const float *__restrict__ dcol, ConvDims d, const unsigned *__restrict__ amax_a,
                                                     const unsigned *__restrict__ amax_b, float *__restrict__ dx) {
    __shared__ float tile[32][33];
    const float inv = 1.0f / (scale_of(*amax_a) * scale_of(*amax_b));
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int xtiles = (d.w + 31) / 32;
    const int x0 = (blockIdx.x % xtiles) * 32, iy = blockIdx.x / xtiles, c0 = blockIdx.y * 32;
    const long long ni = blockIdx.z;
#pragma unroll
    for (int j = 0; j < 4; ++j) { // tile[pixel][channel]
        const int ix = x0 + ty + 8 * j, ci = c0 + tx;
        float sum = 0.0f;
        if (ix < d.w && ci < d.c) {
            for (int ky = 0; ky < d.kh; ++ky) {
                int t = iy + d.pad - ky;
                if (t < 0 || t % d.stride) continue;
                int yo = t / d.stride;
                if (yo >= d.oh) continue;
                for (int kx = 0; kx < d.kw; ++kx) {
                    int u = ix + d.pad - kx;
                    if (u < 0 || u % d.stride) continue;
                    int xo = u / d.stride;
                    if (xo >= d.ow) continue;
                    sum += dcol[((ni * d.oh + yo) * d.ow + xo) * d.k8 + (ci * d.kh + ky) * d.kw + kx];
                }
            }
        }
        tile[ty + 8 * j][tx] = sum * inv;
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int ci = c0 + ty + 8 * j, ix = x0 + tx;
        if (ci < d.c && ix < d.w) dx[((ni * d.c + ci) * d.h + iy) * d.w + ix] = tile[tx][ty + 8 * j];
    }
}

// [rows, cols8] f32 -> [rows, cols] with the scale undone (weight gradient out of its padded accumulator)
__global__ void unscale_rows_kernel(const float *__restrict__ acc, long long rows, int cols, int cols8, const unsigned *__restrict__ amax_a,
                                    const unsigned *__restrict__ amax_b, float *__restrict__ out) {
    const float inv = 1.0f / (scale_of(*amax_a) * scale_of(*amax_b));
    long long total = rows * cols;
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x, stride = (long long)gridDim.x * blockDim.x;
    for (; i < total; i += stride) {
        long long r = i / cols;
        int c = (int)(i - r * cols);
        out[i] = acc[r * cols8 + c] * inv;
    }
}

struct Tmp { // scratch blocks of one call, returned to the context's allocator (stream-ordered reuse) when it ends
    mcb_ctx *ctx;
    std::vector<void *> blocks;
    explicit Tmp(mcb_ctx *c) : ctx(c) {}
    ~Tmp() {
        for (void *p : blocks) mcb_free(ctx, p);
    }
    mcb_status get(size_t bytes, void **out) {
        MCB_TRY(mcb_alloc(ctx, bytes ? bytes : 16, out));
        blocks.push_back(*out);
        return MCB_OK;
    }
};

mcb_status amax_of(mcb_ctx *ctx, const float *x, long long n, unsigned *slot) {
    MCB_TRY(mcb_memset(ctx, slot, 0, sizeof(unsigned)));
    if (n == 0) return MCB_OK;
    amax_kernel<<<mcb_grid_for(ctx, n, kThreads, 8), kThreads, 0, ctx->stream>>>(x, n, slot);
    MCB_LAUNCHED(ctx);
    return MCB_OK;
}

// One launch: D[m, n] (f32, row pitch ldd) = A' B' over the concatenated reduction index of length 3 k (pieces side by side
// for a K-major operand, stacked for an MN-major one: see put3).  The accumulator sees 3 k / 16 additions: for the forward
// and data-gradient products of a convolution (k = c kh kw or the channel count) a few dozen.
mcb_status concat_gemm(mcb_ctx *ctx, const __half *a, int a_mn, long long lda, const __half *b, int b_mn, long long ldb, float *d, long long ldd,
                       long long m, long long n, long long k) {
    TcGemmParams p;
    p.in_dt = MCB_F16;
    p.a = a; p.a_mn_major = a_mn; p.lda = lda;
    p.b = b; p.b_mn_major = b_mn; p.ldb = ldb;
    p.d = d; p.out_dt = MCB_F32; p.ldd = ldd;
    p.m = m; p.n = n; p.k = 3 * k;
    return mcb_tc_gemm(ctx, p);
}

// Three launches accumulating into a zeroed D: for the weight gradient, whose reduction runs over all n oh ow positions.
// The tensor core adds each 16-deep group of products to its f32 accumulator with truncation: an error of about
// (k / 16) * 2^-24 of the sum (measured 4e-5 at k = 8192 per accumulator).  The reduction is therefore cut into slices of
// at most 1024 (64 additions, about 2e-6); the slices meet in f32 adds that round to nearest.
mcb_status split_gemm(mcb_ctx *ctx, const __half *ah, const __half *al, int a_mn, long long lda, const __half *bh, const __half *bl, int b_mn,
                      long long ldb, float *d, long long ldd, long long m, long long n, long long k) {
    MCB_TRY(mcb_memset(ctx, d, 0, sizeof(float) * (size_t)m * (size_t)ldd));
    const __half *as[3] = {ah, ah, al}, *bs[3] = {bh, bl, bh};
    for (int i = 0; i < 3; ++i) {
        TcGemmParams p;
        p.in_dt = MCB_F16;
        p.a = as[i]; p.a_mn_major = a_mn; p.lda = lda;
        p.b = bs[i]; p.b_mn_major = b_mn; p.ldb = ldb;
        p.d = d; p.out_dt = MCB_F32; p.ldd = ldd;
        p.m = m; p.n = n; p.k = k;
        p.accumulate = 1;
        mcb_tc_plan(ctx, m, n, k, true, true, 1, &p.bn, &p.split_k);
        const long long want = (k + 1023) / 1024;
        if (p.split_k < want) p.split_k = (int)(want < 1024 ? want : 1024);
        MCB_TRY(mcb_tc_gemm(ctx, p));
    }
    return MCB_OK;
}

void fill_dims(ConvDims &d, int64_t n, int64_t c, int64_t h, int64_t wd, int64_t o, int64_t kh, int64_t kw, int64_t stride, int64_t pad) {
    d.n = (int)n; d.c = (int)c; d.h = (int)h; d.w = (int)wd; d.o = (int)o; d.kh = (int)kh; d.kw = (int)kw;
    d.stride = (int)stride; d.pad = (int)pad;
    d.oh = (int)((h + 2 * pad - kh) / stride + 1);
    d.ow = (int)((wd + 2 * pad - kw) / stride + 1);
    d.k = d.c * d.kh * d.kw;
    d.k8 = (d.k + 7) / 8 * 8;
    d.m = (long long)d.n * d.oh * d.ow;
}

} // namespace

// Worth the column matrix and three GEMM launches from about 2^24 multiply-adds on; the output channel count must
// give 16-byte rows ([M, O] f16: O % 8 == 0) and the extents must fit the kernels' 32-bit indices.
bool mcb_conv_tc_eligible(mcb_ctx *ctx, int64_t n, int64_t c, int64_t h, int64_t wd, int64_t o, int64_t kh, int64_t kw, int64_t stride, int64_t pad) {
    if (knob_on(ctx, K_CONV_DIRECT)) return false; // test knob: keep the direct kernels
    if (stride <= 0 || pad < 0 || h + 2 * pad < kh || wd + 2 * pad < kw || o % 8) return false;
    ConvDims d;
    fill_dims(d, n, c, h, wd, o, kh, kw, stride, pad);
    const double macs = (double)d.m * d.k * d.o;
    return macs >= (double)(1 << 24) && d.m % 8 == 0 && d.m * d.k8 < (1ll << 40) && (long long)n * c * h * wd < (1ll << 40);
}

mcb_status mcb_conv_tc_forward(mcb_ctx *ctx, const float *x, const float *w, const float *bias, float *out, int64_t n, int64_t c, int64_t h,
                               int64_t wd, int64_t o, int64_t kh, int64_t kw, int64_t stride, int64_t pad) {
    ConvDims d;
    fill_dims(d, n, c, h, wd, o, kh, kw, stride, pad);
    if (d.m == 0 || d.o == 0) return MCB_OK;
    ProfScope prof(ctx, MCB_PROF_CONV, 2.0 * (double)d.m * d.k * d.o, 4.0 * ((double)n * c * h * wd + (double)d.m * d.o));
    Tmp tmp(ctx);
    void *ax, *aw, *col, *wp, *acc;
    MCB_TRY(tmp.get(16, &ax));
    MCB_TRY(tmp.get(16, &aw));
    MCB_TRY(tmp.get(sizeof(__half) * 3 * (size_t)d.m * d.k8, &col));
    MCB_TRY(tmp.get(sizeof(__half) * 3 * (size_t)d.o * d.k8, &wp));
    MCB_TRY(tmp.get(sizeof(float) * (size_t)d.m * d.o, &acc));
    MCB_TRY(amax_of(ctx, x, (long long)n * c * h * wd, (unsigned *)ax));
    MCB_TRY(amax_of(ctx, w, (long long)d.o * d.k, (unsigned *)aw));
    im2col_split_kernel<<<mcb_grid_for(ctx, d.m * (d.k8 / 8), kThreads, 16), kThreads, 0, ctx->stream>>>(x, d, (const unsigned *)ax, (__half *)col);
    MCB_LAUNCHED(ctx);
    // W [O, K]: B-side pieces side by side, [O, 3 K8]
    split_rows_kernel<<<mcb_grid_for(ctx, (long long)d.o * d.k8, kThreads, 8), kThreads, 0, ctx->stream>>>(w, d.o, d.k, d.k8, (const unsigned *)aw, (__half *)wp,
                                                                                                        3ll * d.k8, d.k8, 1);
    MCB_LAUNCHED(ctx);
    MCB_TRY(concat_gemm(ctx, (const __half *)col, 0, 3ll * d.k8, (const __half *)wp, 0, 3ll * d.k8, (float *)acc, d.o, d.m, d.o, d.k8));
    const int plane = d.oh * d.ow;
    rows_to_nchw_kernel<<<dim3((plane + 31) / 32, (d.o + 31) / 32, d.n), 256, 0, ctx->stream>>>((const float *)acc, d, (const unsigned *)ax, (const unsigned *)aw,
                                                                                             bias, out);
    MCB_LAUNCHED(ctx);
    return MCB_OK;
}

mcb_status mcb_conv_tc_backward(mcb_ctx *ctx, const float *x, const float *w, const float *g, float *dx, float *dw, int64_t n, int64_t c, int64_t h,
                                int64_t wd, int64_t o, int64_t kh, int64_t kw, int64_t stride, int64_t pad) {
    ConvDims d;
    fill_dims(d, n, c, h, wd, o, kh, kw, stride, pad);
    if (d.m == 0 || d.o == 0 || (!dx && !dw)) return MCB_OK;
    ProfScope prof(ctx, MCB_PROF_CONV, 2.0 * (double)d.m * d.k * d.o * ((dx ? 1 : 0) + (dw ? 1 : 0)),
                   4.0 * ((double)n * c * h * wd * (dx ? 2 : 1) + (double)d.m * d.o));
    Tmp tmp(ctx);
    void *ag, *gp;
    MCB_TRY(tmp.get(16, &ag));
    MCB_TRY(tmp.get(sizeof(__half) * 3 * (size_t)d.m * d.o, &gp)); // [M, 3 O]: gh | gh | gl
    MCB_TRY(amax_of(ctx, g, d.m * d.o, (unsigned *)ag));
    const int plane = d.oh * d.ow;
    split_nchw_to_rows_kernel<<<dim3((plane + 31) / 32, (d.o + 31) / 32, d.n), 256, 0, ctx->stream>>>(g, d, (const unsigned *)ag, (__half *)gp);
    MCB_LAUNCHED(ctx);
    const __half *gh = (const __half *)gp, *gl = gh + 2 * d.o; // pieces of the side-by-side layout, row pitch 3 O
    if (dx) { // dcol[M, K8] = g[M, O] W[O, K8]: one launch over the concatenated channel index
        void *aw, *wp, *dcol;
        MCB_TRY(tmp.get(16, &aw));
        MCB_TRY(tmp.get(sizeof(__half) * 3 * (size_t)d.o * d.k8, &wp));
        MCB_TRY(tmp.get(sizeof(float) * (size_t)d.m * d.k8, &dcol));
        MCB_TRY(amax_of(ctx, w, (long long)d.o * d.k, (unsigned *)aw));
        // W as the MN-major B operand [reduction = O rows, K8 columns]: B-side pieces stacked, [3 O, K8]
        split_rows_kernel<<<mcb_grid_for(ctx, (long long)d.o * d.k8, kThreads, 8), kThreads, 0, ctx->stream>>>(w, d.o, d.k, d.k8, (const unsigned *)aw, (__half *)wp,
                                                                                                            d.k8, (long long)d.o * d.k8, 1);
        MCB_LAUNCHED(ctx);
        MCB_TRY(concat_gemm(ctx, gh, 0, 3ll * d.o, (const __half *)wp, 1, d.k8, (float *)dcol, d.k8, d.m, d.k8, d.o));
        const int xtiles = (d.w + 31) / 32;
        col2im_kernel<<<dim3(xtiles * d.h, (d.c + 31) / 32, d.n), 256, 0, ctx->stream>>>((const float *)dcol, d, (const unsigned *)ag, (const unsigned *)aw, dx);
        MCB_LAUNCHED(ctx);
    }
    if (dw) { // dW[O, K8] = g^T[O, M] col[M, K8]: long reduction, sliced (see split_gemm)
        void *ax, *col, *acc;
        MCB_TRY(tmp.get(16, &ax));
        MCB_TRY(tmp.get(sizeof(__half) * 3 * (size_t)d.m * d.k8, &col));
        MCB_TRY(tmp.get(sizeof(float) * (size_t)d.o * d.k8, &acc));
        MCB_TRY(amax_of(ctx, x, (long long)n * c * h * wd, (unsigned *)ax));
        im2col_split_kernel<<<mcb_grid_for(ctx, d.m * (d.k8 / 8), kThreads, 16), kThreads, 0, ctx->stream>>>(x, d, (const unsigned *)ax, (__half *)col);
        MCB_LAUNCHED(ctx);
        const __half *ch = (const __half *)col, *cl = ch + 2 * d.k8; // row pitch 3 K8
        MCB_TRY(split_gemm(ctx, gh, gl, 1, 3ll * d.o, ch, cl, 1, 3ll * d.k8, (float *)acc, d.k8, d.o, d.k8, d.m));
        unscale_rows_kernel<<<mcb_grid_for(ctx, (long long)d.o * d.k, kThreads, 8), kThreads, 0, ctx->stream>>>((const float *)acc, d.o, d.k, d.k8,
                                                                                                             (const unsigned *)ag, (const unsigned *)ax, dw);
        MCB_LAUNCHED(ctx);
    }
    return MCB_OK;
}
