// NCHW convolution and max-pooling, forward and backward, in exact f32 on the device
// (host loops on every backend in the reference, autograd/src/host_ops.rs:40-180,341-476).
// Direct kernels: one thread per output element for forward / dx, one block per weight
// element for dw (tree reduction over n*oh*ow terms), column sums for db.
#include "internal.h"

namespace {

struct ConvDims {
    int n, c, h, w, o, kh, kw, stride, pad, oh, ow;
};

__global__ void conv2d_fwd_kernel(const float *__restrict__ x, const float *__restrict__ wt,
                                  const float *__restrict__ bias, float *__restrict__ out, ConvDims d) {
    long long total = (long long)d.n * d.o * d.oh * d.ow;
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    long long step = (long long)gridDim.x * blockDim.x;
    for (; i < total; i += step) {
        int xo = (int)(i % d.ow);
        int yo = (int)((i / d.ow) % d.oh);
        int oi = (int)((i / ((long long)d.ow * d.oh)) % d.o);
        int ni = (int)(i / ((long long)d.ow * d.oh * d.o));
        float sum = bias ? bias[oi] : 0.0f;
        for (int ci = 0; ci < d.c; ++ci)
            for (int ky = 0; ky < d.kh; ++ky) {
                int iy = yo * d.stride + ky - d.pad;
                if (iy < 0 || iy >= d.h) continue;
                for (int kx = 0; kx < d.kw; ++kx) {
                    int ix = xo * d.stride + kx - d.pad;
                    if (ix < 0 || ix >= d.w) continue;
                    sum = fmaf(x[(((long long)ni * d.c + ci) * d.h + iy) * d.w + ix],
                               wt[(((long long)oi * d.c + ci) * d.kh + ky) * d.kw + kx], sum);
                }
            }
        out[i] = sum;
    }
}

// dx[n,c,iy,ix] = sum_{o,ky,kx} g[n,o,y,x] * w[o,c,ky,kx] with y*stride + ky - pad == iy
__global__ void conv2d_dx_kernel(const float *__restrict__ g, const float *__restrict__ wt, float *__restrict__ dx, ConvDims d) {
    long long total = (long long)d.n * d.c * d.h * d.w;
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    long long step = (long long)gridDim.x * blockDim.x;
    for (; i < total; i += step) {
        int ix = (int)(i % d.w);
        int iy = (int)((i / d.w) % d.h);
        int ci = (int)((i / ((long long)d.w * d.h)) % d.c);
        int ni = (int)(i / ((long long)d.w * d.h * d.c));
        float sum = 0.0f;
        for (int oi = 0; oi < d.o; ++oi)
            for (int ky = 0; ky < d.kh; ++ky) {
                int ty = iy + d.pad - ky;
                if (ty < 0 || ty % d.stride) continue;
                int yo = ty / d.stride;
                if (yo >= d.oh) continue;
                for (int kx = 0; kx < d.kw; ++kx) {
                    int tx = ix + d.pad - kx;
                    if (tx < 0 || tx % d.stride) continue;
                    int xo = tx / d.stride;
                    if (xo >= d.ow) continue;
                    sum = fmaf(g[(((long long)ni * d.o + oi) * d.oh + yo) * d.ow + xo],
                               wt[(((long long)oi * d.c + ci) * d.kh + ky) * d.kw + kx], sum);
                }
            }
        dx[i] = sum;
    }
}

// one block per weight element
__global__ void conv2d_dw_kernel(const float *__restrict__ x, const float *__restrict__ g, float *__restrict__ dw, ConvDims d) {
    __shared__ float red[32];
    int wi = blockIdx.x;
    int kx = wi % d.kw;
    int ky = (wi / d.kw) % d.kh;
    int ci = (wi / (d.kw * d.kh)) % d.c;
    int oi = wi / (d.kw * d.kh * d.c);
    long long terms = (long long)d.n * d.oh * d.ow;
    float sum = 0.0f;
    for (long long t = threadIdx.x; t < terms; t += blockDim.x) {
        int xo = (int)(t % d.ow);
        int yo = (int)((t / d.ow) % d.oh);
        int ni = (int)(t / ((long long)d.ow * d.oh));
        int iy = yo * d.stride + ky - d.pad, ix = xo * d.stride + kx - d.pad;
        if (iy < 0 || iy >= d.h || ix < 0 || ix >= d.w) continue;
        sum = fmaf(g[(((long long)ni * d.o + oi) * d.oh + yo) * d.ow + xo],
                   x[(((long long)ni * d.c + ci) * d.h + iy) * d.w + ix], sum);
    }
    sum = block_sum(sum, red);
    if (threadIdx.x == 0) dw[wi] = sum;
}

// bias gradient: block (channel, part) sums the planes of the samples part, part + parts, ...; a second kernel adds the
// parts of each channel in a fixed order
__global__ void conv2d_db_partial_kernel(const float *__restrict__ g, float *__restrict__ partial, ConvDims d) {
    __shared__ float red[32];
    const int oi = blockIdx.x, part = blockIdx.y, parts = gridDim.y;
    const int plane = d.oh * d.ow;
    float sum = 0.0f;
    for (int ni = part; ni < d.n; ni += parts) {
        const float *src = g + ((long long)ni * d.o + oi) * plane;
        for (int r = threadIdx.x; r < plane; r += blockDim.x) sum += src[r];
    }
    sum = block_sum(sum, red);
    if (threadIdx.x == 0) partial[(long long)part * d.o + oi] = sum;
}
__global__ void conv2d_db_final_kernel(const float *__restrict__ partial, int parts, int o, float *__restrict__ db) {
    int oi = blockIdx.x * blockDim.x + threadIdx.x;
    if (oi >= o) return;
    float t = 0.0f;
    for (int p = 0; p < parts; ++p) t += partial[(long long)p * o + oi];
    db[oi] = t;
}

struct PoolDims {
    int nc, h, w, k, stride, pad, oh, ow;
};

__global__ void max_pool_fwd_kernel(const float *__restrict__ x, float *__restrict__ out, PoolDims d) {
    long long total = (long long)d.nc * d.oh * d.ow;
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    long long step = (long long)gridDim.x * blockDim.x;
    for (; i < total; i += step) {
        int xo = (int)(i % d.ow);
        int yo = (int)((i / d.ow) % d.oh);
        long long nc = i / ((long long)d.ow * d.oh);
        float acc = -INFINITY;
        for (int ky = 0; ky < d.k; ++ky) {
            int iy = yo * d.stride + ky - d.pad;
            if (iy < 0 || iy >= d.h) continue;
            for (int kx = 0; kx < d.k; ++kx) {
                int ix = xo * d.stride + kx - d.pad;
                if (ix < 0 || ix >= d.w) continue;
                float v = x[(nc * d.h + iy) * d.w + ix];
                acc = v > acc ? v : acc;
            }
        }
        out[i] = acc;
    }
}

// The reference routes the gradient to the first element of each window row scan that equals
// the window maximum: its `break` leaves only the inner (kx) loop, so a later ky row holding
// the same maximum receives the gradient as well.  Same rule here; dx is zero-filled first.
__global__ void max_pool_bwd_kernel(const float *__restrict__ x, const float *__restrict__ g, float *__restrict__ dx, PoolDims d) {
    long long total = (long long)d.nc * d.oh * d.ow;
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    long long step = (long long)gridDim.x * blockDim.x;
    for (; i < total; i += step) {
        int xo = (int)(i % d.ow);
        int yo = (int)((i / d.ow) % d.oh);
        long long nc = i / ((long long)d.ow * d.oh);
        float best = -INFINITY;
        for (int ky = 0; ky < d.k; ++ky) {
            int iy = yo * d.stride + ky - d.pad;
            if (iy < 0 || iy >= d.h) continue;
            for (int kx = 0; kx < d.k; ++kx) {
                int ix = xo * d.stride + kx - d.pad;
                if (ix < 0 || ix >= d.w) continue;
                float v = x[(nc * d.h + iy) * d.w + ix];
                best = v > best ? v : best;
            }
        }
        float gv = g[i];
        for (int ky = 0; ky < d.k; ++ky) {
            int iy = yo * d.stride + ky - d.pad;
            if (iy < 0 || iy >= d.h) continue;
            for (int kx = 0; kx < d.k; ++kx) {
                int ix = xo * d.stride + kx - d.pad;
                if (ix < 0 || ix >= d.w) continue;
                long long idx = (nc * d.h + iy) * d.w + ix;
                if (x[idx] == best) {
                    atomicAdd(dx + idx, gv);
                    break;
                }
            }
        }
    }
}

// The same rule read from the input's side, for reproducible runs with overlapping windows (stride < kernel): one
// thread per input element visits the windows that cover it in (yo, xo) order and takes a window's gradient when the
// element is that window's maximum and the first such element of its window row.  One writer per element, additions in
// a fixed order, no zero fill.
__global__ void max_pool_bwd_gather_kernel(const float *__restrict__ x, const float *__restrict__ g, float *__restrict__ dx, PoolDims d) {
    long long total = (long long)d.nc * d.h * d.w;
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    long long step = (long long)gridDim.x * blockDim.x;
    for (; i < total; i += step) {
        const int ix = (int)(i % d.w), iy = (int)((i / d.w) % d.h);
        const long long nc = i / ((long long)d.w * d.h);
        const float v = x[i];
        int yo0 = iy + d.pad - d.k + 1, xo0 = ix + d.pad - d.k + 1;
        yo0 = yo0 <= 0 ? 0 : (yo0 + d.stride - 1) / d.stride;
        xo0 = xo0 <= 0 ? 0 : (xo0 + d.stride - 1) / d.stride;
        const int yo1 = min((iy + d.pad) / d.stride, d.oh - 1), xo1 = min((ix + d.pad) / d.stride, d.ow - 1);
        float acc = 0.0f;
        for (int yo = yo0; yo <= yo1; ++yo)
            for (int xo = xo0; xo <= xo1; ++xo) {
                float best = -INFINITY;
                for (int ky = 0; ky < d.k; ++ky) {
                    const int wy = yo * d.stride + ky - d.pad;
                    if (wy < 0 || wy >= d.h) continue;
                    for (int kx = 0; kx < d.k; ++kx) {
                        const int wx = xo * d.stride + kx - d.pad;
                        if (wx < 0 || wx >= d.w) continue;
                        const float u = x[(nc * d.h + wy) * d.w + wx];
                        best = u > best ? u : best;
                    }
                }
                if (!(v == best)) continue;
                bool first = true;
                for (int wx = max(xo * d.stride - d.pad, 0); wx < ix; ++wx) first = first && !(x[(nc * d.h + iy) * d.w + wx] == best);
                if (first) acc += g[(nc * d.oh + yo) * d.ow + xo];
            }
        dx[i] = acc;
    }
}

mcb_status make_conv_dims(mcb_ctx *ctx, ConvDims &d, int64_t n, int64_t c, int64_t h, int64_t wd, int64_t o, int64_t kh,
                          int64_t kw, int64_t stride, int64_t pad) {
    if (stride <= 0 || pad < 0 || h + 2 * pad < kh || wd + 2 * pad < kw)
        return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "conv2d: kernel larger than the padded input or bad stride");
    d.n = (int)n; d.c = (int)c; d.h = (int)h; d.w = (int)wd; d.o = (int)o; d.kh = (int)kh; d.kw = (int)kw;
    d.stride = (int)stride; d.pad = (int)pad;
    d.oh = (int)((h + 2 * pad - kh) / stride + 1);
    d.ow = (int)((wd + 2 * pad - kw) / stride + 1);
    return MCB_OK;
}

} // namespace

extern "C" {

mcb_status mcb_conv2d(mcb_ctx *ctx, const float *x, const float *w, const float *bias, float *out, int64_t n,
                      int64_t c, int64_t h, int64_t wd, int64_t o, int64_t kh, int64_t kw, int64_t stride,
                      int64_t pad) {
    MCB_CHECK_CTX(ctx);
    ConvDims d;
    MCB_TRY(make_conv_dims(ctx, d, n, c, h, wd, o, kh, kw, stride, pad));
    long long total = (long long)d.n * d.o * d.oh * d.ow;
    if (total == 0) return MCB_OK;
    // large convolutions: column matrix + tensor-core GEMMs at f32 accuracy (conv_tc.cu); small ones: direct kernels
    if (mcb_conv_tc_eligible(ctx, n, c, h, wd, o, kh, kw, stride, pad)) return mcb_conv_tc_forward(ctx, x, w, bias, out, n, c, h, wd, o, kh, kw, stride, pad);
    ProfScope prof(ctx, MCB_PROF_CONV, 2.0 * (double)total * d.c * d.kh * d.kw, 4.0 * ((double)n * c * h * wd + (double)total));
    conv2d_fwd_kernel<<<mcb_grid_for(ctx, total, 256, 16), 256, 0, ctx->stream>>>(x, w, bias, out, d);
    MCB_LAUNCHED(ctx);
    return MCB_OK;
}

mcb_status mcb_conv2d_backward(mcb_ctx *ctx, const float *x, const float *w, const float *g, float *dx, float *dw,
                               float *db, int64_t n, int64_t c, int64_t h, int64_t wd, int64_t o, int64_t kh,
                               int64_t kw, int64_t stride, int64_t pad) {
    MCB_CHECK_CTX(ctx);
    ConvDims d;
    MCB_TRY(make_conv_dims(ctx, d, n, c, h, wd, o, kh, kw, stride, pad));
    long long nx = (long long)d.n * d.c * d.h * d.w, nw = (long long)d.o * d.c * d.kh * d.kw;
    if (mcb_conv_tc_eligible(ctx, n, c, h, wd, o, kh, kw, stride, pad) && nx && nw) {
        MCB_TRY(mcb_conv_tc_backward(ctx, x, w, g, dx, dw, n, c, h, wd, o, kh, kw, stride, pad));
        dx = nullptr;
        dw = nullptr; // the bias gradient below is a plain reduction in either case
    }
    ProfScope prof(ctx, MCB_PROF_CONV, 2.0 * (double)d.n * d.o * d.oh * d.ow * d.c * d.kh * d.kw * ((dx ? 1 : 0) + (dw ? 1 : 0)),
                   4.0 * ((double)nx * (dx ? 2 : 1) + (double)d.n * d.o * d.oh * d.ow));
    if (dx && nx) {
        conv2d_dx_kernel<<<mcb_grid_for(ctx, nx, 256, 16), 256, 0, ctx->stream>>>(g, w, dx, d);
        MCB_LAUNCHED(ctx);
    }
    if (dw && nw) {
        conv2d_dw_kernel<<<(unsigned)nw, 256, 0, ctx->stream>>>(x, g, dw, d);
        MCB_LAUNCHED(ctx);
    }
    if (db && d.o) {
        int parts = (ctx->sm_count * 4 + d.o - 1) / d.o;
        if (parts > d.n) parts = d.n;
        if (parts < 1) parts = 1;
        void *scratch;
        MCB_TRY(mcb_scratch(ctx, sizeof(float) * (size_t)parts * d.o, &scratch));
        conv2d_db_partial_kernel<<<dim3((unsigned)d.o, (unsigned)parts), 256, 0, ctx->stream>>>(g, (float *)scratch, d);
        MCB_LAUNCHED(ctx);
        conv2d_db_final_kernel<<<(d.o + 127) / 128, 128, 0, ctx->stream>>>((const float *)scratch, parts, d.o, db);
        MCB_LAUNCHED(ctx);
    }
    return MCB_OK;
}

mcb_status mcb_max_pool2d(mcb_ctx *ctx, const float *x, float *out, int64_t n, int64_t c, int64_t h, int64_t w,
                          int64_t kernel, int64_t stride, int64_t pad) {
    MCB_CHECK_CTX(ctx);
    if (stride <= 0 || h + 2 * pad < kernel || w + 2 * pad < kernel) return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "pool2d: window larger than the padded input");
    PoolDims d{(int)(n * c), (int)h, (int)w, (int)kernel, (int)stride, (int)pad, (int)((h + 2 * pad - kernel) / stride + 1),
               (int)((w + 2 * pad - kernel) / stride + 1)};
    long long total = (long long)d.nc * d.oh * d.ow;
    if (total == 0) return MCB_OK;
    max_pool_fwd_kernel<<<mcb_grid_for(ctx, total, 256, 16), 256, 0, ctx->stream>>>(x, out, d);
    MCB_LAUNCHED(ctx);
    return MCB_OK;
}

mcb_status mcb_max_pool2d_backward(mcb_ctx *ctx, const float *x, const float *g, float *dx, int64_t n, int64_t c,
                                   int64_t h, int64_t w, int64_t kernel, int64_t stride, int64_t pad) {
    MCB_CHECK_CTX(ctx);
    if (stride <= 0 || h + 2 * pad < kernel || w + 2 * pad < kernel) return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "pool2d: window larger than the padded input");
    PoolDims d{(int)(n * c), (int)h, (int)w, (int)kernel, (int)stride, (int)pad, (int)((h + 2 * pad - kernel) / stride + 1),
               (int)((w + 2 * pad - kernel) / stride + 1)};
    if (knob_on(ctx, K_DETERMINISTIC) && stride < kernel) { // overlapping windows would meet in float atomics
        const long long cells = (long long)d.nc * d.h * d.w;
        if (cells == 0) return MCB_OK;
        max_pool_bwd_gather_kernel<<<mcb_grid_for(ctx, cells, 256, 16), 256, 0, ctx->stream>>>(x, g, dx, d);
        MCB_LAUNCHED(ctx);
        return MCB_OK;
    }
    MCB_TRY(mcb_memset(ctx, dx, 0, sizeof(float) * n * c * h * w));
    long long total = (long long)d.nc * d.oh * d.ow;
    if (total == 0) return MCB_OK;
    max_pool_bwd_kernel<<<mcb_grid_for(ctx, total, 256, 16), 256, 0, ctx->stream>>>(x, g, dx, d);
    MCB_LAUNCHED(ctx);
    return MCB_OK;
}

} // extern "C"
