// Elementwise kernels of the training path: binary ops with broadcast, scale, fill,
// unary maps, ReLU / GELU forward and fused backward, casts, in-place accumulate.
// All HBM-bound: 128-bit accesses on the aligned bulk, grid sized in multiples of the
// SM count, grid-stride loops.
#include "common.cuh"
#include "internal.h"

namespace {

constexpr int kThreads = 256;

struct BinDims {
    int rank;
    long long od[8];
    long long as[8]; // element strides of a per output dim (0 where broadcast)
    long long bs[8];
};

template <int OP> __device__ __forceinline__ float bin_op(float x, float y) {
    if (OP == MCB_ADD) return x + y;
    if (OP == MCB_SUB) return x - y;
    if (OP == MCB_MUL) return x * y;
    return x / y;
}

// mode 0: same shape; 1: b is a row vector [cols] against a [rows, cols]; 2: b scalar; 3: a scalar; 4: a row vector
template <int OP>
__global__ void binary_fast_kernel(const float *__restrict__ a, const float *__restrict__ b, float *__restrict__ out,
                                   long long n, long long cols, int mode) {
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    long long stride = (long long)gridDim.x * blockDim.x;
    if (mode == 0 && (n & 3) == 0) {
        long long n4 = n >> 2;
        for (; i < n4; i += stride) {
            float4 x = reinterpret_cast<const float4 *>(a)[i], y = reinterpret_cast<const float4 *>(b)[i], r;
            r.x = bin_op<OP>(x.x, y.x);
            r.y = bin_op<OP>(x.y, y.y);
            r.z = bin_op<OP>(x.z, y.z);
            r.w = bin_op<OP>(x.w, y.w);
            reinterpret_cast<float4 *>(out)[i] = r;
        }
        return;
    }
    for (; i < n; i += stride) {
        float x, y;
        switch (mode) {
        case 0: x = a[i]; y = b[i]; break;
        case 1: x = a[i]; y = b[i % cols]; break;
        case 2: x = a[i]; y = b[0]; break;
        case 3: x = a[0]; y = b[i]; break;
        default: x = a[i % cols]; y = b[i]; break;
        }
        out[i] = bin_op<OP>(x, y);
    }
}

template <int OP>
__global__ void binary_generic_kernel(const float *__restrict__ a, const float *__restrict__ b,
                                      float *__restrict__ out, long long n, BinDims d) {
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    long long stride = (long long)gridDim.x * blockDim.x;
    for (; i < n; i += stride) {
        long long rest = i, ao = 0, bo = 0;
        for (int k = d.rank - 1; k >= 0; --k) {
            long long c = rest % d.od[k];
            rest /= d.od[k];
            ao += c * d.as[k];
            bo += c * d.bs[k];
        }
        out[i] = bin_op<OP>(a[ao], b[bo]);
    }
}

template <typename T> __global__ void add_inplace_kernel(T *__restrict__ dst, const T *__restrict__ src, long long n, int vec) {
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    long long stride = (long long)gridDim.x * blockDim.x;
    long long n4 = vec ? (n >> 2) : 0;
    for (long long j = i; j < n4; j += stride) {
        float4 x = Elem<T>::ld4(dst, j), y = Elem<T>::ld4(src, j);
        Elem<T>::st4(dst, j, make_float4(x.x + y.x, x.y + y.y, x.z + y.z, x.w + y.w));
    }
    for (long long j = (n4 << 2) + i; j < n; j += stride) Elem<T>::st(dst, j, Elem<T>::ld(dst, j) + Elem<T>::ld(src, j));
}

__global__ void scale_kernel(const float *__restrict__ x, float f, float *__restrict__ out, long long n, int vec) {
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    long long stride = (long long)gridDim.x * blockDim.x;
    long long n4 = vec ? (n >> 2) : 0;
    for (long long j = i; j < n4; j += stride) {
        float4 v = reinterpret_cast<const float4 *>(x)[j];
        reinterpret_cast<float4 *>(out)[j] = make_float4(v.x * f, v.y * f, v.z * f, v.w * f);
    }
    for (long long j = (n4 << 2) + i; j < n; j += stride) out[j] = x[j] * f;
}

__global__ void fill_kernel(float *__restrict__ out, float v, long long n) {
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    long long stride = (long long)gridDim.x * blockDim.x;
    for (; i < n; i += stride) out[i] = v;
}

__global__ void unary_kernel(int op, const float *__restrict__ x, float *__restrict__ out, long long n) {
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    long long stride = (long long)gridDim.x * blockDim.x;
    for (; i < n; i += stride) {
        float v = x[i], r;
        switch (op) {
        case MCB_EXP: r = expf(v); break;
        case MCB_LOG: r = logf(v); break;
        case MCB_SIGMOID: r = 1.0f / (1.0f + expf(-v)); break;
        case MCB_SQRT: r = sqrtf(v); break;
        case MCB_SILU: r = v / (1.0f + expf(-v)); break;
        case MCB_ABS: r = fabsf(v); break;
        default: r = -v; break;
        }
        out[i] = r;
    }
}

// ---- activations ----------------------------------------------------------------
struct ReluF {
    static __device__ __forceinline__ float f(float x) { return x > 0.0f ? x : 0.0f; } // NaN -> 0 like f32::max(x, 0)
};
struct GeluF {
    // 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3))), all f32 (cpu/src/kernels.rs:1384-1389)
    static __device__ __forceinline__ float f(float v) {
        const float k = 0.7978845608028654f;
        float v3 = v * v * v;
        return 0.5f * v * (1.0f + tanhf(k * (v + 0.044715f * v3)));
    }
};
struct ReluB {
    static __device__ __forceinline__ float f(float x, float g) { return x > 0.0f ? g : 0.0f; }
};
struct GeluB {
    // d/dx of the tanh form, evaluated with a real tanh.  The reference composes tanh from
    // exp(-2c), which overflows to NaN for x below about -10; this kernel stays finite there.
    static __device__ __forceinline__ float f(float x, float g) {
        const float k = 0.7978845608028654f;
        float xx = x * x;
        float c = k * (x + 0.044715f * xx * x);
        float th = tanhf(c);
        float phi = 0.5f * (1.0f + th);
        float dphi = 0.5f * (1.0f - th * th);
        float coeff = k * (1.0f + 0.044715f * 3.0f * xx);
        return g * (phi + x * dphi * coeff);
    }
};
// The same derivative for bf16 storage: the hardware tanh approximation (relative error about
// 2^-11) is below the bf16 resolution of the result and keeps the kernel bound by memory, not by
// the multi-instruction tanhf.
struct GeluBLowp {
    static __device__ __forceinline__ float f(float x, float g) {
        const float k = 0.7978845608028654f;
        float xx = x * x;
        float c = k * (x + 0.044715f * xx * x);
        float th;
        asm("tanh.approx.f32 %0, %1;" : "=f"(th) : "f"(c));
        float phi = 0.5f * (1.0f + th);
        float dphi = 0.5f * (1.0f - th * th);
        float coeff = k * (1.0f + 0.044715f * 3.0f * xx);
        return g * (phi + x * dphi * coeff);
    }
};

template <typename T, typename Fn> __global__ void map1_kernel(const T *__restrict__ x, T *__restrict__ out, long long n, int vec) {
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    long long stride = (long long)gridDim.x * blockDim.x;
    long long n4 = vec ? (n >> 2) : 0;
    for (long long j = i; j < n4; j += stride) {
        float4 v = Elem<T>::ld4(x, j);
        Elem<T>::st4(out, j, make_float4(Fn::f(v.x), Fn::f(v.y), Fn::f(v.z), Fn::f(v.w)));
    }
    for (long long j = (n4 << 2) + i; j < n; j += stride) Elem<T>::st(out, j, Fn::f(Elem<T>::ld(x, j)));
}

template <typename T, typename Fn>
__global__ void map2_kernel(const T *__restrict__ x, const T *__restrict__ g, T *__restrict__ out, long long n, int vec) {
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    long long stride = (long long)gridDim.x * blockDim.x;
    long long n4 = vec ? (n >> 2) : 0;
    for (long long j = i; j < n4; j += stride) {
        float4 v = Elem<T>::ld4(x, j), w = Elem<T>::ld4(g, j);
        Elem<T>::st4(out, j, make_float4(Fn::f(v.x, w.x), Fn::f(v.y, w.y), Fn::f(v.z, w.z), Fn::f(v.w, w.w)));
    }
    for (long long j = (n4 << 2) + i; j < n; j += stride) Elem<T>::st(out, j, Fn::f(Elem<T>::ld(x, j), Elem<T>::ld(g, j)));
}

// ---- casts ------------------------------------------------------------------------
template <typename S, typename D> __device__ __forceinline__ D cast_one(S v);
template <> __device__ __forceinline__ __nv_bfloat16 cast_one<float, __nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half cast_one<float, __half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ float cast_one<__nv_bfloat16, float>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float cast_one<__half, float>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float cast_one<float, float>(float v) { return v; }

template <typename S, typename D> __global__ void cast_kernel(const S *__restrict__ src, D *__restrict__ dst, long long n) {
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    long long stride = (long long)gridDim.x * blockDim.x;
    for (; i < n; i += stride) dst[i] = cast_one<S, D>(src[i]);
}
template <typename T> __global__ void cast_f32_lp_vec_kernel(const float *__restrict__ src, T *__restrict__ dst, long long n4) {
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    long long stride = (long long)gridDim.x * blockDim.x;
    for (; i < n4; i += stride) Elem<T>::st4(dst, i, reinterpret_cast<const float4 *>(src)[i]);
}
template <typename T> __global__ void cast_lp_f32_vec_kernel(const T *__restrict__ src, float *__restrict__ dst, long long n4) {
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    long long stride = (long long)gridDim.x * blockDim.x;
    for (; i < n4; i += stride) reinterpret_cast<float4 *>(dst)[i] = Elem<T>::ld4(src, i);
}

template <typename Fn>
mcb_status launch_map1(mcb_ctx *ctx, const void *x, void *out, int64_t n, int32_t dt) {
    if (n == 0) return MCB_OK;
    int vec = mcb_aligned16(x) && mcb_aligned16(out);
    ProfScope prof(ctx, MCB_PROF_ELEMENTWISE, 0.0, (double)n * 2.0 * (mcb_is_lp(dt) ? 2.0 : 4.0));
    int grid = mcb_grid_for(ctx, (n + 3) / 4, kThreads);
    if (dt == MCB_F32)
        map1_kernel<float, Fn><<<grid, kThreads, 0, ctx->stream>>>((const float *)x, (float *)out, n, vec);
    else if (dt == MCB_BF16)
        map1_kernel<__nv_bfloat16, Fn><<<grid, kThreads, 0, ctx->stream>>>((const __nv_bfloat16 *)x, (__nv_bfloat16 *)out, n, vec);
    else if (dt == MCB_F16)
        map1_kernel<__half, Fn><<<grid, kThreads, 0, ctx->stream>>>((const __half *)x, (__half *)out, n, vec);
    else
        return mcb_fail(ctx, MCB_UNSUPPORTED_DTYPE, "activation supports f32, bf16 and f16 storage");
    MCB_LAUNCHED(ctx);
    return MCB_OK;
}
template <typename Fn>
mcb_status launch_map2(mcb_ctx *ctx, const void *x, const void *g, void *out, int64_t n, int32_t dt) {
    if (n == 0) return MCB_OK;
    int vec = mcb_aligned16(x) && mcb_aligned16(g) && mcb_aligned16(out);
    ProfScope prof(ctx, MCB_PROF_ELEMENTWISE, 0.0, (double)n * 3.0 * (mcb_is_lp(dt) ? 2.0 : 4.0));
    int grid = mcb_grid_for(ctx, (n + 3) / 4, kThreads);
    if (dt == MCB_F32)
        map2_kernel<float, Fn><<<grid, kThreads, 0, ctx->stream>>>((const float *)x, (const float *)g, (float *)out, n, vec);
    else if (dt == MCB_BF16)
        map2_kernel<__nv_bfloat16, Fn><<<grid, kThreads, 0, ctx->stream>>>((const __nv_bfloat16 *)x, (const __nv_bfloat16 *)g,
                                                                           (__nv_bfloat16 *)out, n, vec);
    else if (dt == MCB_F16)
        map2_kernel<__half, Fn><<<grid, kThreads, 0, ctx->stream>>>((const __half *)x, (const __half *)g, (__half *)out, n, vec);
    else
        return mcb_fail(ctx, MCB_UNSUPPORTED_DTYPE, "activation backward supports f32, bf16 and f16 storage");
    MCB_LAUNCHED(ctx);
    return MCB_OK;
}

// ---- a bf16 [rows, cols] result and its column sums in one pass (the bias gradient of a Linear
// is the column sum of exactly the bf16 gradient its GEMMs read, so both come from one read).
//   MODE 0: out = T(a)               a f32            (cast of an f32 gradient)
//   MODE 1: out = gelu'(a) * b       a = pre-activation, b = upstream gradient, both of type T (bf16 or f16)
//   MODE 2: out = relu'(a) * b
// Lane l of a warp owns columns blockIdx.x*256 + 8l .. +7; the 8 warps of a block take rows
// r0+w, r0+w+8, ...; partial[blockIdx.y][col] receives the block's sum of the ROUNDED outputs.
template <int MODE, typename T>
__global__ void __launch_bounds__(256, 6) map_colsum_kernel(const void *__restrict__ a, const void *__restrict__ b,
                                                         T *__restrict__ out, long long rows, long long cols,
                                                         float *__restrict__ partial) {
    __shared__ float red[8][32][9];
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const long long col = (long long)blockIdx.x * 256 + lane * 8;
    const long long rows_per = (rows + gridDim.y - 1) / gridDim.y;
    const long long r0 = (long long)blockIdx.y * rows_per, r1 = r0 + rows_per < rows ? r0 + rows_per : rows;
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.0f;
    dep_wait();
    dep_trigger();
    if (col < cols) {
#pragma unroll 2
        for (long long r = r0 + w; r < r1; r += 8) {
            const long long e = r * cols + col;
            float v[8];
            if (MODE == 0) {
                const float4 *p = reinterpret_cast<const float4 *>((const float *)a + e);
                float4 lo = p[0], hi = p[1];
                v[0] = lo.x; v[1] = lo.y; v[2] = lo.z; v[3] = lo.w;
                v[4] = hi.x; v[5] = hi.y; v[6] = hi.z; v[7] = hi.w;
            } else {
                uint4 xa = *reinterpret_cast<const uint4 *>((const T *)a + e);
                uint4 xb = *reinterpret_cast<const uint4 *>((const T *)b + e);
                const uint32_t *pa = reinterpret_cast<const uint32_t *>(&xa);
                const uint32_t *pb = reinterpret_cast<const uint32_t *>(&xb);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float2 fa = Lp<T>::unpack2(pa[j]), fb = Lp<T>::unpack2(pb[j]);
                    v[2 * j] = MODE == 1 ? GeluBLowp::f(fa.x, fb.x) : ReluB::f(fa.x, fb.x);
                    v[2 * j + 1] = MODE == 1 ? GeluBLowp::f(fa.y, fb.y) : ReluB::f(fa.y, fb.y);
                }
            }
            uint4 o;
            uint32_t *po = reinterpret_cast<uint32_t *>(&o);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                po[j] = Lp<T>::pack2(v[2 * j], v[2 * j + 1]);
                float2 back = Lp<T>::unpack2(po[j]);
                acc[2 * j] += back.x;
                acc[2 * j + 1] += back.y;
            }
            *reinterpret_cast<uint4 *>(out + e) = o;
        }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) red[w][lane][j] = acc[j];
    __syncthreads();
    // 256 threads = 256 columns of this block: thread t sums column t over the 8 warps
    const int cl = threadIdx.x >> 3, cj = threadIdx.x & 7;
    const long long c = (long long)blockIdx.x * 256 + threadIdx.x;
    if (c < cols) {
        float t = 0.0f;
#pragma unroll
        for (int y = 0; y < 8; ++y) t += red[y][cl][cj];
        partial[(long long)blockIdx.y * cols + c] = t;
    }
}

template <int OP>
mcb_status launch_binary(mcb_ctx *ctx, const float *a, const int64_t *ad, int ar, const float *b, const int64_t *bd,
                         int br, float *out) {
    int r = ar > br ? ar : br;
    BinDims d;
    d.rank = r;
    long long n = 1, an = 1, bn = 1;
    for (int i = 0; i < ar; ++i) an *= ad[i];
    for (int i = 0; i < br; ++i) bn *= bd[i];
    long long astr = 1, bstr = 1;
    for (int i = r - 1; i >= 0; --i) {
        long long x = (i >= r - ar) ? ad[i - (r - ar)] : 1;
        long long y = (i >= r - br) ? bd[i - (r - br)] : 1;
        long long o;
        if (x == y) o = x;
        else if (x == 1) o = y;
        else if (y == 1) o = x;
        else return mcb_fail(ctx, MCB_BROADCAST, "shapes do not broadcast");
        d.od[i] = o;
        d.as[i] = (x == 1) ? 0 : astr;
        d.bs[i] = (y == 1) ? 0 : bstr;
        astr *= x;
        bstr *= y;
        n *= o;
    }
    if (n == 0) return MCB_OK;
    int mode = -1;
    long long cols = 1;
    if (an == n && bn == n) mode = 0;
    else if (bn == 1 && an == n) mode = 2;
    else if (an == 1 && bn == n) mode = 3;
    else if (an == n && br >= 1 && bn == bd[br - 1] && d.od[r - 1] == bn) { mode = 1; cols = bn; }
    else if (bn == n && ar >= 1 && an == ad[ar - 1] && d.od[r - 1] == an) { mode = 4; cols = an; }
    if (mode == 0 && !(mcb_aligned16(a) && mcb_aligned16(b) && mcb_aligned16(out))) mode = 1, cols = n; // scalar path
    int grid = mcb_grid_for(ctx, mode == 0 ? (n + 3) / 4 : n, kThreads);
    if (mode >= 0)
        binary_fast_kernel<OP><<<grid, kThreads, 0, ctx->stream>>>(a, b, out, n, cols, mode);
    else
        binary_generic_kernel<OP><<<grid, kThreads, 0, ctx->stream>>>(a, b, out, n, d);
    MCB_LAUNCHED(ctx);
    return MCB_OK;
}

} // namespace

extern "C" {

mcb_status mcb_binary(mcb_ctx *ctx, int32_t op, const float *a, const int64_t *a_dims, int32_t a_rank,
                      const float *b, const int64_t *b_dims, int32_t b_rank, float *out) {
    MCB_CHECK_CTX(ctx);
    if (a_rank > 8 || b_rank > 8 || a_rank < 0 || b_rank < 0) return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "rank > 8");
    switch (op) {
    case MCB_ADD: return launch_binary<MCB_ADD>(ctx, a, a_dims, a_rank, b, b_dims, b_rank, out);
    case MCB_SUB: return launch_binary<MCB_SUB>(ctx, a, a_dims, a_rank, b, b_dims, b_rank, out);
    case MCB_MUL: return launch_binary<MCB_MUL>(ctx, a, a_dims, a_rank, b, b_dims, b_rank, out);
    case MCB_DIV: return launch_binary<MCB_DIV>(ctx, a, a_dims, a_rank, b, b_dims, b_rank, out);
    default: return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "unknown binary op %d", op);
    }
}

mcb_status mcb_add_inplace(mcb_ctx *ctx, void *dst, const void *src, int64_t n, int32_t dt) {
    MCB_CHECK_CTX(ctx);
    if (n == 0) return MCB_OK;
    int vec = mcb_aligned16(dst) && mcb_aligned16(src);
    ProfScope prof(ctx, MCB_PROF_ELEMENTWISE, 0.0, (double)n * 3.0 * (mcb_is_lp(dt) ? 2.0 : 4.0));
    int grid = mcb_grid_for(ctx, (n + 3) / 4, kThreads);
    if (dt == MCB_F32)
        add_inplace_kernel<float><<<grid, kThreads, 0, ctx->stream>>>((float *)dst, (const float *)src, n, vec);
    else if (dt == MCB_BF16)
        add_inplace_kernel<__nv_bfloat16><<<grid, kThreads, 0, ctx->stream>>>((__nv_bfloat16 *)dst, (const __nv_bfloat16 *)src, n, vec);
    else if (dt == MCB_F16)
        add_inplace_kernel<__half><<<grid, kThreads, 0, ctx->stream>>>((__half *)dst, (const __half *)src, n, vec);
    else
        return mcb_fail(ctx, MCB_UNSUPPORTED_DTYPE, "add_inplace supports f32, bf16 and f16");
    MCB_LAUNCHED(ctx);
    return MCB_OK;
}

mcb_status mcb_scale(mcb_ctx *ctx, const float *x, double factor, float *out, int64_t n) {
    MCB_CHECK_CTX(ctx);
    if (n == 0) return MCB_OK;
    scale_kernel<<<mcb_grid_for(ctx, (n + 3) / 4, kThreads), kThreads, 0, ctx->stream>>>(x, (float)factor, out, n, mcb_aligned16(x) && mcb_aligned16(out));
    MCB_LAUNCHED(ctx);
    return MCB_OK;
}

mcb_status mcb_fill(mcb_ctx *ctx, float *out, float value, int64_t n) {
    MCB_CHECK_CTX(ctx);
    if (n == 0) return MCB_OK;
    fill_kernel<<<mcb_grid_for(ctx, n, kThreads), kThreads, 0, ctx->stream>>>(out, value, n);
    MCB_LAUNCHED(ctx);
    return MCB_OK;
}

mcb_status mcb_unary(mcb_ctx *ctx, int32_t op, const float *x, float *out, int64_t n) {
    MCB_CHECK_CTX(ctx);
    if (op < MCB_EXP || op > MCB_NEG) return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "unknown unary op %d", op);
    if (n == 0) return MCB_OK;
    unary_kernel<<<mcb_grid_for(ctx, n, kThreads), kThreads, 0, ctx->stream>>>(op, x, out, n);
    MCB_LAUNCHED(ctx);
    return MCB_OK;
}

mcb_status mcb_relu(mcb_ctx *ctx, const void *x, void *out, int64_t n, int32_t dt) {
    MCB_CHECK_CTX(ctx);
    return launch_map1<ReluF>(ctx, x, out, n, dt);
}
mcb_status mcb_relu_backward(mcb_ctx *ctx, const void *x, const void *g, void *out, int64_t n, int32_t dt) {
    MCB_CHECK_CTX(ctx);
    return launch_map2<ReluB>(ctx, x, g, out, n, dt);
}
mcb_status mcb_gelu(mcb_ctx *ctx, const void *x, void *out, int64_t n, int32_t dt) {
    MCB_CHECK_CTX(ctx);
    return launch_map1<GeluF>(ctx, x, out, n, dt);
}
mcb_status mcb_gelu_backward(mcb_ctx *ctx, const void *x, const void *g, void *out, int64_t n, int32_t dt) {
    MCB_CHECK_CTX(ctx);
    if (mcb_is_lp(dt)) return launch_map2<GeluBLowp>(ctx, x, g, out, n, dt);
    return launch_map2<GeluB>(ctx, x, g, out, n, dt);
}

mcb_status mcb_cast(mcb_ctx *ctx, const void *src, int32_t src_dt, void *dst, int32_t dst_dt, int64_t n) {
    MCB_CHECK_CTX(ctx);
    if (n == 0) return MCB_OK;
    int grid = mcb_grid_for(ctx, n, kThreads);
    bool vec = (n & 3) == 0 && mcb_aligned16(src) && mcb_aligned16(dst);
    if (src_dt == MCB_F32 && dst_dt == MCB_BF16) {
        if (vec)
            cast_f32_lp_vec_kernel<__nv_bfloat16><<<mcb_grid_for(ctx, n / 4, kThreads), kThreads, 0, ctx->stream>>>((const float *)src, (__nv_bfloat16 *)dst, n / 4);
        else
            cast_kernel<float, __nv_bfloat16><<<grid, kThreads, 0, ctx->stream>>>((const float *)src, (__nv_bfloat16 *)dst, n);
    } else if (src_dt == MCB_BF16 && dst_dt == MCB_F32) {
        if (vec)
            cast_lp_f32_vec_kernel<__nv_bfloat16><<<mcb_grid_for(ctx, n / 4, kThreads), kThreads, 0, ctx->stream>>>((const __nv_bfloat16 *)src, (float *)dst, n / 4);
        else
            cast_kernel<__nv_bfloat16, float><<<grid, kThreads, 0, ctx->stream>>>((const __nv_bfloat16 *)src, (float *)dst, n);
    } else if (src_dt == MCB_F32 && dst_dt == MCB_F16) {
        if (vec)
            cast_f32_lp_vec_kernel<__half><<<mcb_grid_for(ctx, n / 4, kThreads), kThreads, 0, ctx->stream>>>((const float *)src, (__half *)dst, n / 4);
        else
            cast_kernel<float, __half><<<grid, kThreads, 0, ctx->stream>>>((const float *)src, (__half *)dst, n);
    } else if (src_dt == MCB_F16 && dst_dt == MCB_F32) {
        if (vec)
            cast_lp_f32_vec_kernel<__half><<<mcb_grid_for(ctx, n / 4, kThreads), kThreads, 0, ctx->stream>>>((const __half *)src, (float *)dst, n / 4);
        else
            cast_kernel<__half, float><<<grid, kThreads, 0, ctx->stream>>>((const __half *)src, (float *)dst, n);
    } else if (src_dt == MCB_F32 && dst_dt == MCB_F32) {
        cast_kernel<float, float><<<grid, kThreads, 0, ctx->stream>>>((const float *)src, (float *)dst, n);
    } else {
        return mcb_fail(ctx, MCB_UNSUPPORTED_DTYPE, "cast %d -> %d is not supported", src_dt, dst_dt);
    }
    MCB_LAUNCHED(ctx);
    return MCB_OK;
}

} // extern "C"

namespace {
__global__ void fill_from_scalar_kernel(float *__restrict__ out, const float *__restrict__ scalar, double factor, long long n) {
    // product in f64, then narrowed (Ops::full_like_scalar, crates/modern-chainer-core/src/storage.rs:337-345)
    float v = (float)((double)scalar[0] * factor);
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    long long stride = (long long)gridDim.x * blockDim.x;
    for (; i < n; i += stride) out[i] = v;
}
template <typename T>
__global__ void mul_scalar_ptr_kernel(const T *__restrict__ x, const float *__restrict__ scalar, T *__restrict__ out, long long n) {
    float f = scalar[0];
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    long long stride = (long long)gridDim.x * blockDim.x;
    for (; i < n; i += stride) Elem<T>::st(out, i, Elem<T>::ld(x, i) * f);
}
template <typename A, typename B, typename O>
__global__ void add_typed_kernel(const A *__restrict__ a, const B *__restrict__ b, O *__restrict__ out, long long n, int vec) {
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    long long stride = (long long)gridDim.x * blockDim.x;
    long long n4 = vec ? (n >> 2) : 0;
    dep_wait();
    dep_trigger();
    for (long long j = i; j < n4; j += stride) {
        float4 x = Elem<A>::ld4(a, j), y = Elem<B>::ld4(b, j);
        Elem<O>::st4(out, j, make_float4(x.x + y.x, x.y + y.y, x.z + y.z, x.w + y.w));
    }
    for (long long j = (n4 << 2) + i; j < n; j += stride) Elem<O>::st(out, j, Elem<A>::ld(a, j) + Elem<B>::ld(b, j));
}
template <typename A, typename B, typename O>
void launch_add_typed(mcb_ctx *ctx, const void *a, const void *b, void *out, long long n) {
    int vec = mcb_aligned16(a) && mcb_aligned16(b) && mcb_aligned16(out);
    (void)mcb_launch_dep(ctx, add_typed_kernel<A, B, O>, dim3(mcb_grid_for(ctx, (n + 3) / 4, kThreads)), dim3(kThreads), 0, (const A *)a, (const B *)b,
                         (O *)out, n, vec); // a launch error is picked up by the caller's MCB_LAUNCHED
}
} // namespace

mcb_status mcb_fill_from_scalar(mcb_ctx *ctx, float *out, const float *scalar, double factor, int64_t n) {
    if (n == 0) return MCB_OK;
    fill_from_scalar_kernel<<<mcb_grid_for(ctx, n, kThreads), kThreads, 0, ctx->stream>>>(out, scalar, factor, n);
    MCB_LAUNCHED(ctx);
    return MCB_OK;
}

mcb_status mcb_mul_scalar_ptr(mcb_ctx *ctx, const void *x, const float *scalar, void *out, int64_t n, int32_t dt) {
    if (n == 0) return MCB_OK;
    int grid = mcb_grid_for(ctx, n, kThreads);
    if (dt == MCB_F32)
        mul_scalar_ptr_kernel<float><<<grid, kThreads, 0, ctx->stream>>>((const float *)x, scalar, (float *)out, n);
    else if (dt == MCB_BF16)
        mul_scalar_ptr_kernel<__nv_bfloat16><<<grid, kThreads, 0, ctx->stream>>>((const __nv_bfloat16 *)x, scalar, (__nv_bfloat16 *)out, n);
    else if (dt == MCB_F16)
        mul_scalar_ptr_kernel<__half><<<grid, kThreads, 0, ctx->stream>>>((const __half *)x, scalar, (__half *)out, n);
    else
        return mcb_fail(ctx, MCB_UNSUPPORTED_DTYPE, "scalar multiply supports f32, bf16 and f16");
    MCB_LAUNCHED(ctx);
    return MCB_OK;
}

mcb_status mcb_add_typed(mcb_ctx *ctx, const void *a, int32_t a_dt, const void *b, int32_t b_dt, void *out, int32_t out_dt, int64_t n) {
    if (n == 0) return MCB_OK;
    typedef __nv_bfloat16 bf;
    if (a_dt == MCB_F32 && b_dt == MCB_F32 && out_dt == MCB_F32) launch_add_typed<float, float, float>(ctx, a, b, out, n);
    else if (a_dt == MCB_F32 && b_dt == MCB_BF16 && out_dt == MCB_F32) launch_add_typed<float, bf, float>(ctx, a, b, out, n);
    else if (a_dt == MCB_BF16 && b_dt == MCB_F32 && out_dt == MCB_F32) launch_add_typed<bf, float, float>(ctx, a, b, out, n);
    else if (a_dt == MCB_BF16 && b_dt == MCB_BF16 && out_dt == MCB_BF16) launch_add_typed<bf, bf, bf>(ctx, a, b, out, n);
    else if (a_dt == MCB_BF16 && b_dt == MCB_BF16 && out_dt == MCB_F32) launch_add_typed<bf, bf, float>(ctx, a, b, out, n);
    else if (a_dt == MCB_F32 && b_dt == MCB_F16 && out_dt == MCB_F32) launch_add_typed<float, __half, float>(ctx, a, b, out, n);
    else if (a_dt == MCB_F16 && b_dt == MCB_F32 && out_dt == MCB_F32) launch_add_typed<__half, float, float>(ctx, a, b, out, n);
    else if (a_dt == MCB_F16 && b_dt == MCB_F16 && out_dt == MCB_F16) launch_add_typed<__half, __half, __half>(ctx, a, b, out, n);
    else if (a_dt == MCB_F16 && b_dt == MCB_F16 && out_dt == MCB_F32) launch_add_typed<__half, __half, float>(ctx, a, b, out, n);
    else return mcb_fail(ctx, MCB_UNSUPPORTED_DTYPE, "typed add: unsupported storage combination");
    MCB_LAUNCHED(ctx);
    return MCB_OK;
}

bool mcb_map_colsum_supported(const void *a, const void *b, const void *out, int64_t cols) {
    return cols > 0 && cols % 8 == 0 && mcb_aligned16(a) && (!b || mcb_aligned16(b)) && mcb_aligned16(out);
}

namespace {
template <typename T>
cudaError_t launch_map_colsum(mcb_ctx *ctx, int mode, dim3 grid, const void *a, const void *b, void *out, long long rows, long long cols, float *scratch) {
    T *o = (T *)out;
    if (mode == 0) return mcb_launch_dep(ctx, map_colsum_kernel<0, T>, grid, dim3(256), 0, a, b, o, rows, cols, scratch);
    if (mode == 1) return mcb_launch_dep(ctx, map_colsum_kernel<1, T>, grid, dim3(256), 0, a, b, o, rows, cols, scratch);
    return mcb_launch_dep(ctx, map_colsum_kernel<2, T>, grid, dim3(256), 0, a, b, o, rows, cols, scratch);
}
} // namespace

mcb_status mcb_map_colsum(mcb_ctx *ctx, int mode, const void *a, const void *b, void *out_bf16, int64_t rows, int64_t cols,
                          float *colsum_out, int32_t lp_dt) {
    if (!mcb_map_colsum_supported(a, b, out_bf16, cols)) return MCB_UNSUPPORTED;
    if (mode < 0 || mode > 2) return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "map_colsum: unknown mode %d", mode);
    if (!mcb_is_lp(lp_dt)) return mcb_fail(ctx, MCB_UNSUPPORTED_DTYPE, "map_colsum writes bf16 or f16");
    if (rows == 0) return mcb_memset(ctx, colsum_out, 0, sizeof(float) * cols);
    double bytes = (double)rows * cols * (mode == 0 ? 6.0 : 6.0);
    ProfScope prof(ctx, MCB_PROF_ELEMENTWISE, 0.0, bytes);
    int chunks = (int)((cols + 255) / 256);
    int splits = (ctx->sm_count * 6 + chunks - 1) / chunks; // 256-thread blocks, about six per SM
    if (splits > (rows + 15) / 16) splits = (int)((rows + 15) / 16);
    if (splits < 1) splits = 1;
    void *scratch;
    MCB_TRY(mcb_scratch(ctx, sizeof(float) * (size_t)splits * cols, &scratch));
    dim3 grid(chunks, splits);
    if (lp_dt == MCB_BF16) MCB_CUDA(ctx, launch_map_colsum<__nv_bfloat16>(ctx, mode, grid, a, b, out_bf16, rows, cols, (float *)scratch));
    else MCB_CUDA(ctx, launch_map_colsum<__half>(ctx, mode, grid, a, b, out_bf16, rows, cols, (float *)scratch));
    MCB_LAUNCHED(ctx);
    return mcb_partial_sum_final(ctx, (const float *)scratch, splits, cols, colsum_out);
}
