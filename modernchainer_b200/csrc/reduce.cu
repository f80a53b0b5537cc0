// Reduction kernels of the training path: sum_all, sum_to / bias-gradient column sums,
// softmax, LayerNorm forward/backward, softmax-cross-entropy (separate and fused),
// embedding gather / scatter-add.  Row reductions use warp shuffles; cross-row
// reductions are two-stage through a scratch buffer so results do not depend on
// scheduling (no float atomics except the embedding scatter).
#include "common.cuh"
#include <cstdio>

#include "internal.h"

namespace {

constexpr int kThreads = 256;

// ------------------------------------------------------------------ sum_all
__global__ void sum_partial_kernel(const float *__restrict__ x, long long n, double *__restrict__ partial) {
    __shared__ double red[kThreads / 32];
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    long long stride = (long long)gridDim.x * blockDim.x;
    float acc = 0.0f;
    double accd = 0.0;
    int cnt = 0;
    for (; i < n; i += stride) {
        acc += x[i];
        if (++cnt == 64) { // bound the f32 run length, then carry on in f64
            accd += (double)acc;
            acc = 0.0f;
            cnt = 0;
        }
    }
    accd += (double)acc;
    for (int o = 16; o > 0; o >>= 1) accd += __shfl_xor_sync(0xffffffffu, accd, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = accd;
    __syncthreads();
    if (threadIdx.x == 0) {
        double t = 0.0;
        for (int w = 0; w < kThreads / 32; ++w) t += red[w];
        partial[blockIdx.x] = t;
    }
}
// out = (float)(scale * sum(partial[0..m))) in fixed order
__global__ void sum_final_kernel(const double *__restrict__ partial, int m, double scale, float *__restrict__ out) {
    if (threadIdx.x == 0 && blockIdx.x == 0) {
        double t = 0.0;
        for (int i = 0; i < m; ++i) t += partial[i];
        out[0] = (float)(t * scale);
    }
}

// ------------------------------------------------------------------ column sums
// grid (ceil(cols/32), splits), block (32, 8).  partial[split][col].
template <typename T>
__global__ void col_sum_partial_kernel(const T *__restrict__ a, long long rows, long long cols, float *__restrict__ partial) {
    __shared__ float tile[8][33];
    long long col = (long long)blockIdx.x * 32 + threadIdx.x;
    long long rows_per = (rows + gridDim.y - 1) / gridDim.y;
    long long r0 = (long long)blockIdx.y * rows_per, r1 = r0 + rows_per < rows ? r0 + rows_per : rows;
    float acc = 0.0f;
    if (col < cols)
        for (long long r = r0 + threadIdx.y; r < r1; r += 8) acc += Elem<T>::ld(a, r * cols + col);
    tile[threadIdx.y][threadIdx.x] = acc;
    __syncthreads();
    if (threadIdx.y == 0 && col < cols) {
        float t = 0.0f;
#pragma unroll
        for (int y = 0; y < 8; ++y) t += tile[y][threadIdx.x];
        partial[(long long)blockIdx.y * cols + col] = t;
    }
}
// grid (ceil(cols/128), splits), block 256 = 8 warps; lane l of every warp owns columns chunk*128 + 4l .. +3
template <typename T>
__global__ void __launch_bounds__(256) col_sum_vec_kernel(const T *__restrict__ a, long long rows, long long cols,
                                                          float *__restrict__ partial) {
    __shared__ float4 red[8][32];
    int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    long long col = (long long)blockIdx.x * 128 + lane * 4;
    long long rows_per = (rows + gridDim.y - 1) / gridDim.y;
    long long r0 = (long long)blockIdx.y * rows_per, r1 = r0 + rows_per < rows ? r0 + rows_per : rows;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    dep_wait();
    dep_trigger();
    if (col < cols) {
        long long c4 = col >> 2, ld4 = cols >> 2;
#pragma unroll 4
        for (long long r = r0 + w; r < r1; r += 8) {
            float4 v = Elem<T>::ld4(a, r * ld4 + c4);
            acc.x += v.x;
            acc.y += v.y;
            acc.z += v.z;
            acc.w += v.w;
        }
    }
    red[w][lane] = acc;
    __syncthreads();
    if (w == 0 && col < cols) {
        float4 t = red[0][lane];
#pragma unroll
        for (int y = 1; y < 8; ++y) {
            float4 u = red[y][lane];
            t.x += u.x;
            t.y += u.y;
            t.z += u.z;
            t.w += u.w;
        }
        reinterpret_cast<float4 *>(partial + (long long)blockIdx.y * cols)[col >> 2] = t;
    }
}
// out[col] = sum over `parts` partial rows, in a fixed order; block (32, 8): 32 columns, 8 interleaved part groups
__global__ void partial_sum_final_kernel(const float *__restrict__ partial, int parts, long long cols, float *__restrict__ out) {
    __shared__ float red[32][33];
    long long col = (long long)blockIdx.x * 32 + threadIdx.x;
    const int groups = blockDim.y; // 8 or 32 interleaved groups of partial rows
    float t = 0.0f;
    dep_wait();
    dep_trigger();
    if (col < cols) {
#pragma unroll 4
        for (int s = threadIdx.y; s < parts; s += groups) t += partial[(long long)s * cols + col];
    }
    red[threadIdx.y][threadIdx.x] = t;
    __syncthreads();
    if (threadIdx.y == 0 && col < cols) {
        float u = 0.0f;
        for (int y = 0; y < groups; ++y) u += red[y][threadIdx.x];
        out[col] = u;
    }
}
__global__ void col_sum_final_kernel(const float *__restrict__ partial, int splits, long long cols, float *__restrict__ out) {
    long long col = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (col >= cols) return;
    float t = 0.0f;
    for (int s = 0; s < splits; ++s) t += partial[(long long)s * cols + col];
    out[col] = t;
}

// ------------------------------------------------------------------ generic sum_to
// one thread per output element, walking the reduced sub-space
struct SumToWalk {
    int out_rank;        // kept dims
    long long kd[8];     // kept dim sizes (in source order)
    long long ks[8];     // source stride of each kept dim
    int red_rank;
    long long rd[8];     // reduced dim sizes
    long long rs[8];     // source stride of each reduced dim
};
__global__ void sum_to_walk_kernel(const float *__restrict__ a, SumToWalk w, long long n_out, long long n_red,
                                   float *__restrict__ out) {
    long long o = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (o >= n_out) return;
    long long rest = o, base = 0;
    for (int k = w.out_rank - 1; k >= 0; --k) {
        long long c = rest % w.kd[k];
        rest /= w.kd[k];
        base += c * w.ks[k];
    }
    float acc = 0.0f;
    for (long long r = 0; r < n_red; ++r) {
        long long rr = r, off = base;
        for (int k = w.red_rank - 1; k >= 0; --k) {
            long long c = rr % w.rd[k];
            rr /= w.rd[k];
            off += c * w.rs[k];
        }
        acc += a[off];
    }
    out[o] = acc;
}

// ------------------------------------------------------------------ softmax
// Row softmax and its backward with ONE pass over global memory per operand: a row is read once with 128-bit loads
// into shared memory, reduced there (warp shuffles for rows of up to 1024 columns, one warp each, while eight such rows
// fit 48 KB; a whole block for wider rows) and written once.  The backward takes either x (the trait's signature: the probabilities are
// rebuilt in shared memory, one exp per element) or the forward's output y, which the tape keeps, so that
// dx = y (g - sum(y g)) costs no exponential at all.
template <int GROUP> __device__ __forceinline__ float group_sum(float v, float *red) {
    if (GROUP == 32) return warp_sum(v);
    return block_sum(v, red);
}
template <int GROUP> __device__ __forceinline__ float group_max(float v, float *red) {
    if (GROUP == 32) return warp_max(v);
    return block_max(v, red);
}
// copies row `src` (cols floats) into shared `dst`; `vec`: 16-byte aligned and cols % 4 == 0
template <int GROUP> __device__ __forceinline__ void load_row(float *dst, const float *__restrict__ src, int cols, int lane, bool vec) {
    if (vec) {
        const float4 *s4 = reinterpret_cast<const float4 *>(src);
        float4 *d4 = reinterpret_cast<float4 *>(dst);
        for (int j = lane; j < (cols >> 2); j += GROUP) d4[j] = s4[j];
    } else {
        for (int j = lane; j < cols; j += GROUP) dst[j] = src[j];
    }
}
template <int GROUP> __device__ __forceinline__ void store_row(float *__restrict__ dst, const float *src, int cols, int lane, bool vec) {
    if (vec) {
        const float4 *s4 = reinterpret_cast<const float4 *>(src);
        float4 *d4 = reinterpret_cast<float4 *>(dst);
        for (int j = lane; j < (cols >> 2); j += GROUP) d4[j] = s4[j];
    } else {
        for (int j = lane; j < cols; j += GROUP) dst[j] = src[j];
    }
}

// MODE 0: out = softmax(a);  MODE 1: out = backward from x (a = x, b = g);  MODE 2: backward from y (a = y, b = g)
// GROUP 32: one warp per row, 8 rows per block; GROUP 256: one block per row.  Shared memory: rows_per_block * pitch floats
// for a (and the same again for g in the backward modes).
template <int GROUP, int MODE>
__global__ void __launch_bounds__(256) softmax_rows_kernel(const float *__restrict__ a, const float *__restrict__ b, float *__restrict__ out,
                                                           long long rows, int cols, int pitch, int vec) {
    extern __shared__ __align__(16) float srow[];
    __shared__ float red[32];
    constexpr int kRowsPerBlock = 256 / GROUP;
    const int sub = threadIdx.x / GROUP, lane = threadIdx.x % GROUP;
    const long long row = (long long)blockIdx.x * kRowsPerBlock + sub;
    const bool live = row < rows; // a block-wide group (GROUP 256) always has a live row; idle warps of the last block skip
    if (GROUP == 32 && !live) return;
    float *sa = srow + (size_t)sub * pitch, *sg = srow + (size_t)(kRowsPerBlock + sub) * pitch;
    load_row<GROUP>(sa, a + row * cols, cols, lane, vec);
    if (MODE != 0) load_row<GROUP>(sg, b + row * cols, cols, lane, vec);
    if (GROUP == 32) __syncwarp();
    else __syncthreads();
    if (MODE != 2) { // probabilities from the scores, in place in shared memory
        float mx = -INFINITY;
        for (int j = lane; j < cols; j += GROUP) mx = fmaxf(mx, sa[j]);
        mx = group_max<GROUP>(mx, red);
        float sum = 0.0f;
        for (int j = lane; j < cols; j += GROUP) {
            const float e = expf(sa[j] - mx);
            sa[j] = e;
            sum += e;
        }
        sum = group_sum<GROUP>(sum, red);
        const float inv = 1.0f / sum;
        for (int j = lane; j < cols; j += GROUP) sa[j] *= inv;
    }
    if (MODE != 0) {
        float dot = 0.0f;
        for (int j = lane; j < cols; j += GROUP) dot = fmaf(sa[j], sg[j], dot);
        dot = group_sum<GROUP>(dot, red);
        for (int j = lane; j < cols; j += GROUP) sa[j] = sa[j] * (sg[j] - dot);
    }
    if (GROUP == 32) __syncwarp();
    else __syncthreads();
    store_row<GROUP>(out + row * cols, sa, cols, lane, vec);
}

// rows wider than the shared-memory staging allows: three sweeps over global memory (block per row)
__global__ void softmax_wide_kernel(const float *__restrict__ x, const float *__restrict__ g, float *__restrict__ out, long long cols, int mode) {
    __shared__ float red[32];
    const float *s = x + (long long)blockIdx.x * cols;
    const float *gr = g ? g + (long long)blockIdx.x * cols : nullptr;
    float *d = out + (long long)blockIdx.x * cols;
    float mx = 0.0f, inv = 1.0f;
    if (mode != 2) {
        mx = -INFINITY;
        for (long long j = threadIdx.x; j < cols; j += blockDim.x) mx = fmaxf(mx, s[j]);
        mx = block_max(mx, red);
        float sum = 0.0f;
        for (long long j = threadIdx.x; j < cols; j += blockDim.x) sum += expf(s[j] - mx);
        inv = 1.0f / block_sum(sum, red);
    }
    auto prob = [&](long long j) { return mode == 2 ? s[j] : expf(s[j] - mx) * inv; };
    if (mode == 0) {
        for (long long j = threadIdx.x; j < cols; j += blockDim.x) d[j] = prob(j);
        return;
    }
    float dot = 0.0f;
    for (long long j = threadIdx.x; j < cols; j += blockDim.x) dot = fmaf(prob(j), gr[j], dot);
    dot = block_sum(dot, red);
    for (long long j = threadIdx.x; j < cols; j += blockDim.x) d[j] = prob(j) * (gr[j] - dot);
}

// ------------------------------------------------------------------ layer norm
// one warp per row; the row is read from L1/L2 on the second and third sweep.
template <typename OutT>
__global__ void layer_norm_kernel(const float *__restrict__ x, const float *__restrict__ gamma,
                                  const float *__restrict__ beta, float eps, OutT *__restrict__ out,
                                  float *__restrict__ mean_out, float *__restrict__ rstd_out, long long rows, int dim,
                                  int vec) {
    int lane = threadIdx.x & 31;
    long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
    float inv_dim = 1.0f / (float)dim;
    for (long long r = warp; r < rows; r += nwarps) {
        const float *s = x + r * dim;
        OutT *d = out + r * dim;
        float sum = 0.0f;
        if (vec) {
            for (int j = lane; j < (dim >> 2); j += 32) {
                float4 v = reinterpret_cast<const float4 *>(s)[j];
                sum += (v.x + v.y) + (v.z + v.w);
            }
        } else {
            for (int j = lane; j < dim; j += 32) sum += s[j];
        }
        float mean = warp_sum(sum) * inv_dim;
        float var = 0.0f;
        if (vec) {
            for (int j = lane; j < (dim >> 2); j += 32) {
                float4 v = reinterpret_cast<const float4 *>(s)[j];
                float a = v.x - mean, b = v.y - mean, c = v.z - mean, e = v.w - mean;
                var += (a * a + b * b) + (c * c + e * e);
            }
        } else {
            for (int j = lane; j < dim; j += 32) {
                float a = s[j] - mean;
                var += a * a;
            }
        }
        var = warp_sum(var) * inv_dim;
        float rstd = 1.0f / sqrtf(var + eps);
        if (lane == 0) {
            if (mean_out) mean_out[r] = mean;
            if (rstd_out) rstd_out[r] = rstd;
        }
        if (vec) {
            for (int j = lane; j < (dim >> 2); j += 32) {
                float4 v = reinterpret_cast<const float4 *>(s)[j];
                float4 ga = reinterpret_cast<const float4 *>(gamma)[j], be = reinterpret_cast<const float4 *>(beta)[j];
                float4 o = make_float4((v.x - mean) * rstd * ga.x + be.x, (v.y - mean) * rstd * ga.y + be.y,
                                       (v.z - mean) * rstd * ga.z + be.z, (v.w - mean) * rstd * ga.w + be.w);
                Elem<OutT>::st4(d, j, o);
            }
        } else {
            for (int j = lane; j < dim; j += 32) Elem<OutT>::st(d, j, (s[j] - mean) * rstd * gamma[j] + beta[j]);
        }
    }
}

// dx per row plus per-warp partial sums of dgamma / dbeta kept in shared memory:
// smem layout [warps][2][dim]; each block writes its reduced slice to partial[block][2][dim].
template <typename GT>
__global__ void layer_norm_backward_kernel(const float *__restrict__ x, const float *__restrict__ gamma,
                                           const GT *__restrict__ g, float eps, const float *__restrict__ mean_in,
                                           const float *__restrict__ rstd_in, float *__restrict__ dx,
                                           float *__restrict__ partial, long long rows, int dim) {
    extern __shared__ float acc[]; // [warps][2][dim]
    int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
    float *my_dg = acc + (size_t)w * 2 * dim, *my_db = my_dg + dim;
    for (int j = lane; j < dim; j += 32) {
        my_dg[j] = 0.0f;
        my_db[j] = 0.0f;
    }
    long long warp = (long long)blockIdx.x * nw + w;
    long long nwarps = (long long)gridDim.x * nw;
    float fdim = (float)dim, inv_dim = 1.0f / fdim;
    for (long long r = warp; r < rows; r += nwarps) {
        const float *s = x + r * dim;
        const GT *gs = g + r * dim;
        float mean, rstd;
        if (mean_in && rstd_in) {
            mean = mean_in[r];
            rstd = rstd_in[r];
        } else {
            float sum = 0.0f;
            for (int j = lane; j < dim; j += 32) sum += s[j];
            mean = warp_sum(sum) * inv_dim;
            float var = 0.0f;
            for (int j = lane; j < dim; j += 32) {
                float a = s[j] - mean;
                var += a * a;
            }
            rstd = 1.0f / sqrtf(warp_sum(var) * inv_dim + eps);
        }
        float sum_dy = 0.0f, sum_dy_norm = 0.0f;
        for (int j = lane; j < dim; j += 32) {
            float gv = Elem<GT>::ld(gs, j);
            float norm = (s[j] - mean) * rstd;
            float dy = gv * gamma[j];
            sum_dy += dy;
            sum_dy_norm += dy * norm;
            my_dg[j] += gv * norm;
            my_db[j] += gv;
        }
        sum_dy = warp_sum(sum_dy);
        sum_dy_norm = warp_sum(sum_dy_norm);
        for (int j = lane; j < dim; j += 32) {
            float gv = Elem<GT>::ld(gs, j);
            float norm = (s[j] - mean) * rstd;
            float dy = gv * gamma[j];
            dx[r * dim + j] = (fdim * dy - sum_dy - norm * sum_dy_norm) * rstd * inv_dim;
        }
    }
    __syncthreads();
    float *dst = partial + (size_t)blockIdx.x * 2 * dim;
    for (int j = threadIdx.x; j < 2 * dim; j += blockDim.x) {
        float t = 0.0f;
        for (int ww = 0; ww < nw; ++ww) t += acc[(size_t)ww * 2 * dim + j];
        dst[j] = t;
    }
}
__global__ void layer_norm_params_final_kernel(const float *__restrict__ partial, int blocks, int dim,
                                               float *__restrict__ dgamma, float *__restrict__ dbeta) {
    int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= 2 * dim) return;
    float t = 0.0f;
    for (int b = 0; b < blocks; ++b) t += partial[(size_t)b * 2 * dim + j];
    if (j < dim) dgamma[j] = t;
    else dbeta[j - dim] = t;
}

// ------------------------------------------------------------------ softmax cross entropy
// exp for softmax rows: full-precision expf for f32 logits (1e-5 parity with the CPU), the
// hardware exp2 approximation for bf16 logits, whose own rounding is 2^-8
template <typename T> __device__ __forceinline__ float row_exp(float v);
template <> __device__ __forceinline__ float row_exp<float>(float v) { return expf(v); }
template <> __device__ __forceinline__ float row_exp<__nv_bfloat16>(float v) { return __expf(v); }
template <> __device__ __forceinline__ float row_exp<__half>(float v) { return __expf(v); }
// pair of 16-bit logits packed in one word -> two floats (float rows never take these paths)
template <typename T> __device__ __forceinline__ float2 lp_unpack(uint32_t w) { return Lp<T>::unpack2(w); }
template <> __device__ __forceinline__ float2 lp_unpack<float>(uint32_t) { return make_float2(0.0f, 0.0f); }
template <typename T> __device__ __forceinline__ uint32_t lp_pack(float a, float b) { return Lp<T>::pack2(a, b); }
template <> __device__ __forceinline__ uint32_t lp_pack<float>(float, float) { return 0u; }

// per-thread online (max, sum) merged across the block
template <typename T>
__device__ __forceinline__ void row_max_sumexp(const T *__restrict__ row, long long c, float *red, float &mx_out,
                                               float &sum_out) {
    float m = -INFINITY, s = 0.0f;
    // 4 elements per load when the row is wide and aligned: one running-max update per group
    bool vec = ((c & 3) == 0) && ((reinterpret_cast<uintptr_t>(row) & (4 * sizeof(T) - 1)) == 0);
    bool vec8 = sizeof(T) == 2 && ((c & 7) == 0) && ((reinterpret_cast<uintptr_t>(row) & 15) == 0);
    if (vec8) {
        // bf16 rows: 16-byte loads, 8 logits per thread per step
        const uint4 *r8 = reinterpret_cast<const uint4 *>(row);
#pragma unroll 4
        for (long long j = threadIdx.x; j < (c >> 3); j += blockDim.x) {
            uint4 raw = r8[j];
            float f[8];
            unsigned wds[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float2 pr = lp_unpack<T>(wds[q]);
                f[2 * q] = pr.x;
                f[2 * q + 1] = pr.y;
            }
            float gm = fmaxf(fmaxf(fmaxf(f[0], f[1]), fmaxf(f[2], f[3])), fmaxf(fmaxf(f[4], f[5]), fmaxf(f[6], f[7])));
            if (gm > m) {
                s *= row_exp<T>(m - gm);
                m = gm;
            }
            // exp(f - m) as one FMA and one ex2 per logit (this loop is bound by instruction issue, not by HBM)
            const float nml = -m * 1.4426950408889634f;
            float part = 0.0f;
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                float e;
                asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(fmaf(f[q], 1.4426950408889634f, nml)));
                part += e;
            }
            s += part;
        }
    } else if (vec) {
        for (long long j = threadIdx.x; j < (c >> 2); j += blockDim.x) {
            float4 v = Elem<T>::ld4(row, j);
            float gm = fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w));
            if (gm > m) {
                s *= row_exp<T>(m - gm);
                m = gm;
            }
            s += (row_exp<T>(v.x - m) + row_exp<T>(v.y - m)) + (row_exp<T>(v.z - m) + row_exp<T>(v.w - m));
        }
    } else {
        for (long long j = threadIdx.x; j < c; j += blockDim.x) {
            float v = Elem<T>::ld(row, j);
            if (v > m) {
                s = s * row_exp<T>(m - v) + 1.0f;
                m = v;
            } else {
                s += row_exp<T>(v - m);
            }
        }
    }
    float M = block_max(m, red);
    float contrib = (m == -INFINITY) ? 0.0f : s * expf(m - M);
    sum_out = block_sum(contrib, red);
    mx_out = M;
}

__global__ void sce_rows_kernel(const float *__restrict__ x, const void *__restrict__ labels, int label_dt,
                                long long c, float *__restrict__ row_loss, unsigned int *err) {
    __shared__ float red[32];
    long long i = blockIdx.x;
    long long lab = load_index(labels, label_dt, i);
    if (lab < 0 || lab >= c) {
        if (threadIdx.x == 0) {
            atomicOr(err, MCB_DEVERR_LABEL);
            row_loss[i] = 0.0f;
        }
        return;
    }
    const float *row = x + i * c;
    float mx, sum;
    row_max_sumexp<float>(row, c, red, mx, sum);
    if (threadIdx.x == 0) row_loss[i] = (mx + logf(sum)) - row[lab];
}
__global__ void sce_final_kernel(const float *__restrict__ row_loss, long long n, float *__restrict__ loss) {
    __shared__ double red[kThreads];
    double acc = 0.0;
    for (long long i = threadIdx.x; i < n; i += blockDim.x) acc += (double)row_loss[i];
    red[threadIdx.x] = acc;
    __syncthreads();
    for (int o = blockDim.x >> 1; o > 0; o >>= 1) {
        if ((int)threadIdx.x < o) red[threadIdx.x] += red[threadIdx.x + o];
        __syncthreads();
    }
    if (threadIdx.x == 0) loss[0] = (float)(red[0] / (double)n);
}
// fused: row loss + in-place gradient, one DRAM read and one DRAM write of the logits
// `out` may alias `x` (each block reads its whole row before it writes any of it).
// `stats_out` / `stats_in` ([n][2]: row maximum, sum of exp): the loss pass of a training step leaves them for the
// gradient pass, which then needs no reduction over the row and streams it once.
template <typename T>
__global__ void __launch_bounds__(512, 3) sce_fused_kernel(const T *x, T *out, const void *__restrict__ labels, int label_dt, long long n,
                                 long long c, float *__restrict__ row_loss, const float *__restrict__ upstream,
                                 unsigned int *err, float *__restrict__ stats_out, const float *__restrict__ stats_in) {
    __shared__ float red[32];
    long long i = blockIdx.x;
    long long lab = load_index(labels, label_dt, i);
    const T *row = x + i * c;
    T *orow = out + i * c;
    if (lab < 0 || lab >= c) {
        if (threadIdx.x == 0) {
            atomicOr(err, MCB_DEVERR_LABEL);
            if (row_loss) row_loss[i] = 0.0f;
        }
        if (out)
            for (long long j = threadIdx.x; j < c; j += blockDim.x) Elem<T>::st(orow, j, 0.0f);
        return;
    }
    float mx, sum;
    if (stats_in) {
        mx = stats_in[2 * i];
        sum = stats_in[2 * i + 1];
    } else {
        row_max_sumexp<T>(row, c, red, mx, sum);
    }
    if (row_loss) { // the label's logit is read before anyone overwrites it
        float at_label = Elem<T>::ld(row, lab);
        __syncthreads();
        if (threadIdx.x == 0) row_loss[i] = (mx + logf(sum)) - at_label;
    }
    if (threadIdx.x == 0 && stats_out) {
        stats_out[2 * i] = mx;
        stats_out[2 * i + 1] = sum;
    }
    if (!out) return; // loss only
    float up = upstream ? upstream[0] : 1.0f;
    float inv_sum = 1.0f / sum, k = up / (float)n;
    bool vec = ((c & 3) == 0) && (((reinterpret_cast<uintptr_t>(row) | reinterpret_cast<uintptr_t>(orow)) & (4 * sizeof(T) - 1)) == 0);
    const bool vec8 = sizeof(T) == 2 && ((c & 7) == 0) && (((reinterpret_cast<uintptr_t>(row) | reinterpret_cast<uintptr_t>(orow)) & 15) == 0);
    if (vec8) {
        // bf16 rows: 16-byte loads and stores, 8 logits per thread per step, several steps in flight
        const uint4 *r8 = reinterpret_cast<const uint4 *>(row);
        uint4 *o8 = reinterpret_cast<uint4 *>(orow);
#pragma unroll 4
        for (long long j = threadIdx.x; j < (c >> 3); j += blockDim.x) {
            const uint4 raw = r8[j];
            const unsigned wds[4] = {raw.x, raw.y, raw.z, raw.w};
            float p[8];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float2 pr = lp_unpack<T>(wds[q]);
                p[2 * q] = row_exp<T>(pr.x - mx) * inv_sum;
                p[2 * q + 1] = row_exp<T>(pr.y - mx) * inv_sum;
            }
            const long long b = j << 3;
            if (lab >= b && lab < b + 8) {
#pragma unroll
                for (int q = 0; q < 8; ++q)
                    if (lab - b == q) p[q] -= 1.0f;
            }
            unsigned ow[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) ow[q] = lp_pack<T>(p[2 * q] * k, p[2 * q + 1] * k);
            o8[j] = make_uint4(ow[0], ow[1], ow[2], ow[3]);
        }
    } else if (vec) {
        for (long long j = threadIdx.x; j < (c >> 2); j += blockDim.x) {
            float4 v = Elem<T>::ld4(row, j);
            long long b = j << 2;
            float4 p = make_float4(row_exp<T>(v.x - mx) * inv_sum, row_exp<T>(v.y - mx) * inv_sum, row_exp<T>(v.z - mx) * inv_sum,
                                   row_exp<T>(v.w - mx) * inv_sum);
            if (lab >= b && lab < b + 4) {
                int o = (int)(lab - b);
                if (o == 0) p.x -= 1.0f;
                else if (o == 1) p.y -= 1.0f;
                else if (o == 2) p.z -= 1.0f;
                else p.w -= 1.0f;
            }
            Elem<T>::st4(orow, j, make_float4(p.x * k, p.y * k, p.z * k, p.w * k));
        }
    } else {
        for (long long j = threadIdx.x; j < c; j += blockDim.x) {
            float p = row_exp<T>(Elem<T>::ld(row, j) - mx) * inv_sum;
            if (j == lab) p -= 1.0f;
            Elem<T>::st(orow, j, p * k);
        }
    }
}

// Gradient pass over bf16 logits whose row statistics are known: nothing is reduced, so the rows are cut into
// segments of 1024 16-byte chunks and every thread streams four of them (all loads issued before the first
// use).  g = (softmax - onehot) * up / n with the softmax as one FMA and one ex2 per logit:
// p = 2^(v * log2e - (mx * log2e + log2(sum))).  `out` may alias `x`: a chunk is written by the thread that read it.
template <typename T>
__global__ void __launch_bounds__(256) sce_grad_stream_kernel(const uint4 *x, uint4 *out, const void *__restrict__ labels, int label_dt,
                                                              long long n, long long c8, const float *__restrict__ stats,
                                                              const float *__restrict__ upstream, unsigned int *err) {
    const long long row = blockIdx.y;
    const long long j0 = (long long)blockIdx.x * 1024 + threadIdx.x;
    const uint4 *r8 = x + row * c8;
    uint4 *o8 = out + row * c8;
    uint4 raw[4];
    dep_wait();
    dep_trigger();
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        const long long j = j0 + u * 256;
        raw[u] = j < c8 ? r8[j] : make_uint4(0u, 0u, 0u, 0u);
    }
    const long long lab = load_index(labels, label_dt, row);
    const bool bad = lab < 0 || lab >= c8 * 8;
    if (bad && blockIdx.x == 0 && threadIdx.x == 0) atomicOr(err, MCB_DEVERR_LABEL);
    const float mx = stats[2 * row], sum = stats[2 * row + 1];
    const float k = (upstream ? upstream[0] : 1.0f) / (float)n;
    const float c1 = -(mx * 1.4426950408889634f + log2f(sum));
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        const long long j = j0 + u * 256;
        if (j >= c8) continue;
        const unsigned wds[4] = {raw[u].x, raw[u].y, raw[u].z, raw[u].w};
        float p[8];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const float2 pr = Lp<T>::unpack2(wds[q]);
            asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(p[2 * q]) : "f"(fmaf(pr.x, 1.4426950408889634f, c1)));
            asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(p[2 * q + 1]) : "f"(fmaf(pr.y, 1.4426950408889634f, c1)));
        }
        const long long b = j << 3;
        if (lab >= b && lab < b + 8) {
#pragma unroll
            for (int q = 0; q < 8; ++q)
                if (lab - b == q) p[q] -= 1.0f;
        }
        unsigned ow[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) ow[q] = bad ? 0u : Lp<T>::pack2(p[2 * q] * k, p[2 * q + 1] * k);
        o8[j] = make_uint4(ow[0], ow[1], ow[2], ow[3]);
    }
}

// ------------------------------------------------------------------ embedding
__global__ void embedding_kernel(const void *__restrict__ ids, int id_dt, long long n, const float *__restrict__ w,
                                 long long vocab, int dim, float *__restrict__ out, unsigned int *err, int vec) {
    int per_row = vec ? (dim >> 2) : dim;
    long long total = n * per_row;
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    long long stride = (long long)gridDim.x * blockDim.x;
    for (; i < total; i += stride) {
        long long r = i / per_row;
        int j = (int)(i - r * per_row);
        long long id = load_index(ids, id_dt, r);
        bool ok = id >= 0 && id < vocab;
        if (!ok && j == 0) atomicOr(err, MCB_DEVERR_INDEX);
        if (vec) {
            float4 v = ok ? reinterpret_cast<const float4 *>(w + id * dim)[j] : make_float4(0.f, 0.f, 0.f, 0.f);
            reinterpret_cast<float4 *>(out + r * dim)[j] = v;
        } else {
            out[r * dim + j] = ok ? w[id * dim + j] : 0.0f;
        }
    }
}
template <typename GT>
__global__ void embedding_backward_kernel(const void *__restrict__ ids, int id_dt, long long n,
                                          const GT *__restrict__ g, long long vocab, int dim, float *__restrict__ out,
                                          unsigned int *err) {
    long long total = n * dim;
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    long long stride = (long long)gridDim.x * blockDim.x;
    for (; i < total; i += stride) {
        long long r = i / dim;
        int j = (int)(i - r * dim);
        long long id = load_index(ids, id_dt, r);
        if (id < 0 || id >= vocab) {
            if (j == 0) atomicOr(err, MCB_DEVERR_INDEX);
            continue;
        }
        atomicAdd(out + id * dim + j, Elem<GT>::ld(g, i));
    }
}

// Position-ordered scatter for reproducible runs.  The block of token i acts only when no earlier token carries the
// same id; it then adds the gradient rows of every token with that id in position order, which is the order of the
// reference's CPU loop (crates/modern-chainer-cpu/src/kernels.rs:1783-1815).  Every output element has one writer and
// a fixed order of additions, so the result does not depend on scheduling.  Each block reads all n ids: a mode for
// reproducibility, not for speed.  The positions that match are kept as a bit mask in shared memory (n / 8 bytes).
constexpr long long kOrderedEmbeddingMaxTokens = 262144; // 32 KB of mask
template <typename GT>
__global__ void __launch_bounds__(256) embedding_backward_ordered_kernel(const void *__restrict__ ids, int id_dt, long long n, const GT *__restrict__ g,
                                                                         long long vocab, int dim, float *__restrict__ out, unsigned int *err) {
    extern __shared__ unsigned int match_bits[];
    const long long i = blockIdx.x;
    const long long id = load_index(ids, id_dt, i);
    if (id < 0 || id >= vocab) {
        if (threadIdx.x == 0) atomicOr(err, MCB_DEVERR_INDEX);
        return;
    }
    int seen = 0;
    for (long long r = threadIdx.x; r < i && !seen; r += blockDim.x) seen = load_index(ids, id_dt, r) == id;
    if (__syncthreads_or(seen)) return;
    const long long words = (n - i + 31) / 32; // bit b of word w: position i + 32 w + b
    for (long long w = threadIdx.x; w < words; w += blockDim.x) {
        unsigned int bits = 0;
        for (int b = 0; b < 32; ++b) {
            const long long r = i + 32 * w + b;
            if (r < n && load_index(ids, id_dt, r) == id) bits |= 1u << b;
        }
        match_bits[w] = bits;
    }
    __syncthreads();
    for (int j = threadIdx.x; j < dim; j += blockDim.x) {
        float acc = out[id * dim + j];
        for (long long w = 0; w < words; ++w) {
            unsigned int bits = match_bits[w];
            while (bits) {
                const int b = __ffs(bits) - 1;
                bits &= bits - 1;
                acc += Elem<GT>::ld(g, (i + 32 * w + b) * dim + j);
            }
        }
        out[id * dim + j] = acc;
    }
}

bool index_dtype_ok(int dt) { return dt == MCB_I64 || dt == MCB_I32 || dt == MCB_U8; }

} // namespace

// mode 0: softmax; 1: backward from x; 2: backward from the forward's output
mcb_status mcb_softmax_rows(mcb_ctx *ctx, int mode, const float *a, const float *b, float *out, int64_t rows, int64_t cols) {
    if (rows == 0 || cols == 0) return MCB_OK;
    const int operands = mode == 0 ? 1 : 2;
    ProfScope prof(ctx, MCB_PROF_REDUCE, 0.0, 4.0 * (double)rows * cols * (operands + 1));
    const int vec = (cols % 4 == 0) && mcb_aligned16(a) && mcb_aligned16(out) && (!b || mcb_aligned16(b));
    const int pitch = (int)((cols + 3) / 4 * 4);
    constexpr size_t kStage = 48 * 1024 - 256; // dynamic shared memory beside the kernel's static 128 bytes
    if (cols <= 1024 && sizeof(float) * 8 * (size_t)pitch * operands <= kStage) { // one warp per row, eight rows per block
        const size_t smem = sizeof(float) * 8 * (size_t)pitch * operands;
        const unsigned grid = (unsigned)((rows + 7) / 8);
        if (mode == 0) softmax_rows_kernel<32, 0><<<grid, 256, smem, ctx->stream>>>(a, b, out, rows, (int)cols, pitch, vec);
        else if (mode == 1) softmax_rows_kernel<32, 1><<<grid, 256, smem, ctx->stream>>>(a, b, out, rows, (int)cols, pitch, vec);
        else softmax_rows_kernel<32, 2><<<grid, 256, smem, ctx->stream>>>(a, b, out, rows, (int)cols, pitch, vec);
    } else if ((size_t)pitch * operands * sizeof(float) <= kStage) { // one block per row
        const size_t smem = sizeof(float) * (size_t)pitch * operands;
        if (mode == 0) softmax_rows_kernel<256, 0><<<(unsigned)rows, 256, smem, ctx->stream>>>(a, b, out, rows, (int)cols, pitch, vec);
        else if (mode == 1) softmax_rows_kernel<256, 1><<<(unsigned)rows, 256, smem, ctx->stream>>>(a, b, out, rows, (int)cols, pitch, vec);
        else softmax_rows_kernel<256, 2><<<(unsigned)rows, 256, smem, ctx->stream>>>(a, b, out, rows, (int)cols, pitch, vec);
    } else {
        softmax_wide_kernel<<<(unsigned)rows, 256, 0, ctx->stream>>>(a, b, out, cols, mode);
    }
    MCB_LAUNCHED(ctx);
    return MCB_OK;
}

extern "C" {

mcb_status mcb_sum_all(mcb_ctx *ctx, const float *x, int64_t n, float *out) {
    MCB_CHECK_CTX(ctx);
    int grid = mcb_grid_for(ctx, n, kThreads, 4);
    void *scratch;
    MCB_TRY(mcb_scratch(ctx, sizeof(double) * grid, &scratch));
    sum_partial_kernel<<<grid, kThreads, 0, ctx->stream>>>(x, n, (double *)scratch);
    MCB_LAUNCHED(ctx);
    sum_final_kernel<<<1, 32, 0, ctx->stream>>>((const double *)scratch, grid, 1.0, out);
    MCB_LAUNCHED(ctx);
    return MCB_OK;
}

mcb_status mcb_col_sum(mcb_ctx *ctx, const void *a, int32_t dt, int64_t rows, int64_t cols, float *out) {
    MCB_CHECK_CTX(ctx);
    if (cols == 0) return MCB_OK;
    if (rows == 0) return mcb_memset(ctx, out, 0, sizeof(float) * cols);
    ProfScope prof(ctx, MCB_PROF_REDUCE, 0.0, (double)rows * cols * (mcb_is_lp(dt) ? 2.0 : 4.0));
    if ((cols % 4) == 0 && mcb_aligned16(a) && (dt == MCB_F32 || mcb_is_lp(dt))) {
        // wide path: each lane owns 4 consecutive columns (one 8/16-byte load per row), a warp 128 columns
        int chunks = (int)((cols + 127) / 128);
        int splits = (int)((ctx->sm_count * 4 + chunks - 1) / chunks);
        if (splits > (rows + 31) / 32) splits = (int)((rows + 31) / 32);
        if (splits < 1) splits = 1;
        void *scratch;
        MCB_TRY(mcb_scratch(ctx, sizeof(float) * splits * cols, &scratch));
        dim3 grid(chunks, splits);
        if (dt == MCB_F32)
            MCB_CUDA(ctx, mcb_launch_dep(ctx, col_sum_vec_kernel<float>, grid, dim3(256), 0, (const float *)a, (long long)rows, (long long)cols, (float *)scratch));
        else if (dt == MCB_BF16)
            MCB_CUDA(ctx, mcb_launch_dep(ctx, col_sum_vec_kernel<__nv_bfloat16>, grid, dim3(256), 0, (const __nv_bfloat16 *)a, (long long)rows,
                                         (long long)cols, (float *)scratch));
        else
            MCB_CUDA(ctx, mcb_launch_dep(ctx, col_sum_vec_kernel<__half>, grid, dim3(256), 0, (const __half *)a, (long long)rows, (long long)cols,
                                         (float *)scratch));
        MCB_LAUNCHED(ctx);
        MCB_CUDA(ctx, mcb_launch_dep(ctx, partial_sum_final_kernel, dim3((unsigned)((cols + 31) / 32)), dim3(32, 32), 0, (const float *)scratch, splits,
                                     (long long)cols, out));
        MCB_LAUNCHED(ctx);
        return MCB_OK;
    }
    int col_tiles = (int)((cols + 31) / 32);
    int splits = (int)((ctx->sm_count * 8 + col_tiles - 1) / col_tiles);
    if (splits > (rows + 63) / 64) splits = (int)((rows + 63) / 64);
    if (splits < 1) splits = 1;
    void *scratch;
    MCB_TRY(mcb_scratch(ctx, sizeof(float) * splits * cols, &scratch));
    dim3 grid(col_tiles, splits), block(32, 8);
    if (dt == MCB_F32)
        col_sum_partial_kernel<float><<<grid, block, 0, ctx->stream>>>((const float *)a, rows, cols, (float *)scratch);
    else if (dt == MCB_BF16)
        col_sum_partial_kernel<__nv_bfloat16><<<grid, block, 0, ctx->stream>>>((const __nv_bfloat16 *)a, rows, cols, (float *)scratch);
    else if (dt == MCB_F16)
        col_sum_partial_kernel<__half><<<grid, block, 0, ctx->stream>>>((const __half *)a, rows, cols, (float *)scratch);
    else
        return mcb_fail(ctx, MCB_UNSUPPORTED_DTYPE, "col_sum supports f32, bf16 and f16");
    MCB_LAUNCHED(ctx);
    col_sum_final_kernel<<<(int)((cols + 255) / 256), 256, 0, ctx->stream>>>((const float *)scratch, splits, cols, out);
    MCB_LAUNCHED(ctx);
    return MCB_OK;
}

mcb_status mcb_sum_to(mcb_ctx *ctx, const float *a, const int64_t *ad, int32_t ar, const int64_t *td, int32_t tr,
                      float *out) {
    MCB_CHECK_CTX(ctx);
    if (tr > ar || ar > 8 || tr < 0) return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "sum_to target rank %d exceeds source rank %d", tr, ar);
    int shift = ar - tr;
    long long n_src = 1, n_out = 1;
    for (int i = 0; i < ar; ++i) n_src *= ad[i];
    for (int i = 0; i < tr; ++i) n_out *= td[i];
    for (int i = 0; i < tr; ++i)
        if (td[i] != 1 && td[i] != ad[i + shift]) return mcb_fail(ctx, MCB_SHAPE_MISMATCH, "sum_to target does not fold the source shape");
    if (n_out == 0) return MCB_OK;
    if (n_src == n_out) return mcb_memcpy_d2d(ctx, out, a, sizeof(float) * n_src); // equal shapes: a copy
    if (n_src == 0) return mcb_memset(ctx, out, 0, sizeof(float) * n_out);
    if (ar == 2 && tr == 1 && td[0] == ad[1]) return mcb_col_sum(ctx, a, MCB_F32, ad[0], ad[1], out);
    if (n_out == 1) return mcb_sum_all(ctx, a, n_src, out);
    // split source dims into kept and reduced
    SumToWalk w;
    w.out_rank = 0;
    w.red_rank = 0;
    long long stride = 1, n_red = 1;
    long long sstr[8];
    for (int i = ar - 1; i >= 0; --i) {
        sstr[i] = stride;
        stride *= ad[i];
    }
    for (int i = 0; i < ar; ++i) {
        bool kept = i >= shift && td[i - shift] != 1;
        if (kept) {
            w.kd[w.out_rank] = ad[i];
            w.ks[w.out_rank++] = sstr[i];
        } else if (ad[i] != 1) {
            w.rd[w.red_rank] = ad[i];
            w.rs[w.red_rank++] = sstr[i];
            n_red *= ad[i];
        }
    }
    sum_to_walk_kernel<<<(int)((n_out + 127) / 128), 128, 0, ctx->stream>>>(a, w, n_out, n_red, out);
    MCB_LAUNCHED(ctx);
    return MCB_OK;
}

mcb_status mcb_softmax(mcb_ctx *ctx, const float *x, float *out, int64_t rows, int64_t cols) {
    MCB_CHECK_CTX(ctx);
    return mcb_softmax_rows(ctx, 0, x, nullptr, out, rows, cols);
}
mcb_status mcb_softmax_backward(mcb_ctx *ctx, const float *x, const float *g, float *out, int64_t rows, int64_t cols) {
    MCB_CHECK_CTX(ctx);
    return mcb_softmax_rows(ctx, 1, x, g, out, rows, cols);
}
mcb_status mcb_softmax_backward_from_output(mcb_ctx *ctx, const float *y, const float *g, float *out, int64_t rows, int64_t cols) {
    MCB_CHECK_CTX(ctx);
    return mcb_softmax_rows(ctx, 2, y, g, out, rows, cols);
}

mcb_status mcb_layer_norm(mcb_ctx *ctx, const float *x, const float *gamma, const float *beta, double eps, void *out,
                          int32_t out_dt, float *mean, float *rstd, int64_t rows, int64_t dim) {
    MCB_CHECK_CTX(ctx);
    if (rows == 0 || dim == 0) return MCB_OK;
    if (dim > INT32_MAX) return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "layer_norm dim too large");
    int vec = (dim % 4 == 0) && mcb_aligned16(x) && mcb_aligned16(out) && mcb_aligned16(gamma) && mcb_aligned16(beta);
    ProfScope prof(ctx, MCB_PROF_NORM, 0.0, (double)rows * dim * (4.0 + (mcb_is_lp(out_dt) ? 2.0 : 4.0)) + 8.0 * rows);
    if (out_dt == MCB_F32 || mcb_is_lp(out_dt)) {
        mcb_status bulk = mcb_ln_bulk_forward(ctx, x, gamma, beta, eps, out, out_dt, mean, rstd, rows, dim);
        if (bulk != MCB_UNSUPPORTED) return bulk; // enough rows to fill every SM: shared-memory pipeline
        mcb_status fast = mcb_ln_fast_forward(ctx, x, gamma, beta, eps, out, out_dt, mean, rstd, rows, dim);
        if (fast != MCB_UNSUPPORTED) return fast; // rows of up to 1024 aligned elements stay in registers
    }
    int grid = mcb_grid_for(ctx, rows, kThreads / 32, 16);
    if (out_dt == MCB_F32)
        layer_norm_kernel<float><<<grid, kThreads, 0, ctx->stream>>>(x, gamma, beta, (float)eps, (float *)out, mean, rstd, rows, (int)dim, vec);
    else if (out_dt == MCB_BF16)
        layer_norm_kernel<__nv_bfloat16><<<grid, kThreads, 0, ctx->stream>>>(x, gamma, beta, (float)eps, (__nv_bfloat16 *)out, mean, rstd, rows, (int)dim, vec);
    else if (out_dt == MCB_F16)
        layer_norm_kernel<__half><<<grid, kThreads, 0, ctx->stream>>>(x, gamma, beta, (float)eps, (__half *)out, mean, rstd, rows, (int)dim, vec);
    else
        return mcb_fail(ctx, MCB_UNSUPPORTED_DTYPE, "layer_norm output must be f32, bf16 or f16");
    MCB_LAUNCHED(ctx);
    return MCB_OK;
}

mcb_status mcb_layer_norm_backward(mcb_ctx *ctx, const float *x, const float *gamma, const void *g, int32_t g_dt,
                                   double eps, const float *mean, const float *rstd, float *dx, float *dgamma,
                                   float *dbeta, int64_t rows, int64_t dim) {
    return mcb_layer_norm_backward_ex(ctx, x, gamma, g, g_dt, eps, mean, rstd, nullptr, dx, dgamma, dbeta, rows, dim);
}

} // extern "C"

// With `addend` (may alias dx) the input gradient is written as addend + dx; only the pipeline and the
// register-resident kernels do that, so other shapes return MCB_UNSUPPORTED before anything is launched.
mcb_status mcb_layer_norm_backward_ex(mcb_ctx *ctx, const float *x, const float *gamma, const void *g, int32_t g_dt, double eps,
                                      const float *mean, const float *rstd, const float *addend, float *dx, float *dgamma,
                                      float *dbeta, int64_t rows, int64_t dim) {
    MCB_CHECK_CTX(ctx);
    if (dim == 0) return MCB_OK;
    if (rows == 0) {
        MCB_TRY(mcb_memset(ctx, dgamma, 0, sizeof(float) * dim));
        return mcb_memset(ctx, dbeta, 0, sizeof(float) * dim);
    }
    // algorithmic bytes: read x and g, write dx, read the row statistics, write 2*dim parameter sums
    ProfScope prof(ctx, MCB_PROF_NORM, 0.0,
                   (double)rows * dim * (8.0 + (mcb_is_lp(g_dt) ? 2.0 : 4.0) + (addend ? 4.0 : 0.0)) + 8.0 * rows + 8.0 * dim);
    if (g_dt == MCB_F32 || mcb_is_lp(g_dt)) {
        mcb_status bulk = mcb_ln_bulk_backward(ctx, x, gamma, g, g_dt, eps, mean, rstd, addend, dx, dgamma, dbeta, rows, dim);
        if (bulk != MCB_UNSUPPORTED) return bulk;
        mcb_status fast = mcb_ln_fast_backward(ctx, x, gamma, g, g_dt, eps, mean, rstd, addend, dx, dgamma, dbeta, rows, dim);
        if (fast != MCB_UNSUPPORTED) return fast;
    }
    if (addend) return MCB_UNSUPPORTED;
    const size_t smem_cap = 200 * 1024;
    int warps = 8;
    while (warps > 1 && (size_t)warps * 2 * dim * sizeof(float) > smem_cap) warps >>= 1;
    size_t smem = (size_t)warps * 2 * dim * sizeof(float);
    if (smem > smem_cap) return mcb_fail(ctx, MCB_UNSUPPORTED, "layer_norm_backward: dim %lld exceeds the shared-memory staging limit", (long long)dim);
    int grid = mcb_grid_for(ctx, rows, warps, 2);
    void *scratch;
    MCB_TRY(mcb_scratch(ctx, sizeof(float) * (size_t)grid * 2 * dim, &scratch));
    if (g_dt == MCB_F32) {
        MCB_CUDA(ctx, cudaFuncSetAttribute(layer_norm_backward_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_cap));
        layer_norm_backward_kernel<float><<<grid, warps * 32, smem, ctx->stream>>>(x, gamma, (const float *)g, (float)eps, mean, rstd, dx, (float *)scratch, rows, (int)dim);
    } else if (g_dt == MCB_BF16) {
        MCB_CUDA(ctx, cudaFuncSetAttribute(layer_norm_backward_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_cap));
        layer_norm_backward_kernel<__nv_bfloat16><<<grid, warps * 32, smem, ctx->stream>>>(x, gamma, (const __nv_bfloat16 *)g, (float)eps, mean, rstd, dx, (float *)scratch, rows, (int)dim);
    } else if (g_dt == MCB_F16) {
        MCB_CUDA(ctx, cudaFuncSetAttribute(layer_norm_backward_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_cap));
        layer_norm_backward_kernel<__half><<<grid, warps * 32, smem, ctx->stream>>>(x, gamma, (const __half *)g, (float)eps, mean, rstd, dx, (float *)scratch, rows, (int)dim);
    } else {
        return mcb_fail(ctx, MCB_UNSUPPORTED_DTYPE, "layer_norm_backward grad must be f32, bf16 or f16");
    }
    MCB_LAUNCHED(ctx);
    layer_norm_params_final_kernel<<<(int)((2 * dim + 255) / 256), 256, 0, ctx->stream>>>((const float *)scratch, grid, (int)dim, dgamma, dbeta);
    MCB_LAUNCHED(ctx);
    return MCB_OK;
}

extern "C" {

mcb_status mcb_softmax_cross_entropy(mcb_ctx *ctx, const float *logits, const void *labels, int32_t label_dt,
                                     int64_t n, int64_t c, float *loss_out) {
    MCB_CHECK_CTX(ctx);
    if (!index_dtype_ok(label_dt)) return mcb_fail(ctx, MCB_UNSUPPORTED_DTYPE, "labels must be i64, i32 or u8");
    if (n == 0) return mcb_memset(ctx, loss_out, 0, sizeof(float));
    void *scratch;
    MCB_TRY(mcb_scratch(ctx, sizeof(float) * n, &scratch));
    int threads = c >= 4096 ? 512 : (c >= 256 ? 128 : 32);
    sce_rows_kernel<<<(unsigned)n, threads, 0, ctx->stream>>>(logits, labels, label_dt, c, (float *)scratch, ctx->d_err);
    MCB_LAUNCHED(ctx);
    sce_final_kernel<<<1, kThreads, 0, ctx->stream>>>((const float *)scratch, n, loss_out);
    MCB_LAUNCHED(ctx);
    return MCB_OK;
}

mcb_status mcb_softmax_cross_entropy_backward(mcb_ctx *ctx, const float *logits, const void *labels,
                                              int32_t label_dt, int64_t n, int64_t c, float *out) {
    MCB_CHECK_CTX(ctx);
    return mcb_sce_grad(ctx, logits, out, MCB_F32, labels, label_dt, n, c, nullptr, nullptr, nullptr, nullptr);
}

mcb_status mcb_softmax_ce_fused(mcb_ctx *ctx, void *logits, int32_t logits_dt, const void *labels, int32_t label_dt,
                                int64_t n, int64_t c, float *loss_out, const float *upstream) {
    MCB_CHECK_CTX(ctx);
    return mcb_sce_grad(ctx, logits, logits, logits_dt, labels, label_dt, n, c, loss_out, upstream, nullptr, nullptr);
}

mcb_status mcb_embedding(mcb_ctx *ctx, const void *ids, int32_t id_dt, int64_t n, const float *weight, int64_t vocab,
                         int64_t dim, float *out) {
    MCB_CHECK_CTX(ctx);
    if (!index_dtype_ok(id_dt)) return mcb_fail(ctx, MCB_UNSUPPORTED_DTYPE, "ids must be i64, i32 or u8");
    if (n == 0 || dim == 0) return MCB_OK;
    int vec = (dim % 4 == 0) && mcb_aligned16(weight) && mcb_aligned16(out);
    long long total = n * (vec ? dim / 4 : dim);
    embedding_kernel<<<mcb_grid_for(ctx, total, kThreads), kThreads, 0, ctx->stream>>>(ids, id_dt, n, weight, vocab, (int)dim, out, ctx->d_err, vec);
    MCB_LAUNCHED(ctx);
    return MCB_OK;
}

mcb_status mcb_embedding_backward(mcb_ctx *ctx, const void *ids, int32_t id_dt, int64_t n, const void *g,
                                  int32_t g_dt, int64_t vocab, int64_t dim, float *out, int32_t accumulate) {
    MCB_CHECK_CTX(ctx);
    if (!index_dtype_ok(id_dt)) return mcb_fail(ctx, MCB_UNSUPPORTED_DTYPE, "ids must be i64, i32 or u8");
    if (!accumulate) MCB_TRY(mcb_memset(ctx, out, 0, sizeof(float) * vocab * dim));
    if (n == 0 || dim == 0) return MCB_OK;
    if (g_dt != MCB_F32 && g_dt != MCB_BF16 && g_dt != MCB_F16) return mcb_fail(ctx, MCB_UNSUPPORTED_DTYPE, "embedding grad must be f32, bf16 or f16");
    if (knob_on(ctx, K_DETERMINISTIC)) {
        if (n > kOrderedEmbeddingMaxTokens)
            return mcb_fail(ctx, MCB_UNSUPPORTED, "deterministic embedding backward takes at most %lld tokens per call", kOrderedEmbeddingMaxTokens);
        const size_t smem = sizeof(unsigned int) * (size_t)((n + 31) / 32);
        if (g_dt == MCB_F32)
            embedding_backward_ordered_kernel<float><<<(unsigned)n, 256, smem, ctx->stream>>>(ids, id_dt, n, (const float *)g, vocab, (int)dim, out, ctx->d_err);
        else if (g_dt == MCB_BF16)
            embedding_backward_ordered_kernel<__nv_bfloat16><<<(unsigned)n, 256, smem, ctx->stream>>>(ids, id_dt, n, (const __nv_bfloat16 *)g, vocab, (int)dim, out, ctx->d_err);
        else
            embedding_backward_ordered_kernel<__half><<<(unsigned)n, 256, smem, ctx->stream>>>(ids, id_dt, n, (const __half *)g, vocab, (int)dim, out, ctx->d_err);
        MCB_LAUNCHED(ctx);
        return MCB_OK;
    }
    int grid = mcb_grid_for(ctx, n * dim, kThreads);
    if (g_dt == MCB_F32)
        embedding_backward_kernel<float><<<grid, kThreads, 0, ctx->stream>>>(ids, id_dt, n, (const float *)g, vocab, (int)dim, out, ctx->d_err);
    else if (g_dt == MCB_BF16)
        embedding_backward_kernel<__nv_bfloat16><<<grid, kThreads, 0, ctx->stream>>>(ids, id_dt, n, (const __nv_bfloat16 *)g, vocab, (int)dim, out, ctx->d_err);
    else if (g_dt == MCB_F16)
        embedding_backward_kernel<__half><<<grid, kThreads, 0, ctx->stream>>>(ids, id_dt, n, (const __half *)g, vocab, (int)dim, out, ctx->d_err);
    else
        return mcb_fail(ctx, MCB_UNSUPPORTED_DTYPE, "embedding grad must be f32, bf16 or f16");
    MCB_LAUNCHED(ctx);
    return MCB_OK;
}

} // extern "C"

// gradient of the mean cross entropy (times *upstream), optionally with the loss, in one pass
mcb_status mcb_sce_grad(mcb_ctx *ctx, const void *logits, void *out, int32_t dt, const void *labels, int32_t label_dt,
                        int64_t n, int64_t c, float *loss_out, const float *upstream, float *stats_out, const float *stats_in) {
    if (!index_dtype_ok(label_dt)) return mcb_fail(ctx, MCB_UNSUPPORTED_DTYPE, "labels must be i64, i32 or u8");
    if (n == 0) return loss_out ? mcb_memset(ctx, loss_out, 0, sizeof(float)) : MCB_OK;
    if (c == 0) return MCB_OK;
    void *scratch = nullptr;
    if (loss_out) MCB_TRY(mcb_scratch(ctx, sizeof(float) * n, &scratch));
    int threads = c >= 4096 ? 512 : (c >= 256 ? 128 : 32);
    // algorithmic bytes: one read of the logits, one write of the gradient when requested
    ProfScope prof(ctx, MCB_PROF_LOSS, 0.0, (double)n * c * (mcb_is_lp(dt) ? 2.0 : 4.0) * (out ? 2.0 : 1.0) + 8.0 * n);
    if (mcb_is_lp(dt) && out && stats_in && !loss_out && !stats_out && (c % 8) == 0 && n <= 65535 && mcb_aligned16(logits) && mcb_aligned16(out) &&
        !knob_on(ctx, K_SCE_NO_STREAM)) {
        // gradient pass with known row statistics: pure streaming
        const long long c8 = c / 8;
        dim3 grid((unsigned)((c8 + 1023) / 1024), (unsigned)n);
        if (dt == MCB_BF16)
            MCB_CUDA(ctx, mcb_launch_dep(ctx, sce_grad_stream_kernel<__nv_bfloat16>, grid, dim3(256), 0, (const uint4 *)logits, (uint4 *)out, labels,
                                         (int)label_dt, (long long)n, c8, stats_in, upstream, ctx->d_err));
        else
            MCB_CUDA(ctx, mcb_launch_dep(ctx, sce_grad_stream_kernel<__half>, grid, dim3(256), 0, (const uint4 *)logits, (uint4 *)out, labels,
                                         (int)label_dt, (long long)n, c8, stats_in, upstream, ctx->d_err));
        MCB_LAUNCHED(ctx);
        return MCB_OK;
    }
    if (dt == MCB_F32)
        sce_fused_kernel<float><<<(unsigned)n, threads, 0, ctx->stream>>>((const float *)logits, (float *)out, labels, label_dt, n, c, (float *)scratch, upstream, ctx->d_err, stats_out, stats_in);
    else if (dt == MCB_BF16)
        sce_fused_kernel<__nv_bfloat16><<<(unsigned)n, threads, 0, ctx->stream>>>((const __nv_bfloat16 *)logits, (__nv_bfloat16 *)out, labels, label_dt, n, c, (float *)scratch, upstream, ctx->d_err, stats_out, stats_in);
    else if (dt == MCB_F16)
        sce_fused_kernel<__half><<<(unsigned)n, threads, 0, ctx->stream>>>((const __half *)logits, (__half *)out, labels, label_dt, n, c, (float *)scratch, upstream, ctx->d_err, stats_out, stats_in);
    else
        return mcb_fail(ctx, MCB_UNSUPPORTED_DTYPE, "logits must be f32, bf16 or f16");
    MCB_LAUNCHED(ctx);
    if (loss_out) {
        sce_final_kernel<<<1, kThreads, 0, ctx->stream>>>((const float *)scratch, n, loss_out);
        MCB_LAUNCHED(ctx);
    }
    return MCB_OK;
}

// out = (float)(scale * sum(x)) as a device scalar
mcb_status mcb_sum_scaled(mcb_ctx *ctx, const float *x, int64_t n, double scale, float *out) {
    int grid = mcb_grid_for(ctx, n > 0 ? n : 1, kThreads, 4);
    void *scratch;
    MCB_TRY(mcb_scratch(ctx, sizeof(double) * grid, &scratch));
    sum_partial_kernel<<<grid, kThreads, 0, ctx->stream>>>(x, n, (double *)scratch);
    MCB_LAUNCHED(ctx);
    sum_final_kernel<<<1, 32, 0, ctx->stream>>>((const double *)scratch, grid, scale, out);
    MCB_LAUNCHED(ctx);
    return MCB_OK;
}

// out[col] = sum of `parts` rows of partial[parts, cols], in a fixed order (used by fused kernels
// in other files that leave per-block column sums in the context's scratch buffer)
mcb_status mcb_partial_sum_final(mcb_ctx *ctx, const float *partial, int parts, int64_t cols, float *out) {
    MCB_CUDA(ctx, mcb_launch_dep(ctx, partial_sum_final_kernel, dim3((unsigned)((cols + 31) / 32)), dim3(32, 32), 0, partial, parts, (long long)cols, out));
    MCB_LAUNCHED(ctx);
    return MCB_OK;
}

// ------------------------------------------------------------------ allocation-free LayerNorm backward
// The regular LayerNorm backward keeps its per-block partial sums of dgamma / dbeta in a scratch
// buffer that the context allocates on demand.  Code that runs where device allocation is off
// limits (a host that hands the library a stream and fixed buffers and forbids cudaMalloc: a
// real-time loop, a plugin inside a process whose memory is fully pre-partitioned, a region that
// is being recorded and must not change the address space) gets this variant instead: the same
// kernels, with the partial sums in a fixed array that is part of the loaded module.
namespace {
constexpr int kNoAllocMaxDim = 4096;   // widest normalised dimension accepted
constexpr int kNoAllocBlocks = 64;     // row-sweeping blocks (each writes one [2][dim] partial)
// 64 * 2 * 4096 floats = 2 MiB per device that loads the library, held until the process exits
static __device__ __align__(256) float g_ln_noalloc_scratch[kNoAllocBlocks * 2 * kNoAllocMaxDim];

constexpr int kMaxDevices = 64;
float *g_ln_noalloc_ptr[kMaxDevices];   // device address of the array, per device ordinal
bool g_ln_noalloc_ready[kMaxDevices];
std::mutex g_ln_noalloc_mu;
thread_local char g_noalloc_error[256] = "";

mcb_status noalloc_fail(mcb_status st, const char *msg, cudaError_t e = cudaSuccess) {
    if (e != cudaSuccess) snprintf(g_noalloc_error, sizeof(g_noalloc_error), "%s: %s", msg, cudaGetErrorString(e));
    else snprintf(g_noalloc_error, sizeof(g_noalloc_error), "%s", msg);
    return st;
}

// One-time set-up for the current device.  In host code the array's name is only a stand-in for
// the symbol, not a device address; the address a kernel can use comes from cudaGetSymbolAddress.
mcb_status ln_noalloc_setup(int device, float **out) {
    std::lock_guard<std::mutex> lk(g_ln_noalloc_mu);
    if (!g_ln_noalloc_ready[device]) {
        float *ptr = nullptr;
        cudaError_t e = cudaGetSymbolAddress((void **)&ptr, g_ln_noalloc_scratch);
        if (e != cudaSuccess) return noalloc_fail(MCB_BACKEND, "cudaGetSymbolAddress(layer-norm scratch)", e);
        const int smem_cap = 200 * 1024;
        e = cudaFuncSetAttribute(layer_norm_backward_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_cap);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(layer_norm_backward_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_cap);
        if (e != cudaSuccess) return noalloc_fail(MCB_BACKEND, "cudaFuncSetAttribute(layer-norm backward)", e);
        g_ln_noalloc_ptr[device] = ptr;
        g_ln_noalloc_ready[device] = true;
    }
    *out = g_ln_noalloc_ptr[device];
    return MCB_OK;
}
} // namespace

extern "C" const char *mcb_noalloc_last_error(void) { return g_noalloc_error; }

extern "C" mcb_status mcb_layer_norm_backward_noalloc(void *stream, const float *x, const float *gamma, const void *g,
                                                      int32_t g_dt, double eps, const float *mean, const float *rstd,
                                                      float *dx, float *dgamma, float *dbeta, int64_t rows, int64_t dim) {
    g_noalloc_error[0] = 0;
    if (rows < 0 || dim <= 0) return noalloc_fail(MCB_INVALID_ARGUMENT, "layer_norm_backward_noalloc: rows must be >= 0 and dim > 0");
    if (dim > kNoAllocMaxDim)
        return noalloc_fail(MCB_INVALID_ARGUMENT, "layer_norm_backward_noalloc: dim exceeds 4096, the size the built-in scratch array was laid out for");
    if (g_dt != MCB_F32 && g_dt != MCB_BF16) return noalloc_fail(MCB_UNSUPPORTED_DTYPE, "layer_norm_backward_noalloc: grad must be f32 or bf16");
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return noalloc_fail(MCB_BACKEND, "cudaGetDevice", e);
    if (device < 0 || device >= kMaxDevices) return noalloc_fail(MCB_UNSUPPORTED, "layer_norm_backward_noalloc: device ordinal above 63");
    float *scratch = nullptr;
    mcb_status st = ln_noalloc_setup(device, &scratch);
    if (st != MCB_OK) return st;
    cudaStream_t s = (cudaStream_t)stream;
    int warps = 8;
    while (warps > 1 && (size_t)warps * 2 * dim * sizeof(float) > (size_t)200 * 1024) warps >>= 1;
    size_t smem = (size_t)warps * 2 * dim * sizeof(float);
    int64_t want = (rows + warps - 1) / warps;
    int grid = (int)(want < 1 ? 1 : (want > kNoAllocBlocks ? kNoAllocBlocks : want));
    // Every block overwrites its whole [2][dim] slice and the second kernel reads exactly `grid`
    // slices, so nothing left in the array by an earlier call is ever read: no clearing needed.
    if (g_dt == MCB_F32)
        layer_norm_backward_kernel<float><<<grid, warps * 32, smem, s>>>(x, gamma, (const float *)g, (float)eps, mean, rstd, dx, scratch, rows, (int)dim);
    else
        layer_norm_backward_kernel<__nv_bfloat16><<<grid, warps * 32, smem, s>>>(x, gamma, (const __nv_bfloat16 *)g, (float)eps, mean, rstd, dx, scratch, rows, (int)dim);
    e = cudaGetLastError();
    if (e != cudaSuccess) return noalloc_fail(MCB_BACKEND, "layer_norm_backward_noalloc launch", e);
    layer_norm_params_final_kernel<<<(int)((2 * dim + 255) / 256), 256, 0, s>>>(scratch, grid, (int)dim, dgamma, dbeta);
    e = cudaGetLastError();
    if (e != cudaSuccess) return noalloc_fail(MCB_BACKEND, "layer_norm_backward_noalloc launch", e);
    return MCB_OK;
}
