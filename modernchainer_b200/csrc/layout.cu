// Data-layout ops of the tape: 2-D transpose and general axis permutation of f32 tensors.
// The reference does both on the host (download, scalar index loop, upload:
// autograd/src/host_ops.rs:690-777, cpu/src/kernels.rs:306-330); here they are device copies.
// Transpose goes through a 32x33 shared tile so that reads and writes are both coalesced;
// permute walks the OUTPUT linearly (coalesced writes) and gathers.
#include "common.cuh"
#include "internal.h"

namespace {

__global__ void transpose2d_kernel(const float *__restrict__ a, float *__restrict__ out, long long rows, long long cols) {
    __shared__ float tile[32][33];
    long long c0 = (long long)blockIdx.x * 32, r0 = (long long)blockIdx.y * 32;
    // block (32, 8): four passes over the 32 tile rows
    for (int y = threadIdx.y; y < 32; y += 8) {
        long long r = r0 + y, c = c0 + threadIdx.x;
        if (r < rows && c < cols) tile[y][threadIdx.x] = a[r * cols + c];
    }
    __syncthreads();
    for (int y = threadIdx.y; y < 32; y += 8) {
        long long c = c0 + y, r = r0 + threadIdx.x; // out[c, r]
        if (r < rows && c < cols) out[c * rows + r] = tile[threadIdx.x][y];
    }
}

struct PermuteWalk {
    int rank;
    long long od[8]; // output dims
    long long ss[8]; // source stride (elements) of the axis that feeds each output dim
};

__global__ void permute_kernel(const float *__restrict__ a, float *__restrict__ out, long long n, PermuteWalk w) {
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    long long stride = (long long)gridDim.x * blockDim.x;
    for (; i < n; i += stride) {
        long long rest = i, src = 0;
        for (int k = w.rank - 1; k >= 0; --k) {
            long long c = rest % w.od[k];
            rest /= w.od[k];
            src += c * w.ss[k];
        }
        out[i] = a[src];
    }
}

} // namespace

extern "C" {

mcb_status mcb_transpose2d(mcb_ctx *ctx, const float *a, float *out, int64_t rows, int64_t cols) {
    MCB_CHECK_CTX(ctx);
    if (rows < 0 || cols < 0) return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "transpose2d: negative extent");
    if (rows == 0 || cols == 0) return MCB_OK;
    ProfScope prof(ctx, MCB_PROF_ELEMENTWISE, 0.0, 8.0 * (double)rows * (double)cols);
    long long gx = (cols + 31) / 32, gy = (rows + 31) / 32;
    if (gy > 65535) { // very tall: fall back to the gather form
        int64_t dims[2] = {rows, cols};
        int32_t axes[2] = {1, 0};
        return mcb_permute(ctx, a, dims, 2, axes, out);
    }
    transpose2d_kernel<<<dim3((unsigned)gx, (unsigned)gy), dim3(32, 8), 0, ctx->stream>>>(a, out, rows, cols);
    MCB_LAUNCHED(ctx);
    return MCB_OK;
}

mcb_status mcb_permute(mcb_ctx *ctx, const float *a, const int64_t *dims, int32_t rank, const int32_t *axes, float *out) {
    MCB_CHECK_CTX(ctx);
    if (rank < 0 || rank > 8) return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "permute supports up to 8 dimensions, got %d", rank);
    bool seen[8] = {false, false, false, false, false, false, false, false};
    for (int i = 0; i < rank; ++i) {
        if (axes[i] < 0 || axes[i] >= rank || seen[axes[i]]) return mcb_fail(ctx, MCB_INVALID_ARGUMENT, "invalid permute axes");
        seen[axes[i]] = true;
    }
    long long sstr[8], n = 1;
    for (int i = rank - 1; i >= 0; --i) {
        sstr[i] = n;
        n *= dims[i];
    }
    if (n == 0) return MCB_OK;
    PermuteWalk w;
    w.rank = rank;
    for (int i = 0; i < rank; ++i) {
        w.od[i] = dims[axes[i]];
        w.ss[i] = sstr[axes[i]];
    }
    ProfScope prof(ctx, MCB_PROF_ELEMENTWISE, 0.0, 8.0 * (double)n);
    permute_kernel<<<mcb_grid_for(ctx, n, 256), 256, 0, ctx->stream>>>(a, out, n, w);
    MCB_LAUNCHED(ctx);
    return MCB_OK;
}

} // extern "C"
