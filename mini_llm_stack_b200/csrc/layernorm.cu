// Layer norm with a weight and no bias, fused with the pending residual additions.
//
//   v = x[row] + delta[row] + more_rows[row] + more_vec        (each addend optional)
//   h = (v - mean(v)) / sqrt(mean((v - mean(v))^2) + eps) * w
//
// rows == nullptr: every row t; x[t] is replaced by v (the residual stream moves on).
// rows != nullptr: for i < n_rows the row rows[i] is read and h[i] written; x stays.
//
// delta is a tensor of either element type, or (delta_parts > 1) that many float32
// slices part_stride elements apart (a matrix product cut along K), added in the order
// of the slices.  more_rows is float32 [T, d] (a second stream added row by row, e.g.
// the embedding's output at the start of a repeated pass), more_vec one vector [d]
// added to every row.
//
// Everything is float32 with one rounding at the store.  Mean and variance are taken
// in two passes over the row held in shared memory; the order of both sums depends on
// d alone (one block of LN_THREADS threads a row), so a row's result does not depend
// on the batch it is in.
//
// mls_residual_add only settles more_rows / more_vec into x, for a norm of another kind.
#include "common.cuh"

namespace {
constexpr int LN_THREADS = 256;

__global__ void __launch_bounds__(LN_THREADS)
add_layernorm_kernel(float* __restrict__ x, const void* __restrict__ delta, int delta_dtype,
                     int delta_parts, size_t part_stride, const float* __restrict__ more_rows,
                     const void* __restrict__ more_vec, int vec_dtype,
                     const void* __restrict__ w, int w_dtype, float eps, void* __restrict__ h,
                     int h_dtype, int n_rows, int d, const int* __restrict__ rows) {
    chain_release();
    chain_wait();
    extern __shared__ float row_s[];
    __shared__ float scratch[33];
    for (int out_row = blockIdx.x; out_row < n_rows; out_row += gridDim.x) {
        const size_t src = (size_t)(rows ? rows[out_row] : out_row) * d;
        float s = 0.f;
        for (int c = threadIdx.x; c < d; c += LN_THREADS) {
            float v = x[src + c];
            if (delta) {
                float a = load_as_float(delta, src + c, delta_parts > 1 ? MLS_F32 : delta_dtype);
                for (int k = 1; k < delta_parts; ++k)
                    a += ((const float*)delta)[src + c + (size_t)k * part_stride];
                v += a;
            }
            if (more_rows) v += more_rows[src + c];
            if (more_vec) v += load_as_float(more_vec, c, vec_dtype);
            row_s[c] = v;
            if (!rows) x[src + c] = v;
            s += v;
        }
        const float mean = block_sum(s, scratch) / (float)d;
        float q = 0.f;
        for (int c = threadIdx.x; c < d; c += LN_THREADS) {
            const float u = row_s[c] - mean;
            q = fmaf(u, u, q);
        }
        const float var = block_sum(q, scratch) / (float)d;
        const float inv = 1.0f / sqrtf(var + eps);
        for (int c = threadIdx.x; c < d; c += LN_THREADS)
            store_from_float(h, (size_t)out_row * d + c, h_dtype,
                             (row_s[c] - mean) * inv * load_as_float(w, c, w_dtype));
        __syncthreads();                         // row_s is filled again for the next row
    }
}

__global__ void residual_add_kernel(float* __restrict__ x, const float* __restrict__ more_rows,
                                    const void* __restrict__ more_vec, int vec_dtype,
                                    size_t n, int d) {
    chain_release();
    chain_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (size_t)gridDim.x * blockDim.x) {
        float v = x[i];
        if (more_rows) v += more_rows[i];
        if (more_vec) v += load_as_float(more_vec, i % d, vec_dtype);
        x[i] = v;
    }
}

// x += delta (a tensor, the parts of a product cut along K, or nothing); then
// out[t] = [x[t] | other[t]] in the activation type: the input of a projection that reads
// the stream beside a second stream.
__global__ void settle_concat_kernel(float* __restrict__ x, const void* __restrict__ delta,
                                     int delta_dtype, int n_parts, size_t part_stride,
                                     const float* __restrict__ other, void* __restrict__ out,
                                     int out_dtype, size_t n, int d) {
    chain_release();
    chain_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (size_t)gridDim.x * blockDim.x) {
        float v = x[i];
        if (delta) {
            float add = 0.f;
            for (int k = 0; k < n_parts; ++k)
                add += load_as_float(delta, i + (size_t)k * part_stride, delta_dtype);
            v += add;
            x[i] = v;
        }
        const size_t t = i / d, c = i - t * d;
        store_from_float(out, t * 2 * d + c, out_dtype, v);
        store_from_float(out, t * 2 * d + d + c, out_dtype, other[i]);
    }
}
}  // namespace

MLS_API int mls_settle_concat(float* x, const void* delta, int delta_dtype, int delta_parts,
                              long long part_stride, const float* other, void* out,
                              int out_dtype, int n_rows, int d, cudaStream_t stream) {
    if (n_rows <= 0 || d <= 0) return 0;
    const size_t n = (size_t)n_rows * d;
    const int blocks = (int)((n + 255) / 256 < (size_t)(8 * sm_count()) ? (n + 255) / 256
                                                                       : 8 * sm_count());
    MLS_LAUNCH((settle_concat_kernel), dim3(blocks), dim3(256), 0, stream, x, delta, delta_dtype,
               delta_parts < 1 ? 1 : delta_parts, (size_t)part_stride, other, out, out_dtype, n,
               d);
    return launch_status();
}

MLS_API int mls_add_layernorm(float* x, const void* delta, int delta_dtype, int delta_parts,
                              long long part_stride, const float* more_rows, const void* more_vec,
                              int vec_dtype, const void* w, int w_dtype, float eps, void* h,
                              int h_dtype, int n_rows, int d, const int* rows,
                              cudaStream_t stream) {
    if (n_rows <= 0 || d <= 0) return 0;
    const size_t smem = (size_t)d * sizeof(float);
    if (smem > 200 * 1024) return MLS_ERR_UNSUPPORTED;
    if (smem > 48 * 1024) {
        const int rc = (int)cudaFuncSetAttribute(add_layernorm_kernel,
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 (int)smem);
        if (rc) return rc;
    }
    const int blocks = n_rows < 8 * sm_count() ? n_rows : 8 * sm_count();
    MLS_LAUNCH((add_layernorm_kernel), dim3(blocks), dim3(LN_THREADS), smem, stream, x, delta,
               delta_dtype, delta_parts < 1 ? 1 : delta_parts, (size_t)part_stride, more_rows,
               more_vec, vec_dtype, w, w_dtype, eps, h, h_dtype, n_rows, d, rows);
    return launch_status();
}

MLS_API int mls_residual_add(float* x, const float* more_rows, const void* more_vec,
                             int vec_dtype, int n_rows, int d, cudaStream_t stream) {
    if (n_rows <= 0 || d <= 0 || (!more_rows && !more_vec)) return 0;
    const size_t n = (size_t)n_rows * d;
    const int blocks = (int)((n + 255) / 256 < (size_t)(8 * sm_count()) ? (n + 255) / 256
                                                                       : 8 * sm_count());
    MLS_LAUNCH((residual_add_kernel), dim3(blocks), dim3(256), 0, stream, x, more_rows, more_vec,
               vec_dtype, n, d);
    return launch_status();
}
