// Linear recurrences over a matrix state per head, carried from token to token in a
// float32 state slot per request, and what surrounds them.
//
// Per head, with key size e and value size f, the state S is [e, f] and one token does
//
//   read first  (a bonus u on the current token, a decay per key channel and token):
//       o_j = sum_i a_i (S_ij + u_i k_i v_j);   S_ij <- w_i S_ij + k_i v_j
//   write first (one fixed decay a head):
//       S_ij <- g S_ij + k_i v_j;               o_j = sum_i a_i S_ij
//
// with a the "receptance" or query.  mls_linear_scan walks the tokens of every request of
// the step in order, from the state the slot holds, and leaves o [T, H*f] in float32; the
// state goes back to the slot.  A CTA owns 16 columns of one head's S for one request:
// thread (column, row group) keeps every eighth row of its column in registers, a warp holds
// four columns times eight row groups, and the sum over i is the thread's rows in order
// followed by three shuffles: the order never depends on the batch or on how the tokens
// were cut into steps.  Tokens are taken 16 at a time through shared memory.
//
//   mls_scan_finish      o / rms(o) per head (eps inside the root) * weight * silu(gate)
//   mls_rotate_rows      rotation of the first `dims` entries of every head of q and k,
//                        entry i paired with i + dims/2, k then times a constant; float32 out
//   mls_decay_lowrank    w = exp(-exp(W2 tanh(lo) + w0)) from the low-rank pre-activation
//
// State, decays, exponentials, angles' cosines and sines, norms and sums are float32 (the
// angles themselves float64: position * frequency); a, k, v come from the projections.
#include "common.cuh"

namespace {
constexpr int LS_COLS = 16;         // columns of S a CTA owns
constexpr int LS_GROUPS = 8;        // row groups: lanes that share a column
constexpr int LS_THREADS = LS_COLS * LS_GROUPS;
constexpr int LS_TOKENS = 16;       // tokens a pass

template <int RPT>
__global__ void __launch_bounds__(LS_THREADS)
linear_scan_kernel(const void* __restrict__ a_src, int a_dtype, int a_row, int a_off,
                   const void* __restrict__ k_src, int k_dtype, int k_row, int k_off,
                   const void* __restrict__ v_src, int v_dtype, int v_row, int v_off,
                   const float* __restrict__ decay_tok, int decay_row,
                   const float* __restrict__ decay_head,
                   const void* __restrict__ bonus, int bonus_dtype, int read_first,
                   const int* __restrict__ cu_q, const int* __restrict__ state_slot,
                   float* __restrict__ state, long long state_stride,
                   int n_heads, int e, int f, float* __restrict__ out) {
    chain_release();
    chain_wait();
    const int r = blockIdx.z, head = blockIdx.y, col0 = blockIdx.x * LS_COLS;
    const int t0 = cu_q[r], n = cu_q[r + 1] - t0;
    if (n <= 0) return;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int grp = lane & (LS_GROUPS - 1);               // row group: the low three lane bits
    const int col = col0 + warp * 4 + (lane >> 3);
    const bool col_ok = col < f;
    extern __shared__ float smem[];
    float* a_s = smem;                                    // [LS_TOKENS][e]
    float* k_s = a_s + LS_TOKENS * e;
    float* w_s = k_s + LS_TOKENS * e;                     // decays per key channel (read first)
    float* v_s = w_s + (decay_tok ? LS_TOKENS * e : 0);   // [LS_TOKENS][LS_COLS]

    float* S = state + (size_t)state_slot[r] * state_stride + (size_t)head * e * f;
    float s[RPT], ub[RPT];
#pragma unroll
    for (int i = 0; i < RPT; ++i) {
        const int row = i * LS_GROUPS + grp;
        s[i] = (col_ok && row < e) ? S[(size_t)row * f + col] : 0.f;
        ub[i] = (bonus && row < e) ? load_as_float(bonus, (size_t)head * e + row, bonus_dtype) : 0.f;
    }
    const float g = decay_head ? decay_head[head] : 1.f;

    for (int b0 = 0; b0 < n; b0 += LS_TOKENS) {
        const int nb = min(LS_TOKENS, n - b0);
        __syncthreads();
        for (int u = threadIdx.x; u < nb * e; u += LS_THREADS) {
            const int tt = u / e, i = u - tt * e;
            const size_t t = (size_t)(t0 + b0 + tt);
            a_s[u] = load_as_float(a_src, t * a_row + a_off + head * e + i, a_dtype);
            k_s[u] = load_as_float(k_src, t * k_row + k_off + head * e + i, k_dtype);
            if (decay_tok) w_s[u] = decay_tok[t * decay_row + head * e + i];
        }
        for (int u = threadIdx.x; u < nb * LS_COLS; u += LS_THREADS) {
            const int tt = u / LS_COLS, j = u - tt * LS_COLS;
            const size_t t = (size_t)(t0 + b0 + tt);
            v_s[u] = col0 + j < f
                ? load_as_float(v_src, t * v_row + v_off + head * f + col0 + j, v_dtype) : 0.f;
        }
        __syncthreads();
        for (int tt = 0; tt < nb; ++tt) {
            const float vj = v_s[tt * LS_COLS + warp * 4 + (lane >> 3)];
            const float* at = a_s + tt * e + grp;
            const float* kt = k_s + tt * e + grp;
            const float* wt = w_s + tt * e + grp;
            float acc = 0.f;
            if (read_first) {
#pragma unroll
                for (int i = 0; i < RPT; ++i) {
                    if (i * LS_GROUPS + grp < e) {
                        const float ki = kt[i * LS_GROUPS];
                        acc = fmaf(at[i * LS_GROUPS], fmaf(ub[i] * ki, vj, s[i]), acc);
                        s[i] = fmaf(decay_tok ? wt[i * LS_GROUPS] : g, s[i], ki * vj);
                    }
                }
            } else {
#pragma unroll
                for (int i = 0; i < RPT; ++i) {
                    if (i * LS_GROUPS + grp < e) {
                        s[i] = fmaf(decay_tok ? wt[i * LS_GROUPS] : g, s[i], kt[i * LS_GROUPS] * vj);
                        acc = fmaf(at[i * LS_GROUPS], s[i], acc);
                    }
                }
            }
            acc += __shfl_xor_sync(0xffffffffu, acc, 1);
            acc += __shfl_xor_sync(0xffffffffu, acc, 2);
            acc += __shfl_xor_sync(0xffffffffu, acc, 4);
            if (grp == 0 && col_ok)
                out[(size_t)(t0 + b0 + tt) * n_heads * f + (size_t)head * f + col] = acc;
        }
    }
#pragma unroll
    for (int i = 0; i < RPT; ++i) {
        const int row = i * LS_GROUPS + grp;
        if (col_ok && row < e) S[(size_t)row * f + col] = s[i];
    }
}

// One warp a (token, head).
template <typename T>
__global__ void __launch_bounds__(128)
scan_finish_kernel(const float* __restrict__ o, const T* __restrict__ gate, int gate_row,
                   int gate_off, const void* __restrict__ w, int w_dtype, float eps,
                   T* __restrict__ out, int n_tokens, int n_heads, int f) {
    chain_release();
    chain_wait();
    const long long unit = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (unit >= (long long)n_tokens * n_heads) return;
    const int lane = threadIdx.x & 31;
    const int t = (int)(unit / n_heads), head = (int)(unit % n_heads);
    const float* row = o + (size_t)t * n_heads * f + (size_t)head * f;
    float ss = 0.f;
    for (int j = lane; j < f; j += 32) ss = fmaf(row[j], row[j], ss);
    const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)f + eps);
    for (int j = lane; j < f; j += 32) {
        const int c = head * f + j;
        const float z = Elem<T>::load(gate + (size_t)t * gate_row + gate_off + c);
        float v = row[j] * inv;
        if (w) v *= load_as_float(w, c, w_dtype);
        Elem<T>::store(out + (size_t)t * n_heads * f + c, v * (z / (1.0f + expf(-z))));
    }
}

// One block a token; thread (head, i) rotates the pair (i, i + dims/2) of q and of k.
template <typename T>
__global__ void __launch_bounds__(256)
rotate_rows_kernel(const T* __restrict__ src, int src_row, int q_off, int k_off,
                   const int* __restrict__ positions, const double* __restrict__ freq, int dims,
                   float k_scale, float* __restrict__ out, int n_heads, int e) {
    chain_release();
    extern __shared__ float cs[];                        // [dims]: cos | sin
    const int t = blockIdx.x, half = dims / 2;
    chain_wait();
    const int p = positions[t];
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        double s, c;
        sincos((double)p * freq[i], &s, &c);
        cs[i] = (float)c;
        cs[half + i] = (float)s;
    }
    __syncthreads();
    const int width = n_heads * e;
    for (int u = threadIdx.x; u < 2 * width; u += blockDim.x) {
        const int which = u / width, c = u - which * width, i = c % e;
        const T* row = src + (size_t)t * src_row + (which ? k_off : q_off);
        float v = Elem<T>::load(row + c);
        if (i < dims) {
            const bool low = i < half;
            const float m = Elem<T>::load(row + (low ? c + half : c - half));
            const float co = cs[low ? i : i - half], si = cs[half + (low ? i : i - half)];
            v = low ? __fsub_rn(__fmul_rn(v, co), __fmul_rn(m, si))
                    : __fadd_rn(__fmul_rn(v, co), __fmul_rn(m, si));
        }
        out[(size_t)t * 2 * width + u] = which ? v * k_scale : v;
    }
}

// One block a token: lo (float32 [T, rank], before its tanh) -> w [T, channels].
__global__ void __launch_bounds__(256)
decay_lowrank_kernel(const float* __restrict__ lo, int rank, const float* __restrict__ w2,
                     const void* __restrict__ w0, int w0_dtype, float* __restrict__ out,
                     int channels) {
    chain_release();
    extern __shared__ float th[];                        // [rank]
    chain_wait();
    const int t = blockIdx.x;
    for (int i = threadIdx.x; i < rank; i += blockDim.x) th[i] = tanhf(lo[(size_t)t * rank + i]);
    __syncthreads();
    for (int c = threadIdx.x; c < channels; c += blockDim.x) {
        const float* wr = w2 + (size_t)c * rank;
        float z = 0.f;
        for (int i = 0; i < rank; ++i) z = fmaf(wr[i], th[i], z);
        z += load_as_float(w0, c, w0_dtype);
        out[(size_t)t * channels + c] = expf(-expf(z));
    }
}

template <int RPT>
int launch_scan(dim3 grid, size_t smem, cudaStream_t stream, const void* a_src, int a_dtype,
                int a_row, int a_off, const void* k_src, int k_dtype, int k_row, int k_off,
                const void* v_src, int v_dtype, int v_row, int v_off, const float* decay_tok,
                int decay_row, const float* decay_head, const void* bonus, int bonus_dtype,
                int read_first, const int* cu_q, const int* state_slot, float* state,
                long long state_stride, int n_heads, int e, int f, float* out) {
    auto kernel = linear_scan_kernel<RPT>;
    if (smem > 48 * 1024) {
        const int rc = (int)cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 (int)smem);
        if (rc) return rc;
    }
    MLS_LAUNCH(kernel, grid, dim3(LS_THREADS), smem, stream, a_src, a_dtype, a_row, a_off, k_src,
               k_dtype, k_row, k_off, v_src, v_dtype, v_row, v_off, decay_tok, decay_row,
               decay_head, bonus, bonus_dtype, read_first, cu_q, state_slot, state, state_stride,
               n_heads, e, f, out);
    return launch_status();
}
}  // namespace

MLS_API int mls_linear_scan(const void* a_src, int a_dtype, int a_row, int a_off,
                            const void* k_src, int k_dtype, int k_row, int k_off,
                            const void* v_src, int v_dtype, int v_row, int v_off,
                            const float* decay_tok, int decay_row, const float* decay_head,
                            const void* bonus, int bonus_dtype, int read_first, const int* cu_q,
                            const int* state_slot, float* state, long long state_stride,
                            int n_requests, int n_heads, int e, int f, float* out,
                            cudaStream_t stream) {
    if (n_requests <= 0) return 0;
    if (e <= 0 || f <= 0 || e > 32 * LS_GROUPS || (!decay_tok == !decay_head))
        return MLS_ERR_UNSUPPORTED;
    const dim3 grid((f + LS_COLS - 1) / LS_COLS, n_heads, n_requests);
    const size_t smem = (size_t)LS_TOKENS * ((decay_tok ? 3 : 2) * e + LS_COLS) * sizeof(float);
    const int rpt = (e + LS_GROUPS - 1) / LS_GROUPS;
#define LS_GO(R)                                                                                 \
    return launch_scan<R>(grid, smem, stream, a_src, a_dtype, a_row, a_off, k_src, k_dtype, k_row, \
                          k_off, v_src, v_dtype, v_row, v_off, decay_tok, decay_row, decay_head,  \
                          bonus, bonus_dtype, read_first, cu_q, state_slot, state, state_stride,  \
                          n_heads, e, f, out)
    if (rpt <= 2) LS_GO(2);
    if (rpt <= 4) LS_GO(4);
    if (rpt <= 8) LS_GO(8);
    if (rpt <= 16) LS_GO(16);
    LS_GO(32);
#undef LS_GO
}

MLS_API int mls_scan_finish(const float* o, const void* gate, int act_dtype, int gate_row,
                            int gate_off, const void* w, int w_dtype, float eps, void* out,
                            int n_tokens, int n_heads, int f, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    const long long units = (long long)n_tokens * n_heads;
    const int blocks = (int)((units + 3) / 4);
    if (act_dtype == MLS_BF16)
        MLS_LAUNCH((scan_finish_kernel<__nv_bfloat16>), dim3(blocks), dim3(128), 0, stream, o,
                   (const __nv_bfloat16*)gate, gate_row, gate_off, w, w_dtype, eps,
                   (__nv_bfloat16*)out, n_tokens, n_heads, f);
    else
        MLS_LAUNCH((scan_finish_kernel<float>), dim3(blocks), dim3(128), 0, stream, o,
                   (const float*)gate, gate_row, gate_off, w, w_dtype, eps, (float*)out, n_tokens,
                   n_heads, f);
    return launch_status();
}

MLS_API int mls_rotate_rows(const void* src, int src_dtype, int src_row, int q_off, int k_off,
                            const int* positions, const double* freq, int dims, float k_scale,
                            float* out, int n_tokens, int n_heads, int e, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (dims < 0 || dims > e || (dims & 1) || (dims > 0 && !freq)) return MLS_ERR_UNSUPPORTED;
    const size_t smem = (size_t)(dims > 0 ? dims : 1) * sizeof(float);
    if (smem > 48 * 1024) return MLS_ERR_UNSUPPORTED;
    if (src_dtype == MLS_BF16)
        MLS_LAUNCH((rotate_rows_kernel<__nv_bfloat16>), dim3(n_tokens), dim3(256), smem, stream,
                   (const __nv_bfloat16*)src, src_row, q_off, k_off, positions, freq, dims,
                   k_scale, out, n_heads, e);
    else
        MLS_LAUNCH((rotate_rows_kernel<float>), dim3(n_tokens), dim3(256), smem, stream,
                   (const float*)src, src_row, q_off, k_off, positions, freq, dims, k_scale, out,
                   n_heads, e);
    return launch_status();
}

MLS_API int mls_decay_lowrank(const float* lo, int rank, const float* w2, const void* w0,
                              int w0_dtype, float* out, int n_tokens, int channels,
                              cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    const size_t smem = (size_t)rank * sizeof(float);
    if (rank <= 0 || smem > 48 * 1024) return MLS_ERR_UNSUPPORTED;
    MLS_LAUNCH((decay_lowrank_kernel), dim3(n_tokens), dim3(256), smem, stream, lo, rank, w2, w0,
               w0_dtype, out, channels);
    return launch_status();
}
