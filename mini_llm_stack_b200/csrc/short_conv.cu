// Short causal convolutions over time whose last inputs are carried per request, and
// what a mixer does right around them.
//
// A convolution of `taps` taps on a channel, y_t = sum_j w[j] * u_(t - taps + 1 + j) with
// zeros before the sequence's start, needs the taps - 1 inputs before a step's first
// token.  They live in the request's state slot as a tail [taps - 1, channels] of
// float32, oldest first, zero when the slot is claimed (so a tail that reaches before the
// start reads as zeros without a test).  A step reads the tail in the kernel that
// convolves and moves it on in mls_tail_update, a launch of its own, so that no block
// reads what another writes.  "The previous token's row" (a token shift) is the tail of
// a two-tap convolution.
//
//   mls_qk_conv_norm_rope_store   q|k projection (float32) + bias -> convolution ->
//       v := the convolved k (stored in the value pages) -> RMS norm over the whole q
//       row and over the whole k row -> rotation of the first `dims` entries of every
//       head, entry 2i paired with 2i + 1 -> q into the attention's row, k into the pages
//   mls_token_shift_mix           mix_s = h + (h_prev - h) * mu_s for several s at once
//   mls_tail_update               tail := the last taps - 1 inputs after this step
//
// Angles are formed in float64 (position * frequency, frequencies handed over as
// float64) and brought into [-pi, pi] there; their cosine and sine are float32, as are
// sums, norms and the rotation.
#include "common.cuh"
#include "page_tail.cuh"

namespace {
constexpr int SC_THREADS = 256;

// The projection may come as the parts of a product cut along K (float32 [parts][T][C],
// `stride` elements apart): their sum in the order of the parts is the product.
__device__ __forceinline__ float proj_at(const float* __restrict__ proj, size_t i, int n_parts,
                                         size_t stride) {
    float s = proj[i];
    for (int k = 1; k < n_parts; ++k) s += proj[i + (size_t)k * stride];
    return s;
}
__device__ __forceinline__ float4 proj4_at(const float* __restrict__ proj, size_t i, int n_parts,
                                           size_t stride) {
    if (n_parts == 1) return *reinterpret_cast<const float4*>(proj + i);
    return sum_parts4<4>(proj, i, n_parts, stride);      // four parts' loads under way at a time
}

// u_(i) of channel c for the step index i of request rows [row0, ...): from the step's
// rows if i >= 0, else from the tail (i = -1 is the newest tail row).
__device__ __forceinline__ float conv_input(const float* __restrict__ proj, int n_parts,
                                            size_t part_stride, int width, int col,
                                            const void* __restrict__ bias, int w_dtype,
                                            const float* __restrict__ tail, int n_tail,
                                            int channels, int c, int row0, int i) {
    if (i >= 0) {
        float v = proj_at(proj, (size_t)(row0 + i) * width + col, n_parts, part_stride);
        if (bias) v += load_as_float(bias, c, w_dtype);
        return v;
    }
    return tail[(size_t)(n_tail + i) * channels + c];
}

template <typename T>
__global__ void __launch_bounds__(SC_THREADS)
qk_conv_norm_rope_store_kernel(
        const float* __restrict__ proj, int n_parts, long long part_stride,
        const void* __restrict__ bias,
        const void* __restrict__ conv_w, int taps, const void* __restrict__ q_norm,
        const void* __restrict__ k_norm, int w_dtype, float eps,
        float* __restrict__ tail, long long tail_stride, int move_tail,
        const int* __restrict__ state_slot, const int* __restrict__ cu_q,
        const int* __restrict__ req_of_token, const int* __restrict__ positions,
        const double* __restrict__ freq, int rot_dims,
        T* __restrict__ q_out, int q_row, const int* __restrict__ slot_map,
        T* __restrict__ k_pool, T* __restrict__ v_pool, int block_size, long long pool_slots,
        int n_tokens, int n_heads, int n_kv, int hd, int writes, int* status) {
    chain_release();
    extern __shared__ float smem[];
    const int cq = n_heads * hd, ck = n_kv * hd, channels = cq + ck;
    float* y = smem;                       // [channels] convolved, then normalised
    float* cs = y + channels;              // [rot_dims]: cos | sin
    __shared__ float scratch[33];
    const int t = blockIdx.x;
    const int slot = writes ? slot_map[t] : -1;
    const int rest = writes ? page_tail_to_clear(slot_map, t, n_tokens, slot, block_size) : 0;
    chain_wait();
    const int r = req_of_token[t], row0 = cu_q[r], i_t = t - row0, p = positions[t];
    const int n_tail = taps - 1;
    float* my_tail = n_tail > 0 ? tail + (size_t)state_slot[r] * tail_stride : nullptr;
    if (threadIdx.x < rot_dims / 2)
        angle_cos_sin(p, freq[threadIdx.x], cs[threadIdx.x], cs[rot_dims / 2 + threadIdx.x]);
    float ssq = 0.f, ssk = 0.f;
    for (int c = threadIdx.x; c < channels; c += SC_THREADS) {
        float acc;
        if (n_tail > 0) {
            acc = 0.f;
            for (int j = 0; j < taps; ++j) {
                const float u = conv_input(proj, n_parts, (size_t)part_stride, channels, c, bias,
                                           w_dtype, my_tail, n_tail, channels, c, row0,
                                           i_t - n_tail + j);
                acc = fmaf(load_as_float(conv_w, (size_t)c * taps + j, w_dtype), u, acc);
                // a step of one token a request moves its tail on itself: row j - 1 was read
                // by this thread one tap ago
                if (move_tail && j >= 1) my_tail[(size_t)(j - 1) * channels + c] = u;
            }
        } else {
            acc = conv_input(proj, n_parts, (size_t)part_stride, channels, c, bias, w_dtype, nullptr,
                             0, channels, c, row0, i_t);
            if (taps == 1) acc *= load_as_float(conv_w, c, w_dtype);
        }
        y[c] = acc;
        if (c < cq) ssq = fmaf(acc, acc, ssq); else ssk = fmaf(acc, acc, ssk);
    }
    const bool slot_ok = slot >= 0 && slot < pool_slots;
    if (writes && !slot_ok && threadIdx.x == 0) atomicOr(status, MLS_STATUS_BAD_SLOT);
    const float inv_q = 1.0f / sqrtf(block_sum(ssq, scratch) / (float)cq + eps);
    const float inv_k = 1.0f / sqrtf(block_sum(ssk, scratch) / (float)ck + eps);
    // (block_sum's barriers also make y and cs visible to every thread)
    const long long page = slot_ok ? slot / block_size : 0;
    const int off = slot_ok ? slot % block_size : 0;
    const long long n_pages = pool_slots / block_size;
    // values: the convolved keys as they are
    if (writes && slot_ok)
        for (int c = threadIdx.x; c < ck; c += SC_THREADS) {
            const int g = c / hd, e = c - g * hd;
            Elem<T>::store(v_pool + (((size_t)g * n_pages + page) * block_size + off) * hd + e,
                           y[cq + c]);
        }
    // queries and keys: norm, then the rotation of pairs (2i, 2i + 1) below rot_dims
    for (int c = threadIdx.x; c < channels; c += SC_THREADS) {
        const bool is_q = c < cq;
        const int cc = is_q ? c : c - cq;
        const int e = cc % hd;
        const void* nw = is_q ? q_norm : k_norm;
        const float inv = is_q ? inv_q : inv_k;
        float v = y[c] * inv * load_as_float(nw, cc, w_dtype);
        if (e < rot_dims) {
            const int mate = (e & 1) ? c - 1 : c + 1, mcc = (e & 1) ? cc - 1 : cc + 1;
            const float m = y[mate] * inv * load_as_float(nw, mcc, w_dtype);
            const float co = cs[e >> 1], si = cs[rot_dims / 2 + (e >> 1)];
            // even entry: a cos - b sin; odd entry: b cos + a sin
            v = (e & 1) ? __fadd_rn(__fmul_rn(v, co), __fmul_rn(m, si))
                        : __fsub_rn(__fmul_rn(v, co), __fmul_rn(m, si));
        }
        if (is_q) {
            Elem<T>::store(q_out + (size_t)t * q_row + c, v);
        } else if (writes && slot_ok) {
            const int g = cc / hd;
            Elem<T>::store(k_pool + (((size_t)g * n_pages + page) * block_size + off) * hd + e, v);
        }
    }
    if (writes && slot_ok)
        clear_page_tail<T>(rest, slot, block_size, (int)n_pages, n_kv, hd, k_pool, v_pool);
}

// The same with four consecutive channels a thread and step (channels, query channels and
// the head size multiples of four): 16-byte loads of the projection's rows, the taps and
// norm weights of four channels at once, and a rotation whose pairs (2i, 2i + 1) lie inside
// the thread's four values.  The sums run in another order than in the kernel above, so a
// model takes one of the two for all its steps (the choice depends on its sizes alone).
struct Four { float v[4]; };
__device__ __forceinline__ Four load_four(const void* base, size_t i, int dtype) {
    Four r;
    if (dtype == MLS_BF16) {
        const uint2 raw = *reinterpret_cast<const uint2*>((const __nv_bfloat16*)base + i);
        const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
        const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
        r.v[0] = lo.x; r.v[1] = lo.y; r.v[2] = hi.x; r.v[3] = hi.y;
    } else {
        const float4 x = *reinterpret_cast<const float4*>((const float*)base + i);
        r.v[0] = x.x; r.v[1] = x.y; r.v[2] = x.z; r.v[3] = x.w;
    }
    return r;
}
template <typename T>
__device__ __forceinline__ void store_four(T* dst, const float (&v)[4]);
template <>
__device__ __forceinline__ void store_four<float>(float* dst, const float (&v)[4]) {
    *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
}
template <>
__device__ __forceinline__ void store_four<__nv_bfloat16>(__nv_bfloat16* dst, const float (&v)[4]) {
    *reinterpret_cast<uint2*>(dst) = pack_bf16x4(make_float4(v[0], v[1], v[2], v[3]));
}

constexpr int QK_MAX_TAPS = 8;

template <typename T>
__global__ void __launch_bounds__(SC_THREADS, 3)
qk_conv_norm_rope_store_vec4_kernel(
        const float* __restrict__ proj, int n_parts, long long part_stride,
        const void* __restrict__ bias,
        const void* __restrict__ conv_w, int taps, const void* __restrict__ q_norm,
        const void* __restrict__ k_norm, int w_dtype, float eps,
        float* __restrict__ tail, long long tail_stride, int move_tail,
        const int* __restrict__ state_slot, const int* __restrict__ cu_q,
        const int* __restrict__ req_of_token, const int* __restrict__ positions,
        const double* __restrict__ freq, int rot_dims,
        T* __restrict__ q_out, int q_row, const int* __restrict__ slot_map,
        T* __restrict__ k_pool, T* __restrict__ v_pool, int block_size, long long pool_slots,
        int n_tokens, int n_heads, int n_kv, int hd, int writes, int* status) {
    chain_release();
    extern __shared__ float smem[];
    const int cq = n_heads * hd, ck = n_kv * hd, channels = cq + ck, half = rot_dims / 2;
    float* y = smem;                       // [channels] convolved
    float* cs = y + channels;              // [rot_dims]: cos | sin
    __shared__ float sums[SC_THREADS / 32][2];
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int slot = writes ? slot_map[t] : -1;
    const int rest = writes ? page_tail_to_clear(slot_map, t, n_tokens, slot, block_size) : 0;
    chain_wait();
    const int r = req_of_token[t], i_t = t - cu_q[r], p = positions[t];
    const int n_tail = taps > 0 ? taps - 1 : 0;
    float* my_tail = n_tail > 0 ? tail + (size_t)state_slot[r] * tail_stride : nullptr;
    if (threadIdx.x < half)
        angle_cos_sin(p, freq[threadIdx.x], cs[threadIdx.x], cs[half + threadIdx.x]);
    float ssq = 0.f, ssk = 0.f;
    for (int c = threadIdx.x * 4; c < channels; c += blockDim.x * 4) {
        Four b;
        b.v[0] = b.v[1] = b.v[2] = b.v[3] = 0.f;
        if (bias) b = load_four(bias, c, w_dtype);
        float acc[4];
        if (taps == 0) {
            const float4 x = proj4_at(proj, (size_t)t * channels + c, n_parts, (size_t)part_stride);
            acc[0] = x.x + b.v[0]; acc[1] = x.y + b.v[1]; acc[2] = x.z + b.v[2]; acc[3] = x.w + b.v[3];
        } else {
            acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
#pragma unroll
            for (int j = 0; j < QK_MAX_TAPS; ++j) {
                if (j < taps) {
                    const int i = i_t - n_tail + j;
                    float4 x;
                    if (i >= 0) {
                        x = proj4_at(proj, (size_t)(t - n_tail + j) * channels + c, n_parts,
                                     (size_t)part_stride);
                        x.x += b.v[0]; x.y += b.v[1]; x.z += b.v[2]; x.w += b.v[3];
                    } else {
                        x = *reinterpret_cast<const float4*>(my_tail + (size_t)(n_tail + i) * channels + c);
                    }
                    if (move_tail && j >= 1)     // (row j - 1 was read by this thread one tap ago)
                        *reinterpret_cast<float4*>(my_tail + (size_t)(j - 1) * channels + c) = x;
                    const size_t wj = (size_t)c * taps + j;          // [channel][tap]
                    acc[0] = fmaf(load_as_float(conv_w, wj, w_dtype), x.x, acc[0]);
                    acc[1] = fmaf(load_as_float(conv_w, wj + taps, w_dtype), x.y, acc[1]);
                    acc[2] = fmaf(load_as_float(conv_w, wj + 2 * taps, w_dtype), x.z, acc[2]);
                    acc[3] = fmaf(load_as_float(conv_w, wj + 3 * taps, w_dtype), x.w, acc[3]);
                }
            }
        }
        *reinterpret_cast<float4*>(y + c) = make_float4(acc[0], acc[1], acc[2], acc[3]);
        const float s4 = fmaf(acc[0], acc[0], fmaf(acc[1], acc[1], fmaf(acc[2], acc[2], acc[3] * acc[3])));
        if (c < cq) ssq += s4; else ssk += s4;
    }
    const bool slot_ok = slot >= 0 && slot < pool_slots;
    if (writes && !slot_ok && threadIdx.x == 0) atomicOr(status, MLS_STATUS_BAD_SLOT);
    ssq = warp_sum(ssq);
    ssk = warp_sum(ssk);
    if (lane == 0) {
        sums[warp][0] = ssq;
        sums[warp][1] = ssk;
    }
    __syncthreads();
    float tq = 0.f, tk = 0.f;
    for (int wv = 0; wv < (int)(blockDim.x >> 5); ++wv) {       // warps in order
        tq += sums[wv][0];
        tk += sums[wv][1];
    }
    const float inv_q = 1.0f / sqrtf(tq / (float)cq + eps);
    const float inv_k = 1.0f / sqrtf(tk / (float)ck + eps);
    const long long page = slot_ok ? slot / block_size : 0;
    const int off = slot_ok ? slot % block_size : 0;
    const long long n_pages = pool_slots / block_size;
    for (int c = threadIdx.x * 4; c < channels; c += blockDim.x * 4) {
        const bool is_q = c < cq;
        const int cc = is_q ? c : c - cq;
        const int e = cc % hd, g = cc / hd;
        const float inv = is_q ? inv_q : inv_k;
        const float4 raw4 = *reinterpret_cast<const float4*>(y + c);
        const float raw[4] = {raw4.x, raw4.y, raw4.z, raw4.w};
        const Four nw = load_four(is_q ? q_norm : k_norm, cc, w_dtype);
        float v[4];
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) v[q4] = raw[q4] * inv * nw.v[q4];
#pragma unroll
        for (int pr = 0; pr < 2; ++pr) {
            if (e + 2 * pr < rot_dims) {
                const float co = cs[(e >> 1) + pr], si = cs[half + (e >> 1) + pr];
                const float a = v[2 * pr], bb = v[2 * pr + 1];
                v[2 * pr] = __fsub_rn(__fmul_rn(a, co), __fmul_rn(bb, si));
                v[2 * pr + 1] = __fadd_rn(__fmul_rn(bb, co), __fmul_rn(a, si));
            }
        }
        if (is_q) {
            store_four<T>(q_out + (size_t)t * q_row + c, v);
        } else if (writes && slot_ok) {
            const size_t at = (((size_t)g * n_pages + page) * block_size + off) * hd + e;
            store_four<T>(k_pool + at, v);
            store_four<T>(v_pool + at, raw);           // the value: the convolved key as it is
        }
    }
    if (writes && slot_ok)
        clear_page_tail<T>(rest, slot, block_size, (int)n_pages, n_kv, hd, k_pool, v_pool);
}

template <typename T>
__global__ void __launch_bounds__(SC_THREADS)
token_shift_mix_kernel(const T* __restrict__ h, const void* __restrict__ mu, int w_dtype,
                       int n_mix, float* __restrict__ tail, long long tail_stride, int move_tail,
                       const int* __restrict__ state_slot, const int* __restrict__ cu_q,
                       const int* __restrict__ req_of_token, T* __restrict__ out,
                       float* __restrict__ out_f32, int n_tokens, int d) {
    chain_release();
    chain_wait();
    const int t = blockIdx.x;
    const int r = req_of_token[t];
    const bool first = t == cu_q[r];
    float* prev_tail = tail + (size_t)state_slot[r] * tail_stride;
#pragma unroll 4
    for (int c = threadIdx.x; c < d; c += SC_THREADS) {
        const float cur = Elem<T>::load(h + (size_t)t * d + c);
        const float prev = first ? prev_tail[c] : Elem<T>::load(h + (size_t)(t - 1) * d + c);
        const float diff = prev - cur;
        for (int s = 0; s < n_mix; ++s) {
            const float v = fmaf(diff, load_as_float(mu, (size_t)s * d + c, w_dtype), cur);
            // the last mix may be wanted in float32 (it feeds a float32 product)
            if (s == n_mix - 1 && out_f32) out_f32[(size_t)t * d + c] = v;
            else Elem<T>::store(out + ((size_t)s * n_tokens + t) * d + c, v);
        }
        // a step of one token a request: this row is the next step's previous row
        if (move_tail) prev_tail[c] = cur;
    }
}

// One thread a channel walks the tail's rows oldest first: row j becomes the input
// n_tail - j places before the end of the sequence as it is after this step, which is a
// row of this step or, for a short step, the old tail's row j + n (read before that row
// is written, since j + n > j).
template <typename T>
__global__ void __launch_bounds__(SC_THREADS)
tail_update_kernel(const T* __restrict__ src, int width, int col0, const void* __restrict__ bias,
                   int w_dtype, float* __restrict__ tail, long long tail_stride, int n_tail,
                   int channels, const int* __restrict__ state_slot,
                   const int* __restrict__ cu_q) {
    chain_release();
    chain_wait();
    const int r = blockIdx.y;
    const int row0 = cu_q[r], n = cu_q[r + 1] - row0;
    if (n <= 0) return;
    float* my = tail + (size_t)state_slot[r] * tail_stride;
    const int c = blockIdx.x * SC_THREADS + threadIdx.x;
    if (c >= channels) return;
    for (int j = 0; j < n_tail; ++j) {
        const int i = n - n_tail + j;
        float v;
        if (i >= 0) {
            v = Elem<T>::load(src + (size_t)(row0 + i) * width + col0 + c);
            if (bias) v += load_as_float(bias, c, w_dtype);
        } else {
            v = my[(size_t)(j + n) * channels + c];
        }
        my[(size_t)j * channels + c] = v;
    }
}
}  // namespace

MLS_API int mls_qk_conv_norm_rope_store(
        const float* proj, int n_parts, long long part_stride, const void* bias,
        const void* conv_w, int taps, const void* q_norm, const void* k_norm, int w_dtype,
        float eps, float* tail, long long tail_stride, int move_tail,
        const int* state_slot, const int* cu_q, const int* req_of_token, const int* positions,
        const double* freq, int rot_dims, void* q_out, int q_row, int act_dtype,
        const int* slot_map, void* k_pool, void* v_pool, int block_size, long long pool_slots,
        int n_tokens, int n_heads, int n_kv, int hd, int writes, int* status,
        cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (n_parts < 1) n_parts = 1;
    if (taps < 0 || (taps > 1 && !tail) || rot_dims < 0 || rot_dims > hd || (rot_dims & 1) ||
        rot_dims / 2 > SC_THREADS || (rot_dims > 0 && !freq))
        return MLS_ERR_UNSUPPORTED;
    const size_t smem = ((size_t)(n_heads + n_kv) * hd + rot_dims) * sizeof(float);
    if (smem > 200 * 1024) return MLS_ERR_UNSUPPORTED;
    // four channels a thread where every row allows it (the model's sizes alone decide)
    const bool vec4 = (((n_heads * hd) | hd | q_row) & 3) == 0 && (part_stride & 3) == 0 &&
                      taps <= QK_MAX_TAPS &&
                      (taps <= 1 || (tail_stride & 3) == 0);
    // (the block's shape depends on the model's sizes alone, and with it the order of the sums)
    const int threads = (vec4 && (n_heads + n_kv) * hd <= 4096 && rot_dims / 2 <= 128) ? 128 : SC_THREADS;
    if (act_dtype == MLS_BF16) {
        auto kernel = vec4 ? qk_conv_norm_rope_store_vec4_kernel<__nv_bfloat16>
                           : qk_conv_norm_rope_store_kernel<__nv_bfloat16>;
        if (smem > 48 * 1024) {
            const int rc = (int)cudaFuncSetAttribute(
                kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (rc) return rc;
        }
        MLS_LAUNCH(kernel, dim3(n_tokens), dim3(threads), smem, stream, proj, n_parts, part_stride, bias,
                   conv_w, taps, q_norm, k_norm, w_dtype, eps, tail, tail_stride, move_tail, state_slot, cu_q,
                   req_of_token, positions, freq, rot_dims, (__nv_bfloat16*)q_out, q_row, slot_map,
                   (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, block_size, pool_slots,
                   n_tokens, n_heads, n_kv, hd, writes, status);
    } else {
        auto kernel = vec4 ? qk_conv_norm_rope_store_vec4_kernel<float>
                           : qk_conv_norm_rope_store_kernel<float>;
        if (smem > 48 * 1024) {
            const int rc = (int)cudaFuncSetAttribute(
                kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (rc) return rc;
        }
        MLS_LAUNCH(kernel, dim3(n_tokens), dim3(threads), smem, stream, proj, n_parts, part_stride, bias,
                   conv_w, taps, q_norm, k_norm, w_dtype, eps, tail, tail_stride, move_tail, state_slot, cu_q,
                   req_of_token, positions, freq, rot_dims, (float*)q_out, q_row, slot_map,
                   (float*)k_pool, (float*)v_pool, block_size, pool_slots, n_tokens, n_heads,
                   n_kv, hd, writes, status);
    }
    return launch_status();
}

MLS_API int mls_token_shift_mix(const void* h, int act_dtype, const void* mu, int w_dtype,
                                int n_mix, float* tail, long long tail_stride, int move_tail,
                                const int* state_slot, const int* cu_q, const int* req_of_token,
                                void* out, float* out_f32, int n_tokens, int d,
                                cudaStream_t stream) {
    if (n_tokens <= 0 || n_mix <= 0) return 0;
    if (act_dtype == MLS_BF16)
        MLS_LAUNCH((token_shift_mix_kernel<__nv_bfloat16>), dim3(n_tokens), dim3(SC_THREADS), 0,
                   stream, (const __nv_bfloat16*)h, mu, w_dtype, n_mix, tail, tail_stride,
                   move_tail, state_slot, cu_q, req_of_token, (__nv_bfloat16*)out, out_f32, n_tokens, d);
    else
        MLS_LAUNCH((token_shift_mix_kernel<float>), dim3(n_tokens), dim3(SC_THREADS), 0, stream,
                   (const float*)h, mu, w_dtype, n_mix, tail, tail_stride, move_tail, state_slot, cu_q,
                   req_of_token, (float*)out, out_f32, n_tokens, d);
    return launch_status();
}

MLS_API int mls_tail_update(const void* src, int src_dtype, int width, int col0, const void* bias,
                            int w_dtype, float* tail, long long tail_stride, int n_tail,
                            int channels, const int* state_slot, const int* cu_q,
                            int n_requests, cudaStream_t stream) {
    if (n_requests <= 0 || n_tail <= 0 || channels <= 0) return 0;
    const dim3 grid((channels + SC_THREADS - 1) / SC_THREADS, n_requests);
    if (src_dtype == MLS_BF16)
        MLS_LAUNCH((tail_update_kernel<__nv_bfloat16>), grid, dim3(SC_THREADS), 0, stream,
                   (const __nv_bfloat16*)src, width, col0, bias, w_dtype, tail, tail_stride,
                   n_tail, channels, state_slot, cu_q);
    else
        MLS_LAUNCH((tail_update_kernel<float>), grid, dim3(SC_THREADS), 0, stream,
                   (const float*)src, width, col0, bias, w_dtype, tail, tail_stride, n_tail,
                   channels, state_slot, cu_q);
    return launch_status();
}
