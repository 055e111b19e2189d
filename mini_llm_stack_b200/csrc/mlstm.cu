// mLSTM: a matrix memory per head with exponential input and forget gates, carried
// from token to token in a float32 state slot per request.
//
// Per head, with query/key size e and value size f (q pre-scaled by e^-1/2):
//   i = cap * tanh((zi + bi) / cap)                       log input gate
//   g = logsigmoid(cap * tanh((zf + bf) / cap))           log forget gate
//   m' = max(g + m, i)                                    stabiliser, m starts at 0
//   C' = exp(g + m - m') C + exp(i - m') k v^T            C [e, f]
//   n' = exp(g + m - m') n + exp(i - m') k                n [e]
//   num = C'^T q,  den = max(|n' . q|, exp(-m')) + 1e-6
// mls_mlstm_scan walks the tokens of every request of the step in order, from the state
// the slot holds, and leaves num [T, H*f] and den [T, H] (float32); the state goes back
// to the slot.  mls_mlstm_finish then forms o = num / den, divides each head's o by its
// root mean square (eps inside the root), multiplies by the norm weight and by
// sigmoid(gate) and rounds once to the activation type.
//
// A CTA owns FC columns of one head's C for one request and keeps them in registers:
// thread (col, eg) holds a run of rows of its column.  Only the CTA of a
// head's first columns carries n (a thread holds the elements tid, tid + 256, ...); every
// CTA carries its own copy of m (the state row of a head is
// [C (e*f) | n (e) | m (one per column group)]), so no CTA reads what another writes.
// Tokens are taken TB at a time: one pass loads their q, k, v and gates into shared
// memory, then every thread walks the block token by token: the scalar recurrence of m,
// its rows of C, the token's partial output; the partial outputs and the partial n . q
// are added up once a block, in a fixed order.  All gate
// arithmetic, the state and the sums are float32; q, k, v and the gate pre-activations
// come from the projections.  A token's result depends on the tokens before it only
// through the state, never on the batch or on how the sequence was cut into steps.
#include "common.cuh"

namespace {
constexpr int SCAN_THREADS = 256;
constexpr int TB = 16;                      // tokens a pass
constexpr int MAXN = 4;                     // elements of n a thread holds: e <= 1024

__device__ __forceinline__ float soft_cap(float z, float cap) { return cap * tanhf(z / cap); }
__device__ __forceinline__ float log_sigmoid(float z) {
    return fminf(z, 0.f) - log1pf(expf(-fabsf(z)));
}

// 16 bytes of a row as floats.
__device__ __forceinline__ void load16(const float* p, float (&out)[4]) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
}
__device__ __forceinline__ void load16(const __nv_bfloat16* p, float (&out)[8]) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int x = 0; x < 4; ++x) {
        const float2 f2 = __bfloat1622float2(h[x]);
        out[2 * x] = f2.x;
        out[2 * x + 1] = f2.y;
    }
}

// MAXR: most rows of C a thread holds.
template <typename T, int MAXR>
__global__ void __launch_bounds__(SCAN_THREADS, MAXR <= 16 ? 2 : 1)
mlstm_scan_kernel(const T* __restrict__ qkvg, int row_w, int q_off, int k_off, int v_off,
                  const float* __restrict__ gates /* [T, 2H]: zi | zf */,
                  const void* __restrict__ bias_i, const void* __restrict__ bias_f, int b_dtype,
                  float cap, const int* __restrict__ cu_q, const int* __restrict__ state_slot,
                  float* __restrict__ state, long long slot_stride, int n_heads, int e, int f,
                  int fc, int n_groups, float* __restrict__ num, float* __restrict__ den) {
    chain_release();
    chain_wait();
    extern __shared__ float sm[];
    const int grp = blockIdx.x, head = blockIdx.y, req = blockIdx.z;
    const int eg_count = SCAN_THREADS / fc;
    const int col = threadIdx.x % fc, eg = threadIdx.x / fc;
    const int gcol = grp * fc + col;
    const bool active = eg < eg_count && gcol < f;
    const bool first = grp == 0;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float* q_s = sm;                           // [TB][e]
    float* k_s = q_s + TB * e;                 // [TB][e]
    float* v_s = k_s + TB * e;                 // [TB][fc]
    float* part = v_s + TB * fc;               // [TB][eg_count][fc]
    float* gate_s = part + TB * eg_count * fc; // [2][TB]: log input gate, log forget gate
    float* nq_s = gate_s + 2 * TB;             // [TB][8 warps]
    float* m_s = nq_s + TB * 8;                // [TB]: the stabiliser after each token

    const int t0 = cu_q[req], t1 = cu_q[req + 1];
    float* st = state + (size_t)state_slot[req] * slot_stride +
                (size_t)head * ((size_t)e * f + e + n_groups);
    // a thread's rows lie side by side, so that k and q come from shared memory four at a time
    const int rows_per = (e + eg_count - 1) / eg_count;
    const int row0 = eg * rows_per;
    const bool vec = (rows_per & 3) == 0 && (e & 3) == 0;
    float C[MAXR];
#pragma unroll
    for (int r = 0; r < MAXR; ++r) {
        const int row = row0 + r;
        C[r] = (active && r < rows_per && row < e) ? st[(size_t)row * f + gcol] : 0.f;
    }
    float nreg[MAXN];
#pragma unroll
    for (int x = 0; x < MAXN; ++x) {
        const int i = threadIdx.x + x * SCAN_THREADS;
        nreg[x] = (first && i < e) ? st[(size_t)e * f + i] : 0.f;
    }
    float m = st[(size_t)e * f + e + grp];
    const float bi = load_as_float(bias_i, head, b_dtype), bf = load_as_float(bias_f, head, b_dtype);
    const float q_scale = 1.0f / sqrtf((float)e);
    constexpr int V = 16 / (int)sizeof(T);
    const bool vload = e % V == 0 && row_w % V == 0 && q_off % V == 0 && k_off % V == 0 &&
                       reinterpret_cast<uintptr_t>(qkvg) % 16 == 0;

    for (int tb = t0; tb < t1; tb += TB) {
        const int nb = min(TB, t1 - tb);
        // ---- the block's inputs (16 bytes a load where the layout allows)
        if (vload) {
            const int per_row = e / V;
            for (int u = threadIdx.x; u < nb * per_row; u += SCAN_THREADS) {
                const int j = u / per_row, i = (u - j * per_row) * V;
                const T* row = qkvg + (size_t)(tb + j) * row_w + head * e + i;
                float qv[V], kv[V];
                load16(row + q_off, qv);
                load16(row + k_off, kv);
#pragma unroll
                for (int x = 0; x < V; x += 4) {         // e and i are multiples of 4: 16-byte stores
                    *reinterpret_cast<float4*>(q_s + j * e + i + x) = make_float4(
                        qv[x] * q_scale, qv[x + 1] * q_scale, qv[x + 2] * q_scale, qv[x + 3] * q_scale);
                    *reinterpret_cast<float4*>(k_s + j * e + i + x) =
                        make_float4(kv[x], kv[x + 1], kv[x + 2], kv[x + 3]);
                }
            }
        } else {
            for (int u = threadIdx.x; u < nb * e; u += SCAN_THREADS) {
                const int j = u / e, i = u - j * e;
                const T* row = qkvg + (size_t)(tb + j) * row_w;
                q_s[j * e + i] = Elem<T>::load(row + q_off + head * e + i) * q_scale;
                k_s[j * e + i] = Elem<T>::load(row + k_off + head * e + i);
            }
        }
        for (int u = threadIdx.x; u < nb * fc; u += SCAN_THREADS) {
            const int j = u / fc, c = u - j * fc;
            v_s[u] = grp * fc + c < f
                         ? Elem<T>::load(qkvg + (size_t)(tb + j) * row_w + v_off + head * f + grp * fc + c)
                         : 0.f;
        }
        if (threadIdx.x < nb) {
            const float* gr = gates + (size_t)(tb + threadIdx.x) * 2 * n_heads;
            gate_s[threadIdx.x] = soft_cap(gr[head] + bi, cap);
            gate_s[TB + threadIdx.x] = log_sigmoid(soft_cap(gr[n_heads + head] + bf, cap));
        }
        __syncthreads();
        // ---- token by token: the stabiliser (walked by every thread for itself), C and the
        // token's partial output, n and the partial n . q
#pragma unroll 2
        for (int j = 0; j < nb; ++j) {
            const float ig = gate_s[j], fg = gate_s[TB + j];
            const float m_new = fmaxf(fg + m, ig);
            const float keep = expf(fg + m - m_new), take = expf(ig - m_new);
            m = m_new;
            if (threadIdx.x == 0) m_s[j] = m;
            if (active) {
                const float tv = take * v_s[j * fc + col];
                const float* kj = k_s + j * e;
                const float* qj = q_s + j * e;
                // four sums side by side (the order is fixed by the row's place, not by the data)
                float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
                if (vec) {
#pragma unroll
                    for (int r = 0; r < MAXR; r += 4) {
                        if (r < rows_per && row0 + r < e) {
                            const float4 k4 = *reinterpret_cast<const float4*>(kj + row0 + r);
                            const float4 q4 = *reinterpret_cast<const float4*>(qj + row0 + r);
                            C[r] = fmaf(keep, C[r], k4.x * tv);
                            C[r + 1] = fmaf(keep, C[r + 1], k4.y * tv);
                            C[r + 2] = fmaf(keep, C[r + 2], k4.z * tv);
                            C[r + 3] = fmaf(keep, C[r + 3], k4.w * tv);
                            o0 = fmaf(C[r], q4.x, o0);
                            o1 = fmaf(C[r + 1], q4.y, o1);
                            o2 = fmaf(C[r + 2], q4.z, o2);
                            o3 = fmaf(C[r + 3], q4.w, o3);
                        }
                    }
                } else {
#pragma unroll
                    for (int r = 0; r < MAXR; ++r) {
                        const int rr = row0 + r;
                        if (r < rows_per && rr < e) {
                            C[r] = fmaf(keep, C[r], kj[rr] * tv);
                            o0 = fmaf(C[r], qj[rr], o0);
                        }
                    }
                }
                part[(j * eg_count + eg) * fc + col] = (o0 + o1) + (o2 + o3);
            }
            if (first) {
                float nq = 0.f;
#pragma unroll
                for (int x = 0; x < MAXN; ++x) {
                    const int i = threadIdx.x + x * SCAN_THREADS;
                    if (i < e) {
                        nreg[x] = fmaf(keep, nreg[x], take * k_s[j * e + i]);
                        nq = fmaf(nreg[x], q_s[j * e + i], nq);
                    }
                }
                nq = warp_sum(nq);
                if (lane == 0) nq_s[j * 8 + warp] = nq;
            }
        }
        __syncthreads();
        // ---- add up: the column groups' partial outputs, the warps' partial n . q
        for (int u = threadIdx.x; u < nb * fc; u += SCAN_THREADS) {
            const int j = u / fc, c = u - j * fc;
            if (grp * fc + c < f) {
                float s2 = 0.f;
                for (int g2 = 0; g2 < eg_count; ++g2) s2 += part[(j * eg_count + g2) * fc + c];
                num[(size_t)(tb + j) * n_heads * f + (size_t)head * f + grp * fc + c] = s2;
            }
        }
        if (first && threadIdx.x < nb) {
            const int j = threadIdx.x;
            float nq = 0.f;
            for (int w2 = 0; w2 < 8; ++w2) nq += nq_s[j * 8 + w2];
            den[(size_t)(tb + j) * n_heads + head] = fmaxf(fabsf(nq), expf(-m_s[j])) + 1e-6f;
        }
        __syncthreads();
    }
#pragma unroll
    for (int r = 0; r < MAXR; ++r) {
        const int row = row0 + r;
        if (active && r < rows_per && row < e) st[(size_t)row * f + gcol] = C[r];
    }
    if (first) {
#pragma unroll
        for (int x = 0; x < MAXN; ++x) {
            const int i = threadIdx.x + x * SCAN_THREADS;
            if (i < e) st[(size_t)e * f + i] = nreg[x];
        }
    }
    if (threadIdx.x == 0) st[(size_t)e * f + e + grp] = m;
}

template <typename T>
__global__ void mlstm_finish_kernel(const float* __restrict__ num, const float* __restrict__ den,
                                    const T* __restrict__ gate, int gate_row, int g_off,
                                    const void* __restrict__ w, int w_dtype, float eps,
                                    T* __restrict__ out, int n_heads, int f) {
    chain_release();
    chain_wait();
    // one warp a (token, head)
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long unit = (long long)blockIdx.x * (blockDim.x >> 5) + warp;
    const int t = (int)(unit / n_heads), head = (int)(unit % n_heads);
    const float d = den[unit];
    const float* nr = num + (size_t)unit * f;
    float ss = 0.f;
    for (int j = lane; j < f; j += 32) {
        const float o = nr[j] / d;
        ss = fmaf(o, o, ss);
    }
    const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)f + eps);
    for (int j = lane; j < f; j += 32) {
        const float o = nr[j] / d;
        const float z = Elem<T>::load(gate + (size_t)t * gate_row + g_off + head * f + j);
        Elem<T>::store(out + (size_t)unit * f + j,
                       o * inv * load_as_float(w, head * f + j, w_dtype) / (1.0f + expf(-z)));
    }
}

template <typename T, int MAXR>
int launch_scan(const void* qkvg, int row_w, int q_off, int k_off, int v_off, const float* gates,
                const void* bi, const void* bf, int b_dtype, float cap, const int* cu_q,
                const int* state_slot, float* state, long long slot_stride, int n_requests,
                int n_heads, int e, int f, int fc, int n_groups, float* num, float* den,
                cudaStream_t stream) {
    const int eg_count = SCAN_THREADS / fc;
    const size_t smem = (size_t)(2 * TB * e + TB * fc + TB * eg_count * fc + 2 * TB + TB * 8 + TB) *
                        sizeof(float);
    if (smem > 200 * 1024) return MLS_ERR_UNSUPPORTED;
    if (smem > 48 * 1024) {
        const int rc = (int)cudaFuncSetAttribute(mlstm_scan_kernel<T, MAXR>,
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 (int)smem);
        if (rc) return rc;
    }
    MLS_LAUNCH((mlstm_scan_kernel<T, MAXR>), dim3(n_groups, n_heads, n_requests),
               dim3(SCAN_THREADS), smem, stream, (const T*)qkvg, row_w, q_off, k_off, v_off, gates,
               bi, bf, b_dtype, cap, cu_q, state_slot, state, slot_stride, n_heads, e, f, fc,
               n_groups, num, den);
    return launch_status();
}

template <typename T>
int pick_scan(int maxr, const void* qkvg, int row_w, int q_off, int k_off, int v_off,
              const float* gates, const void* bi, const void* bf, int b_dtype, float cap,
              const int* cu_q, const int* state_slot, float* state, long long slot_stride,
              int n_requests, int n_heads, int e, int f, int fc, int n_groups, float* num,
              float* den, cudaStream_t stream) {
#define MLS_SCAN(R)                                                                            \
    return launch_scan<T, R>(qkvg, row_w, q_off, k_off, v_off, gates, bi, bf, b_dtype, cap,    \
                             cu_q, state_slot, state, slot_stride, n_requests, n_heads, e, f,  \
                             fc, n_groups, num, den, stream)
    if (maxr <= 4) MLS_SCAN(4);
    if (maxr <= 8) MLS_SCAN(8);
    if (maxr <= 16) MLS_SCAN(16);
    if (maxr <= 32) MLS_SCAN(32);
    if (maxr <= 64) MLS_SCAN(64);
#undef MLS_SCAN
    return MLS_ERR_UNSUPPORTED;
}
}  // namespace

// Columns of C a CTA owns for heads of (e, f): as many as leave a thread at most 64 rows,
// at most 16 (one prompt then makes enough CTAs for the GPU, two to an SM) and at most f.  The state row of a head is e*f + e + ceil(f / columns)
// floats.
MLS_API int mls_mlstm_columns(int e, int f) {
    int fc = f < 16 ? f : 16;
    while (fc > 1 && (e + (SCAN_THREADS / fc) - 1) / (SCAN_THREADS / fc) > 64) fc = (fc + 1) / 2;
    return fc;
}

MLS_API int mls_mlstm_scan(const void* qkvg, int dtype, int row_w, int q_off, int k_off, int v_off,
                           const float* gates, const void* bias_i, const void* bias_f, int b_dtype,
                           float cap, const int* cu_q, const int* state_slot, float* state,
                           long long slot_stride, int n_requests, int n_heads, int e, int f,
                           float* num, float* den, cudaStream_t stream) {
    if (n_requests <= 0) return 0;
    if (e <= 0 || e > MAXN * SCAN_THREADS || f <= 0 || n_heads <= 0 || n_heads > 65535 ||
        n_requests > 65535)
        return MLS_ERR_UNSUPPORTED;
    const int fc = mls_mlstm_columns(e, f);
    const int eg_count = SCAN_THREADS / fc;
    const int maxr = (e + eg_count - 1) / eg_count;
    const int n_groups = (f + fc - 1) / fc;
    if (dtype == MLS_BF16)
        return pick_scan<__nv_bfloat16>(maxr, qkvg, row_w, q_off, k_off, v_off, gates, bias_i,
                                        bias_f, b_dtype, cap, cu_q, state_slot, state, slot_stride,
                                        n_requests, n_heads, e, f, fc, n_groups, num, den, stream);
    return pick_scan<float>(maxr, qkvg, row_w, q_off, k_off, v_off, gates, bias_i, bias_f, b_dtype,
                            cap, cu_q, state_slot, state, slot_stride, n_requests, n_heads, e, f,
                            fc, n_groups, num, den, stream);
}

MLS_API int mls_mlstm_finish(const float* num, const float* den, const void* gate, int gate_row,
                             int g_off, const void* w, int w_dtype, float eps, void* out, int dtype,
                             int n_tokens, int n_heads, int f, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    const long long units = (long long)n_tokens * n_heads;
    // units is a multiple of nothing in particular: the last block's spare warps would read
    // past the end, so blocks of one warp when it does not divide
    const int warps = units % 4 == 0 ? 4 : 1;
    const int blocks = (int)(units / warps);
    if (dtype == MLS_BF16)
        MLS_LAUNCH((mlstm_finish_kernel<__nv_bfloat16>), dim3(blocks), dim3(32 * warps), 0, stream,
                   num, den, (const __nv_bfloat16*)gate, gate_row, g_off, w, w_dtype, eps,
                   (__nv_bfloat16*)out, n_heads, f);
    else
        MLS_LAUNCH((mlstm_finish_kernel<float>), dim3(blocks), dim3(32 * warps), 0, stream, num, den,
                   (const float*)gate, gate_row, g_off, w, w_dtype, eps, (float*)out, n_heads, f);
    return launch_status();
}
