// Clearing the rest of a page that a request enters in a step (shared by the kernels
// that write a step's tokens into the pages).
#pragma once
#include "common.cuh"

// What lies in a page past its owner's last token is whatever the page's previous owner
// left there.  The attention kernels never count those slots, but the tensor-core ones
// mask the scores, not the values: a probability of 0 times a leftover NaN or Inf would
// still be NaN.  So the slots are cleared when a request enters a page: the token that
// is the last of its request in this step zeroes the rest of its page (keys and values
// of every kv head) if the page's first slot was written in this step too.  Pages are
// owned by one request, so "the next token has the next slot" means "same request", and
// "the token `off` places back has this page's first slot" means the page was entered
// in this step.  Cleared by all threads of one block per token, after chain_wait().
// How many slots after `slot` are to be cleared by token t's block (0: none).  Reads only
// the step's slot map, which no kernel of the step writes: callers ask before chain_wait,
// so that the two loads do not add to what follows the wait.
__device__ __forceinline__ int page_tail_to_clear(const int* __restrict__ slot_map, int t,
                                                  int n_tokens, int slot, int block_size) {
    const int off = slot % block_size;
    const int rest = block_size - 1 - off;
    if (rest <= 0 || slot < 0) return 0;
    const int next = t + 1 < n_tokens ? slot_map[t + 1] : -1;
    const int first = (off > 0 && t - off >= 0) ? slot_map[t - off] : -1;
    if (next == slot + 1) return 0;                                     // not the last one
    if (off > 0 && first != slot - off) return 0;                       // an older page
    return rest;
}
template <typename T>
__device__ __forceinline__ void clear_page_tail(int rest, int slot, int block_size, int n_pages,
                                                int n_kv, int hd, T* __restrict__ k_pool,
                                                T* __restrict__ v_pool) {
    if (rest <= 0) return;
    const int page = slot / block_size, off = slot - page * block_size;
    const size_t row_bytes = (size_t)hd * sizeof(T);
    if (row_bytes % 16 == 0) {
        const int chunks = (int)(row_bytes / 16) * rest;                 // per kv head and pool
        for (int u = threadIdx.x; u < 2 * n_kv * chunks; u += blockDim.x) {
            const int which = u / (n_kv * chunks), w = u - which * n_kv * chunks;
            const int kvh = w / chunks, c = w - kvh * chunks;
            T* base = (which ? v_pool : k_pool) +
                      (((size_t)kvh * n_pages + page) * block_size + off + 1) * hd;
            reinterpret_cast<uint4*>(base)[c] = make_uint4(0u, 0u, 0u, 0u);
        }
    } else {
        const int elems = hd * rest;
        for (int u = threadIdx.x; u < 2 * n_kv * elems; u += blockDim.x) {
            const int which = u / (n_kv * elems), w = u - which * n_kv * elems;
            const int kvh = w / elems, c = w - kvh * elems;
            T* base = (which ? v_pool : k_pool) +
                      (((size_t)kvh * n_pages + page) * block_size + off + 1) * hd;
            Elem<T>::store(base + c, 0.f);
        }
    }
}

