// Token embedding with a hashed table of token pairs added: x[t] = tokens[id[t]] + pairs[row(t)], float32.
// row(t) = (id[t-1] * mul_prev + id[t] * mul_cur) mod buckets; a sequence's first token takes row `buckets` (the table's
// last). The token before a step's first token of a request is per-request state (one int32 per slot): the block of an
// entry's first token reads it and then leaves the entry's last id there for the next step.
#include "common.cuh"

template <typename T>
__global__ void embed_pairs_kernel(const int* __restrict__ ids, const int* __restrict__ pos, const int* __restrict__ tok_entry,
                                   const int* __restrict__ entry_start, const int* __restrict__ entry_slot,
                                   const T* __restrict__ tokens, const T* __restrict__ pairs, int* __restrict__ last_id,
                                   float* __restrict__ out, int width, int vocab, int buckets, long long mul_prev,
                                   long long mul_cur, int* __restrict__ error_flag) {
    dd_launch_dependents();
    dd_grid_wait();
    __shared__ int row_of_pair;
    const int t = blockIdx.x;
    int id = ids[t];
    if (id < 0 || id >= vocab) {
        if (threadIdx.x == 0) atomicOr(error_flag, 1);
        id = min(max(id, 0), vocab - 1);
    }
    if (threadIdx.x == 0) {
        const int e = tok_entry[t];
        const int start = entry_start[e];
        int before = -1;
        if (t == start) {
            int* kept = last_id + entry_slot[e];
            before = *kept;
            int last = ids[entry_start[e + 1] - 1];
            *kept = min(max(last, 0), vocab - 1);
        } else {
            before = min(max(ids[t - 1], 0), vocab - 1);
        }
        row_of_pair = pos[t] == 0 ? buckets : (int)(((long long)before * mul_prev + (long long)id * mul_cur) % buckets);
    }
    __syncthreads();
    const T* a = tokens + (size_t)id * width;
    const T* b = pairs + (size_t)row_of_pair * width;
    float* o = out + (size_t)t * width;
    for (int c = threadIdx.x; c < width; c += blockDim.x) o[c] = dd_to_f32(a[c]) + dd_to_f32(b[c]);
}

// last_id: int32 [slots]; pairs: [buckets + 1, width] in the token table's dtype.
DD_API int dd_embed_pairs(const int* ids, const int* pos, const int* tok_entry, const int* entry_start, const int* entry_slot,
                          const void* tokens, const void* pairs, int* last_id, float* out, int n_tokens, int width, int vocab,
                          int buckets, long long mul_prev, long long mul_cur, int table_dtype, int* error_flag, void* stream) {
    if (n_tokens <= 0) return 0;
    if (width <= 0 || vocab <= 0 || buckets <= 0 || mul_prev < 0 || mul_cur < 0)
        return dd_fail("dd_embed_pairs: bad sizes width=%d vocab=%d buckets=%d", width, vocab, buckets);
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = width >= 1024 ? 256 : 128;
    if (table_dtype == DD_F32)
        dd_launch(embed_pairs_kernel<float>, dim3(n_tokens), dim3(threads), 0, s, ids, pos, tok_entry, entry_start, entry_slot,
                  (const float*)tokens, (const float*)pairs, last_id, out, width, vocab, buckets, mul_prev, mul_cur, error_flag);
    else if (table_dtype == DD_BF16)
        dd_launch(embed_pairs_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(threads), 0, s, ids, pos, tok_entry, entry_start,
                  entry_slot, (const __nv_bfloat16*)tokens, (const __nv_bfloat16*)pairs, last_id, out, width, vocab, buckets,
                  mul_prev, mul_cur, error_flag);
    else
        return dd_fail("dd_embed_pairs: unknown table dtype %d", table_dtype);
    return dd_check_launch("dd_embed_pairs");
}
