// Attention over a compressed latent: what a step's tokens leave in the cache, and the products that stay per head.
//
// A token's down projection is [R latent elements | dr elements of a key part that all heads share]. The cache keeps
// one row per token, [rms(latent) * weight | that key part rotated by the token's position], which is the token's key
// (for every head) and, in its first R elements, its value. dd_latent_prepare writes that row straight into the
// request's page and rotates, in place, the last dr elements of every query head (a query head is [dk | dr]); norm,
// angles, cosines and sines are float32, neighbouring dimensions (2i, 2i + 1) form a pair, the first 2 * n_pairs
// elements of the dr turn and the rest pass unchanged.
//
// Scores against the plain part of a key, (W_uk c) . q, are computed as c . (W_uk^T q): dd_per_head_linear multiplies
// every head's piece of a row by that head's own matrix (out[t, h] = W[h] in[t, h], W [heads, J, I]) and copies `tail`
// further elements through unchanged (the rotated part of a query). The same kernel turns the attention's result, a
// weighted sum of latent rows per head, into the head's value by W_uv. A warp owns an output element for eight tokens:
// its lanes walk the matrix row together (coalesced), products are summed in float32 in an order that does not depend
// on the batch.
#include "common.cuh"

namespace {
template <typename T>
__global__ void __launch_bounds__(128)
latent_prepare_kernel(T* __restrict__ q, int q_stride, int H, int dk, int dr, const T* __restrict__ down, int down_stride,
                      int R, const float* __restrict__ weight, float eps, const float* __restrict__ freqs, int n_pairs,
                      const int* __restrict__ tok_entry, const int* __restrict__ tok_pos, const int* __restrict__ block_table,
                      int max_blocks, T* __restrict__ cache, int n_pages, int page_size, int* __restrict__ error_flag) {
    __shared__ float scratch[4];
    __shared__ float cs[2 * 128];                   // cosines, then sines, of this token's angles
    dd_launch_dependents();
    const int t = blockIdx.x;
    const int pos = tok_pos[t];
    const int block = pos / page_size;
    const int page = (pos >= 0 && block < max_blocks) ? block_table[(size_t)tok_entry[t] * max_blocks + block] : -1;
    for (int i = threadIdx.x; i < n_pairs; i += 128) {
        const float angle = (float)pos * freqs[i];
        cs[i] = cosf(angle);
        cs[128 + i] = sinf(angle);
    }
    dd_grid_wait();
    __syncthreads();
    // every query head's rotated part, in place
    for (int i = threadIdx.x; i < H * n_pairs; i += 128) {
        const int h = i / n_pairs, p = i % n_pairs;
        T* x = q + (size_t)t * q_stride + (size_t)h * (dk + dr) + dk + 2 * p;
        const float a = dd_to_f32(x[0]), b = dd_to_f32(x[1]);
        x[0] = dd_from_f32<T>(a * cs[p] - b * cs[128 + p]);
        x[1] = dd_from_f32<T>(b * cs[p] + a * cs[128 + p]);
    }
    if (page < 0 || page >= n_pages) {
        if (threadIdx.x == 0) atomicOr(error_flag, 2);
        return;
    }
    const T* src = down + (size_t)t * down_stride;
    T* row = cache + ((size_t)page * page_size + pos % page_size) * (R + dr);
    float sq = 0.f;
    for (int c = threadIdx.x; c < R; c += 128) {
        const float v = dd_to_f32(src[c]);
        sq = fmaf(v, v, sq);
    }
    sq = dd_warp_sum(sq);
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = sq;
    __syncthreads();
    const float r = 1.0f / sqrtf((scratch[0] + scratch[1] + scratch[2] + scratch[3]) / (float)R + eps);
    for (int c = threadIdx.x; c < R; c += 128) row[c] = dd_from_f32<T>(dd_to_f32(src[c]) * r * weight[c]);
    for (int p = threadIdx.x; p < dr / 2 + (dr & 1); p += 128) {
        const int c = 2 * p;
        if (p < n_pairs) {
            const float a = dd_to_f32(src[R + c]), b = dd_to_f32(src[R + c + 1]);
            row[R + c] = dd_from_f32<T>(a * cs[p] - b * cs[128 + p]);
            row[R + c + 1] = dd_from_f32<T>(b * cs[p] + a * cs[128 + p]);
        } else {
            row[R + c] = src[R + c];
            if (c + 1 < dr) row[R + c + 1] = src[R + c + 1];
        }
    }
}

constexpr int PH_TOKENS = 8;

template <typename T>
__global__ void __launch_bounds__(128)
per_head_linear_kernel(const T* __restrict__ in, int in_stride, int in_head, const T* __restrict__ w, T* __restrict__ out,
                       int out_stride, int out_head, int n, int I, int J, int tail, int j_per_block) {
    extern __shared__ float rows[];                 // [PH_TOKENS][I]
    dd_launch_dependents();
    const int t0 = blockIdx.x * PH_TOKENS, h = blockIdx.y;
    const int nt = min(PH_TOKENS, n - t0);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    dd_grid_wait();
    for (int i = threadIdx.x; i < PH_TOKENS * I; i += 128) {
        const int tt = i / I, c = i % I;
        rows[i] = tt < nt ? dd_to_f32(in[(size_t)(t0 + tt) * in_stride + (size_t)h * in_head + c]) : 0.f;
    }
    if (blockIdx.z == 0)
        for (int i = threadIdx.x; i < nt * tail; i += 128) {
            const int tt = i / tail, c = i % tail;
            out[(size_t)(t0 + tt) * out_stride + (size_t)h * out_head + J + c] =
                in[(size_t)(t0 + tt) * in_stride + (size_t)h * in_head + I + c];
        }
    __syncthreads();
    const int j0 = blockIdx.z * j_per_block, j1 = min(J, j0 + j_per_block);
    for (int j = j0 + warp; j < j1; j += 4) {
        const T* wr = w + ((size_t)h * J + j) * I;
        float acc[PH_TOKENS];
#pragma unroll
        for (int tt = 0; tt < PH_TOKENS; ++tt) acc[tt] = 0.f;
        for (int c = lane; c < I; c += 32) {
            const float f = dd_to_f32(wr[c]);
#pragma unroll
            for (int tt = 0; tt < PH_TOKENS; ++tt) acc[tt] = fmaf(f, rows[tt * I + c], acc[tt]);
        }
        float mine = 0.f;
#pragma unroll
        for (int tt = 0; tt < PH_TOKENS; ++tt) {
            const float total = dd_warp_sum(acc[tt]);
            if (lane == tt) mine = total;
        }
        if (lane < nt) out[(size_t)(t0 + lane) * out_stride + (size_t)h * out_head + j] = dd_from_f32<T>(mine);
    }
}
}  // namespace

// q: [N, q_stride], head h at h * (dk + dr), its last dr elements are rotated in place. down: [N, down_stride] rows of
// R + dr elements. cache: [n_pages, page_size * (R + dr)]. freqs: float32 [n_pairs], 2 * n_pairs <= dr, at most 128
// pairs. Error bit 2: a token without a page.
DD_API int dd_latent_prepare(void* q, int q_stride, int H, int dk, int dr, const void* down, int down_stride, int R,
                             const float* weight, float eps, const float* freqs, int n_pairs, const int* tok_entry,
                             const int* tok_pos, const int* block_table, int max_blocks, void* cache, int n_pages,
                             int page_size, int n, int dtype, int* error_flag, void* stream) {
    if (n <= 0) return 0;
    if (n_pairs < 0 || n_pairs > 128 || 2 * n_pairs > dr) return dd_fail("dd_latent_prepare: %d pairs do not fit a rotated part of %d (at most 128 pairs)", n_pairs, dr);
    if (H <= 0 || dk < 0 || R <= 0) return dd_fail("dd_latent_prepare: bad sizes");
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == DD_F32)
        dd_launch(latent_prepare_kernel<float>, dim3(n), dim3(128), 0, s, (float*)q, q_stride, H, dk, dr, (const float*)down,
                  down_stride, R, weight, eps, freqs, n_pairs, tok_entry, tok_pos, block_table, max_blocks, (float*)cache, n_pages,
                  page_size, error_flag);
    else if (dtype == DD_BF16)
        dd_launch(latent_prepare_kernel<__nv_bfloat16>, dim3(n), dim3(128), 0, s, (__nv_bfloat16*)q, q_stride, H, dk, dr,
                  (const __nv_bfloat16*)down, down_stride, R, weight, eps, freqs, n_pairs, tok_entry, tok_pos, block_table,
                  max_blocks, (__nv_bfloat16*)cache, n_pages, page_size, error_flag);
    else
        return dd_fail("dd_latent_prepare: unknown dtype %d", dtype);
    return dd_check_launch("dd_latent_prepare");
}

// in: [N, in_stride], head h's I inputs (and `tail` more elements that are copied) at h * in_head; w: [heads, J, I];
// out: [N, out_stride], head h's J outputs (then the tail) at h * out_head. One element type for all three.
DD_API int dd_per_head_linear(const void* in, int in_stride, int in_head, const void* w, void* out, int out_stride,
                              int out_head, int n, int heads, int I, int J, int tail, int dtype, void* stream) {
    if (n <= 0 || heads <= 0) return 0;
    if (I <= 0 || J <= 0 || tail < 0) return dd_fail("dd_per_head_linear: bad sizes");
    const size_t smem = (size_t)PH_TOKENS * I * sizeof(float);
    if (smem > 200 * 1024) return dd_fail("dd_per_head_linear: %d inputs a head are more than a block holds", I);
    cudaStream_t s = (cudaStream_t)stream;
    const int tiles = dd_ceil_div(n, PH_TOKENS);
    // few tokens: a head's outputs are spread over more blocks, so that the matrices stream through many SMs
    int j_per_block = J;
    while (j_per_block > 16 && (long long)tiles * heads * dd_ceil_div(J, j_per_block) < 296) j_per_block = (j_per_block + 1) / 2;
    const dim3 grid(tiles, heads, dd_ceil_div(J, j_per_block));
#define DD_PHL(T)                                                                                                    \
    do {                                                                                                             \
        if (smem > 48 * 1024)                                                                                        \
            cudaFuncSetAttribute(per_head_linear_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);  \
        dd_launch(per_head_linear_kernel<T>, grid, dim3(128), smem, s, (const T*)in, in_stride, in_head, (const T*)w,  \
                  (T*)out, out_stride, out_head, n, I, J, tail, j_per_block);                                        \
    } while (0)
    if (dtype == DD_F32) DD_PHL(float);
    else if (dtype == DD_BF16) DD_PHL(__nv_bfloat16);
    else return dd_fail("dd_per_head_linear: unknown dtype %d", dtype);
#undef DD_PHL
    return dd_check_launch("dd_per_head_linear");
}
