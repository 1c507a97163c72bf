// Small float32 operations on rows of the residual stream and on a projection's output:
//   dd_tanh_norm          out = tanh(alpha * x) * w + b (a norm without statistics), optional row gather
//   dd_add_rows           x += other + vec (another stream and/or one vector for every row)
//   dd_norm_pair_add      x += half * (l / rms(l) * wl + r / rms(r) * wr): two results, each RMS-normed, averaged into the stream
//   dd_wide_norm_rotary   queries and keys RMS-normed over their whole projection (all heads at once, a weight per
//                         element), then the first dimensions of every head rotated by position * frequency
//   dd_sigmoid_gate       x *= sigmoid(gate), element by element, x and gate row views
//   dd_tanh_cap           x = cap * tanh(x / cap)
// Everything is computed in float32 whatever the storage type.
#include "common.cuh"

namespace {
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    v = dd_warp_sum(v);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = (blockDim.x + 31) >> 5;
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float total = 0.f;
    for (int i = 0; i < warps; ++i) total += scratch[i];        // every thread adds in one order
    return total;
}

template <typename T>
__global__ void __launch_bounds__(256)
tanh_norm_kernel(const float* __restrict__ x, const int* __restrict__ row_index, const float* __restrict__ alpha,
                 const float* __restrict__ w, const float* __restrict__ b, T* __restrict__ out, int width) {
    dd_launch_dependents();
    const float a = alpha[0];
    dd_grid_wait();
    const int row = blockIdx.x;
    const float* in = x + (size_t)(row_index ? row_index[row] : row) * width;
    T* o = out + (size_t)row * width;
    if ((width & 3) == 0) {
        for (int c = threadIdx.x * 4; c < width; c += blockDim.x * 4) {
            const float4 v = *reinterpret_cast<const float4*>(in + c);
            const float4 g = *reinterpret_cast<const float4*>(w + c);
            const float4 s = *reinterpret_cast<const float4*>(b + c);
            o[c] = dd_from_f32<T>(fmaf(tanhf(a * v.x), g.x, s.x));
            o[c + 1] = dd_from_f32<T>(fmaf(tanhf(a * v.y), g.y, s.y));
            o[c + 2] = dd_from_f32<T>(fmaf(tanhf(a * v.z), g.z, s.z));
            o[c + 3] = dd_from_f32<T>(fmaf(tanhf(a * v.w), g.w, s.w));
        }
    } else {
        for (int c = threadIdx.x; c < width; c += blockDim.x) o[c] = dd_from_f32<T>(fmaf(tanhf(a * in[c]), w[c], b[c]));
    }
}

__global__ void __launch_bounds__(256)
add_rows_kernel(float* __restrict__ x, const float* __restrict__ other, const float* __restrict__ vec, int width) {
    dd_launch_dependents();
    dd_grid_wait();
    const size_t at = (size_t)blockIdx.x * width;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float v = x[at + c];
        if (other) v += other[at + c];
        if (vec) v += vec[c];
        x[at + c] = v;
    }
}

__global__ void __launch_bounds__(256)
norm_pair_add_kernel(float* __restrict__ x, const float* __restrict__ left, const float* __restrict__ right,
                     const float* __restrict__ wl, const float* __restrict__ wr, float eps, float half, int width) {
    __shared__ float scratch[8];
    dd_launch_dependents();
    dd_grid_wait();
    const size_t at = (size_t)blockIdx.x * width;
    float sl = 0.f, sr = 0.f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const float l = left[at + c], r = right[at + c];
        sl = fmaf(l, l, sl);
        sr = fmaf(r, r, sr);
    }
    const float rl = rsqrtf(block_sum(sl, scratch) / (float)width + eps);
    const float rr = rsqrtf(block_sum(sr, scratch) / (float)width + eps);
    for (int c = threadIdx.x; c < width; c += blockDim.x)
        x[at + c] += half * (left[at + c] * rl * wl[c] + right[at + c] * rr * wr[c]);
}

// A block owns a token. Its cosines and sines are computed once (before the wait for the kernel before: they depend on the
// position only); the token's queries and keys are brought into shared memory as float32 in one pass of 16-byte loads that
// also sums their squares; pairs are rotated there, and one pass of 16-byte stores writes the row back. STAGED false: rows
// that do not fit shared memory, or are not 16-byte aligned, are normed and rotated in place from global memory.
template <typename T, bool STAGED>
__global__ void __launch_bounds__(256)
wide_norm_rotary_kernel(T* __restrict__ q, T* __restrict__ k, int stride, const int* __restrict__ positions,
                        const float* __restrict__ freqs, const float* __restrict__ qw, const float* __restrict__ kw, float eps,
                        int q_heads, int k_heads, int d, int n_pairs, int interleaved) {
    extern __shared__ __align__(16) float wn_shared[];
    __shared__ float sums[2][8];
    constexpr int PIECE = 16 / sizeof(T);
    dd_launch_dependents();
    const int t = blockIdx.x;
    const int nq = q_heads * d, nk = k ? k_heads * d : 0;
    float* cosines = wn_shared;
    float* sines = wn_shared + n_pairs;
    float* row = wn_shared + 2 * n_pairs + ((-2 * n_pairs) & 3);          // [nq + nk], 16-byte aligned
    {
        const float p = (float)positions[t];
        for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) sincosf(p * freqs[i], &sines[i], &cosines[i]);
    }
    dd_grid_wait();
    T* qr = q + (size_t)t * stride;
    T* kr = k ? k + (size_t)t * stride : nullptr;
    float sq = 0.f, sk = 0.f;
    if (STAGED) {
        for (int c = threadIdx.x * PIECE; c < nq + nk; c += blockDim.x * PIECE) {
            const bool is_k = c >= nq;
            const T* src = is_k ? kr + (c - nq) : qr + c;
            T piece[PIECE];
            *reinterpret_cast<uint4*>(piece) = *reinterpret_cast<const uint4*>(src);
            float s = 0.f;
#pragma unroll
            for (int j = 0; j < PIECE; ++j) { const float v = dd_to_f32(piece[j]); row[c + j] = v; s = fmaf(v, v, s); }
            if (is_k) sk += s; else sq += s;
        }
    } else {
        for (int c = threadIdx.x; c < nq; c += blockDim.x) { const float v = dd_to_f32(qr[c]); sq = fmaf(v, v, sq); }
        for (int c = threadIdx.x; c < nk; c += blockDim.x) { const float v = dd_to_f32(kr[c]); sk = fmaf(v, v, sk); }
    }
    sq = dd_warp_sum(sq);
    sk = dd_warp_sum(sk);
    if ((threadIdx.x & 31) == 0) { sums[0][threadIdx.x >> 5] = sq; sums[1][threadIdx.x >> 5] = sk; }
    __syncthreads();
    sq = sk = 0.f;
    for (int i = 0; i < (int)(blockDim.x >> 5); ++i) { sq += sums[0][i]; sk += sums[1][i]; }      // every thread adds in one order
    const float rq = qw ? rsqrtf(sq / (float)nq + eps) : 1.0f;
    const float rk = (kw && nk) ? rsqrtf(sk / (float)nk + eps) : 1.0f;
    // a thread owns whole pairs (and single elements of the unrotated rest), so nothing is read after it was written
    const int per_head = d - n_pairs;               // items of a head: n_pairs pairs, then d - 2 n_pairs single elements
    const int q_items = q_heads * per_head, items = q_items + (k ? k_heads * per_head : 0);
    for (int item = threadIdx.x; item < items; item += blockDim.x) {
        const bool is_k = item >= q_items;
        const int local = is_k ? item - q_items : item;
        const int h = local / per_head, i = local % per_head;
        const float* w = is_k ? kw : qw;
        const float r = is_k ? rk : rq;
        const int base = h * d;
        const int off = is_k ? nq : 0;
        T* dst = is_k ? kr : qr;
        if (i < n_pairs) {
            const int a = base + (interleaved ? 2 * i : i), b = base + (interleaved ? 2 * i + 1 : i + n_pairs);
            float u = (STAGED ? row[off + a] : dd_to_f32(dst[a])) * r, v = (STAGED ? row[off + b] : dd_to_f32(dst[b])) * r;
            if (w) { u *= w[a]; v *= w[b]; }
            const float c = cosines[i], sn = sines[i];
            const float ru = u * c - v * sn, rv = v * c + u * sn;
            if (STAGED) { row[off + a] = ru; row[off + b] = rv; } else { dst[a] = dd_from_f32<T>(ru); dst[b] = dd_from_f32<T>(rv); }
        } else {
            const int a = base + n_pairs + i;
            float u = (STAGED ? row[off + a] : dd_to_f32(dst[a])) * r;
            if (w) u *= w[a];
            if (STAGED) row[off + a] = u; else dst[a] = dd_from_f32<T>(u);
        }
    }
    if (!STAGED) return;
    __syncthreads();
    for (int c = threadIdx.x * PIECE; c < nq + nk; c += blockDim.x * PIECE) {
        T* dst = c >= nq ? kr + (c - nq) : qr + c;
        T piece[PIECE];
#pragma unroll
        for (int j = 0; j < PIECE; ++j) piece[j] = dd_from_f32<T>(row[c + j]);
        *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(piece);
    }
}

// An item is a 16-byte piece of a row (WIDE) or one element; the grid covers all items of all rows.
template <typename T, bool WIDE>
__global__ void __launch_bounds__(256)
sigmoid_gate_kernel(T* __restrict__ x, int x_stride, const T* __restrict__ gate, int gate_stride, int rows, int width) {
    constexpr int PIECE = WIDE ? 16 / sizeof(T) : 1;
    dd_launch_dependents();
    dd_grid_wait();
    const int per_row = width / PIECE;
    const long long item = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (item >= (long long)rows * per_row) return;
    const int r = (int)(item / per_row), c = (int)(item % per_row) * PIECE;
    T* xp = x + (size_t)r * x_stride + c;
    const T* gp = gate + (size_t)r * gate_stride + c;
    if (WIDE) {
        T xs[PIECE], gs[PIECE];
        *reinterpret_cast<uint4*>(xs) = *reinterpret_cast<const uint4*>(xp);
        *reinterpret_cast<uint4*>(gs) = *reinterpret_cast<const uint4*>(gp);
#pragma unroll
        for (int j = 0; j < PIECE; ++j) xs[j] = dd_from_f32<T>(dd_to_f32(xs[j]) / (1.0f + expf(-dd_to_f32(gs[j]))));
        *reinterpret_cast<uint4*>(xp) = *reinterpret_cast<const uint4*>(xs);
    } else {
        *xp = dd_from_f32<T>(dd_to_f32(*xp) / (1.0f + expf(-dd_to_f32(*gp))));
    }
}

__global__ void __launch_bounds__(256) tanh_cap_kernel(float* __restrict__ x, long long n, float cap) {
    dd_launch_dependents();
    dd_grid_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] = cap * tanhf(x[i] / cap);
}
}  // namespace

DD_API int dd_tanh_norm(const float* x, const int* row_index, const float* alpha, const float* w, const float* b, void* out,
                        int rows, int width, int out_dtype, void* stream) {
    if (rows <= 0) return 0;
    if (width <= 0) return dd_fail("dd_tanh_norm: bad width %d", width);
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = width >= 1024 ? 256 : 128;
    if (out_dtype == DD_F32)
        dd_launch(tanh_norm_kernel<float>, dim3(rows), dim3(threads), 0, s, x, row_index, alpha, w, b, (float*)out, width);
    else if (out_dtype == DD_BF16)
        dd_launch(tanh_norm_kernel<__nv_bfloat16>, dim3(rows), dim3(threads), 0, s, x, row_index, alpha, w, b, (__nv_bfloat16*)out, width);
    else
        return dd_fail("dd_tanh_norm: unknown dtype %d", out_dtype);
    return dd_check_launch("dd_tanh_norm");
}

DD_API int dd_add_rows(float* x, const float* other, const float* vec, int rows, int width, void* stream) {
    if (rows <= 0 || (other == nullptr && vec == nullptr)) return 0;
    dd_launch(add_rows_kernel, dim3(rows), dim3(width >= 1024 ? 256 : 128), 0, (cudaStream_t)stream, x, other, vec, width);
    return dd_check_launch("dd_add_rows");
}

DD_API int dd_norm_pair_add(float* x, const float* left, const float* right, const float* wl, const float* wr, float eps,
                            float half, int rows, int width, void* stream) {
    if (rows <= 0) return 0;
    dd_launch(norm_pair_add_kernel, dim3(rows), dim3(width >= 1024 ? 256 : 128), 0, (cudaStream_t)stream, x, left, right, wl, wr,
              eps, half, width);
    return dd_check_launch("dd_norm_pair_add");
}

// q: [N, q_heads * d], k: [N, k_heads * d] (or null), row views of one buffer with row stride `stride`; qw, kw: float32 weights
// over the whole projection (null: that kind is not normed); freqs: n_pairs frequencies (n_pairs may be 0).
DD_API int dd_wide_norm_rotary(void* q, void* k, int stride, const int* positions, const float* freqs, const float* qw,
                               const float* kw, float eps, int n_tokens, int q_heads, int k_heads, int d, int n_pairs,
                               int interleaved, int dtype, void* stream) {
    if (n_tokens <= 0) return 0;
    if (d <= 0 || n_pairs < 0 || 2 * n_pairs > d) return dd_fail("dd_wide_norm_rotary: %d pairs do not fit a head of %d", n_pairs, d);
    cudaStream_t s = (cudaStream_t)stream;
    const int nq = q_heads * d, nk = k ? k_heads * d : 0;
    const int elem = dtype == DD_F32 ? 4 : 2, piece = 16 / elem;
    const size_t table = (size_t)(2 * n_pairs + 3) * sizeof(float);
    // staged: every piece of 16 bytes lies inside q or inside k and is aligned, and the row fits shared memory
    const bool staged = nq % piece == 0 && nk % piece == 0 && stride % piece == 0 && (uintptr_t)q % 16 == 0 &&
                        (k == nullptr || (uintptr_t)k % 16 == 0) && table + (size_t)(nq + nk) * 4 <= 40 * 1024;
    const size_t smem = table + (staged ? (size_t)(nq + nk) * 4 : 0);
    const int threads = (nq + nk) >= 2048 ? 256 : 128;
#define WN_LAUNCH(T, STAGED) dd_launch(wide_norm_rotary_kernel<T, STAGED>, dim3(n_tokens), dim3(threads), smem, s, (T*)q, (T*)k, stride, \
                                       positions, freqs, qw, kw, eps, q_heads, k_heads, d, n_pairs, interleaved)
    if (dtype == DD_F32) { if (staged) WN_LAUNCH(float, true); else WN_LAUNCH(float, false); }
    else if (dtype == DD_BF16) { if (staged) WN_LAUNCH(__nv_bfloat16, true); else WN_LAUNCH(__nv_bfloat16, false); }
    else return dd_fail("dd_wide_norm_rotary: unknown dtype %d", dtype);
#undef WN_LAUNCH
    return dd_check_launch("dd_wide_norm_rotary");
}

DD_API int dd_sigmoid_gate(void* x, int x_stride, const void* gate, int gate_stride, int rows, int width, int dtype, void* stream) {
    if (rows <= 0 || width <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const int elem = dtype == DD_F32 ? 4 : 2, piece = 16 / elem;
    const bool wide = width % piece == 0 && x_stride % piece == 0 && gate_stride % piece == 0 && (uintptr_t)x % 16 == 0 &&
                      (uintptr_t)gate % 16 == 0;
    const long long items = (long long)rows * (wide ? width / piece : width);
    const dim3 grid(dd_ceil_div(items, 128));
#define SG_LAUNCH(T, WIDE) dd_launch(sigmoid_gate_kernel<T, WIDE>, grid, dim3(128), 0, s, (T*)x, x_stride, (const T*)gate, gate_stride, rows, width)
    if (dtype == DD_F32) { if (wide) SG_LAUNCH(float, true); else SG_LAUNCH(float, false); }
    else if (dtype == DD_BF16) { if (wide) SG_LAUNCH(__nv_bfloat16, true); else SG_LAUNCH(__nv_bfloat16, false); }
    else return dd_fail("dd_sigmoid_gate: unknown dtype %d", dtype);
#undef SG_LAUNCH
    return dd_check_launch("dd_sigmoid_gate");
}

DD_API int dd_tanh_cap(float* x, long long n, float cap, void* stream) {
    if (n <= 0) return 0;
    if (!(cap > 0.f)) return dd_fail("dd_tanh_cap: the cap must be positive");
    dd_launch(tanh_cap_kernel, dim3(dd_ceil_div(n, 256)), dim3(256), 0, (cudaStream_t)stream, x, n, cap);
    return dd_check_launch("dd_tanh_cap");
}
