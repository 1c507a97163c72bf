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

template <typename T>
__global__ void __launch_bounds__(256)
wide_norm_rotary_kernel(T* __restrict__ q, T* __restrict__ k, int stride, const int* __restrict__ positions,
                        const float* __restrict__ freqs, const float* __restrict__ qw, const float* __restrict__ kw, float eps,
                        int q_heads, int k_heads, int d, int n_pairs, int interleaved) {
    __shared__ float scratch[8];
    dd_launch_dependents();
    dd_grid_wait();
    const int t = blockIdx.x;
    const float p = (float)positions[t];
    for (int which = 0; which < 2; ++which) {
        T* row = (which ? k : q);
        const int heads = which ? k_heads : q_heads;
        const float* w = which ? kw : qw;
        if (row == nullptr || heads == 0) continue;
        row += (size_t)t * stride;
        const int total = heads * d;
        float r = 1.0f;
        if (w != nullptr) {
            float s = 0.f;
            for (int c = threadIdx.x; c < total; c += blockDim.x) { const float v = dd_to_f32(row[c]); s = fmaf(v, v, s); }
            r = rsqrtf(block_sum(s, scratch) / (float)total + eps);
        }
        // a thread owns whole pairs (and single elements of the unrotated rest), so nothing is read after it was written
        const int per_head = d - n_pairs;           // items of a head: n_pairs pairs, then d - 2 n_pairs single elements
        for (int item = threadIdx.x; item < heads * per_head; item += blockDim.x) {
            const int h = item / per_head, i = item % per_head;
            if (i < n_pairs) {
                const int a = h * d + (interleaved ? 2 * i : i), b = h * d + (interleaved ? 2 * i + 1 : i + n_pairs);
                float u = dd_to_f32(row[a]) * r, v = dd_to_f32(row[b]) * r;
                if (w) { u *= w[a]; v *= w[b]; }
                const float angle = p * freqs[i];
                const float c = cosf(angle), s = sinf(angle);
                row[a] = dd_from_f32<T>(u * c - v * s);
                row[b] = dd_from_f32<T>(v * c + u * s);
            } else {
                const int a = h * d + n_pairs + i;
                float u = dd_to_f32(row[a]) * r;
                if (w) u *= w[a];
                row[a] = dd_from_f32<T>(u);
            }
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(256)
sigmoid_gate_kernel(T* __restrict__ x, int x_stride, const T* __restrict__ gate, int gate_stride, int width) {
    dd_launch_dependents();
    dd_grid_wait();
    T* xr = x + (size_t)blockIdx.x * x_stride;
    const T* gr = gate + (size_t)blockIdx.x * gate_stride;
    for (int c = threadIdx.x; c < width; c += blockDim.x)
        xr[c] = dd_from_f32<T>(dd_to_f32(xr[c]) / (1.0f + expf(-dd_to_f32(gr[c]))));
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
    if (dtype == DD_F32)
        dd_launch(wide_norm_rotary_kernel<float>, dim3(n_tokens), dim3(256), 0, s, (float*)q, (float*)k, stride, positions, freqs,
                  qw, kw, eps, q_heads, k_heads, d, n_pairs, interleaved);
    else if (dtype == DD_BF16)
        dd_launch(wide_norm_rotary_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(256), 0, s, (__nv_bfloat16*)q, (__nv_bfloat16*)k,
                  stride, positions, freqs, qw, kw, eps, q_heads, k_heads, d, n_pairs, interleaved);
    else
        return dd_fail("dd_wide_norm_rotary: unknown dtype %d", dtype);
    return dd_check_launch("dd_wide_norm_rotary");
}

DD_API int dd_sigmoid_gate(void* x, int x_stride, const void* gate, int gate_stride, int rows, int width, int dtype, void* stream) {
    if (rows <= 0 || width <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = width >= 1024 ? 256 : 128;
    if (dtype == DD_F32)
        dd_launch(sigmoid_gate_kernel<float>, dim3(rows), dim3(threads), 0, s, (float*)x, x_stride, (const float*)gate, gate_stride, width);
    else if (dtype == DD_BF16)
        dd_launch(sigmoid_gate_kernel<__nv_bfloat16>, dim3(rows), dim3(threads), 0, s, (__nv_bfloat16*)x, x_stride,
                  (const __nv_bfloat16*)gate, gate_stride, width);
    else
        return dd_fail("dd_sigmoid_gate: unknown dtype %d", dtype);
    return dd_check_launch("dd_sigmoid_gate");
}

DD_API int dd_tanh_cap(float* x, long long n, float cap, void* stream) {
    if (n <= 0) return 0;
    if (!(cap > 0.f)) return dd_fail("dd_tanh_cap: the cap must be positive");
    dd_launch(tanh_cap_kernel, dim3(dd_ceil_div(n, 256)), dim3(256), 0, (cudaStream_t)stream, x, n, cap);
    return dd_check_launch("dd_tanh_cap");
}
