// Streams of earlier layers mixed by learned weights: out = sum over j < n of w[j] * X_j, in float32 and in the order
// of j. The X_j are the planes of one stack [planes, count] (what the embedding and every layer so far has left);
// out may be the stack's next plane. Another kernel of this file blends a row view with another by one learned number:
// v <- (1 - lambda) v + lambda * other, in float32, rounded once (values mixed with those an earlier layer computed
// for the same tokens).
#include "common.cuh"

namespace {
__global__ void __launch_bounds__(256)
weighted_sum4_kernel(const float4* __restrict__ stack, size_t plane4, const float* __restrict__ w, int n,
                     float4* __restrict__ out, size_t count4) {
    dd_launch_dependents();
    dd_grid_wait();
    const size_t i = (size_t)blockIdx.x * 256 + threadIdx.x;
    if (i >= count4) return;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int j = 0; j < n; ++j) {
        const float4 v = stack[(size_t)j * plane4 + i];
        const float f = w[j];
        acc.x = fmaf(f, v.x, acc.x); acc.y = fmaf(f, v.y, acc.y); acc.z = fmaf(f, v.z, acc.z); acc.w = fmaf(f, v.w, acc.w);
    }
    out[i] = acc;
}

__global__ void __launch_bounds__(256)
weighted_sum_kernel(const float* __restrict__ stack, size_t plane, const float* __restrict__ w, int n,
                    float* __restrict__ out, size_t count) {
    dd_launch_dependents();
    dd_grid_wait();
    const size_t i = (size_t)blockIdx.x * 256 + threadIdx.x;
    if (i >= count) return;
    float acc = 0.f;
    for (int j = 0; j < n; ++j) acc = fmaf(w[j], stack[(size_t)j * plane + i], acc);
    out[i] = acc;
}

template <typename T>
__global__ void __launch_bounds__(256)
blend_rows_kernel(T* __restrict__ v, int v_stride, const T* __restrict__ other, int other_stride,
                  const float* __restrict__ lambda, int rows, int width) {
    dd_launch_dependents();
    const float lam = lambda[0];
    dd_grid_wait();
    const size_t i = (size_t)blockIdx.x * 256 + threadIdx.x;
    if (i >= (size_t)rows * width) return;
    const int r = (int)(i / width), c = (int)(i % width);
    T* p = v + (size_t)r * v_stride + c;
    const float a = dd_to_f32(*p), b = dd_to_f32(other[(size_t)r * other_stride + c]);
    *p = dd_from_f32<T>((1.0f - lam) * a + lam * b);
}
}  // namespace

// stack: float32 [planes >= n, count]; w: float32 [n] on the device; out: float32 [count].
DD_API int dd_weighted_sum(const float* stack, long long count, const float* w, int n, float* out, void* stream) {
    if (count <= 0) return 0;
    if (n <= 0) return dd_fail("dd_weighted_sum: nothing to add up (n = %d)", n);
    cudaStream_t s = (cudaStream_t)stream;
    if (count % 4 == 0 && !(((uintptr_t)stack | (uintptr_t)out) & 15)) {
        const long long c4 = count / 4;
        if ((c4 + 255) / 256 > 0x7fffffffLL) return dd_fail("dd_weighted_sum: %lld elements are more than one launch takes", count);
        dd_launch(weighted_sum4_kernel, dim3(dd_ceil_div(c4, 256)), dim3(256), 0, s, (const float4*)stack, (size_t)c4, w, n,
                  (float4*)out, (size_t)c4);
    } else {
        if ((count + 255) / 256 > 0x7fffffffLL) return dd_fail("dd_weighted_sum: %lld elements are more than one launch takes", count);
        dd_launch(weighted_sum_kernel, dim3(dd_ceil_div(count, 256)), dim3(256), 0, s, stack, (size_t)count, w, n, out, (size_t)count);
    }
    return dd_check_launch("dd_weighted_sum");
}

// v, other: row views [rows, width] (strides in elements); lambda: one float32 on the device.
DD_API int dd_blend_rows(void* v, int v_stride, const void* other, int other_stride, const float* lambda, int rows, int width,
                         int dtype, void* stream) {
    if (rows <= 0 || width <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const int grid = dd_ceil_div((long long)rows * width, 256);
    if (dtype == DD_F32)
        dd_launch(blend_rows_kernel<float>, dim3(grid), dim3(256), 0, s, (float*)v, v_stride, (const float*)other, other_stride, lambda, rows, width);
    else if (dtype == DD_BF16)
        dd_launch(blend_rows_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, s, (__nv_bfloat16*)v, v_stride,
                  (const __nv_bfloat16*)other, other_stride, lambda, rows, width);
    else
        return dd_fail("dd_blend_rows: unknown dtype %d", dtype);
    return dd_check_launch("dd_blend_rows");
}
