// RMS norm over the float32 residual stream: y = x / sqrt(mean(x^2) + eps) * (offset + w), eps inside the root,
// the sum of squares and the scaling in float32. `offset` is 0 for a weight stored as the factor itself and 1 for a
// weight stored as its distance from one. Output in the engine dtype. An optional row index gathers rows first (the
// final norm runs only where logits are wanted).
//
// In groups: the row is cut into `groups` equal consecutive stretches and each is divided by its own root mean square;
// the weight multiplies the whole row. With a shift (dd_rmsnorm_shift) the normed row n[t] is blended, in float32 and
// per channel, with the normed row of the token before it in its sequence: out[t] = n[t] + (n[t-1] - n[t]) * mu.
// n[t-1] of a step's first token is the float32 row the request's state slot holds (zeros for a new request); the
// block of that first token also leaves the normed row of the entry's last token there, after it has read the old one,
// so one block alone touches a slot's row. A block norms its own row and the row before it with the same function, so
// n[t-1] has the same bits whether it comes from the state or is computed again.
#include "common.cuh"

namespace {
template <int THREADS>
__device__ __forceinline__ float rms_block_sum(float v, float* scratch) {
    v = dd_warp_sum(v);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float total = 0.f;
#pragma unroll
    for (int w = 0; w < THREADS / 32; ++w) total += scratch[w];
    return total;
}

template <typename TO> struct RmsPack4;
template <> struct RmsPack4<float> {
    __device__ static void store(float* dst, float a, float b, float c, float d) { *reinterpret_cast<float4*>(dst) = make_float4(a, b, c, d); }
};
template <> struct RmsPack4<__nv_bfloat16> {
    __device__ static void store(__nv_bfloat16* dst, float a, float b, float c, float d) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
        uint2 v;
        v.x = *reinterpret_cast<uint32_t*>(&lo);
        v.y = *reinterpret_cast<uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(dst) = v;
    }
};

// Rows whose width is a multiple of 4 and at most 128 * 4 * VPT: the row in registers as float4.
template <typename TO, int VPT>
__global__ void __launch_bounds__(128)
rmsnorm_vec_kernel(const float* __restrict__ x, const int* __restrict__ row_index, const float* __restrict__ weight,
                   TO* __restrict__ out, int width, float eps, float offset) {
    __shared__ float scratch[4];
    dd_launch_dependents();
    const int row = blockIdx.x;
    const int n4 = width >> 2;
    // the weight does not depend on the kernel before: it is in registers before that kernel has finished
    float4 g[VPT];
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int c = threadIdx.x + i * 128;
        g[i] = c < n4 ? __ldg(reinterpret_cast<const float4*>(weight) + c) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    dd_grid_wait();
    const float4* in = reinterpret_cast<const float4*>(x + (size_t)(row_index ? row_index[row] : row) * width);
    float4 v[VPT];
    float sq = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int c = threadIdx.x + i * 128;
        v[i] = c < n4 ? in[c] : make_float4(0.f, 0.f, 0.f, 0.f);
        sq += (v[i].x * v[i].x + v[i].y * v[i].y) + (v[i].z * v[i].z + v[i].w * v[i].w);
    }
    const float r = 1.0f / sqrtf(rms_block_sum<128>(sq, scratch) / (float)width + eps);
    TO* o = out + (size_t)row * width;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int c = threadIdx.x + i * 128;
        if (c < n4)
            RmsPack4<TO>::store(o + 4 * c, v[i].x * r * (offset + g[i].x), v[i].y * r * (offset + g[i].y),
                                v[i].z * r * (offset + g[i].z), v[i].w * r * (offset + g[i].w));
    }
}

template <typename TO, int THREADS>
__global__ void __launch_bounds__(THREADS)
rmsnorm_kernel(const float* __restrict__ x, const int* __restrict__ row_index, const float* __restrict__ weight,
               TO* __restrict__ out, int width, float eps, float offset) {
    __shared__ float scratch[THREADS / 32];
    dd_launch_dependents();
    dd_grid_wait();
    const int row = blockIdx.x;
    const float* in = x + (size_t)(row_index ? row_index[row] : row) * width;
    TO* o = out + (size_t)row * width;
    float sq = 0.f;
    for (int c = threadIdx.x; c < width; c += THREADS) sq += in[c] * in[c];
    const float r = 1.0f / sqrtf(rms_block_sum<THREADS>(sq, scratch) / (float)width + eps);
    for (int c = threadIdx.x; c < width; c += THREADS) o[c] = dd_from_f32<TO>(in[c] * r * (offset + weight[c]));
}
constexpr int MAX_GROUPS = 64;

// The inverse root mean squares of the stretches of row a into ra[0 .. groups), and of row b (if any) into rb (shared
// memory); every thread sees them after. A stretch is cut into 8 / groups pieces (at least one), a warp sums a piece, lane
// by lane in a fixed order, and one thread adds a stretch's pieces: the sum of a row does not depend on which of the two
// rows it is, nor on what the other one is.
template <int THREADS>
__device__ __forceinline__ void group_scales(const float* __restrict__ a, float* ra, const float* __restrict__ b, float* rb,
                                             int width, int groups, float eps, float* partial) {
    const int gw = width / groups, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int pieces = groups >= 8 ? 1 : 8 / groups, piece = (gw + pieces - 1) / pieces;
    const int per_row = groups * pieces;
    // a warp sums the same piece of both rows at once, so that the loads of both are in flight together
    for (int it = warp; it < per_row; it += THREADS / 32) {
        const int g = it / pieces, lo = (it % pieces) * piece, hi = min(gw, lo + piece);
        const float* pa = a + (size_t)g * gw;
        const float* pb = b ? b + (size_t)g * gw : pa;
        float sa = 0.f, sb = 0.f;
        for (int c0 = lo + lane; c0 < hi; c0 += 256) {      // eight loads a row in flight; a zero past the end adds nothing
            float va[8], vb[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) va[k] = c0 + 32 * k < hi ? pa[c0 + 32 * k] : 0.f;
#pragma unroll
            for (int k = 0; k < 8; ++k) vb[k] = b && c0 + 32 * k < hi ? pb[c0 + 32 * k] : 0.f;
#pragma unroll
            for (int k = 0; k < 8; ++k) sa = fmaf(va[k], va[k], sa);
#pragma unroll
            for (int k = 0; k < 8; ++k) sb = fmaf(vb[k], vb[k], sb);
        }
        sa = dd_warp_sum(sa);
        sb = dd_warp_sum(sb);
        if (lane == 0) {
            partial[it] = sa;
            partial[per_row + it] = sb;
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < (b ? 2 : 1) * groups; i += THREADS) {
        const int g = i % groups;
        const float* mine = partial + (i >= groups ? per_row : 0) + g * pieces;
        float total = 0.f;
        for (int j = 0; j < pieces; ++j) total += mine[j];
        (i >= groups ? rb : ra)[g] = 1.0f / sqrtf(total / (float)gw + eps);
    }
    __syncthreads();
}

template <typename TO, int THREADS>
__global__ void __launch_bounds__(THREADS)
rmsnorm_groups_kernel(const float* __restrict__ x, const int* __restrict__ row_index, const float* __restrict__ weight,
                      TO* __restrict__ out, int width, int groups, float eps, float offset) {
    __shared__ float partial[2 * MAX_GROUPS];
    __shared__ float r[MAX_GROUPS];
    dd_launch_dependents();
    dd_grid_wait();
    const int row = blockIdx.x;
    const float* in = x + (size_t)(row_index ? row_index[row] : row) * width;
    TO* o = out + (size_t)row * width;
    group_scales<THREADS>(in, r, nullptr, nullptr, width, groups, eps, partial);
    const int gw = width / groups;
#pragma unroll 4
    for (int c = threadIdx.x; c < width; c += THREADS) o[c] = dd_from_f32<TO>(in[c] * r[c / gw] * (offset + weight[c]));
}

// Explicit roundings, so that a normed value has the same bits whether it is blended at once or kept in the state first
// (the compiler would otherwise contract the products into the subtraction in one place and not in the other).
__device__ __forceinline__ float normed_value(float x, float r, float w) { return __fmul_rn(__fmul_rn(x, r), w); }
__device__ __forceinline__ float blended_value(float n, float p, float mu) { return __fmaf_rn(__fsub_rn(p, n), mu, n); }

template <typename TO, int THREADS>
__global__ void __launch_bounds__(THREADS)
rmsnorm_shift_kernel(const float* __restrict__ x, const float* __restrict__ weight, const float* __restrict__ mu,
                     float* __restrict__ state, const int* __restrict__ tok_entry, const int* __restrict__ entry_start,
                     const int* __restrict__ entry_slot, TO* __restrict__ out, int width, int groups, float eps, float offset) {
    __shared__ float partial[2 * MAX_GROUPS];
    __shared__ float r_own[MAX_GROUPS], r_other[MAX_GROUPS];
    dd_launch_dependents();
    const int t = blockIdx.x;
    const int e = tok_entry[t];
    const int first = entry_start[e], last = entry_start[e + 1] - 1;
    float* kept = state + (size_t)entry_slot[e] * width;
    dd_grid_wait();
    const float* in = x + (size_t)t * width;
    const int gw = width / groups;
    TO* o = out + (size_t)t * width;
    if (t != first) {
        // the token before lies in this step: its normed row again, by the same arithmetic
        const float* before = in - width;
        group_scales<THREADS>(in, r_own, before, r_other, width, groups, eps, partial);
#pragma unroll 4
        for (int c = threadIdx.x; c < width; c += THREADS) {
            const float w = offset + weight[c];
            const float n = normed_value(in[c], r_own[c / gw], w), p = normed_value(before[c], r_other[c / gw], w);
            o[c] = dd_from_f32<TO>(blended_value(n, p, mu[c]));
        }
        return;
    }
    // the first token of its entry in this step: the row before it is the state's; then the state becomes the entry's
    // last normed row (a thread writes only the channels it has read)
    const float* tail = x + (size_t)last * width;
    group_scales<THREADS>(in, r_own, last != t ? tail : nullptr, r_other, width, groups, eps, partial);
    for (int c = threadIdx.x; c < width; c += THREADS) {
        const float w = offset + weight[c];
        const float n = normed_value(in[c], r_own[c / gw], w), p = kept[c];
        o[c] = dd_from_f32<TO>(blended_value(n, p, mu[c]));
        kept[c] = last != t ? normed_value(tail[c], r_other[c / gw], w) : n;
    }
}
}  // namespace

// The norm in groups and the blend with the token before (see the head of this file). state: float32 [slots, width].
DD_API int dd_rmsnorm_shift(const float* x, const float* weight, const float* mu, float* state, const int* tok_entry,
                            const int* entry_start, const int* entry_slot, void* out, int rows, int width, int groups,
                            float eps, float offset, int out_dtype, void* stream) {
    if (rows <= 0) return 0;
    if (width <= 0 || groups <= 0 || groups > MAX_GROUPS || width % groups)
        return dd_fail("dd_rmsnorm_shift: a row of %d does not fall into %d equal stretches (at most %d)", width, groups, MAX_GROUPS);
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == DD_F32)
        dd_launch(rmsnorm_shift_kernel<float, 256>, dim3(rows), dim3(256), 0, s, x, weight, mu, state, tok_entry, entry_start,
                  entry_slot, (float*)out, width, groups, eps, offset);
    else if (out_dtype == DD_BF16)
        dd_launch(rmsnorm_shift_kernel<__nv_bfloat16, 256>, dim3(rows), dim3(256), 0, s, x, weight, mu, state, tok_entry,
                  entry_start, entry_slot, (__nv_bfloat16*)out, width, groups, eps, offset);
    else
        return dd_fail("dd_rmsnorm_shift: unknown output dtype %d", out_dtype);
    return dd_check_launch("dd_rmsnorm_shift");
}

DD_API int dd_rmsnorm_groups(const float* x, const int* row_index, const float* weight, void* out, int rows, int width,
                             int groups, float eps, float offset, int out_dtype, void* stream) {
    if (rows <= 0) return 0;
    if (width <= 0 || groups <= 0 || groups > MAX_GROUPS || width % groups)
        return dd_fail("dd_rmsnorm_groups: a row of %d does not fall into %d equal stretches (at most %d)", width, groups, MAX_GROUPS);
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == DD_F32)
        dd_launch(rmsnorm_groups_kernel<float, 256>, dim3(rows), dim3(256), 0, s, x, row_index, weight, (float*)out, width, groups, eps, offset);
    else if (out_dtype == DD_BF16)
        dd_launch(rmsnorm_groups_kernel<__nv_bfloat16, 256>, dim3(rows), dim3(256), 0, s, x, row_index, weight,
                  (__nv_bfloat16*)out, width, groups, eps, offset);
    else
        return dd_fail("dd_rmsnorm_groups: unknown output dtype %d", out_dtype);
    return dd_check_launch("dd_rmsnorm_groups");
}

DD_API int dd_rmsnorm(const float* x, const int* row_index, const float* weight, void* out, int rows, int width,
                      float eps, float offset, int out_dtype, void* stream) {
    if (rows <= 0) return 0;
    if (width <= 0) return dd_fail("dd_rmsnorm: bad width %d", width);
    if (out_dtype != DD_F32 && out_dtype != DD_BF16) return dd_fail("dd_rmsnorm: unknown output dtype %d", out_dtype);
    cudaStream_t s = (cudaStream_t)stream;
    if (width % 4 == 0 && width <= 128 * 4 * 4 && !(((uintptr_t)x | (uintptr_t)out | (uintptr_t)weight) & 15)) {
        if (out_dtype == DD_F32)
            dd_launch(rmsnorm_vec_kernel<float, 4>, dim3(rows), dim3(128), 0, s, x, row_index, weight, (float*)out, width, eps, offset);
        else
            dd_launch(rmsnorm_vec_kernel<__nv_bfloat16, 4>, dim3(rows), dim3(128), 0, s, x, row_index, weight,
                      (__nv_bfloat16*)out, width, eps, offset);
        return dd_check_launch("dd_rmsnorm");
    }
    if (out_dtype == DD_F32)
        dd_launch(rmsnorm_kernel<float, 256>, dim3(rows), dim3(256), 0, s, x, row_index, weight, (float*)out, width, eps, offset);
    else
        dd_launch(rmsnorm_kernel<__nv_bfloat16, 256>, dim3(rows), dim3(256), 0, s, x, row_index, weight,
                  (__nv_bfloat16*)out, width, eps, offset);
    return dd_check_launch("dd_rmsnorm");
}
