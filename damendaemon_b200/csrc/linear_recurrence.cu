// A gated linear recurrence per channel (a real-gated linear recurrent unit), float32 throughout.
//
//   dd_recurrence_gates   the channels come in `blocks` equal parts; in part b, with u_b the part's inputs of one token,
//                         r = sigmoid(Ra[b] u_b + ba[b]), i = sigmoid(Ri[b] u_b + bi[b]) (Ra[b], Ri[b] square, [out, in]);
//                         a = exp(-gain * r * softplus(lam)), drive = sqrt(1 - a^2) * i * u. Writes 1 - a and drive.
//   dd_linear_scan        S <- S - (1 - a_t) S + drive_t per channel from the request's state, out_t = S * act(y_t) rounded once
//                         (act: 0 none, 1 tanh-gelu)
//
// The gates are sums of float32 products in ascending order of the input channel, whatever else is in the step. The scan
// walks an entry's tokens in order, a thread a channel: a portion and a single token run the same instructions.
#include "common.cuh"

namespace {
constexpr int RG_TOKENS = 16;     // tokens a block of the gate kernel works on
constexpr int RG_OUTS = 128;      // output channels of a block = its threads
constexpr int RG_K = 32;          // input channels staged at a time

__device__ __forceinline__ float rg_softplus(float x) { return x > 20.f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float rg_sigmoid(float x) { return 1.0f / (1.0f + expf(-x)); }

__global__ void __launch_bounds__(RG_OUTS)
recurrence_gates_kernel(const float* __restrict__ u, const float* __restrict__ wa, const float* __restrict__ ba,
                        const float* __restrict__ wi, const float* __restrict__ bi, const float* __restrict__ lam, float gain,
                        float* __restrict__ a_out, float* __restrict__ drive_out, int n_tokens, int width, int bw) {
    __shared__ float us[RG_TOKENS][RG_K];
    __shared__ float was[RG_OUTS][RG_K + 1];
    __shared__ float wis[RG_OUTS][RG_K + 1];
    dd_launch_dependents();
    const int b = blockIdx.y, t0 = blockIdx.x * RG_TOKENS, o0 = blockIdx.z * RG_OUTS;
    const int o = o0 + threadIdx.x;                 // output channel within the part
    const bool live = o < bw;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const float* wa_b = wa + (size_t)b * bw * bw;
    const float* wi_b = wi + (size_t)b * bw * bw;
    float ra[RG_TOKENS], ri[RG_TOKENS];
#pragma unroll
    for (int j = 0; j < RG_TOKENS; ++j) ra[j] = ri[j] = 0.f;
    const float bias_a = live ? ba[b * bw + o] : 0.f, bias_i = live ? bi[b * bw + o] : 0.f;
    const float sp = live ? rg_softplus(lam[b * bw + o]) : 0.f;
    dd_grid_wait();
    for (int k0 = 0; k0 < bw; k0 += RG_K) {
        __syncthreads();
        // weights: a warp reads a stretch of one row at a time (coalesced), rows dealt out over the warps
        for (int r = warp; r < RG_OUTS; r += RG_OUTS / 32) {
            const bool in = o0 + r < bw && k0 + lane < bw;
            was[r][lane] = in ? wa_b[(size_t)(o0 + r) * bw + k0 + lane] : 0.f;
            wis[r][lane] = in ? wi_b[(size_t)(o0 + r) * bw + k0 + lane] : 0.f;
        }
        for (int j = warp; j < RG_TOKENS; j += RG_OUTS / 32)
            us[j][lane] = (t0 + j < n_tokens && k0 + lane < bw) ? u[(size_t)(t0 + j) * width + b * bw + k0 + lane] : 0.f;
        __syncthreads();
#pragma unroll 4
        for (int kk = 0; kk < RG_K; ++kk) {
            const float a = was[threadIdx.x][kk], i = wis[threadIdx.x][kk];
#pragma unroll
            for (int j = 0; j < RG_TOKENS; ++j) {
                ra[j] = fmaf(a, us[j][kk], ra[j]);
                ri[j] = fmaf(i, us[j][kk], ri[j]);
            }
        }
    }
    if (!live) return;
#pragma unroll
    for (int j = 0; j < RG_TOKENS; ++j) {
        if (t0 + j >= n_tokens) break;
        const size_t at = (size_t)(t0 + j) * width + b * bw + o;
        const float r = rg_sigmoid(ra[j] + bias_a), i = rg_sigmoid(ri[j] + bias_i);
        // what is handed on is 1 - a, not a: a decay near one, rounded to float32, would be off by up to 6e-8 of ONE, which
        // over the 1 / (1 - a) tokens a slow channel remembers adds up; 1 - a and 1 - a^2 come from expm1 without cancellation
        const float log_a = -gain * r * sp;
        a_out[at] = -expm1f(log_a);
        drive_out[at] = sqrtf(-expm1f(2.0f * log_a)) * i * u[at];
    }
}

template <typename T>
__global__ void __launch_bounds__(128)
linear_scan_kernel(const float* __restrict__ a, const float* __restrict__ drive, const T* __restrict__ y, int y_stride,
                   const int* __restrict__ entry_start, const int* __restrict__ entry_slot, float* __restrict__ state,
                   T* __restrict__ out, int out_stride, int width, int act) {
    dd_launch_dependents();
    const int e = blockIdx.y, c = blockIdx.x * 128 + threadIdx.x;
    if (c >= width) return;
    const int start = entry_start[e], end = entry_start[e + 1];
    float* sp = state + (size_t)entry_slot[e] * width + c;
    dd_grid_wait();
    float s = *sp;
#pragma unroll 4
    for (int t = start; t < end; ++t) {
        const size_t at = (size_t)t * width + c;
        s = fmaf(-a[at], s, s) + drive[at];              // a holds 1 - decay
        float g = dd_to_f32(y[(size_t)t * y_stride + c]);
        if (act == 1) g = dd_activation(g, DD_ACT_GELU_NEW);
        out[(size_t)t * out_stride + c] = dd_from_f32<T>(s * g);
    }
    *sp = s;
}
}  // namespace

// u: float32 [N, width] contiguous; wa, wi: float32 [blocks, bw, bw]; ba, bi, lam: float32 [width]; a_out (1 - a), drive_out:
// float32 [N, width].
DD_API int dd_recurrence_gates(const float* u, const float* wa, const float* ba, const float* wi, const float* bi, const float* lam,
                               float gain, float* a_out, float* drive_out, int n_tokens, int width, int blocks, void* stream) {
    if (n_tokens <= 0) return 0;
    if (width <= 0 || blocks <= 0 || width % blocks) return dd_fail("dd_recurrence_gates: %d channels do not fall into %d equal parts", width, blocks);
    const int bw = width / blocks;
    const dim3 grid(dd_ceil_div(n_tokens, RG_TOKENS), blocks, dd_ceil_div(bw, RG_OUTS));
    dd_launch(recurrence_gates_kernel, grid, dim3(RG_OUTS), 0, (cudaStream_t)stream, u, wa, ba, wi, bi, lam, gain, a_out, drive_out,
              n_tokens, width, bw);
    return dd_check_launch("dd_recurrence_gates");
}

// a (holding 1 - decay), drive: float32 [N, width]; y: [N, width] row view in `dtype`; state: float32 [slots, width], read and written; out: rows
// of stride out_stride in `dtype`.
DD_API int dd_linear_scan(const float* a, const float* drive, const void* y, int y_stride, const int* entry_start,
                          const int* entry_slot, int n_entries, float* state, void* out, int out_stride, int width, int act,
                          int dtype, void* stream) {
    if (n_entries <= 0 || width <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid(dd_ceil_div(width, 128), n_entries);
    if (dtype == DD_F32)
        dd_launch(linear_scan_kernel<float>, grid, dim3(128), 0, s, a, drive, (const float*)y, y_stride, entry_start, entry_slot, state,
                  (float*)out, out_stride, width, act);
    else if (dtype == DD_BF16)
        dd_launch(linear_scan_kernel<__nv_bfloat16>, grid, dim3(128), 0, s, a, drive, (const __nv_bfloat16*)y, y_stride, entry_start,
                  entry_slot, state, (__nv_bfloat16*)out, out_stride, width, act);
    else
        return dd_fail("dd_linear_scan: unknown dtype %d", dtype);
    return dd_check_launch("dd_linear_scan");
}
