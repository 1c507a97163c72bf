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

constexpr int LS_TOKENS = 16;     // tokens whose operands a thread of the scan requests together

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
    // the operands of the next LS_TOKENS tokens are requested before this chunk's chain of multiply-adds runs: the walk
    // is bound by the loads' latency, not by arithmetic
    float fa[LS_TOKENS], fd[LS_TOKENS], fy[LS_TOKENS];
    auto fetch = [&](int t0) {
#pragma unroll
        for (int k = 0; k < LS_TOKENS; ++k) {
            const int t = min(t0 + k, end - 1);
            fa[k] = a[(size_t)t * width + c];
            fd[k] = drive[(size_t)t * width + c];
            fy[k] = dd_to_f32(y[(size_t)t * y_stride + c]);
        }
    };
    if (start < end) fetch(start);
    for (int t0 = start; t0 < end; t0 += LS_TOKENS) {
        float ca[LS_TOKENS], cd[LS_TOKENS], cy[LS_TOKENS];
#pragma unroll
        for (int k = 0; k < LS_TOKENS; ++k) { ca[k] = fa[k]; cd[k] = fd[k]; cy[k] = fy[k]; }
        if (t0 + LS_TOKENS < end) fetch(t0 + LS_TOKENS);
#pragma unroll
        for (int k = 0; k < LS_TOKENS; ++k) {
            if (t0 + k < end) {
                s = fmaf(-ca[k], s, s) + cd[k];              // a holds 1 - decay
                const float g = act == 1 ? dd_activation(cy[k], DD_ACT_GELU_NEW) : cy[k];
                out[(size_t)(t0 + k) * out_stride + c] = dd_from_f32<T>(s * g);
            }
        }
    }
    *sp = s;
}

// A step of few tokens: a block owns 32 output channels of one part and all the step's tokens, a warp one token, a lane one
// channel. The part's inputs of all tokens lie in shared memory; the two weight matrices' rows of the block's channels pass
// through shared memory 32 input channels at a time, each row's stretch read by one warp in one piece (a lane that streamed
// its own row from global memory would touch 32 lines an instruction). The sums run over the input channels in ascending
// order, the same multiply-adds in the same order as in the tiled kernel, so a token's gates do not depend on which kernel
// computed them.
constexpr int RG_FEW = 16, RG_FEW_OUTS = 32;

__global__ void __launch_bounds__(RG_FEW * RG_FEW_OUTS)
recurrence_gates_few_kernel(const float* __restrict__ u, const float* __restrict__ wa, const float* __restrict__ ba,
                            const float* __restrict__ wi, const float* __restrict__ bi, const float* __restrict__ lam, float gain,
                            float* __restrict__ a_out, float* __restrict__ drive_out, int n_tokens, int width, int bw) {
    extern __shared__ float us[];                   // [n_tokens][bw]
    __shared__ float was[2][RG_FEW_OUTS][RG_K + 1];
    __shared__ float wis[2][RG_FEW_OUTS][RG_K + 1];
    dd_launch_dependents();
    const int b = blockIdx.y, j = threadIdx.x >> 5, lane = threadIdx.x & 31, o0 = blockIdx.x * RG_FEW_OUTS, o = o0 + lane;
    const int warps = blockDim.x >> 5;
    const bool live = o < bw;
    const float* wa_b = wa + (size_t)b * bw * bw;
    const float* wi_b = wi + (size_t)b * bw * bw;
    const float bias_a = live ? ba[b * bw + o] : 0.f, bias_i = live ? bi[b * bw + o] : 0.f;
    const float sp = live ? rg_softplus(lam[b * bw + o]) : 0.f;
    auto stage = [&](int buf, int k0) {             // the weights do not depend on the kernel before
        for (int r = j; r < RG_FEW_OUTS; r += warps) {
            const bool in = o0 + r < bw && k0 + lane < bw;
            was[buf][r][lane] = in ? wa_b[(size_t)(o0 + r) * bw + k0 + lane] : 0.f;
            wis[buf][r][lane] = in ? wi_b[(size_t)(o0 + r) * bw + k0 + lane] : 0.f;
        }
    };
    stage(0, 0);
    dd_grid_wait();
    for (int i = threadIdx.x; i < n_tokens * bw; i += blockDim.x) us[i] = u[(size_t)(i / bw) * width + b * bw + i % bw];
    const float* mine = us + j * bw;
    float ra = 0.f, ri = 0.f;
    int buf = 0;
    for (int k0 = 0; k0 < bw; k0 += RG_K, buf ^= 1) {
        __syncthreads();                            // this stretch is staged; the other buffer has been read
        if (k0 + RG_K < bw) stage(buf ^ 1, k0 + RG_K);
        const int n = min(RG_K, bw - k0);
        for (int kk = 0; kk < n; ++kk) {
            ra = fmaf(was[buf][lane][kk], mine[k0 + kk], ra);
            ri = fmaf(wis[buf][lane][kk], mine[k0 + kk], ri);
        }
    }
    if (!live) return;
    const size_t at = (size_t)j * width + b * bw + o;
    const float r = rg_sigmoid(ra + bias_a), i = rg_sigmoid(ri + bias_i);
    const float log_a = -gain * r * sp;
    a_out[at] = -expm1f(log_a);
    drive_out[at] = sqrtf(-expm1f(2.0f * log_a)) * i * mine[o];
}
}  // namespace

// u: float32 [N, width] contiguous; wa, wi: float32 [blocks, bw, bw]; ba, bi, lam: float32 [width]; a_out (1 - a), drive_out:
// float32 [N, width].
DD_API int dd_recurrence_gates(const float* u, const float* wa, const float* ba, const float* wi, const float* bi, const float* lam,
                               float gain, float* a_out, float* drive_out, int n_tokens, int width, int blocks, void* stream) {
    if (n_tokens <= 0) return 0;
    if (width <= 0 || blocks <= 0 || width % blocks) return dd_fail("dd_recurrence_gates: %d channels do not fall into %d equal parts", width, blocks);
    const int bw = width / blocks;
    if (n_tokens <= RG_FEW && (size_t)n_tokens * bw * sizeof(float) <= 48 * 1024) {
        dd_launch(recurrence_gates_few_kernel, dim3(dd_ceil_div(bw, RG_FEW_OUTS), blocks), dim3(32 * n_tokens), (size_t)n_tokens * bw * sizeof(float),
                  (cudaStream_t)stream, u, wa, ba, wi, bi, lam, gain, a_out, drive_out, n_tokens, width, bw);
        return dd_check_launch("dd_recurrence_gates");
    }
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
