// A state-space mixer with a scalar decay per head (the recurrent form of state-space duality), and the short causal
// convolution over time that feeds it (and other recurrent mixers).
//
//   dd_conv_channels      out[t, c] = act(bias[c] + sum_j taps[c, j] * in[t - (n - 1 - j), c]); the n - 1 inputs before a step's
//                         first token of a request come from its state rows (dd_conv_state_update of delta_rule.cu leaves
//                         them there afterwards); float32 out
//   dd_state_space_scan   per head h (group g = h / (H / G)), from the request's state S [N, dv] (float32):
//                         dt = softplus(dt_in + dt_bias[h]); S <- exp(-exp(A_log[h]) dt) S + dt B_t x_t^T;
//                         y_t = S^T C_t + D[h] x_t
//   dd_gated_group_norm   out = (y * silu(z)) in `groups` equal stretches, each divided by its root mean square, times a weight
//
// Column p of y depends on column p of S only: a block owns (entry, head, a run of columns); a column's N rows are dealt out
// over neighbouring lanes, eight rows each in registers, so the read-out is a few exchanges between lanes. The state lies
// column by column ([slots, H, dv, N rounded up]).
// A portion and a single token run the same instructions in the same order: a prompt cut anywhere gives the same bits.
#include "common.cuh"

namespace {
__device__ __forceinline__ float ss_softplus(float x) { return x > 20.f ? x : log1pf(expf(x)); }

template <typename T>
__global__ void __launch_bounds__(128)
conv_channels_kernel(const T* __restrict__ in, int in_stride, const float* __restrict__ taps_w, const float* __restrict__ bias,
                     int taps, const float* __restrict__ conv_state, const int* __restrict__ tok_entry,
                     const int* __restrict__ entry_start, const int* __restrict__ entry_slot, float* __restrict__ out,
                     int out_stride, int C, int act) {
    dd_launch_dependents();
    const int t = blockIdx.y;
    const int c = blockIdx.x * 128 + threadIdx.x;
    if (c >= C) return;
    float w[16];
    for (int j = 0; j < taps; ++j) w[j] = taps_w[(size_t)c * taps + j];
    float acc = bias ? bias[c] : 0.f;
    dd_grid_wait();
    const int e = tok_entry[t];
    const int at = t - entry_start[e];
    const float* before = conv_state + (size_t)entry_slot[e] * (taps - 1) * C;
    for (int j = 0; j < taps; ++j) {
        const int back = taps - 1 - j;
        const float v = back <= at ? dd_to_f32(in[(size_t)(t - back) * in_stride + c])
                                   : before[(size_t)(taps - 1 + at - back) * C + c];
        acc = fmaf(w[j], v, acc);
    }
    if (act == 1) acc = acc / (1.0f + expf(-acc));
    out[(size_t)t * out_stride + c] = acc;
}

constexpr int SS_THREADS = 128;
constexpr int SS_TOKENS = 16;         // tokens staged together

// LPC lanes share a column; each holds rows sub * 8 .. sub * 8 + 7 of it. The tokens of an entry are staged SS_TOKENS at a
// time in shared memory: B and C rows (padded with zeros to the rows the lanes hold), the block's columns of x, and the step
// size and 1 - decay of every token, which 16 threads compute side by side so that the exponentials and the logarithm do
// not lie on the chain from token to token. While a chunk is worked on, the next one is already on its way in registers.
template <typename T, int LPC>
__global__ void __launch_bounds__(SS_THREADS)
state_space_scan_kernel(const float* __restrict__ xbc, int xbc_stride, const T* __restrict__ dt_in, int dt_stride,
                        const float* __restrict__ dt_bias, const float* __restrict__ a_log, const float* __restrict__ skip,
                        const int* __restrict__ entry_start, const int* __restrict__ entry_slot, float* __restrict__ state,
                        float* __restrict__ out, int H, int G, int N, int dv) {
    constexpr int NP = LPC * 8, COLS = SS_THREADS / LPC;
    constexpr int ROW = 2 * NP + COLS;                                   // staged floats of one token: B, C, x
    constexpr int PER_THREAD = (SS_TOKENS * ROW + SS_THREADS - 1) / SS_THREADS;
    __shared__ __align__(16) float staged[SS_TOKENS * ROW];
    __shared__ float steps[SS_TOKENS], fades[SS_TOKENS];
    dd_launch_dependents();
    const int e = blockIdx.z, h = blockIdx.y, g = h / (H / G);
    const int col0 = blockIdx.x * COLS;
    const int my_col = threadIdx.x / LPC, sub = threadIdx.x % LPC;
    const int col = col0 + my_col;
    const bool live = col < dv;
    const int start = entry_start[e], end = entry_start[e + 1];
    float* sp = state + (((size_t)entry_slot[e] * H + h) * dv + (live ? col : 0)) * NP + sub * 8;
    const float rate = -expf(a_log[h]), bias = dt_bias[h], d_skip = skip[h];
    const int inner = H * dv;
    const int b_from = inner + g * N, c_from = inner + G * N + g * N, x_from = h * dv + col0;
    dd_grid_wait();
    float s[8];
    {
        const float4 a = *reinterpret_cast<const float4*>(sp), b = *reinterpret_cast<const float4*>(sp + 4);
        s[0] = a.x; s[1] = a.y; s[2] = a.z; s[3] = a.w; s[4] = b.x; s[5] = b.y; s[6] = b.z; s[7] = b.w;
    }
    float ahead[PER_THREAD], dt_ahead = 0.f;
    // element i of a chunk: token i / ROW, then B rows [0, NP), C rows [NP, 2 NP), x columns [2 NP, ROW)
    auto fetch = [&](int t0) {
#pragma unroll
        for (int j = 0; j < PER_THREAD; ++j) {
            const int i = threadIdx.x + j * SS_THREADS;
            const int tok = i / ROW, r = i % ROW;
            float v = 0.f;
            if (i < SS_TOKENS * ROW && t0 + tok < end) {
                const float* row = xbc + (size_t)(t0 + tok) * xbc_stride;
                if (r < NP) { if (r < N) v = row[b_from + r]; }
                else if (r < 2 * NP) { if (r - NP < N) v = row[c_from + r - NP]; }
                else if (col0 + r - 2 * NP < dv) v = row[x_from + r - 2 * NP];
            }
            ahead[j] = v;
        }
        if (threadIdx.x < SS_TOKENS && t0 + (int)threadIdx.x < end) dt_ahead = dd_to_f32(dt_in[(size_t)(t0 + threadIdx.x) * dt_stride + h]);
    };
    fetch(start);
    for (int t0 = start; t0 < end; t0 += SS_TOKENS) {
        __syncthreads();                                  // the chunk before has been read
#pragma unroll
        for (int j = 0; j < PER_THREAD; ++j) {
            const int i = threadIdx.x + j * SS_THREADS;
            if (i < SS_TOKENS * ROW) staged[i] = ahead[j];
        }
        if (threadIdx.x < SS_TOKENS) {
            // tokens past the entry's end get a step of zero and no decay: they leave the state as it is, bit for bit
            const bool real = t0 + (int)threadIdx.x < end;
            const float dt = real ? ss_softplus(dt_ahead + bias) : 0.f;
            steps[threadIdx.x] = dt;
            fades[threadIdx.x] = real ? -expm1f(rate * dt) : 0.f;      // 1 - decay: a decay near one would lose its distance from one to rounding
        }
        __syncthreads();
        if (t0 + SS_TOKENS < end) fetch(t0 + SS_TOKENS);
        const int n = min(SS_TOKENS, end - t0);
        // four tokens at a time: the state's chain runs through them one after the other (two multiply-adds a token and
        // row), their read-outs and the exchanges between a column's lanes side by side
        for (int k0 = 0; k0 < n; k0 += 4) {
            float y[4], xs[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float* row = staged + (k0 + i) * ROW;
                const float dt = steps[k0 + i], fade = fades[k0 + i];
                xs[i] = row[2 * NP + my_col];
                const float dtx = dt * xs[i];
                const float4 b0 = *reinterpret_cast<const float4*>(row + sub * 8), b1 = *reinterpret_cast<const float4*>(row + sub * 8 + 4);
                const float4 c0 = *reinterpret_cast<const float4*>(row + NP + sub * 8), c1 = *reinterpret_cast<const float4*>(row + NP + sub * 8 + 4);
                const float bn[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
                const float cn[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
                float acc = 0.f;
#pragma unroll
                for (int r = 0; r < 8; ++r) {
                    s[r] = fmaf(dtx, bn[r], fmaf(-fade, s[r], s[r]));
                    acc = fmaf(s[r], cn[r], acc);
                }
                y[i] = acc;
            }
#pragma unroll
            for (int o = LPC / 2; o > 0; o >>= 1) {
#pragma unroll
                for (int i = 0; i < 4; ++i) y[i] += __shfl_xor_sync(0xffffffffu, y[i], o);
            }
            if (live && sub == 0) {
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    if (k0 + i < n) out[(size_t)(t0 + k0 + i) * inner + h * dv + col] = fmaf(d_skip, xs[i], y[i]);
            }
        }
    }
    if (live) {
        *reinterpret_cast<float4*>(sp) = make_float4(s[0], s[1], s[2], s[3]);
        *reinterpret_cast<float4*>(sp + 4) = make_float4(s[4], s[5], s[6], s[7]);
    }
}

// A block owns a stretch of one token. A thread keeps up to GN_KEEP gated values in registers between the sum of squares and
// the scaling; a stretch longer than the block holds that way is gated again in the second pass (the same instructions).
constexpr int GN_KEEP = 8;

// Entries of one token each (a decode step): nothing to stage; a thread reads its rows of B and C and its column of x
// directly. The arithmetic of a token is that of the staged kernel, instruction for instruction.
template <typename T, int LPC>
__global__ void __launch_bounds__(SS_THREADS)
state_space_single_kernel(const float* __restrict__ xbc, int xbc_stride, const T* __restrict__ dt_in, int dt_stride,
                          const float* __restrict__ dt_bias, const float* __restrict__ a_log, const float* __restrict__ skip,
                          const int* __restrict__ entry_start, const int* __restrict__ entry_slot, float* __restrict__ state,
                          float* __restrict__ out, int H, int G, int N, int dv) {
    constexpr int NP = LPC * 8, COLS = SS_THREADS / LPC;
    dd_launch_dependents();
    const int e = blockIdx.z, h = blockIdx.y, g = h / (H / G);
    const int col = blockIdx.x * COLS + threadIdx.x / LPC, sub = threadIdx.x % LPC;
    const bool live = col < dv;
    const int t = entry_start[e];
    float* sp = state + (((size_t)entry_slot[e] * H + h) * dv + (live ? col : 0)) * NP + sub * 8;
    const float rate = -expf(a_log[h]), bias = dt_bias[h], d_skip = skip[h];
    const int inner = H * dv;
    dd_grid_wait();
    const float4 s0 = *reinterpret_cast<const float4*>(sp), s1 = *reinterpret_cast<const float4*>(sp + 4);
    float s[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
    const float* row = xbc + (size_t)t * xbc_stride;
    const float dt = ss_softplus(dd_to_f32(dt_in[(size_t)t * dt_stride + h]) + bias);
    const float fade = -expm1f(rate * dt);
    const float x = live ? row[h * dv + col] : 0.f;
    const float dtx = dt * x;
    float y = 0.f;
#pragma unroll
    for (int r = 0; r < 8; ++r) {
        const int n = sub * 8 + r;
        const float bn = n < N ? row[inner + g * N + n] : 0.f;
        const float cn = n < N ? row[inner + G * N + g * N + n] : 0.f;
        s[r] = fmaf(dtx, bn, fmaf(-fade, s[r], s[r]));
        y = fmaf(s[r], cn, y);
    }
#pragma unroll
    for (int o = LPC / 2; o > 0; o >>= 1) y += __shfl_xor_sync(0xffffffffu, y, o);
    if (live) {
        if (sub == 0) out[(size_t)t * inner + h * dv + col] = fmaf(d_skip, x, y);
        *reinterpret_cast<float4*>(sp) = make_float4(s[0], s[1], s[2], s[3]);
        *reinterpret_cast<float4*>(sp + 4) = make_float4(s[4], s[5], s[6], s[7]);
    }
}

template <typename T>
__global__ void __launch_bounds__(256)
gated_group_norm_kernel(const float* __restrict__ y, const T* __restrict__ z, int z_stride, const float* __restrict__ w, float eps,
                        T* __restrict__ out, int out_stride, int groups, int inner) {
    __shared__ float scratch[8];
    dd_launch_dependents();
    dd_grid_wait();
    const int t = blockIdx.x, g = blockIdx.y, size = inner / groups;
    const float* yr = y + (size_t)t * inner + g * size;
    const T* zr = z + (size_t)t * z_stride + g * size;
    auto gated = [&](int c) {
        const float gate = dd_to_f32(zr[c]);
        return yr[c] * (gate / (1.0f + expf(-gate)));
    };
    float kept[GN_KEEP];
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < GN_KEEP; ++j) {
        const int c = threadIdx.x + j * blockDim.x;
        kept[j] = c < size ? gated(c) : 0.f;
        sum = fmaf(kept[j], kept[j], sum);
    }
    for (int c = threadIdx.x + GN_KEEP * blockDim.x; c < size; c += blockDim.x) { const float v = gated(c); sum = fmaf(v, v, sum); }
    sum = dd_warp_sum(sum);
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = sum;
    __syncthreads();
    float total = 0.f;
    for (int i = 0; i < (int)(blockDim.x >> 5); ++i) total += scratch[i];
    const float r = rsqrtf(total / (float)size + eps);
    T* o = out + (size_t)t * out_stride + g * size;
#pragma unroll
    for (int j = 0; j < GN_KEEP; ++j) {
        const int c = threadIdx.x + j * blockDim.x;
        if (c < size) o[c] = dd_from_f32<T>(kept[j] * r * w[g * size + c]);
    }
    for (int c = threadIdx.x + GN_KEEP * blockDim.x; c < size; c += blockDim.x) o[c] = dd_from_f32<T>(gated(c) * r * w[g * size + c]);
}

int lanes_per_column(int n) {
    int lanes = 1;
    while (lanes * 8 < n) lanes *= 2;
    return lanes;
}

template <typename T>
int launch_scan(bool single, int lpc, dim3 grid, cudaStream_t s, const float* xbc, int xbc_stride, const T* dt_in, int dt_stride,
                const float* dt_bias, const float* a_log, const float* skip, const int* entry_start, const int* entry_slot,
                float* state, float* out, int H, int G, int N, int dv) {
#define SS_CASE(L) case L: if (single) dd_launch(state_space_single_kernel<T, L>, grid, dim3(SS_THREADS), 0, s, xbc, xbc_stride, dt_in, \
                                                 dt_stride, dt_bias, a_log, skip, entry_start, entry_slot, state, out, H, G, N, dv); \
                   else dd_launch(state_space_scan_kernel<T, L>, grid, dim3(SS_THREADS), 0, s, xbc, xbc_stride, dt_in, dt_stride, \
                                  dt_bias, a_log, skip, entry_start, entry_slot, state, out, H, G, N, dv); break;
    switch (lpc) {
        SS_CASE(1) SS_CASE(2) SS_CASE(4) SS_CASE(8) SS_CASE(16) SS_CASE(32)
        default: return dd_fail("dd_state_space_scan: a state of %d rows is not supported (at most 256)", N);
    }
#undef SS_CASE
    return dd_check_launch("dd_state_space_scan");
}
}  // namespace

// Floats of one column of the state as it is stored (N rounded up to what the lanes of a column hold).
DD_API int dd_state_space_rows(int n) { return lanes_per_column(n) * 8; }

// in: [N, >= C] row view (row stride in_stride); taps_w float32 [C, taps]; bias float32 [C] or null; conv_state float32
// [slots, taps - 1, C]; out float32 rows of stride out_stride. act: 0 none, 1 silu.
DD_API int dd_conv_channels(const void* in, int in_stride, const float* taps_w, const float* bias, int taps, const float* conv_state,
                            const int* tok_entry, const int* entry_start, const int* entry_slot, float* out, int out_stride,
                            int n_tokens, int channels, int act, int dtype, void* stream) {
    if (n_tokens <= 0 || channels <= 0) return 0;
    if (taps < 1 || taps > 16) return dd_fail("dd_conv_channels: %d taps are not supported (1 to 16)", taps);
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid(dd_ceil_div(channels, 128), n_tokens);
    if (dtype == DD_F32)
        dd_launch(conv_channels_kernel<float>, grid, dim3(128), 0, s, (const float*)in, in_stride, taps_w, bias, taps, conv_state,
                  tok_entry, entry_start, entry_slot, out, out_stride, channels, act);
    else if (dtype == DD_BF16)
        dd_launch(conv_channels_kernel<__nv_bfloat16>, grid, dim3(128), 0, s, (const __nv_bfloat16*)in, in_stride, taps_w, bias, taps,
                  conv_state, tok_entry, entry_start, entry_slot, out, out_stride, channels, act);
    else
        return dd_fail("dd_conv_channels: unknown dtype %d", dtype);
    return dd_check_launch("dd_conv_channels");
}

// xbc: float32 [N, H * dv + 2 * G * n_state] rows ([x | B | C], after the convolution and its activation); dt_in: [N, H] row
// view in `dtype`; state: float32 [slots, H, dv, dd_state_space_rows(n_state)], read and written; out: float32 [N, H * dv].
// n_tokens == n_entries (every entry brings one token) takes the kernel without staging.
DD_API int dd_state_space_scan(const float* xbc, int xbc_stride, const void* dt_in, int dt_stride, const float* dt_bias,
                               const float* a_log, const float* skip, const int* entry_start, const int* entry_slot, int n_entries,
                               float* state, float* out, int H, int G, int n_state, int dv, int dtype, void* stream, int n_tokens) {
    if (n_entries <= 0) return 0;
    if (H <= 0 || G <= 0 || H % G || n_state <= 0 || n_state > 256 || dv <= 0)
        return dd_fail("dd_state_space_scan: %d heads in %d groups with a state of %d by %d are not supported", H, G, n_state, dv);
    cudaStream_t s = (cudaStream_t)stream;
    const int lpc = lanes_per_column(n_state);
    const dim3 grid(dd_ceil_div(dv, SS_THREADS / lpc), H, n_entries);
    if (dtype == DD_F32)
        return launch_scan<float>(n_tokens == n_entries, lpc, grid, s, xbc, xbc_stride, (const float*)dt_in, dt_stride, dt_bias, a_log, skip, entry_start,
                                  entry_slot, state, out, H, G, n_state, dv);
    if (dtype == DD_BF16)
        return launch_scan<__nv_bfloat16>(n_tokens == n_entries, lpc, grid, s, xbc, xbc_stride, (const __nv_bfloat16*)dt_in, dt_stride, dt_bias, a_log, skip,
                                          entry_start, entry_slot, state, out, H, G, n_state, dv);
    return dd_fail("dd_state_space_scan: unknown dtype %d", dtype);
}

// y: float32 [N, inner]; z: [N, inner] row view in `dtype`; w: float32 [inner]; out: rows of stride out_stride in `dtype`.
DD_API int dd_gated_group_norm(const float* y, const void* z, int z_stride, const float* w, float eps, void* out, int out_stride,
                               int n_tokens, int groups, int inner, int dtype, void* stream) {
    if (n_tokens <= 0) return 0;
    if (groups <= 0 || inner <= 0 || inner % groups) return dd_fail("dd_gated_group_norm: %d does not fall into %d equal parts", inner, groups);
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid(n_tokens, groups);
    const int size = inner / groups;
    const int threads = size > 1024 ? 256 : (size > 256 ? 128 : (size > 64 ? 64 : 32));
    if (dtype == DD_F32)
        dd_launch(gated_group_norm_kernel<float>, grid, dim3(threads), 0, s, y, (const float*)z, z_stride, w, eps, (float*)out, out_stride,
                  groups, inner);
    else if (dtype == DD_BF16)
        dd_launch(gated_group_norm_kernel<__nv_bfloat16>, grid, dim3(threads), 0, s, y, (const __nv_bfloat16*)z, z_stride, w, eps,
                  (__nv_bfloat16*)out, out_stride, groups, inner);
    else
        return dd_fail("dd_gated_group_norm: unknown dtype %d", dtype);
    return dd_check_launch("dd_gated_group_norm");
}
