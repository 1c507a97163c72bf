// The gated delta rule with a decay per key channel, over per-request state, and what surrounds it.
//
// Per head, token by token, with S [dk, dv] float32 (row i belongs to key channel i):
//     S <- g[:, None] * S;   u = beta * (v - S^T k);   S <- S + k u^T;   o = S^T q
// so the read-out sees the token's own write. Column j of o depends on column j of S only, so a thread block owns
// (entry, head, a run of columns); a column's rows are dealt out over LPC neighbouring lanes, eight rows each in
// registers, and the two dot products of a token are a few exchanges between those lanes (the read-outs' exchanges of
// four tokens run side by side). Tokens are staged 16 at a time by cp.async into two buffers in turn. The state is stored column
// by column ([slots, heads, dv, 8 * LPC], rows past dk stay zero), a thread's rows as two 16-byte pieces. A portion of
// a prompt and a single token run the same instructions in the same order, so a prompt cut anywhere gives the same
// bits.
//
// dd_delta_prepare makes the recurrence's operands, a row of blocks a token, all float32 inside: q, k and v pass a short
// causal convolution over time per channel (taps [channels, n], the last tap is the current token's; the n - 1 inputs
// before a step's first token come from the request's state) and silu; q and k are made unit vectors per head
// (x / sqrt(sum x^2 + 1e-6)), q times dk^-1/2; beta = sigmoid(b); g = exp(-exp(A_log[head]) * softplus(a + dt_bias)).
// dd_conv_state_update then leaves the last n - 1 inputs of every entry in its state rows. dd_delta_finish divides
// every head's o by its root mean square, multiplies by a weight [dv] and by sigmoid(gate) and rounds once.
#include "common.cuh"

namespace {
__device__ __forceinline__ float dr_softplus(float x) { return x > 20.f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float dr_sigmoid(float x) { return 1.0f / (1.0f + expf(-x)); }
template <int BYTES> __device__ __forceinline__ void dr_cp_async(float* dst, const float* src) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    if (BYTES == 16) asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
    else asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(src) : "memory");
}

template <typename T>
__global__ void __launch_bounds__(256)
delta_prepare_kernel(const T* __restrict__ proj, int proj_stride, const T* __restrict__ beta_in, int beta_stride,
                     const float* __restrict__ step_in, const float* __restrict__ conv_w, int taps,
                     const float* __restrict__ conv_state, const float* __restrict__ a_log, const float* __restrict__ dt_bias,
                     const int* __restrict__ tok_entry, const int* __restrict__ entry_start, const int* __restrict__ entry_slot,
                     float* __restrict__ q_out, float* __restrict__ k_out, float* __restrict__ v_out,
                     float* __restrict__ decay_out, float* __restrict__ beta_out, int H, int G, int dk, int dv) {
    // A token's work is dealt out over the gridDim.y blocks of its row: the value channels, decays and step sizes element
    // by element over all their threads, the head vectors of q and k a warp each (convolution, silu and the unit norm stay
    // inside the warp). An element is computed by the same instructions wherever it lands.
    dd_launch_dependents();
    const int t = blockIdx.x;
    const int e = tok_entry[t];
    const int at = t - entry_start[e];              // tokens of this entry before t in this step
    const int qk = G * dk, C = 2 * qk + H * dv;
    const float* before = conv_state + (size_t)entry_slot[e] * (taps - 1) * C;
    dd_grid_wait();
    auto conv = [&](int c) {
        float acc = 0.f;
        for (int j = 0; j < taps; ++j) {
            const int back = taps - 1 - j;          // tap j reads the input `back` tokens ago
            const float in = back <= at ? dd_to_f32(proj[(size_t)(t - back) * proj_stride + c])
                                        : before[(size_t)(taps - 1 + at - back) * C + c];
            acc = fmaf(conv_w[(size_t)c * taps + j], in, acc);
        }
        return acc * dr_sigmoid(acc);
    };
    const int first = blockIdx.y * blockDim.x + threadIdx.x, stride = gridDim.y * blockDim.x;
#pragma unroll 4
    for (int i = first; i < H * dv; i += stride) v_out[(size_t)t * H * dv + i] = conv(2 * qk + i);
#pragma unroll 4
    for (int i = first; i < H * dk; i += stride)
        decay_out[(size_t)t * H * dk + i] = expf(-expf(a_log[i / dk]) * dr_softplus(step_in[(size_t)t * H * dk + i] + dt_bias[i]));
    for (int h = first; h < H; h += stride)
        beta_out[(size_t)t * H + h] = dr_sigmoid(dd_to_f32(beta_in[(size_t)t * beta_stride + h]));
    // unit vectors: a warp a head of q or k; a lane's first four elements stay in registers, further ones are computed again
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    const float q_scale = 1.0f / sqrtf((float)dk);
    for (int vec = blockIdx.y * warps + warp; vec < 2 * G; vec += gridDim.y * warps) {
        const int c0 = vec * dk;
        float y[4], ss = 0.f;
#pragma unroll
        for (int r = 0; r < 4; ++r) y[r] = lane + 32 * r < dk ? conv(c0 + lane + 32 * r) : 0.f;
#pragma unroll
        for (int r = 0; r < 4; ++r) ss = fmaf(y[r], y[r], ss);
        for (int i = lane + 128; i < dk; i += 32) {
            const float x = conv(c0 + i);
            ss = fmaf(x, x, ss);
        }
        ss = dd_warp_sum(ss);
        const float inv = 1.0f / sqrtf(ss + 1e-6f);
        const bool is_q = vec < G;
        float* dst = is_q ? q_out + (size_t)t * qk + (size_t)vec * dk : k_out + (size_t)t * qk + (size_t)(vec - G) * dk;
        const float f = is_q ? inv * q_scale : inv;
#pragma unroll
        for (int r = 0; r < 4; ++r)
            if (lane + 32 * r < dk) dst[lane + 32 * r] = y[r] * f;
        for (int i = lane + 128; i < dk; i += 32) dst[i] = conv(c0 + i) * f;
    }
}

template <typename T>
__global__ void __launch_bounds__(128)
conv_state_update_kernel(const T* __restrict__ proj, int proj_stride, float* __restrict__ conv_state, int taps,
                         const int* __restrict__ entry_start, const int* __restrict__ entry_slot, int C) {
    dd_launch_dependents();
    dd_grid_wait();
    const int e = blockIdx.y;
    const int c = blockIdx.x * 128 + threadIdx.x;
    if (c >= C) return;
    const int start = entry_start[e], n = entry_start[e + 1] - start, keep = taps - 1;
    float* rows = conv_state + (size_t)entry_slot[e] * keep * C;
    // the last `keep` inputs of (what the state held, then this step's); row j takes what lay n rows later, so rows are
    // read before they are overwritten
    for (int j = 0; j < keep; ++j) {
        const int src = j + n;
        rows[(size_t)j * C + c] = src < keep ? rows[(size_t)src * C + c]
                                             : dd_to_f32(proj[(size_t)(start + src - keep) * proj_stride + c]);
    }
}

constexpr int DR_THREADS = 128;
constexpr int DR_TOKENS = 16;          // tokens staged together

template <int LPC>
__global__ void __launch_bounds__(DR_THREADS)
delta_rule_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                  const float* __restrict__ decay, const float* __restrict__ beta, const int* __restrict__ entry_start,
                  const int* __restrict__ entry_slot, float* __restrict__ state, float* __restrict__ out,
                  int H, int G, int dk, int dv) {
    constexpr int DKP = 8 * LPC, COLS = DR_THREADS / LPC;
    constexpr int BUF = DR_TOKENS * (3 * DKP + COLS) + DR_TOKENS;       // floats of one buffer: q, k, decay, v, beta
    extern __shared__ __align__(16) float staged[];                      // two buffers, filled in turn by cp.async
    dd_launch_dependents();
    const int e = blockIdx.z, h = blockIdx.y, g = h / (H / G);
    const int col0 = blockIdx.x * COLS;
    const int my_col = threadIdx.x / LPC, sub = threadIdx.x % LPC;
    const int col = col0 + my_col;
    const bool live = col < dv;
    const int start = entry_start[e], end = entry_start[e + 1];
    // the state is an earlier step's: it is in registers before the kernel before this one has finished
    float* sp = state + (((size_t)entry_slot[e] * H + h) * dv + (live ? col : 0)) * DKP + sub * 8;
    float s[8];
    {
        const float4 a = *reinterpret_cast<const float4*>(sp), b = *reinterpret_cast<const float4*>(sp + 4);
        s[0] = a.x; s[1] = a.y; s[2] = a.z; s[3] = a.w; s[4] = b.x; s[5] = b.y; s[6] = b.z; s[7] = b.w;
    }
    // rows past dk and columns past dv are never copied into: they stay the zeros written here
    if (dk != DKP || col0 + COLS > dv)
        for (int i = threadIdx.x; i < 2 * BUF; i += DR_THREADS) staged[i] = 0.f;
    // 16-byte copies where every row starts on such a boundary
    const bool wide = dk % 4 == 0 && dv % 4 == 0 && !(((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)decay) & 15);
    auto stage = [&](int t0, int buf) {
        const int n = min(DR_TOKENS, end - t0);
        float* bq = staged + buf * BUF;
        float* bk = bq + DR_TOKENS * DKP;
        float* bg = bk + DR_TOKENS * DKP;
        float* bv = bg + DR_TOKENS * DKP;
        float* bb = bv + DR_TOKENS * COLS;
        if (wide) {
            for (int i = threadIdx.x; i < n * (DKP / 4); i += DR_THREADS) {
                const int tt = i / (DKP / 4), r = (i % (DKP / 4)) * 4;
                if (r < dk) {
                    dr_cp_async<16>(bq + tt * DKP + r, q + (size_t)(t0 + tt) * G * dk + (size_t)g * dk + r);
                    dr_cp_async<16>(bk + tt * DKP + r, k + (size_t)(t0 + tt) * G * dk + (size_t)g * dk + r);
                    dr_cp_async<16>(bg + tt * DKP + r, decay + (size_t)(t0 + tt) * H * dk + (size_t)h * dk + r);
                }
            }
            for (int i = threadIdx.x; i < n * (COLS / 4); i += DR_THREADS) {
                const int tt = i / (COLS / 4), c = (i % (COLS / 4)) * 4;
                if (col0 + c < dv) dr_cp_async<16>(bv + tt * COLS + c, v + (size_t)(t0 + tt) * H * dv + (size_t)h * dv + col0 + c);
            }
        } else {
            for (int i = threadIdx.x; i < n * DKP; i += DR_THREADS) {
                const int tt = i / DKP, r = i % DKP;
                if (r < dk) {
                    dr_cp_async<4>(bq + i, q + (size_t)(t0 + tt) * G * dk + (size_t)g * dk + r);
                    dr_cp_async<4>(bk + i, k + (size_t)(t0 + tt) * G * dk + (size_t)g * dk + r);
                    dr_cp_async<4>(bg + i, decay + (size_t)(t0 + tt) * H * dk + (size_t)h * dk + r);
                }
            }
            for (int i = threadIdx.x; i < n * COLS; i += DR_THREADS) {
                const int tt = i / COLS, c = i % COLS;
                if (col0 + c < dv) dr_cp_async<4>(bv + i, v + (size_t)(t0 + tt) * H * dv + (size_t)h * dv + col0 + c);
            }
        }
        if (threadIdx.x < n) dr_cp_async<4>(bb + threadIdx.x, beta + (size_t)(t0 + threadIdx.x) * H + h);
    };
    dd_grid_wait();
    __syncthreads();                                    // the zeros are written before any copy lands
    if (start < end) stage(start, 0);
    asm volatile("cp.async.commit_group;" ::: "memory");
    int buf = 0;
    for (int t0 = start; t0 < end; t0 += DR_TOKENS, buf ^= 1) {
        const int n = min(DR_TOKENS, end - t0);
        if (t0 + DR_TOKENS < end) stage(t0 + DR_TOKENS, buf ^ 1);      // (that buffer's tokens were read before the last barrier)
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 1;" ::: "memory");
        __syncthreads();
        const float* sq = staged + buf * BUF;
        const float* sk = sq + DR_TOKENS * DKP;
        const float* sg = sk + DR_TOKENS * DKP;
        const float* sv = sg + DR_TOKENS * DKP;
        const float* sb = sv + DR_TOKENS * COLS;
        // Four tokens at a time: the state goes through them one after the other (a token's write needs its own
        // exchanged dot product), but their read-outs' exchanges wait until all four are there and then run level by
        // level side by side, so that only the first dot product's exchanges lie on the chain from token to token.
        for (int tt0 = 0; tt0 < n; tt0 += 4) {
            float read[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                read[j] = 0.f;
                const int tt = tt0 + j;
                if (tt < n) {
                    const float4* q4 = reinterpret_cast<const float4*>(sq + tt * DKP + sub * 8);
                    const float4* k4 = reinterpret_cast<const float4*>(sk + tt * DKP + sub * 8);
                    const float4* g4 = reinterpret_cast<const float4*>(sg + tt * DKP + sub * 8);
                    const float4 ka = k4[0], kb = k4[1], ga = g4[0], gb = g4[1], qa = q4[0], qb = q4[1];
                    const float kk[8] = {ka.x, ka.y, ka.z, ka.w, kb.x, kb.y, kb.z, kb.w};
                    const float gg[8] = {ga.x, ga.y, ga.z, ga.w, gb.x, gb.y, gb.z, gb.w};
                    const float qq[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
                    float dot = 0.f;
#pragma unroll
                    for (int r = 0; r < 8; ++r) {
                        s[r] = __fmul_rn(s[r], gg[r]);
                        dot = __fmaf_rn(s[r], kk[r], dot);
                    }
#pragma unroll
                    for (int o = LPC / 2; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
                    const float u = __fmul_rn(sb[tt], __fsub_rn(sv[tt * COLS + my_col], dot));
#pragma unroll
                    for (int r = 0; r < 8; ++r) {
                        s[r] = __fmaf_rn(kk[r], u, s[r]);
                        read[j] = __fmaf_rn(s[r], qq[r], read[j]);
                    }
                }
            }
#pragma unroll
            for (int o = LPC / 2; o > 0; o >>= 1) {
#pragma unroll
                for (int j = 0; j < 4; ++j) read[j] += __shfl_xor_sync(0xffffffffu, read[j], o);
            }
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (tt0 + j < n && live && sub == 0) out[(size_t)(t0 + tt0 + j) * H * dv + (size_t)h * dv + col] = read[j];
        }
        __syncthreads();                                // all have read this buffer before the copies after next fill it
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    if (live) {
        *reinterpret_cast<float4*>(sp) = make_float4(s[0], s[1], s[2], s[3]);
        *reinterpret_cast<float4*>(sp + 4) = make_float4(s[4], s[5], s[6], s[7]);
    }
}

template <typename TO>
__global__ void __launch_bounds__(128)
delta_finish_kernel(const float* __restrict__ o, const float* __restrict__ gate, const float* __restrict__ weight,
                    TO* __restrict__ out, int out_stride, int n, int H, int dv, float eps) {
    dd_launch_dependents();
    dd_grid_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * 4 + warp;        // (token, head)
    if (item >= (long long)n * H) return;
    const int t = (int)(item / H), h = (int)(item % H);
    const float* row = o + (size_t)item * dv;
    const float* gr = gate + (size_t)item * dv;
    float ss = 0.f;
    for (int c = lane; c < dv; c += 32) ss = fmaf(row[c], row[c], ss);
    ss = dd_warp_sum(ss);
    const float r = 1.0f / sqrtf(ss / (float)dv + eps);
    TO* dst = out + (size_t)t * out_stride + (size_t)h * dv;
    for (int c = lane; c < dv; c += 32) dst[c] = dd_from_f32<TO>(row[c] * r * weight[c] * dr_sigmoid(gr[c]));
}

int lanes_per_column(int dk) {
    int lpc = 1;
    while (lpc * 8 < dk) lpc *= 2;
    return lpc;
}
}  // namespace

// Rows of a column as the kernel stores them: the key size rounded up to 8 * (a power of two) (at most 256).
DD_API int dd_delta_state_rows(int dk) { return dk > 0 && dk <= 256 ? 8 * lanes_per_column(dk) : 0; }

// proj: [N, proj_stride] rows whose first 2 * G * dk + H * dv elements are the q, k and v projections; beta_in: a
// [N, H] view; step_in: float32 [N, H * dk]; conv_w: float32 [channels, taps]; conv_state: float32
// [slots, taps - 1, channels]. Outputs float32: q, k [N, G * dk], v [N, H * dv], decay [N, H * dk], beta [N, H].
DD_API int dd_delta_prepare(const void* proj, int proj_stride, const void* beta_in, int beta_stride, const float* step_in,
                            const float* conv_w, int taps, const float* conv_state, const float* a_log, const float* dt_bias,
                            const int* tok_entry, const int* entry_start, const int* entry_slot, float* q_out, float* k_out,
                            float* v_out, float* decay_out, float* beta_out, int n, int H, int G, int dk, int dv, int dtype,
                            void* stream) {
    if (n <= 0) return 0;
    if (taps < 1 || H <= 0 || G <= 0 || H % G || dk <= 0 || dv <= 0) return dd_fail("dd_delta_prepare: bad sizes");
    cudaStream_t s = (cudaStream_t)stream;
    // few tokens: a token's row of blocks grows until the GPU is filled (every thread keeps at least one element)
    const int most = (int)dd_ceil_div((long long)H * (dv + dk), 256);
    int chunks = 1;
    while (chunks < most && (long long)n * chunks < 592) chunks *= 2;
    chunks = chunks < most ? chunks : most;
#define DD_PREP(T)                                                                                                        \
    dd_launch(delta_prepare_kernel<T>, dim3(n, chunks), dim3(256), 0, s, (const T*)proj, proj_stride, (const T*)beta_in,    \
              beta_stride, step_in, conv_w, taps, conv_state, a_log, dt_bias, tok_entry, entry_start, entry_slot, q_out,   \
              k_out, v_out, decay_out, beta_out, H, G, dk, dv)
    if (dtype == DD_F32) DD_PREP(float);
    else if (dtype == DD_BF16) DD_PREP(__nv_bfloat16);
    else return dd_fail("dd_delta_prepare: unknown dtype %d", dtype);
#undef DD_PREP
    return dd_check_launch("dd_delta_prepare");
}

DD_API int dd_conv_state_update(const void* proj, int proj_stride, float* conv_state, int taps, const int* entry_start,
                                const int* entry_slot, int n_entries, int channels, int dtype, void* stream) {
    if (n_entries <= 0 || taps <= 1) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid(dd_ceil_div(channels, 128), n_entries);
    if (dtype == DD_F32)
        dd_launch(conv_state_update_kernel<float>, grid, dim3(128), 0, s, (const float*)proj, proj_stride, conv_state, taps,
                  entry_start, entry_slot, channels);
    else if (dtype == DD_BF16)
        dd_launch(conv_state_update_kernel<__nv_bfloat16>, grid, dim3(128), 0, s, (const __nv_bfloat16*)proj, proj_stride,
                  conv_state, taps, entry_start, entry_slot, channels);
    else
        return dd_fail("dd_conv_state_update: unknown dtype %d", dtype);
    return dd_check_launch("dd_conv_state_update");
}

// q, k: float32 [N, G * dk]; v: [N, H * dv]; decay: [N, H * dk]; beta: [N, H]; state: float32
// [slots, H, dv, dd_delta_state_rows(dk)], read and written; out: float32 [N, H * dv].
DD_API int dd_delta_rule(const float* q, const float* k, const float* v, const float* decay, const float* beta,
                         const int* entry_start, const int* entry_slot, int n_entries, float* state, float* out, int H, int G,
                         int dk, int dv, void* stream) {
    if (n_entries <= 0) return 0;
    if (dk <= 0 || dk > 256 || dv <= 0 || H <= 0 || G <= 0 || H % G)
        return dd_fail("dd_delta_rule: heads of %d by %d are not supported (keys of at most 256)", dk, dv);
    cudaStream_t s = (cudaStream_t)stream;
    const int lpc = lanes_per_column(dk);
    const int cols = DR_THREADS / lpc;
    const dim3 grid(dd_ceil_div(dv, cols), H, n_entries);
    const size_t smem = (size_t)2 * (DR_TOKENS * (3 * 8 * lpc + cols + 1)) * sizeof(float);
#define DD_RULE(L)                                                                                                      \
    do {                                                                                                                \
        if (smem > 48 * 1024)                                                                                           \
            cudaFuncSetAttribute(delta_rule_kernel<L>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);          \
        dd_launch(delta_rule_kernel<L>, grid, dim3(DR_THREADS), smem, s, q, k, v, decay, beta, entry_start, entry_slot,   \
                  state, out, H, G, dk, dv);                                                                            \
    } while (0)
    switch (lpc) {
        case 1: DD_RULE(1); break;
        case 2: DD_RULE(2); break;
        case 4: DD_RULE(4); break;
        case 8: DD_RULE(8); break;
        case 16: DD_RULE(16); break;
        default: DD_RULE(32); break;
    }
#undef DD_RULE
    return dd_check_launch("dd_delta_rule");
}

// o, gate: float32 [N, H * dv]; weight: float32 [dv]; out: [N, out_stride] in out_dtype.
DD_API int dd_delta_finish(const float* o, const float* gate, const float* weight, void* out, int out_stride, int n, int H,
                           int dv, float eps, int out_dtype, void* stream) {
    if (n <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const int grid = dd_ceil_div((long long)n * H, 4);
    if (out_dtype == DD_F32)
        dd_launch(delta_finish_kernel<float>, dim3(grid), dim3(128), 0, s, o, gate, weight, (float*)out, out_stride, n, H, dv, eps);
    else if (out_dtype == DD_BF16)
        dd_launch(delta_finish_kernel<__nv_bfloat16>, dim3(grid), dim3(128), 0, s, o, gate, weight, (__nv_bfloat16*)out,
                  out_stride, n, H, dv, eps);
    else
        return dd_fail("dd_delta_finish: unknown output dtype %d", out_dtype);
    return dd_check_launch("dd_delta_finish");
}
