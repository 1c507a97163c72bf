// Attention over cached latent rows on the tensor cores (mma.sync m16n8k16, float32 accumulate), and the per-head
// matrix products around it.
//
// attention_latent_kernel: one cached row of DK bfloat16 a token is the key of EVERY head, and its first DV elements
// are the value. So the query rows of a block are (token, head) pairs: 64 consecutive pairs of one entry (a run of
// consecutive tokens of one request; a decoded token is a run of one, whose heads alone fill a good part of a tile),
// against key tiles of 64 rows that are copied once for all of them (cp.async; two buffers, or one where that lets two
// blocks share an SM; rows padded by 16 bytes so that ldmatrix is free of bank conflicts at every row length). A warp owns 16 query rows and a slice of the
// value columns; with two slices (DV above 256) both warps of a row compute the same scores. Scores, softmax and the
// weighted sums are float32; the softmax weights meet the values as two bfloat16 terms (the weight rounded, and what
// the rounding left over), so that no weight is rounded to 8 bits. A sink joins the denominator at the end. The keys
// of a row can be cut into splits (grid.y) whose partial sums a second kernel merges: that is how a step of few
// decoded tokens fills the GPU.
//
// per_head_mma_kernel: out[n, h, :] = W[h] x[n, h, :] for every head, tiles of 64 tokens x 128 outputs.
#include "common.cuh"
#include <math_constants.h>

namespace {
constexpr int BKV = 64;

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t* r) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t* r) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float bf16_low(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16_high(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }

// VT: pairs of 8-column value tiles a warp accumulates (VT * 16 value columns a warp). RG: groups of 16 query rows a
// block (4 for prompts; 2 for steps of single tokens with at most 32 heads, whose one token fills half a tile of 64).
template <int VT, int RG>
__global__ void __launch_bounds__(256)
attention_latent_kernel(const __nv_bfloat16* __restrict__ q, int q_stride, const __nv_bfloat16* __restrict__ cache,
                        const int* __restrict__ entry_start, const int* __restrict__ entry_pos0, int n_entries,
                        const int* __restrict__ block_table, int max_blocks, __nv_bfloat16* __restrict__ out,
                        int out_stride, float* __restrict__ part_o, float* __restrict__ part_ml, int H, int DK, int DV,
                        int P, int n_pages, float scale_log2e, int n_splits, int* __restrict__ error_flag,
                        const float* __restrict__ sink, int n_bufs) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int BQ = RG * 16;
    const int NC = DK / 8;                    // 16-byte chunks of a row
    const int KS = DK / 16;                   // k-steps over a row
    const int RB = DK * 2 + 16;               // bytes of a padded row in shared memory
    uint8_t* sQ = smem;
    uint8_t* sK = sQ + BQ * RB;               // [n_bufs][BKV] rows
    dd_launch_dependents();
    dd_grid_wait();

    int e = 0, tile = blockIdx.x, len = 0;
    for (; e < n_entries; ++e) {
        len = entry_start[e + 1] - entry_start[e];
        const int nt = (len * H + BQ - 1) / BQ;
        if (tile < nt) break;
        tile -= nt;
    }
    if (e == n_entries) return;
    const int pair0 = tile * BQ;                              // first (token, head) pair of the tile, within the entry
    const int pairs = min(BQ, len * H - pair0);
    const int tok0 = entry_start[e], pos0 = entry_pos0[e];
    const int pos_last = pos0 + (pair0 + pairs - 1) / H;
    const int* bt = block_table + (size_t)e * max_blocks;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, threads = blockDim.x;
    const int g = lane >> 2, t4 = lane & 3;
    const int rg = warp % RG, vh = warp / RG;                 // the warp's 16 rows, and its slice of the value columns

    for (int idx = tid; idx < BQ * NC; idx += threads) {
        const int r = idx / NC, c = idx % NC;
        uint8_t* dst = sQ + r * RB + c * 16;
        if (r < pairs) {
            const int pr = pair0 + r;
            cp_async16(dst, q + (size_t)(tok0 + pr / H) * q_stride + (size_t)(pr % H) * DK + c * 8);
        } else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
    }
    // The pages of a tile's keys are looked up one tile ahead, a thread a key, into shared memory: the copy loop then has
    // no load that its copies wait for. -1: a key that no query of the tile sees, or one without a page (error bit 2).
    __shared__ int s_page[2][BKV];
    auto find_pages = [&](int kb, int slot) {
        if (tid < BKV) {
            const int key = kb + tid;
            int page = -1;
            if (key <= pos_last) {
                const int blk = key / P;
                page = blk < max_blocks ? bt[blk] : -1;
                if (page < 0 || page >= n_pages) {
                    atomicOr(error_flag, 4);
                    page = -1;
                }
            }
            s_page[slot][tid] = page;
        }
    };
    auto load_k = [&](int kb, int buf, int slot) {
        for (int idx = tid; idx < BKV * NC; idx += threads) {
            const int r = idx / NC, c = idx % NC;
            uint8_t* dst = sK + (buf * BKV + r) * RB + c * 16;
            const int page = s_page[slot][r];
            if (page >= 0) cp_async16(dst, cache + ((size_t)page * P + (kb + r) % P) * DK + c * 8);
            else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);   // 0 * stale NaN would spoil the sum
        }
    };
    // this split's share of the key tiles
    const int all_tiles = pos_last / BKV + 1;
    const int per_split = (all_tiles + n_splits - 1) / n_splits;
    const int tile_lo = blockIdx.y * per_split, tile_hi = min(all_tiles, tile_lo + per_split);

    float o[2 * VT][4], m[2] = {-CUDART_INF_F, -CUDART_INF_F}, l[2] = {0.f, 0.f};
#pragma unroll
    for (int i = 0; i < 2 * VT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    int qpos[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) qpos[i] = pos0 + (pair0 + rg * 16 + g + 8 * i) / H;
    const int mi = lane >> 3;
    const uint32_t q_frag = smem_addr(sQ + (rg * 16 + (mi & 1) * 8 + (lane & 7)) * RB + (mi >> 1) * 16);
    const uint32_t k_frag = (uint32_t)(((mi >> 1) * 8 + (lane & 7)) * RB + (mi & 1) * 16);
    const uint32_t v_frag = (uint32_t)(((mi & 1) * 8 + (lane & 7)) * RB + (mi >> 1) * 16);
    const int col_base = vh * VT * 16;

    find_pages(tile_lo * BKV, 0);
    __syncthreads();
    if (tile_lo < tile_hi) load_k(tile_lo * BKV, 0, 0);
    cp_commit();
    find_pages((tile_lo + 1) * BKV, 1);
    for (int j = tile_lo; j < tile_hi; ++j) {
        const int kb = j * BKV, buf = n_bufs == 2 ? (j - tile_lo) & 1 : 0, slot = (j - tile_lo) & 1;
        cp_wait<0>();
        __syncthreads();                    // tile j has landed, and the pages of tile j + 1 are known to all
        if (n_bufs == 2 && j + 1 < tile_hi) {
            load_k(kb + BKV, buf ^ 1, slot ^ 1);
            cp_commit();
        }
        find_pages(kb + 2 * BKV, slot);     // (tile j's own pages have been used)
        const uint32_t tk = smem_addr(sK + buf * BKV * RB);
        float s[8][4];
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll 2
        for (int ks = 0; ks < KS; ++ks) {
            uint32_t a[4];
            ldmatrix_x4(q_frag + ks * 32, a);
#pragma unroll
            for (int np = 0; np < 4; ++np) {
                uint32_t b[4];
                ldmatrix_x4(tk + np * 16 * RB + k_frag + ks * 32, b);
                mma_bf16(s[2 * np], a, b[0], b[1]);
                mma_bf16(s[2 * np + 1], a, b[2], b[3]);
            }
        }
        float mx[2] = {-CUDART_INF_F, -CUDART_INF_F};
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int key = kb + nt * 8 + 2 * t4 + (i & 1);
                float v = s[nt][i] * scale_log2e;
                if (key > qpos[i >> 1]) v = -CUDART_INF_F;
                s[nt][i] = v;
                mx[i >> 1] = fmaxf(mx[i >> 1], v);
            }
        }
        float corr[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
            const float m_new = fmaxf(m[r], mx[r]);
            corr[r] = m_new == -CUDART_INF_F ? 1.f : exp2f(m[r] - m_new);
            m[r] = m_new;
            l[r] *= corr[r];
        }
        const float msub[2] = {m[0] == -CUDART_INF_F ? 0.f : m[0], m[1] == -CUDART_INF_F ? 0.f : m[1]};
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float p = exp2f(s[nt][i] - msub[i >> 1]);
                s[nt][i] = p;
                l[i >> 1] += p;
            }
        }
#pragma unroll
        for (int i = 0; i < 2 * VT; ++i) {
            o[i][0] *= corr[0]; o[i][1] *= corr[0];
            o[i][2] *= corr[1]; o[i][3] *= corr[1];
        }
#pragma unroll
        for (int kk = 0; kk < BKV / 16; ++kk) {
            uint32_t a[4], a2[4];
            a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
            a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
            a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
            a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
            a2[0] = pack_bf16(s[2 * kk][0] - bf16_low(a[0]), s[2 * kk][1] - bf16_high(a[0]));
            a2[1] = pack_bf16(s[2 * kk][2] - bf16_low(a[1]), s[2 * kk][3] - bf16_high(a[1]));
            a2[2] = pack_bf16(s[2 * kk + 1][0] - bf16_low(a[2]), s[2 * kk + 1][1] - bf16_high(a[2]));
            a2[3] = pack_bf16(s[2 * kk + 1][2] - bf16_low(a[3]), s[2 * kk + 1][3] - bf16_high(a[3]));
            // the rounded weights over all value columns, then the left-overs: two products into one accumulator lie
            // a whole pass apart
#pragma unroll
            for (int dp = 0; dp < VT; ++dp) {
                const int col = col_base + dp * 16;
                if (col < DV) {
                    uint32_t b[4];
                    ldmatrix_x4_trans(tk + kk * 16 * RB + v_frag + col * 2, b);
                    mma_bf16(o[2 * dp], a, b[0], b[1]);
                    mma_bf16(o[2 * dp + 1], a, b[2], b[3]);
                }
            }
#pragma unroll
            for (int dp = 0; dp < VT; ++dp) {
                const int col = col_base + dp * 16;
                if (col < DV) {
                    uint32_t b[4];
                    ldmatrix_x4_trans(tk + kk * 16 * RB + v_frag + col * 2, b);
                    mma_bf16(o[2 * dp], a2, b[0], b[1]);
                    mma_bf16(o[2 * dp + 1], a2, b[2], b[3]);
                }
            }
        }
        __syncthreads();
        if (n_bufs == 1 && j + 1 < tile_hi) {
            load_k(kb + BKV, 0, slot ^ 1);
            cp_commit();
        }
    }
    cp_wait<0>();
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = rg * 16 + g + r * 8;
        if (row >= pairs) continue;
        const int pr = pair0 + row, tok = tok0 + pr / H, h = pr % H;
        if (n_splits > 1) {
            const size_t item = ((size_t)tok * H + h) * n_splits + blockIdx.y;
            if (vh == 0 && t4 == 0) { part_ml[2 * item] = m[r]; part_ml[2 * item + 1] = l[r]; }
            float* dst = part_o + item * DV + 2 * t4;
#pragma unroll
            for (int i = 0; i < 2 * VT; ++i) {
                const int col = col_base + i * 8;
                if (col < DV) *reinterpret_cast<float2*>(dst + col) = make_float2(o[i][2 * r], o[i][2 * r + 1]);
            }
            continue;
        }
        float inv = l[r] > 0.f ? 1.f / l[r] : 0.f;
        if (sink) {
            const float s2 = sink[h] * 1.4426950408889634f, m2 = fmaxf(m[r], s2);
            const float keep = m[r] == -CUDART_INF_F ? 0.f : exp2f(m[r] - m2);
            inv = keep / (l[r] * keep + exp2f(s2 - m2));
        }
        __nv_bfloat16* dst = out + (size_t)tok * out_stride + (size_t)h * DV + 2 * t4;
#pragma unroll
        for (int i = 0; i < 2 * VT; ++i) {
            const int col = col_base + i * 8;
            if (col < DV) *reinterpret_cast<uint32_t*>(dst + col) = pack_bf16(o[i][2 * r] * inv, o[i][2 * r + 1] * inv);
        }
    }
}

// One warp a (token, head): the splits' partial sums, brought to one maximum (the sink's too), added and normed. Lane s
// holds split s's weight (at most 32 splits); a lane adds four neighbouring columns, 16 bytes a load, several in flight.
__global__ void __launch_bounds__(128)
attention_latent_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                              __nv_bfloat16* __restrict__ out, int out_stride, int n_tokens, int H, int DV, int n_splits,
                              const float* __restrict__ sink) {
    dd_launch_dependents();
    dd_grid_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long row = (long long)blockIdx.x * 4 + warp;
    if (row >= (long long)n_tokens * H) return;
    const int t = (int)(row / H), h = (int)(row % H);
    const float* ml = part_ml + (size_t)row * n_splits * 2;
    const float m_mine = lane < n_splits ? ml[2 * lane] : -CUDART_INF_F;
    const float l_mine = lane < n_splits ? ml[2 * lane + 1] : 0.f;
    const float s2 = sink ? sink[h] * 1.4426950408889634f : -CUDART_INF_F;
    float mx = fmaxf(m_mine, s2);
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, d));
    float w = m_mine == -CUDART_INF_F ? 0.f : exp2f(m_mine - mx);
    float total = w * l_mine;
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) total += __shfl_xor_sync(0xffffffffu, total, d);
    if (sink) total += exp2f(s2 - mx);
    w *= total > 0.f ? 1.f / total : 0.f;
    const float* po = part_o + (size_t)row * n_splits * DV;
    __nv_bfloat16* dst = out + (size_t)t * out_stride + (size_t)h * DV;
    for (int c0 = 0; c0 < DV; c0 += 128) {   // (every lane walks the loop: the weights travel by shuffles)
        const int c = c0 + lane * 4;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
        for (int s = 0; s < n_splits; ++s) {
            const float ws = __shfl_sync(0xffffffffu, w, s);
            if (ws != 0.f && c < DV) {       // (a split without visible keys has weight 0)
                const float4 v = *reinterpret_cast<const float4*>(po + (size_t)s * DV + c);
                acc.x = fmaf(ws, v.x, acc.x); acc.y = fmaf(ws, v.y, acc.y); acc.z = fmaf(ws, v.z, acc.z); acc.w = fmaf(ws, v.w, acc.w);
            }
        }
        if (c < DV) {
            *reinterpret_cast<uint32_t*>(dst + c) = pack_bf16(acc.x, acc.y);
            *reinterpret_cast<uint32_t*>(dst + c + 2) = pack_bf16(acc.z, acc.w);
        }
    }
}

// out[n, h * out_head + j] = sum_i w[h][j][i] * in[n, h * in_head + i]; `tail` more elements of a head's input are
// copied behind its outputs. A block: 64 tokens x 128 outputs of one head, the inputs walked in pieces of 32.
constexpr int PM = 64, PN = 128, PK = 32, PRB = PK * 2 + 16;
__global__ void __launch_bounds__(128)
per_head_mma_kernel(const __nv_bfloat16* __restrict__ in, int in_stride, int in_head, const __nv_bfloat16* __restrict__ w,
                    __nv_bfloat16* __restrict__ out, int out_stride, int out_head, int n, int I, int J, int tail) {
    __shared__ __align__(128) uint8_t sA[2][PM * PRB];
    __shared__ __align__(128) uint8_t sB[2][PN * PRB];
    dd_launch_dependents();
    dd_grid_wait();
    const int t0 = blockIdx.x * PM, h = blockIdx.y, j0 = blockIdx.z * PN;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3, mi = lane >> 3;
    const __nv_bfloat16* wh = w + (size_t)h * J * I;
    auto load = [&](int k0, int buf) {
        for (int idx = tid; idx < (PM + PN) * (PK / 8); idx += 128) {
            const int r = idx / (PK / 8), c = idx % (PK / 8);
            const int col = k0 + c * 8;
            if (r < PM) {
                uint8_t* dst = sA[buf] + r * PRB + c * 16;
                if (t0 + r < n && col < I) cp_async16(dst, in + (size_t)(t0 + r) * in_stride + (size_t)h * in_head + col);
                else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
            } else {
                uint8_t* dst = sB[buf] + (r - PM) * PRB + c * 16;
                if (j0 + r - PM < J && col < I) cp_async16(dst, wh + (size_t)(j0 + r - PM) * I + col);
                else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
            }
        }
    };
    float acc[PN / 8][4];
#pragma unroll
    for (int i = 0; i < PN / 8; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
    const int n_steps = (I + PK - 1) / PK;
    load(0, 0);
    cp_commit();
    for (int st = 0; st < n_steps; ++st) {
        const int buf = st & 1;
        if (st + 1 < n_steps) load((st + 1) * PK, buf ^ 1);
        cp_commit();
        cp_wait<1>();
        __syncthreads();
        const uint32_t ta = smem_addr(sA[buf] + (warp * 16 + (mi & 1) * 8 + (lane & 7)) * PRB + (mi >> 1) * 16);
        const uint32_t tb = smem_addr(sB[buf] + ((mi >> 1) * 8 + (lane & 7)) * PRB + (mi & 1) * 16);
#pragma unroll
        for (int ks = 0; ks < PK / 16; ++ks) {
            uint32_t a[4];
            ldmatrix_x4(ta + ks * 32, a);
#pragma unroll
            for (int np = 0; np < PN / 16; ++np) {
                uint32_t b[4];
                ldmatrix_x4(tb + np * 16 * PRB + ks * 32, b);
                mma_bf16(acc[2 * np], a, b[0], b[1]);
                mma_bf16(acc[2 * np + 1], a, b[2], b[3]);
            }
        }
        __syncthreads();
    }
    cp_wait<0>();
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int t = t0 + warp * 16 + g + 8 * r;
        if (t >= n) continue;
        __nv_bfloat16* dst = out + (size_t)t * out_stride + (size_t)h * out_head;
#pragma unroll
        for (int i = 0; i < PN / 8; ++i) {
            const int j = j0 + i * 8 + 2 * t4;
            if (j + 1 < J) *reinterpret_cast<uint32_t*>(dst + j) = pack_bf16(acc[i][2 * r], acc[i][2 * r + 1]);
            else if (j < J) dst[j] = __float2bfloat16(acc[i][2 * r]);
        }
    }
    if (tail > 0 && blockIdx.z == 0)
        for (int idx = tid; idx < PM * tail; idx += 128) {
            const int t = t0 + idx / tail, c = idx % tail;
            if (t < n) out[(size_t)t * out_stride + (size_t)h * out_head + J + c] = in[(size_t)t * in_stride + (size_t)h * in_head + I + c];
        }
}

template <int VT, int RG>
int launch_latent(const void* q, int q_stride, const void* cache, const int* entry_start, const int* entry_pos0, int n_entries,
                  int n_tokens, const int* block_table, int max_blocks, void* out, int out_stride, float* part_o,
                  float* part_ml, int H, int DK, int DV, int P, int n_pages, float scale, int n_splits, int* error_flag,
                  const float* sink, cudaStream_t s) {
    constexpr int BQ = RG * 16;
    // two key buffers, unless only one lets two blocks share an SM: with a warp a scheduler the tensor pipe idles most
    // of the time (measured: 17% active), and a second block fills more of it than a block's own prefetch
    const int half_sm = 113 * 1024;
    const int n_bufs = (BQ + 2 * BKV) * (DK * 2 + 16) > half_sm && (BQ + BKV) * (DK * 2 + 16) <= half_sm ? 1 : 2;
    const int smem = (BQ + n_bufs * BKV) * (DK * 2 + 16);
    static int configured = 0;
    if (smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_latent_kernel<VT, RG>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return dd_fail("dd_attention_latent: shared memory refused: %s", cudaGetErrorString(e));
        configured = smem;
    }
    const int slices = dd_ceil_div(DV, VT * 16);
    // an upper bound of the number of tiles; blocks beyond the real count return at once
    dim3 grid(dd_ceil_div((long long)n_tokens * H, BQ) + n_entries, n_splits);
    dd_launch(attention_latent_kernel<VT, RG>, grid, dim3(32 * RG * slices), (size_t)smem, s, (const __nv_bfloat16*)q, q_stride,
              (const __nv_bfloat16*)cache, entry_start, entry_pos0, n_entries, block_table, max_blocks, (__nv_bfloat16*)out,
              out_stride, part_o, part_ml, H, DK, DV, P, n_pages, scale * 1.4426950408889634f, n_splits, error_flag, sink, n_bufs);
    return dd_check_launch("dd_attention_latent");
}
}  // namespace

// Rows of DK bfloat16 with the value in their first DV: DK and DV multiples of 16, DK at most 576 (a query tile and two
// key tiles fit a block's shared memory), DV at most 512.
DD_API int dd_attention_latent_supported(int dk, int dv, int dtype) {
    return dtype == DD_BF16 && dk > 0 && dv > 0 && dk % 16 == 0 && dv % 16 == 0 && dv <= dk && dk <= 576 && dv <= 512;
}

// The query rows of a tile: 32 where every entry is a single token of at most 32 heads, else 64.
DD_API int dd_attention_latent_tile(int n_tokens, int n_entries, int H) { return n_tokens == n_entries && H <= 32 ? 32 : 64; }

// q: [N, q_stride] rows of H * DK; cache: [n_pages, P * DK]; entries are runs of consecutive tokens of one request
// (entry_start [E+1], entry_pos0 [E], block_table row e). out: [N, out_stride] rows of H * DV. part_o
// [N * H * n_splits * DV] and part_ml [N * H * n_splits * 2] only with n_splits > 1. Error bit 2: a key without a page.
DD_API int dd_attention_latent(const void* q, int q_stride, const void* cache, const int* entry_start, const int* entry_pos0,
                               int n_entries, int n_tokens, const int* block_table, int max_blocks, void* out, int out_stride,
                               float* part_o, float* part_ml, int H, int DK, int DV, int P, int n_pages, float scale,
                               int n_splits, int* error_flag, const float* sink, void* stream) {
    if (n_tokens <= 0 || n_entries <= 0) return 0;
    if (!dd_attention_latent_supported(DK, DV, DD_BF16))
        return dd_fail("dd_attention_latent: rows of %d with values of %d are not supported", DK, DV);
    if (q_stride % 8 || out_stride % 2 || ((uintptr_t)q & 15) || ((uintptr_t)cache & 15) || ((uintptr_t)out & 3))
        return dd_fail("dd_attention_latent: rows must be 16-byte aligned");
    if (n_splits < 1 || n_splits > 32 || (n_splits > 1 && (!part_o || !part_ml))) return dd_fail("dd_attention_latent: bad splits");
    cudaStream_t s = (cudaStream_t)stream;
    int rc;
#define DD_LATENT(VT, RG) launch_latent<VT, RG>(q, q_stride, cache, entry_start, entry_pos0, n_entries, n_tokens, block_table, max_blocks, \
                                        out, out_stride, part_o, part_ml, H, DK, DV, P, n_pages, scale, n_splits, error_flag, sink, s)
    if (dd_attention_latent_tile(n_tokens, n_entries, H) == 32) {
        // single tokens: more warps with fewer value columns each (both slices of a row compute its scores)
        if (DV <= 64) rc = DD_LATENT(4, 2);
        else rc = DD_LATENT(8, 2);
    } else if (DV <= 64) rc = DD_LATENT(4, 4);
    else if (DV <= 128) rc = DD_LATENT(8, 4);
    else rc = DD_LATENT(16, 4);
#undef DD_LATENT
    if (rc || n_splits == 1) return rc;
    dd_launch(attention_latent_merge_kernel, dim3(dd_ceil_div((long long)n_tokens * H, 4)), dim3(128), 0, s, (const float*)part_o,
              (const float*)part_ml, (__nv_bfloat16*)out, out_stride, n_tokens, H, DV, n_splits, sink);
    return dd_check_launch("dd_attention_latent (merge)");
}

DD_API int dd_per_head_mma_supported(int in_stride, int in_head, int out_stride, int out_head, int I, int dtype) {
    return dtype == DD_BF16 && I > 0 && I % 8 == 0 && in_stride % 8 == 0 && in_head % 8 == 0 && out_stride % 2 == 0 && out_head % 2 == 0;
}

DD_API int dd_per_head_mma(const void* in, int in_stride, int in_head, const void* w, void* out, int out_stride, int out_head,
                           int n, int heads, int I, int J, int tail, void* stream) {
    if (n <= 0 || heads <= 0) return 0;
    if (J <= 0 || tail < 0 || heads > 65535 || !dd_per_head_mma_supported(in_stride, in_head, out_stride, out_head, I, DD_BF16))
        return dd_fail("dd_per_head_mma: sizes are not supported");
    if (((uintptr_t)in & 15) || ((uintptr_t)w & 15) || ((uintptr_t)out & 3)) return dd_fail("dd_per_head_mma: rows must be 16-byte aligned");
    dd_launch(per_head_mma_kernel, dim3(dd_ceil_div(n, PM), heads, dd_ceil_div(J, PN)), dim3(128), 0, (cudaStream_t)stream,
              (const __nv_bfloat16*)in, in_stride, in_head, (const __nv_bfloat16*)w, (__nv_bfloat16*)out, out_stride, out_head,
              n, I, J, tail);
    return dd_check_launch("dd_per_head_mma");
}
