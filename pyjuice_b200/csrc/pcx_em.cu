// Mini-batch EM update kernels: tied-flow accumulation, sum-parameter normalise-and-blend, and the
// categorical-leaf update.  All three stream parameters and flows once or twice and are bound by HBM
// bandwidth; threads are laid out along the contiguous dimension of each table (the node index for
// sum parameters, the category index for leaves).
#include "pcx_common.cuh"
#include "../../include/pcx_b200.h"

namespace {

constexpr int NT = 256;

__global__ void tied_accum_kernel(float* __restrict__ flows, int64_t start, int64_t n,
                                  const int64_t* __restrict__ ch_starts, int n_chs) {
    int64_t j = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= n) return;
    float s = 0.0f;
    for (int c = 0; c < n_chs; ++c) s += __ldcs(flows + ch_starts[c] + j);        // all loads first: they overlap
    for (int c = 0; c < n_chs; ++c)                       // moved into the source: running the fold again adds nothing
        if (ch_starts[c] != start) __stcs(flows + ch_starts[c] + j, 0.0f);
    flows[start + j] = s;     // `start` is one of ch_starts: each thread reads its own slot before writing it
}

// One CTA per (node block, tile of MT nodes).  Thread (tx, ty): node m = tx, edges e = ty, ty+EL, ...
// so that a warp reads MT consecutive floats of one edge (the node index is the fastest-varying one).
template <int MT>
__global__ void __launch_bounds__(NT)
em_sum_kernel(float* __restrict__ params, const float* __restrict__ flows,
              const int64_t* __restrict__ blk_par, const int64_t* __restrict__ blk_flow,
              const int32_t* __restrict__ blk_fan, const int32_t* __restrict__ blk_bs,
              int tiles_per_block, float step, float pseudo, int keep_zero) {
    constexpr int EL = NT / MT;
    __shared__ float s_red[EL][MT];
    const int64_t i = blockIdx.x / tiles_per_block;
    const int mt = (int)(blockIdx.x % tiles_per_block);
    const int bs = blk_bs[i];
    const int m = mt * MT + (threadIdx.x % MT);
    const int ty = threadIdx.x / MT;
    const int fan = blk_fan[i];
    const bool live = m < bs;
    const float* f = flows + blk_flow[i] + m;
    float* p = params + blk_par[i] + m;
    const float add = pseudo / (float)fan;

    // eight edges per round: their loads are independent, so a thread has eight (sixteen) in flight instead of one
    constexpr int U = 8;
    float tot = 0.0f;
    if (live) {
        for (int e0 = ty; e0 < fan; e0 += EL * U) {
            float fl[U], pv[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int e = e0 + u * EL;
                fl[u] = (e < fan) ? f[(int64_t)e * bs] : 0.0f;
                pv[u] = (keep_zero && e < fan) ? p[(int64_t)e * bs] : 1.0f;
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int e = e0 + u * EL;
                if (e >= fan) continue;
                if (keep_zero) tot += (pv[u] < 1e-12f) ? 0.0f : fl[u] + add;
                else tot += fl[u];
            }
        }
    }
    s_red[ty][threadIdx.x % MT] = tot;
    __syncthreads();
    for (int s = EL / 2; s > 0; s >>= 1) {
        if (ty < s) s_red[ty][threadIdx.x % MT] += s_red[ty + s][threadIdx.x % MT];
        __syncthreads();
    }
    if (!live) return;
    const float denom = keep_zero ? s_red[0][threadIdx.x % MT] : s_red[0][threadIdx.x % MT] + pseudo;
    for (int e0 = ty; e0 < fan; e0 += EL * U) {
        float fl[U], old[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int e = e0 + u * EL;
            fl[u] = (e < fan) ? f[(int64_t)e * bs] : 0.0f;
            old[u] = (e < fan) ? p[(int64_t)e * bs] : 0.0f;
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int e = e0 + u * EL;
            if (e >= fan) continue;
            const float nw = (fl[u] + add) / denom;
            float upd = (1.0f - step) * old[u] + step * nw;
            if (keep_zero && old[u] < 1e-12f) upd = 0.0f;
            p[(int64_t)e * bs] = upd;
        }
    }
}

// One group of G threads per source node; the group strides over the node's categories.
template <int G>
__global__ void __launch_bounds__(NT)
em_input_cat_kernel(float* __restrict__ params, const float* __restrict__ flows,
                    const int32_t* __restrict__ source_nids, const int32_t* __restrict__ s_pids,
                    const int32_t* __restrict__ s_pfids, const int32_t* __restrict__ node_cats,
                    int64_t n_source, float step, float pseudo, int keep_zero) {
    constexpr int GROUPS = NT / G;
    __shared__ float s_red[NT / 32];
    const int g = threadIdx.x / G, l = threadIdx.x % G;
    const int64_t sidx = (int64_t)blockIdx.x * GROUPS + g;
    const bool live = sidx < n_source;
    int64_t poff = 0, foff = 0;
    int num_cats = 1;
    if (live) {
        int n = source_nids[sidx];
        poff = s_pids[n];
        foff = s_pfids[n];
        num_cats = node_cats[n];
    }
    const float add = pseudo / (float)num_cats;
    float tot = 0.0f;
    if (live) {
        for (int c = l; c < num_cats; c += G) {
            float fl = flows[foff + c];
            if (keep_zero) tot += (params[poff + c] < 1e-12f) ? 0.0f : fl + add;
            else tot += fl;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) tot += __shfl_xor_sync(0xffffffffu, tot, o);
    if (G > 32) {                       // G == NT: one node per CTA, combine the warps
        if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = tot;
        __syncthreads();
        tot = 0.0f;
#pragma unroll
        for (int q = 0; q < NT / 32; ++q) tot += s_red[q];
    }
    if (!live) return;
    const float denom = keep_zero ? tot : tot + pseudo;
    for (int c = l; c < num_cats; c += G) {
        float old = params[poff + c];
        float upd = (1.0f - step) * old + step * (flows[foff + c] + add) / denom;
        if (keep_zero && old < 1e-12f) upd = 0.0f;
        params[poff + c] = upd;
    }
}

// Categorical EM on the transposed shadow of a large table (`flows_t`, `logp_t`: [category, row]; `params`: [row,
// category]; every row is a source vector with C categories).  Two kernels replace three passes over the table (move
// the flows into the [row, category] accumulators, update, rebuild the transposed log-parameter table): the first sums
// every row's flows over the categories, the second works on tiles of 128 rows x 128 categories — 512 contiguous bytes
// per row of either layout, which is what DRAM wants — with the parameter tile going through shared memory, so that
// both layouts are read and written with full-width coalesced accesses.  The flows are left as they are (the caller
// clears or moves them later).  (Tiles of 32 x 32, one CTA per 32 rows, ran at 3.1 TB/s: 128-byte runs strided by
// 16 KB and 128 KB.)
constexpr int EMT = 128;                                 // tile edge
constexpr int EMT_LD = EMT + 1;                          // row pitch of the shared tile: odd, see emt_update_kernel

// part[share, r] = sum over this CTA's categories of flows_t[c, r].  Grid (ceil(R / 128), shares of the categories).
// (No atomics: the row totals are added up in a fixed order, so that data-parallel ranks, which hold bit-identical
// flows after the all-reduce, stay bit-identical after the update.)
constexpr int EMT_MAX_SHARES = 16;
__global__ void __launch_bounds__(256) emt_totals_kernel(float* __restrict__ totals, const float* __restrict__ flows_t,
                                                          int64_t R, int C) {
    __shared__ float s_tot[8][EMT];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t r = (int64_t)blockIdx.x * EMT + 4 * lane;          // four consecutive rows per lane
    const bool vec = (R % 4 == 0) && r + 3 < R;
    float t[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    for (int c0 = (blockIdx.y * 8 + warp) * 8; c0 < C; c0 += gridDim.y * 64) {
        float4 v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int c = c0 + u;
            v[u] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (c < C) {
                const float* src = flows_t + (int64_t)c * R + r;
                if (vec) v[u] = *reinterpret_cast<const float4*>(src);
                else {
                    if (r < R) v[u].x = src[0];
                    if (r + 1 < R) v[u].y = src[1];
                    if (r + 2 < R) v[u].z = src[2];
                    if (r + 3 < R) v[u].w = src[3];
                }
            }
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) { t[0] += v[u].x; t[1] += v[u].y; t[2] += v[u].z; t[3] += v[u].w; }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) s_tot[warp][4 * lane + i] = t[i];
    __syncthreads();
    if (threadIdx.x < EMT) {
        float sum = 0.0f;
#pragma unroll
        for (int w = 0; w < 8; ++w) sum += s_tot[w][threadIdx.x];
        const int64_t rr = (int64_t)blockIdx.x * EMT + threadIdx.x;
        if (rr < R) totals[(int64_t)blockIdx.y * R + rr] = sum;
    }
}

// One tile of 128 rows x 128 categories per CTA (256 threads).  Lane l owns rows l, l + 32, l + 64, l + 96 on the
// transposed side and categories l, l + 32, ... on the parameter side: every global access of a warp is 128 contiguous
// bytes (four of them make up the 512-byte run of the tile), and with a row pitch of 129 floats neither side has a
// shared-memory bank conflict.
__global__ void __launch_bounds__(256) emt_update_kernel(float* __restrict__ params, float* __restrict__ logp_t,
                                                          const float* __restrict__ flows_t, const float* __restrict__ totals,
                                                          int shares, int64_t R, int C, float step, float pseudo) {
    extern __shared__ float s_p[];                       // [128 rows][EMT_LD]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t r0 = (int64_t)blockIdx.x * EMT;
    const int c0 = blockIdx.y * EMT;
    const float add = pseudo / (float)C;
    // parameter tile in: warp -> rows warp, warp + 8, ...
    for (int rr = warp; rr < EMT; rr += 8) {
        const int64_t r = r0 + rr;
        float v[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int c = c0 + lane + 32 * j;
            v[j] = (r < R && c < C) ? params[r * C + c] : 0.0f;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) s_p[rr * EMT_LD + lane + 32 * j] = v[j];
    }
    float inv[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int64_t r = r0 + lane + 32 * i;
        float tot = 0.0f;
        if (r < R)
            for (int sh = 0; sh < shares; ++sh) tot += totals[(int64_t)sh * R + r];
        inv[i] = (r < R) ? 1.0f / (tot + pseudo) : 0.0f;
    }
    __syncthreads();
    // transposed side: warp -> categories warp, warp + 8, ...; two categories per round (eight loads in flight)
    for (int cc0 = warp; cc0 < EMT; cc0 += 16) {
        float f[2][4];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int c = c0 + cc0 + 8 * u;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int64_t r = r0 + lane + 32 * i;
                f[u][i] = (c < C && r < R) ? flows_t[(int64_t)c * R + r] : 0.0f;
            }
        }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int cc = cc0 + 8 * u;
            const int c = c0 + cc;
            if (c >= C) continue;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int64_t r = r0 + lane + 32 * i;
                float* cell = s_p + (lane + 32 * i) * EMT_LD + cc;
                const float upd = (1.0f - step) * (*cell) + step * (f[u][i] + add) * inv[i];
                *cell = upd;
                if (r < R) logp_t[(int64_t)c * R + r] = logf(upd);
            }
        }
    }
    __syncthreads();
    // parameter tile out
    for (int rr = warp; rr < EMT; rr += 8) {
        const int64_t r = r0 + rr;
        if (r >= R) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int c = c0 + lane + 32 * j;
            if (c < C) params[r * C + c] = s_p[rr * EMT_LD + lane + 32 * j];
        }
    }
}

// Flow of a leaf whose variable is not observed: its (linear) flow f spreads over the categories in proportion to the
// parameters, flows[s_pfids + c] += scale * f * params[s_pids + c].  One CTA per source node.
__global__ void __launch_bounds__(NT)
input_cat_missing_kernel(float* __restrict__ flows, const float* __restrict__ params,
                         const float* __restrict__ source_flow, const int32_t* __restrict__ source_nids,
                         const int32_t* __restrict__ s_pids, const int32_t* __restrict__ s_pfids,
                         const int32_t* __restrict__ node_cats, float scale) {
    const int64_t sidx = blockIdx.x;
    const float f = scale * source_flow[sidx];
    if (f == 0.0f) return;
    const int n = source_nids[sidx];
    const float* p = params + (int64_t)s_pids[n];
    float* out = flows + (int64_t)s_pfids[n];
    const int num_cats = node_cats[n];
    for (int c = threadIdx.x; c < num_cats; c += NT) out[c] += f * p[c];      // one writer per (source node, category)
}

}  // namespace

extern "C" {

int pcx_input_cat_missing(float* param_flows, const float* params, const float* source_flow,
                          const int32_t* source_nids, const int32_t* s_pids, const int32_t* s_pfids,
                          const int32_t* node_cats, int64_t n_source, float scale, void* stream) {
    if (n_source <= 0) return 0;
    input_cat_missing_kernel<<<(unsigned)n_source, NT, 0, (cudaStream_t)stream>>>(param_flows, params, source_flow,
                                                                                 source_nids, s_pids, s_pfids, node_cats, scale);
    PCX_LAUNCH_CHECK();
    return 0;
}

int pcx_tied_accum(float* flows, int64_t start, int64_t n, const int64_t* ch_starts, int n_chs, void* stream) {
    if (n <= 0 || n_chs <= 0) return 0;
    tied_accum_kernel<<<(unsigned)pcx_cdiv(n, NT), NT, 0, (cudaStream_t)stream>>>(flows, start, n, ch_starts, n_chs);
    PCX_LAUNCH_CHECK();
    return 0;
}

int pcx_em_sum(float* params, const float* param_flows, const int64_t* blk_par, const int64_t* blk_flow,
               const int32_t* blk_fan, const int32_t* blk_bs, int64_t n_blocks, int max_bs,
               float step, float pseudo, int keep_zero, void* stream) {
    if (n_blocks <= 0) return 0;
    if (max_bs <= 0) return -1;
    cudaStream_t st = (cudaStream_t)stream;
    if (max_bs >= 32) {
        int tiles = (int)pcx_cdiv(max_bs, 32);
        em_sum_kernel<32><<<(unsigned)(n_blocks * tiles), NT, 0, st>>>(params, param_flows, blk_par, blk_flow, blk_fan, blk_bs, tiles, step, pseudo, keep_zero);
    } else if (max_bs >= 8) {
        int tiles = (int)pcx_cdiv(max_bs, 8);
        em_sum_kernel<8><<<(unsigned)(n_blocks * tiles), NT, 0, st>>>(params, param_flows, blk_par, blk_flow, blk_fan, blk_bs, tiles, step, pseudo, keep_zero);
    } else {
        int tiles = max_bs;
        em_sum_kernel<1><<<(unsigned)(n_blocks * tiles), NT, 0, st>>>(params, param_flows, blk_par, blk_flow, blk_fan, blk_bs, tiles, step, pseudo, keep_zero);
    }
    PCX_LAUNCH_CHECK();
    return 0;
}

int pcx_em_input_cat(float* params, const float* param_flows, const int32_t* source_nids,
                     const int32_t* s_pids, const int32_t* s_pfids, const int32_t* node_cats,
                     int64_t n_source, int max_cats, float step, float pseudo, int keep_zero, void* stream) {
    if (n_source <= 0 || max_cats <= 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    if (max_cats > 1024) {
        em_input_cat_kernel<NT><<<(unsigned)n_source, NT, 0, st>>>(params, param_flows, source_nids, s_pids, s_pfids, node_cats, n_source, step, pseudo, keep_zero);
    } else {
        em_input_cat_kernel<32><<<(unsigned)pcx_cdiv(n_source, NT / 32), NT, 0, st>>>(params, param_flows, source_nids, s_pids, s_pfids, node_cats, n_source, step, pseudo, keep_zero);
    }
    PCX_LAUNCH_CHECK();
    return 0;
}

int pcx_em_input_cat_t(float* params, float* logp_t, const float* flows_t, float* totals, int64_t n_rows, int num_cats,
                       float step, float pseudo, void* stream) {
    if (n_rows <= 0 || num_cats <= 0) return 0;
    if (totals == nullptr || (reinterpret_cast<uintptr_t>(flows_t) & 15) != 0) return -1;
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e;
    const int64_t row_tiles = pcx_cdiv(n_rows, EMT);
    int64_t shares = pcx_cdiv(8 * 148, row_tiles);                  // about eight CTAs of 256 threads per SM
    const int64_t max_shares = pcx_cdiv(num_cats, 64);
    if (shares > max_shares) shares = max_shares;
    if (shares > EMT_MAX_SHARES) shares = EMT_MAX_SHARES;
    if (shares < 1) shares = 1;
    emt_totals_kernel<<<dim3((unsigned)row_tiles, (unsigned)shares), 256, 0, st>>>(totals, flows_t, n_rows, num_cats);
    const int smem = EMT * EMT_LD * (int)sizeof(float);
    static PcxOnce done;
    if (!done) {
        e = cudaFuncSetAttribute(emt_update_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
        done = true;
    }
    emt_update_kernel<<<dim3((unsigned)row_tiles, (unsigned)pcx_cdiv(num_cats, EMT)), 256, smem, st>>>(
        params, logp_t, flows_t, totals, (int)shares, n_rows, num_cats, step, pseudo);
    PCX_LAUNCH_CHECK();
    return 0;
}

}  // extern "C"
