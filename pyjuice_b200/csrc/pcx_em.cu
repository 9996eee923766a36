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
// category]; every row is a source vector with C categories).  One kernel replaces three passes over the table (move
// the flows into the [row, category] accumulators, update, rebuild the transposed log-parameter table): a CTA owns 32
// rows; its warps stride over blocks of 32 categories, first for the rows' flow totals, then for the update, in which
// the parameter tile goes through a per-warp shared-memory transpose so that both layouts are read and written with
// coalesced accesses.  The flows are left as they are (the caller clears or moves them later).  (A two-kernel version
// with a four times larger grid -- totals first, then the update -- was measured and was no faster.)
constexpr int EMT_WARPS = 16;
__global__ void __launch_bounds__(EMT_WARPS * 32)
em_input_cat_t_kernel(float* __restrict__ params, float* __restrict__ logp_t, const float* __restrict__ flows_t,
                      int64_t R, int C, float step, float pseudo) {
    extern __shared__ float s_emt[];                     // [EMT_WARPS][32][33] transpose tiles, one per warp
    __shared__ float s_tot[EMT_WARPS][32];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t r0 = (int64_t)blockIdx.x * 32;
    const int64_t r = r0 + lane;
    const bool r_ok = r < R;
    const float add = pseudo / (float)C;

    float tot = 0.0f;
    for (int c0 = warp * 32; c0 < C; c0 += EMT_WARPS * 32) {
        float f[32];
#pragma unroll
        for (int cc = 0; cc < 32; ++cc) f[cc] = (r_ok && c0 + cc < C) ? flows_t[(int64_t)(c0 + cc) * R + r] : 0.0f;
#pragma unroll
        for (int cc = 0; cc < 32; ++cc) tot += f[cc];
    }
    s_tot[warp][lane] = tot;
    __syncthreads();
    tot = 0.0f;
#pragma unroll
    for (int w = 0; w < EMT_WARPS; ++w) tot += s_tot[w][lane];
    const float denom = tot + pseudo;

    float (*tile)[33] = reinterpret_cast<float (*)[33]>(s_emt + warp * 32 * 33);
    for (int c0 = warp * 32; c0 < C; c0 += EMT_WARPS * 32) {
        float f[32];
#pragma unroll
        for (int cc = 0; cc < 32; ++cc) f[cc] = (r_ok && c0 + cc < C) ? flows_t[(int64_t)(c0 + cc) * R + r] : 0.0f;
        const int c = c0 + lane;
#pragma unroll 8
        for (int rr = 0; rr < 32; ++rr) tile[rr][lane] = (r0 + rr < R && c < C) ? params[(r0 + rr) * C + c] : 0.0f;
        __syncwarp();
#pragma unroll
        for (int cc = 0; cc < 32; ++cc) {
            const float upd = (1.0f - step) * tile[lane][cc] + step * (f[cc] + add) / denom;
            tile[lane][cc] = upd;
            if (r_ok && c0 + cc < C) logp_t[(int64_t)(c0 + cc) * R + r] = logf(upd);
        }
        __syncwarp();
#pragma unroll 8
        for (int rr = 0; rr < 32; ++rr)
            if (r0 + rr < R && c < C) params[(r0 + rr) * C + c] = tile[rr][lane];
        __syncwarp();
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

int pcx_em_input_cat_t(float* params, float* logp_t, const float* flows_t, int64_t n_rows, int num_cats, float step,
                       float pseudo, void* stream) {
    if (n_rows <= 0 || num_cats <= 0) return 0;
    const int smem = EMT_WARPS * 32 * 33 * (int)sizeof(float);
    static PcxOnce done;
    if (!done) {
        cudaError_t e = cudaFuncSetAttribute(em_input_cat_t_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
        done = true;
    }
    em_input_cat_t_kernel<<<(unsigned)pcx_cdiv(n_rows, 32), EMT_WARPS * 32, smem, (cudaStream_t)stream>>>(
        params, logp_t, flows_t, n_rows, num_cats, step, pseudo);
    PCX_LAUNCH_CHECK();
    return 0;
}

}  // extern "C"
