// Bandwidth-bound kernels of the circuit path: buffer fills, categorical leaves (forward gather and
// flow scatter) and product layers (gather-add forward, logaddexp-accumulate backward).
//
// Layout: every value buffer is [rows, B] fp32 with the batch innermost, so a warp that walks the
// batch dimension reads and writes whole 128-byte lines.  Product rows are handled four samples per
// thread (float4) whenever B is a multiple of 4.
#include <algorithm>
#include "pcx_common.cuh"
#include "../../include/pcx_b200.h"

namespace {

constexpr int kThreads = 256;

__global__ void fill_kernel(float* __restrict__ p, int64_t n, float v) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    int64_t n4 = n >> 2;
    float4 v4 = make_float4(v, v, v, v);
    if ((reinterpret_cast<uintptr_t>(p) & 15) == 0) {
        for (int64_t k = i; k < n4; k += stride) reinterpret_cast<float4*>(p)[k] = v4;
        for (int64_t k = (n4 << 2) + i; k < n; k += stride) p[k] = v;
    } else {
        for (int64_t k = i; k < n; k += stride) p[k] = v;
    }
}

__global__ void scale_kernel(float* __restrict__ p, int64_t n, float v) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t k = i; k < n; k += stride) p[k] *= v;
}

__global__ void exp_kernel(float* __restrict__ p, int64_t n) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t k = i; k < n; k += stride) p[k] = expf(p[k]);
}

__global__ void root_flows_kernel(float* __restrict__ node_flows, const float* __restrict__ weights,
                                  int64_t root_start, int64_t n, int logspace) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float w = weights ? weights[i] : 1.0f;
    node_flows[root_start + i] = logspace ? logf(w) : w;              // root rows are contiguous: [num_roots, B]
}

// Categorical leaves, general form: one CTA per node, threads walk the batch.  Used when the batch is not a multiple
// of four or a node has too many categories to stage its table in shared memory.  A category id outside the node's
// table (invalid data) must not address outside it: the forward kernel clamps it, the backward kernel adds no flow.
__global__ void input_cat_fwd_kernel(float* __restrict__ node_mars, const float* __restrict__ params,
                                     const void* __restrict__ data, int elsize,
                                     const int32_t* __restrict__ vids, const int32_t* __restrict__ s_pids,
                                     const int32_t* __restrict__ node_cats, int max_cats,
                                     int64_t n_nodes, int64_t node_off, int B) {
    const int64_t n = blockIdx.x;
    const int64_t drow = (int64_t)vids[n] * B;
    const float* prow = params + (int64_t)s_pids[n];
    const int cap = (node_cats ? node_cats[n] : max_cats) - 1;
    float* out = node_mars + (node_off + n) * B;
    for (int b = threadIdx.x; b < B; b += blockDim.x)
        out[b] = logf(prow[min(max(pcx_load_cat(data, elsize, drow + b), 0), cap)]);
}

__global__ void input_cat_bwd_kernel(float* __restrict__ param_flows, const float* __restrict__ node_flows,
                                     const void* __restrict__ data, int elsize,
                                     const int32_t* __restrict__ vids, const int32_t* __restrict__ s_pfids,
                                     const int32_t* __restrict__ node_cats, int max_cats,
                                     int64_t n_nodes, int64_t node_off, int B, int logspace) {
    const int64_t n = blockIdx.x;
    const int64_t drow = (int64_t)vids[n] * B;
    float* frow = param_flows + (int64_t)s_pfids[n];
    const int nc = node_cats ? node_cats[n] : max_cats;
    const float* in = node_flows + (node_off + n) * B;
    for (int b = threadIdx.x; b < B; b += blockDim.x) {
        float f = in[b];
        f = logspace ? expf(f) : f;
        const int c = pcx_load_cat(data, elsize, drow + b);
        if (f != 0.0f && c >= 0 && c < nc) atomicAdd(frow + c, f);
    }
}

// Categorical leaves with the tables of G consecutive nodes staged in shared memory.
//
// A CTA owns G nodes.  Forward: it loads their parameter rows with coalesced reads, takes the logarithm once per
// parameter (not once per sample) and then every thread looks up four consecutive samples per node and writes one
// float4.  Nodes of one variable are consecutive in a layer, so the four category ids are re-read only when the
// variable changes.  Backward: the CTA builds the histograms of its G nodes over the whole batch with shared-memory
// atomics and adds every non-zero bin to the flow accumulators once -- G * num_cats global atomics instead of
// G * B.  Category ids are clamped to the staged table so that invalid data cannot address outside it.
constexpr int kStageThreads = 128;

__device__ __forceinline__ void load_cats4(const void* data, int elsize, int64_t idx, int cap, int* c) {
#pragma unroll
    for (int k = 0; k < 4; ++k) c[k] = min(max(pcx_load_cat(data, elsize, idx + k), 0), cap);
}

__global__ void __launch_bounds__(kStageThreads)
input_cat_fwd_staged(float* __restrict__ node_mars, const float* __restrict__ params,
                     const void* __restrict__ data, int elsize,
                     const int32_t* __restrict__ vids, const int32_t* __restrict__ s_pids,
                     const int32_t* __restrict__ node_cats, int max_cats, int G,
                     int64_t n_nodes, int64_t node_off, int B) {
    extern __shared__ float s_tab[];                       // [G][max_cats] log-parameters
    const int64_t n0 = (int64_t)blockIdx.x * G;
    const int g_end = (int)min((int64_t)G, n_nodes - n0);
    for (int g = 0; g < g_end; ++g) {
        const float* prow = params + (int64_t)s_pids[n0 + g];
        const int nc = min(node_cats[n0 + g], max_cats);
        for (int c = threadIdx.x; c < nc; c += kStageThreads) s_tab[g * max_cats + c] = logf(prow[c]);
        for (int c = nc + threadIdx.x; c < max_cats; c += kStageThreads) s_tab[g * max_cats + c] = PCX_NEG_INF;
    }
    __syncthreads();
    for (int b = (blockIdx.y * kStageThreads + threadIdx.x) * 4; b < B; b += gridDim.y * kStageThreads * 4) {
        int cur = -1, c[4];
        for (int g = 0; g < g_end; ++g) {
            const int v = vids[n0 + g];
            if (v != cur) { load_cats4(data, elsize, (int64_t)v * B + b, max_cats - 1, c); cur = v; }
            const float* t = s_tab + g * max_cats;
            *reinterpret_cast<float4*>(node_mars + (node_off + n0 + g) * B + b) = make_float4(t[c[0]], t[c[1]], t[c[2]], t[c[3]]);
        }
    }
}

__global__ void __launch_bounds__(kStageThreads)
input_cat_bwd_staged(float* __restrict__ param_flows, const float* __restrict__ node_flows,
                     const void* __restrict__ data, int elsize,
                     const int32_t* __restrict__ vids, const int32_t* __restrict__ s_pfids,
                     const int32_t* __restrict__ node_cats, int max_cats, int G,
                     int64_t n_nodes, int64_t node_off, int B, int logspace) {
    extern __shared__ float s_tab[];                       // [G][max_cats] flow histograms
    const int64_t n0 = (int64_t)blockIdx.x * G;
    const int g_end = (int)min((int64_t)G, n_nodes - n0);
    for (int k = threadIdx.x; k < G * max_cats; k += kStageThreads) s_tab[k] = 0.0f;
    __syncthreads();
    for (int b = threadIdx.x * 4; b < B; b += kStageThreads * 4) {
        int cur = -1, c[4];
        for (int g = 0; g < g_end; ++g) {
            const int v = vids[n0 + g];
            if (v != cur) { load_cats4(data, elsize, (int64_t)v * B + b, max_cats - 1, c); cur = v; }
            const float4 q = *reinterpret_cast<const float4*>(node_flows + (node_off + n0 + g) * B + b);
            float f[4] = {q.x, q.y, q.z, q.w};
            float* t = s_tab + g * max_cats;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float x = logspace ? expf(f[k]) : f[k];
                if (x != 0.0f) atomicAdd(t + c[k], x);
            }
        }
    }
    __syncthreads();
    for (int g = 0; g < g_end; ++g) {
        float* frow = param_flows + (int64_t)s_pfids[n0 + g];
        const int nc = min(node_cats[n0 + g], max_cats);
        for (int c = threadIdx.x; c < nc; c += kStageThreads) {
            const float x = s_tab[g * max_cats + c];
            if (x != 0.0f) atomicAdd(frow + c, x);
        }
    }
}

// ---- Categorical leaves with tables too large to stage (tens of thousands of categories) ---------------------------
// The parameter table is [row, category] (a row = the distribution of one source node).  Nodes of one variable are
// consecutive rows, so a lookup of category c for 128 consecutive nodes touches 128 different rows: one 32-byte
// sector per useful float.  These kernels work on a TRANSPOSED shadow instead: logp_T[category, row] (the logarithm is
// taken once per update) and flows_T[category, row], in which the same lookup is 512 contiguous bytes.
//   forward   tile of 128 nodes x 64 samples: per sample a coalesced read of the shadow, staged in shared memory,
//             written out as whole 256-byte pieces of the nodes' rows
//   backward  the same tile read coalesced, then per sample one coalesced reduction into flows_T
//   flush     param_flows[row_pfid[row] + c] += flows_T[c, row]; flows_T = 0   (tiled transpose)
// Flows of tied replicas all land in the source node's row of flows_T, so nothing is left to fold afterwards.
constexpr int kTN = 128, kTS = 64;

__global__ void __launch_bounds__(256)
input_cat_shadow_kernel(float* __restrict__ logp_t, const float* __restrict__ params, int64_t R, int C) {
    __shared__ float tile[32][33];
    const int64_t r0 = (int64_t)blockIdx.x * 32;
    const int c0 = blockIdx.y * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    for (int k = ty; k < 32; k += 8) {
        const int64_t r = r0 + k;
        const int c = c0 + tx;
        tile[k][tx] = (r < R && c < C) ? logf(params[r * C + c]) : 0.0f;
    }
    __syncthreads();
    for (int k = ty; k < 32; k += 8) {
        const int c = c0 + k;
        const int64_t r = r0 + tx;
        if (c < C && r < R) logp_t[(int64_t)c * R + r] = tile[tx][k];
    }
}

__global__ void __launch_bounds__(256)
input_cat_fwd_t_kernel(float* __restrict__ node_mars, const float* __restrict__ logp_t,
                       const void* __restrict__ data, int elsize, const int32_t* __restrict__ vids,
                       const int32_t* __restrict__ prow, int64_t R, int C, int64_t n_nodes, int64_t node_off, int B) {
    __shared__ float tile[kTN][kTS + 1];
    const int64_t n0 = (int64_t)blockIdx.x * kTN;
    const int b0 = blockIdx.y * kTS;
    const int nl = threadIdx.x & (kTN - 1), h = threadIdx.x >> 7;
    const int64_t n = n0 + nl;
    if (n < n_nodes) {
        const int64_t drow = (int64_t)vids[n] * B;
        const int64_t pr = prow[n];
#pragma unroll 8
        for (int s = h * (kTS / 2); s < (h + 1) * (kTS / 2); ++s) {
            const int b = b0 + s;
            float x = 0.0f;
            if (b < B) {
                const int c = min(max(pcx_load_cat(data, elsize, drow + b), 0), C - 1);
                x = logp_t[(int64_t)c * R + pr];
            }
            tile[nl][s] = x;
        }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < kTN * (kTS / 4); idx += 256) {       // B is a multiple of 4
        const int row = idx / (kTS / 4), f = (idx % (kTS / 4)) * 4;
        if (n0 + row < n_nodes && b0 + f < B)
            *reinterpret_cast<float4*>(node_mars + (node_off + n0 + row) * B + b0 + f) =
                make_float4(tile[row][f], tile[row][f + 1], tile[row][f + 2], tile[row][f + 3]);
    }
}

__global__ void __launch_bounds__(256)
input_cat_bwd_t_kernel(float* __restrict__ flows_t, const float* __restrict__ node_flows,
                       const void* __restrict__ data, int elsize, const int32_t* __restrict__ vids,
                       const int32_t* __restrict__ prow, int64_t R, int C, int64_t n_nodes, int64_t node_off, int B,
                       int logspace, int32_t* __restrict__ touched) {
    __shared__ float tile[kTN][kTS + 1];
    const int64_t n0 = (int64_t)blockIdx.x * kTN;
    const int b0 = blockIdx.y * kTS;
    for (int idx = threadIdx.x; idx < kTN * (kTS / 4); idx += 256) {
        const int row = idx / (kTS / 4), f = (idx % (kTS / 4)) * 4;
        float4 q = make_float4(0.f, 0.f, 0.f, 0.f);
        if (n0 + row < n_nodes && b0 + f < B) {
            q = *reinterpret_cast<const float4*>(node_flows + (node_off + n0 + row) * B + b0 + f);
            if (logspace) q = make_float4(__expf(q.x), __expf(q.y), __expf(q.z), __expf(q.w));
        }
        tile[row][f] = q.x; tile[row][f + 1] = q.y; tile[row][f + 2] = q.z; tile[row][f + 3] = q.w;
    }
    __syncthreads();
    const int nl = threadIdx.x & (kTN - 1), h = threadIdx.x >> 7;
    const int64_t n = n0 + nl;
    if (n >= n_nodes) return;
    const int64_t drow = (int64_t)vids[n] * B;
    const int64_t pr = prow[n];
#pragma unroll 4
    for (int s = h * (kTS / 2); s < (h + 1) * (kTS / 2); ++s) {
        const int b = b0 + s;
        if (b >= B) break;
        const float x = tile[nl][s];
        const int c = pcx_load_cat(data, elsize, drow + b);
        if (x != 0.0f && c >= 0 && c < C) {
            atomicAdd(flows_t + (int64_t)c * R + pr, x);
            if (touched[c] == 0) touched[c] = 1;                 // categories whose row of flows_t is not all zero
        }
    }
}

__global__ void __launch_bounds__(256)
input_cat_flush_t_kernel(float* __restrict__ param_flows, float* __restrict__ flows_t,
                         const int64_t* __restrict__ row_pfid, int64_t R, int C, const int32_t* __restrict__ touched) {
    __shared__ float tile[32][33];
    __shared__ int s_any;
    const int64_t r0 = (int64_t)blockIdx.x * 32;
    const int c0 = blockIdx.y * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    if (threadIdx.x == 0) s_any = 0;
    __syncthreads();
    if (threadIdx.x < 32 && c0 + threadIdx.x < C && touched[c0 + threadIdx.x] != 0) s_any = 1;
    __syncthreads();
    if (s_any == 0) return;                                  // no sample of the window carried these categories
    for (int k = ty; k < 32; k += 8) {
        const int c = c0 + k;
        const int64_t r = r0 + tx;
        float x = 0.0f;
        if (c < C && r < R) {
            x = flows_t[(int64_t)c * R + r];
            if (x != 0.0f) flows_t[(int64_t)c * R + r] = 0.0f;
        }
        tile[k][tx] = x;
    }
    __syncthreads();
    for (int k = ty; k < 32; k += 8) {
        const int64_t r = r0 + k;
        const int c = c0 + tx;
        if (r < R && c < C) {
            const float x = tile[tx][k];
            if (x != 0.0f) param_flows[row_pfid[r] + c] += x;
        }
    }
}

// Nodes per CTA of the staged kernels: up to 16, limited by 32 KB of shared memory; 0 = table too large to stage.
inline int stage_group(int max_cats) {
    if (max_cats <= 0) return 0;
    int g = (32 * 1024 / 4) / max_cats;
    return g > 16 ? 16 : g;
}

// Index arithmetic of the product kernels: thread t = (row r, vector column bc) with r = (block i, node j).  The
// divisors are launch constants and almost always powers of two, so the split is two shifts (or two 32-bit
// divisions); launches are cut on the host so that t fits in 32 bits.
struct ProdDiv {
    uint32_t bv, bs;            // vector columns per row, nodes per block
    int lg_bv, lg_bs;           // log2 when a power of two, else -1
};
__device__ __forceinline__ void prod_split(const ProdDiv d, uint32_t t, uint32_t& i, uint32_t& j, uint32_t& bc) {
    const uint32_t r = d.lg_bv >= 0 ? (t >> d.lg_bv) : (t / d.bv);
    bc = t - r * d.bv;
    i = d.lg_bs >= 0 ? (r >> d.lg_bs) : (r / d.bs);
    j = r - i * d.bs;
}

// Product forward.  Thread = (row block i, ROWS nodes j (and j + block / 2) of the block, VEC consecutive samples).
template <int VEC, int ROWS>
__global__ void prod_fwd_kernel(float* __restrict__ element_mars, const float* __restrict__ node_mars,
                                const int32_t* __restrict__ nids, const int32_t* __restrict__ cids,
                                uint32_t total, int64_t block0, ProdDiv d, int n_chs, int B) {
    const uint32_t t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= total) return;
    uint32_t il, j, bc;
    prod_split(d, t, il, j, bc);
    const int64_t i = block0 + il;
    const int b = (int)bc * VEC;
    const int64_t jstep = (int64_t)d.bs * B;
    float acc[ROWS][VEC];
#pragma unroll
    for (int r = 0; r < ROWS; ++r)
#pragma unroll
        for (int v = 0; v < VEC; ++v) acc[r][v] = 0.0f;
    const int32_t* crow = cids + i * n_chs;
    for (int c = 0; c < n_chs; ++c) {
        int32_t cid = crow[c];
        if (cid == 0) continue;
        const float* src = node_mars + ((int64_t)cid + j) * B + b;
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            if (VEC == 4) {
                float4 x = *reinterpret_cast<const float4*>(src + r * jstep);
                acc[r][0] += x.x; acc[r][1] += x.y; acc[r][2] += x.z; acc[r][3] += x.w;
            } else {
                acc[r][0] += src[r * jstep];
            }
        }
    }
    float* dst = element_mars + ((int64_t)nids[i] + j) * B + b;
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
        if (VEC == 4) *reinterpret_cast<float4*>(dst + r * jstep) = make_float4(acc[r][0], acc[r][1], acc[r][2], acc[r][3]);
        else dst[r * jstep] = acc[r][0];
    }
}

// Product backward: log-sum-exp over the parents, then logaddexp into the child's flow.  A thread owns VEC samples of
// ROWS nodes of one block (nodes j and j + block / 2 when ROWS = 2): they share the block's parent list, and the
// thread has twice as many independent loads in flight.  `d.bs` is then half the block size.
template <int VEC, int ROWS>
__global__ void prod_bwd_kernel(float* __restrict__ node_flows, const float* __restrict__ element_flows,
                                const int32_t* __restrict__ u_cids, const int32_t* __restrict__ parids,
                                uint32_t total, int64_t block0, ProdDiv d, int n_pars, int B, int logspace) {
    const uint32_t t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= total) return;
    uint32_t il, j, bc;
    prod_split(d, t, il, j, bc);
    const int64_t i = block0 + il;
    const int b = (int)bc * VEC;
    const int32_t* prow = parids + i * n_pars;
    const int64_t jstep = (int64_t)d.bs * B;            // distance between the thread's rows
    float* dst = node_flows + ((int64_t)u_cids[i] + j) * B + b;
    float cur[ROWS][VEC];                               // requested first: its latency overlaps the parents' loads
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
        if (VEC == 4) {
            const float4 q = *reinterpret_cast<const float4*>(dst + r * jstep);
            cur[r][0] = q.x; cur[r][1] = q.y; cur[r][2] = q.z; cur[r][3] = q.w;
        } else {
            cur[r][0] = dst[r * jstep];
        }
    }

    float mx[ROWS][VEC], sum[ROWS][VEC];
#pragma unroll
    for (int r = 0; r < ROWS; ++r)
#pragma unroll
        for (int v = 0; v < VEC; ++v) { mx[r][v] = PCX_NEG_INF; sum[r][v] = 0.0f; }
    for (int p = 0; p < n_pars; ++p) {
        int32_t pid = prow[p];
        if (pid == 0) continue;
        const float* src = element_flows + ((int64_t)pid + j) * B + b;
        float x[ROWS][VEC];
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            if (VEC == 4) {
                float4 q = *reinterpret_cast<const float4*>(src + r * jstep);
                x[r][0] = q.x; x[r][1] = q.y; x[r][2] = q.z; x[r][3] = q.w;
            } else {
                x[r][0] = src[r * jstep];
            }
        }
#pragma unroll
        for (int r = 0; r < ROWS; ++r)
#pragma unroll
            for (int v = 0; v < VEC; ++v) {
                const float xv = x[r][v];
                if (!logspace) { sum[r][v] += xv; continue; }
                if (xv == PCX_NEG_INF) continue;
                if (xv > mx[r][v]) { sum[r][v] = sum[r][v] * __expf(mx[r][v] - xv) + 1.0f; mx[r][v] = xv; }
                else sum[r][v] += __expf(xv - mx[r][v]);
            }
    }
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
        float out[VEC];
#pragma unroll
        for (int v = 0; v < VEC; ++v) {
            if (logspace) {
                // log(exp(cur) + exp(mx) * sum) around the larger of the two exponents
                const float hi = fmaxf(cur[r][v], mx[r][v]);
                const float s = __expf(cur[r][v] - hi) + sum[r][v] * __expf(mx[r][v] - hi);
                out[v] = (hi == PCX_NEG_INF) ? PCX_NEG_INF : hi + __logf(s);
            } else {
                out[v] = cur[r][v] + sum[r][v];
            }
        }
        if (VEC == 4) *reinterpret_cast<float4*>(dst + r * jstep) = make_float4(out[0], out[1], out[2], out[3]);
        else dst[r * jstep] = out[0];
    }
}

inline int lg2_or_neg(uint32_t v) {
    if (v == 0 || (v & (v - 1)) != 0) return -1;
    int l = 0;
    while ((1u << l) < v) ++l;
    return l;
}
// Cuts `n_blocks` row blocks into launches of fewer than 2^31 threads; `launch(first block, blocks, threads, div)`.
template <typename F>
inline void prod_launches(int64_t n_blocks, int block_size, int bv, F launch) {   // block_size: rows per block per thread set
    ProdDiv d;
    d.bv = (uint32_t)bv; d.bs = (uint32_t)block_size;
    d.lg_bv = lg2_or_neg(d.bv); d.lg_bs = lg2_or_neg(d.bs);
    const int64_t per_block = (int64_t)block_size * bv;
    const int64_t max_blocks = std::max<int64_t>(1, ((int64_t)1 << 31) / per_block - 1);
    for (int64_t b0 = 0; b0 < n_blocks; b0 += max_blocks) {
        const int64_t nb = std::min(max_blocks, n_blocks - b0);
        launch(b0, (uint32_t)(nb * per_block), d);
    }
}

inline int grid_for(int64_t work) {
    int64_t g = pcx_cdiv(work, kThreads);
    return (int)(g < 1 ? 1 : g);
}

}  // namespace

extern "C" {

int pcx_build_arch(void) { return 100; }

int pcx_fill_f32(float* p, int64_t n, float v, void* stream) {
    if (n <= 0) return 0;
    int64_t g = pcx_cdiv(pcx_cdiv(n, 4), kThreads);
    if (g > 148 * 16) g = 148 * 16;
    fill_kernel<<<(int)g, kThreads, 0, (cudaStream_t)stream>>>(p, n, v);
    PCX_LAUNCH_CHECK();
    return 0;
}

int pcx_scale_f32(float* p, int64_t n, float v, void* stream) {
    if (n <= 0) return 0;
    int64_t g = pcx_cdiv(n, kThreads);
    if (g > 148 * 16) g = 148 * 16;
    scale_kernel<<<(int)g, kThreads, 0, (cudaStream_t)stream>>>(p, n, v);
    PCX_LAUNCH_CHECK();
    return 0;
}

int pcx_exp_f32(float* p, int64_t n, void* stream) {
    if (n <= 0) return 0;
    int64_t g = pcx_cdiv(n, kThreads);
    if (g > 148 * 16) g = 148 * 16;
    exp_kernel<<<(int)g, kThreads, 0, (cudaStream_t)stream>>>(p, n);
    PCX_LAUNCH_CHECK();
    return 0;
}

int pcx_set_root_flows(float* node_flows, const float* weights, int64_t root_start, int64_t num_roots,
                       int B, int logspace, void* stream) {
    int64_t n = num_roots * B;
    if (n <= 0) return 0;
    root_flows_kernel<<<grid_for(n), kThreads, 0, (cudaStream_t)stream>>>(node_flows, weights, root_start * B, n, logspace);
    PCX_LAUNCH_CHECK();
    return 0;
}

int pcx_input_cat_fwd(float* node_mars, const float* params, const void* data, int data_elsize,
                      const int32_t* vids, const int32_t* s_pids, const int32_t* node_cats, int max_cats,
                      int64_t n_nodes, int64_t node_off, int B, void* stream) {
    if (data_elsize != 1 && data_elsize != 2 && data_elsize != 4 && data_elsize != 8) return -1;
    if (n_nodes <= 0 || B <= 0) return 0;
    if (max_cats <= 0) return -1;
    const int G = node_cats ? stage_group(max_cats) : 0;
    if (G >= 1 && B % 4 == 0 && (reinterpret_cast<uintptr_t>(node_mars) & 15) == 0) {
        dim3 grid((unsigned)pcx_cdiv(n_nodes, G), (unsigned)pcx_cdiv(B, kStageThreads * 4));
        input_cat_fwd_staged<<<grid, kStageThreads, (size_t)G * max_cats * sizeof(float), (cudaStream_t)stream>>>(
            node_mars, params, data, data_elsize, vids, s_pids, node_cats, max_cats, G, n_nodes, node_off, B);
    } else {
        input_cat_fwd_kernel<<<(unsigned)n_nodes, B >= 256 ? 256 : 128, 0, (cudaStream_t)stream>>>(
            node_mars, params, data, data_elsize, vids, s_pids, node_cats, max_cats, n_nodes, node_off, B);
    }
    PCX_LAUNCH_CHECK();
    return 0;
}

int pcx_input_cat_bwd(float* param_flows, const float* node_flows, const void* data, int data_elsize,
                      const int32_t* vids, const int32_t* s_pfids, const int32_t* node_cats, int max_cats,
                      int64_t n_nodes, int64_t node_off, int B, int logspace, void* stream) {
    if (data_elsize != 1 && data_elsize != 2 && data_elsize != 4 && data_elsize != 8) return -1;
    if (n_nodes <= 0 || B <= 0) return 0;
    if (max_cats <= 0) return -1;
    const int G = node_cats ? stage_group(max_cats) : 0;
    if (G >= 1 && B % 4 == 0 && (reinterpret_cast<uintptr_t>(node_flows) & 15) == 0) {
        input_cat_bwd_staged<<<(unsigned)pcx_cdiv(n_nodes, G), kStageThreads, (size_t)G * max_cats * sizeof(float),
                               (cudaStream_t)stream>>>(
            param_flows, node_flows, data, data_elsize, vids, s_pfids, node_cats, max_cats, G, n_nodes, node_off, B, logspace);
    } else {
        input_cat_bwd_kernel<<<(unsigned)n_nodes, B >= 256 ? 256 : 128, 0, (cudaStream_t)stream>>>(
            param_flows, node_flows, data, data_elsize, vids, s_pfids, node_cats, max_cats, n_nodes, node_off, B, logspace);
    }
    PCX_LAUNCH_CHECK();
    return 0;
}

int pcx_input_cat_shadow(float* logp_t, const float* params, int64_t n_rows, int num_cats, void* stream) {
    if (n_rows <= 0 || num_cats <= 0) return 0;
    dim3 grid((unsigned)pcx_cdiv(n_rows, 32), (unsigned)pcx_cdiv(num_cats, 32));
    input_cat_shadow_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(logp_t, params, n_rows, num_cats);
    PCX_LAUNCH_CHECK();
    return 0;
}

int pcx_input_cat_fwd_t(float* node_mars, const float* logp_t, const void* data, int data_elsize, const int32_t* vids,
                        const int32_t* prow, int64_t n_rows, int num_cats, int64_t n_nodes, int64_t node_off, int B,
                        void* stream) {
    if (data_elsize != 1 && data_elsize != 2 && data_elsize != 4 && data_elsize != 8) return -1;
    if (n_nodes <= 0 || B <= 0) return 0;
    if (B % 4 != 0 || num_cats <= 0 || (reinterpret_cast<uintptr_t>(node_mars) & 15) != 0) return -1;
    dim3 grid((unsigned)pcx_cdiv(n_nodes, kTN), (unsigned)pcx_cdiv(B, kTS));
    input_cat_fwd_t_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(node_mars, logp_t, data, data_elsize, vids, prow,
                                                                   n_rows, num_cats, n_nodes, node_off, B);
    PCX_LAUNCH_CHECK();
    return 0;
}

int pcx_input_cat_bwd_t(float* flows_t, int32_t* touched, const float* node_flows, const void* data, int data_elsize,
                        const int32_t* vids, const int32_t* prow, int64_t n_rows, int num_cats, int64_t n_nodes,
                        int64_t node_off, int B, int logspace, void* stream) {
    if (data_elsize != 1 && data_elsize != 2 && data_elsize != 4 && data_elsize != 8) return -1;
    if (n_nodes <= 0 || B <= 0) return 0;
    if (B % 4 != 0 || num_cats <= 0 || (reinterpret_cast<uintptr_t>(node_flows) & 15) != 0) return -1;
    dim3 grid((unsigned)pcx_cdiv(n_nodes, kTN), (unsigned)pcx_cdiv(B, kTS));
    input_cat_bwd_t_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(flows_t, node_flows, data, data_elsize, vids, prow,
                                                                   n_rows, num_cats, n_nodes, node_off, B, logspace, touched);
    PCX_LAUNCH_CHECK();
    return 0;
}

int pcx_input_cat_flush_t(float* param_flows, float* flows_t, int32_t* touched, const int64_t* row_pfid, int64_t n_rows,
                          int num_cats, void* stream) {
    if (n_rows <= 0 || num_cats <= 0) return 0;
    dim3 grid((unsigned)pcx_cdiv(n_rows, 32), (unsigned)pcx_cdiv(num_cats, 32));
    input_cat_flush_t_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(param_flows, flows_t, row_pfid, n_rows, num_cats, touched);
    PCX_LAUNCH_CHECK();
    cudaError_t e = cudaMemsetAsync(touched, 0, (size_t)num_cats * sizeof(int32_t), (cudaStream_t)stream);
    return e == cudaSuccess ? 0 : (int)e;
}

int pcx_prod_fwd(float* element_mars, const float* node_mars, const int32_t* nids, const int32_t* cids,
                 int64_t n_blocks, int n_chs, int block_size, int B, void* stream) {
    if (n_blocks <= 0 || B <= 0) return 0;
    if (B % 4 == 0) {
        if (block_size % 2 == 0)
            prod_launches(n_blocks, block_size / 2, B / 4, [&](int64_t b0, uint32_t total, ProdDiv d) {
                prod_fwd_kernel<4, 2><<<grid_for(total), kThreads, 0, (cudaStream_t)stream>>>(
                    element_mars, node_mars, nids, cids, total, b0, d, n_chs, B);
            });
        else
            prod_launches(n_blocks, block_size, B / 4, [&](int64_t b0, uint32_t total, ProdDiv d) {
                prod_fwd_kernel<4, 1><<<grid_for(total), kThreads, 0, (cudaStream_t)stream>>>(
                    element_mars, node_mars, nids, cids, total, b0, d, n_chs, B);
            });
    } else {
        prod_launches(n_blocks, block_size, B, [&](int64_t b0, uint32_t total, ProdDiv d) {
            prod_fwd_kernel<1, 1><<<grid_for(total), kThreads, 0, (cudaStream_t)stream>>>(
                element_mars, node_mars, nids, cids, total, b0, d, n_chs, B);
        });
    }
    PCX_LAUNCH_CHECK();
    return 0;
}

int pcx_prod_bwd(float* node_flows, const float* element_flows, const int32_t* u_cids, const int32_t* parids,
                 int64_t n_blocks, int n_pars, int block_size, int B, int logspace, void* stream) {
    if (n_blocks <= 0 || B <= 0) return 0;
    if (B % 4 == 0) {
        if (block_size % 2 == 0)
            prod_launches(n_blocks, block_size / 2, B / 4, [&](int64_t b0, uint32_t total, ProdDiv d) {
                prod_bwd_kernel<4, 2><<<grid_for(total), kThreads, 0, (cudaStream_t)stream>>>(
                    node_flows, element_flows, u_cids, parids, total, b0, d, n_pars, B, logspace);
            });
        else
            prod_launches(n_blocks, block_size, B / 4, [&](int64_t b0, uint32_t total, ProdDiv d) {
                prod_bwd_kernel<4, 1><<<grid_for(total), kThreads, 0, (cudaStream_t)stream>>>(
                    node_flows, element_flows, u_cids, parids, total, b0, d, n_pars, B, logspace);
            });
    } else {
        prod_launches(n_blocks, block_size, B, [&](int64_t b0, uint32_t total, ProdDiv d) {
            prod_bwd_kernel<1, 1><<<grid_for(total), kThreads, 0, (cudaStream_t)stream>>>(
                node_flows, element_flows, u_cids, parids, total, b0, d, n_pars, B, logspace);
        });
    }
    PCX_LAUNCH_CHECK();
    return 0;
}

}  // extern "C"
