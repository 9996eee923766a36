// Bandwidth-bound kernels of the circuit path: buffer fills, categorical leaves (forward gather and
// flow scatter) and product layers (gather-add forward, logaddexp-accumulate backward).
//
// Layout: every value buffer is [rows, B] fp32 with the batch innermost, so a warp that walks the
// batch dimension reads and writes whole 128-byte lines.  Product rows are handled four samples per
// thread (float4) whenever B is a multiple of 4.
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

// Nodes per CTA of the staged kernels: up to 16, limited by 32 KB of shared memory; 0 = table too large to stage.
inline int stage_group(int max_cats) {
    if (max_cats <= 0) return 0;
    int g = (32 * 1024 / 4) / max_cats;
    return g > 16 ? 16 : g;
}

// Product forward.  Thread = (row block i, node j of the block, VEC consecutive samples).
template <int VEC>
__global__ void prod_fwd_kernel(float* __restrict__ element_mars, const float* __restrict__ node_mars,
                                const int32_t* __restrict__ nids, const int32_t* __restrict__ cids,
                                int64_t n_blocks, int n_chs, int block_size, int B) {
    const int bv = B / VEC;
    int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t total = n_blocks * block_size * bv;
    if (t >= total) return;
    int b = (int)(t % bv) * VEC;
    int64_t r = t / bv;
    int j = (int)(r % block_size);
    int64_t i = r / block_size;
    float acc[VEC];
#pragma unroll
    for (int v = 0; v < VEC; ++v) acc[v] = 0.0f;
    const int32_t* crow = cids + i * n_chs;
    for (int c = 0; c < n_chs; ++c) {
        int32_t cid = crow[c];
        if (cid == 0) continue;
        const float* src = node_mars + ((int64_t)cid + j) * B + b;
        if (VEC == 4) {
            float4 x = *reinterpret_cast<const float4*>(src);
            acc[0] += x.x; acc[1] += x.y; acc[2] += x.z; acc[3] += x.w;
        } else {
            acc[0] += src[0];
        }
    }
    float* dst = element_mars + ((int64_t)nids[i] + j) * B + b;
    if (VEC == 4) *reinterpret_cast<float4*>(dst) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    else dst[0] = acc[0];
}

// Product backward: log-sum-exp over the parents, then logaddexp into the child's flow.
template <int VEC>
__global__ void prod_bwd_kernel(float* __restrict__ node_flows, const float* __restrict__ element_flows,
                                const int32_t* __restrict__ u_cids, const int32_t* __restrict__ parids,
                                int64_t n_blocks, int n_pars, int block_size, int B, int logspace) {
    const int bv = B / VEC;
    int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t total = n_blocks * block_size * bv;
    if (t >= total) return;
    int b = (int)(t % bv) * VEC;
    int64_t r = t / bv;
    int j = (int)(r % block_size);
    int64_t i = r / block_size;
    const int32_t* prow = parids + i * n_pars;

    float mx[VEC], sum[VEC];
#pragma unroll
    for (int v = 0; v < VEC; ++v) { mx[v] = PCX_NEG_INF; sum[v] = 0.0f; }
    for (int p = 0; p < n_pars; ++p) {
        int32_t pid = prow[p];
        if (pid == 0) continue;
        const float* src = element_flows + ((int64_t)pid + j) * B + b;
        float x[VEC];
        if (VEC == 4) {
            float4 q = *reinterpret_cast<const float4*>(src);
            x[0] = q.x; x[1] = q.y; x[2] = q.z; x[3] = q.w;
        } else {
            x[0] = src[0];
        }
#pragma unroll
        for (int v = 0; v < VEC; ++v) {
            if (!logspace) { sum[v] += x[v]; continue; }
            if (x[v] == PCX_NEG_INF) continue;
            if (x[v] > mx[v]) { sum[v] = sum[v] * expf(mx[v] - x[v]) + 1.0f; mx[v] = x[v]; }
            else sum[v] += expf(x[v] - mx[v]);
        }
    }
    float* dst = node_flows + ((int64_t)u_cids[i] + j) * B + b;
    float out[VEC];
#pragma unroll
    for (int v = 0; v < VEC; ++v) {
        if (logspace) {
            float inc = (mx[v] == PCX_NEG_INF) ? PCX_NEG_INF : mx[v] + logf(sum[v]);
            out[v] = pcx_logaddexp(dst[v], inc);
        } else {
            out[v] = dst[v] + sum[v];
        }
    }
    if (VEC == 4) *reinterpret_cast<float4*>(dst) = make_float4(out[0], out[1], out[2], out[3]);
    else dst[0] = out[0];
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

int pcx_prod_fwd(float* element_mars, const float* node_mars, const int32_t* nids, const int32_t* cids,
                 int64_t n_blocks, int n_chs, int block_size, int B, void* stream) {
    if (n_blocks <= 0 || B <= 0) return 0;
    if (B % 4 == 0) {
        prod_fwd_kernel<4><<<grid_for(n_blocks * block_size * (B / 4)), kThreads, 0, (cudaStream_t)stream>>>(
            element_mars, node_mars, nids, cids, n_blocks, n_chs, block_size, B);
    } else {
        prod_fwd_kernel<1><<<grid_for(n_blocks * block_size * B), kThreads, 0, (cudaStream_t)stream>>>(
            element_mars, node_mars, nids, cids, n_blocks, n_chs, block_size, B);
    }
    PCX_LAUNCH_CHECK();
    return 0;
}

int pcx_prod_bwd(float* node_flows, const float* element_flows, const int32_t* u_cids, const int32_t* parids,
                 int64_t n_blocks, int n_pars, int block_size, int B, int logspace, void* stream) {
    if (n_blocks <= 0 || B <= 0) return 0;
    if (B % 4 == 0) {
        prod_bwd_kernel<4><<<grid_for(n_blocks * block_size * (B / 4)), kThreads, 0, (cudaStream_t)stream>>>(
            node_flows, element_flows, u_cids, parids, n_blocks, n_pars, block_size, B, logspace);
    } else {
        prod_bwd_kernel<1><<<grid_for(n_blocks * block_size * B), kThreads, 0, (cudaStream_t)stream>>>(
            node_flows, element_flows, u_cids, parids, n_blocks, n_pars, block_size, B, logspace);
    }
    PCX_LAUNCH_CHECK();
    return 0;
}

}  // extern "C"
