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

// One thread per (node, sample); consecutive threads walk the batch.
__global__ void input_cat_fwd_kernel(float* __restrict__ node_mars, const float* __restrict__ params,
                                     const void* __restrict__ data, int elsize,
                                     const int32_t* __restrict__ vids, const int32_t* __restrict__ s_pids,
                                     int64_t n_nodes, int64_t node_off, int B) {
    int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= n_nodes * B) return;
    int64_t n = t / B;
    int b = (int)(t - n * B);
    int cat = pcx_load_cat(data, elsize, (int64_t)vids[n] * B + b);
    node_mars[(node_off + n) * B + b] = logf(params[(int64_t)s_pids[n] + cat]);
}

__global__ void input_cat_bwd_kernel(float* __restrict__ param_flows, const float* __restrict__ node_flows,
                                     const void* __restrict__ data, int elsize,
                                     const int32_t* __restrict__ vids, const int32_t* __restrict__ s_pfids,
                                     int64_t n_nodes, int64_t node_off, int B, int logspace) {
    int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= n_nodes * B) return;
    int64_t n = t / B;
    int b = (int)(t - n * B);
    float f = node_flows[(node_off + n) * B + b];
    f = logspace ? expf(f) : f;
    if (f == 0.0f) return;
    int cat = pcx_load_cat(data, elsize, (int64_t)vids[n] * B + b);
    atomicAdd(param_flows + (int64_t)s_pfids[n] + cat, f);
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
                      const int32_t* vids, const int32_t* s_pids, int64_t n_nodes, int64_t node_off,
                      int B, void* stream) {
    if (data_elsize != 1 && data_elsize != 2 && data_elsize != 4 && data_elsize != 8) return -1;
    if (n_nodes <= 0 || B <= 0) return 0;
    input_cat_fwd_kernel<<<grid_for(n_nodes * B), kThreads, 0, (cudaStream_t)stream>>>(
        node_mars, params, data, data_elsize, vids, s_pids, n_nodes, node_off, B);
    PCX_LAUNCH_CHECK();
    return 0;
}

int pcx_input_cat_bwd(float* param_flows, const float* node_flows, const void* data, int data_elsize,
                      const int32_t* vids, const int32_t* s_pfids, int64_t n_nodes, int64_t node_off,
                      int B, int logspace, void* stream) {
    if (data_elsize != 1 && data_elsize != 2 && data_elsize != 4 && data_elsize != 8) return -1;
    if (n_nodes <= 0 || B <= 0) return 0;
    input_cat_bwd_kernel<<<grid_for(n_nodes * B), kThreads, 0, (cudaStream_t)stream>>>(
        param_flows, node_flows, data, data_elsize, vids, s_pfids, n_nodes, node_off, B, logspace);
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
