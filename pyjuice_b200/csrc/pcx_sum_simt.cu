// Sum-layer kernels, fp32 CUDA-core version: block-sparse log-sum-exp contraction (forward), its
// transposed form (element flows) and the batch contraction that yields parameter flows.
//
// All three are the same shape of work: C[M x N] = sum_k A[m,k] * exp(L[k,n] - shift) with a
// log(...) + shift epilogue (forward / element flows) or a scale-and-accumulate epilogue
// (parameter flows).  A CTA of 256 threads owns one TM x 64 output tile, stages TK = 32 slices of
// both operands in shared memory (the exponentials are taken while staging, once per element) and
// accumulates RM x RN register tiles in fp32.  The running column maximum is carried across
// K-slices and the accumulators are rescaled when it grows, so no second pass over the inputs is
// needed.  Node blocks narrower than 8 (root layers have block size 1) use warp-per-row kernels.
//
// Arithmetic is fp32 throughout (FMA accumulate, expf/logf), the accuracy anchor for the path.
#include "pcx_common.cuh"
#include "../../include/pcx_b200.h"
#include <float.h>

namespace {

constexpr int TB = 64;       // output-tile width (batch for fwd/ele, edges for par)
constexpr int TK = 32;       // contraction slice
constexpr int NT = 256;      // threads per CTA

__device__ __forceinline__ int ilog2(int x) { return 31 - __clz(x); }

// log(flow / value) of one node and sample: flows arrive either in log space or (logspace == 0) linearly.
__device__ __forceinline__ float log_flow_over_mar(float nf, float nm, int logspace) {
    if (!logspace) nf = (nf > 0.0f) ? logf(nf) : PCX_NEG_INF;
    return (nm == PCX_NEG_INF || nf == PCX_NEG_INF) ? PCX_NEG_INF : nf - nm;
}

// -------------------------------------------------------------------------------------------------
// Forward:  node_mars[nid+m, b] = log sum_e params[pid_e + m] * exp(emars[cid_e, b])
// -------------------------------------------------------------------------------------------------
template <int TM, int RM, int RB>
__global__ void __launch_bounds__(NT)
sum_fwd_tiled(float* __restrict__ node_mars, const float* __restrict__ element_mars,
              const float* __restrict__ params, const int32_t* __restrict__ nids,
              const int32_t* __restrict__ cids, const int32_t* __restrict__ pids,
              int K, int block_size, int B) {
    static_assert((TM / RM) * (TB / RB) == NT, "thread tiling must cover the output tile");
    __shared__ __align__(16) float As[TK][TM];
    __shared__ __align__(16) float Bs[TK][TB];
    __shared__ int s_cid[TK], s_pid[TK];
    __shared__ float s_part[NT / TB][TB];
    __shared__ float s_runmax[TB], s_scale[TB];

    const int tid = threadIdx.x;
    const int tiles_m = block_size / TM;
    const int64_t i = blockIdx.x / tiles_m;
    const int m0 = (int)(blockIdx.x % tiles_m) * TM;
    const int b0 = blockIdx.y * TB;

    const int tb = tid % (TB / RB), tm = tid / (TB / RB);
    float acc[RM][RB];
#pragma unroll
    for (int r = 0; r < RM; ++r)
#pragma unroll
        for (int c = 0; c < RB; ++c) acc[r][c] = 0.0f;

    if (tid < TB) s_runmax[tid] = PCX_NEG_INF;

    const int lcol = tid % TB, lrow0 = tid / TB;          // staging role for the L operand
    const bool col_ok = (b0 + lcol) < B;

    for (int k0 = 0; k0 < K; k0 += TK) {
        __syncthreads();                                   // previous slice fully consumed
        if (tid < TK) {
            int k = k0 + tid;
            s_cid[tid] = (k < K) ? cids[i * K + k] : 0;
            s_pid[tid] = (k < K) ? pids[i * K + k] : 0;
        }
        __syncthreads();

        float v[TK / (NT / TB)];
        float vmax = PCX_NEG_INF;
#pragma unroll
        for (int r = 0; r < TK / (NT / TB); ++r) {
            int kk = lrow0 + r * (NT / TB);
            int cid = s_cid[kk];
            v[r] = (col_ok && cid != 0) ? element_mars[(int64_t)cid * B + b0 + lcol] : PCX_NEG_INF;
            vmax = fmaxf(vmax, v[r]);
        }
        s_part[lrow0][lcol] = vmax;
#pragma unroll
        for (int r = 0; r < (TK * TM) / NT; ++r) {
            int idx = tid + r * NT;
            int kk = idx / TM, m = idx % TM;
            As[kk][m] = params[(int64_t)s_pid[kk] + m0 + m];
        }
        __syncthreads();
        if (tid < TB) {
            float old = s_runmax[tid], nw = old;
#pragma unroll
            for (int r = 0; r < NT / TB; ++r) nw = fmaxf(nw, s_part[r][tid]);
            s_scale[tid] = (nw == PCX_NEG_INF) ? 1.0f : expf(old - nw);   // old == -inf -> 0, acc is 0 anyway
            s_runmax[tid] = nw;
        }
        __syncthreads();
        {
            float nw = s_runmax[lcol];
#pragma unroll
            for (int r = 0; r < TK / (NT / TB); ++r) {
                int kk = lrow0 + r * (NT / TB);
                Bs[kk][lcol] = (v[r] == PCX_NEG_INF) ? 0.0f : expf(v[r] - nw);
            }
        }
        float sc[RB];
#pragma unroll
        for (int c = 0; c < RB; ++c) sc[c] = s_scale[tb * RB + c];
#pragma unroll
        for (int r = 0; r < RM; ++r)
#pragma unroll
            for (int c = 0; c < RB; ++c) acc[r][c] *= sc[c];
        __syncthreads();
#pragma unroll 8
        for (int kk = 0; kk < TK; ++kk) {
            float a[RM], b[RB];
#pragma unroll
            for (int r = 0; r < RM; ++r) a[r] = As[kk][tm * RM + r];
#pragma unroll
            for (int c = 0; c < RB; ++c) b[c] = Bs[kk][tb * RB + c];
#pragma unroll
            for (int r = 0; r < RM; ++r)
#pragma unroll
                for (int c = 0; c < RB; ++c) acc[r][c] = fmaf(a[r], b[c], acc[r][c]);
        }
    }

    const int64_t nid = nids[i];
#pragma unroll
    for (int c = 0; c < RB; ++c) {
        int b = b0 + tb * RB + c;
        if (b >= B) continue;
        float mx = s_runmax[tb * RB + c];
#pragma unroll
        for (int r = 0; r < RM; ++r) {
            int m = m0 + tm * RM + r;
            float out = (mx == PCX_NEG_INF) ? PCX_NEG_INF : logf(fmaxf(acc[r][c], 1e-24f)) + mx;
            node_mars[(nid + m) * B + b] = out;
        }
    }
}

// Warp-per-edge-slice version for node blocks of 1, 2 or 4 nodes.
// CTA = (node block, 32 samples); warp w takes edges w, w+8, ...; lane = sample.
template <int BS>
__global__ void __launch_bounds__(NT)
sum_fwd_rows(float* __restrict__ node_mars, const float* __restrict__ element_mars,
             const float* __restrict__ params, const int32_t* __restrict__ nids,
             const int32_t* __restrict__ cids, const int32_t* __restrict__ pids, int K, int B) {
    __shared__ float s_mx[NT / 32][32];
    __shared__ float s_acc[NT / 32][BS][32];
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int64_t i = blockIdx.x;
    const int b = blockIdx.y * 32 + lane;
    float mx = PCX_NEG_INF, acc[BS];
#pragma unroll
    for (int m = 0; m < BS; ++m) acc[m] = 0.0f;
    for (int e = w; e < K; e += NT / 32) {
        int cid = cids[i * K + e];
        if (cid == 0) continue;
        float v = (b < B) ? element_mars[(int64_t)cid * B + b] : PCX_NEG_INF;
        if (v == PCX_NEG_INF) continue;
        int64_t pid = pids[i * K + e];
        float scale = 1.0f, x = 1.0f;
        if (v > mx) { scale = expf(mx - v); mx = v; } else { x = expf(v - mx); }
#pragma unroll
        for (int m = 0; m < BS; ++m) acc[m] = acc[m] * scale + params[pid + m] * x;
    }
    s_mx[w][lane] = mx;
#pragma unroll
    for (int m = 0; m < BS; ++m) s_acc[w][m][lane] = acc[m];
    __syncthreads();
    if (w == 0 && b < B) {
        float gm = PCX_NEG_INF;
#pragma unroll
        for (int q = 0; q < NT / 32; ++q) gm = fmaxf(gm, s_mx[q][lane]);
        const int64_t nid = nids[i];
#pragma unroll
        for (int m = 0; m < BS; ++m) {
            float tot = 0.0f;
#pragma unroll
            for (int q = 0; q < NT / 32; ++q) {
                float qm = s_mx[q][lane];
                if (qm != PCX_NEG_INF) tot += s_acc[q][m][lane] * expf(qm - gm);
            }
            node_mars[(nid + m) * B + b] = (gm == PCX_NEG_INF) ? PCX_NEG_INF : logf(fmaxf(tot, 1e-24f)) + gm;
        }
    }
}

// The same for few rows with very many edges (the root of a wide circuit: one row, thousands of children), where the
// kernel above leaves the machine to a handful of CTAs that each walk hundreds of dependent loads.  CTA = (node
// block, 8 samples); thread = (sample, one of 32 edge lanes); four edges per round, all of their loads issued before
// any is used.
template <int BS>
__global__ void __launch_bounds__(NT)
sum_fwd_rows_deep(float* __restrict__ node_mars, const float* __restrict__ element_mars,
                  const float* __restrict__ params, const int32_t* __restrict__ nids,
                  const int32_t* __restrict__ cids, const int32_t* __restrict__ pids, int K, int B) {
    constexpr int EL = NT / 8;
    __shared__ float s_mx[EL][8];
    __shared__ float s_acc[EL][BS][8];
    const int s = threadIdx.x & 7, el = threadIdx.x >> 3;
    const int64_t i = blockIdx.x;
    const int b = blockIdx.y * 8 + s;
    const int bc = b < B ? b : B - 1;
    float mx = PCX_NEG_INF, acc[BS];
#pragma unroll
    for (int m = 0; m < BS; ++m) acc[m] = 0.0f;
    for (int e0 = el; e0 < K; e0 += 4 * EL) {
        int cid[4];
        int64_t pid[4];
        float v[4], th[4][BS];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int e = e0 + q * EL;
            cid[q] = e < K ? cids[i * K + e] : 0;
            pid[q] = e < K ? pids[i * K + e] : 0;
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            v[q] = element_mars[(int64_t)cid[q] * B + bc];           // row 0 exists (-inf)
#pragma unroll
            for (int m = 0; m < BS; ++m) th[q][m] = params[pid[q] + m];
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            if (cid[q] == 0 || v[q] == PCX_NEG_INF) continue;
            float scale = 1.0f, x = 1.0f;
            if (v[q] > mx) { scale = expf(mx - v[q]); mx = v[q]; } else { x = expf(v[q] - mx); }
#pragma unroll
            for (int m = 0; m < BS; ++m) acc[m] = acc[m] * scale + th[q][m] * x;
        }
    }
    s_mx[el][s] = mx;
#pragma unroll
    for (int m = 0; m < BS; ++m) s_acc[el][m][s] = acc[m];
    __syncthreads();
    if (threadIdx.x < 8 && b < B) {
        float gm = PCX_NEG_INF;
        for (int q = 0; q < EL; ++q) gm = fmaxf(gm, s_mx[q][s]);
        const int64_t nid = nids[i];
#pragma unroll
        for (int m = 0; m < BS; ++m) {
            float tot = 0.0f;
            for (int q = 0; q < EL; ++q) {
                const float qm = s_mx[q][s];
                if (qm != PCX_NEG_INF) tot += s_acc[q][m][s] * expf(qm - gm);
            }
            node_mars[(nid + m) * B + b] = (gm == PCX_NEG_INF) ? PCX_NEG_INF : logf(fmaxf(tot, 1e-24f)) + gm;
        }
    }
}

// -------------------------------------------------------------------------------------------------
// Element flows:  eflows[chid+c, b] = emars[chid+c, b] + log sum_{p,n} params[parpid_p + c*bs + n] * exp(nflow - nmar)
// -------------------------------------------------------------------------------------------------
template <int TM, int RM, int RB>
__global__ void __launch_bounds__(NT)
sum_ele_tiled(float* __restrict__ element_flows, const float* __restrict__ element_mars,
              const float* __restrict__ node_flows, const float* __restrict__ node_mars,
              const float* __restrict__ params, const int32_t* __restrict__ chids,
              const int32_t* __restrict__ parids, const int32_t* __restrict__ parpids,
              int P, int block_size, int ch_block_size, int B, int logspace) {
    static_assert((TM / RM) * (TB / RB) == NT, "thread tiling must cover the output tile");
    __shared__ float As[TK][TM + 1];
    __shared__ __align__(16) float Bs[TK][TB];
    __shared__ int s_row[TK];
    __shared__ int64_t s_par[TK];
    __shared__ float s_part[NT / TB][TB];
    __shared__ float s_runmax[TB], s_scale[TB];

    const int tid = threadIdx.x;
    const int tiles_m = ch_block_size / TM;
    const int64_t i = blockIdx.x / tiles_m;
    const int c0 = (int)(blockIdx.x % tiles_m) * TM;
    const int b0 = blockIdx.y * TB;
    const int lg = ilog2(block_size);
    const int KK = P * block_size;

    const int tb = tid % (TB / RB), tm = tid / (TB / RB);
    float acc[RM][RB];
#pragma unroll
    for (int r = 0; r < RM; ++r)
#pragma unroll
        for (int c = 0; c < RB; ++c) acc[r][c] = 0.0f;
    if (tid < TB) s_runmax[tid] = PCX_NEG_INF;

    const int lcol = tid % TB, lrow0 = tid / TB;
    const bool col_ok = (b0 + lcol) < B;

    for (int k0 = 0; k0 < KK; k0 += TK) {
        __syncthreads();
        if (tid < TK) {
            int k = k0 + tid;
            int row = 0;
            int64_t par = 0;
            if (k < KK) {
                int p = k >> lg, n = k & (block_size - 1);
                int pr = parids[i * P + p];
                if (pr != 0) { row = pr + n; par = (int64_t)parpids[i * P + p] + n; }
            }
            s_row[tid] = row;
            s_par[tid] = par;
        }
        __syncthreads();

        float v[TK / (NT / TB)];
        float vmax = PCX_NEG_INF;
#pragma unroll
        for (int r = 0; r < TK / (NT / TB); ++r) {
            int kk = lrow0 + r * (NT / TB);
            int row = s_row[kk];
            float x = PCX_NEG_INF;
            if (col_ok && row != 0) {
                float nm = node_mars[(int64_t)row * B + b0 + lcol];
                float nf = node_flows[(int64_t)row * B + b0 + lcol];
                x = log_flow_over_mar(nf, nm, logspace);
            }
            v[r] = x;
            vmax = fmaxf(vmax, x);
        }
        s_part[lrow0][lcol] = vmax;
#pragma unroll
        for (int r = 0; r < (TK * TM) / NT; ++r) {
            int idx = tid + r * NT;
            int kk = idx % TK, c = idx / TK;                 // consecutive threads walk n: contiguous in memory
            As[kk][c] = (s_row[kk] != 0) ? params[s_par[kk] + (int64_t)(c0 + c) * block_size] : 0.0f;
        }
        __syncthreads();
        if (tid < TB) {
            float old = s_runmax[tid], nw = old;
#pragma unroll
            for (int r = 0; r < NT / TB; ++r) nw = fmaxf(nw, s_part[r][tid]);
            s_scale[tid] = (nw == PCX_NEG_INF) ? 1.0f : expf(old - nw);
            s_runmax[tid] = nw;
        }
        __syncthreads();
        {
            float nw = s_runmax[lcol];
#pragma unroll
            for (int r = 0; r < TK / (NT / TB); ++r) {
                int kk = lrow0 + r * (NT / TB);
                Bs[kk][lcol] = (v[r] == PCX_NEG_INF) ? 0.0f : expf(v[r] - nw);
            }
        }
        float sc[RB];
#pragma unroll
        for (int c = 0; c < RB; ++c) sc[c] = s_scale[tb * RB + c];
#pragma unroll
        for (int r = 0; r < RM; ++r)
#pragma unroll
            for (int c = 0; c < RB; ++c) acc[r][c] *= sc[c];
        __syncthreads();
#pragma unroll 8
        for (int kk = 0; kk < TK; ++kk) {
            float a[RM], b[RB];
#pragma unroll
            for (int r = 0; r < RM; ++r) a[r] = As[kk][tm * RM + r];
#pragma unroll
            for (int c = 0; c < RB; ++c) b[c] = Bs[kk][tb * RB + c];
#pragma unroll
            for (int r = 0; r < RM; ++r)
#pragma unroll
                for (int c = 0; c < RB; ++c) acc[r][c] = fmaf(a[r], b[c], acc[r][c]);
        }
    }

    const int64_t chid = chids[i];
#pragma unroll
    for (int c = 0; c < RB; ++c) {
        int b = b0 + tb * RB + c;
        if (b >= B) continue;
        float mx = s_runmax[tb * RB + c];
#pragma unroll
        for (int r = 0; r < RM; ++r) {
            int64_t row = chid + c0 + tm * RM + r;
            float em = element_mars[row * B + b];
            float out = (mx == PCX_NEG_INF || em == PCX_NEG_INF || acc[r][c] <= 0.0f)
                            ? PCX_NEG_INF : logf(acc[r][c]) + mx + em;
            element_flows[row * B + b] = logspace ? out : expf(out);
        }
    }
}

// Child blocks of 1, 2 or 4 nodes: CTA = (child block, 32 samples); warps split the (parent, node) pairs.
template <int CBS>
__global__ void __launch_bounds__(NT)
sum_ele_rows(float* __restrict__ element_flows, const float* __restrict__ element_mars,
             const float* __restrict__ node_flows, const float* __restrict__ node_mars,
             const float* __restrict__ params, const int32_t* __restrict__ chids,
             const int32_t* __restrict__ parids, const int32_t* __restrict__ parpids,
             int P, int block_size, int B, int logspace) {
    __shared__ float s_mx[NT / 32][32];
    __shared__ float s_acc[NT / 32][CBS][32];
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int64_t i = blockIdx.x;
    const int b = blockIdx.y * 32 + lane;
    const int lg = ilog2(block_size);
    const int KK = P * block_size;
    float mx = PCX_NEG_INF, acc[CBS];
#pragma unroll
    for (int c = 0; c < CBS; ++c) acc[c] = 0.0f;
    for (int k = w; k < KK; k += NT / 32) {
        int p = k >> lg, n = k & (block_size - 1);
        int pr = parids[i * P + p];
        if (pr == 0 || b >= B) continue;
        float nm = node_mars[(int64_t)(pr + n) * B + b];
        float nf = node_flows[(int64_t)(pr + n) * B + b];
        float v = log_flow_over_mar(nf, nm, logspace);
        if (v == PCX_NEG_INF) continue;
        int64_t pp = (int64_t)parpids[i * P + p] + n;
        float scale = 1.0f, x = 1.0f;
        if (v > mx) { scale = expf(mx - v); mx = v; } else { x = expf(v - mx); }
#pragma unroll
        for (int c = 0; c < CBS; ++c) acc[c] = acc[c] * scale + params[pp + (int64_t)c * block_size] * x;
    }
    s_mx[w][lane] = mx;
#pragma unroll
    for (int c = 0; c < CBS; ++c) s_acc[w][c][lane] = acc[c];
    __syncthreads();
    if (w == 0 && b < B) {
        float gm = PCX_NEG_INF;
#pragma unroll
        for (int q = 0; q < NT / 32; ++q) gm = fmaxf(gm, s_mx[q][lane]);
        const int64_t chid = chids[i];
#pragma unroll
        for (int c = 0; c < CBS; ++c) {
            float tot = 0.0f;
#pragma unroll
            for (int q = 0; q < NT / 32; ++q) {
                float qm = s_mx[q][lane];
                if (qm != PCX_NEG_INF) tot += s_acc[q][c][lane] * expf(qm - gm);
            }
            float em = element_mars[(chid + c) * B + b];
            float out = (gm == PCX_NEG_INF || em == PCX_NEG_INF || tot <= 0.0f) ? PCX_NEG_INF : logf(tot) + gm + em;
            element_flows[(chid + c) * B + b] = logspace ? out : expf(out);
        }
    }
}

// -------------------------------------------------------------------------------------------------
// Parameter flows:  pflows[pfid_e + m] += params[pid_e + m] * sum_b exp(nflow[nid+m,b] - nmar[nid+m,b] + emars[cid_e,b])
// -------------------------------------------------------------------------------------------------
template <int TM, int RM, int RE>
__global__ void __launch_bounds__(NT)
sum_par_tiled(float* __restrict__ param_flows, const float* __restrict__ node_flows,
              const float* __restrict__ node_mars, const float* __restrict__ element_mars,
              const float* __restrict__ params, const int32_t* __restrict__ nids,
              const int32_t* __restrict__ cids, const int32_t* __restrict__ pids,
              const int32_t* __restrict__ pfids, int K, int block_size, int B, int logspace) {
    static_assert((TM / RM) * (TB / RE) == NT, "thread tiling must cover the output tile");
    constexpr int XR = (TM * TK) / NT;      // X elements staged per thread
    constexpr int YR = (TB * TK) / NT;      // Y elements staged per thread
    __shared__ float Xs[TK][TM + 1];
    __shared__ float Ys[TK][TB + 1];
    __shared__ int s_cid[TB];
    __shared__ float s_part[NT / TK][TK];
    __shared__ float s_shift[TK];

    const int tid = threadIdx.x;
    const int tiles_m = block_size / TM;
    const int tiles_e = (K + TB - 1) / TB;
    int64_t bx = blockIdx.x;
    const int et = (int)(bx % tiles_e); bx /= tiles_e;
    const int m0 = (int)(bx % tiles_m) * TM;
    const int64_t i = bx / tiles_m;
    const int e0 = et * TB;
    const int64_t nid = nids[i];

    // compute role: m fastest across threads so that the epilogue's accesses to params / flows coalesce
    const int tm = tid % (TM / RM), te = tid / (TM / RM);
    float acc[RM][RE];
#pragma unroll
    for (int r = 0; r < RM; ++r)
#pragma unroll
        for (int c = 0; c < RE; ++c) acc[r][c] = 0.0f;

    if (tid < TB) {
        int e = e0 + tid;
        s_cid[tid] = (e < K) ? cids[i * K + e] : 0;
    }
    const int lk = tid % TK, lr0 = tid / TK;      // staging role: lane walks the batch (contiguous)

    for (int bb = 0; bb < B; bb += TK) {
        __syncthreads();
        const bool b_ok = (bb + lk) < B;
        float x[XR];
        float xmax = PCX_NEG_INF;
#pragma unroll
        for (int r = 0; r < XR; ++r) {
            int m = lr0 + r * (NT / TK);
            float val = PCX_NEG_INF;
            if (b_ok) {
                float nm = node_mars[(nid + m0 + m) * B + bb + lk];
                float nf = node_flows[(nid + m0 + m) * B + bb + lk];
                val = log_flow_over_mar(nf, nm, logspace);
            }
            x[r] = val;
            xmax = fmaxf(xmax, val);
        }
        s_part[lr0][lk] = xmax;
        float y[YR];
#pragma unroll
        for (int r = 0; r < YR; ++r) {
            int e = lr0 + r * (NT / TK);
            int cid = s_cid[e];
            y[r] = (b_ok && cid != 0) ? element_mars[(int64_t)cid * B + bb + lk] : PCX_NEG_INF;
        }
        __syncthreads();
        if (tid < TK) {
            float s = PCX_NEG_INF;
#pragma unroll
            for (int r = 0; r < NT / TK; ++r) s = fmaxf(s, s_part[r][tid]);
            s_shift[tid] = s;
        }
        __syncthreads();
        const float s = s_shift[lk];
#pragma unroll
        for (int r = 0; r < XR; ++r) {
            int m = lr0 + r * (NT / TK);
            Xs[lk][m] = (s == PCX_NEG_INF || x[r] == PCX_NEG_INF) ? 0.0f : expf(x[r] - s);
        }
#pragma unroll
        for (int r = 0; r < YR; ++r) {
            int e = lr0 + r * (NT / TK);
            Ys[lk][e] = (s == PCX_NEG_INF || y[r] == PCX_NEG_INF) ? 0.0f : fminf(expf(y[r] + s), FLT_MAX);
        }
        __syncthreads();
#pragma unroll 8
        for (int kk = 0; kk < TK; ++kk) {
            float a[RM], b[RE];
#pragma unroll
            for (int r = 0; r < RM; ++r) a[r] = Xs[kk][tm * RM + r];
#pragma unroll
            for (int c = 0; c < RE; ++c) b[c] = Ys[kk][te * RE + c];
#pragma unroll
            for (int r = 0; r < RM; ++r)
#pragma unroll
                for (int c = 0; c < RE; ++c) acc[r][c] = fmaf(a[r], b[c], acc[r][c]);
        }
    }

#pragma unroll
    for (int c = 0; c < RE; ++c) {
        int e = e0 + te * RE + c;
        if (e >= K) continue;
        if (s_cid[te * RE + c] == 0) continue;
        int64_t pid = pids[i * K + e], pfid = pfids[i * K + e];
#pragma unroll
        for (int r = 0; r < RM; ++r) {
            int m = m0 + tm * RM + r;
            float pf = params[pid + m] * acc[r][c];
            if (pf != 0.0f) atomicAdd(param_flows + pfid + m, pf);
        }
    }
}

// Node blocks of 1, 2 or 4 nodes: one warp per (node block, edge); lanes stride over the batch.
template <int BS>
__global__ void __launch_bounds__(NT)
sum_par_rows(float* __restrict__ param_flows, const float* __restrict__ node_flows,
             const float* __restrict__ node_mars, const float* __restrict__ element_mars,
             const float* __restrict__ params, const int32_t* __restrict__ nids,
             const int32_t* __restrict__ cids, const int32_t* __restrict__ pids,
             const int32_t* __restrict__ pfids, int64_t n_blocks, int K, int B, int logspace) {
    const int lane = threadIdx.x & 31;
    const int64_t wid = (int64_t)blockIdx.x * (NT / 32) + (threadIdx.x >> 5);
    if (wid >= n_blocks * K) return;
    const int64_t i = wid / K;
    const int e = (int)(wid % K);
    const int cid = cids[i * K + e];
    if (cid == 0) return;
    const int64_t nid = nids[i];
    float acc[BS];
#pragma unroll
    for (int m = 0; m < BS; ++m) acc[m] = 0.0f;
    for (int b = lane; b < B; b += 32) {
        float em = element_mars[(int64_t)cid * B + b];
        if (em == PCX_NEG_INF) continue;
#pragma unroll
        for (int m = 0; m < BS; ++m) {
            float nm = node_mars[(nid + m) * B + b];
            float nf = node_flows[(nid + m) * B + b];
            float lf = log_flow_over_mar(nf, nm, logspace);
            if (lf != PCX_NEG_INF) acc[m] += fminf(expf(lf + em), FLT_MAX);
        }
    }
#pragma unroll
    for (int m = 0; m < BS; ++m) {
        float v = acc[m];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (lane == 0) {
            float pf = params[(int64_t)pids[i * K + e] + m] * v;
            if (pf != 0.0f) atomicAdd(param_flows + (int64_t)pfids[i * K + e] + m, pf);
        }
    }
}


// ---- other propagation rules (plain kernels, one thread per output) ---------------------------------------------------
// alg 1 "MPE":        value(n) = max_k (log theta[n,k] + child_k);  a parent hands its whole flow to the children that
//                      attain the maximum (|log theta + child - value| < 1e-6), parameter flows likewise.
// alg 2 "GeneralLL":  value(n) = (1 / alpha) * log sum_k (theta[n,k] * exp(child_k))^alpha;  element flows carry the
//                      weights theta^alpha * exp(alpha * (child - value)), parameter flows the ordinary ones.
// alg 0 is the ordinary rule (kept here so that one kernel serves as the reference for the others in tests).
// Reference: layer/kernels/sum_forward_block_sparse.py:83-160, sum_backward_element_block_sparse.py:77-160,
// sum_backward_param_block_sparse.py:57-134.
__global__ void sum_fwd_alg_kernel(float* __restrict__ node_mars, const float* __restrict__ element_mars,
                                   const float* __restrict__ params, const int32_t* __restrict__ nids,
                                   const int32_t* __restrict__ cids, const int32_t* __restrict__ pids,
                                   int64_t n_blocks, int K, int bs, int B, int alg, float alpha) {
    const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= n_blocks * bs * B) return;
    const int b = (int)(t % B);
    const int j = (int)((t / B) % bs);
    const int64_t i = t / ((int64_t)B * bs);
    float mx = PCX_NEG_INF, sum = 0.0f;
    for (int k = 0; k < K; ++k) {
        const int cid = cids[i * K + k];
        if (cid == 0) continue;
        float v = logf(params[(int64_t)pids[i * K + k] + j]) + element_mars[(int64_t)cid * B + b];
        if (alg == 2) v *= alpha;
        if (v == PCX_NEG_INF) continue;
        if (alg == 1) { mx = fmaxf(mx, v); continue; }
        if (v > mx) { sum = sum * expf(mx - v) + 1.0f; mx = v; }
        else sum += expf(v - mx);
    }
    float out = mx;
    if (alg != 1 && mx != PCX_NEG_INF) out = mx + logf(sum);
    if (alg == 2) out /= alpha;
    node_mars[((int64_t)nids[i] + j) * B + b] = out;
}

// weight (log domain) with which parent n hands flow to element e; -inf when none
__device__ __forceinline__ float alg_log_weight(int alg, float alpha, float ltheta, float em, float nm) {
    if (nm == PCX_NEG_INF || em == PCX_NEG_INF || ltheta == PCX_NEG_INF) return PCX_NEG_INF;
    if (alg == 1) return (fabsf(ltheta + em - nm) < 1e-6f) ? 0.0f : PCX_NEG_INF;
    const float w = ltheta + em - nm;
    return alg == 2 ? alpha * w : w;
}

__global__ void sum_ele_alg_kernel(float* __restrict__ element_flows, const float* __restrict__ element_mars,
                                   const float* __restrict__ node_flows, const float* __restrict__ node_mars,
                                   const float* __restrict__ params, const int32_t* __restrict__ chids,
                                   const int32_t* __restrict__ parids, const int32_t* __restrict__ parpids,
                                   int64_t n_blocks, int P, int bs, int cbs, int B, int logspace, int alg, float alpha) {
    const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= n_blocks * cbs * B) return;
    const int b = (int)(t % B);
    const int c = (int)((t / B) % cbs);
    const int64_t i = t / ((int64_t)B * cbs);
    const int64_t erow = (int64_t)chids[i] + c;
    const float em = element_mars[erow * B + b];
    float mx = PCX_NEG_INF, sum = 0.0f;
    for (int p = 0; p < P; ++p) {
        const int par = parids[i * P + p];
        if (par == 0) continue;
        for (int n = 0; n < bs; ++n) {
            const float nf = node_flows[((int64_t)par + n) * B + b];
            const float lf = logspace ? nf : logf(nf);
            const float lw = alg_log_weight(alg, alpha, logf(params[(int64_t)parpids[i * P + p] + (int64_t)c * bs + n]), em,
                                            node_mars[((int64_t)par + n) * B + b]);
            const float v = lf + lw;
            if (v == PCX_NEG_INF || lf == PCX_NEG_INF) continue;
            if (v > mx) { sum = sum * expf(mx - v) + 1.0f; mx = v; }
            else sum += expf(v - mx);
        }
    }
    const float lo = (mx == PCX_NEG_INF) ? PCX_NEG_INF : mx + logf(sum);
    element_flows[erow * B + b] = logspace ? lo : expf(lo);
}

__global__ void sum_par_alg_kernel(float* __restrict__ param_flows, const float* __restrict__ node_flows,
                                   const float* __restrict__ node_mars, const float* __restrict__ element_mars,
                                   const float* __restrict__ params, const int32_t* __restrict__ nids,
                                   const int32_t* __restrict__ cids, const int32_t* __restrict__ pids,
                                   const int32_t* __restrict__ pfids, int64_t n_blocks, int K, int bs, int B,
                                   int logspace, int alg, float alpha) {
    const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= n_blocks * K * bs) return;
    const int j = (int)(t % bs);
    const int k = (int)((t / bs) % K);
    const int64_t i = t / ((int64_t)bs * K);
    const int cid = cids[i * K + k];
    if (cid == 0) return;
    const float ltheta = logf(params[(int64_t)pids[i * K + k] + j]);
    const int64_t nrow = (int64_t)nids[i] + j;
    float acc = 0.0f;
    for (int b = 0; b < B; ++b) {
        const float nf = node_flows[nrow * B + b];
        const float lf = logspace ? nf : logf(nf);
        // GeneralLL: the reference's parameter flows keep the ordinary weight theta * exp(child - value), with the
        // GeneralLL values (sum_backward_param_block_sparse.py:79-134; tests/layer/propagation_algs_test.py:224-236)
        const float lw = alg_log_weight(alg == 2 ? 0 : alg, alpha, ltheta, element_mars[(int64_t)cid * B + b],
                                        node_mars[nrow * B + b]);
        if (lf == PCX_NEG_INF || lw == PCX_NEG_INF) continue;
        acc += expf(lf + lw);
    }
    if (acc != 0.0f) atomicAdd(param_flows + (int64_t)pfids[i * K + k] + j, acc);
}

}  // namespace

// tensor-core dispatch (pcx_sum_tc.cu): returns 1 when it took the call, with the launch status in *rc
int pcx_tc_try_sum_par(float*, const float*, const float*, const float*, const float*, const int32_t*, const int32_t*,
                       const int32_t*, const int32_t*, int64_t, int, int, int, int, cudaStream_t, int*);

extern "C" {

int pcx_sum_fwd(float* node_mars, const float* element_mars, const float* params,
                const int32_t* nids, const int32_t* cids, const int32_t* pids,
                int64_t n_blocks, int K, int block_size, int B, void* stream) {
    if (n_blocks <= 0 || B <= 0) return 0;
    if (block_size <= 0 || (block_size & (block_size - 1)) != 0 || K <= 0) return -1;
    cudaStream_t st = (cudaStream_t)stream;
    if (block_size >= 8) {
        dim3 grid(1, (unsigned)pcx_cdiv(B, TB));
        if (block_size >= 64) {
            grid.x = (unsigned)(n_blocks * (block_size / 64));
            sum_fwd_tiled<64, 4, 4><<<grid, NT, 0, st>>>(node_mars, element_mars, params, nids, cids, pids, K, block_size, B);
        } else if (block_size == 32) {
            grid.x = (unsigned)n_blocks;
            sum_fwd_tiled<32, 2, 4><<<grid, NT, 0, st>>>(node_mars, element_mars, params, nids, cids, pids, K, block_size, B);
        } else if (block_size == 16) {
            grid.x = (unsigned)n_blocks;
            sum_fwd_tiled<16, 1, 4><<<grid, NT, 0, st>>>(node_mars, element_mars, params, nids, cids, pids, K, block_size, B);
        } else {
            grid.x = (unsigned)n_blocks;
            sum_fwd_tiled<8, 1, 2><<<grid, NT, 0, st>>>(node_mars, element_mars, params, nids, cids, pids, K, block_size, B);
        }
    } else if (K >= 512 && n_blocks * pcx_cdiv(B, 32) < 148) {          // few rows, very many edges: spread the edges
        dim3 grid((unsigned)n_blocks, (unsigned)pcx_cdiv(B, 8));
        if (block_size == 4) sum_fwd_rows_deep<4><<<grid, NT, 0, st>>>(node_mars, element_mars, params, nids, cids, pids, K, B);
        else if (block_size == 2) sum_fwd_rows_deep<2><<<grid, NT, 0, st>>>(node_mars, element_mars, params, nids, cids, pids, K, B);
        else sum_fwd_rows_deep<1><<<grid, NT, 0, st>>>(node_mars, element_mars, params, nids, cids, pids, K, B);
    } else {
        dim3 grid((unsigned)n_blocks, (unsigned)pcx_cdiv(B, 32));
        if (block_size == 4) sum_fwd_rows<4><<<grid, NT, 0, st>>>(node_mars, element_mars, params, nids, cids, pids, K, B);
        else if (block_size == 2) sum_fwd_rows<2><<<grid, NT, 0, st>>>(node_mars, element_mars, params, nids, cids, pids, K, B);
        else sum_fwd_rows<1><<<grid, NT, 0, st>>>(node_mars, element_mars, params, nids, cids, pids, K, B);
    }
    PCX_LAUNCH_CHECK();
    return 0;
}

int pcx_sum_bwd_ele(float* element_flows, const float* element_mars, const float* node_flows,
                    const float* node_mars, const float* params,
                    const int32_t* chids, const int32_t* parids, const int32_t* parpids,
                    int64_t n_blocks, int P, int block_size, int ch_block_size, int B, int logspace, void* stream) {
    if (n_blocks <= 0 || B <= 0) return 0;
    if (block_size <= 0 || (block_size & (block_size - 1)) != 0) return -1;
    if (ch_block_size <= 0 || (ch_block_size & (ch_block_size - 1)) != 0 || P <= 0) return -1;
    cudaStream_t st = (cudaStream_t)stream;
#define PCX_ELE_ARGS element_flows, element_mars, node_flows, node_mars, params, chids, parids, parpids, P, block_size
    if (ch_block_size >= 8) {
        dim3 grid(1, (unsigned)pcx_cdiv(B, TB));
        if (ch_block_size >= 64) {
            grid.x = (unsigned)(n_blocks * (ch_block_size / 64));
            sum_ele_tiled<64, 4, 4><<<grid, NT, 0, st>>>(PCX_ELE_ARGS, ch_block_size, B, logspace);
        } else if (ch_block_size == 32) {
            grid.x = (unsigned)n_blocks;
            sum_ele_tiled<32, 2, 4><<<grid, NT, 0, st>>>(PCX_ELE_ARGS, ch_block_size, B, logspace);
        } else if (ch_block_size == 16) {
            grid.x = (unsigned)n_blocks;
            sum_ele_tiled<16, 1, 4><<<grid, NT, 0, st>>>(PCX_ELE_ARGS, ch_block_size, B, logspace);
        } else {
            grid.x = (unsigned)n_blocks;
            sum_ele_tiled<8, 1, 2><<<grid, NT, 0, st>>>(PCX_ELE_ARGS, ch_block_size, B, logspace);
        }
    } else {
        dim3 grid((unsigned)n_blocks, (unsigned)pcx_cdiv(B, 32));
        if (ch_block_size == 4) sum_ele_rows<4><<<grid, NT, 0, st>>>(PCX_ELE_ARGS, B, logspace);
        else if (ch_block_size == 2) sum_ele_rows<2><<<grid, NT, 0, st>>>(PCX_ELE_ARGS, B, logspace);
        else sum_ele_rows<1><<<grid, NT, 0, st>>>(PCX_ELE_ARGS, B, logspace);
    }
#undef PCX_ELE_ARGS
    PCX_LAUNCH_CHECK();
    return 0;
}

int pcx_sum_bwd_par(float* param_flows, const float* node_flows, const float* node_mars,
                    const float* element_mars, const float* params,
                    const int32_t* nids, const int32_t* cids, const int32_t* pids, const int32_t* pfids,
                    int64_t n_blocks, int K, int block_size, int B, int logspace, void* stream) {
    if (n_blocks <= 0 || B <= 0) return 0;
    if (block_size <= 0 || (block_size & (block_size - 1)) != 0 || K <= 0) return -1;
    cudaStream_t st = (cudaStream_t)stream;
    int rc = 0;
    if (pcx_tc_try_sum_par(param_flows, node_flows, node_mars, element_mars, params, nids, cids, pids, pfids,
                           n_blocks, K, block_size, B, logspace, st, &rc)) return rc;
#define PCX_PAR_ARGS param_flows, node_flows, node_mars, element_mars, params, nids, cids, pids, pfids
    if (block_size >= 8) {
        int64_t tiles_e = pcx_cdiv(K, TB);
        if (block_size >= 64) {
            sum_par_tiled<64, 4, 4><<<(unsigned)(n_blocks * (block_size / 64) * tiles_e), NT, 0, st>>>(PCX_PAR_ARGS, K, block_size, B, logspace);
        } else if (block_size == 32) {
            sum_par_tiled<32, 2, 4><<<(unsigned)(n_blocks * tiles_e), NT, 0, st>>>(PCX_PAR_ARGS, K, block_size, B, logspace);
        } else if (block_size == 16) {
            sum_par_tiled<16, 1, 4><<<(unsigned)(n_blocks * tiles_e), NT, 0, st>>>(PCX_PAR_ARGS, K, block_size, B, logspace);
        } else {
            sum_par_tiled<8, 1, 2><<<(unsigned)(n_blocks * tiles_e), NT, 0, st>>>(PCX_PAR_ARGS, K, block_size, B, logspace);
        }
    } else {
        unsigned grid = (unsigned)pcx_cdiv(n_blocks * K, NT / 32);
        if (block_size == 4) sum_par_rows<4><<<grid, NT, 0, st>>>(PCX_PAR_ARGS, n_blocks, K, B, logspace);
        else if (block_size == 2) sum_par_rows<2><<<grid, NT, 0, st>>>(PCX_PAR_ARGS, n_blocks, K, B, logspace);
        else sum_par_rows<1><<<grid, NT, 0, st>>>(PCX_PAR_ARGS, n_blocks, K, B, logspace);
    }
#undef PCX_PAR_ARGS
    PCX_LAUNCH_CHECK();
    return 0;
}

int pcx_sum_fwd_alg(float* node_mars, const float* element_mars, const float* params, const int32_t* nids,
                    const int32_t* cids, const int32_t* pids, int64_t n_blocks, int K, int block_size, int B, int alg,
                    float alpha, void* stream) {
    if (n_blocks <= 0 || B <= 0) return 0;
    if (block_size <= 0 || K <= 0 || alg < 0 || alg > 2 || (alg == 2 && !(alpha > 0.0f))) return -1;
    const int64_t total = n_blocks * block_size * B;
    sum_fwd_alg_kernel<<<(unsigned)pcx_cdiv(total, 256), 256, 0, (cudaStream_t)stream>>>(
        node_mars, element_mars, params, nids, cids, pids, n_blocks, K, block_size, B, alg, alpha);
    PCX_LAUNCH_CHECK();
    return 0;
}

int pcx_sum_bwd_ele_alg(float* element_flows, const float* element_mars, const float* node_flows, const float* node_mars,
                        const float* params, const int32_t* chids, const int32_t* parids, const int32_t* parpids,
                        int64_t n_blocks, int P, int block_size, int ch_block_size, int B, int logspace, int alg,
                        float alpha, void* stream) {
    if (n_blocks <= 0 || B <= 0) return 0;
    if (block_size <= 0 || ch_block_size <= 0 || P <= 0 || alg < 0 || alg > 2 || (alg == 2 && !(alpha > 0.0f))) return -1;
    const int64_t total = n_blocks * ch_block_size * B;
    sum_ele_alg_kernel<<<(unsigned)pcx_cdiv(total, 256), 256, 0, (cudaStream_t)stream>>>(
        element_flows, element_mars, node_flows, node_mars, params, chids, parids, parpids, n_blocks, P, block_size,
        ch_block_size, B, logspace, alg, alpha);
    PCX_LAUNCH_CHECK();
    return 0;
}

int pcx_sum_bwd_par_alg(float* param_flows, const float* node_flows, const float* node_mars, const float* element_mars,
                        const float* params, const int32_t* nids, const int32_t* cids, const int32_t* pids,
                        const int32_t* pfids, int64_t n_blocks, int K, int block_size, int B, int logspace, int alg,
                        float alpha, void* stream) {
    if (n_blocks <= 0 || B <= 0) return 0;
    if (block_size <= 0 || K <= 0 || alg < 0 || alg > 2 || (alg == 2 && !(alpha > 0.0f))) return -1;
    const int64_t total = n_blocks * K * block_size;
    sum_par_alg_kernel<<<(unsigned)pcx_cdiv(total, 256), 256, 0, (cudaStream_t)stream>>>(
        param_flows, node_flows, node_mars, element_mars, params, nids, cids, pids, pfids, n_blocks, K, block_size, B,
        logspace, alg, alpha);
    PCX_LAUNCH_CHECK();
    return 0;
}


}  // extern "C"
