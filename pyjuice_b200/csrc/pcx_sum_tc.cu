// Sum-layer forward and element-flow kernels on the Blackwell tensor cores (tcgen05.mma + TMEM).
//
// Both are log-sum-exp contractions  out[r, b] = log sum_k A[r, k] * exp(L[k, b])  with A >= 0 the sum
// parameters and L log-domain values.  One CTA owns a 128 (rows) x 128 (batch columns) output tile:
//
//   pass 1   thread t < 128 owns batch column t and scans L[:, t] for its maximum mx_t (no cross-thread
//            reduction: the batch is the contiguous dimension, so the scan is also perfectly coalesced);
//   pass 2   per 64-deep K chunk, threads 0..127 turn their column into exp(L - mx_t), threads 128..255
//            fetch one row of A each; both split every fp32 value into bf16 hi + lo and write the four
//            operand tiles (A_hi, A_lo, B_hi, B_lo) straight into shared memory in the K-major core-matrix
//            layout tcgen05.mma consumes; one thread then issues A_hi*B_hi + A_hi*B_lo + A_lo*B_hi into the
//            fp32 TMEM accumulator.  Two smem stages let chunk c+1 be produced while chunk c multiplies;
//            tcgen05.commit -> mbarrier tells when a stage may be overwritten;
//   epilogue warps 0..3 read the accumulator back (tcgen05.ld), apply log(.) + mx_t, transpose through
//            shared memory and store whole 512-byte rows.
//
// The three-term bf16 split keeps ~16 significant bits per factor (relative product error ~2^-16) with fp32
// accumulation; `PCX_SUM_BF16X1` drops to a single bf16 product.  Every mbarrier wait is bounded: on expiry
// the kernel records a status code, stops issuing work, frees its TMEM and returns.
#include "pcx_common.cuh"
#include "pcx_tc.cuh"
#include "../../include/pcx_b200.h"

namespace {

using namespace pcx_tc;

constexpr int BM = 128;          // rows per tile   (UMMA M)
constexpr int BN = 128;          // batch columns per tile (UMMA N)
constexpr int KC = 64;           // contraction depth per smem stage
constexpr int KG = KC / 8;       // 16-byte K groups per stage
constexpr int STAGES = 2;
constexpr int NTH = 256;
constexpr int TILE_BYTES = KG * BM * 16;                 // one operand tile (BM == BN): 8 KB... x2 below
constexpr int STAGE_BYTES = 4 * TILE_BYTES;              // A_hi, A_lo, B_hi, B_lo
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024;  // + alignment slack
static_assert(BM == BN, "operand tiles share one size");
static_assert(STAGES * STAGE_BYTES >= BM * (BN + 1) * 4, "epilogue transpose buffer aliases the stages");

__device__ int g_tc_status = 0;      // 0 ok; otherwise the code of the first bounded wait that gave up

enum Mode { FWD = 0, ELE = 1 };

struct Args {
    float* out;                 // FWD: node_mars            ELE: element_flows
    const float* lsrc;          // FWD: element_mars         ELE: node_flows
    const float* lsrc2;         //                           ELE: node_mars
    const float* emars;         //                           ELE: element_mars (epilogue)
    const float* params;
    const int32_t* rows;        // FWD: nids                 ELE: chids
    const int32_t* kids;        // FWD: cids [n, K]          ELE: parids [n, P]
    const int32_t* kpar;        // FWD: pids [n, K]          ELE: parpids [n, P]
    int K;                      // FWD: table width          ELE: P
    int row_block;              // FWD: block_size           ELE: ch_block_size   (rows per table row, multiple of 128)
    int par_block;              //                           ELE: block_size of the parents
    int B;
    int logspace;
    int terms;                  // 3 = hi*hi + hi*lo + lo*hi, 1 = hi*hi only
};

__device__ __forceinline__ uint32_t pack2(uint16_t a, uint16_t b) { return (uint32_t)a | ((uint32_t)b << 16); }

template <int MODE>
__global__ void __launch_bounds__(NTH, 1) sum_lse_tc_kernel(const Args a) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ uint64_t s_bar[STAGES];
    __shared__ uint32_t s_tmem;
    __shared__ float s_max[BN];
    __shared__ int s_fail;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int tiles_r = a.row_block / BM;
    const int64_t i = blockIdx.x / tiles_r;
    const int r0 = (int)(blockIdx.x % tiles_r) * BM;
    const int b0 = blockIdx.y * BN;
    const int B = a.B;
    // contraction length in elements
    const int KK = (MODE == FWD) ? a.K : a.K * a.par_block;
    const int lg_pb = (MODE == ELE) ? (31 - __clz(a.par_block)) : 0;
    const int n_chunks = (KK + KC - 1) / KC;

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) mbar_init(&s_bar[s], 1);
        fence_mbar_init();
        s_fail = 0;
    }
    if (warp == 0) tmem_alloc(&s_tmem, BN);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = s_tmem;

    // value L[k, col] of this thread's batch column (threads 0..127)
    const int col = b0 + tid;
    const bool col_ok = (tid < BN) && (col < B);
    auto load_l = [&](int k) -> float {
        if (k >= KK) return PCX_NEG_INF;
        if (MODE == FWD) {
            int cid = a.kids[i * a.K + k];
            return cid != 0 ? a.lsrc[(int64_t)cid * B + col] : PCX_NEG_INF;
        } else {
            int p = k >> lg_pb, n = k & (a.par_block - 1);
            int pr = a.kids[i * a.K + p];
            if (pr == 0) return PCX_NEG_INF;
            float nf = a.lsrc[(int64_t)(pr + n) * B + col];
            float nm = a.lsrc2[(int64_t)(pr + n) * B + col];
            if (!a.logspace) nf = (nf > 0.0f) ? logf(nf) : PCX_NEG_INF;
            return (nm == PCX_NEG_INF || nf == PCX_NEG_INF) ? PCX_NEG_INF : nf - nm;
        }
    };

    // ---- pass 1: column maxima ----------------------------------------------------------------------
    float mx = PCX_NEG_INF;
    if (col_ok) {
#pragma unroll 4
        for (int k = 0; k < KK; ++k) mx = fmaxf(mx, load_l(k));
    }
    if (tid < BN) s_max[tid] = mx;

    // ---- pass 2: produce operand tiles, multiply -------------------------------------------------------
    const uint32_t idesc = idesc_bf16_f32(BM, BN);
    bool failed = false;
    for (int c = 0; c < n_chunks; ++c) {
        const int s = c % STAGES, use = c / STAGES;
        uint8_t* st = smem + s * STAGE_BYTES;
        if (c >= STAGES && !failed) {
            if (!mbar_wait(&s_bar[s], (uint32_t)((use - 1) & 1))) { failed = true; s_fail = 1; }
        }
        const int k0 = c * KC;
        if (tid < BN) {
            // B operand: exp(L - mx) of this thread's column, 8 consecutive k per 16-byte store
            uint4* bhi = reinterpret_cast<uint4*>(st + 2 * TILE_BYTES);
            uint4* blo = reinterpret_cast<uint4*>(st + 3 * TILE_BYTES);
#pragma unroll 2
            for (int g = 0; g < KG; ++g) {
                float v[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] = col_ok ? load_l(k0 + g * 8 + j) : PCX_NEG_INF;
                uint16_t h[8], l[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    float x = (v[j] == PCX_NEG_INF) ? 0.0f : expf(v[j] - mx);
                    split_bf16(x, h[j], l[j]);
                }
                bhi[g * BN + tid] = make_uint4(pack2(h[0], h[1]), pack2(h[2], h[3]), pack2(h[4], h[5]), pack2(h[6], h[7]));
                blo[g * BN + tid] = make_uint4(pack2(l[0], l[1]), pack2(l[2], l[3]), pack2(l[4], l[5]), pack2(l[6], l[7]));
            }
        } else {
            // A operand: one row of parameters per thread
            const int r = tid - BN;
            uint4* ahi = reinterpret_cast<uint4*>(st);
            uint4* alo = reinterpret_cast<uint4*>(st + TILE_BYTES);
#pragma unroll 2
            for (int g = 0; g < KG; ++g) {
                float v[8];
                const int kb = k0 + g * 8;
                if (MODE == FWD) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        int k = kb + j;
                        v[j] = (k < KK) ? a.params[(int64_t)a.kpar[i * a.K + k] + r0 + r] : 0.0f;
                    }
                } else {
                    // 8 consecutive parent nodes of one parent block: contiguous in memory (block sizes >= 8)
                    int p = kb >> lg_pb, n = kb & (a.par_block - 1);
                    int pr = (kb < KK) ? a.kids[i * a.K + p] : 0;
                    if (pr != 0) {
                        const float* sp = a.params + (int64_t)a.kpar[i * a.K + p] + (int64_t)(r0 + r) * a.par_block + n;
                        if ((reinterpret_cast<uintptr_t>(sp) & 15) == 0) {
                            const float4* src = reinterpret_cast<const float4*>(sp);
                            float4 q0 = src[0], q1 = src[1];
                            v[0] = q0.x; v[1] = q0.y; v[2] = q0.z; v[3] = q0.w;
                            v[4] = q1.x; v[5] = q1.y; v[6] = q1.z; v[7] = q1.w;
                        } else {
#pragma unroll
                            for (int j = 0; j < 8; ++j) v[j] = sp[j];
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 8; ++j) v[j] = 0.0f;
                    }
                }
                uint16_t h[8], l[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) split_bf16(v[j], h[j], l[j]);
                ahi[g * BM + r] = make_uint4(pack2(h[0], h[1]), pack2(h[2], h[3]), pack2(h[4], h[5]), pack2(h[6], h[7]));
                alo[g * BM + r] = make_uint4(pack2(l[0], l[1]), pack2(l[2], l[3]), pack2(l[4], l[5]), pack2(l[6], l[7]));
            }
        }
        fence_async_smem();
        __syncthreads();
        failed = failed || (s_fail != 0);
        if (tid == 0 && !failed) {
            tc_fence_after_sync();
            const uint32_t sa = smem_u32(st);
#pragma unroll
            for (int ks = 0; ks < KC / 16; ++ks) {
                const uint32_t off = (uint32_t)ks * 2 * BM * 16;       // two K groups per MMA
                const uint64_t dAh = smem_desc(sa + off, BM * 16, 128);
                const uint64_t dAl = smem_desc(sa + TILE_BYTES + off, BM * 16, 128);
                const uint64_t dBh = smem_desc(sa + 2 * TILE_BYTES + off, BN * 16, 128);
                const uint64_t dBl = smem_desc(sa + 3 * TILE_BYTES + off, BN * 16, 128);
                mma_bf16_ss(tmem, dAh, dBh, idesc, (c > 0 || ks > 0) ? 1u : 0u);
                if (a.terms == 3) {
                    mma_bf16_ss(tmem, dAh, dBl, idesc, 1u);
                    mma_bf16_ss(tmem, dAl, dBh, idesc, 1u);
                }
            }
            mma_commit(&s_bar[s]);
        }
    }

    // ---- epilogue --------------------------------------------------------------------------------------
    {
        const int cl = n_chunks - 1;
        if (!failed && !mbar_wait(&s_bar[cl % STAGES], (uint32_t)((cl / STAGES) & 1))) { failed = true; s_fail = 2; }
        // every earlier chunk's multiply has completed too: a commit covers all tcgen05 work issued before it
    }
    __syncthreads();
    failed = failed || (s_fail != 0);
    tc_fence_after_sync();
    float* T = reinterpret_cast<float*>(smem);            // [BM][BN + 1], aliases the (now idle) stages
    if (warp < 4 && !failed) {
        const int row = warp * 32 + lane;
#pragma unroll 1
        for (int cg = 0; cg < BN / 32; ++cg) {
            float v[32];
            tmem_ld32(tmem + ((uint32_t)(warp * 32) << 16) + (uint32_t)(cg * 32), v);
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                float m = s_max[cg * 32 + j];
                float o;
                if (MODE == FWD) o = (m == PCX_NEG_INF) ? PCX_NEG_INF : logf(fmaxf(v[j], 1e-24f)) + m;
                else o = (m == PCX_NEG_INF || v[j] <= 0.0f) ? PCX_NEG_INF : logf(v[j]) + m;
                T[row * (BN + 1) + cg * 32 + j] = o;
            }
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (!failed) {
        const int64_t base_row = (int64_t)a.rows[i] + r0;
        for (int r = warp; r < BM; r += NTH / 32) {
#pragma unroll
            for (int cc = lane; cc < BN; cc += 32) {
                int b = b0 + cc;
                if (b >= B) continue;
                float o = T[r * (BN + 1) + cc];
                if (MODE == ELE) {
                    float em = a.emars[(base_row + r) * B + b];
                    o = (o == PCX_NEG_INF || em == PCX_NEG_INF) ? PCX_NEG_INF : o + em;
                    if (!a.logspace) o = expf(o);
                }
                a.out[(base_row + r) * B + b] = o;
            }
        }
    } else if (tid == 0) {
        atomicCAS(&g_tc_status, 0, 100 * (MODE + 1) + s_fail);
    }
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, BN);
}

int g_sum_mode = 1;      // 0: fp32 CUDA cores only, 1: tensor cores with bf16 hi/lo split, 2: tensor cores, single bf16

template <int MODE>
int launch_tc(const Args& a, int64_t n_blocks, cudaStream_t st) {
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(sum_lse_tc_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    dim3 grid((unsigned)(n_blocks * (a.row_block / BM)), (unsigned)pcx_cdiv(a.B, BN));
    sum_lse_tc_kernel<MODE><<<grid, NTH, SMEM_BYTES, st>>>(a);
    PCX_LAUNCH_CHECK();
    return 0;
}

}  // namespace

// Internal entry points used by pcx_sum_simt.cu's dispatchers; return 1 if the tensor-core path took the call.
int pcx_tc_try_sum_fwd(float* node_mars, const float* element_mars, const float* params, const int32_t* nids,
                       const int32_t* cids, const int32_t* pids, int64_t n_blocks, int K, int block_size, int B,
                       cudaStream_t st, int* rc) {
    if (g_sum_mode == 0 || block_size % BM != 0) return 0;
    Args a{};
    a.out = node_mars; a.lsrc = element_mars; a.params = params; a.rows = nids; a.kids = cids; a.kpar = pids;
    a.K = K; a.row_block = block_size; a.par_block = 1; a.B = B; a.logspace = 1; a.terms = (g_sum_mode == 2) ? 1 : 3;
    *rc = launch_tc<FWD>(a, n_blocks, st);
    return 1;
}

int pcx_tc_try_sum_ele(float* element_flows, const float* element_mars, const float* node_flows, const float* node_mars,
                       const float* params, const int32_t* chids, const int32_t* parids, const int32_t* parpids,
                       int64_t n_blocks, int P, int block_size, int ch_block_size, int B, int logspace,
                       cudaStream_t st, int* rc) {
    if (g_sum_mode == 0 || ch_block_size % BM != 0 || block_size % 8 != 0) return 0;
    Args a{};
    a.out = element_flows; a.lsrc = node_flows; a.lsrc2 = node_mars; a.emars = element_mars; a.params = params;
    a.rows = chids; a.kids = parids; a.kpar = parpids; a.K = P; a.row_block = ch_block_size; a.par_block = block_size;
    a.B = B; a.logspace = logspace; a.terms = (g_sum_mode == 2) ? 1 : 3;
    *rc = launch_tc<ELE>(a, n_blocks, st);
    return 1;
}

extern "C" {

int pcx_set_sum_mode(int mode) {
    if (mode < 0 || mode > 2) return -1;
    g_sum_mode = mode;
    return 0;
}

int pcx_get_status(void) {
    int v = 0;
    cudaError_t e = cudaMemcpyFromSymbol(&v, g_tc_status, sizeof(int));
    return e == cudaSuccess ? v : -(int)e;
}

}  // extern "C"
