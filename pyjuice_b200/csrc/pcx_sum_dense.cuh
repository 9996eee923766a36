// Dense sum layers (tables hundreds to thousands deep, e.g. the 4096 x 4096 transition layers of a large HMM).
//
// For such layers the work of turning child values into tensor-core operands -- column maximum, exp, bf16 hi/lo
// split -- must not be repeated by every 128-row tile (32 tiles share one operand in a 4096-row layer).  The layer is
// therefore run in two steps:
//
//   1. operand pre-pass: one pass over the child rows writes the scaled exponentials as ready-made operand tiles
//      (the K-major core-matrix layout the tensor core reads, hi tile then lo tile) to a scratch buffer, together
//      with the per-sample shifts;
//   2. a plain GEMM over pre-tiled operands: tiles travel global -> shared memory as single bulk copies
//      (cp.async.bulk, completion counted in bytes on an mbarrier), a four-stage ring decouples the copy thread from
//      the thread that issues tcgen05.mma, and four epilogue warps turn the accumulators into log-values / flows.
//
// The same GEMM serves the forward pass, the element flows and the parameter flows (there the contraction runs over
// the batch, and layers that share their parameters -- tied -- are contracted in one go: the batch dimensions of all
// of them are concatenated, so the flows of 127 tied layers are ONE 4096 x 4096 x 32512 product).
//
// Operand precision: both operands are bf16 hi + lo pairs.  The hi and lo parts of the B operand sit side by side in
// one 128-row tile, so that A_hi x [B_hi | B_lo] and A_lo x [B_hi | B_lo] are two MMAs of N = 128 per 16-deep step
// (the cost of an MMA this small is mostly fixed, so two wide ones beat three narrow ones, and lo x lo comes free);
// the epilogue adds accumulator columns j and j + 64.
//
// Accumulation: the tensor core truncates when it adds into its fp32 accumulator, which biases a long sum low.
// Four TMEM accumulators (4 x 128 columns = all of TMEM) take the chunks round-robin and are added in registers at
// the end, which divides the bias by four.
//
// This file is included by pcx_sum_tc.cu (it uses that file's helpers and status word).
#pragma once

namespace {

constexpr int DN = 64;                              // output columns per tile
constexpr int D_A_BYTES = 2 * A_TILE;               // 32 KB: A tile, hi then lo
constexpr int D_B_BYTES = 2 * B_TILE;               // 16 KB: B tile, hi then lo
constexpr int D_STAGE = D_A_BYTES + D_B_BYTES;      // 48 KB
constexpr int D_STAGES = 4;
constexpr int D_SMEM = D_STAGES * D_STAGE + 1024;
constexpr int D_THREADS = 192;                      // warp 0 copies, warp 1 multiplies, warps 2-5 finish
constexpr int D_ACCS = 4;
constexpr int D_ACC_COLS = 2 * DN;                  // hi-part columns, then lo-part columns
constexpr int D_BSLAB = 2 * DN * 16;                // one 8-deep K group of the B tile: 64 hi rows, 64 lo rows

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// One bulk copy global -> this CTA's shared memory; `bar` receives the byte count when the data has landed.
// Both addresses are 16-byte aligned and the size is a multiple of 16 by construction of the tile buffers.
__device__ __forceinline__ void bulk_copy_g2s(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(smem_dst)), "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

enum DenseEpi { D_FWD = 0, D_ELE = 1, D_PAR = 2 };

#ifdef PCX_TRACE
#define PCX_DT(k)                                                                                          \
    do {                                                                                                   \
        const int _slot = blockIdx.x + gridDim.x * blockIdx.y;                                             \
        if (_slot < kTraceItems) {                                                                         \
            long long _t;                                                                                  \
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(_t));                                         \
            g_trace[_slot][(k)] = _t;                                                                      \
        }                                                                                                  \
    } while (0)
#else
#define PCX_DT(k) do { } while (0)
#endif

struct DenseArgs {
    const uint8_t* a_tiles;     // A tile of (row tile mt, chunk c) at a_tiles + (mt * n_chunks + c) * 32 KB
    const uint8_t* b_tiles;     // B tile of (operand row r, chunk c) at b_tiles + (r * n_chunks + c) * 16 KB
    const int32_t* b_group;     // FWD / ELE: group of every table row (rows of a group share their operand)
    int n_chunks;
    int n_ct;                   // FWD / ELE: column tiles (of 64 samples) per group
    int row_block;              // rows per table row (multiple of 128)
    int B;
    int logspace;
    int terms;
    const int32_t* rows;        // FWD: nids   ELE: chids   PAR: nids (unused)
    float* out;                 // FWD: node_mars      ELE: element_flows     PAR: param_flows
    const float* shift;         // FWD / ELE: [n_groups, B] per-sample shifts
    const float* emars;         // ELE: element_mars
    const float* params;        // PAR
    const int32_t* cids;        // PAR: [n_rows, K]
    const int32_t* pids;        // PAR
    const int32_t* pfids;       // PAR
    int K;                      // PAR: table width
};

template <int EPI>
__global__ void __launch_bounds__(D_THREADS, 1) dense_gemm_kernel(const DenseArgs a) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ uint64_t s_full[D_STAGES], s_empty[D_STAGES], s_done;
    __shared__ uint32_t s_tmem;
    __shared__ volatile int s_fail;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int64_t mt = blockIdx.x;                  // 128-row tile
    const int nt = blockIdx.y;                      // FWD / ELE: 64-sample tile      PAR: 64-edge tile
    const int tiles_r = a.row_block / BM;
    const int64_t i = mt / tiles_r;
    const int r0 = (int)(mt % tiles_r) * BM;
    const int n_chunks = a.n_chunks;
    if (tid == 0) PCX_DT(0);

    if (tid == 0) {
        for (int s = 0; s < D_STAGES; ++s) { mbar_init(&s_full[s], 1); mbar_init(&s_empty[s], 1); }
        mbar_init(&s_done, 1);
        fence_mbar_init();
        s_fail = 0;
    }
    if (warp == 0) tmem_alloc(&s_tmem, D_ACCS * D_ACC_COLS);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = s_tmem;
    if (tid == 0) PCX_DT(1);

    const int64_t b_row = (EPI == D_PAR) ? (int64_t)nt : (int64_t)a.b_group[i] * a.n_ct + nt;
    const uint8_t* a_src = a.a_tiles + (size_t)mt * n_chunks * D_A_BYTES;
    const uint8_t* b_src = a.b_tiles + (size_t)b_row * n_chunks * D_B_BYTES;

    if (warp == 0) {
        // ---- copy warp: lane 0 waits for the stage and arms its barrier, twelve lanes each move 4 KB of it --------
        constexpr int PIECE = 4096;
        static_assert(D_STAGE % PIECE == 0 && D_STAGE / PIECE <= 32 && D_A_BYTES % PIECE == 0, "one piece per lane");
        int armed = 0;
        for (int c = 0; c < n_chunks; ++c) {
            const int s = c % D_STAGES;
            int stop = 0;
            if (lane == 0) {
                if (c >= D_STAGES && !mbar_wait(&s_empty[s], (uint32_t)((c / D_STAGES - 1) & 1))) s_fail = 1;
                stop = s_fail;
                if (!stop) mbar_expect_tx(&s_full[s], D_STAGE);
            }
            stop = __shfl_sync(0xffffffffu, stop, 0);
            if (stop) break;
            if (lane < D_STAGE / PIECE) {
                const int off = lane * PIECE;
                const uint8_t* src = (off < D_A_BYTES) ? a_src + (size_t)c * D_A_BYTES + off
                                                       : b_src + (size_t)c * D_B_BYTES + (off - D_A_BYTES);
                bulk_copy_g2s(smem + s * D_STAGE + off, src, PIECE, &s_full[s]);
            }
            armed = c + 1;
        }
        if (lane == 0 && s_fail) {
            // let the copies that are still in flight land before this CTA's shared memory goes away
            for (int c = max(0, armed - D_STAGES); c < armed; ++c)
                mbar_wait(&s_full[c % D_STAGES], (uint32_t)((c / D_STAGES) & 1), 1u << 16);
        }
    } else if (warp == 1) {
        // ---- multiply thread ----------------------------------------------------------------------------
        if (lane == 0) {
            const uint32_t idesc = idesc_bf16_f32(BM, D_ACC_COLS);
            for (int c = 0; c < n_chunks; ++c) {
                const int s = c % D_STAGES;
                if (!mbar_wait(&s_full[s], (uint32_t)((c / D_STAGES) & 1))) { s_fail = 2; break; }
                if (c == 0) PCX_DT(2);
                if (c == n_chunks - 1) PCX_DT(3);
                if (s_fail) break;
                tc_fence_after_sync();
                const uint32_t sa = smem_u32(smem + s * D_STAGE), sb = sa + D_A_BYTES;
                const uint32_t acc = tmem + (uint32_t)((c % D_ACCS) * D_ACC_COLS);
#pragma unroll
                for (int ks = 0; ks < KC / 16; ++ks) {
                    const uint64_t dAh = smem_desc(sa + ks * 2 * (BM * 16), BM * 16, 128);
                    const uint64_t dAl = smem_desc(sa + A_TILE + ks * 2 * (BM * 16), BM * 16, 128);
                    const uint64_t dB = smem_desc(sb + ks * 2 * D_BSLAB, D_BSLAB, 128);
                    mma_bf16_ss(acc, dAh, dB, idesc, (c >= D_ACCS || ks > 0) ? 1u : 0u);
                    if (a.terms == 3) mma_bf16_ss(acc, dAl, dB, idesc, 1u);
                }
                mma_commit(&s_empty[s]);            // the stage is free once these products have read it
            }
            mma_commit(&s_done);
        }
    } else {
        // ---- epilogue warps: TMEM lane quarter warp % 4, one output row per thread --------------------------
        const int lq = warp & 3;
        const int row = lq * 32 + lane;
        bool ok = mbar_wait(&s_done, 0u, 1u << 24);
        if (!ok) s_fail = 3;
        if (tid == 64) PCX_DT(4);
        ok = ok && (s_fail == 0);
        tc_fence_after_sync();
        const int used = n_chunks < D_ACCS ? n_chunks : D_ACCS;
        if (ok) {
#pragma unroll 1
            for (int p = 0; p < DN / 8; ++p) {
                float v[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] = 0.0f;
                for (int q = 0; q < used; ++q) {
                    float t[8], u[8];
                    tmem_ld<8>(tmem + ((uint32_t)(lq * 32) << 16) + (uint32_t)(q * D_ACC_COLS + 8 * p), t);
                    tmem_ld<8>(tmem + ((uint32_t)(lq * 32) << 16) + (uint32_t)(q * D_ACC_COLS + DN + 8 * p), u);
#pragma unroll
                    for (int j = 0; j < 8; ++j) v[j] += t[j] + u[j];
                }
                if (EPI == D_PAR) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const int e = nt * DN + 8 * p + j;
                        if (e >= a.K) continue;
                        if (a.cids[i * a.K + e] == 0) continue;
                        const float pf = a.params[(int64_t)a.pids[i * a.K + e] + r0 + row] * v[j];
                        if (pf != 0.0f) atomicAdd(a.out + (int64_t)a.pfids[i * a.K + e] + r0 + row, pf);
                    }
                } else {
                    const int cb = nt * DN + 8 * p;                // B is a multiple of 64 here
                    const float* sh = a.shift + (int64_t)a.b_group[i] * a.B + cb;
                    const int64_t orow = ((int64_t)a.rows[i] + r0 + row) * a.B + cb;
                    float o[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const float m = sh[j];
                        if (EPI == D_FWD) o[j] = (m == PCX_NEG_INF) ? PCX_NEG_INF : __logf(fmaxf(v[j], 1e-24f)) + m;
                        else o[j] = (m == PCX_NEG_INF || v[j] <= 0.0f) ? PCX_NEG_INF : __logf(v[j]) + m;
                    }
                    if (EPI == D_ELE) {
                        const float4 e0 = *reinterpret_cast<const float4*>(a.emars + orow);
                        const float4 e1 = *reinterpret_cast<const float4*>(a.emars + orow + 4);
                        const float em[8] = {e0.x, e0.y, e0.z, e0.w, e1.x, e1.y, e1.z, e1.w};
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            o[j] = (o[j] == PCX_NEG_INF || em[j] == PCX_NEG_INF) ? PCX_NEG_INF : o[j] + em[j];
                            if (!a.logspace) o[j] = __expf(o[j]);
                        }
                    }
                    float4* dst = reinterpret_cast<float4*>(a.out + orow);
                    dst[0] = make_float4(o[0], o[1], o[2], o[3]);
                    dst[1] = make_float4(o[4], o[5], o[6], o[7]);
                }
            }
        }
        tc_fence_before_sync();
        if (tid == 64) PCX_DT(5);
    }
    __syncthreads();
    if (tid == 0) PCX_DT(6);
    if (tid == 0 && s_fail != 0) atomicCAS(&g_tc_status, 0, 400 + 10 * EPI + s_fail);
    if (warp == 0) tmem_dealloc(tmem, D_ACCS * D_ACC_COLS);
}

// ---- operand pre-passes ------------------------------------------------------------------------------------
// Log-domain value of operand row k at sample b:
//   FWD: element_mars[cids[g, k], b]
//   ELE: node_flows[r, b] - node_mars[r, b] with r = parids[g, k / par_block] + k % par_block
//   PAR (X): node_flows[r, b] - node_mars[r, b] with r = nids[g] + k         (rows of the layer)
struct PrepArgs {
    const float* src;           // FWD: element_mars      ELE / PAR: node_flows
    const float* src2;          // ELE / PAR: node_mars
    const int32_t* kids;        // FWD: cids [n, K]   ELE: parids [n, P]   PAR: nids [n]
    const int32_t* group_row;   // [n_groups] a table row that stands for the group
    int K;                      // table width (FWD: children, ELE: parent blocks)
    int par_block;              // ELE: parent block size; PAR: rows per table row (block size); FWD: 1
    int depth;                  // rows of the operand per group (FWD: K, ELE: K * par_block, PAR: n_rows * block)
    int B;
    int logspace;
    int mode;                   // 0 FWD, 1 ELE, 2 PAR
};

__device__ __forceinline__ float prep_value(const PrepArgs& a, int g, int k, int b) {
    if (k >= a.depth) return PCX_NEG_INF;
    if (a.mode == 0) {
        const int cid = a.kids[(int64_t)a.group_row[g] * a.K + k];
        return cid != 0 ? a.src[(int64_t)cid * a.B + b] : PCX_NEG_INF;
    }
    int64_t r;
    if (a.mode == 1) {
        const int pr = a.kids[(int64_t)a.group_row[g] * a.K + k / a.par_block];
        if (pr == 0) return PCX_NEG_INF;
        r = (int64_t)pr + k % a.par_block;
    } else {
        r = (int64_t)a.kids[k / a.par_block] + k % a.par_block;
    }
    float f = a.src[r * a.B + b];
    const float m = a.src2[r * a.B + b];
    if (!a.logspace) f = (f > 0.0f) ? __logf(f) : PCX_NEG_INF;
    return (m == PCX_NEG_INF || f == PCX_NEG_INF) ? PCX_NEG_INF : f - m;
}

// partial[g][c][b] = max over the 64 operand rows of chunk c.  Grid (n_chunks, ceil(B / 64), n_groups), 256 threads =
// (64 samples, 4 quarters of the chunk's rows).
__global__ void dense_colmax_kernel(const PrepArgs a, float* __restrict__ partial, int n_chunks) {
    __shared__ float s_m[4][64];
    const int c = blockIdx.x, g = blockIdx.z;
    const int lc = threadIdx.x & 63, q = threadIdx.x >> 6;
    const int b = blockIdx.y * 64 + lc;
    const int bc = b < a.B ? b : a.B - 1;
    float m = PCX_NEG_INF;
#pragma unroll
    for (int j = 0; j < 16; ++j) m = fmaxf(m, prep_value(a, g, c * KC + q * 16 + j, bc));
    s_m[q][lc] = m;
    __syncthreads();
    if (q == 0 && b < a.B)
        partial[((int64_t)g * n_chunks + c) * a.B + b] = fmaxf(fmaxf(s_m[0][lc], s_m[1][lc]), fmaxf(s_m[2][lc], s_m[3][lc]));
}

// shift[g][b] = max over the chunks.  Grid (ceil(B / 256), n_groups), 256 threads.
__global__ void dense_shift_kernel(const float* __restrict__ partial, float* __restrict__ shift, int n_chunks, int B) {
    const int b = blockIdx.x * 256 + threadIdx.x, g = blockIdx.y;
    if (b >= B) return;
    float m = PCX_NEG_INF;
    for (int c = 0; c < n_chunks; ++c) m = fmaxf(m, partial[((int64_t)g * n_chunks + c) * B + b]);
    shift[(int64_t)g * B + b] = m;
}

// Operand tiles with the contraction over operand rows (FWD, ELE): tile (g, column tile jt, chunk c) is
// [8 row groups][64 samples hi, 64 samples lo][8 rows] bf16.  Grid (n_chunks, n_ct, n_groups), 256 threads:
// thread = (sample of the tile, two of the eight row groups).
__global__ void dense_rows_tiles_kernel(const PrepArgs a, const float* __restrict__ shift,
                                        uint8_t* __restrict__ tiles, int n_ct, int n_chunks) {
    const int c = blockIdx.x, jt = blockIdx.y, g = blockIdx.z;
    const int lc = threadIdx.x & 63, q = threadIdx.x >> 6;
    const int b = jt * DN + lc;                                     // B is a multiple of 64
    const float mx = shift[(int64_t)g * a.B + b];
    uint8_t* tile = tiles + (((size_t)g * n_ct + jt) * n_chunks + c) * D_B_BYTES;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int grp = q + 4 * h;
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float x = prep_value(a, g, c * KC + grp * 8 + j, b);
            v[j] = (x == PCX_NEG_INF) ? 0.0f : __expf(x - mx);
        }
        uint8_t* dst = tile + grp * D_BSLAB + lc * 16;                 // hi row lc, lo row 64 + lc of the K group
        store_split8(reinterpret_cast<uint4*>(dst), reinterpret_cast<uint4*>(dst + DN * 16), v);
    }
}

// Operand tiles with the contraction over the batch (parameter flows).  X: tile (row tile mt, chunk cc) is
// [8 sample groups][128 rows][8 samples], hi tile then lo tile; Y: tile (edge tile et, chunk cc) is
// [8 sample groups][64 edges hi, 64 edges lo][8 samples].
// shift[b] = max over the layer's rows of (flow - value), from the two kernels above; x = exp(flow - value - shift),
// y = exp(element value + shift).
// Tiles of layer `slot` go to chunk columns slot * cpl + cc of a buffer with `n_chunks` chunk columns per tile row.
// Grid (cpl, row tiles, 1) for X and (cpl, edge tiles, 1) for Y; 256 threads = (8 sample groups, 32 rows).
__global__ void dense_par_x_kernel(const PrepArgs a, const float* __restrict__ shift,
                                   uint8_t* __restrict__ tiles, int n_chunks, int slot, int cpl) {
    const int cc = blockIdx.x, mt = blockIdx.y;
    const int gq = threadIdx.x & 7, rb = threadIdx.x >> 3;
    const int b0 = cc * KC + gq * 8;
    float sh[8];
#pragma unroll
    for (int t = 0; t < 8; ++t) sh[t] = (b0 + t < a.B) ? shift[b0 + t] : PCX_NEG_INF;
    uint8_t* tile = tiles + ((size_t)mt * n_chunks + (size_t)slot * cpl + cc) * D_A_BYTES;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int r = rb + 32 * j;
        float v[8];
#pragma unroll
        for (int t = 0; t < 8; ++t) {
            const float x = (b0 + t < a.B) ? prep_value(a, 0, mt * BM + r, b0 + t) : PCX_NEG_INF;
            v[t] = (x == PCX_NEG_INF || sh[t] == PCX_NEG_INF) ? 0.0f : __expf(x - sh[t]);
        }
        uint8_t* dst = tile + gq * (BM * 16) + r * 16;
        store_split8(reinterpret_cast<uint4*>(dst), reinterpret_cast<uint4*>(dst + A_TILE), v);
    }
}

__global__ void dense_par_y_kernel(const float* __restrict__ element_mars, const int32_t* __restrict__ cids_row,
                                   int K, int B, const float* __restrict__ shift, uint8_t* __restrict__ tiles,
                                   int n_chunks, int slot, int cpl) {
    const int cc = blockIdx.x, et = blockIdx.y;
    const int gq = threadIdx.x & 7, rb = threadIdx.x >> 3;
    const int b0 = cc * KC + gq * 8;
    uint8_t* tile = tiles + ((size_t)et * n_chunks + (size_t)slot * cpl + cc) * D_B_BYTES;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        const int e = et * DN + rb + 32 * j;
        const int cid = (e < K) ? cids_row[e] : 0;
        float v[8];
#pragma unroll
        for (int t = 0; t < 8; ++t) {
            float y = 0.0f;
            if (cid != 0 && b0 + t < B) {
                const float em = element_mars[(int64_t)cid * B + b0 + t];
                const float s = shift[b0 + t];
                y = (em == PCX_NEG_INF || s == PCX_NEG_INF) ? 0.0f : fminf(__expf(em + s), 3.0e38f);
            }
            v[t] = y;
        }
        uint8_t* dst = tile + gq * D_BSLAB + (rb + 32 * j) * 16;
        store_split8(reinterpret_cast<uint4*>(dst), reinterpret_cast<uint4*>(dst + DN * 16), v);
    }
}

template <int EPI>
int launch_dense_gemm(const DenseArgs& a, dim3 grid, cudaStream_t st) {
    static PcxOnce done;
    if (!done) {
        cudaError_t e = cudaFuncSetAttribute(dense_gemm_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, D_SMEM);
        if (e != cudaSuccess) return (int)e;
        done = true;
    }
    dense_gemm_kernel<EPI><<<grid, D_THREADS, D_SMEM, st>>>(a);
    PCX_LAUNCH_CHECK();
    return 0;
}

inline size_t align256(size_t x) { return (x + 255) & ~size_t(255); }

}  // namespace

extern "C" {

int64_t pcx_dense_scratch_bytes(int n_groups, int depth, int B) {
    const int64_t n_chunks = pcx_cdiv(depth, KC), n_ct = pcx_cdiv(B, DN);
    return (int64_t)(align256((size_t)n_groups * n_ct * n_chunks * D_B_BYTES) +
                     align256((size_t)n_groups * n_chunks * B * sizeof(float)) + align256((size_t)n_groups * B * sizeof(float)));
}

static int dense_rows_op(int mode, float* out, const float* src, const float* src2, const float* emars,
                         const void* packed, const int32_t* rows, const int32_t* kids, const int32_t* row_group,
                         const int32_t* group_row, int n_groups, void* scratch, int64_t scratch_bytes,
                         int64_t n_rows, int K, int row_block, int par_block, int B, int logspace, cudaStream_t st) {
    if (n_rows <= 0 || B <= 0) return 0;
    const int depth = (mode == 0) ? K : K * par_block;
    if (row_block % BM != 0 || B % DN != 0 || n_groups <= 0 || depth <= 0) return -1;
    if (scratch == nullptr || (reinterpret_cast<uintptr_t>(scratch) & 255) != 0 ||
        scratch_bytes < pcx_dense_scratch_bytes(n_groups, depth, B)) return -1;
    const int n_chunks = (int)pcx_cdiv(depth, KC), n_ct = B / DN;
    uint8_t* tiles = reinterpret_cast<uint8_t*>(scratch);
    float* partial = reinterpret_cast<float*>(tiles + align256((size_t)n_groups * n_ct * n_chunks * D_B_BYTES));
    float* shift = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(partial) + align256((size_t)n_groups * n_chunks * B * sizeof(float)));

    PrepArgs p{};
    p.src = src; p.src2 = src2; p.kids = kids; p.group_row = group_row; p.K = K;
    p.par_block = (mode == 0) ? 1 : par_block; p.depth = depth; p.B = B; p.logspace = logspace; p.mode = mode;
    dense_colmax_kernel<<<dim3((unsigned)n_chunks, (unsigned)n_ct, (unsigned)n_groups), 256, 0, st>>>(p, partial, n_chunks);
    PCX_LAUNCH_CHECK();
    dense_shift_kernel<<<dim3((unsigned)pcx_cdiv(B, 256), (unsigned)n_groups), 256, 0, st>>>(partial, shift, n_chunks, B);
    PCX_LAUNCH_CHECK();
    dense_rows_tiles_kernel<<<dim3((unsigned)n_chunks, (unsigned)n_ct, (unsigned)n_groups), 256, 0, st>>>(
        p, shift, tiles, n_ct, n_chunks);
    PCX_LAUNCH_CHECK();

    DenseArgs a{};
    a.a_tiles = reinterpret_cast<const uint8_t*>(packed); a.b_tiles = tiles; a.b_group = row_group;
    a.n_chunks = n_chunks; a.n_ct = n_ct; a.row_block = row_block; a.B = B; a.logspace = logspace;
    a.terms = (g_sum_mode == 2) ? 1 : 3; a.rows = rows; a.out = out; a.shift = shift; a.emars = emars;
    dim3 grid((unsigned)(n_rows * (row_block / BM)), (unsigned)n_ct);
    return mode == 0 ? launch_dense_gemm<D_FWD>(a, grid, st) : launch_dense_gemm<D_ELE>(a, grid, st);
}

int pcx_sum_fwd_dense(float* node_mars, const float* element_mars, const void* packed, const int32_t* nids,
                      const int32_t* cids, const int32_t* row_group, const int32_t* group_row, int n_groups,
                      void* scratch, int64_t scratch_bytes, int64_t n_blocks, int K, int block_size, int B,
                      void* stream) {
    return dense_rows_op(0, node_mars, element_mars, nullptr, nullptr, packed, nids, cids, row_group, group_row,
                         n_groups, scratch, scratch_bytes, n_blocks, K, block_size, 1, B, 1, (cudaStream_t)stream);
}

int pcx_sum_bwd_ele_dense(float* element_flows, const float* element_mars, const float* node_flows,
                          const float* node_mars, const void* packed, const int32_t* chids, const int32_t* parids,
                          const int32_t* row_group, const int32_t* group_row, int n_groups, void* scratch,
                          int64_t scratch_bytes, int64_t n_blocks, int P, int block_size, int ch_block_size, int B,
                          int logspace, void* stream) {
    if (block_size % 8 != 0) return -1;
    return dense_rows_op(1, element_flows, node_flows, node_mars, element_mars, packed, chids, parids, row_group,
                         group_row, n_groups, scratch, scratch_bytes, n_blocks, P, ch_block_size, block_size, B,
                         logspace, (cudaStream_t)stream);
}

// Parameter flows, step 1 (once per layer, while element_mars holds that layer's products): operand tiles of the
// layer into chunk columns [slot * cpl, (slot + 1) * cpl) of the X and Y buffers, cpl = ceil(B / 64).
int pcx_sum_par_dense_stage(void* x_tiles, void* y_tiles, float* work /* (ceil(rows / 64) + 1) * B floats */,
                            const float* node_flows, const float* node_mars, const float* element_mars,
                            const int32_t* nids, const int32_t* cids, int64_t n_blocks, int K, int block_size, int B,
                            int n_chunks_total, int slot, int logspace, void* stream) {
    if (n_blocks <= 0 || B <= 0) return 0;
    if (block_size % BM != 0 || K <= 0 || slot < 0) return -1;
    const int cpl = (int)pcx_cdiv(B, KC);
    if ((slot + 1) * cpl > n_chunks_total) return -1;
    cudaStream_t st = (cudaStream_t)stream;
    const int row_chunks = (int)pcx_cdiv(n_blocks * block_size, KC);
    float* partial = work;
    float* shift = work + (size_t)row_chunks * B;
    PrepArgs p{};
    p.src = node_flows; p.src2 = node_mars; p.kids = nids; p.K = 1; p.par_block = block_size;
    p.depth = (int)(n_blocks * block_size); p.B = B; p.logspace = logspace; p.mode = 2;
    dense_colmax_kernel<<<dim3((unsigned)row_chunks, (unsigned)pcx_cdiv(B, 64), 1), 256, 0, st>>>(p, partial, row_chunks);
    PCX_LAUNCH_CHECK();
    dense_shift_kernel<<<dim3((unsigned)pcx_cdiv(B, 256), 1), 256, 0, st>>>(partial, shift, row_chunks, B);
    PCX_LAUNCH_CHECK();
    const int row_tiles = (int)(n_blocks * (block_size / BM));
    dense_par_x_kernel<<<dim3((unsigned)cpl, (unsigned)row_tiles), 256, 0, st>>>(
        p, shift, reinterpret_cast<uint8_t*>(x_tiles), n_chunks_total, slot, cpl);
    PCX_LAUNCH_CHECK();
    // every table row of a dense layer lists the same children (checked by the caller): row 0 stands for all
    dense_par_y_kernel<<<dim3((unsigned)cpl, (unsigned)pcx_cdiv(K, DN)), 256, 0, st>>>(
        element_mars, cids, K, B, shift, reinterpret_cast<uint8_t*>(y_tiles), n_chunks_total, slot, cpl);
    PCX_LAUNCH_CHECK();
    return 0;
}

// Parameter flows, step 2 (once per group of layers that share parameters): one product over all staged chunks.
int pcx_sum_par_dense_gemm(float* param_flows, const float* params, const void* x_tiles, const void* y_tiles,
                           const int32_t* cids, const int32_t* pids, const int32_t* pfids, int64_t n_blocks, int K,
                           int block_size, int n_chunks_total, void* stream) {
    if (n_blocks <= 0 || n_chunks_total <= 0) return 0;
    if (block_size % BM != 0 || K <= 0) return -1;
    DenseArgs a{};
    a.a_tiles = reinterpret_cast<const uint8_t*>(x_tiles); a.b_tiles = reinterpret_cast<const uint8_t*>(y_tiles);
    a.n_chunks = n_chunks_total; a.row_block = block_size; a.terms = (g_sum_mode == 2) ? 1 : 3;
    a.out = param_flows; a.params = params; a.cids = cids; a.pids = pids; a.pfids = pfids; a.K = K;
    dim3 grid((unsigned)(n_blocks * (block_size / BM)), (unsigned)pcx_cdiv(K, DN));
    return launch_dense_gemm<D_PAR>(a, grid, (cudaStream_t)stream);
}

}  // extern "C"
