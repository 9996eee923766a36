// Sum layers with small node blocks (16 ... 64 nodes) on the tensor cores: "sample-major" tiles.
//
// A tcgen05 tile needs 128 rows.  With 32-node blocks the rows of a layer do not share children, so stacking four
// blocks into one row tile would waste the contraction.  Instead the BATCH is the M dimension: a tile is 128 samples
// x NB nodes (NB = 32 or 64: one node block, or the consecutive blocks of a vector that list the same children),
//     D[b, n] = sum_k exp(child[k, b] - max_b) * theta[n, k],
// i.e. the transpose of the row-major tile of pcx_sum_tc.cu.  The operand of exponentials (128 samples x K, K-major)
// is produced by the CTA's threads exactly as there; the parameter operand (NB nodes x K) comes pre-split from
// global memory.  The accumulator has one sample per TMEM lane and one node per column, so the epilogue writes, for
// every node, 32 consecutive samples per warp: fully coalesced without a transpose.
//
// Forward and element flows share the kernel (element flows: the "children" are the parent nodes' flow / value
// ratios, the "nodes" are the child elements, and the element's own value is added at the end).
// Included by pcx_sum_tc.cu.
#pragma once

namespace {

constexpr int SM_SAMPLES = 128;                       // samples per tile (UMMA M)
constexpr int SM_E_TILE = KG * SM_SAMPLES * 16;       // 16 KB: one bf16 [128 x 64] tile of exponentials
constexpr int SM_STAGE = 2 * SM_E_TILE + 2 * B_TILE;  // E hi, E lo, theta hi, theta lo (theta: up to 64 nodes) = 48 KB
static_assert(SM_STAGE == STAGE_BYTES, "same shared-memory budget as the row-major kernels");

struct SmArgs {
    float* out;                 // FWD: node_mars            ELE: element_flows
    const float* src;           // FWD: element_mars         ELE: node_flows
    const float* src2;          //                           ELE: node_mars
    const float* emars;         //                           ELE: element_mars
    const uint4* packed;        // parameter tiles: tile (m, chunk) = [hi | lo] x [8 K groups][NB nodes][8 k] bf16
    const int32_t* first_row;   // [n_tiles_m] first table row of every merged row
    const int32_t* rows;        // FWD: nids                 ELE: chids
    const int32_t* kids;        // FWD: cids [n, K]          ELE: parids [n, P]
    int64_t n_tiles;            // merged rows x sample tiles
    int n_st;                   // sample tiles = ceil(B / 128)
    int K;                      // FWD: table width          ELE: parent blocks per child block
    int par_block;              // FWD: 1                    ELE: parent block size (multiple of 8)
    int B;
    int logspace;
    int terms;
    // Product layer folded in (products of at most two children): FWD: fk = [n, K] pairs of child rows of node_mars
    // per table entry; ELE: fk = [n, child block size] pairs per output element.  nmars = node_mars.  A pair (0, 0)
    // means "no element"; row 0 of node_mars is the dummy node with value 0, so a single child needs no masking.
    const int2* fk;
    const float* nmars;
    int cbs;                    // ELE: child block size (rows of fk per table row)
};

// value of a folded product: sum of its two child rows, -inf when it has no child at all
__device__ __forceinline__ float folded2(const int2 r, const float* nmars_col, int B) {
    const float v = nmars_col[(int64_t)r.x * B] + nmars_col[(int64_t)r.y * B];
    return ((r.x | r.y) != 0) ? v : PCX_NEG_INF;
}

// One CTA walks tiles m * n_st + st (static round-robin: tiles do not depend on each other).
template <int NB, bool ELE>
__global__ void __launch_bounds__(NTH, 2) sum_sm_kernel(const SmArgs a) {
    constexpr int TCOLS = 2 * NB;                      // two accumulators (one per stage)
    constexpr int TH_TILE = 2 * KG * NB * 16;          // bytes of one parameter tile (hi + lo)
    constexpr int HC = NB / 2;                         // epilogue: node columns per thread
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ uint64_t s_bar[STAGES];
    __shared__ uint32_t s_tmem;
    __shared__ float s_part[STAGES][2 * SM_SAMPLES];   // per stage: the two partial maxima of every sample
    __shared__ int s_fail;
    static_assert(STAGES == 2, "two stages, two accumulators");

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) mbar_init(&s_bar[s], 1);
        fence_mbar_init();
        s_fail = 0;
    }
    if (warp == 0) tmem_alloc(&s_tmem, TCOLS);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = s_tmem;
    uint32_t ph[STAGES] = {0, 0};                      // completed phases of the two barriers

    const int B = a.B;
    const int KK = ELE ? a.K * a.par_block : a.K;
    const int lg_pb = ELE ? (31 - __clz(a.par_block)) : 0;
    const int n_chunks = (KK + KC - 1) / KC;
    const int ls = tid & (SM_SAMPLES - 1), h = tid >> 7;       // operand role: sample ls, K groups h, h + 2, ...
    const uint32_t idesc = idesc_bf16_f32(SM_SAMPLES, NB);

    for (int64_t tile = blockIdx.x; tile < a.n_tiles; tile += gridDim.x) {
        const int64_t m = tile / a.n_st;
        const int b0 = (int)(tile % a.n_st) * SM_SAMPLES;
        const int i0 = a.first_row[m];
        const int col = b0 + ls;
        const bool col_ok = col < B;
        const int colc = col_ok ? col : 0;

        // log-domain values of one 8-deep K group (unconditional loads, row 0 exists and is masked afterwards)
        // (entries without a child / parent read the dummy row 0, see the small-table kernel below)
        // four groups at once (the thread's share of one chunk): every index, then every value, then the arithmetic,
        // so that one chunk costs two memory round trips instead of eight
        auto load_groups4 = [&](int kb0, float (*v)[8]) {
            if (!ELE && a.fk != nullptr) {
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                    int2 r[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const int k = kb0 + 16 * t + j;
                        r[j] = (k < KK) ? a.fk[(int64_t)i0 * a.K + k] : make_int2(0, 0);
                    }
#pragma unroll
                    for (int j = 0; j < 8; ++j) v[t][j] = folded2(r[j], a.nmars + colc, B);
                }
            } else if (!ELE) {
                int cid[4][8];
#pragma unroll
                for (int t = 0; t < 4; ++t)
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const int k = kb0 + 16 * t + j;
                        cid[t][j] = (k < KK) ? a.kids[(int64_t)i0 * a.K + k] : 0;
                    }
#pragma unroll
                for (int t = 0; t < 4; ++t)
#pragma unroll
                    for (int j = 0; j < 8; ++j) v[t][j] = a.src[(int64_t)cid[t][j] * B + colc];
            } else {
                int pr[4];
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                    const int kb = kb0 + 16 * t;
                    pr[t] = (kb < KK) ? a.kids[(int64_t)i0 * a.K + (kb >> lg_pb)] : 0;
                }
                float nf[4][8], nm[4][8];
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                    const int64_t row = (int64_t)pr[t] + ((kb0 + 16 * t) & (a.par_block - 1));
#pragma unroll
                    for (int j = 0; j < 8; ++j) { nf[t][j] = a.src[(row + j) * B + colc]; nm[t][j] = a.src2[(row + j) * B + colc]; }
                }
#pragma unroll
                for (int t = 0; t < 4; ++t)
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        float f = nf[t][j];
                        if (!a.logspace) f = __logf(f);
                        v[t][j] = (pr[t] == 0) ? PCX_NEG_INF : f - fmaxf(nm[t][j], -3.0e38f);
                    }
            }
        };
        auto copy_theta = [&](int chunk, uint8_t* st) {
            const uint4* src = a.packed + ((size_t)m * n_chunks + chunk) * (TH_TILE / 16);
            for (int w = tid; w < TH_TILE / 16; w += NTH) cp_async16(st + 2 * SM_E_TILE + w * 16, src + w);
        };
        auto store_group = [&](uint8_t* st, int g, float* v, float mx) {
            const float mxc = (mx == PCX_NEG_INF) ? 0.0f : mx;
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = __expf(v[j] - mxc);
            uint8_t* dst = st + g * (SM_SAMPLES * 16) + ls * 16;
            store_split8(reinterpret_cast<uint4*>(dst), reinterpret_cast<uint4*>(dst + SM_E_TILE), v);
        };
        auto issue = [&](uint8_t* st, uint32_t acc_tmem) {       // one chunk into a fresh accumulator
            const uint32_t sa = smem_u32(st), sb = sa + 2 * SM_E_TILE;
#pragma unroll
            for (int ks = 0; ks < KC / 16; ++ks) {
                const uint64_t dEh = smem_desc(sa + ks * 2 * (SM_SAMPLES * 16), SM_SAMPLES * 16, 128);
                const uint64_t dEl = smem_desc(sa + SM_E_TILE + ks * 2 * (SM_SAMPLES * 16), SM_SAMPLES * 16, 128);
                const uint64_t dTh = smem_desc(sb + ks * 2 * (NB * 16), NB * 16, 128);
                const uint64_t dTl = smem_desc(sb + KG * NB * 16 + ks * 2 * (NB * 16), NB * 16, 128);
                mma_bf16_ss(acc_tmem, dEh, dTh, idesc, ks > 0 ? 1u : 0u);
                if (a.terms == 3) {
                    mma_bf16_ss(acc_tmem, dEh, dTl, idesc, 1u);
                    mma_bf16_ss(acc_tmem, dEl, dTh, idesc, 1u);
                }
            }
        };

        // ---- one pass over the table, 64 entries at a time -------------------------------------------------------
        // Every chunk is scaled by ITS OWN per-sample maximum m_c and multiplied into a fresh accumulator (two
        // accumulators alternate); the threads take chunk c - 1 out of tensor memory while the tensor core works on
        // chunk c and fold it into a running sum held in registers:
        //     M' = max(M, m_c),   acc = acc * exp(M - M') + D_c * exp(m_c - M').
        // The children are therefore gathered once (the gathers are what this kernel spends its time on), and long
        // sums are carried in fp32 registers with round-to-nearest additions.
        const int lq = warp & 3, c0 = (warp >> 2) * HC;
        float acc[HC];
#pragma unroll
        for (int j = 0; j < HC; ++j) acc[j] = 0.0f;
        float M = PCX_NEG_INF;                                   // running maximum of this thread's sample
        float m_prev = PCX_NEG_INF;                              // maximum of the chunk that is still in tensor memory
        bool failed = false;
        auto drain = [&](int c, float m_c) {                     // fold chunk c (accumulator c & 1) into acc
            if (!failed && !mbar_wait(&s_bar[c & 1], (ph[c & 1] + c / STAGES) & 1)) { failed = true; s_fail = 1; }
            tc_fence_after_sync();
            if (failed) return;
            const float Mn = fmaxf(M, m_c);
            const float so = (Mn == PCX_NEG_INF) ? 0.0f : __expf(M - Mn);
            const float sn = (Mn == PCX_NEG_INF) ? 0.0f : __expf(m_c - Mn);
#pragma unroll
            for (int p = 0; p < HC / 8; ++p) {
                float v[8];
                tmem_ld<8>(tmem + (uint32_t)((c & 1) * NB) + ((uint32_t)(lq * 32) << 16) + (uint32_t)(c0 + 8 * p), v);
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[8 * p + j] = acc[8 * p + j] * so + v[j] * sn;
            }
            M = Mn;
            tc_fence_before_sync();
        };
        for (int c = 0; c < n_chunks; ++c) {
            const int s = c % STAGES;
            uint8_t* st = smem + s * SM_STAGE;
            // stage s and accumulator s are free: chunk c - 2 was drained by every thread during iteration c - 1
            copy_theta(c, st);
            float v[4][8];
            load_groups4(c * KC + h * 8, v);
            float mx = PCX_NEG_INF;
#pragma unroll
            for (int t = 0; t < 4; ++t)
#pragma unroll
                for (int j = 0; j < 8; ++j) mx = fmaxf(mx, v[t][j]);
            s_part[s][h * SM_SAMPLES + ls] = mx;
            __syncthreads();
            mx = fmaxf(s_part[s][ls], s_part[s][SM_SAMPLES + ls]);
#pragma unroll
            for (int t = 0; t < 4; ++t) store_group(st, h + 2 * t, v[t], mx);
            cp_async_wait_all();
            fence_async_smem();
            __syncthreads();
            failed = failed || (s_fail != 0);
            if (tid == 0 && !failed) {
                tc_fence_after_sync();
                issue(st, tmem + (uint32_t)(s * NB));
                mma_commit(&s_bar[s]);
            }
            if (c > 0) drain(c - 1, m_prev);
            m_prev = mx;
        }
        drain(n_chunks - 1, m_prev);
#pragma unroll
        for (int s = 0; s < STAGES; ++s) ph[s] += (n_chunks - s + STAGES - 1) / STAGES;
        failed = failed || (s_fail != 0);

        // ---- epilogue: lane = sample, column = node; warps w and w + 4 split the nodes ----------------------------
        if (!failed) {
            const int es = lq * 32 + lane;                       // sample of this thread within the tile (= ls)
            const int b = b0 + es;
            const int64_t base_row = (int64_t)a.rows[i0];        // merged rows are consecutive in the value buffer
            if (b < B) {
#pragma unroll
                for (int j = 0; j < HC; ++j) {
                    const int64_t off = (base_row + c0 + j) * B + b;
                    float o;
                    if (!ELE) o = __logf(fmaxf(acc[j], 1e-24f)) + M;
                    else {
                        const float em = (a.fk != nullptr)
                            ? folded2(a.fk[(int64_t)i0 * a.cbs + c0 + j], a.nmars + b, B) : a.emars[off];
                        o = __logf(acc[j]) + M + em;
                        if (!a.logspace) o = __expf(o);
                    }
                    a.out[off] = o;
                }
            }
        }
        __syncthreads();
        if (s_fail != 0) break;
    }
    if (tid == 0 && s_fail != 0) atomicCAS(&g_tc_status, 0, 500 + s_fail);
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, TCOLS);
}

// Tables at most 64 deep (the common case for small blocks): one thread per sample, one chunk, no cross-thread
// reduction, 21 - 48 KB of shared memory.  A tile is a chain of dependent round trips (index table -> child rows ->
// tensor core -> stores), so the kernel is built to keep many tiles in flight per SM and to shorten the chain:
//  * NG (K groups of 8 held in registers: 4 for tables up to 32 deep, else 8) is a template parameter, so that the
//    32-deep forward instantiation fits eight CTAs on an SM (64 registers), the 32-deep element-flow ones five or
//    six (they also hold the NB element values), and the 64-deep ones four;
//  * the index pairs of a folded product layer are fetched ONE TILE AHEAD into shared memory (every thread of a
//    tile needs the same pairs), which takes their L2 round trip off the chain.
template <int NB, bool ELE, int NG>
constexpr int sm_small_ctas() { return (NG == 4 && !ELE) ? 8 : 4; }     // resident CTAs per SM (registers)

template <int NB, bool ELE, int NG>
__global__ void __launch_bounds__(SM_SAMPLES, sm_small_ctas<NB, ELE, NG>()) sum_sm_small_kernel(const SmArgs a, const int ng) {
    constexpr int TCOLS = NB < 32 ? 32 : NB;
    constexpr int NIDX = 64;                           // index pairs per tile: the table (FWD) or the NB outputs (ELE)
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ uint64_t s_bar;
    __shared__ uint32_t s_tmem;
    __shared__ int s_fail;
    __shared__ int2 s_fk[2][NIDX];

    const int tid = threadIdx.x, warp = tid >> 5;
    if (tid == 0) {
        mbar_init(&s_bar, 1);
        fence_mbar_init();
        s_fail = 0;
    }
    if (warp == 0) tmem_alloc(&s_tmem, TCOLS);

    const int B = a.B;
    const int KK = ELE ? a.K * a.par_block : a.K;
    const int lg_pb = ELE ? (31 - __clz(a.par_block)) : 0;
    const uint32_t idesc = idesc_bf16_f32(SM_SAMPLES, NB);
    const bool folded = a.fk != nullptr;
    const int n_idx = ELE ? NB : KK;                   // pairs per tile
    const int idx_stride = ELE ? a.cbs : a.K;
    // shared memory: E hi [ng][128][16 B], E lo, theta hi [ng][NB][16 B], theta lo
    uint8_t* e_hi = smem;
    uint8_t* e_lo = smem + ng * (SM_SAMPLES * 16);
    uint8_t* t_hi = smem + 2 * ng * (SM_SAMPLES * 16);
    uint8_t* t_lo = t_hi + ng * (NB * 16);

    if (folded && blockIdx.x < a.n_tiles && tid < n_idx)
        s_fk[0][tid] = a.fk[(int64_t)a.first_row[blockIdx.x / a.n_st] * idx_stride + tid];
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = s_tmem;
    uint32_t phase = 0;
    int cur = 0;

    for (int64_t tile = blockIdx.x; tile < a.n_tiles; tile += gridDim.x, cur ^= 1) {
        const int64_t m = tile / a.n_st;
        const int b0 = (int)(tile % a.n_st) * SM_SAMPLES;
        const int i0 = a.first_row[m];
        const int col = b0 + tid;
        const bool col_ok = col < B;
        const int colc = col_ok ? col : 0;
        const int2* fk = s_fk[cur];

        // the next tile's index pairs: requested now, parked in shared memory at the end of this tile
        const int64_t tile_n = tile + gridDim.x;
        int2 fk_next = make_int2(0, 0);
        const bool pre = folded && tile_n < a.n_tiles && tid < n_idx;
        if (pre) fk_next = a.fk[(int64_t)a.first_row[tile_n / a.n_st] * idx_stride + tid];

        // parameter tile: the first ng K groups of the hi half and of the lo half
        {
            const uint4* src = a.packed + (size_t)m * (2 * KG * NB);
            for (int w = tid; w < ng * NB; w += SM_SAMPLES) {
                cp_async16(t_hi + w * 16, src + w);
                cp_async16(t_lo + w * 16, src + KG * NB + w);
            }
        }
        // Values of this thread's sample for every table entry.  Entries without a child / parent (id 0) read row 0,
        // the dummy row, which holds "probability zero" by the buffers' contract (element_mars: -inf); no per-value
        // masking is needed there.  A sample beyond the batch reads column 0 and is never stored.
        float keep[NG][8];
        float mx = PCX_NEG_INF;
        const float* src_col = a.src + colc;
        const float* src2_col = ELE ? a.src2 + colc : nullptr;
#pragma unroll
        for (int g = 0; g < NG; ++g) {
            if (g < ng) {
                const int kb = g * 8;
                if (!ELE && folded) {
                    int2 r[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) r[j] = (kb + j < KK) ? fk[kb + j] : make_int2(0, 0);
#pragma unroll
                    for (int j = 0; j < 8; ++j) keep[g][j] = folded2(r[j], a.nmars + colc, B);
                } else if (!ELE) {
                    int cid[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) cid[j] = (kb + j < KK) ? a.kids[(int64_t)i0 * a.K + kb + j] : 0;
#pragma unroll
                    for (int j = 0; j < 8; ++j) keep[g][j] = src_col[(int64_t)cid[j] * B];
                } else {
                    const int pr = (kb < KK) ? a.kids[(int64_t)i0 * a.K + (kb >> lg_pb)] : 0;
                    const int64_t row = (int64_t)pr + (kb & (a.par_block - 1));
                    float nf[8], nm[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) { nf[j] = src_col[(row + j) * B]; nm[j] = src2_col[(row + j) * B]; }
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        float f = nf[j];
                        if (!a.logspace) f = __logf(f);                              // log(0) = -inf
                        // flow / value in the log domain; (-inf) - (-inf) must read as -inf, hence the clamp
                        keep[g][j] = (pr == 0) ? PCX_NEG_INF : f - fmaxf(nm[j], -3.0e38f);
                    }
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) mx = fmaxf(mx, keep[g][j]);
            }
        }
        const float mxc = (mx == PCX_NEG_INF) ? 0.0f : mx;          // exp(-inf - 0) = 0: no per-value masking either
#pragma unroll
        for (int g = 0; g < NG; ++g) {
            if (g < ng) {
#pragma unroll
                for (int j = 0; j < 8; ++j) keep[g][j] = __expf(keep[g][j] - mxc);
                store_split8(reinterpret_cast<uint4*>(e_hi + g * (SM_SAMPLES * 16) + tid * 16),
                             reinterpret_cast<uint4*>(e_lo + g * (SM_SAMPLES * 16) + tid * 16), keep[g]);
            }
        }
        cp_async_wait_all();
        fence_async_smem();
        __syncthreads();
        if (tid == 0) {
            tc_fence_after_sync();
            for (int ks = 0; ks < ng / 2; ++ks) {
                const uint64_t dEh = smem_desc(smem_u32(e_hi) + ks * 2 * (SM_SAMPLES * 16), SM_SAMPLES * 16, 128);
                const uint64_t dEl = smem_desc(smem_u32(e_lo) + ks * 2 * (SM_SAMPLES * 16), SM_SAMPLES * 16, 128);
                const uint64_t dTh = smem_desc(smem_u32(t_hi) + ks * 2 * (NB * 16), NB * 16, 128);
                const uint64_t dTl = smem_desc(smem_u32(t_lo) + ks * 2 * (NB * 16), NB * 16, 128);
                mma_bf16_ss(tmem, dEh, dTh, idesc, ks > 0 ? 1u : 0u);
                if (a.terms == 3) {
                    mma_bf16_ss(tmem, dEh, dTl, idesc, 1u);
                    mma_bf16_ss(tmem, dEl, dTh, idesc, 1u);
                }
            }
            mma_commit(&s_bar);
        }
        const int64_t base = (int64_t)a.rows[i0] * B + colc;
        // one thread waits for the tensor core, the others sleep in the barrier (128 spinning threads would take
        // issue slots from the other CTAs of the SM)
        if (tid == 0 && !mbar_wait(&s_bar, phase & 1)) s_fail = 2;
        phase += 1;
        __syncthreads();
        const bool failed = s_fail != 0;
        tc_fence_after_sync();
        if (!failed) {
            float* out_col = a.out + base;
            const float* em_col = ELE ? a.emars + base : nullptr;
#pragma unroll
            for (int p = 0; p < NB / 8; ++p) {
                float v[8], em[8];
                if (ELE) {
                    if (folded) {
#pragma unroll
                        for (int j = 0; j < 8; ++j) em[j] = folded2(fk[8 * p + j], a.nmars + colc, B);
                    } else {
#pragma unroll
                        for (int j = 0; j < 8; ++j) em[j] = em_col[(int64_t)(8 * p + j) * B];
                    }
                }
                tmem_ld<8>(tmem + ((uint32_t)(warp * 32) << 16) + (uint32_t)(8 * p), v);    // warp-wide: every lane takes part
                if (!col_ok) continue;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    // log(0) = -inf and -inf + x = -inf take care of empty sums, zero shifts and zero element values
                    float o;
                    if (!ELE) o = __logf(fmaxf(v[j], 1e-24f)) + mx;
                    else {
                        o = __logf(v[j]) + mx + em[j];
                        if (!a.logspace) o = __expf(o);
                    }
                    out_col[(int64_t)(8 * p + j) * B] = o;
                }
            }
        }
        if (pre) s_fk[cur ^ 1][tid] = fk_next;
        tc_fence_before_sync();
        __syncthreads();
        if (s_fail != 0) break;
    }
    if (tid == 0 && s_fail != 0) atomicCAS(&g_tc_status, 0, 510 + s_fail);
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, TCOLS);
}

// Parameter tiles of the sample-major kernels.  One thread per 16-byte (hi) vector: (merged row m, chunk, K group g,
// node r of the tile).  mode 0: theta[n, k] = params[pids[i, k] + n]; mode 1 (element flows, transposed):
// theta[c, (p, n)] = params[parpids[j, p] + c * par_block + n]; i / j = first_row[m] + r / block, n / c = r % block.
__global__ void pack_sm_kernel(uint4* __restrict__ out, const float* __restrict__ params,
                               const int32_t* __restrict__ first_row, const int32_t* __restrict__ kids,
                               const int32_t* __restrict__ kpar, int64_t n_vec, int NB, int block, int K,
                               int par_block, int n_chunks, int mode) {
    int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= n_vec) return;
    const int r = (int)(t % NB);
    const int g = (int)((t / NB) % KG);
    const int64_t tile = t / ((int64_t)NB * KG);
    const int chunk = (int)(tile % n_chunks);
    const int64_t m = tile / n_chunks;
    const int64_t i = (int64_t)first_row[m] + r / block;
    const int n = r % block;
    const int kb = chunk * KC + g * 8;
    float v[8];
    if (mode == 0) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int k = kb + j;
            v[j] = (k < K) ? params[(int64_t)kpar[i * K + k] + n] : 0.0f;
        }
    } else {
        const int KK = K * par_block;
        const int p = kb / par_block, np = kb % par_block;
        const int pr = (kb < KK) ? kids[i * K + p] : 0;
#pragma unroll
        for (int j = 0; j < 8; ++j)
            v[j] = (pr != 0) ? params[(int64_t)kpar[i * K + p] + (int64_t)n * par_block + np + j] : 0.0f;
    }
    uint4* base = out + tile * (2 * KG * NB);
    store_split8(base + g * NB + r, base + KG * NB + g * NB + r, v);
}

// ---- parameter flows of small blocks ------------------------------------------------------------------------------
// pf[n, k] += theta[n, k] * sum_b exp(flow[n,b] - value[n,b] - shift[b]) * exp(child[k,b] + shift[b]).
// The contraction runs over the batch; the MMA's M dimension is the EDGE index k (128 per tile, rows beyond the table
// are zero), N the NB nodes of the merged row.  A CTA (128 threads, four per SM, as sum_par_tc_kernel) walks its share
// of the batch in 32-sample slices; shift[b] is the maximum over the NB nodes.
struct SmParArgs {
    float* param_flows;
    const float* node_flows;
    const float* node_mars;
    const float* element_mars;
    const float* params;
    const int32_t* first_row;   // [n_merged]
    const int32_t* nids;
    const int32_t* cids;        // [n, K]
    const int32_t* pids;
    const int32_t* pfids;
    int K, block, B, logspace, terms, chunks_per_cta;
    const int2* fk;             // product layer folded in: [n, K] pairs of child rows of node_mars (see SmArgs)
};

template <int NB>
__global__ void __launch_bounds__(PNTH, 4) sum_sm_par_kernel(const SmParArgs a) {
    constexpr int NSLAB = NB * 16 + 16;                // padded slab of the node-side tile
    constexpr int N_TILE = PKG * NSLAB;
    constexpr int TCOLS = NB < 32 ? 32 : NB;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ uint64_t s_bar[STAGES];
    __shared__ uint32_t s_tmem;
    __shared__ __align__(16) float s_part[PNTH / 32][PKC];
    __shared__ int s_fail;
    constexpr int STAGE = 2 * X_TILE + 2 * N_TILE;     // edge-side tile (128 rows, as X_TILE) + node-side tile

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int64_t m = blockIdx.x;
    const int e0 = blockIdx.y * BM;
    const int i0 = a.first_row[m];
    const int B = a.B;
    const int total_chunks = (B + PKC - 1) / PKC;
    const int c_begin = blockIdx.z * a.chunks_per_cta;
    const int c_end = min(total_chunks, c_begin + a.chunks_per_cta);

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) mbar_init(&s_bar[s], 1);
        fence_mbar_init();
        s_fail = 0;
    }
    if (warp == 0) tmem_alloc(&s_tmem, TCOLS);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = s_tmem;

    const int g = tid & (PKG - 1), rb = tid / PKG;     // 8-sample group g of the slice, rows rb + 32 j
    const uint32_t idesc = idesc_bf16_f32(BM, NB);
    const int64_t nid0 = a.nids[i0];                   // the merged row's nodes are consecutive
    int cid[4];                                        // this thread's four edge rows
    int2 ch[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int e = e0 + rb + 32 * j;
        cid[j] = (e < a.K) ? a.cids[(int64_t)i0 * a.K + e] : 0;
        ch[j] = (a.fk != nullptr && cid[j] != 0) ? a.fk[(int64_t)i0 * a.K + e] : make_int2(0, 0);
    }
    bool failed = false;

    for (int c = c_begin; c < c_end; ++c) {
        const int it = c - c_begin, s = it % STAGES, use = it / STAGES;
        uint8_t* st = smem + s * STAGE;
        const int bb = c * PKC + g * 8;
        const bool b_ok = bb < B;                      // B is a multiple of 8 here
        const int bbc = b_ok ? bb : 0;

        float y[4][8], x[NB / 32][8];
        if (a.fk != nullptr) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {               // edge side, folded: sum of the product's two child rows
                const float* r0p = a.node_mars + (int64_t)ch[j].x * B + bbc;
                const float* r1p = a.node_mars + (int64_t)ch[j].y * B + bbc;
                const float4 p0 = *reinterpret_cast<const float4*>(r0p), p1 = *reinterpret_cast<const float4*>(r0p + 4);
                const float4 q0 = *reinterpret_cast<const float4*>(r1p), q1 = *reinterpret_cast<const float4*>(r1p + 4);
                const bool any = (ch[j].x | ch[j].y) != 0;
                y[j][0] = any ? p0.x + q0.x : PCX_NEG_INF; y[j][1] = any ? p0.y + q0.y : PCX_NEG_INF;
                y[j][2] = any ? p0.z + q0.z : PCX_NEG_INF; y[j][3] = any ? p0.w + q0.w : PCX_NEG_INF;
                y[j][4] = any ? p1.x + q1.x : PCX_NEG_INF; y[j][5] = any ? p1.y + q1.y : PCX_NEG_INF;
                y[j][6] = any ? p1.z + q1.z : PCX_NEG_INF; y[j][7] = any ? p1.w + q1.w : PCX_NEG_INF;
            }
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) {               // edge side: element values (row 0 = dummy = -inf)
                const float4 q0 = *reinterpret_cast<const float4*>(a.element_mars + (int64_t)cid[j] * B + bbc);
                const float4 q1 = *reinterpret_cast<const float4*>(a.element_mars + (int64_t)cid[j] * B + bbc + 4);
                y[j][0] = q0.x; y[j][1] = q0.y; y[j][2] = q0.z; y[j][3] = q0.w;
                y[j][4] = q1.x; y[j][5] = q1.y; y[j][6] = q1.z; y[j][7] = q1.w;
            }
        }
#pragma unroll
        for (int j = 0; j < NB / 32; ++j) {             // node side: log(flow / value)
            const int64_t off = (nid0 + rb + 32 * j) * B + bbc;
            const float4 f0 = *reinterpret_cast<const float4*>(a.node_flows + off);
            const float4 f1 = *reinterpret_cast<const float4*>(a.node_flows + off + 4);
            const float4 m0 = *reinterpret_cast<const float4*>(a.node_mars + off);
            const float4 m1 = *reinterpret_cast<const float4*>(a.node_mars + off + 4);
            const float nf[8] = {f0.x, f0.y, f0.z, f0.w, f1.x, f1.y, f1.z, f1.w};
            const float nm[8] = {m0.x, m0.y, m0.z, m0.w, m1.x, m1.y, m1.z, m1.w};
#pragma unroll
            for (int t = 0; t < 8; ++t) {
                float f = nf[t];
                if (!a.logspace) f = __logf(f);
                x[j][t] = b_ok ? f - fmaxf(nm[t], -3.0e38f) : PCX_NEG_INF;
            }
        }
        float pm[8];
#pragma unroll
        for (int t = 0; t < 8; ++t) {
            float mm = x[0][t];
#pragma unroll
            for (int j = 1; j < NB / 32; ++j) mm = fmaxf(mm, x[j][t]);
#pragma unroll
            for (int o = PKG; o < 32; o <<= 1) mm = fmaxf(mm, __shfl_xor_sync(0xffffffffu, mm, o));
            pm[t] = mm;
        }
        if (lane < PKG) {
            float4* dst = reinterpret_cast<float4*>(&s_part[warp][lane * 8]);
            dst[0] = make_float4(pm[0], pm[1], pm[2], pm[3]);
            dst[1] = make_float4(pm[4], pm[5], pm[6], pm[7]);
        }
        if (it >= STAGES && !failed && !mbar_wait(&s_bar[s], (uint32_t)((use - 1) & 1))) { failed = true; s_fail = 1; }
        __syncthreads();
        float sh[8];
        {
            const float4 p0 = *reinterpret_cast<const float4*>(&s_part[0][g * 8]);
            const float4 p1 = *reinterpret_cast<const float4*>(&s_part[0][g * 8 + 4]);
            sh[0] = p0.x; sh[1] = p0.y; sh[2] = p0.z; sh[3] = p0.w; sh[4] = p1.x; sh[5] = p1.y; sh[6] = p1.z; sh[7] = p1.w;
#pragma unroll
            for (int w = 1; w < PNTH / 32; ++w) {
                const float4 q0 = *reinterpret_cast<const float4*>(&s_part[w][g * 8]);
                const float4 q1 = *reinterpret_cast<const float4*>(&s_part[w][g * 8 + 4]);
                sh[0] = fmaxf(sh[0], q0.x); sh[1] = fmaxf(sh[1], q0.y); sh[2] = fmaxf(sh[2], q0.z); sh[3] = fmaxf(sh[3], q0.w);
                sh[4] = fmaxf(sh[4], q1.x); sh[5] = fmaxf(sh[5], q1.y); sh[6] = fmaxf(sh[6], q1.z); sh[7] = fmaxf(sh[7], q1.w);
            }
        }
        uint8_t* yhi = st;
        uint8_t* ylo = st + X_TILE;
        uint8_t* xhi = st + 2 * X_TILE;
        uint8_t* xlo = st + 2 * X_TILE + N_TILE;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
#pragma unroll
            for (int t = 0; t < 8; ++t)       // a sample without any flow (shift -inf) contributes nothing
                y[j][t] = (sh[t] == PCX_NEG_INF || !b_ok) ? 0.0f : fminf(__expf(y[j][t] + sh[t]), 3.0e38f);
            const int o = g * XSLAB + (rb + 32 * j) * 16;
            store_split8(reinterpret_cast<uint4*>(yhi + o), reinterpret_cast<uint4*>(ylo + o), y[j]);
        }
#pragma unroll
        for (int j = 0; j < NB / 32; ++j) {
#pragma unroll
            for (int t = 0; t < 8; ++t) x[j][t] = (sh[t] == PCX_NEG_INF) ? 0.0f : __expf(x[j][t] - sh[t]);
            const int o = g * NSLAB + (rb + 32 * j) * 16;
            store_split8(reinterpret_cast<uint4*>(xhi + o), reinterpret_cast<uint4*>(xlo + o), x[j]);
        }
        fence_async_smem();
        __syncthreads();
        failed = failed || (s_fail != 0);
        if (tid == 0 && !failed) {
            tc_fence_after_sync();
            const uint32_t sa = smem_u32(st);
            issue_stage<XSLAB, NSLAB, PKC>(tmem, sa, sa + 2 * X_TILE, idesc, it == 0, a.terms);
            mma_commit(&s_bar[s]);
        }
    }

    const int n_it = c_end - c_begin;
    if (n_it > 0) {
        const int il = n_it - 1;
        if (tid == 0 && !failed && !mbar_wait(&s_bar[il % STAGES], (uint32_t)((il / STAGES) & 1))) s_fail = 2;
    }
    __syncthreads();
    failed = failed || (s_fail != 0);
    tc_fence_after_sync();
    if (!failed && n_it > 0) {
        const int e = e0 + warp * 32 + lane;            // this thread's edge (TMEM lane)
        const bool e_ok = e < a.K && a.cids[(int64_t)i0 * a.K + min(e, a.K - 1)] != 0;
#pragma unroll 1
        for (int p = 0; p < NB / 8; ++p) {
            float v[8];
            tmem_ld<8>(tmem + ((uint32_t)(warp * 32) << 16) + (uint32_t)(8 * p), v);    // warp-wide
            if (!e_ok) continue;
            const int n0 = 8 * p;                       // eight consecutive nodes lie in one block (blocks >= 8 nodes)
            const int64_t i = (int64_t)i0 + n0 / a.block;
            const int nn = n0 % a.block;
            const float* par = a.params + (int64_t)a.pids[i * a.K + e] + nn;
            float* pf = a.param_flows + (int64_t)a.pfids[i * a.K + e] + nn;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float f = par[j] * v[j];
                if (f != 0.0f) atomicAdd(pf + j, f);
            }
        }
    }
    if (failed && tid == 0) atomicCAS(&g_tc_status, 0, 520 + s_fail);
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, TCOLS);
}

// Parameter flows of 32-node blocks whose tables are at most 32 deep (one child block per sum block: the bulk of a
// block-sparse Poon-Domingos layer).  One such table fills a quarter of the 128 edge rows of an MMA tile, so FOUR
// merged rows share a tile: edge rows 32 j .. 32 j + 31 are the edges of row j, node columns 32 j .. 32 j + 31 its
// nodes, and only the four diagonal 32 x 32 blocks of the 128 x 128 product are read back.  The tensor core does
// four times the useful multiplications (it idles anyway); the threads, whose loads and exponentials are what this
// kernel spends its time on, fill both operand tiles completely instead of a quarter of one.
__global__ void __launch_bounds__(PNTH, 3) sum_sm_par_quad_kernel(const SmParArgs a, const int64_t n_merged) {
    constexpr int QN = 32;                             // nodes (and at most edges) per merged row
    constexpr int STAGE = 4 * X_TILE;                  // edge side hi, lo; node side hi, lo (128 rows each)
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ uint64_t s_bar[STAGES];
    __shared__ uint32_t s_tmem;
    __shared__ __align__(16) float s_part[PNTH / 32][4][PKC];      // [warp][row j][sample of the slice]
    __shared__ int s_fail;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int64_t m0 = (int64_t)blockIdx.x * 4;
    const int B = a.B;
    const int total_chunks = (B + PKC - 1) / PKC;
    const int c_begin = blockIdx.z * a.chunks_per_cta;
    const int c_end = min(total_chunks, c_begin + a.chunks_per_cta);

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) mbar_init(&s_bar[s], 1);
        fence_mbar_init();
        s_fail = 0;
    }
    if (warp == 0) tmem_alloc(&s_tmem, 128);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = s_tmem;

    const int g = tid & (PKG - 1), rb = tid / PKG;     // 8-sample group g of the slice; edge rb / node rb of every row j
    const uint32_t idesc = idesc_bf16_f32(BM, 128);
    int2 ch[4];                                        // this thread's edge of the four rows (folded: two child rows)
    int cid[4];
    int64_t nrow[4];                                   // this thread's node of the four rows
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const bool ok = m0 + j < n_merged;
        const int i0 = ok ? a.first_row[m0 + j] : 0;
        cid[j] = (ok && rb < a.K) ? a.cids[(int64_t)i0 * a.K + rb] : 0;
        ch[j] = (a.fk != nullptr && cid[j] != 0) ? a.fk[(int64_t)i0 * a.K + rb] : make_int2(0, 0);
        nrow[j] = ok ? (int64_t)a.nids[i0] + rb : -1;
    }
    bool failed = false;

    for (int c = c_begin; c < c_end; ++c) {
        const int it = c - c_begin, s = it % STAGES, use = it / STAGES;
        uint8_t* st = smem + s * STAGE;
        const int bb = c * PKC + g * 8;
        const bool b_ok = bb < B;                      // B is a multiple of 8 here
        const int bbc = b_ok ? bb : 0;

        float y[4][8], x[4][8];
#pragma unroll
        for (int j = 0; j < 4; ++j) {                   // edge side
            if (a.fk != nullptr) {                      // folded: sum of the product's two child rows
                const float* r0p = a.node_mars + (int64_t)ch[j].x * B + bbc;
                const float* r1p = a.node_mars + (int64_t)ch[j].y * B + bbc;
                const float4 p0 = *reinterpret_cast<const float4*>(r0p), p1 = *reinterpret_cast<const float4*>(r0p + 4);
                const float4 q0 = *reinterpret_cast<const float4*>(r1p), q1 = *reinterpret_cast<const float4*>(r1p + 4);
                const bool any = (ch[j].x | ch[j].y) != 0;
                y[j][0] = any ? p0.x + q0.x : PCX_NEG_INF; y[j][1] = any ? p0.y + q0.y : PCX_NEG_INF;
                y[j][2] = any ? p0.z + q0.z : PCX_NEG_INF; y[j][3] = any ? p0.w + q0.w : PCX_NEG_INF;
                y[j][4] = any ? p1.x + q1.x : PCX_NEG_INF; y[j][5] = any ? p1.y + q1.y : PCX_NEG_INF;
                y[j][6] = any ? p1.z + q1.z : PCX_NEG_INF; y[j][7] = any ? p1.w + q1.w : PCX_NEG_INF;
            } else {                                    // element values (row 0 = dummy = -inf)
                const float4 q0 = *reinterpret_cast<const float4*>(a.element_mars + (int64_t)cid[j] * B + bbc);
                const float4 q1 = *reinterpret_cast<const float4*>(a.element_mars + (int64_t)cid[j] * B + bbc + 4);
                y[j][0] = q0.x; y[j][1] = q0.y; y[j][2] = q0.z; y[j][3] = q0.w;
                y[j][4] = q1.x; y[j][5] = q1.y; y[j][6] = q1.z; y[j][7] = q1.w;
            }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {                   // node side: log(flow / value)
            const bool ok = nrow[j] >= 0 && b_ok;
            const int64_t off = (nrow[j] >= 0 ? nrow[j] : 0) * B + bbc;
            const float4 f0 = *reinterpret_cast<const float4*>(a.node_flows + off);
            const float4 f1 = *reinterpret_cast<const float4*>(a.node_flows + off + 4);
            const float4 m0v = *reinterpret_cast<const float4*>(a.node_mars + off);
            const float4 m1v = *reinterpret_cast<const float4*>(a.node_mars + off + 4);
            const float nf[8] = {f0.x, f0.y, f0.z, f0.w, f1.x, f1.y, f1.z, f1.w};
            const float nm[8] = {m0v.x, m0v.y, m0v.z, m0v.w, m1v.x, m1v.y, m1v.z, m1v.w};
#pragma unroll
            for (int t = 0; t < 8; ++t) {
                float f = nf[t];
                if (!a.logspace) f = __logf(f);
                x[j][t] = ok ? f - fmaxf(nm[t], -3.0e38f) : PCX_NEG_INF;
            }
        }
        // shift of row j and sample t: the maximum over the row's 32 nodes (eight per warp, then across the warps)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float pm[8];
#pragma unroll
            for (int t = 0; t < 8; ++t) {
                float mm = x[j][t];
#pragma unroll
                for (int o = PKG; o < 32; o <<= 1) mm = fmaxf(mm, __shfl_xor_sync(0xffffffffu, mm, o));
                pm[t] = mm;
            }
            if (lane < PKG) {
                float4* dst = reinterpret_cast<float4*>(&s_part[warp][j][lane * 8]);
                dst[0] = make_float4(pm[0], pm[1], pm[2], pm[3]);
                dst[1] = make_float4(pm[4], pm[5], pm[6], pm[7]);
            }
        }
        if (it >= STAGES && !failed && !mbar_wait(&s_bar[s], (uint32_t)((use - 1) & 1))) { failed = true; s_fail = 1; }
        __syncthreads();
        uint8_t* yhi = st;
        uint8_t* ylo = st + X_TILE;
        uint8_t* xhi = st + 2 * X_TILE;
        uint8_t* xlo = st + 3 * X_TILE;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float sh[8];
            {
                const float4 p0 = *reinterpret_cast<const float4*>(&s_part[0][j][g * 8]);
                const float4 p1 = *reinterpret_cast<const float4*>(&s_part[0][j][g * 8 + 4]);
                sh[0] = p0.x; sh[1] = p0.y; sh[2] = p0.z; sh[3] = p0.w; sh[4] = p1.x; sh[5] = p1.y; sh[6] = p1.z; sh[7] = p1.w;
#pragma unroll
                for (int w = 1; w < PNTH / 32; ++w) {
                    const float4 q0 = *reinterpret_cast<const float4*>(&s_part[w][j][g * 8]);
                    const float4 q1 = *reinterpret_cast<const float4*>(&s_part[w][j][g * 8 + 4]);
                    sh[0] = fmaxf(sh[0], q0.x); sh[1] = fmaxf(sh[1], q0.y); sh[2] = fmaxf(sh[2], q0.z); sh[3] = fmaxf(sh[3], q0.w);
                    sh[4] = fmaxf(sh[4], q1.x); sh[5] = fmaxf(sh[5], q1.y); sh[6] = fmaxf(sh[6], q1.z); sh[7] = fmaxf(sh[7], q1.w);
                }
            }
#pragma unroll
            for (int t = 0; t < 8; ++t) {     // a sample without any flow (shift -inf) contributes nothing
                y[j][t] = (sh[t] == PCX_NEG_INF || !b_ok) ? 0.0f : fminf(__expf(y[j][t] + sh[t]), 3.0e38f);
                x[j][t] = (sh[t] == PCX_NEG_INF) ? 0.0f : __expf(x[j][t] - sh[t]);
            }
            const int o = g * XSLAB + (rb + 32 * j) * 16;
            store_split8(reinterpret_cast<uint4*>(yhi + o), reinterpret_cast<uint4*>(ylo + o), y[j]);
            store_split8(reinterpret_cast<uint4*>(xhi + o), reinterpret_cast<uint4*>(xlo + o), x[j]);
        }
        fence_async_smem();
        __syncthreads();
        failed = failed || (s_fail != 0);
        if (tid == 0 && !failed) {
            tc_fence_after_sync();
            const uint32_t sa = smem_u32(st);
            issue_stage<XSLAB, XSLAB, PKC>(tmem, sa, sa + 2 * X_TILE, idesc, it == 0, a.terms);
            mma_commit(&s_bar[s]);
        }
    }

    const int n_it = c_end - c_begin;
    if (n_it > 0) {
        const int il = n_it - 1;
        if (tid == 0 && !failed && !mbar_wait(&s_bar[il % STAGES], (uint32_t)((il / STAGES) & 1))) s_fail = 2;
    }
    __syncthreads();
    failed = failed || (s_fail != 0);
    tc_fence_after_sync();
    if (!failed && n_it > 0) {
        // TMEM lane = edge row: warp w holds the edges of row w; its diagonal block is columns 32 w .. 32 w + 31
        const int e = lane;
        const bool row_ok = m0 + warp < n_merged;
        const int i0 = row_ok ? a.first_row[m0 + warp] : 0;
        const bool e_ok = row_ok && e < a.K && a.cids[(int64_t)i0 * a.K + min(e, a.K - 1)] != 0;
#pragma unroll 1
        for (int p = 0; p < QN / 8; ++p) {
            float v[8];
            tmem_ld<8>(tmem + ((uint32_t)(warp * 32) << 16) + (uint32_t)(warp * QN + 8 * p), v);    // warp-wide
            if (!e_ok) continue;
            const int n0 = 8 * p;                       // eight consecutive nodes lie in one block (blocks >= 8 nodes)
            const int64_t i = (int64_t)i0 + n0 / a.block;
            const int nn = n0 % a.block;
            const float* par = a.params + (int64_t)a.pids[i * a.K + e] + nn;
            float* pf = a.param_flows + (int64_t)a.pfids[i * a.K + e] + nn;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float f = par[j] * v[j];
                if (f != 0.0f) atomicAdd(pf + j, f);
            }
        }
    }
    if (failed && tid == 0) atomicCAS(&g_tc_status, 0, 530 + s_fail);
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, 128);
}

// All sample-major tables of a circuit in one launch: a device array of jobs, the job of a vector is found by binary
// search over vec_begin (the running sum of the jobs' vector counts).
struct SmPackJob {
    uint4* out;
    const int32_t* first_row;
    const int32_t* kids;
    const int32_t* kpar;
    int64_t vec_begin;
    int32_t nb, block, K, par_block, n_chunks, mode;
};
static_assert(sizeof(SmPackJob) == 64, "matches PcxSmPackJob");

__global__ void pack_sm_jobs_kernel(const SmPackJob* __restrict__ jobs, int n_jobs, int64_t n_vec,
                                    const float* __restrict__ params) {
    int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= n_vec) return;
    int lo = 0, hi = n_jobs - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (jobs[mid].vec_begin <= t) lo = mid; else hi = mid - 1;
    }
    const SmPackJob a = jobs[lo];
    t -= a.vec_begin;
    const int NB = a.nb;
    const int r = (int)(t % NB);
    const int g = (int)((t / NB) % KG);
    const int64_t tile = t / ((int64_t)NB * KG);
    const int chunk = (int)(tile % a.n_chunks);
    const int64_t m = tile / a.n_chunks;
    const int64_t i = (int64_t)a.first_row[m] + r / a.block;
    const int n = r % a.block;
    const int kb = chunk * KC + g * 8;
    float v[8];
    if (a.mode == 0) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int k = kb + j;
            v[j] = (k < a.K) ? params[(int64_t)a.kpar[i * a.K + k] + n] : 0.0f;
        }
    } else {
        const int KK = a.K * a.par_block;
        const int p = kb / a.par_block, np = kb % a.par_block;
        const int pr = (kb < KK) ? a.kids[i * a.K + p] : 0;
#pragma unroll
        for (int j = 0; j < 8; ++j)
            v[j] = (pr != 0) ? params[(int64_t)a.kpar[i * a.K + p] + (int64_t)n * a.par_block + np + j] : 0.0f;
    }
    uint4* base = a.out + tile * (2 * KG * NB);
    store_split8(base + g * NB + r, base + KG * NB + g * NB + r, v);
}

template <int NB, bool ELE>
int launch_sm(const SmArgs& a, cudaStream_t st) {
    static PcxOnce done;
    static int sms = 0;
    if (!done) {
        cudaError_t e = cudaFuncSetAttribute(sum_sm_kernel<NB, ELE>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(sum_sm_small_kernel<NB, ELE, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(sum_sm_small_kernel<NB, ELE, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
        if (e != cudaSuccess) return (int)e;
        int dev = 0;
        e = cudaGetDevice(&dev);
        if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess) return (int)e;
        done = true;
    }
    const int depth = ELE ? a.K * a.par_block : a.K;
    if (depth <= KC) {
        const int ng = 2 * (int)pcx_cdiv(depth, 16);                    // K groups actually used (pairs: one MMA step)
        const int bytes = 2 * ng * (SM_SAMPLES * 16) + 2 * ng * (NB * 16) + 1024;
        const int per_sm = ng <= 4 ? sm_small_ctas<NB, ELE, 4>() : sm_small_ctas<NB, ELE, 8>();
        const int64_t grid = a.n_tiles < per_sm * (int64_t)sms ? a.n_tiles : per_sm * (int64_t)sms;
        if (ng <= 4) sum_sm_small_kernel<NB, ELE, 4><<<(unsigned)grid, SM_SAMPLES, bytes, st>>>(a, ng);
        else sum_sm_small_kernel<NB, ELE, 8><<<(unsigned)grid, SM_SAMPLES, bytes, st>>>(a, ng);
        PCX_LAUNCH_CHECK();
        return 0;
    }
    const int64_t grid = a.n_tiles < 2 * (int64_t)sms ? a.n_tiles : 2 * (int64_t)sms;
    sum_sm_kernel<NB, ELE><<<(unsigned)grid, NTH, SMEM_BYTES, st>>>(a);
    PCX_LAUNCH_CHECK();
    return 0;
}

}  // namespace

extern "C" {

int64_t pcx_sm_packed_bytes(int64_t n_merged, int depth, int nb) {
    return n_merged * pcx_cdiv(depth, KC) * 2 * KG * nb * 16;
}

int pcx_pack_sm_params(void* packed, const float* params, const int32_t* first_row, const int32_t* kids,
                       const int32_t* kpar, int64_t n_merged, int nb, int block, int K, int par_block, int mode,
                       void* stream) {
    if (n_merged <= 0) return 0;
    if ((nb != 32 && nb != 64) || block <= 0 || nb % block != 0 || (mode != 0 && mode != 1)) return -1;
    if (mode == 1 && par_block % 8 != 0) return -1;
    const int depth = mode == 0 ? K : K * par_block;
    const int n_chunks = (int)pcx_cdiv(depth, KC);
    const int64_t n_vec = n_merged * n_chunks * KG * nb;
    pack_sm_kernel<<<(unsigned)pcx_cdiv(n_vec, 256), 256, 0, (cudaStream_t)stream>>>(
        reinterpret_cast<uint4*>(packed), params, first_row, kids, kpar, n_vec, nb, block, K, par_block, n_chunks, mode);
    PCX_LAUNCH_CHECK();
    return 0;
}

int pcx_sum_bwd_par_sm(float* param_flows, const float* node_flows, const float* node_mars, const float* element_mars,
                       const float* params, const int32_t* first_row, const int32_t* nids, const int32_t* cids,
                       const int32_t* pids, const int32_t* pfids, const int32_t* fk, int64_t n_merged, int nb,
                       int block, int K, int B, int logspace, void* stream) {
    if (n_merged <= 0 || B <= 0) return 0;
    if ((nb != 32 && nb != 64) || block < 8 || nb % block != 0 || K <= 0 || B % 8 != 0) return -1;
    if (fk == nullptr && element_mars == nullptr) return -1;
    SmParArgs a{param_flows, node_flows, node_mars, element_mars, params, first_row, nids, cids, pids, pfids,
                K, block, B, logspace, (g_sum_mode == 2) ? 1 : 3, 1, reinterpret_cast<const int2*>(fk)};
    const int total_chunks = (int)pcx_cdiv(B, PKC);
    if (nb == 32 && K <= 32) {                                  // four merged rows per tile
        const int64_t quads = pcx_cdiv(n_merged, 4);
        int64_t splits = pcx_cdiv(6 * 148, quads);              // about two waves of three CTAs per SM
        if (splits > total_chunks) splits = total_chunks;
        if (splits < 1) splits = 1;
        a.chunks_per_cta = (int)pcx_cdiv(total_chunks, splits);
        dim3 grid((unsigned)quads, 1, (unsigned)pcx_cdiv(total_chunks, a.chunks_per_cta));
        const int smem = STAGES * 4 * X_TILE + 1024;
        static PcxOnce doneq;
        if (!doneq) {
            cudaError_t e = cudaFuncSetAttribute(sum_sm_par_quad_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
            if (e != cudaSuccess) return (int)e;
            doneq = true;
        }
        sum_sm_par_quad_kernel<<<grid, PNTH, smem, (cudaStream_t)stream>>>(a, n_merged);
        PCX_LAUNCH_CHECK();
        return 0;
    }
    const int64_t base = n_merged * pcx_cdiv(K, BM);
    int64_t splits = pcx_cdiv(8 * 148, base);                  // about two waves of four CTAs per SM
    if (splits > total_chunks) splits = total_chunks;
    if (splits < 1) splits = 1;
    a.chunks_per_cta = (int)pcx_cdiv(total_chunks, splits);
    dim3 grid((unsigned)n_merged, (unsigned)pcx_cdiv(K, BM), (unsigned)pcx_cdiv(total_chunks, a.chunks_per_cta));
    const int smem = STAGES * (2 * X_TILE + 2 * PKG * (nb * 16 + 16)) + 1024;
    static PcxOnce done32, done64;
    cudaError_t e;
    if (nb == 32) {
        if (!done32) {
            e = cudaFuncSetAttribute(sum_sm_par_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
            if (e != cudaSuccess) return (int)e;
            done32 = true;
        }
        sum_sm_par_kernel<32><<<grid, PNTH, smem, (cudaStream_t)stream>>>(a);
    } else {
        if (!done64) {
            e = cudaFuncSetAttribute(sum_sm_par_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
            if (e != cudaSuccess) return (int)e;
            done64 = true;
        }
        sum_sm_par_kernel<64><<<grid, PNTH, smem, (cudaStream_t)stream>>>(a);
    }
    PCX_LAUNCH_CHECK();
    return 0;
}

int pcx_pack_sm_jobs(const void* jobs, int n_jobs, int64_t n_vec, const float* params, void* stream) {
    if (n_jobs <= 0 || n_vec <= 0) return 0;
    pack_sm_jobs_kernel<<<(unsigned)pcx_cdiv(n_vec, 256), 256, 0, (cudaStream_t)stream>>>(
        reinterpret_cast<const SmPackJob*>(jobs), n_jobs, n_vec, params);
    PCX_LAUNCH_CHECK();
    return 0;
}

int pcx_sum_fwd_sm(float* node_mars, const float* element_mars, const void* packed, const int32_t* first_row,
                   const int32_t* nids, const int32_t* cids, const int32_t* fk, int64_t n_merged, int nb, int K, int B,
                   void* stream) {
    if (n_merged <= 0 || B <= 0) return 0;
    if ((nb != 32 && nb != 64) || K <= 0 || (fk == nullptr && element_mars == nullptr)) return -1;
    SmArgs a{};
    a.fk = reinterpret_cast<const int2*>(fk); a.nmars = node_mars;
    a.out = node_mars; a.src = element_mars; a.packed = reinterpret_cast<const uint4*>(packed);
    a.first_row = first_row; a.rows = nids; a.kids = cids; a.n_st = (int)pcx_cdiv(B, SM_SAMPLES);
    a.n_tiles = n_merged * a.n_st; a.K = K; a.par_block = 1; a.B = B; a.logspace = 1;
    a.terms = (g_sum_mode == 2) ? 1 : 3;
    return nb == 32 ? launch_sm<32, false>(a, (cudaStream_t)stream) : launch_sm<64, false>(a, (cudaStream_t)stream);
}

int pcx_sum_bwd_ele_sm(float* element_flows, const float* element_mars, const float* node_flows,
                       const float* node_mars, const void* packed, const int32_t* first_row, const int32_t* chids,
                       const int32_t* parids, const int32_t* fk, int ch_block_size, int64_t n_merged, int nb, int P,
                       int block_size, int B, int logspace, void* stream) {
    if (n_merged <= 0 || B <= 0) return 0;
    if ((nb != 32 && nb != 64) || P <= 0 || block_size % 8 != 0 || (block_size & (block_size - 1)) != 0) return -1;
    if (fk == nullptr && element_mars == nullptr) return -1;
    SmArgs a{};
    a.fk = reinterpret_cast<const int2*>(fk); a.nmars = node_mars; a.cbs = ch_block_size;
    a.out = element_flows; a.src = node_flows; a.src2 = node_mars; a.emars = element_mars;
    a.packed = reinterpret_cast<const uint4*>(packed); a.first_row = first_row; a.rows = chids; a.kids = parids;
    a.n_st = (int)pcx_cdiv(B, SM_SAMPLES); a.n_tiles = n_merged * a.n_st; a.K = P; a.par_block = block_size; a.B = B;
    a.logspace = logspace; a.terms = (g_sum_mode == 2) ? 1 : 3;
    return nb == 32 ? launch_sm<32, true>(a, (cudaStream_t)stream) : launch_sm<64, true>(a, (cudaStream_t)stream);
}

}  // extern "C"
