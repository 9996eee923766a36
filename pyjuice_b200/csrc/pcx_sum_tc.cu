// Sum-layer kernels on the Blackwell tensor cores (tcgen05.mma, fp32 accumulators in TMEM).
//
// Three contractions share one skeleton (a CTA of 256 threads owns a 128-row output tile, stages 64-deep
// operand slices in shared memory in the K-major core-matrix layout and lets one thread issue the MMAs):
//
//   forward        node_mars[r, b]   = log sum_k  theta[r, k] * exp(emars[k, b])            tile 128 x 64 (batch)
//   element flows  eflows[c, b]      = emars[c, b] + log sum_k theta^T[c, k] * exp(nflow[k, b] - nmar[k, b])
//   parameter flows pflow[m, e]     += theta[m, e] * sum_b exp(nflow[m, b] - nmar[m, b] - s_b) * exp(emars[e, b] + s_b)
//                                                                                            tile 128 x 64 (edges)
//
// Operands produced on CUDA cores (the exponentials) are split into bf16 hi + lo and multiplied as
// hi*hi + hi*lo + lo*hi, which keeps ~16 significant bits per factor.  The parameter operand of the first two
// kernels is static between EM updates, so it is pre-split once per update into ready-made 32 KB tile images
// (pcx_pack_sum_params) that the kernels copy into shared memory with cp.async while the exponentials are
// being computed.
//
// Latency, not throughput, bounds these kernels on deep circuits (hundreds of small dependent layers): every
// thread therefore issues all global loads of a slice before touching any of them, the batch column of the
// log-sum-exp kernels is shared by four threads (one 8-row group each per half-slice) so that the column
// maximum needs a single shared-memory exchange, and tables up to 128 deep keep their values in registers
// between the maximum pass and the exponential pass.
//
// Every mbarrier wait is bounded; on expiry the kernel records a status code, skips its remaining tensor-core
// work, frees its TMEM and returns.
#include "pcx_common.cuh"
#include "pcx_tc.cuh"
#include "../../include/pcx_b200.h"
#include <float.h>

namespace {

using namespace pcx_tc;

constexpr int BM = 128;                  // rows per tile (UMMA M)
constexpr int BN = 64;                   // columns per tile (UMMA N)
constexpr int KC = 64;                   // contraction depth per shared-memory stage
constexpr int KG = KC / 8;               // 16-byte K groups per stage
constexpr int STAGES = 2;
constexpr int NTH = 256;
constexpr int A_TILE = KG * BM * 16;     // 16 KB: one bf16 [128 x 64] operand tile
constexpr int B_TILE = KG * BN * 16;     //  8 KB: one bf16 [ 64 x 64] operand tile
constexpr int STAGE_BYTES = 2 * A_TILE + 2 * B_TILE;          // A_hi, A_lo, B_hi, B_lo = 48 KB
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024;
// parameter-flow kernel: 128 threads work on slices of 32 samples, so that four CTAs fit on an SM and hide each
// other's load latency and barrier waits; slabs are padded by 16 B so that the lanes that stage one row write
// different banks
constexpr int PNTH = 128;                // threads
constexpr int PKC = 32;                  // samples (contraction depth) per shared-memory stage
constexpr int PKG = PKC / 8;
constexpr int XSLAB = BM * 16 + 16, YSLAB = BN * 16 + 16;
constexpr int X_TILE = PKG * XSLAB, Y_TILE = PKG * YSLAB;
constexpr int PAR_STAGE_BYTES = 2 * X_TILE + 2 * Y_TILE;
constexpr int PAR_SMEM_BYTES = STAGES * PAR_STAGE_BYTES + 1024;
static_assert(STAGES * STAGE_BYTES >= BM * (64 + 1) * 4, "epilogue transpose buffer aliases the stages");

// Optional phase timestamps of the dataflow launch (development builds only: -DPCX_TRACE).
#ifdef PCX_TRACE
constexpr int kTraceItems = 1 << 16, kTracePoints = 12;
__device__ long long g_trace[kTraceItems][kTracePoints];
#define PCX_T(slot, k)                                                                                     \
    do {                                                                                                   \
        if (threadIdx.x == 0 && (slot) >= 0 && (slot) < kTraceItems) {                                     \
            long long _t;                                                                                  \
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(_t));                                         \
            g_trace[(slot)][(k)] = _t;                                                                     \
        }                                                                                                  \
    } while (0)
#else
#define PCX_T(slot, k) do { } while (0)
#endif

__device__ int g_tc_status = 0;          // 0 ok; otherwise the code of the first bounded wait that gave up


// Eight fp32 values -> eight bf16 "hi" parts and eight bf16 "lo" parts (x ~= hi + lo), two values per conversion.
__device__ __forceinline__ void store_split8(uint4* hi, uint4* lo, const float* x) {
    uint32_t h[4], l[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const __nv_bfloat162 hp = __floats2bfloat162_rn(x[2 * j], x[2 * j + 1]);      // .x (low half) = x[2j]
        h[j] = *reinterpret_cast<const uint32_t*>(&hp);
        const float h0 = __uint_as_float(h[j] << 16), h1 = __uint_as_float(h[j] & 0xffff0000u);
        const __nv_bfloat162 lp = __floats2bfloat162_rn(x[2 * j] - h0, x[2 * j + 1] - h1);
        l[j] = *reinterpret_cast<const uint32_t*>(&lp);
    }
    *hi = make_uint4(h[0], h[1], h[2], h[3]);
    *lo = make_uint4(l[0], l[1], l[2], l[3]);
}

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
    asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 0;" ::: "memory");
}

// Bounded wait until *ctr >= target (acquire): about a second at most with the default limit.
__device__ __forceinline__ bool poll_counter(const int* ctr, int target, uint32_t max_polls = (1u << 21)) {
    for (uint32_t n = 0; n < max_polls; ++n) {
        int v;
        asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(ctr) : "memory");
        if (v >= target) return true;
        if (n > 4096) __nanosleep(256);            // a long wait: stop hammering the counter
    }
    return false;
}
__device__ __forceinline__ void red_release_add(int* ctr, int v) {
    asm volatile("red.release.gpu.global.add.s32 [%0], %1;" ::"l"(ctr), "r"(v) : "memory");
}

// Issue the MMAs of one 64-deep stage: A tiles at `sa` (hi, then lo), B tiles at `sb` (hi, then lo).  A tile is
// KG slabs of [rows][16 B]; consecutive slabs are ASLAB / BSLAB bytes apart (rows * 16, or that plus padding).
template <int ASLAB = BM * 16, int BSLAB = BN * 16, int DEPTH = KC>
__device__ __forceinline__ void issue_stage(uint32_t tmem, uint32_t sa, uint32_t sb, uint32_t idesc, bool first, int terms) {
    constexpr int GROUPS = DEPTH / 8;                 // 16-byte K groups per tile: the lo tile follows the hi tile
#pragma unroll
    for (int ks = 0; ks < DEPTH / 16; ++ks) {
        const uint64_t dAh = smem_desc(sa + ks * 2 * ASLAB, ASLAB, 128);
        const uint64_t dAl = smem_desc(sa + GROUPS * ASLAB + ks * 2 * ASLAB, ASLAB, 128);
        const uint64_t dBh = smem_desc(sb + ks * 2 * BSLAB, BSLAB, 128);
        const uint64_t dBl = smem_desc(sb + GROUPS * BSLAB + ks * 2 * BSLAB, BSLAB, 128);
        mma_bf16_ss(tmem, dAh, dBh, idesc, (!first || ks > 0) ? 1u : 0u);
        if (terms == 3) {
            mma_bf16_ss(tmem, dAh, dBl, idesc, 1u);
            mma_bf16_ss(tmem, dAl, dBh, idesc, 1u);
        }
    }
}

// ---------------------------------------------------------------------------------------------------------
// Parameter pre-split: ready-made A tiles for the forward (MODE 0) and element-flow (MODE 1) kernels
// ---------------------------------------------------------------------------------------------------------
struct PackJob {                // one table whose parameters are to be pre-split; an array of these lives on the device
    uint4* out;                 // [n_rows * tiles_r * n_chunks] tile images of 2 * A_TILE bytes (hi, then lo)
    const int32_t* kids;        // forward: unused                    element flows: parids (0 = padding)
    const int32_t* kpar;        // forward: pids                      element flows: parpids
    int64_t vec_begin;          // index of this job's first 16-byte (hi) vector in the launch-wide enumeration
    int32_t K;                  // table width
    int32_t row_block;          // rows per table row (multiple of 128)
    int32_t par_block;          // element flows: parent block size (multiple of 8)
    int32_t n_chunks;
    int32_t mode;               // 0 forward, 1 element flows
    int32_t pad_;
};

// One thread per 16-byte vector of every job; the job is found by binary search over vec_begin.
__global__ void pack_params_kernel(const PackJob* __restrict__ jobs, int n_jobs, int64_t n_vec,
                                   const float* __restrict__ params) {
    int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= n_vec) return;
    int lo = 0, hi = n_jobs - 1;
    while (lo < hi) {
        int mid = (lo + hi + 1) >> 1;
        if (jobs[mid].vec_begin <= t) lo = mid; else hi = mid - 1;
    }
    const PackJob a = jobs[lo];
    t -= a.vec_begin;
    const int r = (int)(t % BM);
    const int g = (int)((t / BM) % KG);
    int64_t tile = t / (BM * KG);
    const int chunk = (int)(tile % a.n_chunks);
    const int64_t rowtile = tile / a.n_chunks;
    const int tiles_r = a.row_block / BM;
    const int64_t i = rowtile / tiles_r;
    const int r0 = (int)(rowtile % tiles_r) * BM;
    const int kb = chunk * KC + g * 8;
    float v[8];
    if (a.mode == 0) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            int k = kb + j;
            v[j] = (k < a.K) ? params[(int64_t)a.kpar[i * a.K + k] + r0 + r] : 0.0f;
        }
    } else {
        const int KK = a.K * a.par_block;
        const int lg = 31 - __clz(a.par_block);
        int p = kb >> lg, n = kb & (a.par_block - 1);
        int pr = (kb < KK) ? a.kids[i * a.K + p] : 0;
#pragma unroll
        for (int j = 0; j < 8; ++j)
            v[j] = (pr != 0) ? params[(int64_t)a.kpar[i * a.K + p] + (int64_t)(r0 + r) * a.par_block + n + j] : 0.0f;
    }
    uint4* base = a.out + tile * (2 * A_TILE / 16);
    store_split8(base + g * BM + r, base + A_TILE / 16 + g * BM + r, v);
}

// Same conversion for a single table whose record is passed by value (no device-side job array).
__global__ void pack_params_one_kernel(const PackJob a, int64_t n_vec, const float* __restrict__ params) {
    int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= n_vec) return;
    const int r = (int)(t % BM);
    const int g = (int)((t / BM) % KG);
    int64_t tile = t / (BM * KG);
    const int chunk = (int)(tile % a.n_chunks);
    const int64_t rowtile = tile / a.n_chunks;
    const int tiles_r = a.row_block / BM;
    const int64_t i = rowtile / tiles_r;
    const int r0 = (int)(rowtile % tiles_r) * BM;
    const int kb = chunk * KC + g * 8;
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        int k = kb + j;
        v[j] = (k < a.K) ? params[(int64_t)a.kpar[i * a.K + k] + r0 + r] : 0.0f;
    }
    uint4* base = a.out + tile * (2 * A_TILE / 16);
    store_split8(base + g * BM + r, base + A_TILE / 16 + g * BM + r, v);
}

// ---------------------------------------------------------------------------------------------------------
// Forward / element flows
// ---------------------------------------------------------------------------------------------------------
enum Mode { FWD = 0, ELE = 1 };

struct LseArgs {
    float* out;                 // FWD: node_mars            ELE: element_flows
    const float* lsrc;          // FWD: element_mars         ELE: node_flows
    const float* lsrc2;         //                           ELE: node_mars
    const float* emars;         //                           ELE: element_mars (epilogue)
    const uint4* packed;        // pre-split parameter tiles
    const int32_t* rows;        // FWD: nids                 ELE: chids
    const int32_t* kids;        // FWD: cids [n, K]          ELE: parids [n, P]
    int K;
    int row_block;
    int par_block;
    int B;
    int logspace;
    int terms;
    // Product layer folded into this kernel (FC > 0): a product node's value is the sum of FC child rows of
    // node_mars (row 0 = no child), so neither element_mars nor element_flows is touched.
    const int32_t* fkids;       // FWD: [n, K, FC] child rows of every table entry   ELE: [n, row_block, FC] child rows of every output element
    const float* nmars;         // node_mars (fused reads)
    float* nflows_direct;       // ELE: when set, the flow of an element is stored straight to its child rows of node_flows
    int vec;                    // B % 8 == 0 and 16-byte aligned buffers: the epilogue uses 16-byte accesses
};

// Child rows of one table entry (row 0 = no child).
template <int FC>
__device__ __forceinline__ void load_children(const int32_t* idx, int* r) {
#pragma unroll
    for (int c = 0; c < FC; c += 4) {
        const int4 t = *reinterpret_cast<const int4*>(idx + c);
        r[c] = t.x; r[c + 1] = t.y; r[c + 2] = t.z; r[c + 3] = t.w;
    }
}
// Values of the FC child rows at column `col`.  The loads are unconditional (row 0 exists and is simply not used),
// so that a thread can have all loads of several entries in flight at once instead of one per branch.
template <int FC>
__device__ __forceinline__ void load_child_values(const int* r, const float* src, int B, int col, float* v) {
#pragma unroll
    for (int c = 0; c < FC; ++c) v[c] = __ldcg(src + (int64_t)r[c] * B + col);
}
// Sum over the children that exist; -inf when the entry has no child at all.
template <int FC>
__device__ __forceinline__ float combine_children(const int* r, const float* v) {
    float s = 0.0f;
    int any = 0;
#pragma unroll
    for (int c = 0; c < FC; ++c) { s += v[c]; any |= r[c]; }        // row 0 is the dummy node: its value is 0
    return any ? s : PCX_NEG_INF;
}

// Shared-memory state of one tile (declared once per kernel so that every instantiation of the body uses the same).
struct LseShared {
    uint64_t bar[STAGES];
    float part[NTH];            // [threads per column][TN] partial column maxima
    float smax[64];
    int fail;
};

// One CTA = 128 output rows x TN batch columns.  TN in {16, 32, 64} is chosen per launch so that small layers still
// spread over the whole GPU: the per-thread instruction stream is the critical path of these kernels, and a
// narrower tile divides it (256 / TN threads share one column).
//
// `wait_on` (dataflow launches only): a counter that another CTA of the same launch advances when the rows this
// tile reads are complete; the tile proceeds once it has reached `wait_for`.  Everything that does not depend on
// those rows (parameter tiles, index tables) is requested before the wait.  The wait is bounded.
// `ph[s]` counts the completed phases of mbarrier s, so that a CTA can run many tiles on the same barriers.
// Returns false if a bounded wait gave up (the tile's output is then not written).
template <int MODE, bool SMALLK, int FC, int TN>
__device__ __forceinline__ bool lse_tile_body(const LseArgs& a, const int64_t rowtile, const int coltile,
                                              const uint32_t tmem, uint8_t* smem, LseShared& sh, uint32_t* ph,
                                              const int* wait_on, const int wait_for, const int slot = -1) {
    constexpr int TPC = NTH / TN;                      // threads per batch column
    constexpr int NGS = (16 / TPC) > 0 ? (16 / TPC) : 1;    // SMALLK: 8-row groups per thread (the table has <= 16)
    constexpr int BSLAB = TN * 16;                     // bytes of one K group of the B tile
    constexpr int F = FC > 0 ? FC : 4;
    constexpr int HC = TN / 2;                         // epilogue: columns per thread

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int tiles_r = a.row_block / BM;
    const int64_t i = rowtile / tiles_r;
    const int r0 = (int)(rowtile % tiles_r) * BM;
    const int b0 = coltile * TN;
    const int B = a.B;
    const int KK = (MODE == FWD) ? a.K : a.K * a.par_block;
    const int lg_pb = (MODE == ELE) ? (31 - __clz(a.par_block)) : 0;
    const int n_chunks = (KK + KC - 1) / KC;

    // this thread's share of L: batch column `lc`, 8-row groups q, q + TPC, ... of the table
    const int lc = tid % TN, q = tid / TN;
    const int col = b0 + lc;
    const bool col_ok = col < B;
    const int colc = col_ok ? col : 0;

    // Loads are unconditional (row 0 exists and is simply not used) and grouped -- every index of a group, then
    // every value, then the arithmetic -- so that a thread has all loads of a group in flight at once.
    auto group_index = [&](int kb, int (*r)[F]) {                  // child rows of the 8 entries (FWD, folded)
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int k = kb + j;
            if (col_ok && k < KK) load_children<F>(a.fkids + ((int64_t)i * a.K + k) * FC, r[j]);
            else
#pragma unroll
                for (int c = 0; c < F; ++c) r[j][c] = 0;
        }
    };
    auto group_values = [&](const int (*r)[F], float* v) {
        float cv[8][F];
#pragma unroll
        for (int j = 0; j < 8; ++j) load_child_values<F>(r[j], a.nmars, B, colc, cv[j]);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = combine_children<F>(r[j], cv[j]);
    };
    auto parent_of = [&](int kb) -> int {                          // ELE: the parent block of the 8 entries
        return (col_ok && kb < KK) ? a.kids[i * a.K + (kb >> lg_pb)] : 0;
    };
    // ELE: the eight indices of a group lie in one parent block (block sizes are multiples of 8).  The parents'
    // values do not change during the backward pass; only their flows are produced by other tiles.
    auto ele_static = [&](int kb, float* nm) -> int {
        const int pr = parent_of(kb);
        const int64_t row = (int64_t)pr + (kb & (a.par_block - 1));
#pragma unroll
        for (int j = 0; j < 8; ++j) nm[j] = __ldcg(a.lsrc2 + (row + j) * B + colc);
        return pr;
    };
    auto ele_finish = [&](int kb, int pr, const float* nm, float* v) {
        const int64_t row = (int64_t)pr + (kb & (a.par_block - 1));
        float nf[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) nf[j] = __ldcg(a.lsrc + (row + j) * B + colc);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            float f = nf[j];
            if (!a.logspace) f = __logf(f);                                  // log(0) = -inf
            v[j] = (pr == 0) ? PCX_NEG_INF : f - fmaxf(nm[j], -3.0e38f);      // (-inf) - (-inf) reads as -inf
        }
    };
    // raw (log-domain) values of one 8-row group starting at contraction index kb
    auto load_group = [&](int kb, float* v) {
        if (MODE == FWD && FC > 0) {
            int r[8][F];
            group_index(kb, r);
            group_values(r, v);
        } else if (MODE == FWD) {
            int cid[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) cid[j] = (col_ok && kb + j < KK) ? a.kids[i * a.K + kb + j] : 0;
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = __ldcg(a.lsrc + (int64_t)cid[j] * B + colc);
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = (cid[j] != 0) ? v[j] : PCX_NEG_INF;
        } else {
            float nm[8];
            const int pr = ele_static(kb, nm);
            ele_finish(kb, pr, nm, v);
        }
    };
    auto copy_a = [&](int chunk, uint8_t* st) {
        const uint4* src = a.packed + (rowtile * n_chunks + chunk) * (2 * A_TILE / 16);
#pragma unroll
        for (int w = 0; w < 2 * A_TILE / 16 / NTH; ++w) cp_async16(st + (w * NTH + tid) * 16, src + w * NTH + tid);
    };
    // exp(v - mx) of one group -> bf16 hi/lo, written as row `lc` of K group g of the B tile of stage `st`
    auto store_group = [&](uint8_t* st, int g, float* v, float mx) {
        const float mxc = (mx == PCX_NEG_INF) ? 0.0f : mx;     // a column without any mass: every value is -inf
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = __expf(v[j] - mxc);          // exp(-inf - s) = 0
        uint8_t* bt = st + 2 * A_TILE + g * BSLAB + lc * 16;
        store_split8(reinterpret_cast<uint4*>(bt), reinterpret_cast<uint4*>(bt + KG * BSLAB), v);
    };

    // ---- before the wait: parameter tiles and the first group's index table -----------------------------
    float keep[SMALLK ? NGS : 1][8];
    float mx = PCX_NEG_INF;
    int r_first[8][F];
    float nm_first[8];
    int pr_first = 0;
    // epilogue role: this thread finishes HC samples of one output row
    const int erow = (warp & 3) * 32 + lane;
    const bool vec = a.vec != 0;
    int ch[F];
    if (SMALLK) {
        for (int c = 0; c < n_chunks; ++c) copy_a(c, smem + c * STAGE_BYTES);
        if (MODE == FWD && FC > 0) group_index(q * 8, r_first);
        if (MODE == ELE) pr_first = ele_static(q * 8, nm_first);
    }
    if (MODE == ELE && FC > 0 && vec) load_children<F>(a.fkids + ((int64_t)i * a.row_block + r0 + erow) * FC, ch);
    // ELE with 16-column tiles: the values of the 128 output elements (sums of child rows, static during the backward
    // pass) are gathered now, with coalesced loads in the layout of the operand loads, and parked in the part of
    // stage 0 that a 16-column B tile leaves unused; the epilogue reads them from there.
    constexpr bool EMS = (MODE == ELE && FC > 0 && TN == 16);
    float* em_tile = reinterpret_cast<float*>(smem + 2 * A_TILE + 2 * KG * BSLAB);      // [BM][TN + 1]
    static_assert(!EMS || BM * (TN + 1) * 4 <= 2 * B_TILE - 2 * KG * BSLAB, "element values fit beside the B tile");
    if (EMS && vec) {
        int r[8][F];
        float ev[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) load_children<F>(a.fkids + ((int64_t)i * a.row_block + r0 + q * 8 + j) * FC, r[j]);
        group_values(r, ev);
#pragma unroll
        for (int j = 0; j < 8; ++j) em_tile[(q * 8 + j) * (TN + 1) + lc] = ev[j];
    }
    if (wait_on != nullptr) {
        if (tid == 0 && !poll_counter(wait_on, wait_for)) sh.fail = 3;
        __syncthreads();
    }
    PCX_T(slot, 2);

    // ---- pass 1: column maxima (values stay in registers when the table is at most two slices deep) ----
    if (SMALLK) {
#pragma unroll
        for (int h = 0; h < NGS; ++h) {
            const int gi = q + TPC * h;                            // group index within the whole table (< 16)
            if (MODE == FWD && FC > 0 && h == 0) group_values(r_first, keep[0]);
            else if (MODE == ELE && h == 0) ele_finish(q * 8, pr_first, nm_first, keep[0]);
            else if (gi * 8 < KK) load_group(gi * 8, keep[h]);
            else
#pragma unroll
                for (int j = 0; j < 8; ++j) keep[h][j] = PCX_NEG_INF;
#pragma unroll
            for (int j = 0; j < 8; ++j) mx = fmaxf(mx, keep[h][j]);
        }
    } else {
        for (int gi = q; gi * 8 < KK; gi += TPC) {
            float v[8];
            load_group(gi * 8, v);
#pragma unroll
            for (int j = 0; j < 8; ++j) mx = fmaxf(mx, v[j]);
        }
    }
    sh.part[q * TN + lc] = mx;
    __syncthreads();
    PCX_T(slot, 3);
#pragma unroll
    for (int t = 0; t < TPC; ++t) mx = fmaxf(mx, sh.part[t * TN + lc]);
    if (q == 0) sh.smax[lc] = mx;

    const int64_t base_row = (int64_t)a.rows[i] + r0;

    // ---- pass 2: exponentials -> bf16 hi/lo operand tiles, multiply -----------------------------------------
    const uint32_t idesc = idesc_bf16_f32(BM, TN);
    bool failed = false;
    // Deep tables: the tensor core adds every product into its fp32 accumulator with truncation, which biases a
    // sum of hundreds of MMAs low by about 3e-8 per MMA (2e-5 for a 4096-deep table, 2.5e-3 nats after 128 such
    // layers).  So the sum is taken out of TMEM every kFlush chunks (48 MMAs) and carried in registers, where the
    // additions round to nearest; two accumulators alternate, so the tensor core never waits for the read-out.
    constexpr int kFlush = 4;
    constexpr int ACC_COLS = TN < 32 ? 32 : TN;
    const int lq = warp & 3, c0 = (warp >> 2) * HC;    // epilogue role: HC samples of output row lq * 32 + lane
    const int row = lq * 32 + lane;
    float accr[SMALLK ? 1 : HC];
    int drained = 0;
    if (!SMALLK)
#pragma unroll
        for (int j = 0; j < HC; ++j) accr[j] = 0.0f;
    auto drain = [&](int which) {
        if (!SMALLK) {
#pragma unroll
            for (int p = 0; p < HC / 8; ++p) {
                float v[8];
                tmem_ld<8>(tmem + which * ACC_COLS + ((uint32_t)(lq * 32) << 16) + (uint32_t)(c0 + 8 * p), v);
#pragma unroll
                for (int j = 0; j < 8; ++j) accr[8 * p + j] += v[j];
            }
            tc_fence_before_sync();
        }
    };
    if (SMALLK) {
#pragma unroll
        for (int h = 0; h < NGS; ++h) {
            const int gi = q + TPC * h;
            if (gi < n_chunks * KG) store_group(smem + (gi / KG) * STAGE_BYTES, gi % KG, keep[h], mx);
        }
        PCX_T(slot, 4);
        cp_async_wait_all();
        fence_async_smem();
        __syncthreads();
        PCX_T(slot, 5);
        if (tid == 0) {
            tc_fence_after_sync();
            for (int c = 0; c < n_chunks; ++c) {
                const uint32_t sa = smem_u32(smem + c * STAGE_BYTES);
                issue_stage<BM * 16, BSLAB>(tmem, sa, sa + 2 * A_TILE, idesc, c == 0, a.terms);
            }
            mma_commit(&sh.bar[0]);
        }
    } else {
        for (int c = 0; c < n_chunks; ++c) {
            const int s = c % STAGES, use = c / STAGES;
            uint8_t* st = smem + s * STAGE_BYTES;
            if (c >= STAGES && !failed && !mbar_wait(&sh.bar[s], (ph[s] + use - 1) & 1)) { failed = true; sh.fail = 1; }
            // chunk c - 2 is complete: if it closed a group of kFlush chunks, move that group's sum to registers
            if (c >= STAGES && (c - STAGES + 1) % kFlush == 0 && !failed) {
                tc_fence_after_sync();
                drain(((c - STAGES) / kFlush) & 1);
                ++drained;
            }
            copy_a(c, st);
            for (int g = q; g < KG; g += TPC) {
                float v[8];
                load_group(c * KC + g * 8, v);
                store_group(st, g, v, mx);
            }
            cp_async_wait_all();
            fence_async_smem();
            __syncthreads();
            failed = failed || (sh.fail != 0);
            if (tid == 0 && !failed) {
                tc_fence_after_sync();
                const uint32_t sa = smem_u32(st);
                issue_stage<BM * 16, BSLAB>(tmem + ((c / kFlush) & 1) * ACC_COLS, sa, sa + 2 * A_TILE, idesc,
                                            c % kFlush == 0, a.terms);
                mma_commit(&sh.bar[s]);
            }
        }
    }

    // ---- epilogue ------------------------------------------------------------------------------------------
    // Warps w and w + 4 share the TMEM lane quarter w % 4 and take half of the columns each: a thread owns HC
    // consecutive samples of ONE output row.  With B a multiple of 8 it finishes them in registers (one index
    // load per row, 16-byte loads and stores); the indices and the first child values are requested while the
    // tensor core is still working.
    // the values the epilogue adds (children of the output row, their indices were fetched at the start) are
    // requested while the tensor core works
    float4 cq[F][2];
    const int cb0 = (b0 + c0 < B) ? b0 + c0 : 0;       // first column of this thread (clamped for the prefetch)
    if (MODE == ELE && vec && !EMS) {
        if (FC > 0) {
#pragma unroll
            for (int c = 0; c < F; ++c) {
                cq[c][0] = __ldcg(reinterpret_cast<const float4*>(a.nmars + (int64_t)ch[c] * B + cb0));
                cq[c][1] = __ldcg(reinterpret_cast<const float4*>(a.nmars + (int64_t)ch[c] * B + cb0 + 4));
            }
        } else {
            cq[0][0] = __ldcg(reinterpret_cast<const float4*>(a.emars + (base_row + row) * B + cb0));
            cq[0][1] = __ldcg(reinterpret_cast<const float4*>(a.emars + (base_row + row) * B + cb0 + 4));
        }
    }

    {
        const int cl = SMALLK ? 0 : n_chunks - 1;       // the last commit covers every MMA issued before it
        const uint32_t par = SMALLK ? ph[0] : ph[cl % STAGES] + cl / STAGES;
        // one thread waits for the tensor core; the others sleep in the barrier below instead of spinning
        if (tid == 0 && !failed && !mbar_wait(&sh.bar[cl % STAGES], par & 1)) sh.fail = 2;
        if (SMALLK) ph[0] += 1;
        else
#pragma unroll
            for (int s = 0; s < STAGES; ++s) ph[s] += (n_chunks - s + STAGES - 1) / STAGES;
    }
    __syncthreads();
    PCX_T(slot, 6);
    failed = failed || (sh.fail != 0);
    tc_fence_after_sync();
    if (!SMALLK && !failed) {                              // groups of chunks whose sum is still in TMEM
        const int groups = (n_chunks + kFlush - 1) / kFlush;
        for (int g = drained; g < groups; ++g) drain(g & 1);
    }
    if (vec) {
        if (!failed) {
#pragma unroll
            for (int p = 0; p < HC / 8; ++p) {
                const int cb = b0 + c0 + 8 * p;                     // B % 8 == 0: a piece is all in or all out
                float v[8];
                if (SMALLK) tmem_ld<8>(tmem + ((uint32_t)(lq * 32) << 16) + (uint32_t)(c0 + 8 * p), v);
                else
#pragma unroll
                    for (int j = 0; j < 8; ++j) v[j] = accr[SMALLK ? 0 : 8 * p + j];
                if (cb >= B) continue;
                if (MODE == ELE && p > 0 && !EMS) {
                    if (FC > 0) {
#pragma unroll
                        for (int c = 0; c < F; ++c) {
                            cq[c][0] = __ldcg(reinterpret_cast<const float4*>(a.nmars + (int64_t)ch[c] * B + cb));
                            cq[c][1] = __ldcg(reinterpret_cast<const float4*>(a.nmars + (int64_t)ch[c] * B + cb + 4));
                        }
                    } else {
                        cq[0][0] = __ldcg(reinterpret_cast<const float4*>(a.emars + (base_row + row) * B + cb));
                        cq[0][1] = __ldcg(reinterpret_cast<const float4*>(a.emars + (base_row + row) * B + cb + 4));
                    }
                }
                float o[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const float m = sh.smax[c0 + 8 * p + j];
                    // log(0) = -inf and -inf + x = -inf cover empty sums and columns without mass
                    if (MODE == FWD) o[j] = __logf(fmaxf(v[j], 1e-24f)) + m;
                    else o[j] = __logf(v[j]) + m;
                }
                if (MODE == ELE) {
                    float em[8];
                    if (EMS) {
#pragma unroll
                        for (int j = 0; j < 8; ++j) em[j] = em_tile[row * (TN + 1) + c0 + 8 * p + j];
                    } else if (FC > 0) {
                        int any = 0;
#pragma unroll
                        for (int j = 0; j < 8; ++j) em[j] = 0.0f;
#pragma unroll
                        for (int c = 0; c < F; ++c) {
                            const bool on = ch[c] != 0;
                            any |= ch[c];
                            em[0] += on ? cq[c][0].x : 0.0f; em[1] += on ? cq[c][0].y : 0.0f;
                            em[2] += on ? cq[c][0].z : 0.0f; em[3] += on ? cq[c][0].w : 0.0f;
                            em[4] += on ? cq[c][1].x : 0.0f; em[5] += on ? cq[c][1].y : 0.0f;
                            em[6] += on ? cq[c][1].z : 0.0f; em[7] += on ? cq[c][1].w : 0.0f;
                        }
                        if (!any) {
#pragma unroll
                            for (int j = 0; j < 8; ++j) em[j] = PCX_NEG_INF;
                        }
                    } else {
                        em[0] = cq[0][0].x; em[1] = cq[0][0].y; em[2] = cq[0][0].z; em[3] = cq[0][0].w;
                        em[4] = cq[0][1].x; em[5] = cq[0][1].y; em[6] = cq[0][1].z; em[7] = cq[0][1].w;
                    }
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        o[j] = o[j] + em[j];
                        if (!a.logspace) o[j] = __expf(o[j]);
                    }
                }
                const float4 o0 = make_float4(o[0], o[1], o[2], o[3]), o1 = make_float4(o[4], o[5], o[6], o[7]);
                if (MODE == ELE && FC > 0 && a.nflows_direct != nullptr) {
                    // every child of this element has it as its only parent: its flow IS the element's flow
#pragma unroll
                    for (int c = 0; c < F; ++c) {
                        if (ch[c] != 0) {
                            float4* dst = reinterpret_cast<float4*>(a.nflows_direct + (int64_t)ch[c] * B + cb);
                            dst[0] = o0; dst[1] = o1;
                        }
                    }
                } else {
                    float4* dst = reinterpret_cast<float4*>(a.out + (base_row + row) * B + cb);
                    dst[0] = o0; dst[1] = o1;
                }
            }
        }
        tc_fence_before_sync();
    } else {
        // general batch sizes: through a shared-memory transpose, one sample per thread and step
        float* T = reinterpret_cast<float*>(smem);            // [BM][TN + 1], aliases the (now idle) stages
        if (!failed) {
            float v[HC];
            if (SMALLK) tmem_ld<HC>(tmem + ((uint32_t)(lq * 32) << 16) + (uint32_t)c0, v);
            else
#pragma unroll
                for (int j = 0; j < HC; ++j) v[j] = accr[SMALLK ? 0 : j];
#pragma unroll
            for (int j = 0; j < HC; ++j) {
                const float m = sh.smax[c0 + j];
                float o;
                if (MODE == FWD) o = (m == PCX_NEG_INF) ? PCX_NEG_INF : __logf(fmaxf(v[j], 1e-24f)) + m;
                else o = (m == PCX_NEG_INF || v[j] <= 0.0f) ? PCX_NEG_INF : __logf(v[j]) + m;
                T[row * (TN + 1) + c0 + j] = o;
            }
        }
        tc_fence_before_sync();
        __syncthreads();
        if (!failed) {
            constexpr int ITERS = BM * TN / NTH, UB = 4;
            for (int it0 = 0; it0 < ITERS; it0 += UB) {
                // four outputs per thread at a time: all their loads first, then the arithmetic and the stores
                float o[UB], em[UB], cv[UB][F];
                int chs[UB][F];
#pragma unroll
                for (int u = 0; u < UB; ++u) {
                    const int flat = (it0 + u) * NTH + tid;
                    const int r = flat / TN, cc = flat % TN;
                    o[u] = T[r * (TN + 1) + cc];
                    if (MODE == ELE && FC > 0) load_children<F>(a.fkids + ((int64_t)i * a.row_block + r0 + r) * FC, chs[u]);
                }
                if (MODE == ELE) {
#pragma unroll
                    for (int u = 0; u < UB; ++u) {
                        const int flat = (it0 + u) * NTH + tid;
                        const int r = flat / TN, b = b0 + flat % TN;
                        const int bc = b < B ? b : 0;
                        if (FC > 0) load_child_values<F>(chs[u], a.nmars, B, bc, cv[u]);
                        else em[u] = a.emars[(base_row + r) * B + bc];
                    }
                }
#pragma unroll
                for (int u = 0; u < UB; ++u) {
                    const int flat = (it0 + u) * NTH + tid;
                    const int r = flat / TN, b = b0 + flat % TN;
                    if (b >= B) continue;
                    float ov = o[u];
                    if (MODE == ELE) {
                        const float e = (FC > 0) ? combine_children<F>(chs[u], cv[u]) : em[u];
                        ov = (ov == PCX_NEG_INF || e == PCX_NEG_INF) ? PCX_NEG_INF : ov + e;
                        if (!a.logspace) ov = __expf(ov);
                        if (FC > 0 && a.nflows_direct != nullptr) {
#pragma unroll
                            for (int c = 0; c < F; ++c)
                                if (chs[u][c] != 0) a.nflows_direct[(int64_t)chs[u][c] * B + b] = ov;
                            continue;
                        }
                    }
                    a.out[(base_row + r) * B + b] = ov;
                }
            }
        }
    }
    if (failed && tid == 0) atomicCAS(&g_tc_status, 0, 100 * (MODE + 1) + sh.fail);
    PCX_T(slot, 8);
    return !failed;
}

// Barriers, status word and TMEM of a CTA; returns the TMEM base address.
template <int TCOLS>
__device__ __forceinline__ uint32_t lse_cta_setup(LseShared& sh, uint32_t* s_tmem) {
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) mbar_init(&sh.bar[s], 1);
        fence_mbar_init();
        sh.fail = 0;
    }
    if (threadIdx.x < 32) tmem_alloc(s_tmem, TCOLS);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    return *s_tmem;
}

template <int MODE, bool SMALLK, int FC, int TN>
__global__ void __launch_bounds__(NTH, 2) sum_lse_tc_kernel(const LseArgs a) {
    constexpr int TCOLS = 2 * (TN < 32 ? 32 : TN);     // TMEM columns: two accumulators (see kFlush)
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ LseShared sh;
    __shared__ uint32_t s_tmem;
    const uint32_t tmem = lse_cta_setup<TCOLS>(sh, &s_tmem);
    uint32_t ph[STAGES] = {0, 0};
    lse_tile_body<MODE, SMALLK, FC, TN>(a, blockIdx.x, blockIdx.y, tmem, smem, sh, ph, nullptr, 0);
    __syncthreads();
    if (threadIdx.x < 32) tmem_dealloc(tmem, TCOLS);
}

// ---------------------------------------------------------------------------------------------------------
// Dataflow launch: every tile of a run of consecutive layers in ONE launch
// ---------------------------------------------------------------------------------------------------------
// Deep, narrow circuits (a tree-shaped model has one layer per level of the tree) spend their time in launch
// boundaries: a layer with a handful of 128-row blocks cannot fill 148 SMs, and the next layer cannot start before
// the last tile of this one has drained.  Batch columns are independent of one another, though, so the only true
// dependency of tile (layer l, rows, columns j) is on the tiles of earlier layers with the same columns j.
//
// Work items (table, row tile, column tile) are enumerated layer by layer and claimed from a global counter in that
// order.  A counter per (level, column tile) counts finished row tiles; an item of level t waits until the counter
// of (t - 1, j) is complete, which, by induction, means every earlier level is complete for columns j.  An item is
// only ever claimed after all items it can wait for have been claimed by CTAs that are already running, so the
// scheme cannot deadlock whatever the number of resident CTAs; each wait is bounded all the same.
struct ChainJob {
    const uint4* packed;
    const int32_t* rows;
    const int32_t* kids;
    const int32_t* fkids;
    int64_t item_begin;
    int32_t K, row_block, par_block, n_rowtiles;
    int32_t level, prev_total;
};
static_assert(sizeof(ChainJob) == 64, "matches PcxChainJob");

template <int MODE, int FC, int TN>
__global__ void __launch_bounds__(NTH, 2)
sum_chain_kernel(LseArgs a, const ChainJob* jobs, int n_jobs, int64_t n_items, int n_ct, int* ctrl) {
    constexpr int TCOLS = 2 * (TN < 32 ? 32 : TN);
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ LseShared sh;
    __shared__ uint32_t s_tmem;
    __shared__ int64_t s_item;
    constexpr int kJobsInSmem = 128;
    __shared__ __align__(16) ChainJob s_jobs[kJobsInSmem];   // copied with 16-byte accesses                    // small job tables are searched on chip
    if (n_jobs <= kJobsInSmem) {
        const uint4* src = reinterpret_cast<const uint4*>(jobs);
        uint4* dst = reinterpret_cast<uint4*>(s_jobs);
        for (int k = threadIdx.x; k < n_jobs * (int)(sizeof(ChainJob) / 16); k += NTH) dst[k] = src[k];
        jobs = s_jobs;
    }
    const uint32_t tmem = lse_cta_setup<TCOLS>(sh, &s_tmem);
    uint32_t ph[STAGES] = {0, 0};
    int* done = ctrl + 64;                                      // [level][column tile] finished row tiles
    unsigned long long* queue = reinterpret_cast<unsigned long long*>(ctrl);
    // thread 0 claims one item ahead: the round trip of the claim overlaps the work on the current item
    unsigned long long next = 0;
    if (threadIdx.x == 0) next = atomicAdd(queue, 1ull);
    for (;;) {
        if (threadIdx.x == 0) s_item = (int64_t)next;
        __syncthreads();
        const int64_t item = s_item;
        if (item >= n_items) break;
        if (threadIdx.x == 0) next = atomicAdd(queue, 1ull);
        PCX_T((int)item, 0);
        int lo = 0, hi = n_jobs - 1;
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (jobs[mid].item_begin <= item) lo = mid; else hi = mid - 1;
        }
        const ChainJob j = jobs[lo];
        a.packed = j.packed; a.rows = j.rows; a.kids = j.kids; a.fkids = j.fkids;
        a.K = j.K; a.row_block = j.row_block; a.par_block = j.par_block;
        const int64_t t = item - j.item_begin;
        const int ct = (int)(t / j.n_rowtiles);                 // column-tile major: lane 0 of a level is claimed first
        const int64_t rt = t % j.n_rowtiles;
        const int* wait_on = (j.level > 0) ? done + (j.level - 1) * n_ct + ct : nullptr;
        const int KK = (MODE == FWD) ? j.K : j.K * j.par_block;
        PCX_T((int)item, 1);
        if (KK <= 2 * KC) lse_tile_body<MODE, true, FC, TN>(a, rt, ct, tmem, smem, sh, ph, wait_on, j.prev_total, (int)item);
        else lse_tile_body<MODE, false, FC, TN>(a, rt, ct, tmem, smem, sh, ph, wait_on, j.prev_total, (int)item);
        // publish: the barrier orders every thread's stores before thread 0's release (a tile that gave up still
        // counts, so that the launch drains; the status word tells the host)
        __syncthreads();
        if (threadIdx.x == 0) red_release_add(done + j.level * n_ct + ct, 1);
        PCX_T((int)item, 9);
#ifdef PCX_TRACE
        if (threadIdx.x == 0 && item < kTraceItems) { g_trace[item][10] = j.level; g_trace[item][11] = blockIdx.x; }
#endif
    }
    __syncthreads();
    if (threadIdx.x < 32) tmem_dealloc(tmem, TCOLS);
}

// ---------------------------------------------------------------------------------------------------------
// Parameter flows
// ---------------------------------------------------------------------------------------------------------
struct ParArgs {
    float* param_flows;
    const float* node_flows;
    const float* node_mars;
    const float* element_mars;
    const float* params;
    const int32_t* nids;
    const int32_t* cids;
    const int32_t* pids;
    const int32_t* pfids;
    int K;
    int block_size;
    int B;
    int logspace;
    int terms;
    int chunks_per_cta;         // 64-sample slices handled by one CTA (the batch is split across blockIdx.z)
    const int32_t* fkids;       // FC > 0: [n, K, FC] child rows of node_mars whose sum is the value of table entry (i, e)
};

template <int FC>
__device__ __forceinline__ void par_tile_body(const ParArgs& a, const int64_t rowtile, const int etile, const int zsplit) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ uint64_t s_bar[STAGES];
    __shared__ uint32_t s_tmem;
    __shared__ __align__(16) float s_part[PNTH / 32][PKC];
    __shared__ int s_cid[BN], s_pid[BN], s_pfid[BN];
    __shared__ int s_fail;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int tiles_r = a.block_size / BM;
    const int64_t i = rowtile / tiles_r;
    const int r0 = (int)(rowtile % tiles_r) * BM;
    const int e0 = etile * BN;
    const int B = a.B;
    const int total_chunks = (B + PKC - 1) / PKC;
    const int c_begin = zsplit * a.chunks_per_cta;
    const int c_end = min(total_chunks, c_begin + a.chunks_per_cta);

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) mbar_init(&s_bar[s], 1);
        fence_mbar_init();
        s_fail = 0;
    }
    if (tid < BN) {
        const int e = e0 + tid;
        const bool ok = e < a.K;
        s_cid[tid] = ok ? a.cids[i * a.K + e] : 0;
        s_pid[tid] = ok ? a.pids[i * a.K + e] : 0;
        s_pfid[tid] = ok ? a.pfids[i * a.K + e] : 0;
    }
    if (warp == 0) tmem_alloc(&s_tmem, BN);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = s_tmem;
    const int64_t nid = (int64_t)a.nids[i] + r0;

    // staging role: 8-sample group g of the slice, rows rb + 32 j
    const int g = tid & (PKG - 1), rb = tid / PKG;
    const uint32_t idesc = idesc_bf16_f32(BM, BN);
    bool failed = false;

    // child rows of this thread's two table entries: the same for every slice of the batch
    constexpr int FK = FC > 0 ? FC : 4;
    int chr[2][FK];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        if (FC > 0 && s_cid[rb + 32 * j] != 0) load_children<FK>(a.fkids + ((int64_t)i * a.K + e0 + rb + 32 * j) * FC, chr[j]);
        else
#pragma unroll
            for (int c = 0; c < FK; ++c) chr[j][c] = 0;
    }

    for (int c = c_begin; c < c_end; ++c) {
        const int it = c - c_begin, s = it % STAGES, use = it / STAGES;
        uint8_t* st = smem + s * PAR_STAGE_BYTES;
        const int bb = c * PKC + g * 8;                 // first sample of this thread's group
        const bool b_ok = bb < B;                      // B is a multiple of 8: a group is all-in or all-out

        // issue every load of the slice first
        float x[4][8], y[2][8];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int64_t off = (nid + rb + 32 * j) * B + bb;
            if (b_ok) {
                const float4 f0 = *reinterpret_cast<const float4*>(a.node_flows + off);
                const float4 f1 = *reinterpret_cast<const float4*>(a.node_flows + off + 4);
                const float4 m0 = *reinterpret_cast<const float4*>(a.node_mars + off);
                const float4 m1 = *reinterpret_cast<const float4*>(a.node_mars + off + 4);
                const float nf[8] = {f0.x, f0.y, f0.z, f0.w, f1.x, f1.y, f1.z, f1.w};
                const float nm[8] = {m0.x, m0.y, m0.z, m0.w, m1.x, m1.y, m1.z, m1.w};
#pragma unroll
                for (int t = 0; t < 8; ++t) {
                    float f = nf[t];
                    if (!a.logspace) f = __logf(f);                        // log(0) = -inf
                    x[j][t] = f - fmaxf(nm[t], -3.0e38f);                   // (-inf) - (-inf) reads as -inf
                }
            } else {
#pragma unroll
                for (int t = 0; t < 8; ++t) x[j][t] = PCX_NEG_INF;
            }
        }
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int cid = s_cid[rb + 32 * j];
            if (FC > 0) {
                // the product node's value is recomputed from its children (no element buffer involved); loads are
                // unconditional -- row 0 exists and is not used -- so that all of them are in flight together
                constexpr int F = FC > 0 ? FC : 4;
                int r[F];
#pragma unroll
                for (int c = 0; c < F; ++c) r[c] = b_ok ? chr[j][c] : 0;
                const int bbc = b_ok ? bb : 0;
                float4 q[F][2];
#pragma unroll
                for (int c = 0; c < F; ++c) {
                    q[c][0] = __ldcg(reinterpret_cast<const float4*>(a.node_mars + (int64_t)r[c] * B + bbc));
                    q[c][1] = __ldcg(reinterpret_cast<const float4*>(a.node_mars + (int64_t)r[c] * B + bbc + 4));
                }
                int any = 0;
#pragma unroll
                for (int t = 0; t < 8; ++t) y[j][t] = 0.0f;
#pragma unroll
                for (int c = 0; c < F; ++c) {                               // row 0 is the dummy node: value 0
                    any |= r[c];
                    y[j][0] += q[c][0].x; y[j][1] += q[c][0].y; y[j][2] += q[c][0].z; y[j][3] += q[c][0].w;
                    y[j][4] += q[c][1].x; y[j][5] += q[c][1].y; y[j][6] += q[c][1].z; y[j][7] += q[c][1].w;
                }
                if (!any) {
#pragma unroll
                    for (int t = 0; t < 8; ++t) y[j][t] = PCX_NEG_INF;
                }
            } else if (b_ok && cid != 0) {
                const float4 q0 = *reinterpret_cast<const float4*>(a.element_mars + (int64_t)cid * B + bb);
                const float4 q1 = *reinterpret_cast<const float4*>(a.element_mars + (int64_t)cid * B + bb + 4);
                y[j][0] = q0.x; y[j][1] = q0.y; y[j][2] = q0.z; y[j][3] = q0.w;
                y[j][4] = q1.x; y[j][5] = q1.y; y[j][6] = q1.z; y[j][7] = q1.w;
            } else {
#pragma unroll
                for (int t = 0; t < 8; ++t) y[j][t] = PCX_NEG_INF;
            }
        }
        // per-sample shift = max over the 128 rows of the tile of log(flow / value)
        float pm[8];
#pragma unroll
        for (int t = 0; t < 8; ++t) {
            float m = fmaxf(fmaxf(x[0][t], x[1][t]), fmaxf(x[2][t], x[3][t]));
#pragma unroll
            for (int o = PKG; o < 32; o <<= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
            pm[t] = m;
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
        uint8_t* xhi = st;
        uint8_t* xlo = st + X_TILE;
        uint8_t* yhi = st + 2 * X_TILE;
        uint8_t* ylo = st + 2 * X_TILE + Y_TILE;
        float shc[8];                                   // a sample without any flow: every x is -inf, shift by 0
#pragma unroll
        for (int t = 0; t < 8; ++t) shc[t] = (sh[t] == PCX_NEG_INF) ? 0.0f : sh[t];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
#pragma unroll
            for (int t = 0; t < 8; ++t) x[j][t] = __expf(x[j][t] - shc[t]);   // exp(-inf - s) = 0
            const int o = g * XSLAB + (rb + 32 * j) * 16;
            store_split8(reinterpret_cast<uint4*>(xhi + o), reinterpret_cast<uint4*>(xlo + o), x[j]);
        }
#pragma unroll
        for (int j = 0; j < 2; ++j) {
#pragma unroll
            for (int t = 0; t < 8; ++t) y[j][t] = fminf(__expf(y[j][t] + sh[t]), 3.0e38f);   // sh = -inf: exp(-inf) = 0
            const int o = g * YSLAB + (rb + 32 * j) * 16;
            store_split8(reinterpret_cast<uint4*>(yhi + o), reinterpret_cast<uint4*>(ylo + o), y[j]);
        }
        fence_async_smem();
        __syncthreads();
        failed = failed || (s_fail != 0);
        if (tid == 0 && !failed) {
            tc_fence_after_sync();
            const uint32_t sa = smem_u32(st);
            issue_stage<XSLAB, YSLAB, PKC>(tmem, sa, sa + 2 * X_TILE, idesc, it == 0, a.terms);
            mma_commit(&s_bar[s]);
        }
    }

    const int n_it = c_end - c_begin;
    if (n_it > 0) {
        const int il = n_it - 1;
        if (!failed && !mbar_wait(&s_bar[il % STAGES], (uint32_t)((il / STAGES) & 1))) { failed = true; s_fail = 2; }
    }
    __syncthreads();
    failed = failed || (s_fail != 0);
    tc_fence_after_sync();
    if (warp < 4 && !failed && n_it > 0) {
        const int row = warp * 32 + lane;
#pragma unroll 1
        for (int cg = 0; cg < BN / 32; ++cg) {
            float v[32];
            tmem_ld32(tmem + ((uint32_t)(warp * 32) << 16) + (uint32_t)(cg * 32), v);
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                const int e = cg * 32 + j;
                if (s_cid[e] == 0) continue;
                const float pf = a.params[(int64_t)s_pid[e] + r0 + row] * v[j];
                if (pf != 0.0f) atomicAdd(a.param_flows + (int64_t)s_pfid[e] + r0 + row, pf);
            }
        }
    }
    if (failed && tid == 0) atomicCAS(&g_tc_status, 0, 300 + s_fail);
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, BN);
}

template <int FC>
__global__ void __launch_bounds__(PNTH, 4) sum_par_tc_kernel(const ParArgs a) {
    par_tile_body<FC>(a, blockIdx.x, blockIdx.y, blockIdx.z);
}

// Every table of the circuit in ONE launch.  Parameter-flow tiles of different layers are independent of each
// other (they only read node values / flows and add into disjoint or atomically shared accumulators), so once the
// chain of element-flow kernels has produced all node flows, the whole circuit's parameter flows form one large
// grid instead of one small launch per layer.
struct ParJob {
    const int32_t* nids;
    const int32_t* cids;
    const int32_t* pids;
    const int32_t* pfids;
    const int32_t* fkids;
    int64_t item_begin;         // first work item (CTA) of this table in the launch-wide enumeration
    int32_t K;
    int32_t block_size;
    int32_t e_tiles;            // ceil(K / 64)
    int32_t splits;             // batch splits per (row tile, edge tile)
};

template <int FC>
__global__ void __launch_bounds__(PNTH, 4)
sum_par_tc_batched(const ParJob* __restrict__ jobs, int n_jobs, ParArgs a) {
    const int64_t w = blockIdx.x;
    int lo = 0, hi = n_jobs - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (jobs[mid].item_begin <= w) lo = mid; else hi = mid - 1;
    }
    const ParJob j = jobs[lo];
    a.nids = j.nids; a.cids = j.cids; a.pids = j.pids; a.pfids = j.pfids; a.fkids = j.fkids;
    a.K = j.K; a.block_size = j.block_size;
    int64_t t = w - j.item_begin;
    const int z = (int)(t % j.splits); t /= j.splits;
    const int et = (int)(t % j.e_tiles);
    par_tile_body<FC>(a, t / j.e_tiles, et, z);
}

// One warp exercises the give-up branch of the two bounded waits the tensor-core kernels use: it waits, with a small
// explicit limit, on a counter that nothing advances (which = 0) or on an mbarrier that no copy or MMA ever arrives
// on (which = 1), records the status code 900 + which and returns normally.
__device__ int g_probe_counter = 0;
__global__ void bounded_wait_probe_kernel(int which, uint32_t max_polls) {
    __shared__ uint64_t bar;
    if (threadIdx.x != 0) return;
    bool ok;
    if (which == 0) {
        ok = poll_counter(&g_probe_counter, 1, max_polls);
    } else {
        mbar_init(&bar, 1);
        fence_mbar_init();
        ok = mbar_wait(&bar, 0u, max_polls);
        mbar_inval(&bar);
    }
    if (!ok) atomicCAS(&g_tc_status, 0, 900 + which);
}

// Built-in scratch of the allocation-free forward entry point: room for PCX_NOALLOC_MAX_TILES pre-split parameter
// tiles.  Every GPU that loads the library reserves it until the process exits.
__device__ __align__(256) unsigned char g_noalloc_tiles[(size_t)PCX_NOALLOC_MAX_TILES * 2 * A_TILE];
constexpr int kMaxDevices = 64;
// Device address of the scratch, per device ordinal.  Written without a lock: two host threads that make the first
// call on one device at the same time both resolve the same address and store the same value.
unsigned char* g_noalloc_ptr[kMaxDevices] = {nullptr};

thread_local int g_sum_mode = 1;      // per host thread; 0: fp32 CUDA cores only, 1: tensor cores with bf16 hi/lo split, 2: tensor cores, single bf16

template <typename Kern>
int configure_once(Kern kern, bool* done) {
    if (!*done) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        *done = true;
    }
    return 0;
}

template <int MODE, int FC, int TN>
int launch_lse_tn(const LseArgs& a, int64_t n_rows, cudaStream_t st) {
    static PcxOnce done_small, done_big;
    const int KK = (MODE == FWD) ? a.K : a.K * a.par_block;
    dim3 grid((unsigned)(n_rows * (a.row_block / BM)), (unsigned)pcx_cdiv(a.B, TN));
    if (KK <= 2 * KC) {
        int rc = configure_once(sum_lse_tc_kernel<MODE, true, FC, TN>, &done_small);
        if (rc) return rc;
        sum_lse_tc_kernel<MODE, true, FC, TN><<<grid, NTH, SMEM_BYTES, st>>>(a);
    } else {
        int rc = configure_once(sum_lse_tc_kernel<MODE, false, FC, TN>, &done_big);
        if (rc) return rc;
        sum_lse_tc_kernel<MODE, false, FC, TN><<<grid, NTH, SMEM_BYTES, st>>>(a);
    }
    PCX_LAUNCH_CHECK();
    return 0;
}

// Tile width: the widest of 64 / 32 / 16 columns that still gives about one CTA per SM.
template <int MODE, int FC>
int launch_lse_fc(const LseArgs& a, int64_t n_rows, cudaStream_t st) {
    const int64_t row_tiles = n_rows * (a.row_block / BM);
    if (row_tiles * pcx_cdiv(a.B, 64) >= 148) return launch_lse_tn<MODE, FC, 64>(a, n_rows, st);
    if (row_tiles * pcx_cdiv(a.B, 32) >= 148) return launch_lse_tn<MODE, FC, 32>(a, n_rows, st);
    return launch_lse_tn<MODE, FC, 16>(a, n_rows, st);
}

// 16-byte accesses in the epilogue need whole groups of eight samples and aligned buffers.
inline int lse_vec_ok(const LseArgs& a) {
    auto al = [](const void* p) { return p == nullptr || (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    return (a.B % 8 == 0 && al(a.out) && al(a.nmars) && al(a.emars) && al(a.nflows_direct)) ? 1 : 0;
}

template <int MODE>
int launch_lse(const LseArgs& a_in, int64_t n_rows, int fc, cudaStream_t st) {
    LseArgs a = a_in;
    a.vec = lse_vec_ok(a);
    switch (fc) {
        case 0: return launch_lse_fc<MODE, 0>(a, n_rows, st);
        case 4: return launch_lse_fc<MODE, 4>(a, n_rows, st);
        case 8: return launch_lse_fc<MODE, 8>(a, n_rows, st);
        default: return -1;
    }
}

template <int MODE, int FC, int TN>
int launch_chain_tn(const LseArgs& a, const ChainJob* jobs, int n_jobs, int64_t n_items, int n_ct, int* ctrl,
                    int n_ctas, cudaStream_t st) {
    static PcxOnce done;
    int rc = configure_once(sum_chain_kernel<MODE, FC, TN>, &done);
    if (rc) return rc;
    sum_chain_kernel<MODE, FC, TN><<<n_ctas, NTH, SMEM_BYTES, st>>>(a, jobs, n_jobs, n_items, n_ct, ctrl);
    PCX_LAUNCH_CHECK();
    return 0;
}

template <int MODE, int FC>
int launch_chain_fc(const LseArgs& a, const ChainJob* jobs, int n_jobs, int64_t n_items, int tn, int n_ct, int* ctrl,
                    int n_ctas, cudaStream_t st) {
    switch (tn) {
        case 64: return launch_chain_tn<MODE, FC, 64>(a, jobs, n_jobs, n_items, n_ct, ctrl, n_ctas, st);
        case 32: return launch_chain_tn<MODE, FC, 32>(a, jobs, n_jobs, n_items, n_ct, ctrl, n_ctas, st);
        case 16: return launch_chain_tn<MODE, FC, 16>(a, jobs, n_jobs, n_items, n_ct, ctrl, n_ctas, st);
        default: return -1;
    }
}

}  // namespace

// Used by the dispatchers in pcx_sum_simt.cu.
int pcx_tc_sum_mode() { return g_sum_mode; }

template <int FC>
static int launch_par_fc(const ParArgs& a, dim3 grid, cudaStream_t st) {
    static PcxOnce done;
    if (!done) {
        cudaError_t e = cudaFuncSetAttribute(sum_par_tc_kernel<FC>, cudaFuncAttributeMaxDynamicSharedMemorySize, PAR_SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        done = true;
    }
    sum_par_tc_kernel<FC><<<grid, PNTH, PAR_SMEM_BYTES, st>>>(a);
    cudaError_t e = cudaGetLastError();
    return (e == cudaSuccess) ? 0 : (int)e;
}

int pcx_tc_launch_par(float* param_flows, const float* node_flows, const float* node_mars, const float* element_mars,
                      const float* params, const int32_t* nids, const int32_t* cids, const int32_t* pids,
                      const int32_t* pfids, const int32_t* fkids, int fc, int64_t n_blocks, int K, int block_size,
                      int B, int logspace, cudaStream_t st) {
    ParArgs a{param_flows, node_flows, node_mars, element_mars, params, nids, cids, pids, pfids,
              K, block_size, B, logspace, (g_sum_mode == 2) ? 1 : 3, 1, fkids};
    const int64_t base = n_blocks * (block_size / BM) * pcx_cdiv(K, BN);
    const int total_chunks = (int)pcx_cdiv(B, PKC);
    int64_t splits = pcx_cdiv(4 * 148, base);                  // aim at four CTAs per SM
    if (splits > total_chunks) splits = total_chunks;
    if (splits < 1) splits = 1;
    a.chunks_per_cta = (int)pcx_cdiv(total_chunks, splits);
    dim3 grid((unsigned)(n_blocks * (block_size / BM)), (unsigned)pcx_cdiv(K, BN),
              (unsigned)pcx_cdiv(total_chunks, a.chunks_per_cta));
    switch (fc) {
        case 0: return launch_par_fc<0>(a, grid, st);
        case 4: return launch_par_fc<4>(a, grid, st);
        case 8: return launch_par_fc<8>(a, grid, st);
        default: return -1;
    }
}

int pcx_tc_try_sum_par(float* param_flows, const float* node_flows, const float* node_mars, const float* element_mars,
                       const float* params, const int32_t* nids, const int32_t* cids, const int32_t* pids,
                       const int32_t* pfids, int64_t n_blocks, int K, int block_size, int B, int logspace,
                       cudaStream_t st, int* rc) {
    if (g_sum_mode == 0 || block_size % BM != 0 || B % 8 != 0) return 0;
    *rc = pcx_tc_launch_par(param_flows, node_flows, node_mars, element_mars, params, nids, cids, pids, pfids,
                            nullptr, 0, n_blocks, K, block_size, B, logspace, st);
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

int pcx_clear_status(void) {
    const int v = 0;
    cudaError_t e = cudaMemcpyToSymbol(g_tc_status, &v, sizeof(int));
    return e == cudaSuccess ? 0 : (int)e;
}

int pcx_probe_bounded_wait(int which, int max_polls, void* stream) {
    if ((which != 0 && which != 1) || max_polls < 1 || max_polls > (1 << 16)) return -1;
    bounded_wait_probe_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(which, (uint32_t)max_polls);
    PCX_LAUNCH_CHECK();
    return 0;
}

int64_t pcx_packed_tile_count(int64_t n_rows, int K, int row_block, int par_block, int mode) {
    if (row_block % BM != 0) return 0;
    const int64_t KK = (mode == 0) ? K : (int64_t)K * par_block;
    return n_rows * (row_block / BM) * pcx_cdiv(KK, KC);
}

int pcx_pack_sum_params(const void* jobs, int n_jobs, int64_t n_vec, const float* params, void* stream) {
    if (n_jobs <= 0 || n_vec <= 0) return 0;
    const unsigned grid = (unsigned)pcx_cdiv(n_vec, 256);
    pack_params_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(reinterpret_cast<const PackJob*>(jobs), n_jobs, n_vec, params);
    PCX_LAUNCH_CHECK();
    return 0;
}

int pcx_sum_fwd_packed(float* node_mars, const float* element_mars, const void* packed,
                       const int32_t* nids, const int32_t* cids, int64_t n_blocks, int K, int block_size, int B,
                       void* stream) {
    if (n_blocks <= 0 || B <= 0) return 0;
    if (block_size % BM != 0 || K <= 0) return -1;
    LseArgs a{};
    a.out = node_mars; a.lsrc = element_mars; a.packed = reinterpret_cast<const uint4*>(packed);
    a.rows = nids; a.kids = cids; a.K = K; a.row_block = block_size; a.par_block = 1; a.B = B; a.logspace = 1;
    a.terms = (g_sum_mode == 2) ? 1 : 3;
    return launch_lse<FWD>(a, n_blocks, 0, (cudaStream_t)stream);
}

int pcx_sum_fwd_noalloc(float* node_mars, const float* element_mars, const float* params,
                        const int32_t* nids, const int32_t* cids, const int32_t* pids,
                        int64_t n_blocks, int K, int block_size, int B, void* stream) {
    if (n_blocks <= 0 || B <= 0) return 0;
    if (block_size % BM != 0 || K <= 0) return -1;
    const int64_t tiles = n_blocks * (block_size / BM) * pcx_cdiv(K, KC);
    if (tiles > PCX_NOALLOC_MAX_TILES) return PCX_ERR_SCRATCH_TOO_SMALL;

    // Set-up, once per device: in host code the array's name is only a handle, the kernels need its device address.
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= kMaxDevices) return -1;
    if (g_noalloc_ptr[dev] == nullptr) {
        void* ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_noalloc_tiles);
        if (e != cudaSuccess) return (int)e;
        g_noalloc_ptr[dev] = static_cast<unsigned char*>(ptr);
    }
    unsigned char* scratch = g_noalloc_ptr[dev];
    cudaStream_t st = (cudaStream_t)stream;

    // 1) split the parameters of this table into the scratch (every byte of the tiles used is rewritten, padding
    //    included, so nothing depends on what an earlier call left there)
    PackJob job{};
    job.out = reinterpret_cast<uint4*>(scratch); job.kids = cids; job.kpar = pids; job.vec_begin = 0;
    job.K = K; job.row_block = block_size; job.par_block = 1; job.n_chunks = (int)pcx_cdiv(K, KC); job.mode = 0;
    const int64_t n_vec = tiles * KG * BM;
    pack_params_one_kernel<<<(unsigned)pcx_cdiv(n_vec, 256), 256, 0, st>>>(job, n_vec, params);
    PCX_LAUNCH_CHECK();

    // 2) the tensor-core forward kernel, reading the tiles it was just given
    LseArgs a{};
    a.out = node_mars; a.lsrc = element_mars; a.packed = reinterpret_cast<const uint4*>(scratch);
    a.rows = nids; a.kids = cids; a.K = K; a.row_block = block_size; a.par_block = 1; a.B = B; a.logspace = 1;
    a.terms = (g_sum_mode == 2) ? 1 : 3;
    return launch_lse<FWD>(a, n_blocks, 0, st);
}

int pcx_sum_fwd_fused(float* node_mars, const void* packed, const int32_t* nids, const int32_t* cids,
                      const int32_t* fkids, int fc, int64_t n_blocks, int K, int block_size, int B, void* stream) {
    if (n_blocks <= 0 || B <= 0) return 0;
    if (block_size % BM != 0 || K <= 0 || (fc != 4 && fc != 8)) return -1;
    LseArgs a{};
    a.out = node_mars; a.nmars = node_mars; a.fkids = fkids; a.packed = reinterpret_cast<const uint4*>(packed);
    a.rows = nids; a.kids = cids; a.K = K; a.row_block = block_size; a.par_block = 1; a.B = B; a.logspace = 1;
    a.terms = (g_sum_mode == 2) ? 1 : 3;
    return launch_lse<FWD>(a, n_blocks, fc, (cudaStream_t)stream);
}

int pcx_sum_bwd_ele_fused(float* element_flows, float* node_flows, const float* node_mars, const void* packed,
                          const int32_t* chids, const int32_t* parids, const int32_t* fkids, int fc, int direct,
                          int64_t n_blocks, int P, int block_size, int ch_block_size, int B, int logspace,
                          void* stream) {
    if (n_blocks <= 0 || B <= 0) return 0;
    if (ch_block_size % BM != 0 || block_size % 8 != 0 || P <= 0 || (fc != 4 && fc != 8)) return -1;
    LseArgs a{};
    a.out = element_flows; a.lsrc = node_flows; a.lsrc2 = node_mars; a.nmars = node_mars; a.fkids = fkids;
    a.nflows_direct = direct ? node_flows : nullptr;
    a.packed = reinterpret_cast<const uint4*>(packed); a.rows = chids; a.kids = parids; a.K = P;
    a.row_block = ch_block_size; a.par_block = block_size; a.B = B; a.logspace = logspace;
    a.terms = (g_sum_mode == 2) ? 1 : 3;
    return launch_lse<ELE>(a, n_blocks, fc, (cudaStream_t)stream);
}

int pcx_sum_bwd_par_fused(float* param_flows, const float* node_flows, const float* node_mars, const float* params,
                          const int32_t* nids, const int32_t* cids, const int32_t* pids, const int32_t* pfids,
                          const int32_t* fkids, int fc, int64_t n_blocks, int K, int block_size, int B, int logspace,
                          void* stream) {
    if (n_blocks <= 0 || B <= 0) return 0;
    if (block_size % BM != 0 || B % 8 != 0 || K <= 0 || (fc != 4 && fc != 8)) return -1;
    return pcx_tc_launch_par(param_flows, node_flows, node_mars, nullptr, params, nids, cids, pids, pfids, fkids, fc,
                             n_blocks, K, block_size, B, logspace, (cudaStream_t)stream);
}

int pcx_sum_chain(int mode, float* node_mars, float* node_flows, const void* jobs, int n_jobs, int64_t n_items,
                  int n_levels, int tn, int fc, int B, int logspace, int* ctrl, int64_t ctrl_len, void* stream) {
    if (n_jobs <= 0 || n_items <= 0 || B <= 0) return 0;
    if ((mode != 0 && mode != 1) || (fc != 4 && fc != 8) || n_levels <= 0) return -1;
    const int n_ct = (int)pcx_cdiv(B, tn);
    const int64_t need = 64 + (int64_t)n_levels * n_ct;
    if (ctrl == nullptr || ctrl_len < need || (reinterpret_cast<uintptr_t>(ctrl) & 7) != 0) return -1;
    cudaStream_t st = (cudaStream_t)stream;
    int dev = 0, sms = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return (int)e;
    e = cudaMemsetAsync(ctrl, 0, (size_t)need * sizeof(int), st);
    if (e != cudaSuccess) return (int)e;
    LseArgs a{};
    a.nmars = node_mars; a.B = B; a.terms = (g_sum_mode == 2) ? 1 : 3;
    if (mode == 0) { a.out = node_mars; a.logspace = 1; }
    else { a.lsrc = node_flows; a.lsrc2 = node_mars; a.nflows_direct = node_flows; a.logspace = logspace; }
    a.vec = lse_vec_ok(a);
    const int n_ctas = (int)(n_items < 2 * (int64_t)sms ? n_items : 2 * (int64_t)sms);
    const ChainJob* cj = reinterpret_cast<const ChainJob*>(jobs);
    if (mode == 0) {
        return fc == 4 ? launch_chain_fc<FWD, 4>(a, cj, n_jobs, n_items, tn, n_ct, ctrl, n_ctas, st)
                       : launch_chain_fc<FWD, 8>(a, cj, n_jobs, n_items, tn, n_ct, ctrl, n_ctas, st);
    }
    return fc == 4 ? launch_chain_fc<ELE, 4>(a, cj, n_jobs, n_items, tn, n_ct, ctrl, n_ctas, st)
                   : launch_chain_fc<ELE, 8>(a, cj, n_jobs, n_items, tn, n_ct, ctrl, n_ctas, st);
}

#ifdef PCX_TRACE
int pcx_trace_read(long long* host, int n_items) {
    if (n_items > kTraceItems) n_items = kTraceItems;
    cudaError_t e = cudaMemcpyFromSymbol(host, g_trace, (size_t)n_items * kTracePoints * sizeof(long long));
    return (int)e;
}
#endif

int pcx_sum_bwd_par_batched(float* param_flows, const float* node_flows, const float* node_mars, const float* params,
                            const void* jobs, int n_jobs, int64_t n_items, int fc, int B, int chunks_per_cta,
                            int logspace, void* stream) {
    if (n_jobs <= 0 || n_items <= 0 || B <= 0) return 0;
    if (B % 8 != 0 || chunks_per_cta <= 0 || (fc != 4 && fc != 8)) return -1;
    ParArgs a{};
    a.param_flows = param_flows; a.node_flows = node_flows; a.node_mars = node_mars; a.params = params;
    a.B = B; a.logspace = logspace; a.terms = (g_sum_mode == 2) ? 1 : 3; a.chunks_per_cta = chunks_per_cta;
    static PcxOnce done4, done8;
    cudaError_t e;
    if (fc == 4) {
        if (!done4) {
            e = cudaFuncSetAttribute(sum_par_tc_batched<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, PAR_SMEM_BYTES);
            if (e != cudaSuccess) return (int)e;
            done4 = true;
        }
        sum_par_tc_batched<4><<<(unsigned)n_items, PNTH, PAR_SMEM_BYTES, (cudaStream_t)stream>>>(
            reinterpret_cast<const ParJob*>(jobs), n_jobs, a);
    } else {
        if (!done8) {
            e = cudaFuncSetAttribute(sum_par_tc_batched<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, PAR_SMEM_BYTES);
            if (e != cudaSuccess) return (int)e;
            done8 = true;
        }
        sum_par_tc_batched<8><<<(unsigned)n_items, PNTH, PAR_SMEM_BYTES, (cudaStream_t)stream>>>(
            reinterpret_cast<const ParJob*>(jobs), n_jobs, a);
    }
    PCX_LAUNCH_CHECK();
    return 0;
}

int pcx_sum_bwd_ele_packed(float* element_flows, const float* element_mars, const float* node_flows,
                           const float* node_mars, const void* packed, const int32_t* chids, const int32_t* parids,
                           int64_t n_blocks, int P, int block_size, int ch_block_size, int B, int logspace,
                           void* stream) {
    if (n_blocks <= 0 || B <= 0) return 0;
    if (ch_block_size % BM != 0 || block_size % 8 != 0 || P <= 0) return -1;
    LseArgs a{};
    a.out = element_flows; a.lsrc = node_flows; a.lsrc2 = node_mars; a.emars = element_mars;
    a.packed = reinterpret_cast<const uint4*>(packed); a.rows = chids; a.kids = parids; a.K = P;
    a.row_block = ch_block_size; a.par_block = block_size; a.B = B; a.logspace = logspace;
    a.terms = (g_sum_mode == 2) ? 1 : 3;
    return launch_lse<ELE>(a, n_blocks, 0, (cudaStream_t)stream);
}

}  // extern "C"

#include "pcx_sum_dense.cuh"
#include "pcx_sum_dense2.cuh"
#include "pcx_sum_sm.cuh"
