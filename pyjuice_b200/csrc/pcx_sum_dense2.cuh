// Dense sum layers, wide tiles: the second generation of the two-step dense path (pcx_sum_dense.cuh).
//
// What changed and why.  The first version multiplied 128 x 64 tiles: every 32 KB parameter tile was fetched once
// per 64 samples, so a 4096 x 4096 layer at 256 samples moved 400 MB from L2 to the SMs per pass and ran at the
// per-SM copy rate, not at the tensor-core rate.  Here an output tile is 128 rows x up to 256 samples (all samples
// of a rank for the usual batch sizes), so a parameter tile is fetched ONCE per layer and pass; the machine is
// filled by splitting the contraction over the 2, 4 or 8 CTAs of a thread-block cluster instead (split-K): after the
// main loop every CTA sends, through distributed shared memory, the columns of its partial accumulator that a peer
// owns, and each CTA finishes its own share of the columns, adding the partial tiles in rank order (so results are
// reproducible bit for bit) -- no global scratch, no counters, and the epilogue runs on every SM.  The only waits
// between CTAs are the hardware's cluster barriers (the CTAs of a cluster are resident together by construction).
//
//   operand pre-pass   ONE kernel per layer and pass: a CTA owns 8 samples and ALL operand rows; it gathers the
//                      log-domain values (the product layer is folded in: a product's value is the sum of its
//                      children's rows), keeps them in shared memory, reduces the per-sample maximum, and writes
//                      exp(value - max) as bf16 hi / lo operand tiles.  No element_mars, no separate maximum pass.
//   GEMM               warp 0 streams 32-deep operand slices with bulk copies into a ring of 4-8 stages, one thread
//                      of warp 1 issues three tcgen05.mma per 16-deep step (hi x hi, hi x lo, lo x hi; N = 64, 128
//                      or 256) into a TMEM accumulator, warps 2-5 finish: log + shift (forward), + element value and
//                      a direct store into the children's flow rows (element flows, product backward folded in),
//                      or parameter * sum -> atomic add (parameter flows).
//   parameter flows    as before ONE product per group of layers that share parameters, contraction over the
//                      concatenated batches; its operands (X = exp(flow - value - shift) and Y = exp(child value
//                      + shift)) are staged per layer by one kernel; samples of consecutive layers are packed
//                      back to back, so small per-rank batches (data parallelism) do not pad the contraction.
//
// B operand tile of (group g, column tile jt, chunk c): [8 K-groups][DN samples][8 x bf16] hi, then the same for lo
// (2 * DN * 128 bytes).  A tiles are the pre-split parameter tiles of pcx_pack_sum_params (unchanged).
//
// This file is included by pcx_sum_tc.cu after pcx_sum_dense.cuh and uses their helpers and the status word.
#pragma once

namespace {

constexpr int W_STEP = 32;                          // contraction depth per pipeline stage
constexpr int W_A_HALF = (W_STEP / 8) * BM * 16;    // 8 KB: hi (or lo) part of the A operand of one stage
constexpr int W_THREADS = 192;                      // warp 0 copies, warp 1 multiplies, warps 2-5 finish
constexpr int W_PREP_THREADS = 512;
constexpr int W_PREP_SAMPLES = 8;                   // samples per pre-pass CTA (one 32-byte sector per row)
constexpr int W_MAX_DEPTH = 6144;                   // operand rows the pre-pass can hold in shared memory

template <int DN>
struct WideCfg {
    static constexpr int B_HALF = (W_STEP / 8) * DN * 16;               // hi (or lo) part of the B operand of one stage
    static constexpr int STAGE = 2 * W_A_HALF + 2 * B_HALF;            // DN = 256: 48 KB, 128: 32 KB, 64: 24 KB
    static constexpr int STAGES = (DN == 256) ? 4 : ((DN == 128) ? 6 : 8);
    static constexpr int SMEM = STAGES * STAGE + 1024;
    static constexpr int B_TILE = 2 * 8 * DN * 16;                     // one 64-deep operand tile, hi then lo
};

enum WideEpi { W_FWD = 0, W_ELE = 1, W_PAR = 2 };

struct WideArgs {
    const uint8_t* a_tiles;     // A tile of (row tile mt, chunk c) at a_tiles + (mt * n_chunks + c) * 32 KB
    const uint8_t* b_tiles;     // B tile of (operand row r, chunk c) at b_tiles + (r * n_chunks + c) * B_TILE
    const int32_t* b_group;     // FWD / ELE: group of every table row (rows of a group share their operand)
    int n_chunks;               // 64-deep chunks of the whole contraction
    int splits;                 // CTAs per output tile along the contraction (divides n_chunks)
    int n_ct;                   // FWD / ELE: column tiles per group
    int row_block;              // rows per table row (multiple of 128)
    int B;
    int logspace;
    int terms;
    const int32_t* rows;        // FWD: nids   ELE: chids
    float* out;                 // FWD: node_mars   ELE: element_flows (unless direct)   PAR: param_flows
    const float* shift;         // FWD / ELE: [n_groups, B] per-sample shifts
    const float* emars;         // ELE, products not folded: element_mars
    const float* nmars;         // ELE, products folded: node_mars (an element's value = sum of its children's rows)
    float* nflows;              // ELE, direct: node_flows (an element's flow is stored into its children's rows)
    const int32_t* fkids;       // ELE, folded: [n_rows * row_block][fc] child rows of every element (0 = none)
    int fc;
    int direct;
    const float* params;        // PAR
    const int32_t* cids;        // PAR: [n_rows, K]
    const int32_t* pids;        // PAR
    const int32_t* pfids;       // PAR
    int K;                      // PAR: table width
};

// ---- programmatic dependent launch --------------------------------------------------------------------------------
// A pass over a deep circuit is a chain of short kernels (pre-pass, GEMM, pre-pass, GEMM, ...), each of which needs
// all of its predecessor's output.  Launched with the programmatic-serialization attribute, a kernel may become
// resident while its predecessor is still running and set itself up (barriers, tensor memory, index arithmetic); it
// then waits here until the predecessor has completed and its writes are visible.  `launch_dependents` lets the
// successor start that early.  Off (plain stream order) when pcx_set_dependent_launch(0) was called.
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void griddep_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
int g_wide_pdl = 1;

// ---- L2 residency -----------------------------------------------------------------------------------------------------
// The parameter tiles of a layer are read once per pass and, for tied layers, again by the next layer a few tens of
// microseconds later: they are fetched with an evict-last policy so that the operand tiles and value rows streaming
// through L2 in between do not push them out.
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
    return p;
}
// Streaming (evict-first) variant of store_split8 for operands that are written once and read much later.
__device__ __forceinline__ void store_split8_streaming(uint4* hi, uint4* lo, const float* x) {
    uint32_t h[4], l[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const __nv_bfloat162 hp = __floats2bfloat162_rn(x[2 * j], x[2 * j + 1]);
        h[j] = *reinterpret_cast<const uint32_t*>(&hp);
        const float h0 = __uint_as_float(h[j] << 16), h1 = __uint_as_float(h[j] & 0xffff0000u);
        const __nv_bfloat162 lp = __floats2bfloat162_rn(x[2 * j] - h0, x[2 * j + 1] - h1);
        l[j] = *reinterpret_cast<const uint32_t*>(&lp);
    }
    __stcs(hi, make_uint4(h[0], h[1], h[2], h[3]));
    __stcs(lo, make_uint4(l[0], l[1], l[2], l[3]));
}
__device__ __forceinline__ void bulk_copy_g2s_hint(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar,
                                                   uint64_t policy) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
                 ::"r"(smem_u32(smem_dst)), "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar)), "l"(policy) : "memory");
}

// ---- thread-block cluster helpers (the CTAs that share one output tile) -----------------------------------------
__device__ __forceinline__ uint32_t cluster_cta_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// Barrier over all threads of all CTAs of the cluster (release / acquire); every warp must arrive converged.
__device__ __forceinline__ void cluster_sync_all() {
    __syncwarp();
    asm volatile("barrier.cluster.arrive.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.aligned;" ::: "memory");
}
// Address of `smem_addr` (an address in this CTA's shared memory) in the shared memory of the CTA with rank `rank`.
__device__ __forceinline__ uint32_t cluster_map(uint32_t smem_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_store(uint32_t addr, float v) {
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}

// Element flows: value of the element in row (i, r0 + row) for the 32 columns from b0 on, and its child rows.
__device__ __forceinline__ void wide_gather_em(const WideArgs& a, int64_t i, int r0, int row, int b0, float* em, int* fk) {
    const int nv = min(32, a.B - b0);
    if (a.fkids != nullptr) {                                        // element value = sum of the children's rows
        const int64_t erow = i * a.row_block + r0 + row;
        bool any = false;
#pragma unroll
        for (int q = 0; q < 8; ++q) { fk[q] = (q < a.fc) ? a.fkids[erow * a.fc + q] : 0; any = any || fk[q] != 0; }
#pragma unroll
        for (int j = 0; j < 32; ++j) em[j] = any ? 0.0f : PCX_NEG_INF;
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            if (fk[q] != 0) {
                const float* src = a.nmars + (int64_t)fk[q] * a.B + b0;
#pragma unroll
                for (int j = 0; j < 32; j += 4) {
                    if (j < nv) {
                        const float4 c4 = *reinterpret_cast<const float4*>(src + j);
                        em[j] += c4.x; em[j + 1] += c4.y; em[j + 2] += c4.z; em[j + 3] += c4.w;
                    }
                }
            }
        }
    } else {
        const int64_t orow = ((int64_t)a.rows[i] + r0 + row) * a.B + b0;
#pragma unroll
        for (int q = 0; q < 8; ++q) fk[q] = 0;
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
            if (j < nv) {
                const float4 e4 = *reinterpret_cast<const float4*>(a.emars + orow + j);
                em[j] = e4.x; em[j + 1] = e4.y; em[j + 2] = e4.z; em[j + 3] = e4.w;
            }
        }
    }
}

// Epilogue of one row and 32 consecutive columns.
template <int EPI, int DN>
__device__ __forceinline__ void wide_finish(const WideArgs& a, int64_t i, int r0, int row, int nt, int cb, const float* v,
                                            const float* pre_em = nullptr, const int* pre_fk = nullptr) {
    if (EPI == W_PAR) {
#pragma unroll 4
        for (int j = 0; j < 32; ++j) {
            const int e = nt * DN + cb + j;
            if (e >= a.K) break;
            if (a.cids[i * a.K + e] == 0) continue;
            const float pf = a.params[(int64_t)a.pids[i * a.K + e] + r0 + row] * v[j];
            if (pf != 0.0f) atomicAdd(a.out + (int64_t)a.pfids[i * a.K + e] + r0 + row, pf);
        }
        return;
    }
    const int b0 = nt * DN + cb;
    if (b0 >= a.B) return;
    const float* sh = a.shift + (int64_t)a.b_group[i] * a.B + b0;
    const int64_t erow = i * a.row_block + r0 + row;                 // index of this output row in its table
    const int64_t orow = ((int64_t)a.rows[i] + r0 + row) * a.B + b0;
    const int nv = min(32, a.B - b0);                                // valid columns: B is a multiple of 4
    float o[32];
#pragma unroll
    for (int j = 0; j < 32; j += 4) {
        if (j < nv) {
            const float4 m4 = *reinterpret_cast<const float4*>(sh + j);
            const float m[4] = {m4.x, m4.y, m4.z, m4.w};
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                const float x = v[j + t];
                if (EPI == W_FWD) o[j + t] = (m[t] == PCX_NEG_INF) ? PCX_NEG_INF : __logf(fmaxf(x, 1e-24f)) + m[t];
                else o[j + t] = (m[t] == PCX_NEG_INF || x <= 0.0f) ? PCX_NEG_INF : __logf(x) + m[t];
            }
        }
    }
    if (EPI == W_FWD) {
#pragma unroll
        for (int j = 0; j < 32; j += 4)
            if (j < nv) *reinterpret_cast<float4*>(a.out + orow + j) = make_float4(o[j], o[j + 1], o[j + 2], o[j + 3]);
        return;
    }
    // element flows: the element's value (gathered here, or already gathered while the main loop ran), then the stores
    float em[32];
    int fk[8];
    if (pre_em != nullptr) {
#pragma unroll
        for (int j = 0; j < 32; ++j) em[j] = pre_em[j];
#pragma unroll
        for (int q = 0; q < 8; ++q) fk[q] = pre_fk[q];
    } else {
        wide_gather_em(a, i, r0, row, b0, em, fk);
    }
#pragma unroll
    for (int j = 0; j < 32; ++j) {
        if (j < nv) {
            o[j] = (o[j] == PCX_NEG_INF || em[j] == PCX_NEG_INF) ? PCX_NEG_INF : o[j] + em[j];
            if (!a.logspace) o[j] = __expf(o[j]);
        }
    }
    if (a.fkids != nullptr && a.direct) {                             // every child has this one parent: plain stores
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            if (fk[q] != 0) {
                float* dst = a.nflows + (int64_t)fk[q] * a.B + b0;
#pragma unroll
                for (int j = 0; j < 32; j += 4)
                    if (j < nv) *reinterpret_cast<float4*>(dst + j) = make_float4(o[j], o[j + 1], o[j + 2], o[j + 3]);
            }
        }
    } else {
#pragma unroll
        for (int j = 0; j < 32; j += 4)
            if (j < nv) *reinterpret_cast<float4*>(a.out + orow + j) = make_float4(o[j], o[j + 1], o[j + 2], o[j + 3]);
    }
}

template <int EPI, int DN>
__global__ void __launch_bounds__(W_THREADS, 1) wide_gemm_kernel(const WideArgs a) {
    using C = WideCfg<DN>;
    constexpr int ACCS = (EPI == W_PAR) ? 2 : 1;         // the long contraction of the parameter flows alternates two
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ uint64_t s_full[C::STAGES], s_empty[C::STAGES], s_done;
    __shared__ uint32_t s_tmem;
    __shared__ volatile int s_fail;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int64_t mt = blockIdx.x;                  // 128-row tile
    const int nt = blockIdx.y;                      // FWD / ELE: sample tile      PAR: edge tile
    const int split = blockIdx.z;
    const int tiles_r = a.row_block / BM;
    const int64_t i = mt / tiles_r;
    const int r0 = (int)(mt % tiles_r) * BM;
    const int chunks_here = a.n_chunks / a.splits;
    const int c_begin = split * chunks_here;
    const int n_steps = chunks_here * (KC / W_STEP);

    if (tid == 0) {
        for (int s = 0; s < C::STAGES; ++s) { mbar_init(&s_full[s], 1); mbar_init(&s_empty[s], 1); }
        mbar_init(&s_done, 1);
        fence_mbar_init();
        s_fail = 0;
    }
    if (warp == 0) tmem_alloc(&s_tmem, (ACCS * DN < 32) ? 32 : ACCS * DN);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = s_tmem;
    griddep_wait();                                 // everything above overlapped the previous kernel's tail
    griddep_launch_dependents();

    const int64_t b_row = (EPI == W_PAR) ? (int64_t)nt : (int64_t)a.b_group[i] * a.n_ct + nt;
    const uint8_t* a_src = a.a_tiles + ((size_t)mt * a.n_chunks + c_begin) * (2 * A_TILE);
    const uint8_t* b_src = a.b_tiles + ((size_t)b_row * a.n_chunks + c_begin) * C::B_TILE;

    if (warp == 0) {
        // ---- copy warp: lane 0 waits for the stage and arms its barrier, four lanes move one piece each -------------
        int armed = 0;
        const uint64_t keep = l2_policy_evict_last();
        for (int t = 0; t < n_steps; ++t) {
            const int s = t % C::STAGES;
            int stop = 0;
            if (lane == 0) {
                if (t >= C::STAGES && !mbar_wait(&s_empty[s], (uint32_t)((t / C::STAGES - 1) & 1))) s_fail = 1;
                stop = s_fail;
                if (!stop) mbar_expect_tx(&s_full[s], C::STAGE);
            }
            stop = __shfl_sync(0xffffffffu, stop, 0);
            if (stop) break;
            const int c = t / (KC / W_STEP), h = t % (KC / W_STEP);
            uint8_t* dst = smem + s * C::STAGE;
            const uint8_t* a_at = a_src + (size_t)c * (2 * A_TILE) + h * W_A_HALF;
            const uint8_t* b_at = b_src + (size_t)c * C::B_TILE + h * C::B_HALF;
            if (EPI == W_PAR) {                      // staged operands, shared by the CTAs of a wave only: default policy
                if (lane == 0) bulk_copy_g2s(dst, a_at, W_A_HALF, &s_full[s]);
                if (lane == 1) bulk_copy_g2s(dst + W_A_HALF, a_at + A_TILE, W_A_HALF, &s_full[s]);
            } else {                                 // parameter tiles: keep them for the next (tied) layer
                if (lane == 0) bulk_copy_g2s_hint(dst, a_at, W_A_HALF, &s_full[s], keep);
                if (lane == 1) bulk_copy_g2s_hint(dst + W_A_HALF, a_at + A_TILE, W_A_HALF, &s_full[s], keep);
            }
            if (lane == 2) bulk_copy_g2s(dst + 2 * W_A_HALF, b_at, C::B_HALF, &s_full[s]);
            if (lane == 3) bulk_copy_g2s(dst + 2 * W_A_HALF + C::B_HALF, b_at + C::B_TILE / 2, C::B_HALF, &s_full[s]);
            armed = t + 1;
        }
        if (lane == 0 && s_fail) {
            // let the copies that are still in flight land before this CTA's shared memory goes away
            for (int t = max(0, armed - C::STAGES); t < armed; ++t)
                mbar_wait(&s_full[t % C::STAGES], (uint32_t)((t / C::STAGES) & 1), 1u << 16);
        }
    } else if (warp == 1) {
        // ---- multiply thread ----------------------------------------------------------------------------
        if (lane == 0) {
            const uint32_t idesc = idesc_bf16_f32(BM, DN);
            for (int t = 0; t < n_steps; ++t) {
                const int s = t % C::STAGES;
                if (!mbar_wait(&s_full[s], (uint32_t)((t / C::STAGES) & 1))) { s_fail = 2; break; }
                if (s_fail) break;
                tc_fence_after_sync();
                const uint32_t sa = smem_u32(smem + s * C::STAGE), sb = sa + 2 * W_A_HALF;
                const uint32_t acc = tmem + (uint32_t)((t % ACCS) * DN);
#pragma unroll
                for (int ks = 0; ks < W_STEP / 16; ++ks) {
                    const uint64_t dAh = smem_desc(sa + ks * 2 * (BM * 16), BM * 16, 128);
                    const uint64_t dAl = smem_desc(sa + W_A_HALF + ks * 2 * (BM * 16), BM * 16, 128);
                    const uint64_t dBh = smem_desc(sb + ks * 2 * (DN * 16), DN * 16, 128);
                    const uint64_t dBl = smem_desc(sb + C::B_HALF + ks * 2 * (DN * 16), DN * 16, 128);
                    mma_bf16_ss(acc, dAh, dBh, idesc, (t >= ACCS || ks > 0) ? 1u : 0u);
                    if (a.terms == 3) {
                        mma_bf16_ss(acc, dAh, dBl, idesc, 1u);
                        mma_bf16_ss(acc, dAl, dBh, idesc, 1u);
                    }
                }
                mma_commit(&s_empty[s]);            // the stage is free once these products have read it
            }
            mma_commit(&s_done);
        }
    }
    if (warp < 2 && a.splits > 1) {         // the cluster barriers of the epilogue count every thread of the cluster
        cluster_sync_all();
        cluster_sync_all();
    }
    if (warp >= 2) {
        // ---- epilogue warps: TMEM lane quarter warp % 4, one output row per thread --------------------------
        const int lq = warp & 3;
        const int row = lq * 32 + lane;
        // Element flows, tile split over 4 or 8 CTAs: this CTA finishes at most 64 columns, and what the epilogue needs
        // beside the accumulator -- the elements' values, gathered from their child rows -- does not depend on the
        // products.  Fetch it now, while the main loop runs, instead of after it.
        const int QW0 = DN / a.splits;
        const bool pre = (EPI == W_ELE) && a.splits > 1 && QW0 <= 64;
        float em0[32], em1[32];
        int fk0[8];
        if (pre) {
            const int c0 = nt * DN + (int)cluster_cta_rank() * QW0;
            if (c0 < a.B) wide_gather_em(a, i, r0, row, c0, em0, fk0);
            if (QW0 == 64 && c0 + 32 < a.B) wide_gather_em(a, i, r0, row, c0 + 32, em1, fk0);
        }
        bool ok = mbar_wait(&s_done, 0u, 1u << 24);
        if (!ok) s_fail = 3;
        ok = ok && (s_fail == 0);
        tc_fence_after_sync();
        const uint32_t tbase = tmem + ((uint32_t)(lq * 32) << 16);
        const int used = n_steps < ACCS ? n_steps : ACCS;
        if (a.splits == 1) {
            if (ok) {
#pragma unroll 1
                for (int cb = 0; cb < DN; cb += 32) {
                    float v[32];
                    tmem_ld<32>(tbase + (uint32_t)cb, v);
                    if (ACCS == 2 && used == 2) {
                        float u[32];
                        tmem_ld<32>(tbase + (uint32_t)(DN + cb), u);
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] += u[j];
                    }
                    wide_finish<EPI, DN>(a, i, r0, row, nt, cb, v);
                }
            }
        } else {
            // split contraction: this CTA finishes columns [rank * QW, (rank + 1) * QW) of the tile.  Peers' stage
            // buffers are free once every CTA's products are complete (first cluster barrier); the partial columns a
            // peer owns go into its shared memory as recv[sender][column][row]; after the second barrier the partials
            // are added in rank order.
            const int QW = DN / a.splits;
            const uint32_t me = cluster_cta_rank();
            cluster_sync_all();
            const uint32_t recv = smem_u32(smem);
            for (int r = 0; r < a.splits; ++r) {
                if ((uint32_t)r == me) continue;
                const uint32_t dst = cluster_map(recv + (uint32_t)(((int)me * QW) * BM + row) * 4u, (uint32_t)r);
#pragma unroll 1
                for (int cb = 0; cb < QW; cb += 32) {
                    float v[32];
                    if (ok) tmem_ld<32>(tbase + (uint32_t)(r * QW + cb), v);
                    else {
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = 0.0f;
                    }
#pragma unroll
                    for (int j = 0; j < 32; ++j) cluster_store(dst + (uint32_t)((cb + j) * BM) * 4u, v[j]);
                }
            }
            cluster_sync_all();
            const float* mine = reinterpret_cast<const float*>(smem);
            if (ok) {
#pragma unroll 1
                for (int cb = 0; cb < QW; cb += 32) {
                    float own[32], v[32];
                    tmem_ld<32>(tbase + (uint32_t)((int)me * QW + cb), own);
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = 0.0f;
                    for (int q = 0; q < a.splits; ++q) {          // rank order: the sum is reproducible
                        if ((uint32_t)q == me) {
#pragma unroll
                            for (int j = 0; j < 32; ++j) v[j] += own[j];
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j) v[j] += mine[((q * QW) + cb + j) * BM + row];
                        }
                    }
                    if (pre) wide_finish<EPI, DN>(a, i, r0, row, nt, (int)me * QW + cb, v, cb == 0 ? em0 : em1, fk0);
                    else wide_finish<EPI, DN>(a, i, r0, row, nt, (int)me * QW + cb, v);
                }
            }
        }
        tc_fence_before_sync();
    }
    __syncthreads();
    if (tid == 0 && s_fail != 0) atomicCAS(&g_tc_status, 0, 600 + 10 * EPI + s_fail);
    if (warp == 0) tmem_dealloc(tmem, (ACCS * DN < 32) ? 32 : ACCS * DN);
}

// ---- operand pre-passes --------------------------------------------------------------------------------------
struct WidePrepArgs {
    const float* src;           // FWD: element_mars, or node_mars when products are folded     ELE / PAR: node_flows
    const float* src2;          // ELE / PAR: node_mars
    const int32_t* kids;        // FWD: cids [n, K]   ELE: parids [n, P]   PAR: nids [n]
    const int32_t* fkids;       // FWD folded: [n * K][fc] child rows of every listed element
    const int32_t* group_row;   // [n_groups] a table row that stands for the group (PAR: unused)
    int fc;
    int K;                      // table width (FWD: children, ELE: parent blocks, PAR: 1)
    int par_block;              // ELE: parent block size   PAR: block size   FWD: 1
    int depth;                  // operand rows per group
    int depth_pad;              // rounded up to whole 64-deep chunks
    int B;
    int logspace;
    int mode;                   // 0 FWD, 1 ELE, 2 PAR
    int DN, n_ct, n_chunks;     // FWD / ELE tile geometry
    uint8_t* tiles;             // FWD / ELE: operand tiles     PAR: X tiles
    float* shift;               // FWD / ELE: [n_groups, B]
    // PAR only
    uint8_t* y_tiles;
    const float* emars;         // products not folded
    const int32_t* cids_row;    // [Kfw] children of the layer's rows (every row lists the same)
    const int32_t* fk_row;      // folded: [Kfw][fc]
    int Kfw;
    int n_chunks_total, slot;
    int cs;                     // CTAs (one cluster) that share the operand rows of a group
};

// Eight consecutive samples of operand row k, in the log domain.  Every load is unconditional (row 0 of each value
// buffer exists; what it holds is replaced by a select), so that the loads of several rows are in flight together.
template <int FC>
__device__ __forceinline__ void wide_prep_value(const WidePrepArgs& a, int g, int k, int b0, float* v) {
    const bool in = k < a.depth;
    if (a.mode == 0) {
        const int64_t at = (int64_t)a.group_row[g] * a.K + (in ? k : 0);
        if (FC == 0) {
            const int cid = in ? a.kids[at] : 0;
            const float4 p = *reinterpret_cast<const float4*>(a.src + (int64_t)cid * a.B + b0);
            const float4 q = *reinterpret_cast<const float4*>(a.src + (int64_t)cid * a.B + b0 + 4);
            const float x[8] = {p.x, p.y, p.z, p.w, q.x, q.y, q.z, q.w};
#pragma unroll
            for (int s = 0; s < 8; ++s) v[s] = cid != 0 ? x[s] : PCX_NEG_INF;
            return;
        }
        int fk[FC > 0 ? FC : 1];
        bool any = false;
#pragma unroll
        for (int j = 0; j < FC; ++j) { fk[j] = in ? a.fkids[at * FC + j] : 0; any = any || fk[j] != 0; }
        float4 p[FC > 0 ? FC : 1], q[FC > 0 ? FC : 1];
#pragma unroll
        for (int j = 0; j < FC; ++j) {
            p[j] = *reinterpret_cast<const float4*>(a.src + (int64_t)fk[j] * a.B + b0);
            q[j] = *reinterpret_cast<const float4*>(a.src + (int64_t)fk[j] * a.B + b0 + 4);
        }
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int j = 0; j < FC; ++j) {
            if (fk[j] != 0) {
                acc[0] += p[j].x; acc[1] += p[j].y; acc[2] += p[j].z; acc[3] += p[j].w;
                acc[4] += q[j].x; acc[5] += q[j].y; acc[6] += q[j].z; acc[7] += q[j].w;
            }
        }
#pragma unroll
        for (int s = 0; s < 8; ++s) v[s] = any ? acc[s] : PCX_NEG_INF;
        return;
    }
    const int kk = in ? k : 0;
    int pr;
    if (a.mode == 1) pr = a.kids[(int64_t)a.group_row[g] * a.K + kk / a.par_block];
    else pr = a.kids[kk / a.par_block];
    const bool live = in && pr != 0;
    const int64_t r = live ? (int64_t)pr + kk % a.par_block : 0;
    const float4 f0 = *reinterpret_cast<const float4*>(a.src + r * a.B + b0);
    const float4 f1 = *reinterpret_cast<const float4*>(a.src + r * a.B + b0 + 4);
    const float4 m0 = *reinterpret_cast<const float4*>(a.src2 + r * a.B + b0);
    const float4 m1 = *reinterpret_cast<const float4*>(a.src2 + r * a.B + b0 + 4);
    const float f[8] = {f0.x, f0.y, f0.z, f0.w, f1.x, f1.y, f1.z, f1.w};
    const float m[8] = {m0.x, m0.y, m0.z, m0.w, m1.x, m1.y, m1.z, m1.w};
#pragma unroll
    for (int s = 0; s < 8; ++s) {
        float x = f[s];
        if (!a.logspace) x = (x > 0.0f) ? __logf(x) : PCX_NEG_INF;
        v[s] = (!live || m[s] == PCX_NEG_INF || x == PCX_NEG_INF) ? PCX_NEG_INF : x - m[s];
    }
}

// The operand rows of a group are split over the `cs` CTAs of a cluster (whole 64-row chunks each); every CTA stages
// the log-domain values of ITS rows for the eight samples in shared memory ([8][ld] floats) and the per-sample maximum
// over ALL rows is formed by exchanging the CTAs' maxima through distributed shared memory.  Returns it in sh[0..8).
template <int FC>
__device__ __forceinline__ void wide_prep_stage(const WidePrepArgs& a, int g, int b0, int k_begin, int rows_here,
                                                float* s_val, int ld, float* s_red, float* s_peer, float* sh) {
    const int tid = threadIdx.x;
    float mx[8];
#pragma unroll
    for (int s = 0; s < 8; ++s) mx[s] = PCX_NEG_INF;
    for (int k = tid; k < rows_here; k += 2 * W_PREP_THREADS) {      // two rows per round: their loads overlap
        const int k2 = k + W_PREP_THREADS;
        float v[8], w[8];
        wide_prep_value<FC>(a, g, k_begin + k, b0, v);
        wide_prep_value<FC>(a, g, k2 < rows_here ? k_begin + k2 : a.depth, b0, w);
#pragma unroll
        for (int s = 0; s < 8; ++s) { s_val[s * ld + k] = v[s]; mx[s] = fmaxf(mx[s], v[s]); }
        if (k2 < rows_here) {
#pragma unroll
            for (int s = 0; s < 8; ++s) { s_val[s * ld + k2] = w[s]; mx[s] = fmaxf(mx[s], w[s]); }
        }
    }
#pragma unroll
    for (int s = 0; s < 8; ++s)
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx[s] = fmaxf(mx[s], __shfl_xor_sync(0xffffffffu, mx[s], o));
    if ((tid & 31) == 0) {
#pragma unroll
        for (int s = 0; s < 8; ++s) s_red[(tid >> 5) * 8 + s] = mx[s];
    }
    __syncthreads();
    if (a.cs > 1) {
        const uint32_t me = cluster_cta_rank();
        if (tid < 8) {
            float m = PCX_NEG_INF;
#pragma unroll
            for (int w = 0; w < W_PREP_THREADS / 32; ++w) m = fmaxf(m, s_red[w * 8 + tid]);
            for (int r = 0; r < a.cs; ++r)
                cluster_store(cluster_map(smem_u32(s_peer + me * 8 + tid), (uint32_t)r), m);
        }
        cluster_sync_all();
#pragma unroll
        for (int s = 0; s < 8; ++s) {
            float m = PCX_NEG_INF;
            for (int r = 0; r < a.cs; ++r) m = fmaxf(m, s_peer[r * 8 + s]);
            sh[s] = m;
        }
    } else {
#pragma unroll
        for (int s = 0; s < 8; ++s) {
            float m = PCX_NEG_INF;
#pragma unroll
            for (int w = 0; w < W_PREP_THREADS / 32; ++w) m = fmaxf(m, s_red[w * 8 + s]);
            sh[s] = m;
        }
    }
}

// FWD / ELE operand tiles (contraction over operand rows).  Grid (ceil(B / 8), n_groups, cs), clusters of cs along z,
// 512 threads.
template <int FC>
__global__ void __launch_bounds__(W_PREP_THREADS) wide_prep_rows_kernel(const WidePrepArgs a) {
    extern __shared__ float s_dyn[];
    __shared__ float s_red[(W_PREP_THREADS / 32) * 8];
    __shared__ float s_peer[8 * 8];
    const int tid = threadIdx.x, g = blockIdx.y;
    const int b0 = blockIdx.x * W_PREP_SAMPLES;                      // B is a multiple of 8
    const int rows_here = a.depth_pad / a.cs;
    const int k_begin = blockIdx.z * rows_here;
    const int ld = rows_here + 4;
    float sh[8];
    griddep_wait();
    griddep_launch_dependents();
    wide_prep_stage<FC>(a, g, b0, k_begin, rows_here, s_dyn, ld, s_red, s_peer, sh);
    if (blockIdx.z == 0 && tid < 8) a.shift[(int64_t)g * a.B + b0 + tid] = sh[tid];

    const int tile_bytes = 2 * 8 * a.DN * 16;
    for (int it = tid; it < rows_here; it += W_PREP_THREADS) {       // (rows / 8) K-groups x 8 samples
        const int s = it & 7, kl = it >> 3;
        const float4 p = *reinterpret_cast<const float4*>(s_dyn + s * ld + kl * 8);
        const float4 q = *reinterpret_cast<const float4*>(s_dyn + s * ld + kl * 8 + 4);
        const float x[8] = {p.x, p.y, p.z, p.w, q.x, q.y, q.z, q.w};
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = (x[j] == PCX_NEG_INF || sh[s] == PCX_NEG_INF) ? 0.0f : __expf(x[j] - sh[s]);
        const int kg = k_begin / 8 + kl;
        const int b = b0 + s;
        const int jt = b / a.DN, bl = b % a.DN;
        uint8_t* tile = a.tiles + (((size_t)g * a.n_ct + jt) * a.n_chunks + (kg >> 3)) * tile_bytes;
        uint8_t* dst = tile + (size_t)(kg & 7) * (a.DN * 16) + bl * 16;
        store_split8(reinterpret_cast<uint4*>(dst), reinterpret_cast<uint4*>(dst + tile_bytes / 2), v);
    }
}

// Parameter-flow operands of one layer (contraction over the batch), into the columns of slot `slot`:
// X tile (row tile mt, chunk cc): [8 sample groups][128 rows][8 samples] hi, lo; Y tile (edge tile et of 256, chunk cc):
// [8 sample groups][256 edges][8 samples] hi, lo.  The concatenated sample index of (slot, b) is slot * B + b.
// Grid (ceil(B / 8), 1, cs), clusters of cs along z (rows and edges are split over the cluster), 512 threads.
template <int FC>
__global__ void __launch_bounds__(W_PREP_THREADS) wide_prep_par_kernel(const WidePrepArgs a) {
    extern __shared__ float s_dyn[];
    __shared__ float s_red[(W_PREP_THREADS / 32) * 8];
    __shared__ float s_peer[8 * 8];
    const int tid = threadIdx.x;
    const int b0 = blockIdx.x * W_PREP_SAMPLES;
    const int rows_here = a.depth_pad / a.cs;
    const int k_begin = blockIdx.z * rows_here;
    const int ld = rows_here + 4;
    float sh[8];
    griddep_wait();
    griddep_launch_dependents();
    wide_prep_stage<0>(a, 0, b0, k_begin, rows_here, s_dyn, ld, s_red, s_peer, sh);   // mode 2: flow - value of the layer's rows

    const int64_t q0 = (int64_t)a.slot * a.B + b0;
    const int64_t cc = q0 / KC;
    const int sg = (int)(q0 % KC) / 8;
    for (int rl = tid; rl < rows_here; rl += W_PREP_THREADS) {
        const int r = k_begin + rl;
        if (r >= a.depth) break;
        float v[8];
#pragma unroll
        for (int s = 0; s < 8; ++s) {
            const float x = s_dyn[s * ld + rl];
            v[s] = (x == PCX_NEG_INF || sh[s] == PCX_NEG_INF) ? 0.0f : __expf(x - sh[s]);
        }
        uint8_t* tile = a.tiles + ((size_t)(r / BM) * a.n_chunks_total + cc) * (2 * A_TILE);
        uint8_t* dst = tile + sg * (BM * 16) + (r % BM) * 16;
        store_split8_streaming(reinterpret_cast<uint4*>(dst), reinterpret_cast<uint4*>(dst + A_TILE), v);
    }
    constexpr int EN = 256;
    const int e_per = (a.Kfw + a.cs - 1) / a.cs;
    const int e_end = min(a.Kfw, (int)(blockIdx.z + 1) * e_per);
    for (int e = blockIdx.z * e_per + tid; e < e_end; e += W_PREP_THREADS) {
        float em[8];
        bool live;
        if (FC == 0) {
            const int cid = a.cids_row[e];
            live = cid != 0;
            const float4 p = *reinterpret_cast<const float4*>(a.emars + (int64_t)cid * a.B + b0);
            const float4 q = *reinterpret_cast<const float4*>(a.emars + (int64_t)cid * a.B + b0 + 4);
            em[0] = p.x; em[1] = p.y; em[2] = p.z; em[3] = p.w; em[4] = q.x; em[5] = q.y; em[6] = q.z; em[7] = q.w;
        } else {
            live = false;
#pragma unroll
            for (int s = 0; s < 8; ++s) em[s] = 0.0f;
            int fk[FC > 0 ? FC : 1];
            float4 p[FC > 0 ? FC : 1], q[FC > 0 ? FC : 1];
#pragma unroll
            for (int j = 0; j < FC; ++j) fk[j] = a.fk_row[(int64_t)e * FC + j];
#pragma unroll
            for (int j = 0; j < FC; ++j) {
                p[j] = *reinterpret_cast<const float4*>(a.src2 + (int64_t)fk[j] * a.B + b0);
                q[j] = *reinterpret_cast<const float4*>(a.src2 + (int64_t)fk[j] * a.B + b0 + 4);
            }
#pragma unroll
            for (int j = 0; j < FC; ++j) {
                if (fk[j] != 0) {
                    live = true;
                    em[0] += p[j].x; em[1] += p[j].y; em[2] += p[j].z; em[3] += p[j].w;
                    em[4] += q[j].x; em[5] += q[j].y; em[6] += q[j].z; em[7] += q[j].w;
                }
            }
        }
        float v[8];
#pragma unroll
        for (int s = 0; s < 8; ++s)
            v[s] = (!live || em[s] == PCX_NEG_INF || sh[s] == PCX_NEG_INF) ? 0.0f : fminf(__expf(em[s] + sh[s]), 3.0e38f);
        uint8_t* tile = a.y_tiles + ((size_t)(e / EN) * a.n_chunks_total + cc) * (2 * 8 * EN * 16);
        uint8_t* dst = tile + sg * (EN * 16) + (e % EN) * 16;
        store_split8_streaming(reinterpret_cast<uint4*>(dst), reinterpret_cast<uint4*>(dst + 8 * EN * 16), v);
    }
}

// CTAs per group that share the operand rows of a pre-pass (= its cluster size): whole 64-row chunks each.
inline int wide_prep_cluster(int n_chunks) {
    int cs = 1;
    while (cs < 4 && n_chunks % (cs * 2) == 0 && n_chunks / (cs * 2) >= 4) cs *= 2;
    return cs;
}

template <typename Kern>
int wide_launch_prep(Kern kern, const WidePrepArgs& p, dim3 grid, size_t smem, cudaStream_t st) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(W_PREP_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    int n_attr = 0;
    if (grid.z > 1) {
        attr[n_attr].id = cudaLaunchAttributeClusterDimension;
        attr[n_attr].val.clusterDim.x = 1;
        attr[n_attr].val.clusterDim.y = 1;
        attr[n_attr].val.clusterDim.z = grid.z;
        ++n_attr;
    }
    if (g_wide_pdl) {
        attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
        ++n_attr;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n_attr;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, p);
    if (e != cudaSuccess) return (int)e;
    PCX_LAUNCH_CHECK();
    return 0;
}

// Tile width in samples.  Batches of 64 and fewer also take 128-column tiles (the rest is padding): a 64-column tile can
// only be split two ways along the contraction (a CTA finishes at least 32 columns), which leaves 64 CTAs to stream
// the parameter image of a 4096-row layer, and that stream, not the padded multiplications, is what the time goes into.
inline int wide_dn(int B) { return B > 128 ? 256 : 128; }

// CTAs per output tile along the contraction (= cluster size): enough to fill the machine, a power of two that divides
// the chunks and leaves every CTA at least 32 columns of the tile to finish.
inline int wide_splits(int64_t tiles, int n_chunks, int DN) {
    int s = 1;
    while (s < 8 && s * 2 <= DN / 32 && tiles * (s * 2) <= 160 && n_chunks % (s * 2) == 0 && n_chunks / (s * 2) >= 2) s *= 2;
    return s;
}

template <typename Kern>
int wide_set_smem(Kern kern, int bytes, bool* done) {
    if (!*done) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
        if (e != cudaSuccess) return (int)e;
        *done = true;
    }
    return 0;
}

template <int EPI, int DN>
int launch_wide_gemm(const WideArgs& a, dim3 grid, cudaStream_t st) {
    static PcxOnce done;
    int rc = wide_set_smem(wide_gemm_kernel<EPI, DN>, WideCfg<DN>::SMEM, &done);
    if (rc != 0) return rc;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(W_THREADS);
    cfg.dynamicSmemBytes = WideCfg<DN>::SMEM;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    int n_attr = 0;
    if (grid.z > 1) {
        attr[n_attr].id = cudaLaunchAttributeClusterDimension;       // the CTAs that split one tile's contraction
        attr[n_attr].val.clusterDim.x = 1;
        attr[n_attr].val.clusterDim.y = 1;
        attr[n_attr].val.clusterDim.z = grid.z;
        ++n_attr;
    }
    if (g_wide_pdl) {
        attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
        ++n_attr;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n_attr;
    cudaError_t e = cudaLaunchKernelEx(&cfg, wide_gemm_kernel<EPI, DN>, a);
    if (e != cudaSuccess) return (int)e;
    PCX_LAUNCH_CHECK();
    return 0;
}

template <int EPI>
int launch_wide_gemm_dn(const WideArgs& a, int DN, dim3 grid, cudaStream_t st) {
    if (DN == 256) return launch_wide_gemm<EPI, 256>(a, grid, st);
    return launch_wide_gemm<EPI, 128>(a, grid, st);          // wide_dn() yields 256 or 128
}

template <int FC>
int launch_wide_prep_rows(const WidePrepArgs& p, dim3 grid, size_t smem, cudaStream_t st) {
    static PcxOnce done;
    int rc = wide_set_smem(wide_prep_rows_kernel<FC>, (W_MAX_DEPTH + 4) * 8 * (int)sizeof(float), &done);
    if (rc != 0) return rc;
    return wide_launch_prep(wide_prep_rows_kernel<FC>, p, grid, smem, st);
}

template <int FC>
int launch_wide_prep_par(const WidePrepArgs& p, dim3 grid, size_t smem, cudaStream_t st) {
    static PcxOnce done;
    int rc = wide_set_smem(wide_prep_par_kernel<FC>, (W_MAX_DEPTH + 4) * 8 * (int)sizeof(float), &done);
    if (rc != 0) return rc;
    return wide_launch_prep(wide_prep_par_kernel<FC>, p, grid, smem, st);
}

struct WideScratch {
    uint8_t* tiles;
    float* shift;
    int64_t total;
};

inline WideScratch wide_scratch(void* base, int n_groups, int depth, int B) {
    const int DN = wide_dn(B);
    const int64_t n_chunks = pcx_cdiv(depth, KC), n_ct = pcx_cdiv(B, DN);
    const size_t t = align256((size_t)n_groups * n_ct * n_chunks * (2 * 8 * DN * 16));
    const size_t s = align256((size_t)n_groups * B * sizeof(float));
    WideScratch w;
    uint8_t* b = reinterpret_cast<uint8_t*>(base);
    w.tiles = b;
    w.shift = reinterpret_cast<float*>(b + t);
    w.total = (int64_t)(t + s);
    return w;
}

// Measurement hook: when set (per host thread), the two-kernel operators record this event between their operand
// pre-pass and their GEMM, so that a caller timing the call with events of its own can tell the two kernels apart.
thread_local cudaEvent_t g_wide_stage_event = nullptr;

// Shared host part of the forward pass and the element flows.
static int wide_rows_op(int mode, float* out, const float* src, const float* src2, const float* emars, float* nflows,
                        const void* packed, const int32_t* rows, const int32_t* kids, const int32_t* fkids_prep,
                        const int32_t* fkids_epi, int fc, int direct, const int32_t* row_group, const int32_t* group_row,
                        int n_groups, void* scratch, int64_t scratch_bytes, int64_t n_rows, int K,
                        int row_block, int par_block, int B, int logspace, cudaStream_t st) {
    if (n_rows <= 0 || B <= 0) return 0;
    const int depth = (mode == 0) ? K : K * par_block;
    if (row_block % BM != 0 || B % 8 != 0 || n_groups <= 0 || depth <= 0 || depth > W_MAX_DEPTH) return -1;
    if (fc != 0 && fc != 2 && fc != 4 && fc != 8) return -1;
    const int64_t row_tiles = n_rows * (row_block / BM);
    const WideScratch w = wide_scratch(scratch, n_groups, depth, B);
    if (scratch == nullptr || (reinterpret_cast<uintptr_t>(scratch) & 255) != 0 || scratch_bytes < w.total) return -1;
    const int DN = wide_dn(B);
    const int n_chunks = (int)pcx_cdiv(depth, KC), n_ct = (int)pcx_cdiv(B, DN);
    const int splits = wide_splits(row_tiles * n_ct, n_chunks, DN);

    WidePrepArgs p{};
    p.src = src; p.src2 = src2; p.kids = kids; p.fkids = fkids_prep; p.group_row = group_row; p.fc = fc; p.K = K;
    p.par_block = (mode == 0) ? 1 : par_block; p.depth = depth; p.depth_pad = n_chunks * KC; p.B = B;
    p.logspace = logspace; p.mode = mode; p.DN = DN; p.n_ct = n_ct; p.n_chunks = n_chunks; p.tiles = w.tiles;
    p.shift = w.shift;
    p.cs = wide_prep_cluster(n_chunks);
    const dim3 pgrid((unsigned)(B / W_PREP_SAMPLES), (unsigned)n_groups, (unsigned)p.cs);
    const size_t psmem = (size_t)(p.depth_pad / p.cs + 4) * 8 * sizeof(float);
    int rc;
    const int pfc = (mode == 0 && fkids_prep != nullptr) ? fc : 0;
    if (pfc == 0) rc = launch_wide_prep_rows<0>(p, pgrid, psmem, st);
    else if (pfc == 2) rc = launch_wide_prep_rows<2>(p, pgrid, psmem, st);
    else if (pfc == 4) rc = launch_wide_prep_rows<4>(p, pgrid, psmem, st);
    else rc = launch_wide_prep_rows<8>(p, pgrid, psmem, st);
    if (rc != 0) return rc;
    if (g_wide_stage_event != nullptr) cudaEventRecord(g_wide_stage_event, st);      // measurement hook, see pcx_set_stage_event

    WideArgs a{};
    a.a_tiles = reinterpret_cast<const uint8_t*>(packed); a.b_tiles = w.tiles; a.b_group = row_group;
    a.n_chunks = n_chunks; a.splits = splits; a.n_ct = n_ct; a.row_block = row_block; a.B = B; a.logspace = logspace;
    a.terms = (g_sum_mode == 2) ? 1 : 3; a.rows = rows; a.out = out; a.shift = w.shift; a.emars = emars;
    a.nmars = src2; a.nflows = nflows; a.fkids = fkids_epi; a.fc = fc; a.direct = direct;
    const dim3 grid((unsigned)row_tiles, (unsigned)n_ct, (unsigned)splits);
    return mode == 0 ? launch_wide_gemm_dn<W_FWD>(a, DN, grid, st) : launch_wide_gemm_dn<W_ELE>(a, DN, grid, st);
}

}  // namespace

extern "C" {

int pcx_set_stage_event(void* event) {
    g_wide_stage_event = reinterpret_cast<cudaEvent_t>(event);
    return 0;
}

int pcx_set_dependent_launch(int on) {
    g_wide_pdl = on ? 1 : 0;
    return 0;
}

int64_t pcx_dense2_scratch_bytes(int n_groups, int depth, int B) {
    return wide_scratch(nullptr, n_groups, depth, B).total;
}

int pcx_sum_fwd_dense2(float* node_mars, const float* element_mars, const void* packed, const int32_t* nids,
                       const int32_t* cids, const int32_t* fkids, int fc, const int32_t* row_group,
                       const int32_t* group_row, int n_groups, void* scratch, int64_t scratch_bytes,
                       int64_t n_blocks, int K, int block_size, int B, void* stream) {
    if (fkids == nullptr && element_mars == nullptr) return -1;
    const float* src = fkids != nullptr ? node_mars : element_mars;
    return wide_rows_op(0, node_mars, src, nullptr, nullptr, nullptr, packed, nids, cids, fkids, nullptr,
                        fkids != nullptr ? fc : 0, 0, row_group, group_row, n_groups, scratch, scratch_bytes,
                        n_blocks, K, block_size, 1, B, 1, (cudaStream_t)stream);
}

int pcx_sum_bwd_ele_dense2(float* element_flows, const float* element_mars, float* node_flows, const float* node_mars,
                           const void* packed, const int32_t* chids, const int32_t* parids, const int32_t* fkids,
                           int fc, int direct, const int32_t* row_group, const int32_t* group_row, int n_groups,
                           void* scratch, int64_t scratch_bytes, int64_t n_blocks, int P,
                           int block_size, int ch_block_size, int B, int logspace, void* stream) {
    if (block_size % 8 != 0) return -1;
    if (fkids == nullptr && (element_mars == nullptr || element_flows == nullptr)) return -1;
    if (fkids != nullptr && !direct && element_flows == nullptr) return -1;
    return wide_rows_op(1, element_flows, node_flows, node_mars, element_mars, node_flows, packed, chids, parids, nullptr,
                        fkids, fkids != nullptr ? fc : 0, direct, row_group, group_row, n_groups, scratch, scratch_bytes,
                        n_blocks, P, ch_block_size, block_size, B, logspace, (cudaStream_t)stream);
}

int pcx_sum_par_dense2_stage(void* x_tiles, void* y_tiles, const float* node_flows, const float* node_mars,
                             const float* element_mars, const int32_t* nids, const int32_t* cids_row,
                             const int32_t* fkids_row, int fc, int64_t n_blocks, int K, int block_size, int B,
                             int n_chunks_total, int slot, int logspace, void* stream) {
    if (n_blocks <= 0 || B <= 0) return 0;
    const int64_t rows = n_blocks * block_size;
    if (block_size % BM != 0 || K <= 0 || slot < 0 || B % 8 != 0 || rows > W_MAX_DEPTH) return -1;
    if (((int64_t)slot + 1) * B > (int64_t)n_chunks_total * KC) return -1;
    if (fkids_row == nullptr && element_mars == nullptr) return -1;
    if (fkids_row != nullptr && fc != 2 && fc != 4 && fc != 8) return -1;
    WidePrepArgs p{};
    p.src = node_flows; p.src2 = node_mars; p.kids = nids; p.K = 1; p.par_block = block_size; p.depth = (int)rows;
    p.depth_pad = (int)pcx_cdiv(rows, KC) * KC; p.B = B; p.logspace = logspace; p.mode = 2;
    p.tiles = reinterpret_cast<uint8_t*>(x_tiles); p.y_tiles = reinterpret_cast<uint8_t*>(y_tiles);
    p.emars = element_mars; p.cids_row = cids_row; p.fk_row = fkids_row; p.fc = fc; p.Kfw = K;
    p.n_chunks_total = n_chunks_total; p.slot = slot;
    p.cs = wide_prep_cluster(p.depth_pad / KC);
    const dim3 grid((unsigned)(B / W_PREP_SAMPLES), 1, (unsigned)p.cs);
    const size_t smem = (size_t)(p.depth_pad / p.cs + 4) * 8 * sizeof(float);
    cudaStream_t st = (cudaStream_t)stream;
    if (fkids_row == nullptr) return launch_wide_prep_par<0>(p, grid, smem, st);
    if (fc == 2) return launch_wide_prep_par<2>(p, grid, smem, st);
    if (fc == 4) return launch_wide_prep_par<4>(p, grid, smem, st);
    return launch_wide_prep_par<8>(p, grid, smem, st);
}

int pcx_sum_par_dense2_gemm(float* param_flows, const float* params, const void* x_tiles, const void* y_tiles,
                            const int32_t* cids, const int32_t* pids, const int32_t* pfids, int64_t n_blocks, int K,
                            int block_size, int n_chunks_total, void* stream) {
    if (n_blocks <= 0 || n_chunks_total <= 0) return 0;
    if (block_size % BM != 0 || K <= 0) return -1;
    WideArgs a{};
    a.a_tiles = reinterpret_cast<const uint8_t*>(x_tiles); a.b_tiles = reinterpret_cast<const uint8_t*>(y_tiles);
    a.n_chunks = n_chunks_total; a.splits = 1; a.row_block = block_size; a.terms = (g_sum_mode == 2) ? 1 : 3;
    a.out = param_flows; a.params = params; a.cids = cids; a.pids = pids; a.pfids = pfids; a.K = K;
    const dim3 grid((unsigned)(n_blocks * (block_size / BM)), (unsigned)pcx_cdiv(K, 256), 1);
    return launch_wide_gemm<W_PAR, 256>(a, grid, (cudaStream_t)stream);
}

}  // extern "C"
