/*
 * pcx_b200.h — C ABI of the sm_100a kernels behind the compiled probabilistic-circuit
 * forward / backward / mini-batch-EM path.
 *
 * Every entry point replaces one kernel family of PyJuice; the citation after each
 * declaration names the reference launcher (or Triton kernel) whose work it takes over.
 * Paths are relative to the PyJuice source tree (src/pyjuice/...).
 *
 * Conventions
 *   - all pointers are DEVICE pointers; sizes and scalars are passed by value;
 *   - value buffers are row-major [rows, B] fp32 with the batch innermost;
 *   - index tables are int32 copies of the compiled int64 tables (host checks the range);
 *     id 0 in a child / parent / parameter table means padding;
 *   - kernels are enqueued on `stream` (a cudaStream_t passed as void*), never allocate,
 *     never synchronise, and write in place;
 *   - return value: 0 on success, a cudaError_t value if the launch was rejected,
 *     -1 for an argument the kernel family does not support.
 */
#ifndef PCX_B200_H
#define PCX_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Library / build identification: returns the compute capability it was built for (100). */
int pcx_build_arch(void);

/* Arithmetic of the sum-layer contractions, held PER CALLING HOST THREAD (two threads that drive two circuits never
 * change each other's arithmetic; the Python host sets it before every call from the circuit's own attribute): 0 = fp32 CUDA cores everywhere; 1 (default) = tensor
 * cores (tcgen05, fp32 accumulate) with every fp32 factor split into bf16 hi + lo (three products) wherever the
 * block sizes allow a 128-row tile, fp32 CUDA cores elsewhere; 2 = as 1 with a single bf16 product.
 * Takes over the role of the reference's force_use_bf16 / force_use_fp32 switches (layer/sum_layer.py:752-771). */
int pcx_set_sum_mode(int mode);
/* 0, or the code of the first tensor-core kernel whose bounded barrier wait ran out (synchronises the device). */
int pcx_get_status(void);
/* Reset that status word to 0 (after the caller has dealt with the failure). */
int pcx_clear_status(void);
/* Self-test of the failure path: one warp waits, for at most `max_polls` (<= 65536) polls, on a counter that
 * nothing advances (which = 0) or on an mbarrier nothing arrives on (which = 1), gives up, records status
 * 900 + which and returns; the context stays usable.  The reference's kernels have no such path: their barrier
 * waits are unbounded loops (layer/kernels/c/tlmm_forward_sum.cu:55-61). */
int pcx_probe_bounded_wait(int which, int max_polls, void* stream);

/* p[i] = v  /  p[i] *= v  for i < n.
 * Replaces the buffer resets of model/tensorcircuit.py:357-359, 528-529, 1761-1773 and the
 * `param_flows *= flows_memory` of model/tensorcircuit.py:1411-1412, layer/input_layer.py:299-300. */
int pcx_fill_f32(float* p, int64_t n, float v, void* stream);
int pcx_scale_f32(float* p, int64_t n, float v, void* stream);
/* p[i] = exp(p[i]); used to hand linear-space flows to callers that ask for logspace_flows=False. */
int pcx_exp_f32(float* p, int64_t n, void* stream);

/* Flow-carrying entry points take `logspace`: 1 = flow buffers hold log-flows (the default regime),
 * 0 = they hold linear flows (PyJuice's logspace_flows=False).  Arithmetic is done in log space either way;
 * the flag only changes how flows are read and written. */

/* node_flows[root rows, b] = w (linear) or log w (log space), w = weights ? weights[r*B+b] : 1
 * (model/tensorcircuit.py:537-552). */
int pcx_set_root_flows(float* node_flows, const float* weights, int64_t root_start, int64_t num_roots,
                       int B, int logspace, void* stream);

/* Categorical leaves, forward:  node_mars[node_off+n, b] = log params[s_pids[n] + data[vids[n], b]].
 * data is [V, B], element size data_elsize in {1,2,4,8} (unsigned 8-bit or signed wider).
 * node_cats[n] = number of categories of node n, max_cats their maximum: when the tables of a few nodes fit in
 * shared memory (and B % 4 == 0) they are staged there; node_cats may be NULL (always the general kernel).
 * Replaces InputLayer.forward + Categorical.fw_mar_fn
 * (layer/input_layer.py:318-380, 1148-1187; nodes/distributions/categorical.py:82-91). */
int pcx_input_cat_fwd(float* node_mars, const float* params, const void* data, int data_elsize,
                      const int32_t* vids, const int32_t* s_pids, const int32_t* node_cats, int max_cats,
                      int64_t n_nodes, int64_t node_off, int B, void* stream);

/* Categorical leaves, backward:  param_flows[s_pfids[n] + data[vids[n], b]] += flow(node_off+n, b)  (linear value).
 * Replaces InputLayer.backward + Categorical.bk_flow_fn / cat_backward.cu
 * (layer/input_layer.py:449-548; nodes/distributions/categorical.py:93-120;
 *  layer/kernels/c/input_layers/cat_backward.cu:24-52). */
int pcx_input_cat_bwd(float* param_flows, const float* node_flows, const void* data, int data_elsize,
                      const int32_t* vids, const int32_t* s_pfids, const int32_t* node_cats, int max_cats,
                      int64_t n_nodes, int64_t node_off, int B, int logspace, void* stream);

/* Categorical leaves with very large tables (too many categories to stage a node's table in shared memory): the same
 * two operators on a transposed shadow of the parameter table.  logp_t[c * n_rows + r] = log params[r * num_cats + c]
 * (pcx_input_cat_shadow, once per parameter update); prow[n] = row of node n (= s_pids[n] / num_cats); flows are
 * accumulated into flows_t[c * n_rows + r] (zero-initialised by the caller) and moved into the reference's layout by
 * pcx_input_cat_flush_t: param_flows[row_pfid[r] + c] += flows_t[c, r], flows_t = 0; `touched` ([num_cats] int32, zero
 * at first) marks the categories that received flow, so that the flush skips the others.  Flows of tied replicas all
 * land in their source row.  B must be a multiple of 4.  Replace, like the two entry points above, Categorical.fw_mar_fn /
 * bk_flow_fn (nodes/distributions/categorical.py:82-120) and layer/kernels/c/input_layers/cat_backward.cu:24-52,
 * whose histogram does not cover tied or large tables (layer/input_layer.py:304-316). */
int pcx_input_cat_shadow(float* logp_t, const float* params, int64_t n_rows, int num_cats, void* stream);
int pcx_input_cat_fwd_t(float* node_mars, const float* logp_t, const void* data, int data_elsize, const int32_t* vids,
                        const int32_t* prow, int64_t n_rows, int num_cats, int64_t n_nodes, int64_t node_off, int B,
                        void* stream);
int pcx_input_cat_bwd_t(float* flows_t, int32_t* touched, const float* node_flows, const void* data, int data_elsize,
                        const int32_t* vids, const int32_t* prow, int64_t n_rows, int num_cats, int64_t n_nodes,
                        int64_t node_off, int B, int logspace, void* stream);
int pcx_input_cat_flush_t(float* param_flows, float* flows_t, int32_t* touched, const int64_t* row_pfid, int64_t n_rows,
                          int num_cats, void* stream);

/* Product layer forward:  element_mars[nids[i]+j, b] = sum_c node_mars[cids[i,c]+j, b]   (cids == 0 skipped).
 * Replaces ProdLayer.forward -> _forward_backward_kernel_2d
 * (layer/prod_layer.py:161-205, 263-369; layer/kernels/prod.py:156-226 with accum=False). */
int pcx_prod_fwd(float* element_mars, const float* node_mars, const int32_t* nids, const int32_t* cids,
                 int64_t n_blocks, int n_chs, int block_size, int B, void* stream);

/* Product layer backward:
 *   node_flows[u_cids[i]+j, b] = logaddexp(node_flows[...], logsumexp_p element_flows[parids[i,p]+j, b])
 *   (plain sums when logspace == 0).
 * Replaces ProdLayer.backward (layer/prod_layer.py:207-238; layer/kernels/prod.py:192-226 with
 * accum=True, prop_logsumexp=True). */
int pcx_prod_bwd(float* node_flows, const float* element_flows, const int32_t* u_cids, const int32_t* parids,
                 int64_t n_blocks, int n_pars, int block_size, int B, int logspace, void* stream);

/* Sum layer forward, one partition:
 *   node_mars[nids[i]+m, b] = log sum_e params[pids[i,e]+m] * exp(element_mars[cids[i,e], b]),  m < block_size.
 * K is the padded fan-in (table width).  Replaces SumLayer._forward_block_sparse / _forward_sparse and the
 * kernels they pick (layer/sum_layer.py:551-1056; layer/kernels/sum_forward_block_sparse.py:25-170;
 * layer/kernels/sum_forward_sparse.py:24-107; layer/kernels/c/tlmm_forward_sum.cu:123-194;
 * layer/kernels/c/smallbatch_forward_sum.cu:30-73). */
int pcx_sum_fwd(float* node_mars, const float* element_mars, const float* params,
                const int32_t* nids, const int32_t* cids, const int32_t* pids,
                int64_t n_blocks, int K, int block_size, int B, void* stream);

/* Pre-split parameter tiles for the tensor-core kernels.  The parameter operand of the forward and element-flow
 * contractions only changes at EM updates, so it is converted once per update into bf16 hi/lo tile images of
 * 32 KB (one per 128-row tile and 64-deep slice of the contraction) that the kernels copy straight into shared
 * memory.  One launch serves every table of the circuit: `jobs` is a DEVICE array of n_jobs PcxPackJob records,
 * n_vec the total number of 16-byte vectors (sum over jobs of tiles * 1024).  `pcx_packed_tile_count` * 32768
 * bytes is the size of a job's `out`.  No counterpart in the reference (its kernels convert on the fly:
 * layer/kernels/c/tlmm_forward_sum.cu:140-166). */
typedef struct PcxPackJob {
    void* out;                /* device: tile images */
    const int32_t* kids;      /* device: mode 1: parids [n_rows, K] (0 = padding); mode 0: unused */
    const int32_t* kpar;      /* device: mode 0: pids [n_rows, K]; mode 1: parpids [n_rows, K] */
    int64_t vec_begin;        /* running sum of tiles * 1024 over the preceding jobs */
    int32_t K;                /* table width */
    int32_t row_block;        /* mode 0: block_size; mode 1: ch_block_size (multiple of 128) */
    int32_t par_block;        /* mode 1: block_size of the parents (multiple of 8); mode 0: 1 */
    int32_t n_chunks;         /* ceil(contraction length / 64) */
    int32_t mode;             /* 0 forward, 1 element flows */
    int32_t pad_;
} PcxPackJob;
int64_t pcx_packed_tile_count(int64_t n_rows, int K, int row_block, int par_block, int mode);
int pcx_pack_sum_params(const void* jobs, int n_jobs, int64_t n_vec, const float* params, void* stream);

/* pcx_sum_fwd / pcx_sum_bwd_ele on the tensor cores (tcgen05 + TMEM), reading pre-split parameter tiles.
 * Need block_size % 128 == 0 (forward) or ch_block_size % 128 == 0 and block_size % 8 == 0 (element flows). */
int pcx_sum_fwd_packed(float* node_mars, const float* element_mars, const void* packed,
                       const int32_t* nids, const int32_t* cids, int64_t n_blocks, int K, int block_size, int B,
                       void* stream);
int pcx_sum_bwd_ele_packed(float* element_flows, const float* element_mars, const float* node_flows,
                           const float* node_mars, const void* packed, const int32_t* chids, const int32_t* parids,
                           int64_t n_blocks, int P, int block_size, int ch_block_size, int B, int logspace,
                           void* stream);

/* Product layer folded into the sum kernels.  In the reference a product layer is its own kernel that writes
 * element_mars, read back by the sum layer above it and recomputed during the backward pass
 * (model/tensorcircuit.py:395-411, 590-591; layer/prod_layer.py:161-238).  These variants take, instead of an element
 * buffer, the child rows of every product node: `fkids` is [n_blocks, K, fc] (forward, parameter flows: the fc
 * node_mars rows whose sum is the value of table entry (i, k); 0 = none) or [n_blocks, ch_block_size, fc] (element
 * flows: the children of every output element), fc in {2, 4, 8}.  With direct != 0 the element-flow kernel stores
 * each element's flow straight into its children's rows of node_flows (valid when every such child has exactly one
 * parent in the whole circuit), which replaces the product-layer backward kernel as well. */
int pcx_sum_fwd_fused(float* node_mars, const void* packed, const int32_t* nids, const int32_t* cids,
                      const int32_t* fkids, int fc, int64_t n_blocks, int K, int block_size, int B, void* stream);
int pcx_sum_bwd_ele_fused(float* element_flows, float* node_flows, const float* node_mars, const void* packed,
                          const int32_t* chids, const int32_t* parids, const int32_t* fkids, int fc, int direct,
                          int64_t n_blocks, int P, int block_size, int ch_block_size, int B, int logspace,
                          void* stream);
int pcx_sum_bwd_par_fused(float* param_flows, const float* node_flows, const float* node_mars, const float* params,
                          const int32_t* nids, const int32_t* cids, const int32_t* pids, const int32_t* pfids,
                          const int32_t* fkids, int fc, int64_t n_blocks, int K, int block_size, int B, int logspace,
                          void* stream);

/* ---- Dense layers (tables hundreds to thousands deep, e.g. 4096 x 4096 HMM transition layers) ----------------------
 * Two steps per call: an operand pre-pass (column maxima, exp, bf16 hi/lo split, written as ready-made operand tiles to
 * `scratch`) and a GEMM over pre-tiled operands (bulk copies global -> shared memory, four-stage ring, tcgen05, eight
 * TMEM accumulators).  Requirements: block sizes multiples of 128 (parents: of 8), B a multiple of 64, parameters
 * pre-split with pcx_pack_sum_params.  Rows of the table that list the same children (parents) share one operand:
 * row_group[i] is the group of table row i, group_row[g] one row of group g.  `scratch` is caller-owned, 256-byte
 * aligned, at least pcx_dense_scratch_bytes(n_groups, depth, B) bytes (depth = K, or P * block_size for the element
 * flows).  Same results as pcx_sum_fwd / pcx_sum_bwd_ele (layer/sum_layer.py:551-929, 1369-1719). */
int64_t pcx_dense_scratch_bytes(int n_groups, int depth, int B);
int pcx_sum_fwd_dense(float* node_mars, const float* element_mars, const void* packed, const int32_t* nids,
                      const int32_t* cids, const int32_t* row_group, const int32_t* group_row, int n_groups,
                      void* scratch, int64_t scratch_bytes, int64_t n_blocks, int K, int block_size, int B,
                      void* stream);
int pcx_sum_bwd_ele_dense(float* element_flows, const float* element_mars, const float* node_flows,
                          const float* node_mars, const void* packed, const int32_t* chids, const int32_t* parids,
                          const int32_t* row_group, const int32_t* group_row, int n_groups, void* scratch,
                          int64_t scratch_bytes, int64_t n_blocks, int P, int block_size, int ch_block_size, int B,
                          int logspace, void* stream);

/* Parameter flows of dense layers (layer/sum_layer.py:1721-2080).  The contraction runs over the batch; layers that
 * share their parameter and flow tables (tied layers) are contracted in ONE product whose contraction dimension is
 * the concatenation of their batches.  Step 1, once per layer while element_mars holds that layer's products:
 * pcx_sum_par_dense_stage writes the layer's operand tiles into chunk columns [slot * cpl, (slot + 1) * cpl),
 * cpl = ceil(B / 64), of x_tiles ([row tiles][n_chunks_total] tiles of 32 KB) and y_tiles ([ceil(K / 64)]
 * [n_chunks_total] tiles of 16 KB); every table row must list the same children (cids = the row of table row 0);
 * `work` holds (ceil(n_blocks * block_size / 64) + 1) * B floats.  Step 2, once per group: pcx_sum_par_dense_gemm adds
 * params[pids[i,e] + n] * sum_b x[n,b] y[e,b] to param_flows[pfids[i,e] + n]. */
int pcx_sum_par_dense_stage(void* x_tiles, void* y_tiles, float* work, const float* node_flows,
                            const float* node_mars, const float* element_mars, const int32_t* nids,
                            const int32_t* cids, int64_t n_blocks, int K, int block_size, int B, int n_chunks_total,
                            int slot, int logspace, void* stream);
int pcx_sum_par_dense_gemm(float* param_flows, const float* params, const void* x_tiles, const void* y_tiles,
                           const int32_t* cids, const int32_t* pids, const int32_t* pfids, int64_t n_blocks, int K,
                           int block_size, int n_chunks_total, void* stream);

/* ---- Dense layers, wide tiles ----------------------------------------------------------------------------------
 * Same contractions as the four entry points above with output tiles of 128 rows x up to 256 samples (a parameter
 * tile is fetched once per layer and pass) and the contraction split over several CTAs per tile; preferred whenever
 * B is a multiple of 8 and the operand has at most 6144 rows.  The product layer can be folded in: with `fkids`
 * ([table rows * K][fc] for the forward pass, [child rows][fc] for the element flows; fc = 2, 4 or 8 child rows of
 * every product, 0 = none) a product's value is gathered from node_mars and element_mars / element_flows are not
 * used; with `direct` (every child row has exactly one parent product) an element's flow is stored straight into its
 * children's rows of node_flows.  `scratch`: pcx_dense2_scratch_bytes(n_groups, depth, B) bytes, 256-byte aligned.
 * The CTAs that split one tile's contraction form a thread-block cluster and exchange partial sums through
 * distributed shared memory.
 * Replace, like the entry points above: SumLayer._forward_block_sparse / _backward_block_sparse_ele_flows /
 * _backward_block_sparse_par_flows (layer/sum_layer.py:551-929, 1369-1719, 1721-2080), with ProdLayer.forward /
 * backward folded in (layer/prod_layer.py:161-238). */
/* The sum-layer operators under the reference's other propagation rules (`propagation_alg`, layer/sum_layer.py:
 * 367-412, 414-543; kernels layer/kernels/sum_forward_block_sparse.py:83-160, sum_backward_element_block_sparse.py:
 * 77-160, sum_backward_param_block_sparse.py:57-134), plain fp32 CUDA-core kernels with the table layout of
 * pcx_sum_fwd / pcx_sum_bwd_ele / pcx_sum_bwd_par.  alg 0 = "LL" (the ordinary rule), 1 = "MPE" (value = max_k
 * log theta + child; a parent's flow goes to the children and parameters that attain the maximum, |log theta +
 * child - value| < 1e-6), 2 = "GeneralLL" (value = (1 / alpha) log sum_k (theta exp(child))^alpha; element flows
 * weighted by theta^alpha exp(alpha (child - value)), parameter flows by theta exp(child - value)). */
int pcx_sum_fwd_alg(float* node_mars, const float* element_mars, const float* params, const int32_t* nids,
                    const int32_t* cids, const int32_t* pids, int64_t n_blocks, int K, int block_size, int B, int alg,
                    float alpha, void* stream);
int pcx_sum_bwd_ele_alg(float* element_flows, const float* element_mars, const float* node_flows, const float* node_mars,
                        const float* params, const int32_t* chids, const int32_t* parids, const int32_t* parpids,
                        int64_t n_blocks, int P, int block_size, int ch_block_size, int B, int logspace, int alg,
                        float alpha, void* stream);
int pcx_sum_bwd_par_alg(float* param_flows, const float* node_flows, const float* node_mars, const float* element_mars,
                        const float* params, const int32_t* nids, const int32_t* cids, const int32_t* pids,
                        const int32_t* pfids, int64_t n_blocks, int K, int block_size, int B, int logspace, int alg,
                        float alpha, void* stream);

/* Measurement hook (per calling host thread): while `event` (a cudaEvent_t created with timing) is set,
 * pcx_sum_fwd_dense2 and pcx_sum_bwd_ele_dense2 record it on their stream between the operand pre-pass kernel and the
 * GEMM kernel, so that a benchmark that brackets the call with two events of its own gets the duration of each of
 * the two kernels.  NULL switches it off (default).  No counterpart in the reference. */
int pcx_set_stage_event(void* event);
/* The wide-tile kernels are launched with programmatic stream serialization (a kernel sets itself up while its
 * predecessor drains, then waits for it); 0 switches that off, e.g. to compare timings. */
int pcx_set_dependent_launch(int on);
int64_t pcx_dense2_scratch_bytes(int n_groups, int depth, int B);
int pcx_sum_fwd_dense2(float* node_mars, const float* element_mars, const void* packed, const int32_t* nids,
                       const int32_t* cids, const int32_t* fkids, int fc, const int32_t* row_group,
                       const int32_t* group_row, int n_groups, void* scratch, int64_t scratch_bytes,
                       int64_t n_blocks, int K, int block_size, int B, void* stream);
int pcx_sum_bwd_ele_dense2(float* element_flows, const float* element_mars, float* node_flows, const float* node_mars,
                           const void* packed, const int32_t* chids, const int32_t* parids, const int32_t* fkids,
                           int fc, int direct, const int32_t* row_group, const int32_t* group_row, int n_groups,
                           void* scratch, int64_t scratch_bytes, int64_t n_blocks, int P,
                           int block_size, int ch_block_size, int B, int logspace, void* stream);
/* Parameter flows: step 1 writes the operands of one layer at sample positions [slot * B, (slot + 1) * B) of the
 * concatenated batch (x_tiles: [row tiles][n_chunks_total] tiles of 32 KB; y_tiles: [ceil(K / 256)][n_chunks_total]
 * tiles of 64 KB; both zero-filled once by the caller; n_chunks_total = ceil(layers * B / 64)); `cids_row` / `fkids_row`
 * are the children of table row 0 (every row lists the same).  Step 2 is one product per group of tied layers. */
int pcx_sum_par_dense2_stage(void* x_tiles, void* y_tiles, const float* node_flows, const float* node_mars,
                             const float* element_mars, const int32_t* nids, const int32_t* cids_row,
                             const int32_t* fkids_row, int fc, int64_t n_blocks, int K, int block_size, int B,
                             int n_chunks_total, int slot, int logspace, void* stream);
int pcx_sum_par_dense2_gemm(float* param_flows, const float* params, const void* x_tiles, const void* y_tiles,
                            const int32_t* cids, const int32_t* pids, const int32_t* pfids, int64_t n_blocks, int K,
                            int block_size, int n_chunks_total, void* stream);

/* ---- Small node blocks (32 or 64 nodes) on the tensor cores: sample-major tiles -----------------------------------
 * A tile is 128 samples x nb nodes (nb = 32 or 64): one node block, or two consecutive 32-node blocks whose table rows
 * are identical and whose node ids are consecutive ("merged row"; first_row[m] = its first table row).  The batch is
 * the MMA's M dimension, so blocks need not share children to fill a tile.  Parameters are pre-split per merged row
 * with pcx_pack_sm_params (mode 0: forward tables nids/cids/pids, block = block size; mode 1: element-flow tables
 * chids/parids/parpids, block = child block size, par_block = block size of the parents) into a caller-owned buffer
 * of pcx_sm_packed_bytes(n_merged, depth, nb) bytes (depth = K, or P * par_block).  Same results as pcx_sum_fwd /
 * pcx_sum_bwd_ele (layer/sum_layer.py:551-929, 1369-1719).
 * Product layer folded in (products of at most two children): pass `fk` instead of reading element_mars -- pairs of
 * child rows of node_mars, [n, K, 2] per table entry for the forward pass and the parameter flows, [n, child block
 * size, 2] per output element for the element flows ((0, 0) = no element); fk == NULL reads element_mars. */
int64_t pcx_sm_packed_bytes(int64_t n_merged, int depth, int nb);
int pcx_pack_sm_params(void* packed, const float* params, const int32_t* first_row, const int32_t* kids,
                       const int32_t* kpar, int64_t n_merged, int nb, int block, int K, int par_block, int mode,
                       void* stream);
/* Parameter flows of small blocks on the tensor cores (layer/sum_layer.py:1721-2080): the contraction runs over the
 * batch, the MMA's M dimension is the edge index (128 per tile), N the nb nodes of the merged row.  B must be a multiple
 * of 8; element_mars row 0 must hold -inf (the dummy element). */
int pcx_sum_bwd_par_sm(float* param_flows, const float* node_flows, const float* node_mars, const float* element_mars,
                       const float* params, const int32_t* first_row, const int32_t* nids, const int32_t* cids,
                       const int32_t* pids, const int32_t* pfids, const int32_t* fk, int64_t n_merged, int nb,
                       int block, int K, int B, int logspace, void* stream);
/* The same conversion for many tables in one launch: `jobs` is a DEVICE array of n_jobs records, vec_begin the running
 * sum of n_merged * n_chunks * 8 * nb over the preceding jobs, n_vec the total. */
typedef struct PcxSmPackJob {
    void* out;
    const int32_t* first_row;
    const int32_t* kids;
    const int32_t* kpar;
    int64_t vec_begin;
    int32_t nb, block, K, par_block, n_chunks, mode;
} PcxSmPackJob;
int pcx_pack_sm_jobs(const void* jobs, int n_jobs, int64_t n_vec, const float* params, void* stream);
int pcx_sum_fwd_sm(float* node_mars, const float* element_mars, const void* packed, const int32_t* first_row,
                   const int32_t* nids, const int32_t* cids, const int32_t* fk, int64_t n_merged, int nb, int K, int B,
                   void* stream);
int pcx_sum_bwd_ele_sm(float* element_flows, const float* element_mars, const float* node_flows,
                       const float* node_mars, const void* packed, const int32_t* first_row, const int32_t* chids,
                       const int32_t* parids, const int32_t* fk, int ch_block_size, int64_t n_merged, int nb, int P,
                       int block_size, int B, int logspace, void* stream);

/* Forward (mode 0) or element flows (mode 1) of a RUN of consecutive layers in one launch, product layers folded in
 * (as pcx_sum_fwd_fused / pcx_sum_bwd_ele_fused with direct stores).  Tiles are work items claimed from a device
 * counter in layer order; a tile of level t starts as soon as the tiles of level t - 1 that cover the same batch
 * columns are finished, so layers overlap and no launch boundary separates them.  `jobs` is a DEVICE array of
 * PcxChainJob records ordered by level (level 0 is processed first: the lowest layer for mode 0, the highest for
 * mode 1); a job holds n_rowtiles * ceil(B / tn) items, `item_begin` is the running sum, `prev_total` the number of
 * row tiles of the previous level (all its jobs together).  tn in {16, 32, 64} is the tile width in samples.
 * `ctrl` is caller-owned device scratch of ctrl_len >= 64 + n_levels * ceil(B / tn) ints (8-byte aligned); it is
 * cleared on the stream by this call.  The reference runs one kernel launch per layer partition
 * (layer/sum_layer.py:367-412, 414-543). */
typedef struct PcxChainJob {
    const void* packed;       /* pre-split parameter tiles of the table (pcx_pack_sum_params) */
    const int32_t* rows;      /* mode 0: nids      mode 1: chids */
    const int32_t* kids;      /* mode 0: cids      mode 1: parids */
    const int32_t* fkids;     /* mode 0: [n, K, fc]   mode 1: [n, ch_block_size, fc] child rows */
    int64_t item_begin;
    int32_t K;                /* mode 0: table width      mode 1: parent blocks per child block */
    int32_t row_block;        /* mode 0: block size       mode 1: child block size */
    int32_t par_block;        /* mode 0: 1                mode 1: block size of the parents */
    int32_t n_rowtiles;       /* n_rows * row_block / 128 */
    int32_t level;
    int32_t prev_total;
} PcxChainJob;
int pcx_sum_chain(int mode, float* node_mars, float* node_flows, const void* jobs, int n_jobs, int64_t n_items,
                  int n_levels, int tn, int fc, int B, int logspace, int* ctrl, int64_t ctrl_len, void* stream);

/* Parameter flows of MANY tables in one launch (product layers folded in, as pcx_sum_bwd_par_fused).  Tiles of
 * different layers do not depend on one another, so after the backward sweep has produced every node flow the whole
 * circuit's parameter flows run as one grid.  `jobs` is a DEVICE array of n_jobs PcxParJob records; a table
 * contributes n_rows * (block_size / 128) * e_tiles * splits work items, `item_begin` is the running sum over the
 * preceding jobs, n_items the total.  Every work item handles `chunks_per_cta` 32-sample slices of the batch
 * (splits = ceil(ceil(B / 32) / chunks_per_cta), the same for every job).  In the reference this is one kernel
 * launch per layer partition (layer/sum_layer.py:520-541). */
typedef struct PcxParJob {
    const int32_t* nids;
    const int32_t* cids;
    const int32_t* pids;
    const int32_t* pfids;
    const int32_t* fkids;     /* [n_rows, K, fc] */
    int64_t item_begin;
    int32_t K;
    int32_t block_size;
    int32_t e_tiles;          /* ceil(K / 64) */
    int32_t splits;
} PcxParJob;
int pcx_sum_bwd_par_batched(float* param_flows, const float* node_flows, const float* node_mars, const float* params,
                            const void* jobs, int n_jobs, int64_t n_items, int fc, int B, int chunks_per_cta,
                            int logspace, void* stream);

/* Sum layer forward on the tensor cores for hosts that must not allocate.  [No counterpart in the reference.]
 *
 * Same result as pcx_sum_fwd_packed, same arguments as pcx_sum_fwd.  Some callers cannot obtain device memory at
 * the moment they need this kernel: code running inside a stream capture or a real-time loop where cudaMalloc
 * (which synchronises the device) is forbidden, a plugin living in a process whose memory pool belongs to another
 * framework, a thin FFI host with no allocator binding at all.  The tensor-core kernel needs the parameters of the
 * table pre-split into bf16 hi/lo tiles; here that scratch is a fixed array inside the library
 * (PCX_NOALLOC_MAX_TILES tiles of 32 KB = 8 MiB, held by every GPU that loads the library until the process
 * exits), filled by a first kernel on `stream` and consumed by the second.  Nothing is allocated or freed.
 *
 *   - needs block_size % 128 == 0; n_blocks * (block_size / 128) * ceil(K / 64) tiles must fit, otherwise
 *     PCX_ERR_SCRATCH_TOO_SMALL is returned and nothing is launched;
 *   - the first call on each device looks up the array's device address (with that device current) and caches it per
 *     device ordinal without a lock — two host threads making that first call together store the same value; make
 *     that first call before starting any stream capture;
 *   - all calls share the one array: calls that may overlap on the GPU (different streams, no ordering) race on
 *     it and must be serialised by the caller.  Each call rewrites every tile it uses, padding included, so a call
 *     never depends on what an earlier one left behind. */
#define PCX_NOALLOC_MAX_TILES 256
#define PCX_ERR_SCRATCH_TOO_SMALL (-2)
int pcx_sum_fwd_noalloc(float* node_mars, const float* element_mars, const float* params,
                        const int32_t* nids, const int32_t* cids, const int32_t* pids,
                        int64_t n_blocks, int K, int block_size, int B, void* stream);

/* Sum layer backward, element flows, one backward partition:
 *   element_flows[chids[i]+c, b] = element_mars[chids[i]+c, b]
 *        + log sum_{p, n} params[parpids[i,p] + c*block_size + n] * exp(node_flows[parids[i,p]+n, b] - node_mars[parids[i,p]+n, b])
 * for c < ch_block_size; P is the padded number of parent blocks.
 * Replaces SumLayer._backward_block_sparse_ele_flows / _backward_sparse_ele_flows
 * (layer/sum_layer.py:1369-1719, 2135-2380; layer/kernels/sum_backward_element_block_sparse.py:25-190;
 *  layer/kernels/c/ele_backward_sum.cu:113-159; layer/kernels/c/smallbatch_ele_backward.cu:47-97). */
int pcx_sum_bwd_ele(float* element_flows, const float* element_mars, const float* node_flows,
                    const float* node_mars, const float* params,
                    const int32_t* chids, const int32_t* parids, const int32_t* parpids,
                    int64_t n_blocks, int P, int block_size, int ch_block_size, int B, int logspace, void* stream);

/* Sum layer backward, parameter flows, one forward partition:
 *   param_flows[pfids[i,e]+m] += params[pids[i,e]+m] * sum_b exp(node_flows[nids[i]+m, b] - node_mars[nids[i]+m, b] + element_mars[cids[i,e], b]).
 * Accumulates (atomically) into param_flows.  Replaces SumLayer._backward_block_sparse_par_flows /
 * _backward_sparse_par_flows (layer/sum_layer.py:1744-2080, 2380-2620;
 * layer/kernels/sum_backward_param_block_sparse.py:25-142; layer/kernels/c/par_backward_sum.cu:4-207;
 * layer/kernels/c/smallbatch_par_backward.cu:31-68). */
int pcx_sum_bwd_par(float* param_flows, const float* node_flows, const float* node_mars,
                    const float* element_mars, const float* params,
                    const int32_t* nids, const int32_t* cids, const int32_t* pids, const int32_t* pfids,
                    int64_t n_blocks, int K, int block_size, int B, int logspace, void* stream);

/* flows[start + j] = sum_c flows[ch_starts[c] + j], j < n, and every other accumulator is cleared (in place on
 * `flows`; the source's own range is one of the ch_starts), so a second call changes nothing.  Replaces InputLayer._pflow_accum_kernel (layer/input_layer.py:755-783, 1391-1411)
 * and cum_par_flows_kernel (model/backend/parflow_fusing.py:80-112). */
int pcx_tied_accum(float* flows, int64_t start, int64_t n, const int64_t* ch_starts, int n_chs, void* stream);

/* EM update of sum parameters.  One descriptor row per node block:
 *   blk_par[i], blk_flow[i] first parameter / flow of the block, blk_fan[i] real fan-in (child nodes),
 *   blk_bs[i] block size.  For node m of block i:
 *     tot = sum_e flows[blk_flow + e*bs + m]
 *     theta[blk_par + e*bs + m] = (1-step)*theta + step*(flow + pseudo/fan)/(tot + pseudo)
 *   (keep_zero != 0: parameters < 1e-12 stay 0 and do not receive the pseudocount).
 * Replaces em_par_update -> cum_pflow_kernel + em_par_update_kernel
 * (model/backend/par_update.py:173-256, 296-326). */
int pcx_em_sum(float* params, const float* param_flows, const int64_t* blk_par, const int64_t* blk_flow,
               const int32_t* blk_fan, const int32_t* blk_bs, int64_t n_blocks, int max_bs,
               float step, float pseudo, int keep_zero, void* stream);

/* EM update of categorical leaf parameters, one row of node_cats[n] categories per source node n:
 *   theta[s_pids[n]+c] = (1-step)*theta + step*(flows[s_pfids[n]+c] + pseudo/num_cats)/(sum_c flows + pseudo).
 * node_cats is indexed by layer-local node id; max_cats only selects the launch shape.
 * Replaces InputLayer.mini_batch_em -> _em_kernel + Categorical.{small,large}_ncats_em_fn
 * (layer/input_layer.py:785-813, 1414-1436; nodes/distributions/categorical.py:191-272). */
int pcx_em_input_cat(float* params, const float* param_flows, const int32_t* source_nids,
                     const int32_t* s_pids, const int32_t* s_pfids, const int32_t* node_cats,
                     int64_t n_source, int max_cats, float step, float pseudo, int keep_zero, void* stream);

/* Categorical EM for a layer whose flows were accumulated in the transposed shadow (pcx_input_cat_bwd_t) and whose
 * [row, category] accumulators hold nothing else: params[r, c] <- (1 - step) * params[r, c] + step * (flows_t[c, r] +
 * pseudo / C) / (sum_c flows_t[c, r] + pseudo), and logp_t[c, r] <- log of the new value, in two short kernels (instead of
 * pcx_input_cat_flush_t + pcx_em_input_cat + pcx_input_cat_shadow).  `totals`: caller-owned scratch of 16 * n_rows floats
 * (partial row totals, added in a fixed order: no atomics, results repeat bit for bit); flows_t 16-byte aligned and left unchanged.  The update itself is
 * that of the reference's categorical EM kernels (nodes/distributions/categorical.py:192-229, 231-272). */
int pcx_em_input_cat_t(float* params, float* logp_t, const float* flows_t, float* totals, int64_t n_rows, int num_cats,
                       float step, float pseudo, void* stream);
/* Flows of unobserved categorical leaves: param_flows[s_pfids[n] + c] += scale * source_flow[k] * params[s_pids[n] + c]
 * for the k-th source node n = source_nids[k] and every category c (source_flow: the linear flow of the node plus
 * that of the nodes tied to it).  Used by the top-down probabilities of the rescaled EM update.  Replaces
 * InputLayer.add_missing_flows / Categorical.bk_flow_mask_fn (layer/input_layer.py:894-968,
 * nodes/distributions/categorical.py:123-160). */
int pcx_input_cat_missing(float* param_flows, const float* params, const float* source_flow,
                          const int32_t* source_nids, const int32_t* s_pids, const int32_t* s_pfids,
                          const int32_t* node_cats, int64_t n_source, float scale, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* PCX_B200_H */
