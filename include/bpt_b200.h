/*
 * bpt_b200 — C ABI of the B200 (sm_100a) implementation of BP-Transformer's graph
 * attention hot path.  Plain pointers and sizes only; every pointer named "device" must
 * be device memory of the current CUDA device, every launch goes to the given stream and
 * no entry point synchronises unless it says so.  All functions return 0 on success and a
 * BPT_ERR_* code otherwise; bpt_last_error() gives the message of the calling thread's
 * last failure.
 *
 * Each entry point names the reference interface it replaces (paths are relative to the
 * yzh119/BPT source tree).
 */
#ifndef BPT_B200_H_
#define BPT_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void *bpt_stream_t; /* a cudaStream_t */

enum {
    BPT_OK = 0,
    BPT_ERR_INVALID = 1,     /* bad argument (null pointer, negative size, unsupported shape) */
    BPT_ERR_CUDA = 2,        /* a CUDA runtime call or launch failed */
    BPT_ERR_WORKSPACE = 3,   /* workspace too small */
    BPT_ERR_UNSUPPORTED = 4, /* dtype / head-dim combination without a kernel */
    BPT_ERR_OVERFLOW = 5     /* a size does not fit the 32-bit indices of the fused path */
};

/* Element types of feature tensors. Accumulation is fp32 (fp64 for BPT_F64). */
enum { BPT_F32 = 0, BPT_F64 = 1, BPT_BF16 = 2, BPT_F16 = 3 };

const char *bpt_last_error(void);
int bpt_version(void);

/* ------------------------------------------------------------------------------------
 * Binary-partition graph construction.
 * Replaces BinaryPartition.__cinit__/build_graph, graph_builder/builder.pyx:29-116.
 * Results are bit-identical to that code for the same (length, triu, step, clip_dist).
 * ---------------------------------------------------------------------------------- */

/* Level table (host only, no GPU work): builder.pyx:41-56.  n_nodes_arr and shift are host
 * arrays of at least 64 entries; entry j is the size / first node id of level j. */
int bpt_bp_levels(int64_t length, uint32_t *n_nodes_arr, uint32_t *shift,
                  int64_t *n_nodes, int *n_levels);

/* Bytes of device workspace bpt_bp_count needs. */
size_t bpt_bp_count_workspace_bytes(int64_t length);

/* Per-leaf edge counts and their exclusive prefix sum (builder.pyx:64-116 replayed without
 * writing).  leaf_offsets: device int64[length+1]; leaf_offsets[i] is the edge id of leaf
 * i's first edge, leaf_offsets[length] the edge count.  If n_edges_host is not NULL the
 * call waits for the stream and stores the edge count there. */
int bpt_bp_count(int64_t length, int triu, int step, int clip_dist, int64_t *leaf_offsets,
                 void *workspace, size_t workspace_bytes, int64_t *n_edges_host,
                 bpt_stream_t stream);

/* Writes the edge list in the reference's emission order (builder.pyx:64-116) and the
 * node positions (builder.pyx:46-47,57-62).  src/dst get v_shift added, which is how
 * get_edges(v_shift) (builder.pyx:137-140) and the block-diagonal batching of
 * graph/lm.py:59-98 place a sequence inside a batch.  Outputs are device arrays of
 * n_edges (src, dst, etype) and n_nodes (pos) entries; index_bytes selects int32 (4) or
 * int64 (8) elements.  Any of the output pointers may be NULL. */
int bpt_bp_fill(int64_t length, int triu, int step, int clip_dist,
                const int64_t *leaf_offsets, int64_t v_shift, int index_bytes,
                void *src, void *dst, void *etype, void *pos, bpt_stream_t stream);

/* Baseline graphs of the reference's dense / strided configurations: `length` token nodes plus
 * one root node (id `length`) that every token feeds.  Same two-step protocol and outputs as
 * bpt_bp_count / bpt_bp_fill (workspace size: bpt_bp_count_workspace_bytes(length)).
 * bpt_fc_*: FullyConnected(length, triu, window), graph_builder/builder.pyx:228-274 (every
 * token attends to the tokens within `window` positions, left only when triu; edge type
 * 2j-1 / 2j for distance j to the left / right).
 * bpt_oas_*: OpenAISparse(length, stride, c), builder.pyx:154-196 (causal: a token attends to
 * its stride block up to itself and to the last c tokens before every earlier block boundary). */
int bpt_fc_count(int64_t length, int triu, int64_t window, int64_t *leaf_offsets, void *workspace,
                 size_t workspace_bytes, int64_t *n_edges_host, bpt_stream_t stream);
int bpt_fc_fill(int64_t length, int triu, int64_t window, const int64_t *leaf_offsets, int64_t v_shift,
                int index_bytes, void *src, void *dst, void *etype, void *pos, bpt_stream_t stream);
int bpt_oas_count(int64_t length, int64_t stride, int64_t c, int64_t *leaf_offsets, void *workspace,
                  size_t workspace_bytes, int64_t *n_edges_host, bpt_stream_t stream);
int bpt_oas_fill(int64_t length, int64_t stride, int64_t c, const int64_t *leaf_offsets, int64_t v_shift,
                 int index_bytes, void *src, void *dst, void *etype, void *pos, bpt_stream_t stream);

/* Sentence-aligned cross graph (decoder -> encoder memory, graph/mt.py:318-321; premise <->
 * hypothesis, graph/nli.py:84-87): a list of dense blocks.  blocks[b] = {first source id, number
 * of sources, first destination id, number of destinations} (device int64[n_blocks][4]; zero-size
 * blocks are skipped by giving them equal offsets), edge_offsets[n_blocks + 1] = running sum of
 * sources x destinations (device int64).  Edge order inside a block as in the reference: source
 * slow, destination fast.  src/dst: device arrays of n_edges int32 or int64. */
int bpt_dense_blocks_fill(const int64_t *blocks, const int64_t *edge_offsets, int64_t n_blocks, int64_t n_edges,
                          int index_bytes, void *src, void *dst, bpt_stream_t stream);

/* ------------------------------------------------------------------------------------
 * CSR extraction.  Replaces get_csrs(), graph/base.py:71-86 (two COO->CSR conversions and
 * two partition_csr calls).  Entries of a row are in ascending edge-id order.
 * ---------------------------------------------------------------------------------- */

size_t bpt_coo_to_csr_workspace_bytes(int64_t n_edges, int64_t n_rows);

/* key[e] = row of edge e, other[e] = its column; index_bytes = 4 or 8 for every array.
 * indptr[n_rows+1], indices[n_edges] = other[eid], eid[n_edges]. */
int bpt_coo_to_csr(const void *key, const void *other, int64_t n_edges, int64_t n_rows,
                   int index_bytes, void *indptr, void *indices, void *eid,
                   void *workspace, size_t workspace_bytes, bpt_stream_t stream);

size_t bpt_partition_csr_workspace_bytes(int64_t n_rows);

/* partition_csr(indptr, chunk_size), graph_builder/builder.pyx:305-321, in two steps.
 * Count: chunk_offsets device int64[n_rows+1] (first chunk id of every row; last entry =
 * number of chunks).  If n_chunks_host is not NULL the call waits for the stream. */
int bpt_partition_csr_count(const int64_t *indptr, int64_t n_rows, int chunk_size,
                            int64_t *chunk_offsets, void *workspace, size_t workspace_bytes,
                            int64_t *n_chunks_host, bpt_stream_t stream);
/* Fill: row int64[n_chunks], indptr_out int64[n_chunks+1]. */
int bpt_partition_csr_fill(const int64_t *indptr, int64_t n_rows, int chunk_size,
                           const int64_t *chunk_offsets, int64_t n_chunks, int64_t *row,
                           int64_t *indptr_out, bpt_stream_t stream);

/* ------------------------------------------------------------------------------------
 * The eight graph operators.  Replace the functions exported by graph_kernel/graphop.cpp:
 * 216-225 (kernels in graph_kernel/graphop_kernel.cu).  `row`/`indptr` are the chunk
 * arrays of partition_csr (n_chunks and n_chunks+1 entries, rows non-decreasing), `eid`
 * maps CSR position to edge id, `indices` is the other endpoint; all int64, device.
 * Feature tensors are contiguous (N,h,d) / (E,h); dtype is a BPT_* element type.
 * Unlike the reference no operator uses floating-point atomics: results are bitwise
 * reproducible.  Outputs indexed by edge id are written only at edge ids that occur in
 * `eid`; the caller zero-fills them first if the CSR does not cover every edge (the
 * reference allocates them with at::zeros, graphop_kernel.cu:248,284).
 * ---------------------------------------------------------------------------------- */

/* maskedmm_csr_forward, graphop.cpp:16-30 / graphop_kernel.cu:269-304:
 * y[eid[j],h] = sum_d A[row_of(j),h,d] * B[indices[j],h,d]. */
int bpt_maskedmm_csr_forward(const int64_t *row, const int64_t *indptr, const int64_t *eid,
                             const int64_t *indices, int64_t n_chunks,
                             const void *A, const void *B, void *y,
                             int h, int d, int dtype, bpt_stream_t stream);

/* maskedmm_csr_backward, graphop.cpp:104-131 / graphop_kernel.cu:355-409:
 * dA[r] = sum over the (row,...) CSR of dy * B[indices]; dB[c] = sum over the (col,...)
 * CSR of dy * A[indices].  n_rows_a / n_rows_b: rows of dA / dB (zero-filled by the call
 * for rows without edges). */
int bpt_maskedmm_csr_backward(const int64_t *row, const int64_t *indptr_r, const int64_t *eid_r,
                              const int64_t *indices_r, int64_t n_chunks_r,
                              const int64_t *col, const int64_t *indptr_c, const int64_t *eid_c,
                              const int64_t *indices_c, int64_t n_chunks_c,
                              const void *A, const void *B, const void *dy,
                              void *dA, void *dB, int64_t n_rows_a, int64_t n_rows_b,
                              int h, int d, int dtype, bpt_stream_t stream);

/* node_mul_edge_forward, graphop.cpp:38-51 / graphop_kernel.cu:235-266:
 * y[eid[j],h] = sum_d A[row_of(j),h,d] * B[eid[j],d]. */
int bpt_node_mul_edge_forward(const int64_t *row, const int64_t *indptr, const int64_t *eid,
                              int64_t n_chunks, const void *A, const void *B, void *y,
                              int h, int d, int dtype, bpt_stream_t stream);

/* node_mul_edge_backward, graphop.cpp:133-154 / graphop_kernel.cu:306-351:
 * dA[r,h,:] = sum_j dy[eid[j],h] * B[eid[j],:]; dB[eid[j],:] = sum_h dy[eid[j],h] * A[r,h,:]. */
int bpt_node_mul_edge_backward(const int64_t *row, const int64_t *indptr, const int64_t *eid,
                               int64_t n_chunks, const void *A, const void *B, const void *dy,
                               void *dA, void *dB, int64_t n_rows_a,
                               int h, int d, int dtype, bpt_stream_t stream);

/* sparse_softmax_forward, graphop.cpp:59-70 / graphop_kernel.cu:411-463:
 * softmax of x over the entries of each CSR row, per head. */
int bpt_sparse_softmax_forward(const int64_t *row, const int64_t *indptr, const int64_t *eid,
                               int64_t n_chunks, const void *x, void *y,
                               int h, int dtype, bpt_stream_t stream);

/* sparse_softmax_backward, graphop.cpp:156-171 / graphop_kernel.cu:465-507:
 * dx = y * (dy - sum_row(dy*y)). */
int bpt_sparse_softmax_backward(const int64_t *row, const int64_t *indptr, const int64_t *eid,
                                int64_t n_chunks, const void *y, const void *dy, void *dx,
                                int h, int dtype, bpt_stream_t stream);

/* vector_spmm_forward, graphop.cpp:80-95 / graphop_kernel.cu:509-542:
 * y[r,h,:] = sum_j edata[eid[j],h] * x[indices[j],h,:]; rows without edges get zero. */
int bpt_vector_spmm_forward(const int64_t *row, const int64_t *indptr, const int64_t *eid,
                            const int64_t *indices, int64_t n_chunks,
                            const void *edata, const void *x, void *y, int64_t n_rows_y,
                            int h, int d, int dtype, bpt_stream_t stream);

/* vector_spmm_backward, graphop.cpp:173-214 / graphop_kernel.cu:544-600:
 * dedata[eid[j],h] = sum_d dy[r,h,d] * x[indices[j],h,d] over the (row,...) CSR;
 * dx[c,h,:] = sum_j edata[eid_t[j],h] * dy[indices_t[j],h,:] over the transposed CSR.
 * Every chunk of the transposed CSR is processed (the reference sizes that launch with
 * the other CSR's chunk count, graphop_kernel.cu:566,588). */
int bpt_vector_spmm_backward(const int64_t *row, const int64_t *indptr, const int64_t *eid,
                             const int64_t *indices, int64_t n_chunks,
                             const int64_t *col, const int64_t *indptr_t, const int64_t *eid_t,
                             const int64_t *indices_t, int64_t n_chunks_t,
                             const void *edata, const void *dy, const void *x,
                             void *dedata, void *dx, int64_t n_rows_x,
                             int h, int d, int dtype, bpt_stream_t stream);

/* ------------------------------------------------------------------------------------
 * Fused graph attention.  One call replaces the reference's operator chain
 *   masked_mm -> node_mul_edge -> (e_rel + e)/sqrt(d_k) -> sparse_softmax -> vec_spmm
 * of BPTBlock.forward, modules/attention.py:66-77 (dropout off), i.e. per destination i
 *   o[i,h,:] = sum_e softmax_e(scale * <q[i,h], k[src_e,h] + ak[etype_e]>) * v[src_e,h,:]
 * over i's incoming edges, and bpt_attn_backward its gradient (what autograd builds from
 * modules/op.py:10-58).  Edge scores never reach HBM in the forward; no floating-point
 * atomics anywhere, so results are bitwise reproducible.
 *
 * The graph is given as a plan: a device blob built once per graph from the COO edge list
 * (src, dst, etype: int32, edge id = position), holding the int32 in-CSR, out-CSR, per-type
 * buckets and the work lists the kernels walk.  counts_host[12] (host memory, filled by
 * bpt_attn_plan_build, which waits for the stream) must be passed back to the other calls.
 * etype may be NULL (all edges type 0); every etype must be < n_etypes, every src < n_src and every
 * dst < n_nodes: bpt_attn_plan_build checks all three on the device first and returns
 * BPT_ERR_INVALID, with nothing built, when one is out of range.
 * Destinations and sources may be different node sets: dst ids index n_nodes rows (q, o, lse,
 * dq), src ids index n_src rows (k, v, dk, dv).  Self-attention has n_src == n_nodes; the
 * reference's cross-attention (BPTMemBlock, modules/attention.py:144-168) and a shard of a long
 * sequence attending to gathered K/V have not.
 * ---------------------------------------------------------------------------------- */

/* Dropout on the attention weights, the reference's drop_att between sparse_softmax and vec_spmm
 * (modules/attention.py:73): with rate r an edge's weight for one head is zeroed with probability r and
 * the kept ones are scaled by 1 / (1 - r), after the softmax normalisation.  The mask is a hash of
 * (destination, source, head, seed): the forward and the backward of one layer call must be given the same
 * seed, nothing is stored between them, and results stay bitwise reproducible for a fixed seed.  Parallel
 * edges between one pair of nodes share their bit.  A NULL pointer or rate 0 switches dropout off.
 * bpt_attn_dropout_mask writes the mask (1 = kept) for edges in edge-id order, (n_edges, h) bytes. */
typedef struct {
    double rate;   /* in [0, 1) */
    uint64_t seed;
} bpt_dropout_t;
int bpt_attn_dropout_mask(const int32_t *src, const int32_t *dst, int64_t n_edges, int h,
                          const bpt_dropout_t *dropout, uint8_t *mask, bpt_stream_t stream);

size_t bpt_attn_plan_bytes(int64_t n_nodes, int64_t n_src, int64_t n_edges, int n_etypes);
size_t bpt_attn_plan_workspace_bytes(int64_t n_nodes, int64_t n_src, int64_t n_edges, int n_etypes);
int bpt_attn_plan_build(const int32_t *src, const int32_t *dst, const int32_t *etype,
                        int64_t n_edges, int64_t n_nodes, int64_t n_src, int n_etypes, void *plan,
                        size_t plan_bytes, void *workspace, size_t workspace_bytes,
                        int32_t *counts_host, bpt_stream_t stream);

/* Scratch bytes of bpt_attn_forward (backward == 0) or bpt_attn_backward (backward != 0). */
size_t bpt_attn_workspace_bytes(int64_t n_nodes, int64_t n_edges, const int32_t *counts_host,
                                int h, int d, int backward);

/* q, o: (n_nodes, h, d), k, v: (n_src, h, d) of `dtype` (BPT_F32, BPT_BF16 or BPT_F16; d <= 128);
 * ak: (n_etypes, d) of `dtype` or NULL for no relative-position term; lse: fp32
 * (n_nodes, h), natural-log sum of exponentials of each row's scaled scores (-inf for a
 * row without incoming edges, whose o is 0). */
int bpt_attn_forward(const void *plan, const int32_t *counts_host, int64_t n_nodes,
                     int64_t n_edges, int n_etypes, const void *q, const void *k, const void *v,
                     const void *ak, double scale, void *o, float *lse, int h, int d, int dtype,
                     void *workspace, size_t workspace_bytes, const bpt_dropout_t *dropout, bpt_stream_t stream);

/* lse: the forward's output; d_o: gradient of o.  dq: (n_nodes, h, d), dk, dv: (n_src, h, d),
 * or both NULL to skip them;
 * dak: fp32 (n_etypes, d), required when ak is given.  The forward's o is not needed: the
 * row term <dO, O> of the softmax gradient is recomputed in fp32 from the probabilities. */
int bpt_attn_backward(const void *plan, const int32_t *counts_host, int64_t n_nodes,
                      int64_t n_edges, int n_etypes, const void *q, const void *k, const void *v,
                      const void *ak, double scale, const float *lse,
                      const void *d_o, void *dq, void *dk, void *dv, float *dak, int h, int d,
                      int dtype, void *workspace, size_t workspace_bytes, const bpt_dropout_t *dropout,
                      bpt_stream_t stream);

/* ------------------------------------------------------------------------------------
 * Tensor-core forward (bf16, head dim 64).  Same result as bpt_attn_forward within bf16
 * tolerance; the graph is given as a tile plan.  No counterpart in the reference beyond the
 * operator chain named at bpt_attn_forward.
 *
 * bpt_tile_plan_create is the planner on the host (pure integer code, no GPU needed;
 * bpt_tile_plan_create_device below makes the same plan on the device).  It takes the in-CSR as
 * host int32 arrays (in_indptr[n_nodes+1], in_src[n_edges], in_etype[n_edges] or NULL) and
 * covers the attention matrix with groups: a sorted list of source columns shared by up to
 * 8 m-blocks of <= 16 destination rows, each m-block holding a dense matrix of edge types
 * over those columns.  `group_rows` consecutive rows form a dense group when their union of
 * sources has at most `max_cols` columns and edges >= min_density * rows * columns; other
 * rows are bucketed by block of `col_block` consecutive sources: the rows of a bucket form a
 * group of their own or, with join_dense != 0, join the dense group that already stages
 * those sources; a group holds at most `max_mblocks` (<= 8) m-blocks, more spill into a
 * copy of the group; rows of at most
 * `simt_max_degree` edges outside dense groups are listed as whole-row items
 * {row, begin, end, -1} for the CUDA-core kernel instead.
 * bpt_tile_plan_sizes fills sizes[12] = {groups, m-blocks, column entries, etype cells, split
 * rows, slots, t_max, max_cols_pad, max m-blocks per group, max QR slots per group, row
 * items, dense groups}.  bpt_tile_plan_export copies groups (8 int32 each), mblocks (56 int32
 * each), cols (int32), et (uint8 if et_bytes == 1, which needs every type < 255, else
 * uint16), split_rows and row_items (4 int32 each) into host arrays of those sizes, to be
 * uploaded as they are; cell_pos (int32 per etype cell, may be NULL) is the cell's edge
 * payload: in_payload[j] of CSR entry j, or j itself when in_payload is NULL, -1 without an
 * edge.  et is stored [chunk][16][64] per m-block; cell_pos holds the same cells per chunk in
 * the order the tensor-core lanes read them: cell (r, c) of a chunk at
 * (((c / 32) * 4 + (c % 32) / 8) * 32 + (r % 8) * 4 + (c % 8) / 2) * 4 + (r / 8) * 2 + (c & 1).  The same planner serves the transposed problem (rows = sources): feed it the
 * out-CSR with in_payload = each entry's position in the in-CSR.
 * bpt_export_in_csr / bpt_export_out_csr copy the in-CSR (indptr, src, etype; a row's entries
 * ordered by source, then by edge id) / out-CSR (indptr over n_src rows, dst, position in the
 * in-CSR; a row's entries in edge-id order) of a bpt_attn_plan_build plan to host arrays (they
 * wait for the stream).
 * ---------------------------------------------------------------------------------- */
void *bpt_tile_plan_create(const int32_t *in_indptr, const int32_t *in_src, const int32_t *in_etype,
                           const int32_t *in_payload, int64_t n_nodes, int64_t n_edges, double min_density, int max_cols,
                           int group_rows, int col_block, int simt_max_degree, int max_mblocks,
                           int join_dense);
int bpt_tile_plan_sizes(const void *handle, int64_t *sizes);
int bpt_tile_plan_export(const void *handle, int32_t *groups, int32_t *mblocks, int32_t *cols, void *et,
                         int et_bytes, int32_t *cell_pos, int32_t *split_rows, int32_t *row_items);
void bpt_tile_plan_destroy(void *handle);

/* The same planner on the device (replaces, for a batch shape not seen before, the per-batch host work
 * of graph/base.py:71-86 plus the export, host planning and upload of the calls above).  Reads the
 * in-CSR (transposed = 0: rows = destinations, cells carry edge types) or the out-CSR (transposed = 1:
 * rows = sources, cells carry positions in the in-CSR) of a bpt_attn_plan_build plan where it lies and
 * produces, array for array, what bpt_tile_plan_create + bpt_tile_plan_export produce for the same
 * parameters with simt_max_degree = 0 and join_dense = 0.  It allocates its own device memory
 * (temporaries are freed before it returns, the plan's arrays by bpt_tile_plan_device_destroy) and
 * waits for the stream three times to learn array sizes.  bpt_tile_plan_device_sizes fills sizes[13]:
 * the twelve of bpt_tile_plan_sizes and the largest edge type (-1 without edges).
 * bpt_tile_plan_device_export copies into DEVICE arrays of those sizes (any of them may be NULL) and
 * waits for the stream. */
void *bpt_tile_plan_create_device(const void *attn_plan, const int32_t *counts_host, int64_t n_nodes,
                                  int64_t n_edges, int n_etypes, int transposed, double min_density,
                                  int max_cols, int group_rows, int col_block, int max_mblocks,
                                  bpt_stream_t stream);
/* The same with the column space given as `n_segs` segments (col_seg_starts_host: n_segs + 1 ascending HOST
 * values from 0 to the number of columns: the node offsets of the graphs of a block-diagonal batch,
 * graph/lm.py:59-98).  Blocks of `col_block` consecutive columns are then counted from each segment's start,
 * so every graph of the batch is cut where it is cut when planned alone (a 64-leaf span of the second
 * sequence no longer straddles two blocks because the first sequence has an odd number of nodes): fewer
 * rows spread over several tiles.  n_segs = 0 is bpt_tile_plan_create_device.  The host planner gives the
 * same plan when its column ids are shifted the same way and the exported column lists shifted back. */
void *bpt_tile_plan_create_device_aligned(const void *attn_plan, const int32_t *counts_host, int64_t n_nodes,
                                          int64_t n_edges, int n_etypes, int transposed,
                                          const int64_t *col_seg_starts_host, int n_segs, double min_density,
                                          int max_cols, int group_rows, int col_block, int max_mblocks,
                                          bpt_stream_t stream);
int bpt_tile_plan_device_sizes(const void *handle, int64_t *sizes);
int bpt_tile_plan_device_export(const void *handle, int32_t *groups, int32_t *mblocks, int32_t *cols,
                                void *et, int et_bytes, int32_t *cell_pos, int32_t *split_rows,
                                bpt_stream_t stream);
void bpt_tile_plan_device_destroy(void *handle);
int bpt_export_in_csr(const void *plan, const int32_t *counts_host, int64_t n_nodes, int64_t n_edges,
                      int n_etypes, int32_t *in_indptr_host, int32_t *in_src_host, int32_t *in_etype_host,
                      bpt_stream_t stream);

int bpt_export_out_csr(const void *plan, const int32_t *counts_host, int64_t n_nodes, int64_t n_edges,
                       int n_etypes, int32_t *out_indptr_host, int32_t *out_dst_host,
                       int32_t *out_inpos_host, bpt_stream_t stream);

/* Device copies of an exported tile plan and the matching bpt_tile_plan_sizes entries. */
typedef struct {
    const int32_t *groups, *mblocks, *cols;
    const void *et;          /* edge types per cell, uint8 or uint16 (et_bytes); may be NULL for transposed plans */
    const int32_t *cell_pos; /* edge payload per cell; may be NULL for the forward */
    const int32_t *split_rows, *row_items;
    int64_t n_groups, n_split, n_slots, n_row_items;
    int32_t et_bytes, max_cols_pad, t_max, reserved;
} bpt_tile_plan_t;

/* Shared memory per block that the tile kernels of bpt_attn_forward_tc / bpt_attn_backward_tc need
 * for a tile plan with these sizes (t_max = 0 without embed_ak).  A plan whose need exceeds the
 * 227 KB a block can have (very many edge types: the per-head tables grow with t_max) is refused
 * by those calls with BPT_ERR_UNSUPPORTED; callers ask here first and use bpt_attn_forward /
 * bpt_attn_backward instead.  Host-only, no CUDA call. */
size_t bpt_attn_tc_smem_bytes(int max_cols_pad, int t_max, int et_bytes);

size_t bpt_attn_forward_tc_workspace_bytes(int64_t n_slots, int h);

/* groups, mblocks, cols, et, split_rows, row_items: device copies of the exported arrays;
 * attn_plan / counts_host: the bpt_attn_plan_build plan of the same graph (its in-CSR is what
 * row_items index; may be NULL when there are no row items); the size arguments are the
 * matching entries of bpt_tile_plan_sizes.  q, o: (n_nodes, h, 64), k, v: (n_src, h, 64) bf16,
 * 16-byte aligned; ak: (n_etypes, 64) bf16 or NULL; lse fp32 (n_nodes, h). */
int bpt_attn_forward_tc(const int32_t *groups, int64_t n_groups, const int32_t *mblocks,
                        const int32_t *cols, const void *et, int et_bytes, const int32_t *split_rows,
                        int64_t n_split, int64_t n_slots, const int32_t *row_items,
                        int64_t n_row_items, const void *attn_plan, const int32_t *counts_host,
                        int64_t n_nodes, int64_t n_edges, int max_cols_pad, int t_max,
                        int max_mblocks, int max_qr_slots, int n_etypes, const void *q,
                        const void *k, const void *v, const void *ak, double scale, void *o,
                        float *lse, int h, int d, int dtype, void *workspace,
                        size_t workspace_bytes, const bpt_dropout_t *dropout, bpt_stream_t stream);

/* The whole backward on the tensor-core path (bf16, head dim 64): dst_tiles = the forward's tile
 * plan exported WITH cell_pos and without row items, src_tiles = the transposed tile plan
 * (bpt_tile_plan_create fed with the out-CSR of bpt_export_out_csr: indptr over n_src rows, dst
 * as columns, in_etype = NULL, in_payload = positions in the in-CSR; exported with cell_pos),
 * attn_plan / counts_host = the bpt_attn_plan_build plan of the
 * same graph.  o and lse are the forward's outputs (delta = <dO, O> per row here).  Runs the
 * destination-side tile kernel (per edge and head one word {bf16 p, bf16 dS} into the workspace,
 * K part of dQ), then the relative-position part of dQ and d embed_ak (a per-row table of dS
 * summed by edge type followed by two cuBLAS GEMMs when the tiles use at most 256 edge types,
 * per-edge CUDA-core kernels otherwise), then the
 * source-side tile kernel (dK, dV).  Single writer per output element, fixed summation orders. */
size_t bpt_attn_backward_tc_workspace_bytes(const bpt_tile_plan_t *dst_tiles, const bpt_tile_plan_t *src_tiles,
                                            const int32_t *counts_host, int64_t n_nodes, int64_t n_edges,
                                            int h);
int bpt_attn_backward_tc(const bpt_tile_plan_t *dst_tiles, const bpt_tile_plan_t *src_tiles,
                         const void *attn_plan, const int32_t *counts_host, int64_t n_nodes,
                         int64_t n_edges, int n_etypes, const void *q, const void *k, const void *v,
                         const void *ak, double scale, const void *o, const float *lse, const void *d_o,
                         void *dq, void *dk, void *dv, float *dak, int h, int d, int dtype,
                         void *workspace, size_t workspace_bytes, const bpt_dropout_t *dropout, bpt_stream_t stream);

/* ------------------------------------------------------------------------------------
 * Forward on the 5th-generation tensor cores (tcgen05.mma with accumulators in tensor memory; bf16, head
 * dim 64).  Same result as bpt_attn_forward_tc within bf16 tolerance and the same operator chain of the
 * reference (modules/attention.py:66-77).  `tiles` is a tile plan made by bpt_tile_plan_create with
 * group_rows = 128 and max_mblocks = 8 (a thread block owns 128 destination rows, one per thread and
 * tensor-memory lane), exported with 8-bit cells and without row items; at most 248 edge types when ak
 * is given.  The first 16 bytes of the workspace hold a status word that the kernel sets to 1 when one of
 * its bounded waits ran out (the block then frees its tensor memory and returns; results are invalid):
 * zero them once, read them with bpt_attn_forward_tc5_status (which waits for the stream).
 * bpt_attn_forward_tc5_smem_bytes: shared memory per block for a plan with these sizes (host only).
 * ---------------------------------------------------------------------------------- */
size_t bpt_attn_forward_tc5_smem_bytes(int max_cols_pad, int t_max);
size_t bpt_attn_forward_tc5_workspace_bytes(int64_t n_slots, int h);
int bpt_attn_forward_tc5(const bpt_tile_plan_t *tiles, int64_t n_nodes, int n_etypes, const void *q, const void *k,
                         const void *v, const void *ak, double scale, void *o, float *lse, int h, int d, int dtype,
                         void *workspace, size_t workspace_bytes, bpt_stream_t stream);
int bpt_attn_forward_tc5_status(const void *workspace, int32_t *status_host, bpt_stream_t stream);

/* ------------------------------------------------------------------------------------
 * Forward for fp32 tensors on tensor cores (head dim 64), same result as bpt_attn_forward within its
 * fp32 tolerance and the same operator chain of the reference (modules/attention.py:66-77): the tile
 * plan of bpt_attn_forward_tc (exported without row items; 8- or 16-bit cells), every product run as
 * three TF32 products on operands split into a TF32 head and an fp32 remainder.  q, o: (n_nodes, h, 64),
 * k, v: (n_src, h, 64), ak: (n_etypes, 64) or NULL, all fp32 and 16-byte aligned; lse fp32 (n_nodes, h).
 * The workspace is that of bpt_attn_forward_tc_workspace_bytes.
 * bpt_attn_forward_tc32_smem_bytes: shared memory per block for a plan with these sizes (host only).
 * ---------------------------------------------------------------------------------- */
size_t bpt_attn_forward_tc32_smem_bytes(int max_cols_pad, int t_max, int et_bytes);
int bpt_attn_forward_tc32(const bpt_tile_plan_t *tiles, int64_t n_nodes, int n_etypes, const void *q, const void *k,
                          const void *v, const void *ak, double scale, void *o, float *lse, int h, int d,
                          void *workspace, size_t workspace_bytes, const bpt_dropout_t *dropout,
                          bpt_stream_t stream);

/* Backward for fp32 tensors with the destination side on tensor cores (head dim 64), same gradients as
 * bpt_attn_backward within its fp32 tolerance (the backward of the operator chain of
 * modules/attention.py:66-77, graphop.py:42-47, 84-92, 130-137).  `tiles` is the forward's tile plan with
 * cell positions, `src_tiles` the transposed tile plan (with cell positions) or NULL; attn_plan /
 * counts_host the bpt_attn_plan_build plan of the same graph (its type buckets drive the embed_ak
 * passes, which stay on the CUDA-core kernels, as does the source side when src_tiles is NULL).  The
 * destination-side tile kernel recomputes p and dp = <dO, v> per edge with three TF32 products per
 * product, takes delta = <dO, O> from the forward's output o, and accumulates the K part of dQ; the
 * source-side tile kernel accumulates dK and dV from the per-edge scratch.  dk and dv may both be NULL; dak is required when ak is given and must be zeroed by the caller. */
size_t bpt_attn_backward_tc32_workspace_bytes(const bpt_tile_plan_t *tiles, const bpt_tile_plan_t *src_tiles,
                                              const int32_t *counts_host, int64_t n_nodes, int64_t n_edges, int h);
int bpt_attn_backward_tc32(const bpt_tile_plan_t *tiles, const bpt_tile_plan_t *src_tiles, const void *attn_plan,
                           const int32_t *counts_host, int64_t n_nodes, int64_t n_edges, int n_etypes, const void *q, const void *k,
                           const void *v, const void *ak, double scale, const void *o, const float *lse,
                           const void *d_o, void *dq, void *dk, void *dv, float *dak, int h, int d,
                           void *workspace, size_t workspace_bytes, const bpt_dropout_t *dropout,
                           bpt_stream_t stream);

/* Bytes of device memory built into the library as scratch for bpt_attn_forward_static. */
#define BPT_ATTN_STATIC_SCRATCH_BYTES (8u << 20)

/* No counterpart in the reference.  bpt_attn_forward for callers that must not allocate
 * device memory while they run: code replaying a fixed memory plan, a host thread that
 * shares the GPU with a framework whose allocator it cannot call into, a service that
 * pre-sizes everything at start-up.  Same arguments and results as bpt_attn_forward, minus
 * the workspace: the scratch for rows split over several work items is a fixed
 * BPT_ATTN_STATIC_SCRATCH_BYTES (8 MiB) array inside the library image, resident on every
 * GPU that loads the library until the process exits.  The call allocates and frees
 * nothing.  A graph whose split rows need more than that (about ten sequences of n = 8192,
 * k = 4 at 8 heads x 64; one sequence of n = 65536 does not fit) is rejected with
 * BPT_ERR_WORKSPACE and nothing is launched.
 * The first call on each device looks up the array's device address (the device must be
 * current, as for every call here); make that first call outside any stream capture.
 * All calls on a device share the one array: nothing in it has to be zero beforehand
 * (every slot that is read is written earlier in the same call), but two calls that may run
 * at the same time on one GPU, on different streams or from different threads, overwrite
 * each other's partial results; order them on one stream or with events. */
int bpt_attn_forward_static(const void *plan, const int32_t *counts_host, int64_t n_nodes,
                            int64_t n_edges, int n_etypes, const void *q, const void *k,
                            const void *v, const void *ak, double scale, void *o, float *lse,
                            int h, int d, int dtype, bpt_stream_t stream);

/* ------------------------------------------------------------------------------------
 * y = LayerNorm(x + r) over the last dimension in one pass (r may be NULL: plain LayerNorm).
 * The blocks of modules/attention.py end each half with norm(h + sublayer(h))
 * (attention.py:79-81, 141, 168-171); the reference spells it with torch operators.
 * x, r, y: (n_rows, dim) of `dtype` (BPT_F32, BPT_BF16, BPT_F16), gamma, beta: (dim) of the same
 * type (either may be NULL), all 16-byte aligned; dim a multiple of 8, at most 4096.  Statistics in
 * fp32, biased variance, as torch.nn.LayerNorm.
 * ---------------------------------------------------------------------------------- */
int bpt_add_layer_norm(const void *x, const void *r, const void *gamma, const void *beta, double eps, void *y,
                       int64_t n_rows, int dim, int dtype, bpt_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* BPT_B200_H_ */
