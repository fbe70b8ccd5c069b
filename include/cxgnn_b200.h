/*
 * cxgnn_b200.h — C ABI of libcxgnn_b200.so, the sm_100a aggregation engine that
 * stands in for the kernels behind the `cxgnncomp_backend` extension module of
 * CxGNN-Compute (src/cpp/python_bindings/binding.cpp:14-130).
 *
 * Conventions, all entry points:
 *   - plain C, `extern "C"`; every pointer is a DEVICE pointer unless the
 *     parameter name ends in `_host`;
 *   - returns CXG_OK (0) or a negative CXG_E* code; never exits, aborts, resets
 *     the device or throws; `cxg_last_error_string()` gives the reason for the
 *     last failure on the calling thread;
 *   - no allocation and no synchronisation: scratch memory is passed in by the
 *     caller (`*_workspace_size` tells how much) and kernels are enqueued on
 *     `stream` (a `cudaStream_t` passed as `void*`; NULL = the legacy default
 *     stream, which is what the reference launches on);
 *   - CSR_Layer graph format of the reference: `ptr[n_dst+1]`, `idx[nnz]`, row r
 *     holds the source ids of destination r; features are row-major and
 *     contiguous.
 */
#ifndef CXGNN_B200_H_
#define CXGNN_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ------------------------------------------------------- */
#define CXG_OK 0
#define CXG_EINVAL (-1)       /* bad size, flag or combination of arguments   */
#define CXG_ENULL (-2)        /* a required pointer is NULL                   */
#define CXG_EUNSUPPORTED (-3) /* valid request that this build does not cover */
#define CXG_ECUDA (-4)        /* a CUDA call or kernel launch failed          */
#define CXG_EWORKSPACE (-5)   /* workspace missing or too small               */
#define CXG_ETIMEOUT (-6)     /* a bounded device-side wait ran out           */
#define CXG_ELIMIT (-7)       /* size beyond a fixed limit of the entry point */

/* ---- element types ------------------------------------------------------ */
#define CXG_F32 0
#define CXG_BF16 1

/* ---- reductions ----------------------------------------------------------*/
#define CXG_SUM 0
#define CXG_MEAN 1

/* ---- flags of cxg_spmm_csr ---------------------------------------------- */
#define CXG_SPMM_ACCUMULATE 1u /* y[row] += result instead of y[row] = result */
/* Row-fetch variant of the tiled kernel, kept for measurement; results are
   bit-identical. Default: 16-byte async copies into shared memory. */
#define CXG_SPMM_BULK_ROWS 4u /* one bulk async copy (TMA) per row into shared
                                 memory, completion on an mbarrier             */
/* Test hook of the bulk-copy variant: the first stage of the first tile announces 16 bytes
   that no copy delivers, so that its bounded wait runs out and the time-out path (status
   CXG_ETIMEOUT, kernels return, nothing written out of bounds) can be exercised. Use it
   with a short cxg_set_wait_limit_cycles. */
#define CXG_SPMM_TEST_STALL 8u
/* Measurement aid: rows of 128 / 256 / 512 bytes without edge values normally take a leaner
   instantiation of the tiled walk; this flag keeps them on the general one. Same results. */
#define CXG_SPMM_GENERIC_WALK 16u
/* The tiled kernel normally keeps six persistent CTAs on every SM; with this flag it keeps four, so
   that a kernel launched from another stream meanwhile (the copy kernel of a collective that overlaps
   this aggregation) finds room on every SM instead of waiting for this kernel to end. Same results. */
#define CXG_SPMM_SHARE_SMS 32u
/* Index-stream variant of the lean walk (rows of 128 / 256 / 512 bytes): the source ids of a tile are staged
   into shared memory by the bulk-copy unit (one 512-byte `cp.async.bulk` per 128 int32 / 64 int64 ids, two
   chunks per warp, the next one requested while the current one is read, completion on an mbarrier with a
   bounded wait) instead of being loaded by the lanes one stage ahead. Needs a 16-byte aligned `idx`; ignored
   otherwise and on the general walk. Same results bit for bit. CXG_SPMM_TEST_STALL makes every warp's first
   chunk announce 16 bytes that never arrive. */
#define CXG_SPMM_TMA_INDEX 64u

const char *cxg_last_error_string(void);
int cxg_abi_version(void);
/* Kernels launched by this library in this process so far (all threads). */
long long cxg_kernel_launch_count(void);

/*
 * Description of one CSR aggregation  y[t(r), h, :] (+)= red_{e in row r} v[e,h] * x[s(e), h, :]
 * shared by the SpMM entry points below.
 *
 *   ptr        int64 (ptr_bytes 8) or int32 (ptr_bytes 4), n_dst+1 entries
 *   idx        int64 (idx_bytes 8) or int32 (idx_bytes 4), source id per edge
 *   x          [n_src, heads, feat]  dtype
 *   y          [n_out, heads, feat]  dtype
 *   edge_val   optional float32 [nnz, heads]; NULL = all ones
 *   edge_mask  optional uint8/bool [nnz]; 0 = skip the edge          (selective_aggr)
 *   edge_rel   optional int32 [nnz]; source row becomes rel*rel_stride + idx  (aggr_rel)
 *   targets    optional int64 [n_dst]; output row of CSR row r; NULL = r      (target_aggr)
 *   reduce     CXG_SUM or CXG_MEAN (mean divides by the row's edge count; rows
 *              without edges give 0)
 *
 * Arithmetic: one fp32 accumulator per (row, column), edges added strictly in
 * CSR order (fma when an edge value is given). Rows longer than the split
 * threshold are cut into fixed segments whose partial sums are added in segment
 * order, so results never depend on scheduling.
 */
typedef struct cxg_spmm_desc {
  const void *ptr;
  const void *idx;
  const void *x;
  void *y;
  const float *edge_val;
  const uint8_t *edge_mask;
  const int32_t *edge_rel;
  const int64_t *targets;
  int64_t n_dst;
  int64_t nnz;
  int64_t rel_stride;
  int32_t feat;
  int32_t heads;
  int32_t dtype;
  int32_t ptr_bytes;
  int32_t idx_bytes;
  int32_t reduce;
  uint32_t flags;
  int32_t split_edges; /* rows with more edges are split; 0 = default (256) */
} cxg_spmm_desc;

/*
 * The kernels never spin without a limit: a wait on an mbarrier (the bulk-copy variant of cxg_spmm_csr,
 * the pipeline of cxg_typed_matmul) gives up after a cycle limit (default 2^31 cycles, about a second;
 * cxg_set_wait_limit_cycles changes it for the launches that follow, 0 restores the default), records that
 * in the call's workspace and returns. These two read the record: they WAIT for everything queued on
 * `stream`, then return CXG_OK, CXG_ETIMEOUT (a wait ran out) or, for cxg_spmm_csr, CXG_EINVAL (ptr[n_dst]
 * was larger than desc->nnz: the kernels read only the declared edges); in both failure cases the result of
 * the call that used `workspace` last is incomplete. Optional: nothing else in the library synchronises.
 */
int cxg_set_wait_limit_cycles(long long cycles);
int cxg_spmm_csr_status(const void *workspace, void *stream);
int cxg_typed_matmul_status(const void *workspace, void *stream);

/*
 * Weight gradient of the typed linear: dW[r] = sum over the positions m with rel[m] == r of x[ix(m), :]^T g[ig(m), :],
 * dW float32 [num_rel, k, n]. Positions are those of cxg_typed_matmul (sorted by relation, every aligned block of 128
 * one relation); ix(m) = idx[m] (NULL: m), ig(m) = idx_g[m] (NULL: ix(m)); a position counts only when ix(m) is in
 * [0, x_rows) and ig(m) in [0, g_rows). Replaces the per-relation loop of torch.mm over row sets in
 * TypedLinearE2EOP.backward (cxgnncomp/typed_linear.py:115-137) by one launch on the tensor cores (a contraction
 * over positions, both operands MN-major) plus a fixed-order reduction of per-CTA partial sums: no atomics. An
 * accumulator in tensor memory takes a few thousand positions at most and the partial sums are added in ordinary
 * fp32, so the error does not grow with the number of rows. precision 1 = plain bf16 / TF32 products, 2 =
 * error-compensated TF32 for fp32 inputs (1e-5 class). Shapes: k == 128, n * element size a multiple of 128 bytes,
 * n <= 256, one stage within shared memory (CXG_EUNSUPPORTED otherwise). cxg_typed_wgrad_status reads back whether a
 * bounded wait ran out.
 */
int cxg_typed_wgrad_workspace_size(int num_rel, int k, int n, size_t *bytes);
/* Test hook: the first tile of every CTA is never handed to the tensor-core role, so the bounded waits for it run out
   (status CXG_ETIMEOUT, all roles leave, tensor memory is released). Use it with a short cxg_set_wait_limit_cycles. */
#define CXG_WGRAD_TEST_STALL 1u
int cxg_typed_wgrad(const void *x, const void *g, const int64_t *rel, const int64_t *idx, const int64_t *idx_g,
                    int64_t m, int64_t x_rows, int64_t g_rows, int k, int n, int num_rel, int dtype, int precision,
                    uint32_t flags, float *dw, void *workspace, size_t workspace_bytes, void *stream);
int cxg_typed_wgrad_status(const void *workspace, void *stream);

/*
 * Scratch bytes needed by cxg_spmm_csr for a graph with n_dst rows and nnz
 * edges at row width heads*feat (split_edges as in the descriptor). Upper bound;
 * depends on sizes only.
 */
int cxg_spmm_csr_workspace_size(int64_t n_dst, int64_t nnz, int32_t feat,
                                int32_t heads, int32_t split_edges,
                                size_t *bytes);

/*
 * CSR SpMM forward. Replaces, depending on the optional fields of `desc`:
 *   sage_sum_forward / sage_mean_forward            src/cpp/src/aggr.cu:385-393
 *   sage_sum_forward_edge_value (1 head / H heads)  src/cpp/src/aggr.cu:377-383
 *   run_spmm_configurable{,_int32}                  src/cpp/src/spmm_host.cu:6-55,99-156
 *   spmm_multihead, Naive schedule                  src/cpp/src/spmm_host.cu:158-181
 *   selective_aggr                                  src/cpp/src/aggr.cu:478-492
 *   target_aggr                                     src/cpp/src/aggr.cu:450-463
 *   aggr_rel                                        src/cpp/src/rel_spmm.cu:37-70
 * The workspace holds the split plan of long rows and their partial sums; it is
 * rebuilt on every call and carries no state between calls.
 */
int cxg_spmm_csr(const cxg_spmm_desc *desc, void *workspace,
                 size_t workspace_bytes, void *stream);

/*
 * CSR SpMM backward for the aggregation `desc` describes (desc->y is unused,
 * desc->x is the forward input and only needed for dval):
 *   dx[s(e),h,:]  += v[e,h] * dy[t(r),h,:]     (divided by the row's edge count for mean)
 *   dval[e,h]      = <dy[t(r),h,:], x[s(e),h,:]>
 * dy has desc->dtype; dx [n_src, heads, feat] and dval [nnz, heads] are float32,
 * either may be NULL. dx is ADDED INTO, so the caller zero-fills it first (the
 * reference does: torch::zeros_like, src/cpp/src/aggr.cu:196). The additions
 * into dx are vector atomics whose order is not fixed, as in the reference.
 * Replaces sageBackwardImpl (src/cpp/src/aggr.cu:189-273), run_spmm_configurable_bwd
 * (src/cpp/src/spmm_host.cu:57-97), spmm_multihead_bwd (spmm_host.cu:198-214),
 * selective_aggr_bwd / target_aggr_backward (aggr.cu:465-509) and aggr_rel's
 * backward (src/cpp/src/rel_spmm.cu:106-135).
 */
int cxg_spmm_csr_backward(const cxg_spmm_desc *desc, const void *dy, float *dx,
                          float *dval, void *stream);

/*
 * Transposed graph of a CSR_Layer graph, built on the device by a stable radix sort of the edges by
 * source id (no atomics, same result on every run; equal to a stable sort of idx):
 *   t_ptr [n_src + 1] int64    transposed row of source s = [t_ptr[s], t_ptr[s+1])
 *   t_idx [nnz]  (idx width)   destination (forward row) of every transposed edge, ascending inside a row
 *   t_eid [nnz]  (idx width)   forward edge id of every transposed edge (optional, may be NULL)
 *   inv_deg [n_dst] float      1 / max(1, edges of forward row r) (optional, may be NULL)
 * Only the first min(ptr[n_dst], nnz) edges are read. With it dX = A^T dY runs on cxg_spmm_csr over
 * (t_ptr, t_idx) instead of the atomic scatter of the reference's backward kernels
 * (src/cpp/src/aggr_kernel.cu:188-249); the reference has no transpose of its own: AggrOP.backward
 * assumes a symmetric graph instead (cxgnncomp/graph_conv.py:57-77). nnz < 2^31, n_src < 2^32.
 */
int cxg_csr_transpose_workspace_size(int64_t nnz, size_t *bytes);
int cxg_csr_transpose(const void *ptr, const void *idx, int ptr_bytes, int idx_bytes,
                      int64_t n_dst, int64_t n_src, int64_t nnz, int64_t *t_ptr, void *t_idx,
                      void *t_eid, float *inv_deg, void *workspace, size_t workspace_bytes,
                      void *stream);

/*
 * Edge softmax of GAT. For every destination d and head h over the edges e of row d:
 *   t = att_dst[d,h] + att_src[idx[e],h];  t = max(t, t*slope)      (LeakyReLU)
 *   out[e,h] = exp(t - max_row t) / sum_row exp(t - max_row t);     mask[e,h] = t > 0
 * att_dst [n_dst, heads], att_src [n_src, heads], out [nnz, heads] float32, mask
 * [nnz, heads] bytes. Replaces edge_attention / EdgeSoftMaxFunction::forward and
 * edge_softmax_fwd (src/cpp/src/edge_softmax.cu:3-42,97-132). Same summation order per
 * row as the reference for rows of up to 1024 edges; exp is the accurate expf where the
 * reference uses the fast __expf. Workspace: cxg_edge_softmax_workspace_size bytes.
 */
int cxg_edge_softmax_workspace_size(int64_t n_dst, int64_t nnz, size_t *bytes);
int cxg_edge_softmax_forward(const void *ptr, const void *idx, int ptr_bytes,
                             int idx_bytes, const float *att_dst,
                             const float *att_src, float *out, uint8_t *mask,
                             int64_t n_dst, int64_t nnz, int heads, float slope,
                             void *workspace, size_t workspace_bytes, void *stream);

/*
 * Backward of the edge softmax (edge_softmax_bwd, src/cpp/src/edge_softmax.cu:44-95,
 * 143-170): with s = sum_row out*grad, tmp = out*(grad - s), times slope where mask is 0;
 * grad_src[idx[e],h] += tmp (atomic); grad_dst[d,h] = sum_row tmp, written only for rows
 * that have both mask values (it is zero otherwise). grad_dst [n_dst, heads] and grad_src
 * [n_src, heads] must be zero-filled by the caller, as the reference does.
 */
int cxg_edge_softmax_backward(const void *ptr, const void *idx, int ptr_bytes,
                              int idx_bytes, const float *grad, const uint8_t *mask,
                              const float *out, float *grad_dst, float *grad_src,
                              int64_t n_dst, int64_t nnz, int heads, float slope,
                              void *workspace, size_t workspace_bytes, void *stream);

/*
 * Fused GAT aggregation: score, LeakyReLU, edge softmax and weighted neighbour sum in one walk over the edges,
 * without any [nnz, heads] array in memory. Replaces, for one layer, the sequence edge_attention ->
 * sage_sum_forward_edge_value / SpMMValOP of MyGATConv.forward_many (cxgnncomp/graph_conv.py:458-496,
 * src/cpp/src/edge_softmax.cu:3-95, src/cpp/src/aggr_kernel.cu:155-186,443-491).
 *   forward:  y[r,h,:] = sum_e p[e,h] x[idx[e],h,:],  p = softmax over row r of leaky(a_dst[r,h] + a_src[idx[e],h]);
 *             also row_max[r,h] and row_sum[r,h] (max and sum of exp(t - max) of the row; -1e30 / 0 for rows
 *             without edges), which is all the backward needs to recompute p.
 *   backward: walks the TRANSPOSED graph (t_ptr over the n_src sources, t_idx = destinations, as
 *             cxg_csr_transpose builds it): dx [n_src, heads, c], d_a_src [n_src, heads] (both written, fixed
 *             order) and d_a_dst [n_dst, heads]. With t_eid (the forward edge of every transposed edge, third
 *             output of cxg_csr_transpose, width idx_bytes) and fwd_ptr (row pointers of the forward graph,
 *             fwd_ptr_bytes wide) every edge's score gradient is parked at its forward position in the
 *             workspace and d_a_dst[r] is the sum over row r's edges in a fixed order: every output is the
 *             same on every run (about 14 % more time for a layer's forward + backward at the GAT configuration).
 *             With both NULL d_a_dst is zeroed and added into with atomics, like the reference's grad_src.
 * x [n_src, heads, c], y / dy [n_dst, heads, c] float32; heads a power of two <= 16; heads * c * 4 must be
 * 128, 256 or 512 bytes (CXG_EUNSUPPORTED otherwise: use the separate kernels). exp is the fast __expf, like
 * the reference's fast-math build; results agree with the three-pass formulation to fp32 rounding, not bit
 * for bit (the running maximum changes the order of the roundings).
 */
int cxg_gat_fused_workspace_size(int64_t n_dst, int64_t nnz, int heads, int c, size_t *bytes);
int cxg_gat_fused_forward(const void *ptr, const void *idx, int ptr_bytes, int idx_bytes, const float *x,
                          const float *a_src, const float *a_dst, float *y, float *row_max, float *row_sum,
                          int64_t n_dst, int64_t nnz, int heads, int c, float slope, void *workspace,
                          size_t workspace_bytes, void *stream);
int cxg_gat_fused_backward(const void *t_ptr, const void *t_idx, int ptr_bytes, int idx_bytes,
                           const float *dy, const float *y, const float *x, const float *a_src,
                           const float *a_dst, const float *row_max, const float *row_sum, float *dx,
                           float *d_a_src, float *d_a_dst, int64_t n_src, int64_t n_dst, int64_t nnz,
                           int heads, int c, float slope, const void *t_eid, const void *fwd_ptr,
                           int fwd_ptr_bytes, void *workspace, size_t workspace_bytes, void *stream);

/*
 * SDDMM on an edge list: out[e,h] = <src_feat[src[e],h,:], dst_feat[dst[e],:]>, src_feat
 * [n_src, heads, feat], out [n_edge, heads]. dst_per_head = 0: dst_feat is [n_dst, feat]
 * as in run_sddmm / sddmm_multihead (src/cpp/src/sddmm_host.cu:4-14, sddmm_kernel.cu:3-25);
 * dst_per_head = 1: dst_feat is [n_dst, heads, feat] (the head-wise product that the
 * gradient of a multi-head SpMM with respect to its edge values needs).
 */
int cxg_sddmm_coo(const void *src, const void *dst, int idx_bytes,
                  const float *src_feat, const float *dst_feat, float *out,
                  int64_t n_edge, int feat, int heads, int dst_per_head,
                  void *stream);

/* out[e] = 1 / (edges of e's row): edge_value_degree (src/cpp/src/edge_softmax.cu:186-214). */
int cxg_edge_value_degree(const void *ptr, int ptr_bytes, float *out, int64_t n_dst,
                          void *stream);

/* y[d] = sum over row d of x[idx[e]]: spmv (src/cpp/src/edge_softmax.cu:216-244). */
int cxg_spmv_csr(const void *ptr, const void *idx, int ptr_bytes, int idx_bytes,
                 const float *x, float *y, int64_t n_dst, void *stream);

/*
 * Generalised SpMM of the dgSPARSE surface, GSpMM_u (val = NULL) and GSpMM_u_e
 * (src/cpp/include/dgsparse.h:14-131, src/cpp/src/dgsparse.cu:324-475, python_bindings/binding.cpp:87-119):
 * y[r, c] = REDUCE over the edges e of row r of COMPUTE(val[e], x[idx[e], c]), fp32, edges in CSR order.
 * The accumulator starts at 0, (float)INT_MIN or (float)INT_MAX; rows without edges give 0; mean divides
 * by the edge count. compute: add v + x, sub x - v, mul v * x (fused into the sum), div x / v.
 */
#define CXG_ROP_SUM 0
#define CXG_ROP_MAX 1
#define CXG_ROP_MIN 2
#define CXG_ROP_MEAN 3
#define CXG_COP_ADD 0
#define CXG_COP_SUB 1
#define CXG_COP_MUL 2
#define CXG_COP_DIV 3
int cxg_gspmm_csr(const void *ptr, const void *idx, int ptr_bytes, int idx_bytes, const float *val,
                  const float *x, float *y, int64_t n_dst, int feat, int reduce_op, int compute_op,
                  void *stream);

/*
 * The two attention scores of a GAT layer in one pass over the transformed features
 * (cxgnncomp/graph_conv.py:470-474: `(x_src * att_src).sum(-1)`, `(x_dst * att_dst).sum(-1)`):
 * alpha_src[n, h] = <feat[n, h, :], att_src[h, :]> for n < n_src, alpha_dst[n, h] = <feat[n, h, :], att_dst[h, :]>
 * for n < n_dst <= n_src. feat [n_src, heads, c] fp32. The backward writes
 * grad_feat[n, h, :] = g_src[n, h] * att_src[h, :] + (n < n_dst) * g_dst[n, h] * att_dst[h, :].
 */
int cxg_gat_scores(const float *feat, const float *att_src, const float *att_dst, float *alpha_src,
                   float *alpha_dst, int64_t n_src, int64_t n_dst, int heads, int c, void *stream);
int cxg_gat_scores_backward(const float *g_src, const float *g_dst, const float *att_src,
                            const float *att_dst, float *grad_feat, int64_t n_src, int64_t n_dst,
                            int heads, int c, void *stream);
/*
 * Gradients of the two attention vectors of the same step (the reference leaves them to autograd through the
 * multiply + sum pairs): grad_att_src[h, :] = sum_n g_src[n, h] feat[n, h, :] over n < n_src,
 * grad_att_dst[h, :] = sum_n g_dst[n, h] feat[n, h, :] over n < n_dst, both [heads, c], in one pass over feat with a
 * fixed two-level order of additions (contiguous row chunks, then the chunks in order).
 */
int cxg_gat_att_grad_workspace_size(int heads, int c, size_t *bytes);
int cxg_gat_att_grad(const float *feat, const float *g_src, const float *g_dst, float *grad_att_src,
                     float *grad_att_dst, int64_t n_src, int64_t n_dst, int heads, int c, void *workspace,
                     size_t workspace_bytes, void *stream);

/*
 * out[c] = sum over the n_row rows of x[r, c] (x row-major [n_row, width], dtype CXG_F32 or CXG_BF16, out float32):
 * the gradient of the bias that MyGATConv / MyGCNConv add to every output row (cxgnncomp/graph_conv.py:493-494,
 * 543-545, 622-623; the reference leaves it to autograd's sum). Fixed two-level order of additions (contiguous row chunks,
 * then the chunks in order), no atomics.
 */
int cxg_column_sum_workspace_size(int width, size_t *bytes);
int cxg_column_sum(const void *x, int dtype, int64_t n_row, int width, float *out, void *workspace,
                   size_t workspace_bytes, void *stream);

/*
 * out[r, f] = sum over heads of in[r, h, f] (heads added in order into one fp32 accumulator): the head
 * reduction of spmm_multihead's PreReduce / Optimal schedules, which return [n, feat]
 * (src/cpp/src/spmm_host.cu:158-196).
 */
int cxg_head_sum(const void *in, void *out, int64_t n_row, int heads, int feat, int dtype,
                 void *stream);

/*
 * gather / GatherFunction (src/cpp/src/aggr.cu:42-62,395-448). backward = 0:
 * out[dest[e],:] += in[e,:] (out [n_node, feat] zero-filled by the caller, atomic adds);
 * backward = 1: out[e,:] = in[dest[e],:].
 */
int cxg_gather_edges(const float *in, const void *dest, int idx_bytes, float *out,
                     int64_t n_edge, int feat, int backward, void *stream);

/*
 * Relation-bucket padding: pad_rel / pad_rel_idx (src/cpp/src/stitch_kernel.cu:3-53).
 * rel (int64, length base + num_rel*(thres-1)) holds the relation of every item in
 * rel[0..base); pad slot t belongs to relation t/(thres-1) and is turned into a member of it
 * while that relation's count is short of a multiple of thres, else into the dummy relation
 * num_rel. idx (optional, same length) gets -1 in every pad slot. count: int64 [num_rel].
 */
int cxg_pad_rel(int64_t *rel, int64_t *idx, const int64_t *count, int thres,
                int num_rel, int64_t base, void *stream);

/*
 * Typed linear, one output row per item, exact fp32 (fma in k order):
 *   src == NULL:              out[i]      += x[i]      . W[types[i]]   typed_linear
 *   src != NULL, dst == NULL: out[i]      += x[src[i]] . W[types[i]]   typed_linear_s2e
 *   src and dst:              out[dst[i]] += x[src[i]] . W[types[i]]   typed_linear_s2d (atomic)
 * (run_typed_linear{,_s2e,_s2d}, src/cpp/src/rel_spmm.cu:231-358). x [n_rows_x, k],
 * W [num_rel, k, n], types int32 [num].
 */
int cxg_typed_linear(const float *x, const float *w, float *out, const int32_t *types,
                     const int64_t *src, const int64_t *dst, int64_t num,
                     int64_t n_rows_x, int k, int n, int num_rel, void *stream);

/*
 * y[d,:] = sum over row d of x[idx[e],:] . W[rel[e]]: aggr_rgcn_direct_func
 * (src/cpp/src/rel_spmm.cu:138-181,442-467). rel int32 [nnz], fp32.
 */
int cxg_rgcn_direct(const void *ptr, const void *idx, int ptr_bytes, int idx_bytes,
                    const int32_t *rel, const float *x, const float *w, float *y,
                    int64_t n_dst, int k, int n, void *stream);

/*
 * out[i, :] = in[rows[i], :] for rows of row_bytes bytes (even; 16-byte accesses when pointers and
 * row size allow): the pack step of the needed-rows feature exchange between GPUs, the reference's
 * "densify" (test/1-kernels/test_mgpu_model.py:227-331). rows int64 [n_rows].
 */
int cxg_gather_rows(const void *in, const int64_t *rows, void *out, int64_t n_rows,
                    int64_t row_bytes, void *stream);

/*
 * Peer mappings for the exchange between the GPUs of one node (one process per GPU). cxg_ipc_export gives the
 * 64-byte CUDA IPC handle of the allocation that holds `ptr` and ptr's offset inside it; the other process calls
 * cxg_ipc_open WITH ITS OWN GPU CURRENT and receives the base of a mapping of that allocation in its own context
 * (lazy peer access over NVLink; the mapping is probed with a small copy before it is handed out), to be released
 * with cxg_ipc_close. An allocation can be opened once per process. cxg_copy_async is a device-to-device
 * cudaMemcpyAsync (copy engines) for moving packed rows into such a mapping.
 *
 * cxg_put_rows fuses the pack step with the transfer: row i of the list goes to peer q = the segment
 * [seg_start[q], seg_start[q+1]) that holds i, at peer_base[q] + (i - seg_start[q]) * row_bytes, where peer_base[q]
 * points into a mapping obtained from cxg_ipc_open (already offset to the first row q expects from this rank).
 * Plain 16-byte stores over NVLink, all peers written concurrently; no send buffer, no collective kernel.
 * peer_base_host and seg_start_host (n_peer and n_peer + 1 entries) are HOST arrays. The caller orders the step
 * across ranks (nobody may still read the destination; the receiver may read it once every sender's kernel has
 * completed). Replaces the pack + NCCL send / receive pair of the reference's "densify" exchange
 * (test/1-kernels/test_mgpu_model.py:227-331). n_peer <= 16, row_bytes a multiple of 16.
 */
int cxg_ipc_export(const void *ptr, unsigned char *handle64, int64_t *offset_bytes);
int cxg_ipc_open(const unsigned char *handle64, void **base);
int cxg_ipc_close(void *base);
int cxg_copy_async(void *dst, const void *src, int64_t bytes, void *stream);
int cxg_put_rows(const void *in, const int64_t *rows, void *const *peer_base_host,
                 const int64_t *seg_start_host, int n_peer, int64_t row_bytes, void *stream);


/*
 * Neighbour sampling for mini-batches in the CSR_Layer format (the step the reference takes from its
 * external loader: neighbor_sample at cxgnncomp/data_preparation.py:214-215, test/ae/E2_spmm/perf-spmm.py:45-46).
 * For frontier node v = frontier[i] with in-degree d: out[out_ptr[i] .. out_ptr[i] + min(d, fanout)) receives
 * min(d, fanout) distinct in-neighbours of v (global ids), in the order of v's CSR row; all of them when
 * d <= fanout, else a uniform subset drawn by Floyd's algorithm from a counter-based generator keyed by
 * (seed, v). out_ptr is the caller's exclusive prefix sum of min(d, fanout). fanout <= 64.
 */
/* counts[i] = min(in-degree of frontier[i], fanout): the row lengths whose prefix sum is out_ptr below. */
int cxg_sample_counts(const void *graph_ptr, int ptr_bytes, const int64_t *frontier, int64_t n_front,
                      int fanout, int64_t *counts, void *stream);
int cxg_sample_neighbors(const void *graph_ptr, const void *graph_idx, int ptr_bytes, int idx_bytes,
                         const int64_t *frontier, int64_t n_front, int fanout,
                         const int64_t *out_ptr, int64_t *out, uint64_t seed, void *stream);

/*
 * Renumbering of sampled neighbours into batch-local ids (what the reference's loader does before it hands
 * over a CSR_Layer batch). local_of [num_nodes] int64 maps global id -> position in the batch, -1 outside it.
 * cxg_renumber_claim appends every id of picked[] that has no position yet to fresh[] exactly once (in no
 * fixed order; *n_fresh, a device counter, receives how many) and marks it as claimed (-2). The caller reads
 * n_fresh, sorts fresh[0 .. n_fresh) and calls cxg_renumber_assign: local_of[fresh_sorted[i]] = base + i, then
 * out[i] = local_of[picked[i]]. fresh needs room for min(n_picked, num_nodes) entries.
 */
int cxg_renumber_claim(const int64_t *picked, int64_t n_picked, int64_t *local_of, int64_t *fresh,
                       int64_t *n_fresh, void *stream);
int cxg_renumber_assign(const int64_t *fresh_sorted, int64_t n_fresh, int64_t base,
                        const int64_t *picked, int64_t n_picked, int64_t *local_of, int64_t *out,
                        void *stream);

/*
 * topo_sort (src/cpp/src/schedule.cu:72-124, python_bindings/binding.cpp:33) on HOST arrays: nodes in
 * the order a breadth-first release by remaining in-degree gives; ptr/idx list the out-edges, degree
 * the in-degrees. Cycles are stepped through as the reference does (degree-1 nodes, then the first
 * node of the smallest remaining degree). order [n_node]; *n_order = nodes released.
 */
int cxg_topo_sort_host(const int64_t *ptr_host, const int64_t *idx_host,
                       const int64_t *degree_host, int64_t n_node, int64_t *order_host,
                       int64_t *n_order);

/*
 * Per-relation sub-graphs on the host: rel_schedule (src/cpp/src/schedule.cu:5-63).
 * All pointers are HOST pointers; outputs are caller-allocated, row-major per relation:
 * sub_ptr [num_rel][n_dst+1], sub_idx [num_rel][nnz], sub_target [num_rel][n_dst],
 * counts [num_rel][2] = (rows kept, edges kept), n_in_layer [num_rel][num_layer].
 */
int cxg_rel_schedule_host(const int64_t *ptr_host, const int64_t *idx_host,
                          const int32_t *rel_host, int64_t n_dst,
                          const int64_t *num_node_in_layer_host, int num_layer,
                          int num_rel, int64_t *sub_ptr_host, int64_t *sub_idx_host,
                          int64_t *sub_target_host, int64_t *counts_host,
                          int64_t *n_in_layer_host);

/*
 * Typed matmul: C[oc(m),:] = A[ia(m),:] . W[rel[m]] for m in [0, m), where every aligned
 * block of 128 positions holds one relation (rel[m] >= num_rel marks padding),
 *   ia(m) = src_idx ? src_idx[m] : m          (positions with ia outside [0, m_valid) are padding)
 *   oc(m) = dst_idx ? dst_idx[m] : (src_idx && !seq_output ? ia(m) : m).
 * Replaces typed_matmul and its four Triton kernels (cxgnncomp/codegen/
 * triton_typed_matmul.py:145-860). A [*, k], W [num_rel, k, n], C [*, n] of dtype (fp32/bf16).
 * precision 1: tcgen05 tensor cores, fp32 accumulation in tensor memory (bf16 inputs, or fp32
 * inputs as TF32 like the reference's tl.dot: about 1e-3 relative); precision 2: fp32 inputs with
 * error-compensated TF32 (every operand split into two TF32 terms, three products per term summed in
 * the same accumulator: fp32 accuracy, about 1e-6; same as 1 for bf16). Both need k % 16 == 0
 * (bf16) / % 8 (fp32), n % 16 == 0, n <= 256. precision 0: exact fp32 fma of every product (no
 * tensor cores), any k, n.
 * flags: CXG_TMM_SEQ_OUTPUT as above; CXG_TMM_ATOMIC_F32 adds the rows into C, which is then
 * float32 [*, n] whatever dtype is (vector atomics; rows of C may be hit by many positions, e.g.
 * oc = destination node of an edge, which fuses the segment sum of the RGCN layer into the
 * matmul; the caller zero-fills C; the order of the additions is not fixed).
 */
#define CXG_TMM_SEQ_OUTPUT 1
#define CXG_TMM_ATOMIC_F32 2
/* Dense mode: C[r * m + i, :] = A[i, :] . W[r] for every row i < m and EVERY relation r (C is [num_rel * m, n]):
   the "transform every node with every relation's weight" step of TypedLinearS2DMMAggrOP
   (cxgnncomp/typed_linear.py:191-221) as one launch. rel, src_idx, dst_idx must be NULL, m_valid == m,
   precision 1 or 2. */
#define CXG_TMM_ALL_RELATIONS 8
/* Measurement aid: the dense mode normally fetches the tiles of A with tiled bulk tensor copies (boxes of 128 rows x
   128 bytes, 128-byte swizzle); this flag keeps the 16-byte asynchronous copies. Same results. */
#define CXG_TMM_NO_TMA 16
/* Measurement aid: rows gathered by index (read once each) are fetched by the bulk tensor copy unit in its gathering
   form (tile::gather4, four rows of 128 bytes per request) instead of 16-byte asynchronous copies. Same results;
   slower on every shape measured, hence not the default. */
#define CXG_TMM_GATHER4 32
/* Test hook: the first tile of every CTA is never handed to the tensor-core role, so the bounded
   waits for it run out (status CXG_ETIMEOUT, all roles leave, tensor memory is released). Use it
   with a short cxg_set_wait_limit_cycles. */
#define CXG_TMM_TEST_STALL 4
int cxg_typed_matmul_workspace_size(int num_rel, int k, int n, int dtype, size_t *bytes);
int cxg_typed_matmul(const void *a, const void *w, void *c, const int64_t *rel,
                     const int64_t *src_idx, const int64_t *dst_idx, int64_t m,
                     int64_t m_valid, int k, int n, int num_rel, int dtype,
                     int precision, int flags, void *workspace,
                     size_t workspace_bytes, void *stream);

/*
 * cxg_spmm_csr without a caller-provided workspace. No counterpart in the reference
 * (its kernels need no scratch memory); added for callers that cannot allocate
 * device memory at call time or cannot pass a scratch buffer across their binding:
 * plugins inside a host program whose memory pool owns the device, serving loops
 * that must avoid the device-wide synchronisation of cudaMalloc / cudaFree, thin
 * FFI bindings that carry only the operator's tensors.
 *
 * The scratch lives in one fixed array of CXG_SPMM_STATIC_SCRATCH_BYTES inside the
 * library, present on every GPU that loads the library until the process exits.
 *   - A request that needs more scratch than that is refused with CXG_ELIMIT (the
 *     message gives the need); nothing is launched. As a guide, 32 MiB covers the
 *     169,343-node / 2.33M-edge graph at 128 fp32 features (about 15 MiB).
 *   - All calls share the array. Its previous contents do not matter, but calls
 *     that overlap on the GPU (other streams, other host threads) corrupt each
 *     other: order them on the device.
 *   - The array used is the one of the CURRENT device (cudaGetDevice at the time of the call); `stream`
 *     must belong to that device. The first call on each device looks the array's device address up
 *     (cudaGetSymbolAddress).
 *   - It never calls cudaMalloc, cudaFree or any other allocating routine.
 * Results are those of cxg_spmm_csr, bit for bit. cxg_spmm_csr_static_status is cxg_spmm_csr_status for
 * the built-in array of the current device (the caller never sees its address).
 */
#define CXG_SPMM_STATIC_SCRATCH_BYTES (32u << 20)
int cxg_spmm_csr_static(const cxg_spmm_desc *desc, void *stream);
int cxg_spmm_csr_static_status(void *stream);

#ifdef __cplusplus
}
#endif
#endif /* CXGNN_B200_H_ */
