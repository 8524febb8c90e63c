/*
 * tango_b200 -- C ABI of the B200 (sm_100a) library behind Tango's quantized
 * GNN-training operators.
 *
 * Every entry point is `extern "C"`, takes plain device pointers and sizes,
 * launches on the CUDA stream it is given (a cudaStream_t passed as void*),
 * never allocates or frees device memory, never synchronises the device and
 * never exits the process: it returns TANGO_OK (0) or a negative error code
 * (see tango_strerror).  All pointers are device pointers unless a comment says
 * "host".  The device that owns the pointers must be current in the calling
 * thread.  No global mutable state is kept, so the library may be entered from
 * several host threads (PyTorch's autograd thread runs the backward calls).
 * The exceptions are named where they are declared: tango_qgemm_dw_noalloc
 * (scratch inside the library) and the tango_peer_* set-up helpers of the
 * multi-GPU section (they create and map shared buffers, once, on the host).
 *
 * Each declaration cites the reference interface it replaces as file:line
 * inside the Tango repository (cuda/src/cuda.cpp holds its pybind table).
 *
 * Layout conventions
 *   - matrices are row-major with an explicit leading dimension (elements);
 *   - int8 feature/operand matrices use a leading dimension that is a multiple
 *     of 16 bytes on the fast paths; columns in [cols, ld) must be zero (the
 *     quantizers here write them as zero);
 *   - sparse structure is CSR with int32 `indptr`/`indices`; an optional
 *     `edge_ids` array maps a CSR slot to the id of the edge stored there;
 *   - scales are 1-element fp32 tensors in device memory, as in the reference.
 */
#ifndef TANGO_B200_H_
#define TANGO_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TANGO_OK 0
#define TANGO_EINVAL (-1)   /* bad argument (null pointer, negative size, bad mode) */
#define TANGO_EALIGN (-2)   /* pointer or leading dimension not aligned as required */
#define TANGO_ECUDA (-3)    /* a CUDA runtime/driver call failed (see tango_last_cuda_error) */
#define TANGO_ETIMEOUT (-4) /* a bounded device-side wait expired (reported via status word) */
#define TANGO_ESIZE (-5)    /* size beyond what the entry point supports */

#define TANGO_ROUND_TRUNC 0      /* (int8)(x/s): the reference's fused forward GEMM, cuda/src/iterator.h:155-164 */
#define TANGO_ROUND_NEAREST 1    /* rint + clamp: the reference's quantize kernel, cuda/src/quantization.cu:6-35 */
#define TANGO_ROUND_STOCHASTIC 2 /* floor(x/s + u), u from Philox4x32-10 keyed by (seed, call) -- not in the reference */

#define TANGO_OP_ADD 0
#define TANGO_OP_SUB 1
#define TANGO_OP_MUL 2
#define TANGO_OP_DIV 3

typedef void *tango_stream_t; /* cudaStream_t */

/* Library version (major*10000 + minor*100 + patch). */
int tango_version(void);
/* Static string for an error code. */
const char *tango_strerror(int code);
/* cudaError_t of the last failing CUDA call made by this thread inside the library (0 if none). */
int tango_last_cuda_error(void);

/* ---------------------------------------------------------------- quantisation */

/* scale[0] = max|x| / 127 over a [rows, cols] fp32 matrix with leading dimension ld.
 * If row_scale != NULL the maximum is taken over x[r,c] * row_scale[r].
 * Replaces get_scale (cuda/src/cuda.cpp:186, cuda/src/quantization.cu:45-93). */
int tango_absmax_scale(const float *x, int64_t rows, int64_t cols, int64_t ld, const float *row_scale,
                       float *scale, tango_stream_t stream);

/* q[r,c] = round_mode(x[r,c] * (1/scale[0])) clamped to [-127,127]; columns [cols, ldq) of q are set to 0.
 * row_scale (optional) multiplies x[r,:] first.  `seed`/`call` key the stochastic stream; the random
 * number of element (r,c) depends only on (seed, call, r*cols + c).  `step` (optional, here and in the two entry
 * points below that take it) points to a device word whose value, shifted left by 32, is added to `call` when the
 * kernel runs: scalar arguments are frozen when a launch is captured in a CUDA graph, a device word is not, so a
 * training loop that replays a graph bumps that word once per step to draw fresh random numbers.
 * Replaces quantize (cuda/src/cuda.cpp:185, cuda/src/quantization.cu:17-43). */
int tango_quantize(const float *x, int64_t rows, int64_t cols, int64_t ldx, const float *row_scale,
                   const float *scale, int8_t *q, int64_t ldq, int mode, uint64_t seed, uint64_t call,
                   const uint64_t *step, tango_stream_t stream);

/* out[c, r] = nearest(x[r, c] / scale[0]) for x fp32 [nrow, ncol] contiguous -> int8 [ncol, nrow] contiguous.
 * Replaces transpose_quant (cuda/src/cuda.cpp:187, cuda/src/quantization.cu:95-167). */
int tango_quantize_transpose(const float *x, int64_t nrow, int64_t ncol, const float *scale, int8_t *out,
                             tango_stream_t stream);

/* Backward of y = relu(.): the masked gradient m[r,c] = (y[r,c] > 0 ? g[r,c] : 0) is consumed without being written.
 * tango_relu_grad_stats: scale[0] = max |m[r,c] * row_scale[r]| / 127 and, if colsum != NULL, colsum[c] = sum_r m[r,c]
 * (the bias gradient), added in a fixed order through `scratch` (tango_relu_grad_stats_scratch_bytes).
 * tango_quantize_relu_grad: q = round_mode(m * row_scale[r] / scale[0]), q rows padded to ldq (multiple of 16).
 * They replace the torch ops between the aggregation's backward and its quantizer in the reference's layer
 * (ReLU backward, `grad_output.sum(0)`, `* norm`, get_scale, quantize: evaluation/test_gcn.py:123-137,
 * cuda/SPMM.py:18-24) with two passes over g and y. */
int64_t tango_relu_grad_stats_scratch_bytes(int64_t rows, int64_t cols);
int tango_relu_grad_stats(const float *g, int64_t ldg, const float *y, int64_t ldy, int64_t rows, int64_t cols,
                          const float *row_scale, float *scale, float *colsum, void *scratch, int64_t scratch_bytes,
                          tango_stream_t stream);
int tango_quantize_relu_grad(const float *g, int64_t ldg, const float *y, int64_t ldy, int64_t rows, int64_t cols,
                             const float *row_scale, const float *scale, int8_t *q, int64_t ldq, int mode,
                             uint64_t seed, uint64_t call, const uint64_t *step, tango_stream_t stream);

/* ---------------------------------------------------------------- int8 GEMMs (tcgen05 kind::i8) */

/* Bytes of scratch tango_qgemm_dw needs for an [n, k] weight gradient. */
int64_t tango_qgemm_dw_workspace_bytes(int64_t n, int64_t k);

/* Y[M,N] = float(Xq[M,K] . Wq[N,K]^T) * (sx[0]*sw[0]) (+ bias[N]); if scale_y != NULL it must hold 0 on entry and
 * receives max|Y|/127.  `status` is a 1-int device word that receives TANGO_ETIMEOUT if a bounded wait expires.
 * Replaces the GEMM + epilogue of QGEMM_forward (cuda/src/cuda.cpp:11-16,183, cuda/src/QGEMM_forward.cu:125-157). */
int tango_qgemm_nt(const int8_t *xq, int64_t ldx, const int8_t *wq, int64_t ldw, int64_t m, int64_t n, int64_t k,
                   const float *sx, const float *sw, const float *bias, float *y, int64_t ldy, float *scale_y,
                   int *status, tango_stream_t stream);

/* The reference's fused forward: quantises X[M,K] (times row_scale[r] if given) and W[N,K] with the given rounding
 * mode and the scales sx, sw, writes the int8 copies xq, wq that the backward pass re-uses, and computes the GEMM
 * above.  Stochastic mode draws X with `call`, W with `call`+1.  (The reference quantizes on load inside the GEMM,
 * cuda/src/iterator.h:155-164; here the quantizer is a separate streaming kernel in front of the TMA-fed GEMM -- a
 * quantize-on-load producer for the tcgen05 kernel was built, was bit-exact and measured 3x slower.)
 * Replaces QGEMM_forward (cuda/src/cuda.cpp:183, cuda/kernels.py:79-94). */
int tango_qgemm_forward(const float *x, int64_t ldx_f, const float *row_scale, const float *w, int64_t ldw_f,
                        int64_t m, int64_t n, int64_t k, const float *sx, const float *sw, int8_t *xq, int64_t ldxq,
                        int8_t *wq, int64_t ldwq, const float *bias, float *y, int64_t ldy, float *scale_y, int mode,
                        uint64_t seed, uint64_t call, const uint64_t *step, int *status, tango_stream_t stream);

/* dX[M,K] = float(dYq[M,N] . Wq[N,K]) * (sdy[0]*sw[0]), then row r times row_scale[r] if row_scale != NULL (the
 * backward of a left normalisation folded into the epilogue).
 * Replaces QGEMM_backward_gradX (cuda/src/cuda.cpp:191, cuda/src/QGEMM_backward.cu:21-48). */
int tango_qgemm_dx(const int8_t *dyq, int64_t lddy, const int8_t *wq, int64_t ldw, int64_t m, int64_t n, int64_t k,
                   const float *sdy, const float *sw, const float *row_scale, float *dx, int64_t lddx, int *status,
                   tango_stream_t stream);

/* dW[N,K] = float(dYq^T[N,M] . Xq[M,K]) * (sdy[0]*sx[0]); split over M with int32 atomics into `workspace`
 * (tango_qgemm_dw_workspace_bytes; contents on entry are irrelevant), then dequantised.
 * Replaces QGEMM_backward_gradW (cuda/src/cuda.cpp:192, cuda/src/QGEMM_backward.cu:50-113). */
int tango_qgemm_dw(const int8_t *dyq, int64_t lddy, const int8_t *xq, int64_t ldx, int64_t m, int64_t n, int64_t k,
                   const float *sdy, const float *sx, float *dw, int64_t lddw, void *workspace,
                   int64_t workspace_bytes, int *status, tango_stream_t stream);

/* Weight gradient for callers that have no device memory to lend and must not allocate any: same result as
 * tango_qgemm_dw, but the split-K scratch is a fixed 4 MiB array that lives inside the library image, so no
 * workspace argument exists and no cudaMalloc / cudaFree (nor any allocating library routine) is called.  This has
 * no counterpart in the reference.  It is meant for hosts where allocation is off the table at call time: a
 * runtime that has handed all device memory to its own pool and gives plug-ins no allocator handle, or a
 * latency-sensitive loop that cannot tolerate the implicit device-wide synchronisation of cudaMalloc/cudaFree.
 * Limits and rules:
 *   - n * round_up(k, 4) must not exceed tango_qgemm_dw_noalloc_max_elems() (1,048,576 int32); larger problems
 *     return TANGO_ESIZE and must use tango_qgemm_dw with caller memory;
 *   - every GPU that loads the library holds the 4 MiB until the process exits;
 *   - the first call on a device looks up the array's device address (cudaGetSymbolAddress, once per device, under a
 *     mutex); make that first call before starting any stream capture;
 *   - all calls on a device share the one array: it still holds the previous call's partial sums, each call clears
 *     the part it uses first, and two calls that overlap on the GPU (different streams) race -- serialise them. */
int tango_qgemm_dw_noalloc(const int8_t *dyq, int64_t lddy, const int8_t *xq, int64_t ldx, int64_t m, int64_t n,
                           int64_t k, const float *sdy, const float *sx, float *dw, int64_t lddw, int *status,
                           tango_stream_t stream);
/* Capacity of the built-in scratch of tango_qgemm_dw_noalloc in int32 elements. */
int64_t tango_qgemm_dw_noalloc_max_elems(void);

/* ---------------------------------------------------------------- SpMM (CSR, int8 features, int32 accumulation) */

/* Optional schedule for rows too long for one warp.  A row whose degree exceeds `split_threshold` is cut into
 * `n_units` units (vrow, begin, end, slot) stored as int32 quadruples; each unit adds its partial sums into
 * int32 scratch `ws` ([n_heavy * nseg, ws_ld]) and the rows listed in `heavy_rows` ([n_heavy]) are finished by a
 * second kernel.  With n_units == 0 every row is handled by one warp (the units/heavy_rows/ws fields are ignored). */
typedef struct tango_spmm_plan {
    const int32_t *units;      /* [n_units, 4] */
    int64_t n_units;
    const int32_t *heavy_rows; /* [n_heavy] */
    int64_t n_heavy;
    int32_t *ws;               /* [n_heavy * nseg, ws_ld] int32 scratch, 16-byte aligned */
    int64_t ws_ld;             /* >= round_up(F, 16), a multiple of 4 */
    int32_t split_threshold;
    const int32_t *row_order;  /* optional [n_rows]: warp w works on row row_order[w] (e.g. rows sorted by degree, so
                                  that the warps of a CTA finish together); NULL = natural order */
    int64_t n_long_rows;       /* with row_order: rows row_order[0, n_long_rows) get one warp each, the shorter rows
                                  after them are handled by groups of lanes (several rows per warp); -1 = all long */
    /* Optional dense hub region (tango_spmm_copy_u only; all zero / NULL = none).  With rows ranked by length and
     * columns by how often they are referenced, the adjacency of a power-law graph is dense in its top-left corner:
     * that staircase-shaped region is multiplied as dense 0/1 int8 tiles on the tensor cores instead of being
     * gathered edge by edge.  Row tile i (128 rows: heavy rows 128 i .. 128 i + 127, i.e. the first dense_rows entries
     * of heavy_rows in order) owns a run of stored 128 x 128 tiles; dense_units lists work items (row tile, index of
     * the first stored tile, first column tile, number of tiles); column tile k covers the feature rows
     * dense_cols[128 k .. 128 k + 127].  Every work item adds partial[r, :] = sum_c tile[r, c] * Nq[dense_cols[c], :]
     * (exact int32) into the scratch row of its heavy rows.  The CSR handed to the entry point must then hold only
     * the edges OUTSIDE the region, every region row must be listed in heavy_rows (its remaining edges are covered by
     * units, possibly none) and row_order must list the heavy rows first: its first n_skip_rows entries are left to
     * units + finalize. */
    const int8_t *dense_a;       /* [dense_n_tiles * 128, 128] int8: the stored tiles, row-major, entries = multiplicity */
    int64_t dense_n_tiles;
    const int32_t *dense_units;  /* [dense_n_units, 4] int32, 16-byte aligned */
    int64_t dense_n_units;
    int64_t dense_rows;          /* multiple of 128, <= n_heavy */
    const int32_t *dense_cols;   /* [dense_n_cols] feature-row id of every column of the region */
    int64_t dense_n_cols;        /* multiple of 128 */
    int8_t *dense_b;             /* scratch [dense_n_cols, round_up(f, 16)] int8: the region's feature rows, packed */
    int *dense_status;           /* optional device word that receives TANGO_ETIMEOUT if a bounded wait of the GEMM expires */
    int64_t n_skip_rows;         /* leading entries of row_order owned by units + finalize (0 without a dense region) */
} tango_spmm_plan;

/* out[v,:] = sum_k scales[k] * float(sum_{j in segment k of row v} Nq[indices[j], :]) for v < n_rows.
 * `indptr` has n_rows*nseg + 1 entries: row v owns the nseg consecutive segments v*nseg .. v*nseg+nseg-1, segment k
 * holding the neighbours that live on shard k (nseg = 1 and one scale on a single GPU).  Optional fused epilogue:
 * out = act((acc) * row_scale[v] + bias[:]) with relu != 0 selecting max(.,0); out_absmax (optional, must hold 0)
 * receives max|out|/127.  Replaces csr_SPMM (cuda/src/cuda.cpp:194, cuda/src/SPMM.cu:23-68). */
int tango_spmm_copy_u(const int32_t *indptr, const int32_t *indices, int64_t n_rows, int nseg, const int8_t *nq,
                      int64_t ldn, int64_t f, const float *scales, const float *row_scale, const float *bias,
                      int relu, float *out, int64_t ldo, float *out_absmax, const tango_spmm_plan *plan /* host */,
                      tango_stream_t stream);

/* out[v,h,:] = scale[0] * float(sum_j Eq[eid(j), h] * Nq[indices[j], h, :]); Nq is [*, H*D] with leading dimension
 * ldn, Eq is int8 [E, H] contiguous in edge-id order, eid(j) = edge_ids ? edge_ids[j] : j.
 * Replaces multi_cusparse_SPMM (cuda/src/cuda.cpp:138-160,196, cuda/src/SPMM.cu:70-130, cuda/kernels.py:122-136). */
int tango_spmm_u_mul_e(const int32_t *indptr, const int32_t *indices, const int32_t *edge_ids, int64_t n_rows,
                       const int8_t *nq, int64_t ldn, int h, int d, const int8_t *eq, const float *scale, float *out,
                       int64_t ldo, const tango_spmm_plan *plan /* host */, tango_stream_t stream);

/* out[v,:] = scale[0] * float(sum_{j in row v} Zq[eid(j), :]) -- sum of the int8 edge features incident to a node.
 * Replaces incidence_SPMM (cuda/src/cuda.cpp:198, cuda/src/SPMM.cu:259-303). */
int tango_spmm_incidence(const int32_t *indptr, const int32_t *edge_ids, int64_t n_rows, const int8_t *zq, int64_t ldz,
                         int64_t f, const float *scale, float *out, int64_t ldo, const tango_spmm_plan *plan /* host */,
                         tango_stream_t stream);

/* ---------------------------------------------------------------- SDDMM */

/* out[e,h] = float(sum_d Uq[src[e],h,d] * Vq[dst[e],h,d]) * (su[0]*sv[0]); out is [E, H] contiguous.
 * out_absmax (optional, must hold 0) receives max|out|/127.
 * Replaces mySDDMM_int8 with op "dot" (cuda/src/cuda.cpp:201, cuda/src/SDDMM.cu:8-47,124-153). */
int tango_sddmm_dot(const int32_t *src, const int32_t *dst, int64_t n_edges, const int8_t *uq, int64_t ldu,
                    const int8_t *vq, int64_t ldv, int h, int d, const float *su, const float *sv, float *out,
                    float *out_absmax, tango_stream_t stream);

/* The same product, walked row by row of a CSR/CSC instead of edge by edge: for every slot j of row r
 *   out[eid(j), h] = float(sum_d Uq[indices[j],h,d] * Vq[r,h,d]) * (su[0]*sv[0])
 * (edge_ids == NULL: slot j is edge j).  With the CSC (rows = destinations, indices = sources) this is exactly
 * tango_sddmm_dot; V's row stays in registers and only U is gathered, so half as many bytes move, and rows longer
 * than plan->split_threshold are cut into the plan's slices (no scratch needed; plan may be NULL).  Needs rows of
 * both operands padded to 16 (or 4) bytes with zero pad, h*d <= 512, and for h > 1 a head width d that is a
 * power-of-two multiple of 16 (or 4) bytes; otherwise returns TANGO_EALIGN and the caller uses tango_sddmm_dot.
 * Replaces mySDDMM_int8 with op "dot" (cuda/src/cuda.cpp:201, cuda/src/SDDMM.cu:8-47,124-153). */
int tango_sddmm_dot_rows(const int32_t *indptr, const int32_t *indices, const int32_t *edge_ids, int64_t n_rows,
                         const int8_t *uq, int64_t ldu, const int8_t *vq, int64_t ldv, int h, int d, const float *su,
                         const float *sv, float *out, float *out_absmax, const tango_spmm_plan *plan /* host */,
                         tango_stream_t stream);

/* out[e,:] = op(float(Uq[src[e],:])*su[0], float(Vq[dst[e],:])*sv[0]) over `dim` features; out is [E, dim] contiguous.
 * Replaces mySDDMM_int8 with op add/sub/mul/div (cuda/src/cuda.cpp:201, cuda/src/SDDMM.cu:49-100,154-176). */
int tango_sddmm_elementwise(int op, const int32_t *src, const int32_t *dst, int64_t n_edges, const int8_t *uq,
                            int64_t ldu, const int8_t *vq, int64_t ldv, int64_t dim, const float *su, const float *sv,
                            float *out, float *out_absmax, tango_stream_t stream);

/* ---------------------------------------------------------------- fused GAT edge pipeline */

/* For every destination row v of a CSC (indptr, indices = source ids, edge_ids):
 *   z[j] = leaky_relu(float(elq[indices[j],h])*sl[0] + float(erq[v,h])*sr[0], slope)
 *   a[eid(j),h] = exp(z[j]-max_v)/sum_v
 * i.e. the reference's sddmm_u_add_v -> LeakyReLU -> dgl edge_softmax chain (evaluation/test_gat.py:141-146,
 * cuda/SDDMM.py:10-20) in one pass; `a` is fp32 [E, H] in edge-id order; elq / erq are contiguous int8 [N, H], H <= 8.
 * Optional schedule: with row_order (rows by decreasing degree) the first n_block_rows rows get a whole CTA each, the
 * others a warp; row_order == NULL means one warp per row in natural order.  The optional *_absmax word of the four
 * edge-softmax entry points (must hold 0) receives max|output|/127, i.e. the scale the quantizer of the next operator
 * would otherwise compute with a pass of its own (get_scale, cuda/src/quantization.cu:79-93). */
int tango_gat_edge_softmax(const int32_t *indptr, const int32_t *indices, const int32_t *edge_ids,
                           const int32_t *row_order, int64_t n_block_rows, int64_t n_rows, const int8_t *elq,
                           const int8_t *erq, int h, const float *sl, const float *sr, float slope, float *a,
                           float *a_absmax, tango_stream_t stream);

/* Gradient of the pass above with respect to the edge logits: for every destination row and head
 *   dz[eid(j),h] = a_j * (da_j - sum_k a_k da_k) * (z_j > 0 ? 1 : slope)
 * (softmax backward, then LeakyReLU backward with z recomputed from the int8 operands).  `a`, `da`, `dz` are fp32
 * [E, H] in edge-id order; elq / erq are contiguous int8 [N, H].  Replaces the autograd backward of
 * dgl.ops.edge_softmax and nn.LeakyReLU in the reference's GAT layer (evaluation/test_gat.py:144-146). */
int tango_gat_edge_softmax_bwd(const int32_t *indptr, const int32_t *indices, const int32_t *edge_ids,
                               const int32_t *row_order, int64_t n_block_rows, int64_t n_rows, const int8_t *elq,
                               const int8_t *erq, int h, const float *sl, const float *sr, float slope, const float *a,
                               const float *da, float *dz, float *dz_absmax, tango_stream_t stream);

/* The same attention weights without an fp32 copy of them, in two steps.  The reference materialises the logits, the
 * weights and their transposed int8 copy as E x H tensors (evaluation/test_gat.py:141-152, cuda/SPMM.py:38-47); here
 * step 1 keeps only the softmax statistics of every destination row, row_m[v,h] = max_j z_j and
 * row_inv[v,h] = 1 / sum_j exp(z_j - max) (fp32 [N, H]; rows without edges are left untouched), and a_absmax
 * (optional, must hold 0) receives max|a| / 127 -- the largest weight of a row is exp(0) * row_inv, so the int8 scale
 * of `a` is known before any weight is formed.  Step 2 writes aq[eid(j),h] = round_mode(exp(z_j - row_m) * row_inv /
 * a_scale[0]) clamped to [-127,127], int8 [E, H] in edge-id order: exactly what quantising the fp32 weights of
 * tango_gat_edge_softmax with that scale gives, rounding stream included (element index eid * H + h).  The
 * gradient pass recomputes the weights from the statistics instead of reading them. */
int tango_gat_edge_softmax_stats(const int32_t *indptr, const int32_t *indices, const int32_t *row_order,
                                 int64_t n_block_rows, int64_t n_rows, const int8_t *elq, const int8_t *erq, int h,
                                 const float *sl, const float *sr, float slope, float *row_m, float *row_inv,
                                 float *a_absmax, tango_stream_t stream);
int tango_gat_edge_softmax_quantized(const int32_t *indptr, const int32_t *indices, const int32_t *edge_ids,
                                     const int32_t *row_order, int64_t n_block_rows, int64_t n_rows, const int8_t *elq,
                                     const int8_t *erq, int h, const float *sl, const float *sr, float slope,
                                     const float *row_m, const float *row_inv, const float *a_scale, int8_t *aq,
                                     int mode, uint64_t seed, uint64_t call, const uint64_t *step,
                                     tango_stream_t stream);
int tango_gat_edge_softmax_bwd_stats(const int32_t *indptr, const int32_t *indices, const int32_t *edge_ids,
                                     const int32_t *row_order, int64_t n_block_rows, int64_t n_rows, const int8_t *elq,
                                     const int8_t *erq, int h, const float *sl, const float *sr, float slope,
                                     const float *row_m, const float *row_inv, const float *da, float *dz,
                                     float *dz_absmax, tango_stream_t stream);

/* Edge softmax of plain fp32 scores: for every destination row v (CSC order) and head h
 *   a[eid(j),h] = softmax_j( z[eid(j),h] * zmul )     over the incoming edges j of v,
 * z and a fp32 [E, H] in edge-id order (edge_ids == NULL: slot j is edge j), h <= 8; zmul folds a constant factor
 * such as HGT's 1/sqrt(d_k) into the pass.  Same row schedule arguments as tango_gat_edge_softmax.  Replaces
 * dgl.ops.edge_softmax(g, t, norm_by='dst') (evaluation/test_HGT.py:59-60, evaluation/test_gat.py:146). */
int tango_edge_softmax(const int32_t *indptr, const int32_t *edge_ids, const int32_t *row_order,
                       int64_t n_block_rows, int64_t n_rows, const float *z, int h, float zmul, float *a,
                       float *a_absmax, tango_stream_t stream);

/* Gradient of tango_edge_softmax with respect to z: dz[eid(j),h] = a_j * (da_j - sum_k a_k da_k) * zmul.
 * Replaces the autograd backward of dgl.ops.edge_softmax. */
int tango_edge_softmax_bwd(const int32_t *indptr, const int32_t *edge_ids, const int32_t *row_order,
                           int64_t n_block_rows, int64_t n_rows, int h, float zmul, const float *a, const float *da,
                           float *dz, float *dz_absmax, tango_stream_t stream);

/* ---------------------------------------------------------------- multi-GPU exchange over peer memory */

/* None of the entry points of this section has a counterpart in the reference, which is single-GPU.  They serve the
 * row-partitioned aggregation (every GPU needs the int8 rows of all GPUs): instead of quantizing locally and then
 * all-gathering, the quantizer stores every 16-byte piece of row r straight into the gathered table of every GPU of
 * the node, at tables[k] + (row0 + r) * ldq (tables: DEVICE array of n_tables base pointers, peer memory mapped into
 * this process, e.g. through CUDA IPC; row0 = first row of this rank's shard in the gathered table; ldq a multiple
 * of 16).  Plain stores over NVLink, no multicast, no loads from peer memory.  Arguments otherwise as for
 * tango_quantize / tango_quantize_relu_grad.  A tango_peer_sync on the same stream must follow before any GPU reads
 * its table. */
int tango_quantize_push(const float *x, int64_t rows, int64_t cols, int64_t ldx, const float *row_scale,
                        const float *scale, int8_t *const *tables /* device */, int n_tables, int64_t row0,
                        int64_t ldq, int mode, uint64_t seed, uint64_t call, const uint64_t *step,
                        tango_stream_t stream);
int tango_quantize_relu_grad_push(const float *g, int64_t ldg, const float *y, int64_t ldy, int64_t rows, int64_t cols,
                                  const float *row_scale, const float *scale, int8_t *const *tables /* device */,
                                  int n_tables, int64_t row0, int64_t ldq, int mode, uint64_t seed, uint64_t call,
                                  const uint64_t *step, tango_stream_t stream);

/* Set-up helpers for buffers that the other processes of the node map (host side, once per buffer; the operator
 * entry points themselves still never allocate).  tango_peer_alloc: cudaMalloc + zero fill on the current device and
 * the 64-byte CUDA IPC handle of the allocation; tango_peer_open: maps another process's buffer for kernels of the
 * CURRENT device (peer access is enabled on demand) and returns its address in this process; tango_peer_close /
 * tango_peer_free undo them. */
int tango_peer_alloc(int64_t bytes, void **ptr, unsigned char *handle64);
int tango_peer_open(const unsigned char *handle64, void **ptr);
int tango_peer_close(void *ptr);
int tango_peer_free(void *ptr);

/* Lets kernels of the current device store to and load from memory of `peer_device` (cudaDeviceEnablePeerAccess;
 * already enabled counts as success).  TANGO_EINVAL if the two devices cannot reach each other. */
int tango_enable_peer_access(int peer_device);

/* Barrier + all-reduce(max) of one non-negative float among the `world` GPUs of a node, in one single-CTA launch.
 * slots: DEVICE array of `world` pointers, slots[k] = rank k's array of 2 * world 64-bit words (zero-initialised once,
 * mapped by every rank); round_word: this rank's device word counting the rounds (zero-initialised; all ranks must
 * call the same number of times); val_in / val_out may be NULL (pure barrier).  On return from the kernel everything
 * that the other ranks wrote to this GPU's memory before their call is visible to later kernels of this stream.
 * The wait is bounded: limit_ns nanoseconds (<= 0 selects the default of 2 s).  On expiry *status = TANGO_ETIMEOUT,
 * val_out receives the maximum over the ranks that did arrive, and the kernel returns; the round still counts, so a
 * rank that was merely late meets the others again at the next call.  The limit is also the largest skew between
 * ranks that a training loop may have at a rendezvous (a rank that spends longer than this between two steps, e.g.
 * in an evaluation pass that only it runs, makes the others time out). */
int tango_peer_sync(uint64_t *const *slots /* device */, int rank, int world, uint64_t *round_word, const float *val_in,
                    float *val_out, int *status, int64_t limit_ns, tango_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* TANGO_B200_H_ */
