/*
 * pbg_b200.h -- C ABI of the B200 (sm_100a) training-step library for PyTorch-BigGraph.
 *
 * The library takes the slot of the reference's native module `torchbiggraph._C`
 * (torchbiggraph/util.cpp:425-460, loaded in torchbiggraph/train_gpu.py:41-46) and runs, on
 * the device, what the reference runs as PyTorch ops inside
 * `Trainer._process_one_batch` (torchbiggraph/train_cpu.py:86-112) for every batch that
 * `process_in_batches` (torchbiggraph/batching.py:91-125) hands it.
 *
 * Conventions
 *   - plain C types only; every buffer is a raw pointer owned by the caller and alive for the
 *     duration of the call.  "dev" pointers are device memory on the context's GPU, "host"
 *     pointers are host memory (pinned memory makes the copies asynchronous).
 *   - every function returns a pbg_status; 0 is success.  pbg_last_error(ctx) gives the text.
 *     Nothing aborts, nothing spins without a bound.
 *   - one context per GPU and per host thread; calls on one context are serialised on the
 *     stream given at creation (0 = the legacy default stream).
 *   - embedding tables are dense row-major float32 [num_rows, dim]; RowAdagrad state is one
 *     float32 per row (torchbiggraph/row_adagrad.py:34-40).  The lhs and rhs table may be the
 *     same memory (same entity type and partition): pass the same pointers.
 *   - operator parameters are float32 tables [num_rels, dim]; complex_diagonal rows are
 *     [real | imag] (torchbiggraph/operators.py:128-157).  Their AsyncAdagrad accumulators
 *     (torchbiggraph/async_adagrad.py:75-85) have the same shape.
 */
#ifndef PBG_B200_H
#define PBG_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
  PBG_OK = 0,
  PBG_ERR_BAD_ARGUMENT = 1,   /* null pointer, negative size, inconsistent shapes            */
  PBG_ERR_UNSUPPORTED = 2,    /* a plugin / option this library has no device code for        */
  PBG_ERR_INDEX_RANGE = 3,    /* an entity or relation id outside its table (reported by the
                                 kernels through a flag; the offending rows are skipped)      */
  PBG_ERR_TIMEOUT = 4,        /* a bounded device-side wait ran out                           */
  PBG_ERR_CUDA = 5,           /* a CUDA runtime call failed; text in pbg_last_error           */
  PBG_ERR_NO_DEVICE = 6,      /* no CUDA device / wrong architecture                          */
  PBG_ERR_TOO_LARGE = 7       /* a size beyond a stated maximum                               */
} pbg_status;

/* OPERATORS registry names (torchbiggraph/operators.py:46-157) */
typedef enum { PBG_OP_NONE = 0, PBG_OP_DIAGONAL = 1, PBG_OP_TRANSLATION = 2,
               PBG_OP_COMPLEX_DIAGONAL = 3, PBG_OP_LINEAR = 4, PBG_OP_AFFINE = 5 } pbg_operator;
/* COMPARATORS registry names (torchbiggraph/model.py:156-303) */
typedef enum { PBG_CMP_DOT = 0, PBG_CMP_COS = 1, PBG_CMP_L2 = 2, PBG_CMP_SQUARED_L2 = 3 } pbg_comparator;
/* LOSS_FUNCTIONS registry names (torchbiggraph/losses.py:50-161) */
typedef enum { PBG_LOSS_LOGISTIC = 0, PBG_LOSS_RANKING = 1, PBG_LOSS_SOFTMAX = 2 } pbg_loss;
/* arithmetic of the score / gradient contractions */
typedef enum {
  PBG_PREC_FP32 = 0,     /* fp32 FMA on the CUDA cores; the rtol 1e-4 tier                    */
  PBG_PREC_TF32X3 = 1,   /* tcgen05 TF32 tensor cores, 3-term error-compensated split, fp32
                            accumulation in tensor memory; the rtol 1e-4 tier                 */
  PBG_PREC_TF32 = 2,     /* tcgen05 TF32 tensor cores, single pass; the rtol 1e-3 tier        */
  PBG_PREC_BF16X6 = 3,   /* tcgen05 bf16 tensor cores on three bf16 planes per fp32 operand
                            (x = b0 + b1 + b2, 24 mantissa bits), the six plane products of
                            order <= 2, fp32 accumulation in tensor memory; the rtol 1e-4 tier.
                            Not for the linear / affine operators: pbg_create refuses those.
                            Pays where the contractions dominate (large chunks, dim >= 400):
                            the planes are 6 bytes per operand value where fp32 is 4          */
  PBG_PREC_BF16X3 = 4    /* the same on TWO planes per operand (x ~ b0 + b1, 16 mantissa bits) and the
                            three plane products b0.b0 + b0.b1 + b1.b0: half the tensor-core work
                            and 4 bytes per operand value.  Every product carries a relative
                            error of about 2^-17 (the dropped terms), some 30 times that of fp32
                            rounding; sums of such products stay inside rtol 1e-4 unless they
                            cancel heavily.  Not for linear / affine.                            */
} pbg_precision;

/* The keys of ConfigSchema (torchbiggraph/config.py:158-230, 318-359, 411-425) that the
 * training step reads. */
typedef struct {
  int32_t dim;                /* dimension                                                     */
  int32_t op;                 /* pbg_operator of the relation(s)                               */
  int32_t comparator;         /* pbg_comparator                                                */
  int32_t loss;               /* pbg_loss                                                      */
  int32_t dynamic_relations;  /* 0: one relation per batch, operator on the rhs only
                                 (model.py:666-703); 1: per-edge relation, two operator
                                 tables, two one-sided passes (model.py:705-758)               */
  int32_t num_rels;           /* rows of the operator tables                                   */
  int32_t num_batch_negs;
  int32_t num_uniform_negs;
  int32_t disable_lhs_negs;
  int32_t disable_rhs_negs;
  int32_t precision;          /* pbg_precision                                                 */
  int32_t max_batch_size;     /* largest number of edges in one batch (batch_size)             */
  int32_t batches_in_flight;  /* k >= 1: batches of one wave read the tables as they were when
                                 the wave started and their k optimizer steps are applied in
                                 batch order (deterministic HOGWILD, train_cpu.py:861-884);
                                 1 = the reference's sequential semantics                      */
  float margin;               /* ranking loss margin                                           */
  float lr;                   /* RowAdagrad learning rate                                      */
  float relation_lr;          /* AsyncAdagrad learning rate of operator parameters
                                 (train_cpu.py:224-228: relation_lr if set, else lr)           */
  float regularization_coef;  /* N3 regularizer weight (torchbiggraph/regularizers.py:51-97),
                                 0 = off; not with linear / affine operators                   */
  float max_norm;             /* > 0: a looked-up row longer than this enters the step scaled by
                                 max_norm / (norm + 1e-7), and the table keeps the scaled row
                                 (F.embedding(max_norm=...), torchbiggraph/model.py:57-61);
                                 0 = off                                                        */
} pbg_config;

/* One resident (lhs partition, rhs partition) bucket.  Pointers are device memory. */
typedef struct {
  float *lhs_emb;   float *lhs_state;  int64_t lhs_rows;   /* [lhs_rows, dim], [lhs_rows]      */
  float *rhs_emb;   float *rhs_state;  int64_t rhs_rows;   /* may equal the lhs_* pointers     */
  float *rhs_op;    float *rhs_op_state;                   /* [num_rels, dim] or NULL (op none)*/
  float *lhs_op;    float *lhs_op_state;                   /* dynamic relations only, else NULL*/
  const float *relation_weights;                           /* HOST array [num_rels] (standard
                                                              mode) or [1] (dynamic); NULL = 1 */
  /* config.global_emb (torchbiggraph/model.py:433-441, 486-492): one trained vector per entity
   * type, added to every row of that type before the operator; standard relations only.
   * [dim] vector and its AsyncAdagrad accumulator per side, NULL = none.  The rhs pointers equal
   * the lhs pointers when both sides are of one entity type (one vector, the gradients of both
   * sides add up). */
  float *lhs_global;  float *lhs_global_state;
  float *rhs_global;  float *rhs_global_state;
} pbg_bucket;

/* One batch of a call: edges [offset, offset + count) of the edge arrays, all of relation
 * `rel` in standard mode (batching.py:21-79); `rel` is ignored with dynamic relations. */
typedef struct { int64_t offset; int32_t count; int32_t rel; } pbg_batch;

/* Stats of one batch (torchbiggraph/train_cpu.py:95-101). */
typedef struct { float loss; float reg; int64_t violators_lhs; int64_t violators_rhs; int64_t count; } pbg_batch_stats;

typedef struct pbg_context pbg_context;

/* Library / build information; usable without a GPU. */
const char *pbg_version(void);
const char *pbg_status_string(int status);

/* Creates the per-GPU context (workspace sized from cfg; stream = a cudaStream_t cast to
 * void*, NULL for the default stream).  Replaces the per-process set-up of
 * GPUProcess.__init__ / run (torchbiggraph/train_gpu.py:101-135). */
int pbg_create(const pbg_config *cfg, int device, void *stream, pbg_context **out);
int pbg_destroy(pbg_context *ctx);
const char *pbg_last_error(const pbg_context *ctx);
/* Workspace bytes the context holds on the device. */
int64_t pbg_workspace_bytes(const pbg_context *ctx);
/* lr / relation_lr / margin may change between calls (checkpoint reload, schedules). */
int pbg_set_hyperparameters(pbg_context *ctx, float lr, float relation_lr, float margin);

/* Trains `num_batches` batches on the bucket: the device-side replacement of the loop
 * `for batch_edges in batcher(...): trainer.process_one_batch(model, batch_edges)`
 * (torchbiggraph/batching.py:121-122 -> train_cpu.py:86-112).  The batches are taken in order
 * in ceil(num_batches / batches_in_flight) waves of equal size (sizes differ by at most one, the
 * larger waves first); a call with at most batches_in_flight batches is one wave.
 *   lhs, rhs, rel : device int64 arrays of `num_edges` partition-local row ids / relation ids
 *                   (rel may be NULL in standard mode).
 *   batches       : HOST array of num_batches descriptors.
 *   uniform_lhs / uniform_rhs : device int64 [num_batches, chunks_per_batch, num_uniform_negs]
 *                   row ids of the uniformly sampled negatives, chunks_per_batch =
 *                   ceil(max_batch_size / chunk_size); NULL = draw them on the device from
 *                   `seed` (the reference draws them with torch.randint, model.py:70-75).
 *   stats_out     : HOST array of num_batches entries, filled when the call returns
 *                   (the call synchronises the stream once, at its end), or NULL to skip the
 *                   read-back and stay asynchronous (use pbg_read_stats later).
 */
int pbg_train_batches(pbg_context *ctx, const pbg_bucket *bucket,
                      const int64_t *lhs_dev, const int64_t *rhs_dev, const int64_t *rel_dev,
                      int64_t num_edges, const pbg_batch *batches, int32_t num_batches,
                      const int64_t *uniform_lhs_dev, const int64_t *uniform_rhs_dev,
                      uint64_t seed, pbg_batch_stats *stats_out);

/* Same, with the edge arrays (and optional uniform ids) in HOST memory: copies them to the
 * device asynchronously on the context's stream ahead of the first wave (8 to 24 bytes per
 * edge, against ~50 KB per edge of table traffic).  This is the call that stands where
 * GPUProcess.do_one_job moves a bucket's edges to the GPU and trains on them
 * (torchbiggraph/train_gpu.py:243-266). */
int pbg_train_batches_host(pbg_context *ctx, const pbg_bucket *bucket,
                           const int64_t *lhs_host, const int64_t *rhs_host, const int64_t *rel_host,
                           int64_t num_edges, const pbg_batch *batches, int32_t num_batches,
                           const int64_t *uniform_lhs_host, const int64_t *uniform_rhs_host,
                           uint64_t seed, pbg_batch_stats *stats_out);

/* Per-edge weights (EdgeList.weight of the reference: every loss multiplies the loss of a positive
 * and of its negatives by the edge's weight, torchbiggraph/losses.py:65-78, 104-113, 145-157).
 * weights_dev: DEVICE float array parallel to the edge arrays of the NEXT pbg_train_batches,
 * pbg_train_batches_host or pbg_eval_batch call on this context; that call uses it and clears
 * it.  NULL clears it at once.  Without this call every edge weighs 1. */
int pbg_set_edge_weights(pbg_context *ctx, const float *weights_dev);

/* Sum of the stats of every batch trained since the last call of this function (device
 * accumulators read back once; Stats.sum in torchbiggraph/stats.py:39-47). */
int pbg_read_stats(pbg_context *ctx, pbg_batch_stats *sum_out);

/* Forward pass only: MultiRelationEmbedder.forward (torchbiggraph/model.py:624-762) for one
 * batch.  Outputs are device float32: lhs_pos / rhs_pos [count]; lhs_neg / rhs_neg
 * [count, neg_cols] with neg_cols as returned by pbg_neg_columns (masked entries hold -1e9,
 * model.py:836-839).  A side whose negatives are disabled gets neg_cols == 0. */
int pbg_score_batch(pbg_context *ctx, const pbg_bucket *bucket,
                    const int64_t *lhs_dev, const int64_t *rhs_dev, const int64_t *rel_dev,
                    int32_t count, int32_t rel,
                    const int64_t *uniform_lhs_dev, const int64_t *uniform_rhs_dev, uint64_t seed,
                    float *lhs_pos, float *rhs_pos, float *lhs_neg, float *rhs_neg);
/* Chunk size and negative columns for a batch of `count` edges (model.py:648-656). */
int pbg_neg_columns(const pbg_context *ctx, int32_t count, int32_t *chunk_size, int32_t *chunks,
                    int32_t *lhs_neg_cols, int32_t *rhs_neg_cols);

/* Evaluation of one batch: RankingEvaluator._process_one_batch (torchbiggraph/eval.py:43-81).
 * Forward pass as pbg_score_batch, then per side rank = 1 + #(neg >= pos) of every edge, and the
 * Stats the reference returns, as sums over the batch (the caller averages over count, as
 * Stats.average does): loss (calc_loss, batching.py:139-150), pos_rank, mrr, r1, r10, r50 are the
 * mean over the enabled sides of the per-side sums (average_of_sums, stats.py:19-20); auc is
 * count x the mean of the per-side randomized AUCs (util.py:415-428: `count` random
 * positive / negative pairs per side, drawn on the device from `seed`).  Nothing is updated. */
typedef struct { float loss; double pos_rank, mrr, r1, r10, r50, auc; int64_t count; } pbg_eval_stats;
int pbg_eval_batch(pbg_context *ctx, const pbg_bucket *bucket,
                   const int64_t *lhs_dev, const int64_t *rhs_dev, const int64_t *rel_dev,
                   int32_t count, int32_t rel,
                   const int64_t *uniform_lhs_dev, const int64_t *uniform_rhs_dev, uint64_t seed,
                   pbg_eval_stats *stats_out);

/* The same evaluation for relations with all_negs=True (torchbiggraph/model.py:582-617, 648-650): the negatives
 * of a side are ALL rows of its table, one chunk holds the whole batch, and the score of an edge against its
 * own true entity is ignored.  rank = 1 + #(candidates scoring >= the positive) over lhs_rows - 1 (rhs_rows - 1)
 * candidates; the loss is calc_loss over those score rows; Stats as pbg_eval_batch returns them.  The score rows
 * are never stored: the table is scored in slabs of 8192 rows.  num_batch_negs / num_uniform_negs of the
 * context are not used.  Not for the linear / affine operators. */
int pbg_eval_batch_all_negs(pbg_context *ctx, const pbg_bucket *bucket,
                            const int64_t *lhs_dev, const int64_t *rhs_dev, const int64_t *rel_dev,
                            int32_t count, int32_t rel, uint64_t seed, pbg_eval_stats *stats_out);

/* The sparse-row optimizer step alone: RowAdagrad.step on a sparse gradient
 * (torchbiggraph/row_adagrad.py:80-96).  rows: device int64 [n] (duplicates allowed, they are
 * summed first), grads: device float32 [n, dim]. */
int pbg_row_adagrad(pbg_context *ctx, float *emb, float *state, int64_t num_rows,
                    const int64_t *rows_dev, const float *grads_dev, int32_t n, float lr);

/* The same sparse RowAdagrad step for callers that cannot allocate device memory: a trainer that
 * has given all of HBM to its partitions, a process under an allocator that owns the device, or
 * code that cannot afford the device-wide synchronisation cudaMalloc / cudaFree imply.  It has no
 * counterpart in the reference (there the step is RowAdagrad.step on tensors PyTorch allocates).
 * It takes no context and calls no allocating routine: its scratch (sort buffers, digit
 * counters, error word; about 1 MB) is a fixed array inside the library that every GPU which
 * loads the library holds until the process exits.
 *   - at most 16384 gradient rows per call (n <= 16384), dim a multiple of 4 up to 2048; larger
 *     sizes return PBG_ERR_TOO_LARGE / PBG_ERR_UNSUPPORTED and touch nothing;
 *   - the first call on a device looks up the array's device address (with that device
 *     current); make that first call before any stream capture is begun;
 *   - all calls on a device share the one array: two calls whose kernels overlap on the GPU
 *     (different streams or host threads) race.  Serialise them.
 *   - the call returns after synchronising `stream` (a cudaStream_t, NULL = default stream);
 *     PBG_ERR_INDEX_RANGE reports row ids outside [0, num_rows), which are skipped. */
int pbg_row_adagrad_static(float *emb, float *state, int64_t num_rows, int32_t dim,
                           const int64_t *rows_dev, const float *grads_dev, int32_t n, float lr,
                           void *stream);

/* ---- The edge-list utilities of the reference's native module torchbiggraph._C (torchbiggraph/util.cpp:425-460),
 * on the device.  Any context serves (its configuration is not read); all pointers are device memory unless
 * stated; every call returns after synchronising the context's stream. ---- */

/* reverse_permutation (util.cpp:103-125): out[perm[i]] = i.  perm, out: int64 [n]. */
int pbg_reverse_permutation(pbg_context *ctx, const int64_t *perm_dev, int64_t n, int64_t *out_dev);

/* shuffle (util.cpp:127-220): row i of the table moves to row perm[i].  The reference permutes in place by
 * following cycles on host threads; here `in` and `out` are two different buffers of rows x row_bytes bytes
 * (the Python wrapper keeps the in-place interface).  A permutation value outside [0, rows) gives
 * PBG_ERR_INDEX_RANGE ("Permutation has out-of-bound values", util.cpp:200-202); that row is skipped. */
int pbg_shuffle_rows(pbg_context *ctx, const void *in_dev, void *out_dev, int64_t rows, int64_t row_bytes,
                     const int64_t *perm_dev);

/* randperm (util.cpp:14-101; also where the trainers call torch.randperm for the per-bucket edge shuffle,
 * train_cpu.py:857-859, train_gpu.py:245): a uniformly random permutation of [0, n) fixed by `seed`, int64 [n].
 * The reference's stream is a Mersenne Twister per host thread (its output depends on the thread count); this
 * one sorts 44-bit hashes of (seed, index).  n < 2^31. */
int pbg_randperm(pbg_context *ctx, int64_t n, uint64_t seed, int64_t *out_dev);

/* sub_bucket (util.cpp:260-423): splits a bucket's edges into num_lhs_sub_parts x num_rhs_sub_parts sub-buckets.
 * An entity's offset goes through the permutation of its relation's entity type; the permuted offset divided by
 * ceil(count / parts) is its sub-partition, the remainder its offset there.  Outputs hold the sub-buckets one
 * after the other in (i, j) row-major order, every edge at its sub-partition offsets, in input order inside a
 * sub-bucket -- the layout the reference returns as views (util.cpp:344-362).
 *   lhs_in / rhs_in / rel_in, lhs_out / rhs_out / rel_out : device int64 [num_edges]
 *   lhs_entity_counts / rhs_entity_counts                 : HOST int64 [num_relations]
 *   lhs_perms / rhs_perms                                 : HOST arrays [num_relations] of DEVICE int64 pointers
 *   dynamic_relations                                     : 1 = every edge uses entry 0 of the per-relation arrays
 *   sub_bucket_counts                                     : HOST int64 [parts_l * parts_r], edges per sub-bucket
 * A relation id outside [0, num_relations) gives PBG_ERR_INDEX_RANGE ("rel > numRelations", util.cpp:320-322). */
int pbg_sub_bucket(pbg_context *ctx, const int64_t *lhs_in, const int64_t *rhs_in, const int64_t *rel_in, int64_t num_edges,
                   int32_t num_relations, const int64_t *lhs_entity_counts, const int64_t *const *lhs_perms,
                   const int64_t *rhs_entity_counts, const int64_t *const *rhs_perms,
                   int64_t *lhs_out, int64_t *rhs_out, int64_t *rel_out,
                   int32_t num_lhs_sub_parts, int32_t num_rhs_sub_parts, int32_t dynamic_relations,
                   int64_t *sub_bucket_counts);

/* Kernel launches issued by this context since creation (for launch accounting). */
int64_t pbg_launch_count(const pbg_context *ctx);

/* Per-kernel-class device timing with CUDA events on the context's stream (the reference only
 * keeps wall-clock sections per bucket, torchbiggraph/train_cpu.py:614-703).  While enabled every
 * class of launches of every wave is bracketed by an event pair, which costs a little
 * throughput: switch it on for a measuring pass only.  pbg_kernel_times synchronises the
 * stream, adds up the pairs recorded since the last read and clears them.
 * enable = 1: pairs on the streams as the library uses them (the two halves of a wave run on two
 * streams and their classes overlap: a pair then spans whatever ran beside its kernels);
 * enable = 2: the halves are launched one after the other on the context's stream, so that a pair
 * brackets its kernels alone -- the durations to hold against a roofline.
 * Classes: 0 sort keys + radix sort, 1 gather/operator/prepare, 2 score contraction, 3 loss,
 * 4 gradient contractions, 5 optimizer updates, 6 stats.  ms_out / launches_out: HOST arrays of
 * PBG_NUM_KERNEL_CLASSES entries. */
#define PBG_NUM_KERNEL_CLASSES 7
int pbg_set_profiling(pbg_context *ctx, int enable);
int pbg_kernel_times(pbg_context *ctx, double *ms_out, int64_t *launches_out);

#ifdef __cplusplus
}
#endif
#endif /* PBG_B200_H */
