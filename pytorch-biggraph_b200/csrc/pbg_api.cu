// C ABI of the library (include/pbg_b200.h): context, workspace carving, and the per-wave launch
// sequence  keys -> sort -> gather -> score -> loss -> gradient products -> optimizer steps -> stats.
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "pbg_common.cuh"


struct pbg_context {
  pbg_config cfg;
  int device;
  cudaStream_t stream;
  std::string err;
  // static geometry
  int Dp, Pm, U, Mm, Ms, Cm, spb, kmax;
  // workspace
  char *ws = nullptr;
  size_t ws_bytes = 0;
  WaveBufs bufs;           // workspace pointers (table pointers filled per call)
  SortPlan sort[2];        // double-buffered: wave w+1 is sorted on `side` while wave w trains
  cudaStream_t side = nullptr;      // key build + sort of the next wave
  cudaStream_t part2 = nullptr;     // second half of a wave's gather / score / loss / gradient kernels
  cudaEvent_t ev_wave = nullptr, ev_part2 = nullptr, ev_joined = nullptr, ev_stats = nullptr;
  cudaEvent_t ev_sorted[2] = {nullptr, nullptr}, ev_updated[2] = {nullptr, nullptr}, ev_inputs = nullptr;
  pbg_batch_stats *stats_dev = nullptr;
  int stats_cap = 0;
  double *sum_dev = nullptr;
  double *eval_dev = nullptr;
  int *errflag = nullptr;
  void *tcplan = nullptr;       // tensor maps of the tcgen05 contractions
  void *pairplan = nullptr;     // tensor maps of the fused score + loss kernel (standard relations, plane tiers)
  bool fused = false;           // training runs gather -> fused score / loss -> dual gradient product
  bool fused_halves = false;    // ... as two halves of the wave on two streams (PBG_HALVES=1; for comparisons)
  float *psum = nullptr;        // partial gradient rows of hub rows, indexed by slot position
  long long *hublist = nullptr;
  int *hubcnt = nullptr;
  long long *bigtab = nullptr;  // batch boundaries of the rows with 256 and more slots in a wave
  cudaStream_t upd_side = nullptr;                          // operator-row kernels that run beside the embedding rows' update
  cudaEvent_t ev_upd_fork = nullptr, ev_upd_join = nullptr;
  long long *edge_dev[3] = {nullptr, nullptr, nullptr};
  long long edge_cap = 0;
  long long *uni_dev[2] = {nullptr, nullptr};
  long long uni_cap = 0;
  long long launches = 0;
  unsigned long long batches_done = 0;
  // scratch of the edge-list utilities (pbg_randperm, pbg_sub_bucket): grown on demand
  SortPlan esort = {{nullptr, nullptr}, {nullptr, nullptr}, nullptr, 0, 0};
  char *esort_mem = nullptr;
  long long *etab_dev = nullptr;      // per-relation tables of a sub_bucket call + its counts
  long long etab_cap = 0;
  char *allnegs_mem = nullptr;        // scratch of pbg_eval_batch_all_negs, allocated at its first call
  SortPlan csort = {{nullptr, nullptr}, {nullptr, nullptr}, nullptr, 0, 0};   // call-wide sort of all waves' slots
  char *csort_mem = nullptr;
  int split_min_k = 2;                // waves of at least this many batches run as two halves on two streams (PBG_SPLIT_MIN_K)
  int group_sort_mode = -1;           // PBG_CALL_SORT: 1 = always sort waves in groups, 0 = never, unset = where it pays
  std::vector<cudaEvent_t> ev_group;  // one per group of waves sorted together
  // optional event timing per kernel class
  const float *edge_w = nullptr;   // per-edge weights for the next train / eval call (pbg_set_edge_weights)
  bool profiling = false;
  bool profile_serial = false;   // profiling mode 2: one stream, so that an event pair brackets one kernel class alone
  struct Span { int cls; int launches; cudaEvent_t a, b; };
  std::vector<Span> spans;
  std::vector<cudaEvent_t> event_pool;
};

// Brackets the launches of one kernel class with an event pair when profiling is on.
struct ClassTimer {
  pbg_context *c; int cls; cudaEvent_t a = nullptr, b = nullptr;
  static cudaEvent_t get(pbg_context *c) {
    cudaEvent_t e;
    if (!c->event_pool.empty()) { e = c->event_pool.back(); c->event_pool.pop_back(); return e; }
    cudaEventCreate(&e);
    return e;
  }
  cudaStream_t st;
  ClassTimer(pbg_context *c_, int cls_, cudaStream_t st_ = nullptr) : c(c_), cls(cls_), st(st_ ? st_ : c_->stream) {
    if (c->profiling) { a = get(c); b = get(c); cudaEventRecord(a, st); }
  }
  void done(int launches) {
    c->launches += launches;
    if (c->profiling) { cudaEventRecord(b, st); c->spans.push_back({cls, launches, a, b}); }
  }
};

static int fail(pbg_context *c, int code, const char *fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  if (c) c->err = buf;
  return code;
}
#define CU(c, call)                                                                          \
  do {                                                                                       \
    cudaError_t e_ = (call);                                                                 \
    if (e_ != cudaSuccess) return fail(c, PBG_ERR_CUDA, "%s: %s", #call, cudaGetErrorString(e_)); \
  } while (0)

extern "C" const char *pbg_version(void) { return "pbg_b200 0.1 (sm_100a)"; }
extern "C" const char *pbg_status_string(int s) {
  switch (s) {
    case PBG_OK: return "ok";
    case PBG_ERR_BAD_ARGUMENT: return "bad argument";
    case PBG_ERR_UNSUPPORTED: return "unsupported plugin or option";
    case PBG_ERR_INDEX_RANGE: return "entity or relation id out of range";
    case PBG_ERR_TIMEOUT: return "bounded device wait ran out";
    case PBG_ERR_CUDA: return "CUDA error";
    case PBG_ERR_NO_DEVICE: return "no usable CUDA device";
    case PBG_ERR_TOO_LARGE: return "size beyond a stated maximum";
  }
  return "unknown status";
}
extern "C" const char *pbg_last_error(const pbg_context *c) { return c ? c->err.c_str() : "null context"; }
extern "C" int64_t pbg_workspace_bytes(const pbg_context *c) { return c ? (int64_t)c->ws_bytes : 0; }
extern "C" int64_t pbg_launch_count(const pbg_context *c) { return c ? c->launches : 0; }

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

static int chunk_geometry(const pbg_config &cfg, int *Pm, int *Cm) {
  int B = cfg.max_batch_size;
  int lim = cfg.num_batch_negs > 0 ? cfg.num_batch_negs : cfg.num_uniform_negs;
  if (lim <= 0) return PBG_ERR_BAD_ARGUMENT;
  *Pm = lim < B ? lim : B;
  *Cm = (B + *Pm - 1) / *Pm;
  return PBG_OK;
}

extern "C" int pbg_create(const pbg_config *cfg, int device, void *stream, pbg_context **out) {
  if (!cfg || !out) return PBG_ERR_BAD_ARGUMENT;
  *out = nullptr;
  pbg_context *c = new pbg_context();
  c->cfg = *cfg;
  c->device = device;
  c->stream = (cudaStream_t)stream;
  *out = c;   // returned even on failure so that the caller can read the error text
  if (cfg->dim <= 0 || cfg->dim % 4 != 0 || cfg->dim > 2048)
    return fail(c, PBG_ERR_UNSUPPORTED, "dimension %d: this build needs a multiple of 4 up to 2048", cfg->dim);
  if (cfg->op < PBG_OP_NONE || cfg->op > PBG_OP_AFFINE) return fail(c, PBG_ERR_BAD_ARGUMENT, "unknown operator %d", cfg->op);
  const bool matrix_op = cfg->op == PBG_OP_LINEAR || cfg->op == PBG_OP_AFFINE;
  if (matrix_op && cfg->dynamic_relations)
    return fail(c, PBG_ERR_UNSUPPORTED, "operator %s with dynamic relations (one matrix per edge) has no device code",
                cfg->op == PBG_OP_LINEAR ? "linear" : "affine");
  if (matrix_op && cfg->regularization_coef != 0.f)
    return fail(c, PBG_ERR_UNSUPPORTED, "Regularizer not implemented for this operator");   /* operators.py:39-40 */
  if (cfg->op == PBG_OP_COMPLEX_DIAGONAL && cfg->dim % 8 != 0)
    return fail(c, PBG_ERR_UNSUPPORTED, "complex_diagonal needs a dimension that is a multiple of 8 (got %d)", cfg->dim);
  if (cfg->comparator < PBG_CMP_DOT || cfg->comparator > PBG_CMP_SQUARED_L2) return fail(c, PBG_ERR_BAD_ARGUMENT, "unknown comparator %d", cfg->comparator);
  if (cfg->loss < PBG_LOSS_LOGISTIC || cfg->loss > PBG_LOSS_SOFTMAX) return fail(c, PBG_ERR_BAD_ARGUMENT, "unknown loss %d", cfg->loss);
  if (cfg->num_batch_negs < 0 || cfg->num_uniform_negs < 0 || cfg->max_batch_size <= 0 || cfg->num_rels <= 0)
    return fail(c, PBG_ERR_BAD_ARGUMENT, "negative or zero size in config");
  if (cfg->batches_in_flight < 1 || cfg->batches_in_flight > PBG_KMAX)
    return fail(c, PBG_ERR_BAD_ARGUMENT, "batches_in_flight must be in [1, %d]", PBG_KMAX);
  if ((size_t)cfg->batches_in_flight * ((cfg->dim + 127) / 128) * 512 > 227 * 1024)
    return fail(c, PBG_ERR_TOO_LARGE, "batches_in_flight %d with dimension %d: the per-batch totals of a hub row exceed shared memory (at most 28 batches above dimension 1024)",
                cfg->batches_in_flight, cfg->dim);
  if (cfg->precision < PBG_PREC_FP32 || cfg->precision > PBG_PREC_BF16X3) return fail(c, PBG_ERR_BAD_ARGUMENT, "unknown precision %d", cfg->precision);
  const bool planes = cfg->precision == PBG_PREC_BF16X6 || cfg->precision == PBG_PREC_BF16X3;
  const size_t npl = cfg->precision == PBG_PREC_BF16X3 ? 2 : 3;
  if (planes && matrix_op)
    return fail(c, PBG_ERR_UNSUPPORTED, "the bf16-plane precisions do not cover the linear / affine operators; use tf32x3");
  if (chunk_geometry(*cfg, &c->Pm, &c->Cm) != PBG_OK)
    return fail(c, PBG_ERR_BAD_ARGUMENT, "num_batch_negs and num_uniform_negs are both 0: no chunk size (model.py:648-656)");

  int ndev = 0;
  if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev <= device || device < 0)
    return fail(c, PBG_ERR_NO_DEVICE, "CUDA device %d not available", device);
  CU(c, cudaSetDevice(device));
  cudaDeviceProp prop;
  CU(c, cudaGetDeviceProperties(&prop, device));
  if (prop.major != 10) return fail(c, PBG_ERR_NO_DEVICE, "device %d is sm_%d%d; this library is built for sm_100a only", device, prop.major, prop.minor);

  c->kmax = cfg->batches_in_flight;
  c->U = cfg->num_uniform_negs;
  c->Mm = c->Pm + c->U;
  c->Ms = (c->Mm + 3) / 4 * 4;
  c->Dp = (cfg->dim + 31) / 32 * 32;
  c->spb = cfg->dynamic_relations ? c->Cm * (2 * c->Mm + 4 * c->Pm) : c->Cm * 2 * c->Mm;
  const bool dyn = cfg->dynamic_relations != 0;
  size_t nblk = (size_t)c->kmax * c->Cm;
  size_t nN = nblk * c->Mm, nQ = nblk * c->Pm;
  long long nocc = (long long)c->kmax * c->spb;
  if (nocc > (1ll << 30)) return fail(c, PBG_ERR_TOO_LARGE, "wave of %lld row slots is beyond 2^30", nocc);

  // ---- carve the workspace ------------------------------------------------------------------
  size_t off = 0;
  auto take = [&](size_t bytes) { size_t o = off; off = align_up(off + bytes, 256); return o; };
  size_t oReg = 0, oRscale = 0;
  size_t oX[4], oAux[4], oG[4], oS[2], oSpos[2], oCoef[4], oLoss[2], oViol[2], oRank[2];
  oX[0] = take(nN * c->Dp * 4); oX[1] = take(nN * c->Dp * 4);
  oAux[0] = take(nN * 4); oAux[1] = take(nN * 4);
  if (dyn) { oX[2] = take(nQ * c->Dp * 4); oX[3] = take(nQ * c->Dp * 4); oAux[2] = take(nQ * 4); oAux[3] = take(nQ * 4); }
  else { oX[2] = oX[1]; oX[3] = oX[0]; oAux[2] = oAux[1]; oAux[3] = oAux[0]; }
  oG[0] = take(nN * c->Dp * 4); oG[1] = take(nN * c->Dp * 4);
  if (dyn) { oG[2] = take(nQ * c->Dp * 4); oG[3] = take(nQ * c->Dp * 4); }
  else { oG[2] = oG[0]; oG[3] = oG[1]; }            // standard relations have no GQ arrays
  const int Ma = (c->Mm + 3) / 4 * 4;
  size_t oA[2] = {0, 0};
  if (!dyn) {
    for (int s2 = 0; s2 < 2; ++s2) oA[s2] = take(nN * Ma * 4);
  }
  const int Dpb = (cfg->dim + 7) / 8 * 8, Kb = (c->Mm + 7) / 8 * 8;
  size_t oXB[4] = {0, 0, 0, 0}, oAB[2] = {0, 0}, oTB[2] = {0, 0};
  // Standard relations under the dot / cos comparators with one score tile per chunk block: the fused
  // score + loss kernel and the dual gradient product (pbg_pair.cu).  Measured on a B200 it wins at dimension 100
  // (+2.5 % and +5 % on the two such workloads, fewer and shorter launches) and loses at dimension 1024 (-4 %: the
  // dual product's second operand costs more there than the merged coefficient matrix it saves), so it is the
  // default up to dimension 256.  PBG_FUSED=1 / 0 in the environment forces one or the other.
  {
    const char *env = getenv("PBG_FUSED");
    const bool eligible = planes && !dyn && !matrix_op && cfg->comparator < PBG_CMP_L2 && c->Pm <= 128 && c->Mm <= 256;
    c->fused = eligible && (env && (env[0] == '0' || env[0] == '1') ? env[0] == '1' : cfg->dim <= 256);
    const char *envh = getenv("PBG_HALVES");
    c->fused_halves = envh && envh[0] == '1';
    const char *envk = getenv("PBG_SPLIT_MIN_K");
    if (envk && atoi(envk) >= 2) c->split_min_k = atoi(envk);
    const char *envs = getenv("PBG_CALL_SORT");
    if (envs && (envs[0] == '0' || envs[0] == '1')) c->group_sort_mode = envs[0] - '0';
  }
  if (planes) {
    oXB[0] = take(nN * npl * Dpb * 2); oXB[1] = take(nN * npl * Dpb * 2);
    if (dyn) { oXB[2] = take(nQ * npl * Dpb * 2); oXB[3] = take(nQ * npl * Dpb * 2); oTB[0] = take(nQ * npl * Kb * 2); oTB[1] = take(nQ * npl * Kb * 2); }
    else { oXB[2] = oXB[1]; oXB[3] = oXB[0]; oAB[0] = take(nN * npl * Kb * 2); oAB[1] = take(nN * npl * Kb * 2); }
    if (c->fused)
      for (int p = 0; p < 2; ++p) oTB[p] = take(nQ * npl * Kb * 2);
  }
  for (int p = 0; p < 2; ++p) {
    oS[p] = take(nQ * c->Ms * 4); oSpos[p] = take(nQ * 4); oLoss[p] = take(nQ * 4); oViol[p] = take(nQ * 4);
    if (p == 0) { oReg = take(nQ * 4); oRscale = take(nN * 4); }
    oRank[p] = take(nQ * 4);
  }
  oCoef[0] = take(nN * 4); oCoef[1] = take(nN * 4); oCoef[2] = take(nQ * 4); oCoef[3] = take(nQ * 4);
  size_t oRel = take(nblk * 8 * (size_t)cfg->dim * 4);
  size_t oGlobPart = take(nblk * 2 * 8 * (size_t)cfg->dim * 4);
  const size_t opw = matrix_op ? (size_t)cfg->dim * cfg->dim + (cfg->op == PBG_OP_AFFINE ? cfg->dim : 0) : (size_t)cfg->dim;
  size_t oR1 = 0, oR2 = 0, oDA = 0;
  if (matrix_op) { oR1 = take(nN * c->Dp * 4); oR2 = take(nN * c->Dp * 4); oDA = take((size_t)c->kmax * opw * 4); }
  size_t oK[2][2], oV[2][2], oH[2];
  for (int s = 0; s < 2; ++s) {
    oK[s][0] = take((size_t)nocc * 8); oK[s][1] = take((size_t)nocc * 8);
    oV[s][0] = take((size_t)nocc * 4); oV[s][1] = take((size_t)nocc * 4);
    oH[s] = take(pbg_sort_hist_entries((int)nocc) * 4);
  }
  size_t oSum = take(8 * sizeof(double)), oErr = take(256), oEval = take(8 * sizeof(double));
  size_t oPsum = take((size_t)nocc * c->Dp * 4), oHub = take(((size_t)nocc / 8 + 64) * 8), oHubCnt = take(256);
  size_t oBigTab = take(pbg_bigtab_bytes((long long)nocc));
  // dynamic relations with a (vector) operator: the operator-row gradient of every edge, written by the pull-back pass
  size_t oGR[2] = {0, 0};
  const bool keep_gr = dyn && cfg->op != PBG_OP_NONE && !matrix_op;
  if (keep_gr) { oGR[0] = take(nQ * c->Dp * 4); oGR[1] = take(nQ * c->Dp * 4); }
  c->ws_bytes = off;
  CU(c, cudaMalloc(&c->ws, c->ws_bytes));
  CU(c, cudaMemsetAsync(c->ws, 0, c->ws_bytes, c->stream));
  WaveBufs &b = c->bufs;
  memset(&b, 0, sizeof b);
  for (int a = 0; a < 4; ++a) {
    b.X[a] = (float *)(c->ws + oX[a]);
    b.aux[a] = (float *)(c->ws + oAux[a]);
    b.GX[a] = (float *)(c->ws + oG[a]);
    b.coef[a] = (float *)(c->ws + oCoef[a]);
  }
  for (int p = 0; p < 2; ++p) b.A[p] = dyn ? nullptr : (float *)(c->ws + oA[p]);
  b.Ma = Ma;
  b.Dpb = Dpb; b.Kb = Kb; b.npl = (int)npl;
  for (int a = 0; a < 4; ++a) b.XB[a] = planes ? (unsigned short *)(c->ws + oXB[a]) : nullptr;
  for (int p = 0; p < 2; ++p) {
    b.AB[p] = (planes && !dyn) ? (unsigned short *)(c->ws + oAB[p]) : nullptr;
    b.TB[p] = (planes && (dyn || c->fused)) ? (unsigned short *)(c->ws + oTB[p]) : nullptr;
  }
  b.xrows[0] = b.xrows[1] = c->Mm;
  b.xrows[2] = b.xrows[3] = dyn ? c->Pm : c->Mm;
  for (int t = 0; t < 2; ++t) b.GR[t] = keep_gr ? (float *)(c->ws + oGR[t]) : nullptr;
  b.grows[0] = b.grows[1] = c->Mm;
  b.grows[2] = b.grows[3] = c->Pm;
  for (int p = 0; p < 2; ++p) {
    b.S[p] = (float *)(c->ws + oS[p]);
    b.spos[p] = (float *)(c->ws + oSpos[p]);
    b.lossrow[p] = (float *)(c->ws + oLoss[p]);
    if (p == 0) { b.regrow = (float *)(c->ws + oReg); b.rscale = (float *)(c->ws + oRscale); }
    b.violrow[p] = (int *)(c->ws + oViol[p]);
    b.rankrow[p] = (int *)(c->ws + oRank[p]);
  }
  b.relpart = (float *)(c->ws + oRel);
  b.globpart = (float *)(c->ws + oGlobPart);
  b.R1 = matrix_op ? (float *)(c->ws + oR1) : nullptr;
  b.R2 = matrix_op ? (float *)(c->ws + oR2) : nullptr;
  b.dA = matrix_op ? (float *)(c->ws + oDA) : nullptr;
  for (int s = 0; s < 2; ++s) {
    c->sort[s].keys[0] = (unsigned long long *)(c->ws + oK[s][0]);
    c->sort[s].keys[1] = (unsigned long long *)(c->ws + oK[s][1]);
    c->sort[s].vals[0] = (unsigned int *)(c->ws + oV[s][0]);
    c->sort[s].vals[1] = (unsigned int *)(c->ws + oV[s][1]);
    c->sort[s].hist = (unsigned int *)(c->ws + oH[s]);
    c->sort[s].max_n = (int)nocc;
    c->sort[s].result = 0;
    CU(c, cudaEventCreateWithFlags(&c->ev_sorted[s], cudaEventDisableTiming));
    CU(c, cudaEventCreateWithFlags(&c->ev_updated[s], cudaEventDisableTiming));
  }
  CU(c, cudaEventCreateWithFlags(&c->ev_inputs, cudaEventDisableTiming));
  CU(c, cudaStreamCreateWithFlags(&c->side, cudaStreamNonBlocking));
  CU(c, cudaStreamCreateWithFlags(&c->part2, cudaStreamNonBlocking));
  CU(c, cudaEventCreateWithFlags(&c->ev_wave, cudaEventDisableTiming));
  CU(c, cudaEventCreateWithFlags(&c->ev_part2, cudaEventDisableTiming));
  CU(c, cudaEventCreateWithFlags(&c->ev_joined, cudaEventDisableTiming));
  CU(c, cudaEventCreateWithFlags(&c->ev_stats, cudaEventDisableTiming));
  if (!(getenv("PBG_REL_ASIDE") && getenv("PBG_REL_ASIDE")[0] == '0')) {        // PBG_REL_ASIDE=0: everything on one stream (for comparisons)
    CU(c, cudaStreamCreateWithFlags(&c->upd_side, cudaStreamNonBlocking));
    CU(c, cudaEventCreateWithFlags(&c->ev_upd_fork, cudaEventDisableTiming));
    CU(c, cudaEventCreateWithFlags(&c->ev_upd_join, cudaEventDisableTiming));
  }
  c->sum_dev = (double *)(c->ws + oSum);
  c->errflag = (int *)(c->ws + oErr);
  c->eval_dev = (double *)(c->ws + oEval);
  b.errflag = c->errflag;
  c->psum = (float *)(c->ws + oPsum);
  c->hublist = (long long *)(c->ws + oHub);
  c->hubcnt = (int *)(c->ws + oHubCnt);
  c->bigtab = (long long *)(c->ws + oBigTab);
  if (cfg->precision != PBG_PREC_FP32) {
    WaveDims gd;
    memset(&gd, 0, sizeof gd);
    gd.D = cfg->dim; gd.Dp = c->Dp; gd.Pm = c->Pm; gd.U = c->U; gd.Mm = c->Mm; gd.Ms = c->Ms; gd.Cm = c->Cm;
    gd.dynamic = dyn;
    c->tcplan = pbg_tc_plan_create(gd, b, (int)nblk, cfg->precision);
    if (!c->tcplan) return fail(c, PBG_ERR_CUDA, "could not encode the TMA tensor maps of the tensor-core contractions");
    if (c->fused) {
      c->pairplan = pbg_pair_plan_create(gd, b, (int)nblk);
      if (!c->pairplan) return fail(c, PBG_ERR_CUDA, "could not encode the TMA tensor maps of the fused score kernel");
    }
  }
  CU(c, cudaStreamSynchronize(c->stream));
  return PBG_OK;
}

extern "C" int pbg_destroy(pbg_context *c) {
  if (!c) return PBG_OK;
  cudaSetDevice(c->device);
  if (c->ws) cudaFree(c->ws);
  if (c->tcplan) pbg_tc_plan_destroy(c->tcplan);
  if (c->pairplan) pbg_pair_plan_destroy(c->pairplan);
  if (c->stats_dev) cudaFree(c->stats_dev);
  for (int i = 0; i < 3; ++i) if (c->edge_dev[i]) cudaFree(c->edge_dev[i]);
  for (int i = 0; i < 2; ++i) if (c->uni_dev[i]) cudaFree(c->uni_dev[i]);
  if (c->esort_mem) cudaFree(c->esort_mem);
  if (c->allnegs_mem) cudaFree(c->allnegs_mem);
  if (c->csort_mem) cudaFree(c->csort_mem);
  for (auto e : c->ev_group) cudaEventDestroy(e);
  if (c->etab_dev) cudaFree(c->etab_dev);
  for (int s = 0; s < 2; ++s) {
    if (c->ev_sorted[s]) cudaEventDestroy(c->ev_sorted[s]);
    if (c->ev_updated[s]) cudaEventDestroy(c->ev_updated[s]);
  }
  if (c->ev_inputs) cudaEventDestroy(c->ev_inputs);
  if (c->side) cudaStreamDestroy(c->side);
  if (c->part2) cudaStreamDestroy(c->part2);
  if (c->upd_side) cudaStreamDestroy(c->upd_side);
  if (c->ev_upd_fork) cudaEventDestroy(c->ev_upd_fork);
  if (c->ev_upd_join) cudaEventDestroy(c->ev_upd_join);
  if (c->ev_wave) cudaEventDestroy(c->ev_wave);
  if (c->ev_part2) cudaEventDestroy(c->ev_part2);
  if (c->ev_joined) cudaEventDestroy(c->ev_joined);
  if (c->ev_stats) cudaEventDestroy(c->ev_stats);
  for (auto &s : c->spans) { cudaEventDestroy(s.a); cudaEventDestroy(s.b); }
  for (auto e : c->event_pool) cudaEventDestroy(e);
  delete c;
  return PBG_OK;
}

extern "C" int pbg_set_hyperparameters(pbg_context *c, float lr, float relation_lr, float margin) {
  if (!c) return PBG_ERR_BAD_ARGUMENT;
  c->cfg.lr = lr; c->cfg.relation_lr = relation_lr; c->cfg.margin = margin;
  return PBG_OK;
}

extern "C" int pbg_neg_columns(const pbg_context *c, int32_t count, int32_t *chunk_size, int32_t *chunks,
                               int32_t *lhs_neg_cols, int32_t *rhs_neg_cols) {
  if (!c || count < 0) return PBG_ERR_BAD_ARGUMENT;
  int lim = c->cfg.num_batch_negs > 0 ? c->cfg.num_batch_negs : c->cfg.num_uniform_negs;
  int P = count < lim ? count : lim;
  int cols = c->cfg.num_batch_negs > 0 ? P + c->U : c->U;
  if (chunk_size) *chunk_size = P;
  if (chunks) *chunks = P > 0 ? (count + P - 1) / P : 0;
  if (lhs_neg_cols) *lhs_neg_cols = c->cfg.disable_lhs_negs ? 0 : cols;
  if (rhs_neg_cols) *rhs_neg_cols = c->cfg.disable_rhs_negs ? 0 : cols;
  return PBG_OK;
}

#define PBG_CALL_SORT_MAX (1ll << 23)     // most slots of a call whose waves are sorted in groups (the buffers hold all of them: 24 bytes per slot)
#define PBG_SORT_GROUP_SLOTS (1ll << 19)  // slots sorted at a time

static int ensure_call_sort(pbg_context *c, long long n) {
  if (n <= c->csort.max_n) return PBG_OK;
  if (c->csort_mem) { cudaFree(c->csort_mem); c->csort_mem = nullptr; c->csort.max_n = 0; }
  const long long cap = n + n / 8 + 1024;
  const size_t kb = align_up((size_t)cap * 8, 256), vb = align_up((size_t)cap * 4, 256);
  const size_t hb = align_up(pbg_sort_hist_entries((int)cap) * 4, 256);
  CU(c, cudaMalloc(&c->csort_mem, 2 * kb + 2 * vb + hb));
  char *p = c->csort_mem;
  c->csort.keys[0] = (unsigned long long *)p; c->csort.keys[1] = (unsigned long long *)(p + kb);
  c->csort.vals[0] = (unsigned int *)(p + 2 * kb); c->csort.vals[1] = (unsigned int *)(p + 2 * kb + vb);
  c->csort.hist = (unsigned int *)(p + 2 * kb + 2 * vb);
  c->csort.max_n = (int)cap;
  return PBG_OK;
}

static int bit_length(unsigned long long v) { int b = 0; while (v) { ++b; v >>= 1; } return b < 1 ? 1 : b; }

// Fills the per-call parts of dims / bufs from the bucket.
static int bind_bucket(pbg_context *c, const pbg_bucket *bk, WaveDims &d, WaveBufs &w) {
  const pbg_config &cfg = c->cfg;
  if (!bk || !bk->lhs_emb || !bk->rhs_emb) return fail(c, PBG_ERR_BAD_ARGUMENT, "bucket without embedding tables");
  if (bk->lhs_rows <= 0 || bk->rhs_rows <= 0) return fail(c, PBG_ERR_BAD_ARGUMENT, "bucket with an empty table");
  if (((uintptr_t)bk->lhs_emb | (uintptr_t)bk->rhs_emb) & 15) return fail(c, PBG_ERR_BAD_ARGUMENT, "embedding tables must be 16-byte aligned");
  bool has_op = cfg.op != PBG_OP_NONE;
  if (has_op && !bk->rhs_op) return fail(c, PBG_ERR_BAD_ARGUMENT, "operator configured but bucket has no rhs_op table");
  if (has_op && cfg.dynamic_relations && !bk->lhs_op) return fail(c, PBG_ERR_BAD_ARGUMENT, "dynamic relations need the lhs_op table");
  memset(&d, 0, sizeof d);
  d.D = cfg.dim; d.Dp = c->Dp; d.Pm = c->Pm; d.U = c->U; d.Mm = c->Mm; d.Ms = c->Ms; d.Cm = c->Cm;
  d.op = cfg.op; d.cmp = cfg.comparator; d.loss = cfg.loss; d.dynamic = cfg.dynamic_relations != 0;
  d.batch_negs = cfg.num_batch_negs > 0;
  d.neg_enabled[0] = !cfg.disable_lhs_negs; d.neg_enabled[1] = !cfg.disable_rhs_negs;
  d.num_batch_negs = cfg.num_batch_negs; d.spb = c->spb; d.margin = cfg.margin; d.reg_coef = cfg.regularization_coef; d.max_norm = cfg.max_norm > 0.f ? cfg.max_norm : 0.f;
  d.matrix_op = cfg.op == PBG_OP_LINEAR || cfg.op == PBG_OP_AFFINE;
  d.opw = d.matrix_op ? cfg.dim * cfg.dim + (cfg.op == PBG_OP_AFFINE ? cfg.dim : 0) : cfg.dim;
  d.n_rows[0] = bk->lhs_rows; d.n_rows[1] = bk->rhs_rows;
  d.shared_table = bk->lhs_emb == bk->rhs_emb;
  if (d.shared_table && bk->lhs_rows != bk->rhs_rows) return fail(c, PBG_ERR_BAD_ARGUMENT, "shared table with different row counts");
  d.num_rels = cfg.num_rels;
  unsigned long long emb_keys = (unsigned long long)bk->lhs_rows + (d.shared_table ? 0ull : (unsigned long long)bk->rhs_rows);
  d.key_rel_base = emb_keys;
  d.key_invalid = emb_keys + ((d.dynamic && has_op) ? 2ull * cfg.num_rels : 0ull);
  w = c->bufs;
  w.ew = nullptr;
  w.glob[0] = bk->lhs_global; w.glob[1] = bk->rhs_global;
  w.gacc[0] = bk->lhs_global_state; w.gacc[1] = bk->rhs_global_state;
  w.glob_shared = bk->lhs_global != nullptr && bk->lhs_global == bk->rhs_global;
  if ((bk->lhs_global || bk->rhs_global) && cfg.dynamic_relations)
    return fail(c, PBG_ERR_UNSUPPORTED, "global embeddings cannot be combined with dynamic relations (model.py:488-489)");
  if (((uintptr_t)bk->lhs_global | (uintptr_t)bk->rhs_global) & 15) return fail(c, PBG_ERR_BAD_ARGUMENT, "global embeddings must be 16-byte aligned");
  if (bk->lhs_emb == bk->rhs_emb && bk->lhs_global != bk->rhs_global)
    return fail(c, PBG_ERR_BAD_ARGUMENT, "one table read through two different global embeddings");
  w.W[0] = bk->lhs_emb; w.G[0] = bk->lhs_state; w.W[1] = bk->rhs_emb; w.G[1] = bk->rhs_state;
  w.theta[0] = has_op ? bk->rhs_op : nullptr; w.acc[0] = has_op ? bk->rhs_op_state : nullptr;
  w.theta[1] = (has_op && d.dynamic) ? bk->lhs_op : nullptr; w.acc[1] = (has_op && d.dynamic) ? bk->lhs_op_state : nullptr;
  return PBG_OK;
}

static int check_errflag(pbg_context *c) {
  int flag = 0;
  CU(c, cudaMemcpyAsync(&flag, c->errflag, sizeof flag, cudaMemcpyDeviceToHost, c->stream));
  CU(c, cudaStreamSynchronize(c->stream));
  if (flag) {
    cudaMemsetAsync(c->errflag, 0, sizeof(int), c->stream);
    if (flag & 2) return fail(c, PBG_ERR_TIMEOUT, "a bounded device-side wait ran out (flag %d)", flag);
    return fail(c, PBG_ERR_INDEX_RANGE, "an entity or relation id was outside its table; those rows were skipped");
  }
  return PBG_OK;
}

static int run_forward(pbg_context *c, const WaveDims &d, const WaveBatches &wb, const WaveBufs &w, cudaStream_t st) {
  {
    ClassTimer t(c, 1, st);
    int n = launch_gather(d, wb, w, st);
    if (d.matrix_op) n += launch_matrix_forward(d, wb, w, st) + launch_postop(d, wb, w, st);   // z = A x (+ t), prepare, positive score
    t.done(n);
  }
  ClassTimer t(c, 2, st);
  if (c->cfg.precision == PBG_PREC_FP32) t.done(launch_score_simt(d, wb, w, st));
  else t.done(launch_score_tc(d, wb, w, c->tcplan, st));
  return PBG_OK;
}

// gather -> score -> loss -> gradient products of the chunk blocks [d.blk0, d.blk0 + d.nblk) on `st`
static void run_part(pbg_context *c, const WaveDims &d, const WaveBatches &wb, const WaveBufs &w, cudaStream_t st) {
  if (c->fused) {
    { ClassTimer t(c, 1, st); t.done(launch_gather(d, wb, w, st)); }
    { ClassTimer t(c, 2, st); t.done(launch_pair_score(d, wb, w, c->pairplan, st)); }      // scores, loss, coefficient planes
    if (d.reg_coef != 0.f) { ClassTimer t(c, 3, st); t.done(launch_reg_value(d, wb, w, st)); }
    ClassTimer t(c, 4, st);
    t.done(launch_grad_dual_tc(d, wb, w, c->tcplan, st));
    return;
  }
  run_forward(c, d, wb, w, st);
  { ClassTimer t(c, 3, st); t.done(launch_loss(d, wb, w, st) + (d.reg_coef != 0.f ? launch_reg_value(d, wb, w, st) : 0)); }
  ClassTimer t(c, 4, st);
  int n = c->cfg.precision == PBG_PREC_FP32 ? launch_grad_simt(d, wb, w, st) : launch_grad_tc(d, wb, w, c->tcplan, st);
  if (d.matrix_op) n += launch_gz_rows(d, wb, w, st) + launch_matrix_backward(d, wb, w, st);   // back through A
  t.done(n);
}

extern "C" int pbg_set_profiling(pbg_context *c, int enable) {
  if (!c) return PBG_ERR_BAD_ARGUMENT;
  c->profiling = enable != 0;
  c->profile_serial = enable == 2;
  return PBG_OK;
}

extern "C" int pbg_kernel_times(pbg_context *c, double *ms_out, int64_t *launches_out) {
  if (!c || !ms_out || !launches_out) return PBG_ERR_BAD_ARGUMENT;
  CU(c, cudaSetDevice(c->device));
  CU(c, cudaStreamSynchronize(c->stream));
  for (int i = 0; i < PBG_NUM_KERNEL_CLASSES; ++i) { ms_out[i] = 0.0; launches_out[i] = 0; }
  for (auto &s : c->spans) {
    float ms = 0.f;
    if (cudaEventElapsedTime(&ms, s.a, s.b) == cudaSuccess) { ms_out[s.cls] += ms; launches_out[s.cls] += s.launches; }
    c->event_pool.push_back(s.a);
    c->event_pool.push_back(s.b);
  }
  c->spans.clear();
  return PBG_OK;
}

extern "C" int pbg_train_batches(pbg_context *c, const pbg_bucket *bk, const int64_t *lhs, const int64_t *rhs,
                                 const int64_t *rel, int64_t num_edges, const pbg_batch *batches,
                                 int32_t num_batches, const int64_t *ul, const int64_t *ur, uint64_t seed,
                                 pbg_batch_stats *stats_out) {
  if (!c) return PBG_ERR_BAD_ARGUMENT;
  if (num_batches == 0) return PBG_OK;
  if (!lhs || !rhs || !batches || num_batches < 0 || num_edges < 0) return fail(c, PBG_ERR_BAD_ARGUMENT, "null edge arrays or batch list");
  CU(c, cudaSetDevice(c->device));
  WaveDims d;
  WaveBufs w;
  int rc = bind_bucket(c, bk, d, w);
  if (rc) return rc;
  if (!bk->lhs_state || !bk->rhs_state) return fail(c, PBG_ERR_BAD_ARGUMENT, "bucket without RowAdagrad state");
  if (d.op != PBG_OP_NONE && (!bk->rhs_op_state || (d.dynamic && !bk->lhs_op_state)))
    return fail(c, PBG_ERR_BAD_ARGUMENT, "operator tables without AsyncAdagrad state");
  if ((bk->lhs_global && !bk->lhs_global_state) || (bk->rhs_global && !bk->rhs_global_state))
    return fail(c, PBG_ERR_BAD_ARGUMENT, "global embeddings without AsyncAdagrad state");
  if (d.dynamic && d.op != PBG_OP_NONE && !rel) return fail(c, PBG_ERR_BAD_ARGUMENT, "dynamic relations need the rel array");
  for (int i = 0; i < num_batches; ++i) {
    const pbg_batch &b = batches[i];
    if (b.count < 0 || b.count > c->cfg.max_batch_size || b.offset < 0 || b.offset + b.count > num_edges)
      return fail(c, PBG_ERR_BAD_ARGUMENT, "batch %d: offset %lld count %d outside [0, %lld] or above max_batch_size %d", i,
                  (long long)b.offset, b.count, (long long)num_edges, c->cfg.max_batch_size);
    if (!d.dynamic && (b.rel < 0 || b.rel >= c->cfg.num_rels))
      return fail(c, PBG_ERR_INDEX_RANGE, "batch %d: relation %d outside [0, %d)", i, b.rel, c->cfg.num_rels);
  }
  w.lhs = (const long long *)lhs; w.rhs = (const long long *)rhs; w.rel = (const long long *)rel;
  w.ul = (const long long *)ul; w.ur = (const long long *)ur;
  w.ew = c->edge_w; c->edge_w = nullptr;                    // per-edge weights apply to one call
  w.seed = seed ^ (c->batches_done * 0x9E3779B97F4A7C15ull);
  if (stats_out && num_batches > c->stats_cap) {
    if (c->stats_dev) cudaFree(c->stats_dev);
    c->stats_dev = nullptr;
    int cap = num_batches + num_batches / 2 + 64;
    CU(c, cudaMalloc(&c->stats_dev, (size_t)cap * sizeof(pbg_batch_stats)));
    c->stats_cap = cap;
  }
  const int bits = bit_length(d.key_invalid);
  // The sort keys depend on the edge and negative ids only, never on the tables: the key build
  // and radix sort of a wave run on the side stream and overlap the previous wave's kernels.
  CU(c, cudaEventRecord(c->ev_inputs, c->stream));
  CU(c, cudaStreamWaitEvent(c->side, c->ev_inputs, 0));
  // The batches are dealt to the fewest waves that hold them, as evenly as possible: 270 batches at
  // 14 in flight are 20 waves of 14 or 13 rather than 19 full ones and a wave of 4 that would pay
  // the same launches and joins for a quarter of the work.
  const int nwaves = (num_batches + c->kmax - 1) / c->kmax;
  const int kbase = num_batches / nwaves, kextra = num_batches % nwaves;
  std::vector<WaveBatches> wbs((size_t)nwaves);
  std::vector<int> kks((size_t)nwaves);
  std::vector<long long> slot0((size_t)nwaves + 1, 0);
  for (int wv = 0, b0 = 0; wv < nwaves; ++wv) {
    const int kk = kbase + (wv < kextra ? 1 : 0);
    WaveBatches &wb = wbs[wv];
    memset(&wb, 0, sizeof wb);
    for (int i = 0; i < kk; ++i) {
      const pbg_batch &b = batches[b0 + i];
      wb.off[i] = b.offset; wb.n[i] = b.count; wb.gidx[i] = b0 + i;
      wb.rel[i] = d.dynamic ? 0 : b.rel;
      int wi = d.dynamic ? 0 : b.rel;
      wb.wrel[i] = bk->relation_weights ? bk->relation_weights[wi] : 1.0f;
    }
    kks[wv] = kk;
    slot0[wv + 1] = slot0[wv] + (long long)kk * d.spb;
    b0 += kk;
  }
  // Waves are sorted several at a time: the slots of a group of waves, keyed by (wave in the group, row), go through
  // one radix sort of a few passes -- instead of a dozen launches of a few microseconds per wave, which on small
  // dimensions (a wave of 56,000 slots of 100 floats) are a large part of the step.  The sorted list is the per-wave
  // lists one after the other; the wave tags are masked off again.  Groups hold about PBG_SORT_GROUP_SLOTS slots, so
  // that the first update of a call waits for a short sort only and the later groups are sorted beside the training
  // of the earlier ones.  This pays where a wave's own sort needs three or more passes (keys above 22 bits: two
  // partitions of millions of rows; measured +4.5 % on such a bucket at dimension 100); with two passes per wave the
  // larger sort kernels of a group get in the way of the training kernels on the other stream more than the saved
  // launches give back (-8 % on a 100,000-row graph), so those calls, and calls of a single wave, sort wave by wave.
  // PBG_CALL_SORT=1 / 0 in the environment forces one or the other.
  const long long wave_slots = (long long)c->kmax * d.spb;
  int group = (int)((PBG_SORT_GROUP_SLOTS + wave_slots - 1) / wave_slots);
  // the first update of a call waits for the first group's sort, which nothing hides: a call of few waves (a half
  // sub-bucket of the several-GPU schedule is ten) is cut into at least four groups, of two waves or more
  if (group > (nwaves + 3) / 4) group = (nwaves + 3) / 4;
  if (group < 2) group = 2;
  if (group > nwaves) group = nwaves;
  if (group < 1) group = 1;
  const int wave_bits = bit_length((unsigned long long)(group - 1));
  const bool wanted = c->group_sort_mode == 1 || (c->group_sort_mode < 0 && bits > 22);
  const bool call_sort = wanted && nwaves > 1 && group > 1 && slot0[nwaves] <= PBG_CALL_SORT_MAX && bits + wave_bits <= 44;
  const int ngroups = call_sort ? (nwaves + group - 1) / group : 0;
  SortPlan *csp = nullptr;
  if (call_sort) {
    int rcs = ensure_call_sort(c, slot0[nwaves]);
    if (rcs) return rcs;
    csp = &c->csort;
    while ((int)c->ev_group.size() < ngroups) {
      cudaEvent_t e;
      CU(c, cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
      c->ev_group.push_back(e);
    }
    for (int gi = 0; gi < ngroups; ++gi) {
      const int w0 = gi * group, w1 = w0 + group < nwaves ? w0 + group : nwaves;
      const long long off = slot0[w0], cnt = slot0[w1] - slot0[w0];
      ClassTimer t(c, 0, c->side);
      int n = 0;
      for (int wv = w0; wv < w1; ++wv) {
        WaveDims dw = d;
        dw.k = kks[wv]; dw.nblk = kks[wv] * d.Cm; dw.nocc = kks[wv] * d.spb; dw.blk0 = 0;
        n += launch_build_keys(dw, wbs[wv], w, csp->keys[0] + slot0[wv], csp->vals[0] + slot0[wv], c->side, (unsigned long long)(wv - w0) << bits);
      }
      SortPlan gsp = *csp;                                    // the group's part of the buffers; the counters are shared (one stream)
      gsp.keys[0] += off; gsp.keys[1] += off; gsp.vals[0] += off; gsp.vals[1] += off;
      n += pbg_sort(gsp, (int)cnt, bits + wave_bits, c->side);
      csp->result = gsp.result;                               // the same number of passes for every group
      n += launch_mask_keys(gsp.keys[gsp.result], cnt, (1ull << bits) - 1ull, c->side);
      t.done(n);
      CU(c, cudaEventRecord(c->ev_group[gi], c->side));
    }
  }
  int wave = 0;
  for (int b0 = 0; b0 < num_batches; ++wave) {
    const int kk = kks[wave];
    const WaveBatches &wb = wbs[wave];
    d.k = kk; d.nblk = kk * d.Cm; d.nocc = kk * d.spb;
    SortPlan &sp = c->sort[wave & 1];
    if (!call_sort) {
      if (wave >= 2) CU(c, cudaStreamWaitEvent(c->side, c->ev_updated[wave & 1], 0));   // buffers free again
      ClassTimer t(c, 0, c->side);
      int n = launch_build_keys(d, wb, w, sp.keys[0], sp.vals[0], c->side);
      t.done(n + pbg_sort(sp, d.nocc, bits, c->side));
      CU(c, cudaEventRecord(c->ev_sorted[wave & 1], c->side));
    }
    // The batches of a wave all read the tables as the wave found them, so its forward / backward
    // kernels can run as two independent halves on two streams: the memory-bound kernels of one
    // half fill the SMs' idle issue slots while the other half's contractions run.
    d.blk0 = 0;
    if (c->fused && !c->fused_halves) {
      // the fused score kernel computes both problems of a chunk block in one CTA: a wave of 14 batches of 10
      // chunks is one round of 140 CTAs, where its halves would each leave half of the SMs idle
      run_part(c, d, wb, w, c->stream);
    } else if (kk >= c->split_min_k && c->profile_serial) {
      int ka = (kk + 1) / 2;
      WaveDims da = d, db = d;
      da.nblk = ka * d.Cm;
      db.blk0 = ka * d.Cm; db.nblk = (kk - ka) * d.Cm;
      run_part(c, da, wb, w, c->stream);
      run_part(c, db, wb, w, c->stream);
    } else if (kk >= c->split_min_k) {
      int ka = (kk + 1) / 2;
      WaveDims da = d, db = d;
      da.nblk = ka * d.Cm;
      db.blk0 = ka * d.Cm; db.nblk = (kk - ka) * d.Cm;
      CU(c, cudaEventRecord(c->ev_wave, c->stream));          // previous wave's update is in front of this
      CU(c, cudaStreamWaitEvent(c->part2, c->ev_wave, 0));
      run_part(c, db, wb, w, c->part2);
      CU(c, cudaEventRecord(c->ev_part2, c->part2));
      run_part(c, da, wb, w, c->stream);
      CU(c, cudaStreamWaitEvent(c->stream, c->ev_part2, 0));
    } else {
      run_part(c, d, wb, w, c->stream);
    }
    // The per-batch statistics need the loss rows of both halves and nothing of the update: they are
    // summed on the second stream while the update runs on the first.
    const bool stats_aside = kk >= c->split_min_k && !c->profile_serial;
    if (stats_aside) {
      CU(c, cudaEventRecord(c->ev_joined, c->stream));
      CU(c, cudaStreamWaitEvent(c->part2, c->ev_joined, 0));
      { ClassTimer t(c, 6, c->part2); t.done(launch_stats(d, wb, w, stats_out ? c->stats_dev : nullptr, c->sum_dev, c->part2)); }
      CU(c, cudaEventRecord(c->ev_stats, c->part2));
    }
    CU(c, cudaStreamWaitEvent(c->stream, call_sort ? c->ev_group[wave / group] : c->ev_sorted[wave & 1], 0));
    {
      ClassTimer t(c, 5);
      const unsigned long long *wkeys = call_sort ? csp->keys[csp->result] + slot0[wave] : sp.keys[sp.result];
      const unsigned int *wvals = call_sort ? csp->vals[csp->result] + slot0[wave] : sp.vals[sp.result];
      t.done(launch_update(d, wb, w, wkeys, wvals, c->cfg.lr, c->cfg.relation_lr, c->psum, c->hublist, c->hubcnt, c->bigtab, c->stream,
                           c->upd_side, c->ev_upd_fork, c->ev_upd_join));
    }
    CU(c, cudaEventRecord(c->ev_updated[wave & 1], c->stream));
    if (stats_aside) CU(c, cudaStreamWaitEvent(c->stream, c->ev_stats, 0));   // the next wave rewrites the loss rows
    else { ClassTimer t(c, 6); t.done(launch_stats(d, wb, w, stats_out ? c->stats_dev : nullptr, c->sum_dev, c->stream)); }
    b0 += kk;
  }
  c->batches_done += (unsigned long long)num_batches;
  CU(c, pbg_take_launch_error());
  if (stats_out) {
    CU(c, cudaMemcpyAsync(stats_out, c->stats_dev, (size_t)num_batches * sizeof(pbg_batch_stats),
                          cudaMemcpyDeviceToHost, c->stream));
    return check_errflag(c);
  }
  return PBG_OK;
}

static int grow_i64(pbg_context *c, long long **p, long long need) {
  if (*p) cudaFree(*p);
  *p = nullptr;
  CU(c, cudaMalloc(p, (size_t)need * sizeof(long long)));
  return PBG_OK;
}

extern "C" int pbg_train_batches_host(pbg_context *c, const pbg_bucket *bk, const int64_t *lhs, const int64_t *rhs,
                                      const int64_t *rel, int64_t num_edges, const pbg_batch *batches,
                                      int32_t num_batches, const int64_t *ul, const int64_t *ur, uint64_t seed,
                                      pbg_batch_stats *stats_out) {
  if (!c) return PBG_ERR_BAD_ARGUMENT;
  if (num_batches == 0) return PBG_OK;
  if (!lhs || !rhs || num_edges < 0) return fail(c, PBG_ERR_BAD_ARGUMENT, "null edge arrays");
  CU(c, cudaSetDevice(c->device));
  if (num_edges > c->edge_cap) {
    long long cap = num_edges + num_edges / 4 + 1024;
    for (int i = 0; i < 3; ++i) { int rc = grow_i64(c, &c->edge_dev[i], cap); if (rc) return rc; }
    c->edge_cap = cap;
  }
  size_t eb = (size_t)num_edges * sizeof(long long);
  CU(c, cudaMemcpyAsync(c->edge_dev[0], lhs, eb, cudaMemcpyHostToDevice, c->stream));
  CU(c, cudaMemcpyAsync(c->edge_dev[1], rhs, eb, cudaMemcpyHostToDevice, c->stream));
  if (rel) CU(c, cudaMemcpyAsync(c->edge_dev[2], rel, eb, cudaMemcpyHostToDevice, c->stream));
  long long *uld = nullptr, *urd = nullptr;
  if (ul || ur) {
    long long per = (long long)num_batches * c->Cm * c->U;
    if (per > c->uni_cap) {
      for (int i = 0; i < 2; ++i) { int rc = grow_i64(c, &c->uni_dev[i], per + 1024); if (rc) return rc; }
      c->uni_cap = per + 1024;
    }
    if (ul) { CU(c, cudaMemcpyAsync(c->uni_dev[0], ul, (size_t)per * 8, cudaMemcpyHostToDevice, c->stream)); uld = c->uni_dev[0]; }
    if (ur) { CU(c, cudaMemcpyAsync(c->uni_dev[1], ur, (size_t)per * 8, cudaMemcpyHostToDevice, c->stream)); urd = c->uni_dev[1]; }
  }
  return pbg_train_batches(c, bk, (const int64_t *)c->edge_dev[0], (const int64_t *)c->edge_dev[1],
                           rel ? (const int64_t *)c->edge_dev[2] : nullptr, num_edges, batches, num_batches,
                           (const int64_t *)uld, (const int64_t *)urd, seed, stats_out);
}

extern "C" int pbg_set_edge_weights(pbg_context *c, const float *weights_dev) {
  if (!c) return PBG_ERR_BAD_ARGUMENT;
  c->edge_w = weights_dev;
  return PBG_OK;
}

extern "C" int pbg_read_stats(pbg_context *c, pbg_batch_stats *out) {
  if (!c || !out) return PBG_ERR_BAD_ARGUMENT;
  CU(c, cudaSetDevice(c->device));
  double s[5];
  CU(c, cudaMemcpyAsync(s, c->sum_dev, sizeof s, cudaMemcpyDeviceToHost, c->stream));
  CU(c, cudaMemsetAsync(c->sum_dev, 0, sizeof s, c->stream));
  int rc = check_errflag(c);
  out->loss = (float)s[0]; out->reg = (float)s[4];
  out->violators_lhs = (int64_t)(s[1] + 0.5); out->violators_rhs = (int64_t)(s[2] + 0.5); out->count = (int64_t)(s[3] + 0.5);
  return rc;
}

extern "C" int pbg_score_batch(pbg_context *c, const pbg_bucket *bk, const int64_t *lhs, const int64_t *rhs,
                               const int64_t *rel, int32_t count, int32_t relidx, const int64_t *ul,
                               const int64_t *ur, uint64_t seed, float *lhs_pos, float *rhs_pos, float *lhs_neg,
                               float *rhs_neg) {
  if (!c) return PBG_ERR_BAD_ARGUMENT;
  if (count == 0) return PBG_OK;
  if (!lhs || !rhs || !lhs_pos || !rhs_pos || count < 0 || count > c->cfg.max_batch_size)
    return fail(c, PBG_ERR_BAD_ARGUMENT, "bad score_batch arguments (count %d, max_batch_size %d)", count, c->cfg.max_batch_size);
  CU(c, cudaSetDevice(c->device));
  WaveDims d;
  WaveBufs w;
  int rc = bind_bucket(c, bk, d, w);
  if (rc) return rc;
  if (!d.dynamic && (relidx < 0 || relidx >= c->cfg.num_rels)) return fail(c, PBG_ERR_INDEX_RANGE, "relation %d outside [0, %d)", relidx, c->cfg.num_rels);
  if (d.dynamic && d.op != PBG_OP_NONE && !rel) return fail(c, PBG_ERR_BAD_ARGUMENT, "dynamic relations need the rel array");
  if ((d.neg_enabled[0] && !lhs_neg) || (d.neg_enabled[1] && !rhs_neg)) return fail(c, PBG_ERR_BAD_ARGUMENT, "null negative-score output");
  w.lhs = (const long long *)lhs; w.rhs = (const long long *)rhs; w.rel = (const long long *)rel;
  w.ul = (const long long *)ul; w.ur = (const long long *)ur; w.seed = seed;
  WaveBatches wb;
  memset(&wb, 0, sizeof wb);
  wb.n[0] = count; wb.rel[0] = d.dynamic ? 0 : relidx; wb.wrel[0] = 1.0f;
  d.k = 1; d.nblk = d.Cm; d.nocc = d.spb;
  d.blk0 = 0;
  run_forward(c, d, wb, w, c->stream);
  c->launches += launch_export_scores(d, wb, w, lhs_pos, rhs_pos, lhs_neg, rhs_neg, c->stream);
  CU(c, pbg_take_launch_error());
  return check_errflag(c);
}

extern "C" int pbg_eval_batch(pbg_context *c, const pbg_bucket *bk, const int64_t *lhs, const int64_t *rhs,
                              const int64_t *rel, int32_t count, int32_t relidx, const int64_t *ul, const int64_t *ur,
                              uint64_t seed, pbg_eval_stats *out) {
  if (!c || !out) return PBG_ERR_BAD_ARGUMENT;
  memset(out, 0, sizeof *out);
  if (count == 0) return PBG_OK;
  if (!lhs || !rhs || count < 0 || count > c->cfg.max_batch_size)
    return fail(c, PBG_ERR_BAD_ARGUMENT, "bad eval_batch arguments (count %d, max_batch_size %d)", count, c->cfg.max_batch_size);
  CU(c, cudaSetDevice(c->device));
  WaveDims d;
  WaveBufs w;
  int rc = bind_bucket(c, bk, d, w);
  if (rc) return rc;
  if (!d.dynamic && (relidx < 0 || relidx >= c->cfg.num_rels)) return fail(c, PBG_ERR_INDEX_RANGE, "relation %d outside [0, %d)", relidx, c->cfg.num_rels);
  if (d.dynamic && d.op != PBG_OP_NONE && !rel) return fail(c, PBG_ERR_BAD_ARGUMENT, "dynamic relations need the rel array");
  w.lhs = (const long long *)lhs; w.rhs = (const long long *)rhs; w.rel = (const long long *)rel;
  w.ew = c->edge_w; c->edge_w = nullptr;
  w.ul = (const long long *)ul; w.ur = (const long long *)ur; w.seed = seed;
  WaveBatches wb;
  memset(&wb, 0, sizeof wb);
  wb.n[0] = count; wb.rel[0] = d.dynamic ? 0 : relidx;
  wb.wrel[0] = bk->relation_weights ? bk->relation_weights[d.dynamic ? 0 : relidx] : 1.0f;
  d.k = 1; d.nblk = d.Cm; d.nocc = d.spb; d.blk0 = 0;
  run_forward(c, d, wb, w, c->stream);
  c->launches += launch_eval(d, wb, w, c->eval_dev, c->stream);
  CU(c, pbg_take_launch_error());
  double h[8];
  CU(c, cudaMemcpyAsync(h, c->eval_dev, sizeof h, cudaMemcpyDeviceToHost, c->stream));
  rc = check_errflag(c);
  int sides = (d.neg_enabled[0] ? 1 : 0) + (d.neg_enabled[1] ? 1 : 0);
  double div = sides > 0 ? sides : 1;
  // the reference averages the two sides' sums (average_of_sums) and averages the two AUCs
  out->loss = (float)h[0];
  out->pos_rank = h[1] / div; out->mrr = h[2] / div; out->r1 = h[3] / div; out->r10 = h[4] / div; out->r50 = h[5] / div;
  out->auc = sides > 0 ? (h[6] + h[7]) / div : 0.0;          // = count * mean(side AUCs): averaged over count by the caller
  out->count = count;
  return rc;
}

#define PBG_ALLNEGS_SLAB 8192     // candidate rows transformed and scored at a time

extern "C" int pbg_eval_batch_all_negs(pbg_context *c, const pbg_bucket *bk, const int64_t *lhs, const int64_t *rhs,
                                       const int64_t *rel, int32_t count, int32_t relidx, uint64_t seed, pbg_eval_stats *out) {
  if (!c || !out) return PBG_ERR_BAD_ARGUMENT;
  memset(out, 0, sizeof *out);
  if (count == 0) return PBG_OK;
  if (!lhs || !rhs || count < 0 || count > c->cfg.max_batch_size)
    return fail(c, PBG_ERR_BAD_ARGUMENT, "bad eval_batch_all_negs arguments (count %d, max_batch_size %d)", count, c->cfg.max_batch_size);
  CU(c, cudaSetDevice(c->device));
  WaveDims d;
  WaveBufs w;
  int rc = bind_bucket(c, bk, d, w);
  if (rc) return rc;
  if (d.matrix_op) return fail(c, PBG_ERR_UNSUPPORTED, "ranking against all entities has no device code for the linear / affine operators");
  if (!d.dynamic && (relidx < 0 || relidx >= c->cfg.num_rels)) return fail(c, PBG_ERR_INDEX_RANGE, "relation %d outside [0, %d)", relidx, c->cfg.num_rels);
  if (d.dynamic && d.op != PBG_OP_NONE && !rel) return fail(c, PBG_ERR_BAD_ARGUMENT, "dynamic relations need the rel array");
  if (!c->allnegs_mem) CU(c, cudaMalloc(&c->allnegs_mem, pbg_allnegs_bytes(c->cfg.max_batch_size, c->Dp, PBG_ALLNEGS_SLAB)));
  w.lhs = (const long long *)lhs; w.rhs = (const long long *)rhs; w.rel = (const long long *)rel;
  w.ew = c->edge_w; c->edge_w = nullptr;
  w.seed = seed;
  const float wrel = bk->relation_weights ? bk->relation_weights[d.dynamic ? 0 : relidx] : 1.0f;
  c->launches += launch_allnegs_eval(d, w, c->allnegs_mem, count, PBG_ALLNEGS_SLAB, d.dynamic ? 0 : relidx, wrel, c->eval_dev, c->stream);
  CU(c, pbg_take_launch_error());
  double h[8];
  CU(c, cudaMemcpyAsync(h, c->eval_dev, sizeof h, cudaMemcpyDeviceToHost, c->stream));
  rc = check_errflag(c);
  int sides = (d.neg_enabled[0] ? 1 : 0) + (d.neg_enabled[1] ? 1 : 0);
  double div = sides > 0 ? sides : 1;
  out->loss = (float)h[0];
  out->pos_rank = h[1] / div; out->mrr = h[2] / div; out->r1 = h[3] / div; out->r10 = h[4] / div; out->r50 = h[5] / div;
  out->auc = sides > 0 ? (h[6] + h[7]) / div : 0.0;
  out->count = count;
  return rc;
}

extern "C" int pbg_row_adagrad(pbg_context *c, float *emb, float *state, int64_t num_rows, const int64_t *rows,
                               const float *grads, int32_t n, float lr) {
  if (!c) return PBG_ERR_BAD_ARGUMENT;
  if (n == 0) return PBG_OK;
  if (!emb || !state || !rows || !grads || n < 0 || num_rows <= 0) return fail(c, PBG_ERR_BAD_ARGUMENT, "bad row_adagrad arguments");
  SortPlan &sp = c->sort[0];
  if (n > sp.max_n) return fail(c, PBG_ERR_TOO_LARGE, "%d gradient rows exceed this context's sort capacity %d", n, sp.max_n);
  CU(c, cudaSetDevice(c->device));
  c->launches += launch_iota_keys((const long long *)rows, num_rows, n, sp.keys[0], sp.vals[0], c->errflag, c->stream);
  c->launches += pbg_sort(sp, n, bit_length((unsigned long long)num_rows), c->stream);
  c->launches += launch_row_adagrad_sorted(emb, state, c->cfg.dim, sp.keys[sp.result], sp.vals[sp.result],
                                           grads, n, lr, (unsigned long long)num_rows, c->stream);
  CU(c, pbg_take_launch_error());
  return check_errflag(c);
}

// ---- edge-list utilities (torchbiggraph/util.cpp) -------------------------------------------------
static int check_errflag_edges(pbg_context *c, const char *what) {
  int flag = 0;
  CU(c, cudaMemcpyAsync(&flag, c->errflag, sizeof flag, cudaMemcpyDeviceToHost, c->stream));
  CU(c, cudaStreamSynchronize(c->stream));
  if (flag) {
    cudaMemsetAsync(c->errflag, 0, sizeof(int), c->stream);
    if (flag & 4) return fail(c, PBG_ERR_INDEX_RANGE, "%s: rel > numRelations", what);
    return fail(c, PBG_ERR_INDEX_RANGE, "%s: a value lies outside its table; those elements were skipped", what);
  }
  return PBG_OK;
}

// sort scratch for n (key, value) pairs
static int ensure_edge_sort(pbg_context *c, long long n) {
  if (n > 0x7fffffffll) return fail(c, PBG_ERR_TOO_LARGE, "%lld elements are beyond the 2^31 - 1 one call sorts", n);
  if (n <= c->esort.max_n) return PBG_OK;
  if (c->esort_mem) { cudaFree(c->esort_mem); c->esort_mem = nullptr; c->esort.max_n = 0; }
  const long long cap = n + n / 4 + 1024 > 0x7fffffffll ? 0x7fffffffll : n + n / 4 + 1024;
  const size_t kb = align_up((size_t)cap * 8, 256), vb = align_up((size_t)cap * 4, 256);
  const size_t hb = align_up(pbg_sort_hist_entries((int)cap) * 4, 256);
  CU(c, cudaMalloc(&c->esort_mem, 2 * kb + 2 * vb + hb));
  char *p = c->esort_mem;
  c->esort.keys[0] = (unsigned long long *)p; c->esort.keys[1] = (unsigned long long *)(p + kb);
  c->esort.vals[0] = (unsigned int *)(p + 2 * kb); c->esort.vals[1] = (unsigned int *)(p + 2 * kb + vb);
  c->esort.hist = (unsigned int *)(p + 2 * kb + 2 * vb);
  c->esort.max_n = (int)cap;
  return PBG_OK;
}

extern "C" int pbg_reverse_permutation(pbg_context *c, const int64_t *perm, int64_t n, int64_t *out) {
  if (!c) return PBG_ERR_BAD_ARGUMENT;
  if (n == 0) return PBG_OK;
  if (!perm || !out || n < 0) return fail(c, PBG_ERR_BAD_ARGUMENT, "bad reverse_permutation arguments");
  CU(c, cudaSetDevice(c->device));
  c->launches += launch_reverse_permutation((const long long *)perm, n, (long long *)out, c->errflag, c->stream);
  CU(c, pbg_take_launch_error());
  return check_errflag_edges(c, "reverse_permutation");
}

extern "C" int pbg_shuffle_rows(pbg_context *c, const void *in, void *out, int64_t rows, int64_t row_bytes, const int64_t *perm) {
  if (!c) return PBG_ERR_BAD_ARGUMENT;
  if (rows == 0 || row_bytes == 0) return PBG_OK;
  if (!in || !out || !perm || rows < 0 || row_bytes < 0 || in == out) return fail(c, PBG_ERR_BAD_ARGUMENT, "bad shuffle arguments (in and out must be different buffers)");
  CU(c, cudaSetDevice(c->device));
  c->launches += launch_shuffle_rows(in, out, rows, row_bytes, (const long long *)perm, c->errflag, c->stream);
  CU(c, pbg_take_launch_error());
  int rc = check_errflag_edges(c, "shuffle");
  if (rc == PBG_ERR_INDEX_RANGE) c->err = "Permutation has out-of-bound values";      // util.cpp:200-202
  return rc;
}

extern "C" int pbg_randperm(pbg_context *c, int64_t n, uint64_t seed, int64_t *out) {
  if (!c) return PBG_ERR_BAD_ARGUMENT;
  if (n == 0) return PBG_OK;
  if (!out || n < 0) return fail(c, PBG_ERR_BAD_ARGUMENT, "bad randperm arguments");
  CU(c, cudaSetDevice(c->device));
  int rc = ensure_edge_sort(c, n);
  if (rc) return rc;
  c->launches += launch_randperm(c->esort, n, seed, (long long *)out, c->stream);
  CU(c, pbg_take_launch_error());
  CU(c, cudaStreamSynchronize(c->stream));
  return PBG_OK;
}

extern "C" int pbg_sub_bucket(pbg_context *c, const int64_t *lhs_in, const int64_t *rhs_in, const int64_t *rel_in, int64_t num_edges,
                              int32_t num_relations, const int64_t *lhs_entity_counts, const int64_t *const *lhs_perms,
                              const int64_t *rhs_entity_counts, const int64_t *const *rhs_perms, int64_t *lhs_out,
                              int64_t *rhs_out, int64_t *rel_out, int32_t num_lhs_sub_parts, int32_t num_rhs_sub_parts,
                              int32_t dynamic_relations, int64_t *sub_bucket_counts) {
  if (!c) return PBG_ERR_BAD_ARGUMENT;
  const int R = num_relations, nl = num_lhs_sub_parts, nr = num_rhs_sub_parts;
  if (R <= 0 || !lhs_entity_counts || !rhs_entity_counts || !lhs_perms || !rhs_perms || !sub_bucket_counts)
    return fail(c, PBG_ERR_BAD_ARGUMENT, "Inconsistent num_relations");                 // util.cpp:277-281
  if (nl <= 0 || nr <= 0 || nl > 127 || nr > 127) return fail(c, PBG_ERR_BAD_ARGUMENT, "sub-partition counts must be in [1, 127] (int8 in the reference)");
  if (num_edges < 0 || (num_edges > 0 && (!lhs_in || !rhs_in || !rel_in || !lhs_out || !rhs_out || !rel_out)))
    return fail(c, PBG_ERR_BAD_ARGUMENT, "null edge arrays");
  CU(c, cudaSetDevice(c->device));
  int rc = ensure_edge_sort(c, num_edges);
  if (rc) return rc;
  const long long need = 6ll * R + (long long)nl * nr;
  if (need > c->etab_cap) {
    if (c->etab_dev) cudaFree(c->etab_dev);
    c->etab_dev = nullptr;
    CU(c, cudaMalloc(&c->etab_dev, (size_t)(need + 64) * sizeof(long long)));
    c->etab_cap = need + 64;
  }
  std::vector<long long> tab((size_t)need, 0);
  for (int r = 0; r < R; ++r) {
    if (!lhs_perms[r] || !rhs_perms[r] || lhs_entity_counts[r] <= 0 || rhs_entity_counts[r] <= 0)
      return fail(c, PBG_ERR_BAD_ARGUMENT, "relation %d: null permutation or empty entity type", r);
    tab[r] = (long long)(uintptr_t)lhs_perms[r];
    tab[R + r] = (long long)(uintptr_t)rhs_perms[r];
    tab[2 * R + r] = lhs_entity_counts[r];
    tab[3 * R + r] = rhs_entity_counts[r];
    tab[4 * R + r] = (lhs_entity_counts[r] + nl - 1) / nl;                               // util.cpp:296-315
    tab[5 * R + r] = (rhs_entity_counts[r] + nr - 1) / nr;
  }
  CU(c, cudaMemcpyAsync(c->etab_dev, tab.data(), (size_t)6 * R * sizeof(long long), cudaMemcpyHostToDevice, c->stream));
  CU(c, cudaStreamSynchronize(c->stream));                                               // tab is a local: the copy must have left it
  long long *counts_dev = c->etab_dev + 6 * R;
  c->launches += launch_sub_bucket(c->esort, (const long long *)lhs_in, (const long long *)rhs_in, (const long long *)rel_in, num_edges, R,
                                   c->etab_dev, nl, nr, dynamic_relations != 0, (long long *)lhs_out, (long long *)rhs_out,
                                   (long long *)rel_out, counts_dev, c->errflag, c->stream);
  CU(c, pbg_take_launch_error());
  CU(c, cudaMemcpyAsync(sub_bucket_counts, counts_dev, (size_t)nl * nr * sizeof(long long), cudaMemcpyDeviceToHost, c->stream));
  return check_errflag_edges(c, "sub_bucket");
}
