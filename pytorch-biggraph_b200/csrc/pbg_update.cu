// Optimizer steps of one wave.
//
// The sorted occurrence list (pbg_sort.cu) puts all gradient slots of a table row next to each
// other, in batch order.  A warp keeps a row in registers, and for every batch of the wave that
// touched it sums the slots' gradients -- each taken back through comparator.prepare and the
// relation operator on the fly -- and applies one optimizer step:
//   embedding rows  RowAdagrad   G += mean(g^2); w -= lr g / (sqrt(G) + 1e-10)
//                                (torchbiggraph/row_adagrad.py:84-96; duplicates are summed first,
//                                 the `coalesce` of line 83)
//   operator rows   AsyncAdagrad G += g^2 elementwise; theta -= lr_rel g / (sqrt(G) + 1e-10)
//                                (torchbiggraph/async_adagrad.py:75-85)
// A row is read once and written once per wave however many batches touched it, and the
// optimizer state never leaves HBM.  Everything is summed in a fixed order: results are
// reproducible run to run.
#include "pbg_common.cuh"

#define UPD_WARPS 8

// Everything needed to pull one gradient slot back to the embedding row it came from.
// CMPK >= 0 fixes the comparator at compile time, OPK == 0 states that the operator does not scale
// the gradient (none / translation): the kernels instantiated that way carry no dead branches.
template <int VEC, int CMPK = -1, int OPK = -1>
#define REL_UNKNOWN (-(1ll << 62))
struct SlotGrad {
  const float *g, *y;      // gradient row, prepared operand row
  const float *theta;      // operator row or null
  float dotgy, inv, cf;    // cos: <g', y> and 1/|z|; l2 family: coefficient of y
  float rc;                // N3 regularizer weight if the slot is an adjusted positive row, else 0
  bool rcplx;              // ... with the complex modulus (complex_diagonal)
  int op, cmp, D;

  // gstage: the gradient row already staged in shared memory (null: read it from global memory)
  // pre_op: (linear / affine only) stop at the operator output instead of reading the finished
  //         gradient of the raw row from R2
  // rl_known: (dynamic relations) the slot's relation id where the caller has looked it up already (REL_UNKNOWN: look
  //           it up here); reg_known: 1 / 0 = the slot is / is not a regularized row (-1: work it out here)
  __device__ __forceinline__ void init(const WaveDims &d, const WaveBatches &wb, const WaveBufs &w,
                                       int a, int blk, int r, int b, int lane, const float *gstage = nullptr,
                                       bool pre_op = false, long long rl_known = REL_UNKNOWN, int reg_known = -1) {
    D = d.D; op = OPK == 0 ? PBG_OP_NONE : d.op; cmp = CMPK >= 0 ? CMPK : d.cmp;
    size_t xr = (size_t)blk * w.xrows[a] + r, gr = (size_t)blk * w.grows[a] + r;
    y = w.X[a] + xr * d.Dp;
    g = gstage ? gstage : w.GX[a] + gr * d.Dp;
    theta = nullptr;
    cf = 0.f; inv = 1.f; dotgy = 0.f;
    rc = 0.f; rcplx = d.op == PBG_OP_COMPLEX_DIAGONAL;
    if (d.reg_coef != 0.f) {
      // regularized rows: the edges of the chunk (not the uniform negatives) in every operand array
      if (reg_known >= 0) { if (reg_known) rc = d.reg_coef; }
      else {
        BlockInfo rbi = block_info(d, wb, blk);
        if (r < rbi.n && (a >= ARR_Q0 || r < d.Pm)) rc = d.reg_coef;
      }
    }
    if (d.matrix_op) {
      op = PBG_OP_NONE;
      if (a == ARR_N1 && !pre_op) {            // R2 already holds d(loss)/d(raw row)
        if (!gstage) g = w.R2 + gr * d.Dp;
        cmp = PBG_CMP_DOT;
        return;
      }
    }
    if (OPK != 0 && op != PBG_OP_NONE) {
      if (!d.dynamic) {
        if ((a == ARR_N1 || a == ARR_Q0) && w.theta[0]) theta = w.theta[0] + (size_t)wb.rel[b] * D;
      } else if (a == ARR_Q0 || a == ARR_Q1) {
        long long rl = rl_known;
        if (rl == REL_UNKNOWN) {
          BlockInfo bi = block_info(d, wb, blk);
          rl = w.rel[bi.e0 + r];
        }
        const float *tab = w.theta[a == ARR_Q0 ? 0 : 1];
        if (tab && rl >= 0 && rl < d.num_rels) theta = tab + (size_t)rl * D;
      }
    }
    const int cmp = CMPK >= 0 ? CMPK : this->cmp;
    if (cmp >= PBG_CMP_L2) {
      // dynamic: ga = T.N - rowsum(T) a ;  gb = T^T.Q - colsum(T) b.  standard: g = A.N' - rowsum(A) y
      const float *cp = (a == ARR_N0) ? w.coef[0] : (a == ARR_N1) ? w.coef[1] : (a == ARR_Q0) ? w.coef[2] : w.coef[3];
      cf = cp[gr];
    } else if (cmp == PBG_CMP_COS) {
      inv = w.aux[a][xr];
      float s = 0.f;
#pragma unroll
      for (int c = 0; c < VEC; ++c) {
        int dd = c * 128 + lane * 4;
        if (dd < D) s += f4dot(graw(dd), yv(dd));
      }
      dotgy = warp_sum(s);
    }
  }
  __device__ __forceinline__ float4 yv(int dd) const {
    return ld4(y + dd);
  }
  // gradient w.r.t. the operator output z at elements [dd, dd+4)
  // gradient that reaches the prepared row: from the contractions, plus the regularizer's own
  __device__ __forceinline__ float4 graw(int dd) const {
    float4 v = ld4(g + dd);
    if (rc != 0.f) v = v + n3_grad4(y, dd, D, rcplx) * rc;
    return v;
  }
  __device__ __forceinline__ float4 gz(int dd) const {
    float4 v = graw(dd);
    const int cmp = CMPK >= 0 ? CMPK : this->cmp;
    if (cmp >= PBG_CMP_L2) v = v - yv(dd) * cf;
    else if (cmp == PBG_CMP_COS) v = (v - yv(dd) * dotgy) * inv;   // (g - y <g,y>) / |z|
    return v;
  }
  // gradient w.r.t. the embedding row at elements [dd, dd+4)
  __device__ __forceinline__ float4 gx(int dd) const {
    float4 v = gz(dd);
    if (OPK == 0 || theta == nullptr || op == PBG_OP_TRANSLATION) return v;
    float4 t = ld4(theta + dd);
    if (op == PBG_OP_DIAGONAL) return v * t;
    int h = D >> 1;
    int dp = dd < h ? dd + h : dd - h;
    float4 vp = gz(dp), tp = ld4(theta + dp);
    // gx_re = g_re p_re + g_im p_im ;  gx_im = -g_re p_im + g_im p_re
    return dd < h ? v * t + vp * tp : v * tp - vp * t;
  }
};

// d(loss)/d(operator row) contributed by one slot whose operand went through the operator:
// needs the gradient at the operator output (gz) and the raw embedding row x.
template <int VEC, int CMPK = -1>
__device__ __forceinline__ float4 op_param_grad(const SlotGrad<VEC, CMPK, -1> &sg, const float *x, float xscale, int dd,
                                                const float *xadd = nullptr) {
  // xadd: global embedding added to the raw row before the operator (null: none)
  float4 v = sg.gz(dd);
  if (sg.op == PBG_OP_TRANSLATION) return v;
  auto raw = [&](int e) {
    float4 r = ld4(x + e) * xscale;
    if (xadd) r = r + ld4(xadd + e);
    return r;
  };
  float4 xv = raw(dd);
  if (sg.op == PBG_OP_DIAGONAL) return v * xv;
  int h = sg.D >> 1;
  int dp = dd < h ? dd + h : dd - h;
  float4 vp = sg.gz(dp), xp = raw(dp);
  // d real = g_re a_re + g_im a_im ;  d imag = -g_re a_im + g_im a_re
  return dd < h ? v * xv + vp * xp : v * xp - vp * xv;
}

// ------------------------------------------------------------------------------------------------
// Segmented optimizer step over the sorted slot list.
//
// The list is cut into tiles of TILE slots, one warp per tile (after issuing L2 prefetches for the
// gradient and table rows of its slots); the warp reads the keys of slots
// [t0-32, t0+32) and the values of [t0, t0+32) in two coalesced loads and finds segment (= table
// row) boundaries with ballots.
//   * a row with at most SHORT_MAX slots is handled entirely by the warp whose tile holds its first
//     slot: row and state in registers, one optimizer step per batch that touched it;
//   * a longer row (a hub of the graph) is summed tile by tile: every warp writes, for each
//     (batch, tile) run of its slots, one partial gradient row to psum[first slot of the run]; the
//     warp that holds the head registers the row in hublist, and hub_update_kernel finishes it
//     with one CTA per row (eight warps add the partial rows of a batch in a fixed order).
// RULE selects the table and its optimizer: embedding rows / RowAdagrad, or (dynamic relations)
// operator rows / AsyncAdagrad.
// ------------------------------------------------------------------------------------------------
#define TILE 4
#define SHORT_MAX 24
#define HUB_BIG 256     // rows with at least this many slots in a wave get their batches summed by separate CTAs
// hublist holds nocc / 8 + 64 entries; a hub row has more than SHORT_MAX slots, so the rows themselves need fewer than
// nocc / 16 + 32 of them and the list of big rows (at most nocc / HUB_BIG) lives in the rest.  hubcnt[0] counts hub
// rows, hubcnt[1] big rows.
__device__ __forceinline__ long long *hub_biglist(long long *hublist, int nocc) { return hublist + nocc / 16 + 32; }
__device__ __forceinline__ const long long *hub_biglist(const long long *hublist, int nocc) { return hublist + nocc / 16 + 32; }
enum { RULE_EMB = 0, RULE_REL = 1 };

template <int VEC, int RULE>
struct RowState {
  float4 v[VEC], a[VEC];     // row; per-element accumulator (RULE_REL only)
  float G;                   // per-row accumulator (RULE_EMB only)
  float *prow, *pacc;

  // where the row and its optimizer state live
  __device__ __forceinline__ void locate(const WaveDims &d, const WaveBufs &w, unsigned long long key) {
    const int D = d.D;
    if (RULE == RULE_EMB) {
      int side = (!d.shared_table && key >= (unsigned long long)d.n_rows[0]) ? 1 : 0;
      long long row = (long long)(side ? key - (unsigned long long)d.n_rows[0] : key);
      prow = w.W[side] + (size_t)row * D;
      pacc = w.G[side] + row;
    } else {
      unsigned long long rk = key - d.key_rel_base;
      int t = rk >= (unsigned long long)d.num_rels ? 1 : 0;
      long long rl = (long long)(rk - (unsigned long long)t * d.num_rels);
      prow = w.theta[t] + (size_t)rl * D;
      pacc = w.acc[t] + (size_t)rl * D;
    }
  }
  __device__ __forceinline__ void load(const WaveDims &d, const WaveBufs &w, unsigned long long key, int lane) {
    const int D = d.D;
    locate(d, w, key);
    if (RULE == RULE_EMB) G = *pacc;
#pragma unroll
    for (int c = 0; c < VEC; ++c) {
      int dd = c * 128 + lane * 4;
      v[c] = dd < D ? ld4(prow + dd) : f4zero();
      if (RULE == RULE_REL) a[c] = dd < D ? ld4(pacc + dd) : f4zero();
    }
    if (RULE == RULE_EMB && d.max_norm > 0.f) {
      // the lookup of this wave used the row scaled to max_norm (F.embedding(max_norm=...), model.py:57-61;
      // same arithmetic as the gather): the table keeps the scaled row, the optimizer steps start from it
      float ss = 0.f;
#pragma unroll
      for (int c = 0; c < VEC; ++c) ss += f4dot(v[c], v[c]);
      float norm = sqrtf(warp_sum(ss));
      if (norm > d.max_norm) {
        float sc = d.max_norm / (norm + 1e-7f);
#pragma unroll
        for (int c = 0; c < VEC; ++c) v[c] = v[c] * sc;
      }
    }
  }
  // one optimizer step with the summed gradient g of one batch
  __device__ __forceinline__ void step(const float4 (&g)[VEC], float lr, float invD) {
    if (RULE == RULE_EMB) {
      float ss = 0.f;
#pragma unroll
      for (int c = 0; c < VEC; ++c) ss += f4dot(g[c], g[c]);
      ss = warp_sum(ss);
      G += ss * invD;
      float stepv = lr / (sqrtf(G) + PBG_ADAGRAD_EPS);
#pragma unroll
      for (int c = 0; c < VEC; ++c) v[c] = v[c] - g[c] * stepv;
    } else {
#pragma unroll
      for (int c = 0; c < VEC; ++c) {
        a[c] = a[c] + g[c] * g[c];
        v[c].x -= lr * g[c].x / (sqrtf(a[c].x) + PBG_ADAGRAD_EPS);
        v[c].y -= lr * g[c].y / (sqrtf(a[c].y) + PBG_ADAGRAD_EPS);
        v[c].z -= lr * g[c].z / (sqrtf(a[c].z) + PBG_ADAGRAD_EPS);
        v[c].w -= lr * g[c].w / (sqrtf(a[c].w) + PBG_ADAGRAD_EPS);
      }
    }
  }
  // RowAdagrad step of an embedding row whose batch's mean squared gradient is known already
  __device__ __forceinline__ void step_with_norm(const float4 (&g)[VEC], float lr, float mean_sq) {
    G += mean_sq;
    float stepv = lr / (sqrtf(G) + PBG_ADAGRAD_EPS);
#pragma unroll
    for (int c = 0; c < VEC; ++c) v[c] = v[c] - g[c] * stepv;
  }
  __device__ __forceinline__ void store(int D, int lane) {
#pragma unroll
    for (int c = 0; c < VEC; ++c) {
      int dd = c * 128 + lane * 4;
      if (dd < D) { st4(prow + dd, v[c]); if (RULE == RULE_REL) st4(pacc + dd, a[c]); }
    }
    if (RULE == RULE_EMB && lane == 0) *pacc = G;
  }
};

// acc += the contribution of one slot to its row's gradient
template <int VEC, int RULE, int CMPK = -1, int OPK = -1>
__device__ __forceinline__ void add_slot(float4 (&acc)[VEC], const WaveDims &d, const WaveBatches &wb,
                                         const WaveBufs &w, const Occ &oc, int lane, const float *gstage = nullptr,
                                         long long rl_known = REL_UNKNOWN, int reg_known = -1) {
  const int D = d.D;
  if (RULE == RULE_EMB) {
    SlotGrad<VEC, CMPK, OPK> sg;
    sg.init(d, wb, w, oc.a, oc.blk, oc.r, oc.b, lane, gstage, false, rl_known, reg_known);
#pragma unroll
    for (int c = 0; c < VEC; ++c) {
      int dd = c * 128 + lane * 4;
      if (dd < D) acc[c] = acc[c] + sg.gx(dd);
    }
  } else {
    SlotGrad<VEC, CMPK, -1> sg;
    int qa = oc.a == ARR_R0 ? ARR_Q0 : ARR_Q1;             // slot that carried the operator
    int na = oc.a == ARR_R0 ? ARR_N1 : ARR_N0;             // its operator-free copy (raw row)
    sg.init(d, wb, w, qa, oc.blk, oc.r, oc.b, lane, nullptr, false, rl_known, reg_known);
    size_t nrow = (size_t)oc.blk * w.xrows[na] + oc.r;
    const float *x = w.X[na] + nrow * d.Dp;
    float xscale = (CMPK >= 0 ? CMPK : d.cmp) == PBG_CMP_COS ? 1.0f / w.aux[na][nrow] : 1.0f;
#pragma unroll
    for (int c = 0; c < VEC; ++c) {
      int dd = c * 128 + lane * 4;
      if (dd < D) {
        acc[c] = acc[c] + op_param_grad<VEC, CMPK>(sg, x, xscale, dd);
        // N3 regularizer on the edge's own parameter row (still as the wave found it in global memory)
        if (d.reg_coef != 0.f && sg.theta) acc[c] = acc[c] + n3_grad4(sg.theta, dd, D, d.op == PBG_OP_COMPLEX_DIAGONAL) * d.reg_coef;
      }
    }
  }
}

// Embedding rows: 4 warps per CTA, each with TILE row buffers in shared memory that it fills with
// bulk asynchronous copies (cp.async.bulk, completion on the warp's mbarrier): the gradient rows
// of a whole tile are in flight at once instead of one dependent 16-byte-per-lane load at a time.
#define TILE_WARPS_EMB 4
#define UPD_WAIT_LIMIT 4000000

// MODE 1 (plain): the slot's gradient row is already the gradient of the table row (dot comparator, no
// operator or a translation) -- compiled without the comparator / operator pull-back, whose
// predicated-off copies in the unrolled loops cost more issue slots than the additions themselves.
// MODE 2: cos comparator with no operator or a translation, comparator fixed at compile time.
// MODE 3: dot comparator fixed at compile time, any operator (the pull-back through complex_diagonal
// evaluates the comparator's part twice per element).
// MODE 0: everything decided at run time.
// Resident CTAs per SM: rows of up to 256 floats with an operator or a non-trivial comparator are bound by the latency
// of a slot's chain of loads, not by bytes, and gain from twice the warps at the price of a few dozen bytes of spills
// (dimension 200, dynamic complex_diagonal / l2: update 55.8 -> 52.5 ms per 2.16 M edges); the wide rows stay at the
// register count that keeps them spill-free.
template <int VEC, int RULE, int MODE>
__global__ void __launch_bounds__(32 * (RULE == RULE_EMB ? TILE_WARPS_EMB : UPD_WARPS), RULE == RULE_EMB ? (VEC == 2 ? 6 : 3) : (VEC == 2 ? 4 : 2))
tile_update_kernel(WaveDims d, WaveBatches wb, WaveBufs w, const unsigned long long *__restrict__ keys,
                   const unsigned int *__restrict__ vals, float lr, float *__restrict__ psum,
                   long long *__restrict__ hublist, int *__restrict__ hubcnt) {
  constexpr int WARPS = RULE == RULE_EMB ? TILE_WARPS_EMB : UPD_WARPS;
  constexpr bool PLAIN = MODE == 1;
  constexpr bool STAGED = RULE == RULE_EMB || PLAIN;          // (the plain form of the operator rows stages its GR rows too)
  extern __shared__ __align__(128) float stage_all[];        // [WARPS][TILE][Dp] (STAGED only)
  __shared__ __align__(8) unsigned long long sbar[WARPS];
  const unsigned FULL = 0xffffffffu;
  const unsigned long long SENT = ~0ull;
  int lane = threadIdx.x & 31;
  const int wl = threadIdx.x >> 5;
  long long t0 = ((long long)blockIdx.x * WARPS + wl) * TILE;
  if (t0 >= d.nocc) return;
  float *stage = STAGED ? stage_all + (size_t)wl * TILE * d.Dp : nullptr;
  const uint32_t bar = (uint32_t)__cvta_generic_to_shared(&sbar[wl]);
  uint32_t phase = 0;
  int staged_lo = 0, staged_hi = 0;                           // window slots whose rows are in `stage`
  if (STAGED) {
    if (lane == 0) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" :: "r"(bar));
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
  }
  const int D = d.D;
  const float invD = 1.0f / (float)D;
  const unsigned long long lo = RULE == RULE_EMB ? 0ull : d.key_rel_base;
  const unsigned long long hi = RULE == RULE_EMB ? d.key_rel_base : d.key_invalid;
  long long pa = t0 - 32 + lane, pb = t0 + lane;
  unsigned long long kA = pa >= 0 ? keys[pa] : SENT;
  unsigned long long kB = pb < d.nocc ? keys[pb] : SENT;
  unsigned int vB = pb < d.nocc ? vals[pb] : 0u;
  const int bB = (int)(vB / (unsigned int)d.spb);              // batch of this lane's slot
  // Every lane resolves its own slot once -- the integer divisions of the decoding, and with dynamic relations the
  // relation id of the slot's edge (a load that the operator row's address depends on) -- so that the slot-by-slot
  // loop below starts from shuffles instead of redoing both as one dependent chain per slot.
  Occ ocB; ocB.b = bB; ocB.a = 0; ocB.blk = 0; ocB.r = 0;
  long long rlB = REL_UNKNOWN;
  int regB = -1;
  if ((!PLAIN || RULE == RULE_REL) && pb < d.nocc && kB < hi) {
    ocB = occ_decode(d, (int)vB);
    if (!PLAIN && (d.dynamic || d.reg_coef != 0.f)) {
      const int qa = ocB.a == ARR_R0 ? ARR_Q0 : ocB.a == ARR_R1 ? ARR_Q1 : ocB.a;
      BlockInfo bi = block_info(d, wb, ocB.blk);
      if (d.dynamic && d.op != PBG_OP_NONE && (qa == ARR_Q0 || qa == ARR_Q1) && ocB.r < bi.n) rlB = w.rel[bi.e0 + ocB.r];
      regB = (ocB.r < bi.n && (qa >= ARR_Q0 || ocB.r < d.Pm)) ? 1 : 0;
    }
  }
  if (__shfl_sync(FULL, kB, TILE - 1) < lo) return;          // tile holds only the other rule's rows
  // Copies the gradient rows of window slots j0 .. j0+cnt-1 (cnt <= TILE) into the stage buffers and
  // waits for them; the wait is bounded (bit 1 of the error word when it runs out).
  auto stage_rows = [&](int j0, int cnt) {
    __syncwarp();                                            // everyone is done with the old rows
    const int src = j0 + (lane < cnt ? lane : 0);
    Occ oc;
    oc.a = __shfl_sync(FULL, ocB.a, src); oc.blk = __shfl_sync(FULL, ocB.blk, src); oc.r = __shfl_sync(FULL, ocB.r, src);
    unsigned int v = __shfl_sync(FULL, vB, src);
    if (lane == 0) {
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(bar), "r"((uint32_t)(cnt * d.D * 4)) : "memory");
    }
    __syncwarp();
    if (lane < cnt) {
      if (PLAIN && RULE == RULE_EMB) oc = occ_decode(d, (int)v);   // the plain embedding kernel decodes only what it stages
      const float *g;
      if (RULE == RULE_REL) g = w.GR[oc.a == ARR_R1 ? 1 : 0] + ((size_t)oc.blk * d.Pm + oc.r) * d.Dp;
      else {
        const float *gbase = (d.matrix_op && oc.a == ARR_N1) ? w.R2 : w.GX[oc.a];
        g = gbase + ((size_t)oc.blk * w.grows[oc.a] + oc.r) * d.Dp;
      }
      uint32_t dst = (uint32_t)__cvta_generic_to_shared(stage + (size_t)lane * d.Dp);
      asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                   :: "r"(dst), "l"(g), "r"((uint32_t)(d.D * 4)), "r"(bar) : "memory");
    }
    bool done = false;
    for (int it = 0; it < UPD_WAIT_LIMIT && !done; ++it) {
      uint32_t ok;
      asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
                   : "=r"(ok) : "r"(bar), "r"(phase) : "memory");
      done = ok != 0;
    }
    if (!done && lane == 0) atomicOr(w.errflag, 2);
    phase ^= 1u;
    staged_lo = j0; staged_hi = j0 + cnt;
  };
  if (RULE == RULE_EMB) {
    // get the rows this tile will need moving towards L2 before the dependent loads start
#pragma unroll
    for (int i = 0; i < TILE; ++i) {
      unsigned long long key = __shfl_sync(FULL, kB, i);
      if (key >= hi) break;
      int side = (!d.shared_table && key >= (unsigned long long)d.n_rows[0]) ? 1 : 0;
      const float *wr = w.W[side] + (size_t)(side ? key - (unsigned long long)d.n_rows[0] : key) * D;
      for (int f = lane * 32; f < D; f += 1024) asm volatile("prefetch.global.L2 [%0];" :: "l"(wr + f));
    }
    int nvalid = __popc(__ballot_sync(FULL, lane < TILE && kB < hi));
    if (nvalid > 0) stage_rows(0, nvalid);
  } else if (STAGED) {
    // operator rows, plain form: the tile's slots of this rule (they follow the embedding rows' slots in the sorted list)
    const int first = __popc(__ballot_sync(FULL, lane < TILE && kB < lo));
    const int nvalid = __popc(__ballot_sync(FULL, lane < TILE && kB >= lo && kB < hi));
    if (nvalid > 0) stage_rows(first, nvalid);
  }
  int i = 0;
  while (i < TILE) {
    unsigned long long key = __shfl_sync(FULL, kB, i);
    if (key >= hi) return;                                   // sorted: nothing of this rule follows
    if (key < lo) { ++i; continue; }
    unsigned fm = __ballot_sync(FULL, kB == key);
    unsigned rest = ~(fm >> i);
    int run = rest ? __ffs(rest) - 1 : 32 - i;               // slots i .. i+run-1 of the window share the key
    bool hits_end = i + run >= 32;
    int back = 0;
    if (i == 0) back = __clz(~__ballot_sync(FULL, kA == key)); // slots of this row just before the tile
    bool head_here = back == 0;
    bool hub = hits_end || back == 32 || back + run > SHORT_MAX;
    if (!hub && !head_here) { i += run; continue; }          // short row owned by an earlier tile
    int nproc = hub ? (run < TILE - i ? run : TILE - i) : run;
    RowState<VEC, RULE> rs;
    if (!hub) rs.load(d, w, key, lane);
    float4 acc[VEC];
#pragma unroll
    for (int c = 0; c < VEC; ++c) acc[c] = f4zero();
    int cur_b = -1, run_start = 0;
    for (int j = i; j <= i + nproc; ++j) {
      bool in = j < i + nproc;
      Occ oc;
      if (in) {
        oc.b = __shfl_sync(FULL, ocB.b, j);
        if (!PLAIN || RULE == RULE_REL) { oc.a = __shfl_sync(FULL, ocB.a, j); oc.blk = __shfl_sync(FULL, ocB.blk, j); oc.r = __shfl_sync(FULL, ocB.r, j); }
      }
      if (cur_b >= 0 && (!in || oc.b != cur_b)) {             // a batch of this row is complete
        if (hub) {
          float *dst = psum + (size_t)(t0 + run_start) * d.Dp;
#pragma unroll
          for (int c = 0; c < VEC; ++c) {
            int dd = c * 128 + lane * 4;
            if (dd < D) st4(dst + dd, acc[c]);
          }
        } else {
          rs.step(acc, lr, invD);
        }
#pragma unroll
        for (int c = 0; c < VEC; ++c) acc[c] = f4zero();
      }
      if (!in) break;
      if (oc.b != cur_b) { cur_b = oc.b; run_start = j; }
      const float *gs = nullptr;
      if (STAGED) {
        if (j >= staged_hi) {                                 // a short row that runs past the tile
          int left = i + nproc - j;
          stage_rows(j, left < TILE ? left : TILE);
        }
        gs = stage + (size_t)(j - staged_lo) * d.Dp;
      }
      if (PLAIN) {
        // the staged row: the slot's gradient row, or for operator rows the edge's row of GR (dyn_pullback_kernel)
#pragma unroll
        for (int c = 0; c < VEC; ++c) {
          int dd = c * 128 + lane * 4;
          if (dd < D) acc[c] = acc[c] + ld4(gs + dd);
        }
      } else {
        const long long rl = __shfl_sync(FULL, rlB, j);
        const int reg = __shfl_sync(FULL, regB, j);
        if (MODE == 2) add_slot<VEC, RULE, PBG_CMP_COS, 0>(acc, d, wb, w, oc, lane, gs, rl, reg);
        else if (MODE == 3) add_slot<VEC, RULE, PBG_CMP_DOT, -1>(acc, d, wb, w, oc, lane, gs, rl, reg);
        else add_slot<VEC, RULE>(acc, d, wb, w, oc, lane, gs, rl, reg);
      }
    }
    if (!hub) rs.store(D, lane);
    else if (head_here && lane == 0) {
      const long long head = t0 + i;
      hublist[atomicAdd(hubcnt, 1)] = head;
      // a row's slots are contiguous in the sorted list: it has HUB_BIG or more of them exactly when the slot
      // HUB_BIG - 1 places after its head still carries its key; those few rows go on a second list
      if (head + HUB_BIG - 1 < (long long)d.nocc && keys[head + HUB_BIG - 1] == key)
        hub_biglist(hublist, d.nocc)[atomicAdd(hubcnt + 1, 1)] = head;
    }
    i += nproc;
  }
}

// End of the prefix of [lo, hi) on which pred holds (pred must hold on a prefix only).  The whole CTA
// probes blockDim.x evenly spaced positions per round: two rounds for any wave size instead of a
// chain of ~16 dependent loads by one thread.  Every thread returns the same value.
template <class Pred>
__device__ __forceinline__ long long coop_prefix_end(long long lo, long long hi, Pred pred) {
  while (lo < hi) {
    long long stride = (hi - lo + blockDim.x - 1) / blockDim.x;
    long long pos = lo + (long long)threadIdx.x * stride;
    int cnt = __syncthreads_count(pos < hi && pred(pos));
    if (cnt == 0) return lo;
    long long nhi = lo + (long long)cnt * stride;
    lo = lo + (long long)(cnt - 1) * stride + 1;
    if (nhi < hi) hi = nhi;
    if (stride == 1) return hi;
  }
  return hi;
}

// The same for one warp: 32 probes per round.  Every lane returns the same value.
template <class Pred>
__device__ __forceinline__ long long warp_prefix_end(long long lo, long long hi, Pred pred) {
  const int lane = threadIdx.x & 31;
  while (lo < hi) {
    long long stride = (hi - lo + 31) / 32;
    long long pos = lo + (long long)lane * stride;
    int cnt = __popc(__ballot_sync(0xffffffffu, pos < hi && pred(pos)));
    if (cnt == 0) return lo;
    long long nhi = lo + (long long)cnt * stride;
    lo = lo + (long long)(cnt - 1) * stride + 1;
    if (nhi < hi) hi = nhi;
    if (stride == 1) return hi;
  }
  return hi;
}

// The few rows that collect hundreds of slots per wave (the top nodes of a power-law partition)
// would keep one CTA of hub_update_kernel busy long after every other row is done.  One CTA per
// (big row, batch) adds that batch's partial rows up first -- warp w takes runs w, w + 8, ..., the
// eight sums are added in warp order -- and leaves the total in the batch's first partial row, so
// that hub_update_kernel reads one row per batch of a big row.
template <int VEC>
__global__ void __launch_bounds__(32 * UPD_WARPS)
hub_reduce_kernel(WaveDims d, const unsigned long long *__restrict__ keys, const unsigned int *__restrict__ vals,
                  float *__restrict__ psum, const long long *__restrict__ hublist, const int *__restrict__ hubcnt,
                  long long *__restrict__ bigtab) {
  extern __shared__ __align__(16) float part[];              // [UPD_WARPS][VEC * 128]
  const int lane = threadIdx.x & 31, wl = threadIdx.x >> 5;
  const int D = d.D;
  const long long *biglist = hub_biglist(hublist, d.nocc);
  const long long items = (long long)hubcnt[1] * d.k;        // the tile kernel listed the big rows
  for (long long item = blockIdx.x; item < items; item += gridDim.x) {
    const int h = (int)(item / d.k), b = (int)(item % d.k);
    const long long head = biglist[h];
    const unsigned long long key = keys[head];
    const long long end = coop_prefix_end(head + HUB_BIG, (long long)d.nocc, [&](long long pos) { return keys[pos] == key; });
    // where batch b starts and ends inside the row.  hub_update_kernel reads the answers from bigtab[h] ([b] = first
    // slot of batch b or -1, [PBG_KMAX] = end of the row) instead of searching again.  (Both searches in the same
    // rounds, half of the CTA each, measured slower: 14.2 against 11.8 us.)
    const long long q = coop_prefix_end(head, end, [&](long long pos) { return (int)(vals[pos] / (unsigned int)d.spb) < b; });
    const long long eb = coop_prefix_end(q, end, [&](long long pos) { return (int)(vals[pos] / (unsigned int)d.spb) <= b; });
    if (threadIdx.x == 0) {
      bigtab[(size_t)h * (PBG_KMAX + 1) + b] = q < eb ? q : -1;
      if (b == 0) bigtab[(size_t)h * (PBG_KMAX + 1) + PBG_KMAX] = end;
    }
    if (q >= eb) continue;
    const long long ftb = (q / TILE + 1) * TILE;
    const long long nruns = 1 + (eb > ftb ? (eb - 1 - ftb) / TILE + 1 : 0);
    if (nruns == 1) continue;
    float4 acc[VEC];
#pragma unroll
    for (int c = 0; c < VEC; ++c) acc[c] = f4zero();
    // warp w takes runs w, w + 8, ...: four of its partial rows in flight at a time, added in run order
    for (long long r0 = wl; r0 < nruns; r0 += 4 * UPD_WARPS) {
      const float *src[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        long long r = r0 + (long long)u * UPD_WARPS;
        src[u] = r < nruns ? psum + (size_t)(r == 0 ? q : ftb + (r - 1) * TILE) * d.Dp : nullptr;
      }
#pragma unroll
      for (int c = 0; c < VEC; ++c) {
        int dd = c * 128 + lane * 4;
        if (dd < D) {
          float4 v[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) v[u] = src[u] ? ld4(src[u] + dd) : f4zero();
#pragma unroll
          for (int u = 0; u < 4; ++u) acc[c] = acc[c] + v[u];
        }
      }
    }
#pragma unroll
    for (int c = 0; c < VEC; ++c) st4(&part[(size_t)wl * VEC * 128 + c * 128 + lane * 4], acc[c]);
    __syncthreads();
    float *dst = psum + (size_t)q * d.Dp;
    for (int dd = threadIdx.x * 4; dd < D; dd += 4 * blockDim.x) {
      float4 t = ld4(&part[dd]);
#pragma unroll
      for (int u = 1; u < UPD_WARPS; ++u) t = t + ld4(&part[(size_t)u * VEC * 128 + dd]);
      st4(dst + dd, t);
    }
    __syncthreads();
  }
}

// One CTA per hub row.  Its slots [head, end) are in batch order.  One probe per thread over the row's first 256
// slots gives, in a single round of loads, the row's end and where each of its batches starts (rows of 256 and more
// slots: searches); then warp w adds up the partial rows of batches w, w+8, ... (a batch's slots [q, eb) were summed
// by the tile warps in runs that start at q and at every multiple of TILE inside (q, eb)) into tot[batch][] and,
// for embedding rows, takes the batch's squared norm while it has the sum in registers; warp 0 applies the optimizer
// steps in batch order from shared memory.  All sums run in a fixed order.
template <int VEC, int RULE>
__global__ void __launch_bounds__(32 * UPD_WARPS)
hub_update_kernel(WaveDims d, WaveBatches wb, WaveBufs w, const unsigned long long *__restrict__ keys,
                  const unsigned int *__restrict__ vals, float lr, const float *__restrict__ psum,
                  const long long *__restrict__ hublist, const int *__restrict__ hubcnt,
                  const long long *__restrict__ bigtab) {
  static_assert(32 * UPD_WARPS == HUB_BIG, "one probe per thread covers exactly the rows that are not big");
  extern __shared__ __align__(16) float tot[];               // [k][VEC * 128]
  __shared__ long long bstart[PBG_KMAX + 1];
  __shared__ float bnorm[PBG_KMAX];                           // mean squared gradient of a batch (embedding rows)
  __shared__ int sbatch[32 * UPD_WARPS];
  __shared__ unsigned long long skey;
  __shared__ long long bend;
  const int lane = threadIdx.x & 31, wl = threadIdx.x >> 5;
  const int D = d.D;
  const float invD = 1.0f / (float)D;
  const int nh = hubcnt[0], nbig = hubcnt[1];
  const long long *biglist = hub_biglist(hublist, d.nocc);
  // the big rows first (theirs is the longest chain of dependent loads), then the list of all hub rows without them
  for (int item = blockIdx.x; item < nbig + nh; item += gridDim.x) {
    const bool from_big = item < nbig;
    const long long head = from_big ? biglist[item] : hublist[item - nbig];
    const long long p = head + threadIdx.x;
    const unsigned long long kp = p < (long long)d.nocc ? keys[p] : ~0ull;
    const int bp = p < (long long)d.nocc ? (int)(vals[p] / (unsigned int)d.spb) : -1;
    // what hub_reduce_kernel found out about a big row: the starts of its batches and its end, one load each
    long long tabv = -1;
    if (from_big && threadIdx.x <= PBG_KMAX) tabv = bigtab[(size_t)item * (PBG_KMAX + 1) + threadIdx.x];
    if (threadIdx.x == 0) skey = kp;
    for (int i = threadIdx.x; i <= PBG_KMAX; i += blockDim.x) bstart[i] = -1;
    __syncthreads();
    const unsigned long long key = skey;
    const bool in = kp == key;
    sbatch[threadIdx.x] = in ? bp : -1;
    if (wl == 0) {
      // the row these steps start from: on its way to L2 while the sums are made
      RowState<VEC, RULE> where;
      where.locate(d, w, key);
      for (int f = lane * 32; f < D; f += 1024) {
        asm volatile("prefetch.global.L2 [%0];" :: "l"(where.prow + f));
        if (RULE == RULE_REL) asm volatile("prefetch.global.L2 [%0];" :: "l"(where.pacc + f));
      }
    }
    const int cnt = __syncthreads_count(in);                  // slots of the row among the first 256 (they are contiguous)
    const bool big = cnt == (int)blockDim.x;                  // hub_reduce_kernel left one row per batch
    if (big && !from_big) continue;                           // taken from the list of big rows
    long long end = head + cnt;
    if (!big) {
      if (in && (threadIdx.x == 0 || sbatch[threadIdx.x - 1] != bp)) bstart[bp] = p;     // first slot of batch bp
    } else {
      if (threadIdx.x < d.k) bstart[threadIdx.x] = tabv;
      if (threadIdx.x == PBG_KMAX) bend = tabv;
    }
    __syncthreads();
    if (big) end = bend;
    // ---- per-batch totals ----
    for (int bq = wl; bq < d.k; bq += UPD_WARPS) {
      long long q = bstart[bq];
      if (q < 0) continue;
      long long eb = end;
      for (int nb = bq + 1; nb < d.k; ++nb) if (bstart[nb] >= 0) { eb = bstart[nb]; break; }
      long long ftb = (q / TILE + 1) * TILE;
      long long nruns = big ? 1 : 1 + (eb > ftb ? (eb - 1 - ftb) / TILE + 1 : 0);
      float4 acc[VEC];
#pragma unroll
      for (int c = 0; c < VEC; ++c) acc[c] = f4zero();
      // four partial rows in flight at a time; they are still added in run order
      for (long long r0 = 0; r0 < nruns; r0 += 4) {
        const float *src[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          long long r = r0 + u;
          long long start = r == 0 ? q : ftb + (r - 1) * TILE;
          src[u] = r < nruns ? psum + (size_t)start * d.Dp : nullptr;
        }
#pragma unroll
        for (int c = 0; c < VEC; ++c) {
          int dd = c * 128 + lane * 4;
          if (dd < D) {
            float4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) v[u] = src[u] ? ld4(src[u] + dd) : f4zero();
#pragma unroll
            for (int u = 0; u < 4; ++u) acc[c] = acc[c] + v[u];
          }
        }
      }
#pragma unroll
      for (int c = 0; c < VEC; ++c) st4(&tot[(size_t)bq * VEC * 128 + c * 128 + lane * 4], acc[c]);
      if (RULE == RULE_EMB) {
        // the same expression, on the same values, as RowState::step evaluates
        float ss = 0.f;
#pragma unroll
        for (int c = 0; c < VEC; ++c) ss += f4dot(acc[c], acc[c]);
        ss = warp_sum(ss);
        if (lane == 0) bnorm[bq] = ss * invD;
      }
    }
    __syncthreads();
    // ---- optimizer steps in batch order ----
    // Every thread steps four columns of the row through all batches (the batch norms are known, so nothing in a
    // step crosses columns): the same arithmetic per element, in the same order, as one warp stepping whole rows --
    // which took eight times as long, one dependent instruction stream of a lone warp.  (A row that max_norm has to
    // rescale first needs its norm: that case keeps the one-warp form.)
    // With more hub rows than CTAs (a small graph, where every row is one) the kernel is bound by the instructions it
    // executes, not by one row's chain, and the one-warp form executes fewer.
    if ((RULE == RULE_EMB && d.max_norm > 0.f) || nh + nbig > (int)gridDim.x) {
      if (wl == 0) {
        RowState<VEC, RULE> rs;
        rs.load(d, w, key, lane);
        for (int bq = 0; bq < d.k; ++bq) {
          if (bstart[bq] < 0) continue;
          float4 g[VEC];
#pragma unroll
          for (int c = 0; c < VEC; ++c) g[c] = ld4(&tot[(size_t)bq * VEC * 128 + c * 128 + lane * 4]);
          if (RULE == RULE_EMB) rs.step_with_norm(g, lr, bnorm[bq]);
          else rs.step(g, lr, invD);
        }
        rs.store(D, lane);
      }
    } else {
      RowState<VEC, RULE> where;
      where.locate(d, w, key);
      const float G0 = RULE == RULE_EMB ? *where.pacc : 0.f;
      float Gl = G0;
      for (int dd = threadIdx.x * 4; dd < D; dd += 4 * blockDim.x) {
        float4 v = ld4(where.prow + dd), a = f4zero();
        if (RULE == RULE_REL) a = ld4(where.pacc + dd);
        Gl = G0;
        for (int bq = 0; bq < d.k; ++bq) {
          if (bstart[bq] < 0) continue;
          const float4 g = ld4(&tot[(size_t)bq * VEC * 128 + dd]);
          if (RULE == RULE_EMB) {
            Gl += bnorm[bq];
            const float stepv = lr / (sqrtf(Gl) + PBG_ADAGRAD_EPS);
            v = v - g * stepv;
          } else {
            a = a + g * g;
            v.x -= lr * g.x / (sqrtf(a.x) + PBG_ADAGRAD_EPS);
            v.y -= lr * g.y / (sqrtf(a.y) + PBG_ADAGRAD_EPS);
            v.z -= lr * g.z / (sqrtf(a.z) + PBG_ADAGRAD_EPS);
            v.w -= lr * g.w / (sqrtf(a.w) + PBG_ADAGRAD_EPS);
          }
        }
        st4(where.prow + dd, v);
        if (RULE == RULE_REL) st4(where.pacc + dd, a);
      }
      if (RULE == RULE_EMB && threadIdx.x == 0) {
        // (thread 0 owns columns 0..3 of every row, so its Gl went through all batches)
        *where.pacc = Gl;
      }
    }
    __syncthreads();
  }
}

// Standard relations: every rhs row of a batch went through the same operator row.  Stage 1: one
// CTA per chunk sums the parameter gradient of its rows (N1 slots: chunk rows + uniform rows)
// into relpart[b][c][D] (the eight warps added up in shared memory); the raw rows are re-read from the rhs table, which this wave has not
// updated yet.  Stage 2 (relupdate_std_kernel) adds the chunks up and steps theta, batch by batch.
template <int VEC>
__global__ void __launch_bounds__(32 * UPD_WARPS) relgrad_std_kernel(WaveDims d, WaveBatches wb, WaveBufs w) {
  int lane = threadIdx.x & 31, wl = threadIdx.x >> 5;
  int blk = blockIdx.x;
  BlockInfo bi = block_info(d, wb, blk);
  const int D = d.D;
  float4 acc[VEC];
#pragma unroll
  for (int c = 0; c < VEC; ++c) acc[c] = f4zero();
  int items = d.Mm;                                          // the chunk's rhs rows: GN1 slots
  if (bi.n > 0) {
    for (int it = wl; it < items; it += UPD_WARPS) {
      int a = ARR_N1;
      int r = it;
      long long row = slot_row(d, wb, w, bi, 1, r);
      if (row < 0 || row >= d.n_rows[1]) continue;
      SlotGrad<VEC> sg;
      sg.init(d, wb, w, a, blk, r, bi.b, lane);
      const float *x = w.W[1] + (size_t)row * D;
      const float xsc = d.max_norm > 0.f ? w.rscale[(size_t)blk * d.Mm + r] : 1.0f;    // the raw row entered the operator scaled
#pragma unroll
      for (int c = 0; c < VEC; ++c) {
        int dd = c * 128 + lane * 4;
        if (dd < D) acc[c] = acc[c] + op_param_grad<VEC>(sg, x, xsc, dd, w.glob[1]);
      }
    }
  }
  if (d.reg_coef != 0.f && wl == 0 && bi.n > 0) {
    // N3 regularizer on the relation's parameters: sum(params^3) * number of chunks
    // (regularizers.py:88-92), i.e. once per chunk block; theta is still the wave's snapshot here
    const float *th = w.theta[0] + (size_t)wb.rel[bi.b] * D;
#pragma unroll
    for (int c = 0; c < VEC; ++c) {
      int dd = c * 128 + lane * 4;
      if (dd < D) acc[c] = acc[c] + n3_grad4(th, dd, D, d.op == PBG_OP_COMPLEX_DIAGONAL) * d.reg_coef;
    }
  }
  // the eight warps' sums are added in warp order: one partial row per chunk block, so that the
  // single-CTA stage 2 reads Cm rows per batch instead of 8 Cm (its loads are one dependent chain)
  extern __shared__ __align__(16) float wpart_raw[];
  float (*wpart)[VEC * 128] = reinterpret_cast<float (*)[VEC * 128]>(wpart_raw);
#pragma unroll
  for (int c = 0; c < VEC; ++c) st4(&wpart[wl][c * 128 + lane * 4], acc[c]);
  __syncthreads();
  float *out = w.relpart + (size_t)blk * D;
  for (int dd = threadIdx.x * 4; dd < D; dd += 4 * blockDim.x) {
    float4 t = ld4(&wpart[0][dd]);
#pragma unroll
    for (int u = 1; u < UPD_WARPS; ++u) t = t + ld4(&wpart[u][dd]);
    st4(out + dd, t);
  }
}

__global__ void relupdate_std_kernel(WaveDims d, WaveBatches wb, WaveBufs w, float lr) {
  int dd = blockIdx.x * blockDim.x + threadIdx.x;
  if (dd >= d.D) return;
  // The gradient sums of all batches first: these loads do not depend on the steps, and with the
  // batch loop innermost they are all in flight together (one dependent chain of k * Cm loads took
  // 76 us per wave).  Chunks are added in the same order as before.
  float g[PBG_KMAX];
#pragma unroll
  for (int b = 0; b < PBG_KMAX; ++b) g[b] = 0.f;
  for (int c = 0; c < d.Cm; ++c) {
#pragma unroll
    for (int b = 0; b < PBG_KMAX; ++b)
      if (b < d.k) g[b] += w.relpart[((size_t)b * d.Cm + c) * d.D + dd];
  }
  // the steps in batch order; the row of the relation in hand stays in registers
  int cur = -1;
  float a = 0.f, th = 0.f;
#pragma unroll
  for (int b = 0; b < PBG_KMAX; ++b) {
    if (b >= d.k || wb.n[b] <= 0) continue;
    int rl = wb.rel[b];
    if (rl < 0 || rl >= d.num_rels) continue;
    if (rl != cur) {
      if (cur >= 0) { w.acc[0][(size_t)cur * d.D + dd] = a; w.theta[0][(size_t)cur * d.D + dd] = th; }
      cur = rl;
      a = w.acc[0][(size_t)rl * d.D + dd]; th = w.theta[0][(size_t)rl * d.D + dd];
    }
    a += g[b] * g[b];
    th -= lr * g[b] / (sqrtf(a) + PBG_ADAGRAD_EPS);
  }
  if (cur >= 0) { w.acc[0][(size_t)cur * d.D + dd] = a; w.theta[0][(size_t)cur * d.D + dd] = th; }
}

// linear / affine operators: turns GN1 rows (gradient w.r.t. the prepared operand) into the
// gradient w.r.t. the operator output, in place; slots without a row get zeros.  The two
// contractions of launch_matrix_backward read the result.
template <int VEC>
__global__ void __launch_bounds__(32 * UPD_WARPS) gz_rows_kernel(WaveDims d, WaveBatches wb, WaveBufs w) {
  int lane = threadIdx.x & 31;
  long long item = (long long)blockIdx.x * UPD_WARPS + (threadIdx.x >> 5);
  if (item >= (long long)d.nblk * d.Mm) return;
  int lb = (int)(item / d.Mm), r = (int)(item - (long long)lb * d.Mm);
  const int blk = d.blk0 + lb;
  BlockInfo bi = block_info(d, wb, blk);
  const int D = d.D;
  float *row = w.GX[ARR_N1] + ((size_t)blk * d.Mm + r) * d.Dp;
  long long id = slot_row(d, wb, w, bi, 1, r);
  float4 v[VEC];
  if (id < 0 || id >= d.n_rows[1]) {
#pragma unroll
    for (int c = 0; c < VEC; ++c) v[c] = f4zero();
  } else {
    SlotGrad<VEC> sg;
    sg.init(d, wb, w, ARR_N1, blk, r, bi.b, lane, nullptr, true);
#pragma unroll
    for (int c = 0; c < VEC; ++c) {
      int dd = c * 128 + lane * 4;
      v[c] = dd < D ? sg.gz(dd) : f4zero();
    }
  }
  __syncwarp();
#pragma unroll
  for (int c = 0; c < VEC; ++c) {
    int dd = c * 128 + lane * 4;
    if (dd < D) st4(row + dd, v[c]);
  }
}

int launch_gz_rows(const WaveDims &d, const WaveBatches &wb, const WaveBufs &w, cudaStream_t st) {
  long long items = (long long)d.nblk * d.Mm;
  int ctas = (int)((items + UPD_WARPS - 1) / UPD_WARPS);
  int vec = (d.D + 127) / 128;
#define GZ(V) gz_rows_kernel<V><<<ctas, 32 * UPD_WARPS, 0, st>>>(d, wb, w)
  if (vec <= 1) GZ(1); else if (vec <= 2) GZ(2); else if (vec <= 4) GZ(4); else if (vec <= 8) GZ(8); else GZ(16);
#undef GZ
  return 1;
}

// AsyncAdagrad on the matrix (and translation) of the batch's relation, batch by batch
// (async_adagrad.py:75-85).  dA[b] comes from launch_matrix_backward; the gradient of an affine
// translation is the column sum of the batch's GN1 rows.
__global__ void relupdate_matrix_kernel(WaveDims d, WaveBatches wb, WaveBufs w, float lr) {
  long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= d.opw) return;
  const long long DD = (long long)d.D * d.D;
  for (int b = 0; b < d.k; ++b) {
    if (wb.n[b] <= 0) continue;
    int rl = wb.rel[b];
    if (rl < 0 || rl >= d.num_rels) continue;
    float g;
    if (e < DD) g = w.dA[(size_t)b * d.opw + e];
    else {
      int dd = (int)(e - DD);
      g = 0.f;
      const float *rows = w.GX[ARR_N1] + (size_t)b * d.Cm * d.Mm * d.Dp + dd;
      for (int r = 0; r < d.Cm * d.Mm; ++r) g += rows[(size_t)r * d.Dp];
    }
    size_t idx = (size_t)rl * d.opw + e;
    float a = w.acc[0][idx] + g * g;
    w.acc[0][idx] = a;
    w.theta[0][idx] -= lr * g / (sqrtf(a) + PBG_ADAGRAD_EPS);
  }
}

// Global embeddings (config.global_emb): the vector of an entity type is added to every row of that
// type before the operator, so its gradient is the sum of the row gradients of all slots of its
// side(s).  Stage 1: one CTA per chunk block, warp w sums the slots w, w + 8, ... of the lhs and of
// the rhs operand array, the eight sums are added in warp order into globpart[blk][side][D]; stage 2
// adds the partial sums of a batch
// in a fixed order and applies the dense AsyncAdagrad step, batch after batch
// (torchbiggraph/async_adagrad.py:75-85; the vector is one of model.parameters(), train_cpu.py:215-230).
template <int VEC>
__global__ void __launch_bounds__(32 * UPD_WARPS) globgrad_kernel(WaveDims d, WaveBatches wb, WaveBufs w) {
  extern __shared__ __align__(16) float wpart_raw[];
  float (*wpart)[VEC * 128] = reinterpret_cast<float (*)[VEC * 128]>(wpart_raw);
  int lane = threadIdx.x & 31, wl = threadIdx.x >> 5;
  int blk = blockIdx.x;
  BlockInfo bi = block_info(d, wb, blk);
  const int D = d.D;
#pragma unroll 1
  for (int side = 0; side < 2; ++side) {
    float4 acc[VEC];
#pragma unroll
    for (int c = 0; c < VEC; ++c) acc[c] = f4zero();
    if (bi.n > 0 && w.glob[side]) {
      for (int r = wl; r < d.Mm; r += UPD_WARPS) {
        long long row = slot_row(d, wb, w, bi, side, r);
        if (row < 0 || row >= d.n_rows[side]) continue;
        SlotGrad<VEC> sg;
        sg.init(d, wb, w, side == 0 ? ARR_N0 : ARR_N1, blk, r, bi.b, lane);
#pragma unroll
        for (int c = 0; c < VEC; ++c) {
          int dd = c * 128 + lane * 4;
          if (dd < D) acc[c] = acc[c] + sg.gx(dd);
        }
      }
    }
    __syncthreads();                                   // wpart of the previous side has been read
#pragma unroll
    for (int c = 0; c < VEC; ++c) st4(&wpart[wl][c * 128 + lane * 4], acc[c]);
    __syncthreads();
    float *out = w.globpart + ((size_t)blk * 2 + side) * D;
    for (int dd = threadIdx.x * 4; dd < D; dd += 4 * blockDim.x) {
      float4 t = ld4(&wpart[0][dd]);
#pragma unroll
      for (int u = 1; u < UPD_WARPS; ++u) t = t + ld4(&wpart[u][dd]);
      st4(out + dd, t);
    }
  }
}

__global__ void globupdate_kernel(WaveDims d, WaveBatches wb, WaveBufs w, float lr) {
  int dd = blockIdx.x * blockDim.x + threadIdx.x;
  if (dd >= d.D) return;
  // gradient sums of all batches first (independent loads, all in flight), then the steps in batch order
  float g0[PBG_KMAX], g1[PBG_KMAX];
#pragma unroll
  for (int b = 0; b < PBG_KMAX; ++b) { g0[b] = 0.f; g1[b] = 0.f; }
  for (int c = 0; c < d.Cm; ++c) {
#pragma unroll
    for (int b = 0; b < PBG_KMAX; ++b) {
      if (b < d.k) {
        const float *part = w.globpart + (((size_t)b * d.Cm + c) * 2) * d.D + dd;
        if (w.glob[0]) g0[b] += part[0];
        if (w.glob[1]) g1[b] += part[d.D];
      }
    }
  }
  const bool two = !w.glob_shared && w.glob[1] != nullptr;       // a second vector of its own
  const bool one = w.glob[0] != nullptr;
  float a0 = 0.f, v0 = 0.f, a1 = 0.f, v1 = 0.f;
  if (one) { a0 = w.gacc[0][dd]; v0 = w.glob[0][dd]; }
  if (two) { a1 = w.gacc[1][dd]; v1 = w.glob[1][dd]; }
#pragma unroll
  for (int b = 0; b < PBG_KMAX; ++b) {
    if (b >= d.k || wb.n[b] <= 0) continue;
    float gs0 = g0[b], gs1 = g1[b];
    if (w.glob_shared) { gs0 += gs1; gs1 = 0.f; }
    if (one) { a0 += gs0 * gs0; v0 -= lr * gs0 / (sqrtf(a0) + PBG_ADAGRAD_EPS); }
    if (two) { a1 += gs1 * gs1; v1 -= lr * gs1 / (sqrtf(a1) + PBG_ADAGRAD_EPS); }
  }
  if (one) { w.gacc[0][dd] = a0; w.glob[0][dd] = v0; }
  if (two) { w.gacc[1][dd] = a1; w.glob[1][dd] = v1; }
}

int launch_matrix_update(const WaveDims &d, const WaveBatches &wb, const WaveBufs &w, float lr, cudaStream_t st) {
  relupdate_matrix_kernel<<<(d.opw + 255) / 256, 256, 0, st>>>(d, wb, w, lr);
  return 1;
}

// Standard relations under the cos comparator with no operator or a translation: the pull-back of a slot's gradient
// through the normalisation, g <- (g - y <g, y>) / |z|, needs nothing but the slot's own rows.  Done here for all
// slots at once, one warp per slot, in place -- the same expression SlotGrad::gz evaluates -- it leaves the sorted,
// row-by-row update kernel nothing to do per slot but add (its plain form), instead of a dot product, a warp reduction
// and two more row reads inside that kernel's chain of dependent steps.
template <int VEC>
__global__ void __launch_bounds__(32 * UPD_WARPS) cos_pullback_kernel(WaveDims d, WaveBatches wb, WaveBufs w) {
  const int lane = threadIdx.x & 31;
  long long item = (long long)blockIdx.x * UPD_WARPS + (threadIdx.x >> 5);
  const long long per_side = (long long)d.nblk * d.Mm;
  if (item >= 2 * per_side) return;
  const int side = item >= per_side ? 1 : 0;
  item -= (long long)side * per_side;
  const int lb = (int)(item / d.Mm), r = (int)(item - (long long)lb * d.Mm);
  const int blk = d.blk0 + lb;
  BlockInfo bi = block_info(d, wb, blk);
  if (bi.n <= 0) return;
  const long long id = slot_row(d, wb, w, bi, side, r);
  if (id < 0 || id >= d.n_rows[side]) return;
  const int a = side ? ARR_N1 : ARR_N0;
  SlotGrad<VEC, PBG_CMP_COS, 0> sg;
  sg.init(d, wb, w, a, blk, r, bi.b, lane);
  float4 v[VEC];
#pragma unroll
  for (int c = 0; c < VEC; ++c) {
    int dd = c * 128 + lane * 4;
    v[c] = dd < d.D ? sg.gz(dd) : f4zero();
  }
  __syncwarp();
  float *row = w.GX[a] + ((size_t)blk * w.grows[a] + r) * d.Dp;
#pragma unroll
  for (int c = 0; c < VEC; ++c) {
    int dd = c * 128 + lane * 4;
    if (dd < d.D) st4(row + dd, v[c]);
  }
}

// Dynamic relations with a diagonal, translation or complex_diagonal operator (no regularizer): everything a gradient
// slot contributes is worked out here for all slots at once, one warp per slot -- the gradient of the table row
// (comparator and operator pull-back: SlotGrad::gx) written over the slot's own gradient row, and for the slots that
// went through an operator the gradient of the edge's operator row (op_param_grad) into GR -- so that both sorted,
// row-by-row update kernels run in their plain form (add the slot's row) instead of evaluating ~570 instructions and a
// chain of dependent loads per slot.  The expressions are the ones those kernels evaluated.
template <int VEC>
__global__ void __launch_bounds__(32 * UPD_WARPS, VEC <= 2 ? 4 : 2) dyn_pullback_kernel(WaveDims d, WaveBatches wb, WaveBufs w) {
  const int lane = threadIdx.x & 31;
  long long item = (long long)blockIdx.x * UPD_WARPS + (threadIdx.x >> 5);
  const long long nN = (long long)d.nblk * d.Mm, nQ = (long long)d.nblk * d.Pm;
  if (item >= 2 * nN + 2 * nQ) return;
  int a, rows;
  if (item < nN) { a = ARR_N0; rows = d.Mm; }
  else if ((item -= nN) < nN) { a = ARR_N1; rows = d.Mm; }
  else if ((item -= nN) < nQ) { a = ARR_Q0; rows = d.Pm; }
  else { item -= nQ; a = ARR_Q1; rows = d.Pm; }
  const int lb = (int)(item / rows), r = (int)(item - (long long)lb * rows);
  const int blk = d.blk0 + lb;
  BlockInfo bi = block_info(d, wb, blk);
  if (bi.n <= 0) return;
  // the entity of the slot: N arrays hold lhs / rhs rows (chunk, then uniform), Q0 = op_rhs(rhs), Q1 = op_lhs(lhs)
  const int side = (a == ARR_N0 || a == ARR_Q1) ? 0 : 1;
  if (a >= ARR_Q0 && r >= bi.n) return;
  const long long id = slot_row(d, wb, w, bi, side, r);
  if (id < 0 || id >= d.n_rows[side]) {
    // an entity id outside its table (the call reports it): the edge's operator-row slot may still be a valid one
    // (its key depends on the relation id only), so it gets a zero gradient rather than whatever the row held
    if (a >= ARR_Q0 && w.GR[a - ARR_Q0]) {
      float *prow0 = w.GR[a - ARR_Q0] + ((size_t)blk * d.Pm + r) * d.Dp;
      for (int dd = lane * 4; dd < d.D; dd += 128) st4(prow0 + dd, f4zero());
    }
    return;
  }
  SlotGrad<VEC> sg;
  sg.init(d, wb, w, a, blk, r, bi.b, lane);
  const int D = d.D;
  float4 gxv[VEC], pg[VEC];
  const bool param = a >= ARR_Q0 && sg.theta != nullptr;
#pragma unroll
  for (int c = 0; c < VEC; ++c) {
    int dd = c * 128 + lane * 4;
    gxv[c] = dd < D ? sg.gx(dd) : f4zero();
    pg[c] = f4zero();
  }
  if (param) {
    const int na = a == ARR_Q0 ? ARR_N1 : ARR_N0;              // the slot's operator-free copy (prepared raw row)
    const size_t nrow = (size_t)blk * w.xrows[na] + r;
    const float *x = w.X[na] + nrow * d.Dp;
    const float xscale = d.cmp == PBG_CMP_COS ? 1.0f / w.aux[na][nrow] : 1.0f;
#pragma unroll
    for (int c = 0; c < VEC; ++c) {
      int dd = c * 128 + lane * 4;
      if (dd < D) pg[c] = op_param_grad<VEC>(sg, x, xscale, dd);
    }
  }
  __syncwarp();
  float *row = w.GX[a] + ((size_t)blk * w.grows[a] + r) * d.Dp;
  float *prow = a >= ARR_Q0 ? w.GR[a - ARR_Q0] + ((size_t)blk * d.Pm + r) * d.Dp : nullptr;
#pragma unroll
  for (int c = 0; c < VEC; ++c) {
    int dd = c * 128 + lane * 4;
    if (dd < D) {
      st4(row + dd, gxv[c]);
      if (param) st4(prow + dd, pg[c]);
    }
  }
}

struct UpdateScratch { float *psum; long long *hublist; int *hubcnt; long long *bigtab; cudaStream_t side; cudaEvent_t fork, join; };

template <int VEC>
static int launch_update_vec(const WaveDims &d_in, const WaveBatches &wb, const WaveBufs &w,
                             const unsigned long long *keys, const unsigned int *vals, float lr, float rel_lr,
                             const UpdateScratch &us, cudaStream_t st) {
  WaveDims d = d_in;            // (the comparator becomes dot once the cos pull-back has been applied to all slots, below)
  int launches = 0;
  long long warps = ((long long)d.nocc + TILE - 1) / TILE;
  int ctas = (int)((warps + UPD_WARPS - 1) / UPD_WARPS);
  int ctas_emb = (int)((warps + TILE_WARPS_EMB - 1) / TILE_WARPS_EMB);
  size_t stage_smem = (size_t)TILE_WARPS_EMB * TILE * d.Dp * sizeof(float);
  const int hub_ctas = 296;     // (two and four times as many measured the same: the kernels take as long as their longest row)
  size_t hub_smem = (size_t)d.k * VEC * 128 * sizeof(float);            // per-batch totals of one hub row
  size_t red_smem = (size_t)UPD_WARPS * VEC * 128 * sizeof(float);       // eight partial sums of one batch of a big row
  // the attribute is set once for the largest wave this row width allows in 227 KB
  size_t hub_smem_max = (size_t)PBG_KMAX * VEC * 128 * sizeof(float);
  if (hub_smem_max > 227 * 1024) hub_smem_max = 227 * 1024;
  // per device (a process may hold contexts on several GPUs); a failed opt-in makes the launch fail,
  // which the caller's cudaGetLastError reports
  const int tile_smem_max = (int)((size_t)TILE_WARPS_EMB * TILE * VEC * 128 * sizeof(float));
  pbg_opt_in_smem((const void *)hub_update_kernel<VEC, RULE_EMB>, (int)hub_smem_max);
  pbg_opt_in_smem((const void *)hub_reduce_kernel<VEC>, (int)red_smem);
  pbg_opt_in_smem((const void *)relgrad_std_kernel<VEC>, (int)red_smem);
  pbg_opt_in_smem((const void *)globgrad_kernel<VEC>, (int)red_smem);
  pbg_opt_in_smem((const void *)tile_update_kernel<VEC, RULE_EMB, 0>, tile_smem_max);
  pbg_opt_in_smem((const void *)tile_update_kernel<VEC, RULE_EMB, 1>, tile_smem_max);
  pbg_opt_in_smem((const void *)tile_update_kernel<VEC, RULE_EMB, 2>, tile_smem_max);
  pbg_opt_in_smem((const void *)tile_update_kernel<VEC, RULE_EMB, 3>, tile_smem_max);
  bool has_op = d.op != PBG_OP_NONE && w.theta[0] != nullptr;
  const bool has_glob = w.glob[0] || w.glob[1];
  // Standard relations under a translation: the operator row's two kernels (one CTA per chunk block, then ONE CTA that
  // steps the row batch after batch: 35 + 37 us of latency per wave at dimension 100) touch nothing the embedding
  // rows' kernels read or write -- the pull-back through a translation is the identity and its parameter gradient
  // is the sum of the rhs rows' gradients -- so they run on a side stream beside them.
  const bool cos_first = !d.dynamic && d.cmp == PBG_CMP_COS && !d.matrix_op && d.reg_coef == 0.f && !has_glob &&
                         (d.op == PBG_OP_NONE || d.op == PBG_OP_TRANSLATION);
  if (cos_first) {
    const long long rows2 = 2ll * d.nblk * d.Mm;
    cos_pullback_kernel<VEC><<<(unsigned)((rows2 + UPD_WARPS - 1) / UPD_WARPS), 32 * UPD_WARPS, 0, st>>>(d_in, wb, w);
    ++launches;
    d.cmp = PBG_CMP_DOT;        // what the gradient slots hold now is the gradient of the operator's output
  }
  // (rows of more than 1024 floats keep the per-slot form: the staging buffers of the plain operator-row kernel would
  // not fit in shared memory)
  const bool dyn_first = d.dynamic && has_op && !d.matrix_op && d.reg_coef == 0.f && !has_glob && w.GR[0] != nullptr && VEC <= 8;
  if (dyn_first) {
    const long long rows4 = 2ll * d.nblk * d.Mm + 2ll * d.nblk * d.Pm;
    dyn_pullback_kernel<VEC><<<(unsigned)((rows4 + UPD_WARPS - 1) / UPD_WARPS), 32 * UPD_WARPS, 0, st>>>(d_in, wb, w);
    ++launches;
    d.cmp = PBG_CMP_DOT;        // the gradient slots hold the gradients of the table rows now
  }
  const bool rel_side = has_op && !d.dynamic && !d.matrix_op && d.op == PBG_OP_TRANSLATION && !has_glob && us.side != nullptr;
  if (has_op && !d.dynamic && !d.matrix_op) {
    if (rel_side) {
      cudaEventRecord(us.fork, st);
      cudaStreamWaitEvent(us.side, us.fork, 0);
      relgrad_std_kernel<VEC><<<d.nblk, 32 * UPD_WARPS, red_smem, us.side>>>(d, wb, w);
      relupdate_std_kernel<<<(d.D + 127) / 128, 128, 0, us.side>>>(d, wb, w, rel_lr);
      cudaEventRecord(us.join, us.side);
      launches += 2;
    } else {
      relgrad_std_kernel<VEC><<<d.nblk, 32 * UPD_WARPS, red_smem, st>>>(d, wb, w);
      ++launches;
    }
  }
  // gradient sums of the global embeddings: before any operator parameter of this wave is stepped
  if (has_glob) {
    globgrad_kernel<VEC><<<d.nblk, 32 * UPD_WARPS, red_smem, st>>>(d, wb, w);
    ++launches;
  }
  cudaMemsetAsync(us.hubcnt, 0, 2 * sizeof(int), st);
  // the gradient slot is the row's gradient as it stands: dot comparator, and no operator or a translation
  const bool plain = dyn_first || (d.cmp == PBG_CMP_DOT && !d.matrix_op && d.reg_coef == 0.f && (d.op == PBG_OP_NONE || d.op == PBG_OP_TRANSLATION));
  if (plain) tile_update_kernel<VEC, RULE_EMB, 1><<<ctas_emb, 32 * TILE_WARPS_EMB, stage_smem, st>>>(d, wb, w, keys, vals, lr, us.psum, us.hublist, us.hubcnt);
  else if (d.cmp == PBG_CMP_COS && !d.matrix_op && d.reg_coef == 0.f && (d.op == PBG_OP_NONE || d.op == PBG_OP_TRANSLATION))
    tile_update_kernel<VEC, RULE_EMB, 2><<<ctas_emb, 32 * TILE_WARPS_EMB, stage_smem, st>>>(d, wb, w, keys, vals, lr, us.psum, us.hublist, us.hubcnt);
  else if (d.cmp == PBG_CMP_DOT && !d.matrix_op && d.reg_coef == 0.f)
    tile_update_kernel<VEC, RULE_EMB, 3><<<ctas_emb, 32 * TILE_WARPS_EMB, stage_smem, st>>>(d, wb, w, keys, vals, lr, us.psum, us.hublist, us.hubcnt);
  else tile_update_kernel<VEC, RULE_EMB, 0><<<ctas_emb, 32 * TILE_WARPS_EMB, stage_smem, st>>>(d, wb, w, keys, vals, lr, us.psum, us.hublist, us.hubcnt);
  hub_reduce_kernel<VEC><<<2 * hub_ctas, 32 * UPD_WARPS, red_smem, st>>>(d, keys, vals, us.psum, us.hublist, us.hubcnt, us.bigtab);
  hub_update_kernel<VEC, RULE_EMB><<<hub_ctas, 32 * UPD_WARPS, hub_smem, st>>>(d, wb, w, keys, vals, lr, us.psum, us.hublist, us.hubcnt, us.bigtab);
  ++launches;
  launches += 2;
  if (has_op) {
    if (d.dynamic) {
      pbg_opt_in_smem((const void *)hub_update_kernel<VEC, RULE_REL>, (int)hub_smem_max);
      cudaMemsetAsync(us.hubcnt, 0, 2 * sizeof(int), st);
      if (dyn_first) {
        const size_t rel_smem = (size_t)UPD_WARPS * TILE * d.Dp * sizeof(float);
        pbg_opt_in_smem((const void *)tile_update_kernel<VEC, RULE_REL, 1>, (int)((size_t)UPD_WARPS * TILE * VEC * 128 * sizeof(float)));
        tile_update_kernel<VEC, RULE_REL, 1><<<ctas, 32 * UPD_WARPS, rel_smem, st>>>(d, wb, w, keys, vals, rel_lr, us.psum, us.hublist, us.hubcnt);
      }
      else if (d.cmp == PBG_CMP_DOT && d.reg_coef == 0.f)
        tile_update_kernel<VEC, RULE_REL, 3><<<ctas, 32 * UPD_WARPS, 0, st>>>(d, wb, w, keys, vals, rel_lr, us.psum, us.hublist, us.hubcnt);
      else
        tile_update_kernel<VEC, RULE_REL, 0><<<ctas, 32 * UPD_WARPS, 0, st>>>(d, wb, w, keys, vals, rel_lr, us.psum, us.hublist, us.hubcnt);
      hub_reduce_kernel<VEC><<<2 * hub_ctas, 32 * UPD_WARPS, red_smem, st>>>(d, keys, vals, us.psum, us.hublist, us.hubcnt, us.bigtab);
      hub_update_kernel<VEC, RULE_REL><<<hub_ctas, 32 * UPD_WARPS, hub_smem, st>>>(d, wb, w, keys, vals, rel_lr, us.psum, us.hublist, us.hubcnt, us.bigtab);
      ++launches;
      launches += 2;
    } else if (d.matrix_op) {
      launches += launch_matrix_update(d, wb, w, rel_lr, st);
    } else if (rel_side) {
      cudaStreamWaitEvent(st, us.join, 0);
    } else {
      relupdate_std_kernel<<<(d.D + 127) / 128, 128, 0, st>>>(d, wb, w, rel_lr);
      ++launches;
    }
  }
  if (has_glob) {
    globupdate_kernel<<<(d.D + 127) / 128, 128, 0, st>>>(d, wb, w, rel_lr);
    ++launches;
  }
  pbg_note_launch();
  return launches;
}

int launch_update(const WaveDims &d, const WaveBatches &wb, const WaveBufs &w, const unsigned long long *keys,
                  const unsigned int *vals, float lr, float rel_lr, float *psum, long long *hublist, int *hubcnt,
                  long long *bigtab, cudaStream_t st, cudaStream_t side, cudaEvent_t fork, cudaEvent_t join) {
  UpdateScratch us{psum, hublist, hubcnt, bigtab, side, fork, join};
  int vec = (d.D + 127) / 128;
  if (vec <= 1) return launch_update_vec<1>(d, wb, w, keys, vals, lr, rel_lr, us, st);
  if (vec <= 2) return launch_update_vec<2>(d, wb, w, keys, vals, lr, rel_lr, us, st);
  if (vec <= 4) return launch_update_vec<4>(d, wb, w, keys, vals, lr, rel_lr, us, st);
  if (vec <= 8) return launch_update_vec<8>(d, wb, w, keys, vals, lr, rel_lr, us, st);
  return launch_update_vec<16>(d, wb, w, keys, vals, lr, rel_lr, us, st);
}

// Stand-alone sparse RowAdagrad step (row_adagrad.py:80-96): rows sorted with duplicates adjacent,
// vals[q] = index of the gradient row.
template <int VEC>
__global__ void __launch_bounds__(32 * UPD_WARPS)
row_adagrad_sorted_kernel(float *emb, float *state, int D, const unsigned long long *__restrict__ keys,
                          const unsigned int *__restrict__ vals, const float *__restrict__ grads, int n,
                          float lr, unsigned long long key_invalid) {
  int lane = threadIdx.x & 31;
  long long pos = (long long)blockIdx.x * UPD_WARPS + (threadIdx.x >> 5);
  if (pos >= n) return;
  unsigned long long key = keys[pos];
  if (key >= key_invalid) return;
  if (pos > 0 && keys[pos - 1] == key) return;
  float4 acc[VEC];
#pragma unroll
  for (int c = 0; c < VEC; ++c) acc[c] = f4zero();
  for (long long q = pos; q < n && keys[q] == key; ++q) {
    const float *g = grads + (size_t)vals[q] * D;
#pragma unroll
    for (int c = 0; c < VEC; ++c) {
      int dd = c * 128 + lane * 4;
      if (dd < D) acc[c] = acc[c] + ld4(g + dd);
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < VEC; ++c) ss += f4dot(acc[c], acc[c]);
  ss = warp_sum(ss);
  float G = state[key] + ss / (float)D;
  float stepv = lr / (sqrtf(G) + PBG_ADAGRAD_EPS);
  float *wrow = emb + (size_t)key * D;
#pragma unroll
  for (int c = 0; c < VEC; ++c) {
    int dd = c * 128 + lane * 4;
    if (dd < D) st4(wrow + dd, ld4(wrow + dd) - acc[c] * stepv);
  }
  if (lane == 0) state[key] = G;
}

int launch_row_adagrad_sorted(float *emb, float *state, int dim, const unsigned long long *keys,
                              const unsigned int *vals, const float *grads, int n, float lr,
                              unsigned long long key_invalid, cudaStream_t st) {
  int ctas = (n + UPD_WARPS - 1) / UPD_WARPS;
  int vec = (dim + 127) / 128;
#define RA(V) row_adagrad_sorted_kernel<V><<<ctas, 32 * UPD_WARPS, 0, st>>>(emb, state, dim, keys, vals, grads, n, lr, key_invalid)
  if (vec <= 1) RA(1); else if (vec <= 2) RA(2); else if (vec <= 4) RA(4); else if (vec <= 8) RA(8); else RA(16);
#undef RA
  return 1;
}
