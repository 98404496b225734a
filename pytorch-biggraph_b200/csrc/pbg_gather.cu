// Row gather fused with the relation operator and comparator.prepare: builds the operand tiles
// of one wave (see pbg_common.cuh for the layout) straight from the embedding tables, one warp
// per row slot, 16-byte loads and stores.  Replaces, for a whole wave at once,
//   F.embedding gathers                 torchbiggraph/model.py:57-61, 645-646
//   sample_entities                     torchbiggraph/model.py:70-75
//   adjust_embs (operator + prepare)    torchbiggraph/model.py:478-506, operators.py:49-157, 197-338
//   zero padding of the last chunk      torchbiggraph/model.py:787-800
//   the positive scores                 torchbiggraph/model.py:177, 267-274
// and emits the sort keys that group gradient slots by table row.
#include "pbg_common.cuh"

#define GATHER_WARPS 8

template <int VEC>
__device__ __forceinline__ void load_row(float4 (&v)[VEC], const float *row, int D, int lane) {
#pragma unroll
  for (int c = 0; c < VEC; ++c) {
    int d = c * 128 + lane * 4;
    v[c] = d < D ? ld4(row + d) : f4zero();
  }
}
// F.embedding(max_norm=...) (torchbiggraph/model.py:57-61): a looked-up row whose 2-norm exceeds
// max_norm is used scaled by max_norm / (norm + 1e-7).  Here the scale is applied in registers and
// returned; the table itself is rewritten by the update kernel, which owns each touched row alone
// (RowState::load applies the same scale before the optimizer steps) -- rewriting it from the gather
// would let the duplicates of a row read it half-scaled.
template <int VEC>
__device__ __forceinline__ float renorm_row(float4 (&v)[VEC], float max_norm) {
  if (max_norm <= 0.f) return 1.0f;
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < VEC; ++c) ss += f4dot(v[c], v[c]);
  float norm = sqrtf(warp_sum(ss));
  if (!(norm > max_norm)) return 1.0f;
  float sc = max_norm / (norm + 1e-7f);
#pragma unroll
  for (int c = 0; c < VEC; ++c) v[c] = v[c] * sc;
  return sc;
}
// row += the global embedding of the row's entity type (config.global_emb; model.py:486-492), if any
template <int VEC>
__device__ __forceinline__ void add_global(float4 (&v)[VEC], const float *glob, int D, int lane) {
  if (!glob) return;
#pragma unroll
  for (int c = 0; c < VEC; ++c) {
    int d = c * 128 + lane * 4;
    if (d < D) v[c] = v[c] + ld4(glob + d);
  }
}
template <int VEC>
__device__ __forceinline__ void store_row(float *row, const float4 (&v)[VEC], int D, int lane) {
#pragma unroll
  for (int c = 0; c < VEC; ++c) {
    int d = c * 128 + lane * 4;
    if (d < D) st4(row + d, v[c]);
  }
}
template <int VEC>
__device__ __forceinline__ void put_row(float *base, size_t off, const float4 (&v)[VEC], int D, int lane) {
  store_row<VEC>(base + off, v, D, lane);
}
// bf16-plane tier: the three planes of operand row r of block blk in array a
template <int VEC>
__device__ __forceinline__ void put_row_planes(const WaveBufs &w, int a, int blk, int r, const float4 (&v)[VEC], int D, int lane) {
  const size_t plane = (size_t)w.xrows[a] * w.Dpb;
  unsigned short *x = w.XB[a] + ((size_t)blk * w.npl * w.xrows[a] + r) * w.Dpb;
  const bool three = w.npl > 2;
#pragma unroll
  for (int c = 0; c < VEC; ++c) {
    int dd = c * 128 + lane * 4;
    if (dd < D) {
      uint2 p0, p1, p2;
      bf16_planes4(v[c], p0, p1, p2);
      *(uint2 *)(x + dd) = p0; *(uint2 *)(x + plane + dd) = p1;
      if (three) *(uint2 *)(x + 2 * plane + dd) = p2;
    }
  }
}
template <int VEC>
__device__ __forceinline__ void zero_row_planes(const WaveBufs &w, int a, int blk, int r, int D, int lane) {
  const size_t plane = (size_t)w.xrows[a] * w.Dpb;
  unsigned short *x = w.XB[a] + ((size_t)blk * w.npl * w.xrows[a] + r) * w.Dpb;
  const bool three = w.npl > 2;
#pragma unroll
  for (int c = 0; c < VEC; ++c) {
    int dd = c * 128 + lane * 4;
    if (dd < D) {
      *(uint2 *)(x + dd) = make_uint2(0, 0); *(uint2 *)(x + plane + dd) = make_uint2(0, 0);
      if (three) *(uint2 *)(x + 2 * plane + dd) = make_uint2(0, 0);
    }
  }
}
template <int VEC>
__device__ __forceinline__ void zero_row(float *row, int D, int lane) {
#pragma unroll
  for (int c = 0; c < VEC; ++c) {
    int d = c * 128 + lane * 4;
    if (d < D) st4(row + d, f4zero());
  }
}

// z = op(x; theta).  complex_diagonal pairs element d with d +- D/2, which lives in another
// lane: the partner chunk is re-read from memory (an L1 hit).
template <int VEC>
__device__ __forceinline__ void apply_operator(float4 (&z)[VEC], const float4 (&x)[VEC], const float *xrow,
                                               const float *theta, int op, int D, int lane, const float *glob = nullptr, float rsc = 1.0f) {
  int h = D >> 1;
#pragma unroll
  for (int c = 0; c < VEC; ++c) {
    int d = c * 128 + lane * 4;
    if (d >= D) { z[c] = f4zero(); continue; }
    if (op == PBG_OP_NONE || theta == nullptr) { z[c] = x[c]; continue; }
    float4 t = ld4(theta + d);
    if (op == PBG_OP_DIAGONAL) z[c] = x[c] * t;
    else if (op == PBG_OP_TRANSLATION) z[c] = x[c] + t;
    else {  // complex_diagonal: theta = [real | imag]
      int dp = d < h ? d + h : d - h;
      float4 xp = ld4(xrow + dp) * rsc, tp = ld4(theta + dp);
      if (glob) xp = xp + ld4(glob + dp);
      z[c] = d < h ? x[c] * t - xp * tp      // re = a_re p_re - a_im p_im
                   : xp * t + x[c] * tp;     // im = a_re p_im + a_im p_re
    }
  }
}

// comparator.prepare in place; returns the per-row auxiliary value kept for the later kernels
// (cos: 1/|z|, l2 family: |y|^2, dot: 0).
template <int VEC>
__device__ __forceinline__ float prepare_row(float4 (&z)[VEC], int cmp) {
  if (cmp == PBG_CMP_DOT) return 0.f;
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < VEC; ++c) ss += f4dot(z[c], z[c]);
  ss = warp_sum(ss);
  if (cmp != PBG_CMP_COS) return ss;
  float inv = 1.0f / sqrtf(ss);          // no epsilon: a zero row gives inf/NaN as in model.py:191-192
#pragma unroll
  for (int c = 0; c < VEC; ++c) z[c] = z[c] * inv;
  return inv;
}

template <int VEC>
__device__ __forceinline__ float positive_score(const float4 (&a)[VEC], const float4 (&b)[VEC], int cmp) {
  float s = 0.f;
  if (cmp == PBG_CMP_DOT || cmp == PBG_CMP_COS) {
#pragma unroll
    for (int c = 0; c < VEC; ++c) s += f4dot(a[c], b[c]);
    return warp_sum(s);
  }
#pragma unroll
  for (int c = 0; c < VEC; ++c) { float4 df = a[c] - b[c]; s += f4dot(df, df); }
  s = warp_sum(s);
  return cmp == PBG_CMP_L2 ? -sqrtf(fmaxf(s, 1e-30f)) : -s;
}

template <int VEC, bool PL>
__global__ void __launch_bounds__(32 * GATHER_WARPS, VEC >= 8 ? 2 : 3) gather_kernel(WaveDims d, WaveBatches wb, WaveBufs w) {
  int lane = threadIdx.x & 31;
  long long item = (long long)blockIdx.x * GATHER_WARPS + (threadIdx.x >> 5);
  if (item >= (long long)d.nblk * d.Mm) return;
  int lb = (int)(item / d.Mm), r = (int)(item - (long long)lb * d.Mm);
  const int blk = d.blk0 + lb;
  BlockInfo bi = block_info(d, wb, blk);
  const int D = d.D;
  size_t nrow = (size_t)blk * d.Mm + r;
  const size_t noff = nrow * d.Dp;
  float *n0 = w.X[ARR_N0] + noff, *n1 = w.X[ARR_N1] + noff;
  float4 x[VEC], z[VEC], y0[VEC], y1[VEC];

  if (r < d.Pm) {                                           // ---- an edge of the chunk ----------
    size_t qrow = (size_t)blk * d.Pm + r;
    const size_t qoff = qrow * d.Dp;
    float *q0 = d.dynamic ? w.X[ARR_Q0] + qoff : nullptr;
    float *q1 = d.dynamic ? w.X[ARR_Q1] + qoff : nullptr;
    long long il = -1, ir = -1, rl = d.dynamic ? 0 : wb.rel[bi.b];
    bool ok = r < bi.n;
    if (ok) {
      il = w.lhs[bi.e0 + r];
      ir = w.rhs[bi.e0 + r];
      if (d.dynamic && d.op != PBG_OP_NONE) rl = w.rel[bi.e0 + r];
      if (il < 0 || il >= d.n_rows[0] || ir < 0 || ir >= d.n_rows[1] ||
          (d.op != PBG_OP_NONE && (rl < 0 || rl >= d.num_rels))) {
        if (lane == 0) atomicOr(w.errflag, 1);
        ok = false;
      }
    }
    if (!ok) {                                              // padding row: exact zeros
      zero_row<VEC>(n0, D, lane);
      zero_row<VEC>(n1, D, lane);
      if (d.matrix_op) zero_row<VEC>(w.R1 + noff, D, lane);
      if (d.dynamic) { zero_row<VEC>(q0, D, lane); zero_row<VEC>(q1, D, lane); }
      if (PL) {
        zero_row_planes<VEC>(w, ARR_N0, blk, r, D, lane); zero_row_planes<VEC>(w, ARR_N1, blk, r, D, lane);
        if (d.dynamic) { zero_row_planes<VEC>(w, ARR_Q0, blk, r, D, lane); zero_row_planes<VEC>(w, ARR_Q1, blk, r, D, lane); }
      }
      if (lane == 0) {
        w.aux[ARR_N0][nrow] = 0.f; w.aux[ARR_N1][nrow] = 0.f;
        if (d.dynamic) { w.aux[ARR_Q0][qrow] = 0.f; w.aux[ARR_Q1][qrow] = 0.f; }
        w.spos[0][qrow] = 0.f; w.spos[1][qrow] = 0.f;
      }
      return;
    }
    const float *xl = w.W[0] + (size_t)il * D, *xr = w.W[1] + (size_t)ir * D;
    const float *th0 = (d.op != PBG_OP_NONE && w.theta[0]) ? w.theta[0] + (size_t)rl * D : nullptr;
    // lhs row without operator -> N0
    load_row<VEC>(x, xl, D, lane);
    const float scl = renorm_row<VEC>(x, d.max_norm);
    add_global<VEC>(x, w.glob[0], D, lane);
#pragma unroll
    for (int c = 0; c < VEC; ++c) y0[c] = x[c];
    float a0 = prepare_row<VEC>(y0, d.cmp);
    put_row<VEC>(w.X[ARR_N0], noff, y0, D, lane);
    if (PL) put_row_planes<VEC>(w, ARR_N0, blk, r, y0, D, lane);
    if (d.matrix_op) {
      // linear / affine: the raw rhs row goes to R1; operator, prepare and the positive score
      // follow in the contraction and postop_kernel
      load_row<VEC>(x, xr, D, lane);
      renorm_row<VEC>(x, d.max_norm);
      add_global<VEC>(x, w.glob[1], D, lane);
      store_row<VEC>(w.R1 + noff, x, D, lane);
      if (lane == 0) w.aux[ARR_N0][nrow] = a0;
    } else if (!d.dynamic) {
      // rhs row through the operator -> N1; one positive score shared by both problems
      load_row<VEC>(x, xr, D, lane);
      const float scr = renorm_row<VEC>(x, d.max_norm);
      if (d.max_norm > 0.f && lane == 0) w.rscale[nrow] = scr;
      add_global<VEC>(x, w.glob[1], D, lane);
      apply_operator<VEC>(y1, x, xr, th0, d.op, D, lane, w.glob[1], scr);
      float a1 = prepare_row<VEC>(y1, d.cmp);
      put_row<VEC>(w.X[ARR_N1], noff, y1, D, lane);
      if (PL) put_row_planes<VEC>(w, ARR_N1, blk, r, y1, D, lane);
      float s = positive_score<VEC>(y0, y1, d.cmp);
      if (lane == 0) {
        w.aux[ARR_N0][nrow] = a0; w.aux[ARR_N1][nrow] = a1;
        w.spos[0][qrow] = s; w.spos[1][qrow] = s;
      }
    } else {
      const float *th1 = (d.op != PBG_OP_NONE && w.theta[1]) ? w.theta[1] + (size_t)rl * D : nullptr;
      // op_lhs(lhs row) -> Q1 (x still holds the lhs row)
      apply_operator<VEC>(z, x, xl, th1, d.op, D, lane, nullptr, scl);
      float aq1 = prepare_row<VEC>(z, d.cmp);
      put_row<VEC>(w.X[ARR_Q1], qoff, z, D, lane);
      if (PL) put_row_planes<VEC>(w, ARR_Q1, blk, r, z, D, lane);
      // rhs row without operator -> N1
      load_row<VEC>(x, xr, D, lane);
      const float scr = renorm_row<VEC>(x, d.max_norm);
#pragma unroll
      for (int c = 0; c < VEC; ++c) y1[c] = x[c];
      float a1 = prepare_row<VEC>(y1, d.cmp);
      put_row<VEC>(w.X[ARR_N1], noff, y1, D, lane);
      if (PL) put_row_planes<VEC>(w, ARR_N1, blk, r, y1, D, lane);
      float s1 = positive_score<VEC>(y1, z, d.cmp);         // problem 1: c(rhs, op_lhs(lhs))
      // op_rhs(rhs row) -> Q0
      apply_operator<VEC>(z, x, xr, th0, d.op, D, lane, nullptr, scr);
      float aq0 = prepare_row<VEC>(z, d.cmp);
      put_row<VEC>(w.X[ARR_Q0], qoff, z, D, lane);
      if (PL) put_row_planes<VEC>(w, ARR_Q0, blk, r, z, D, lane);
      float s0 = positive_score<VEC>(y0, z, d.cmp);         // problem 0: c(lhs, op_rhs(rhs))
      if (lane == 0) {
        w.aux[ARR_N0][nrow] = a0; w.aux[ARR_N1][nrow] = a1;
        w.aux[ARR_Q0][qrow] = aq0; w.aux[ARR_Q1][qrow] = aq1;
        w.spos[0][qrow] = s0; w.spos[1][qrow] = s1;
      }
    }
    return;
  }
  // ---- a uniformly drawn negative row, one per side ------------------------------------------
#pragma unroll
  for (int side = 0; side < 2; ++side) {
    float *dst = side == 0 ? n0 : n1;
    long long id = slot_row(d, wb, w, bi, side, r);
    if (id >= d.n_rows[side]) { if (lane == 0) atomicOr(w.errflag, 1); id = -1; }
    if (id < 0) {
      zero_row<VEC>(dst, D, lane);
      if (PL) zero_row_planes<VEC>(w, side, blk, r, D, lane);
      if (side == 1 && d.matrix_op) zero_row<VEC>(w.R1 + noff, D, lane);
      if (lane == 0) w.aux[side][nrow] = 0.f;
      continue;
    }
    const float *xrow = w.W[side] + (size_t)id * D;
    load_row<VEC>(x, xrow, D, lane);
    const float scu = renorm_row<VEC>(x, d.max_norm);
    if (side == 1 && d.max_norm > 0.f && lane == 0) w.rscale[nrow] = scu;
    add_global<VEC>(x, w.glob[side], D, lane);
    if (side == 1 && d.matrix_op) { store_row<VEC>(w.R1 + noff, x, D, lane); continue; }
    const float *th = nullptr;
    if (side == 1 && !d.dynamic && d.op != PBG_OP_NONE && w.theta[0]) {
      int rl = wb.rel[bi.b];
      if (rl >= 0 && rl < d.num_rels) th = w.theta[0] + (size_t)rl * D;
    }
    apply_operator<VEC>(z, x, xrow, th, d.op, D, lane, w.glob[side], scu);
    float a = prepare_row<VEC>(z, d.cmp);
    put_row<VEC>(w.X[side], noff, z, D, lane);
    if (PL) put_row_planes<VEC>(w, side, blk, r, z, D, lane);
    if (lane == 0) w.aux[side][nrow] = a;
  }
}

// The same work when nothing has to be computed on the way -- standard relations, no operator, dot
// comparator: the operand rows are plain copies of the table rows, and the positive score is their
// dot product.  Both rows of a slot (lhs side, rhs side) are loaded at once, which doubles the bytes
// a warp keeps in flight, and the kernel carries none of the operator / prepare code of the general
// one (half the registers, three CTAs per SM instead of two).
template <int VEC, bool PL>
__global__ void __launch_bounds__(32 * GATHER_WARPS, VEC >= 16 ? 1 : VEC >= 8 ? 3 : 4) gather_plain_kernel(WaveDims d, WaveBatches wb, WaveBufs w) {
  int lane = threadIdx.x & 31;
  long long item = (long long)blockIdx.x * GATHER_WARPS + (threadIdx.x >> 5);
  if (item >= (long long)d.nblk * d.Mm) return;
  int lb = (int)(item / d.Mm), r = (int)(item - (long long)lb * d.Mm);
  const int blk = d.blk0 + lb;
  BlockInfo bi = block_info(d, wb, blk);
  const int D = d.D;
  size_t nrow = (size_t)blk * d.Mm + r;
  const size_t noff = nrow * d.Dp;
  float *n0 = w.X[ARR_N0] + noff, *n1 = w.X[ARR_N1] + noff;
  long long i0, i1;
  const bool edge = r < d.Pm;
  if (edge) {
    bool ok = r < bi.n;
    i0 = ok ? w.lhs[bi.e0 + r] : -1;
    i1 = ok ? w.rhs[bi.e0 + r] : -1;
    if (ok && (i0 < 0 || i0 >= d.n_rows[0] || i1 < 0 || i1 >= d.n_rows[1])) {
      if (lane == 0) atomicOr(w.errflag, 1);
      ok = false;
    }
    if (!ok) i0 = i1 = -1;                                  // padding row: exact zeros on both sides
  } else {
    i0 = slot_row(d, wb, w, bi, 0, r);
    i1 = slot_row(d, wb, w, bi, 1, r);
    if (i0 >= d.n_rows[0]) { if (lane == 0) atomicOr(w.errflag, 1); i0 = -1; }
    if (i1 >= d.n_rows[1]) { if (lane == 0) atomicOr(w.errflag, 1); i1 = -1; }
  }
  float4 a[VEC], b[VEC];
#pragma unroll
  for (int c = 0; c < VEC; ++c) {
    int dd = c * 128 + lane * 4;
    a[c] = (i0 >= 0 && dd < D) ? ld4(w.W[0] + (size_t)i0 * D + dd) : f4zero();
  }
#pragma unroll
  for (int c = 0; c < VEC; ++c) {
    int dd = c * 128 + lane * 4;
    b[c] = (i1 >= 0 && dd < D) ? ld4(w.W[1] + (size_t)i1 * D + dd) : f4zero();
  }
  if (i0 >= 0) add_global<VEC>(a, w.glob[0], D, lane);       // padding rows stay exact zeros
  if (i1 >= 0) add_global<VEC>(b, w.glob[1], D, lane);
  if (PL) {
    // bf16-plane tier: the contractions read the planes, nothing reads the fp32 operand rows
    const size_t plane = (size_t)d.Mm * w.Dpb;
    unsigned short *x0 = w.XB[0] + ((size_t)blk * w.npl * d.Mm + r) * w.Dpb, *x1 = w.XB[1] + ((size_t)blk * w.npl * d.Mm + r) * w.Dpb;
    const bool three = w.npl > 2;
#pragma unroll
    for (int c = 0; c < VEC; ++c) {
      int dd = c * 128 + lane * 4;
      if (dd < D) {
        uint2 p0, p1, p2;
        bf16_planes4(a[c], p0, p1, p2);
        *(uint2 *)(x0 + dd) = p0; *(uint2 *)(x0 + plane + dd) = p1;
        if (three) *(uint2 *)(x0 + 2 * plane + dd) = p2;
        bf16_planes4(b[c], p0, p1, p2);
        *(uint2 *)(x1 + dd) = p0; *(uint2 *)(x1 + plane + dd) = p1;
        if (three) *(uint2 *)(x1 + 2 * plane + dd) = p2;
      }
    }
  } else {
    store_row<VEC>(n0, a, D, lane);
    store_row<VEC>(n1, b, D, lane);
  }
  float s = 0.f;
  if (edge) {
#pragma unroll
    for (int c = 0; c < VEC; ++c) s += f4dot(a[c], b[c]);
    s = warp_sum(s);
  }
  if (lane == 0) {
    w.aux[ARR_N0][nrow] = 0.f; w.aux[ARR_N1][nrow] = 0.f;
    if (edge) { size_t q = (size_t)blk * d.Pm + r; w.spos[0][q] = s; w.spos[1][q] = s; }
  }
}

// linear / affine operators: R2 holds A.x for every rhs row of the chunk blocks; this kernel adds
// the translation (affine), applies comparator.prepare, writes the operand row to N1 and, for the
// chunk's edges, the positive score against the lhs row already in N0.
template <int VEC>
__global__ void __launch_bounds__(32 * GATHER_WARPS) postop_kernel(WaveDims d, WaveBatches wb, WaveBufs w) {
  int lane = threadIdx.x & 31;
  long long item = (long long)blockIdx.x * GATHER_WARPS + (threadIdx.x >> 5);
  if (item >= (long long)d.nblk * d.Mm) return;
  int lb = (int)(item / d.Mm), r = (int)(item - (long long)lb * d.Mm);
  const int blk = d.blk0 + lb;
  BlockInfo bi = block_info(d, wb, blk);
  const int D = d.D;
  size_t nrow = (size_t)blk * d.Mm + r, noff = nrow * d.Dp;
  long long id = slot_row(d, wb, w, bi, 1, r);
  bool ok = id >= 0 && id < d.n_rows[1];
  if (ok && r < d.Pm) {                         // the edge's lhs id must be valid too (gather zeroed the rows otherwise)
    long long il = w.lhs[bi.e0 + r];
    ok = il >= 0 && il < d.n_rows[0];
  }
  float4 z[VEC], y0[VEC];
  if (!ok) {
    zero_row<VEC>(w.X[ARR_N1] + noff, D, lane);
    if (lane == 0) {
      w.aux[ARR_N1][nrow] = 0.f;
      if (r < d.Pm) { size_t q = (size_t)blk * d.Pm + r; w.spos[0][q] = 0.f; w.spos[1][q] = 0.f; }
    }
    return;
  }
  load_row<VEC>(z, w.R2 + noff, D, lane);
  if (d.op == PBG_OP_AFFINE) {
    const float *t = w.theta[0] + (size_t)wb.rel[bi.b] * d.opw + (size_t)D * D;
#pragma unroll
    for (int c = 0; c < VEC; ++c) {
      int dd = c * 128 + lane * 4;
      if (dd < D) z[c] = z[c] + ld4(t + dd);
    }
  }
  float a1 = prepare_row<VEC>(z, d.cmp);
  store_row<VEC>(w.X[ARR_N1] + noff, z, D, lane);
  if (lane == 0) w.aux[ARR_N1][nrow] = a1;
  if (r < d.Pm) {
    load_row<VEC>(y0, w.X[ARR_N0] + noff, D, lane);
    float s = positive_score<VEC>(y0, z, d.cmp);
    size_t q = (size_t)blk * d.Pm + r;
    if (lane == 0) { w.spos[0][q] = s; w.spos[1][q] = s; }
  }
}

int launch_postop(const WaveDims &d, const WaveBatches &wb, const WaveBufs &w, cudaStream_t st) {
  long long items = (long long)d.nblk * d.Mm;
  int ctas = (int)((items + GATHER_WARPS - 1) / GATHER_WARPS);
  int vec = (d.D + 127) / 128;
  if (vec <= 1) postop_kernel<1><<<ctas, 32 * GATHER_WARPS, 0, st>>>(d, wb, w);
  else if (vec <= 2) postop_kernel<2><<<ctas, 32 * GATHER_WARPS, 0, st>>>(d, wb, w);
  else if (vec <= 4) postop_kernel<4><<<ctas, 32 * GATHER_WARPS, 0, st>>>(d, wb, w);
  else if (vec <= 8) postop_kernel<8><<<ctas, 32 * GATHER_WARPS, 0, st>>>(d, wb, w);
  else postop_kernel<16><<<ctas, 32 * GATHER_WARPS, 0, st>>>(d, wb, w);
  return 1;
}

int launch_gather(const WaveDims &d, const WaveBatches &wb, const WaveBufs &w, cudaStream_t st) {
  long long items = (long long)d.nblk * d.Mm;
  int ctas = (int)((items + GATHER_WARPS - 1) / GATHER_WARPS);
  int vec = (d.D + 127) / 128;
  const bool plain = !d.dynamic && !d.matrix_op && d.max_norm <= 0.f && d.cmp == PBG_CMP_DOT && (d.op == PBG_OP_NONE || w.theta[0] == nullptr);
  if (plain && w.XB[0] && d.reg_coef == 0.f) {      // planes only: nothing reads the fp32 operand rows then
    if (vec <= 1) gather_plain_kernel<1, true><<<ctas, 32 * GATHER_WARPS, 0, st>>>(d, wb, w);
    else if (vec <= 2) gather_plain_kernel<2, true><<<ctas, 32 * GATHER_WARPS, 0, st>>>(d, wb, w);
    else if (vec <= 4) gather_plain_kernel<4, true><<<ctas, 32 * GATHER_WARPS, 0, st>>>(d, wb, w);
    else if (vec <= 8) gather_plain_kernel<8, true><<<ctas, 32 * GATHER_WARPS, 0, st>>>(d, wb, w);
    else gather_plain_kernel<16, true><<<ctas, 32 * GATHER_WARPS, 0, st>>>(d, wb, w);
    return 1;
  }
  if (plain && !w.XB[0]) {
    if (vec <= 1) gather_plain_kernel<1, false><<<ctas, 32 * GATHER_WARPS, 0, st>>>(d, wb, w);
    else if (vec <= 2) gather_plain_kernel<2, false><<<ctas, 32 * GATHER_WARPS, 0, st>>>(d, wb, w);
    else if (vec <= 4) gather_plain_kernel<4, false><<<ctas, 32 * GATHER_WARPS, 0, st>>>(d, wb, w);
    else if (vec <= 8) gather_plain_kernel<8, false><<<ctas, 32 * GATHER_WARPS, 0, st>>>(d, wb, w);
    else gather_plain_kernel<16, false><<<ctas, 32 * GATHER_WARPS, 0, st>>>(d, wb, w);
    return 1;
  }
  if (w.XB[0]) {
    if (vec <= 1) gather_kernel<1, true><<<ctas, 32 * GATHER_WARPS, 0, st>>>(d, wb, w);
    else if (vec <= 2) gather_kernel<2, true><<<ctas, 32 * GATHER_WARPS, 0, st>>>(d, wb, w);
    else if (vec <= 4) gather_kernel<4, true><<<ctas, 32 * GATHER_WARPS, 0, st>>>(d, wb, w);
    else if (vec <= 8) gather_kernel<8, true><<<ctas, 32 * GATHER_WARPS, 0, st>>>(d, wb, w);
    else gather_kernel<16, true><<<ctas, 32 * GATHER_WARPS, 0, st>>>(d, wb, w);
    return 1;
  }
  if (vec <= 1) gather_kernel<1, false><<<ctas, 32 * GATHER_WARPS, 0, st>>>(d, wb, w);
  else if (vec <= 2) gather_kernel<2, false><<<ctas, 32 * GATHER_WARPS, 0, st>>>(d, wb, w);
  else if (vec <= 4) gather_kernel<4, false><<<ctas, 32 * GATHER_WARPS, 0, st>>>(d, wb, w);
  else if (vec <= 8) gather_kernel<8, false><<<ctas, 32 * GATHER_WARPS, 0, st>>>(d, wb, w);
  else gather_kernel<16, false><<<ctas, 32 * GATHER_WARPS, 0, st>>>(d, wb, w);
  return 1;
}

// One thread per occurrence slot: the sort key is the table row the slot's gradient belongs to.
//   lhs-table rows            key = row
//   rhs-table rows            key = row (+ lhs rows when the tables differ)
//   operator-table rows       key = key_rel_base + table * num_rels + rel   (dynamic relations)
//   slots without gradient    key = key_invalid (sorts to the end)
__global__ void build_keys_kernel(WaveDims d, WaveBatches wb, WaveBufs w, unsigned long long *keys,
                                  unsigned int *vals) {
  int o = blockIdx.x * blockDim.x + threadIdx.x;
  if (o >= d.nocc) return;
  Occ q = occ_decode(d, o);
  BlockInfo bi = block_info(d, wb, q.blk);
  unsigned long long key = d.key_invalid;
  unsigned long long rbase = d.shared_table ? 0ull : (unsigned long long)d.n_rows[0];
  if (q.a == ARR_N0 || q.a == ARR_N1) {
    int side = q.a == ARR_N0 ? 0 : 1;
    long long row = slot_row(d, wb, w, bi, side, q.r);
    if (row >= 0 && row < d.n_rows[side]) key = (side ? rbase : 0ull) + (unsigned long long)row;
  } else if (q.r < bi.n) {
    long long e = bi.e0 + q.r;
    if (q.a == ARR_Q0) {
      long long row = w.rhs[e];
      if (row >= 0 && row < d.n_rows[1]) key = rbase + (unsigned long long)row;
    } else if (q.a == ARR_Q1) {
      long long row = w.lhs[e];
      if (row >= 0 && row < d.n_rows[0]) key = (unsigned long long)row;
    } else if (d.dynamic && d.op != PBG_OP_NONE) {
      long long rl = w.rel[e];
      int t = q.a == ARR_R0 ? 0 : 1;
      if (rl >= 0 && rl < d.num_rels) key = d.key_rel_base + (unsigned long long)t * d.num_rels + (unsigned long long)rl;
    }
  }
  keys[o] = key;
  vals[o] = (unsigned int)o;
}

int launch_build_keys(const WaveDims &d, const WaveBatches &wb, const WaveBufs &w,
                      unsigned long long *keys, unsigned int *vals, cudaStream_t st) {
  build_keys_kernel<<<(d.nocc + 255) / 256, 256, 0, st>>>(d, wb, w, keys, vals);
  return 1;
}
