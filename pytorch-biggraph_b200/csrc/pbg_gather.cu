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
// `tag` is OR-ed into every key (the wave's number above the key bits when a whole call is sorted at once).
__global__ void build_keys_kernel(WaveDims d, WaveBatches wb, WaveBufs w, unsigned long long *keys,
                                  unsigned int *vals, unsigned long long tag) {
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
  keys[o] = key | tag;
  vals[o] = (unsigned int)o;
}

int launch_build_keys(const WaveDims &d, const WaveBatches &wb, const WaveBufs &w,
                      unsigned long long *keys, unsigned int *vals, cudaStream_t st, unsigned long long tag) {
  build_keys_kernel<<<(d.nocc + 255) / 256, 256, 0, st>>>(d, wb, w, keys, vals, tag);
  return 1;
}

// keys[i] &= mask: drops the wave tags once the call-wide sort has grouped the slots by wave
__global__ void mask_keys_kernel(unsigned long long *keys, long long n, unsigned long long mask) {
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) keys[i] &= mask;
}
int launch_mask_keys(unsigned long long *keys, long long n, unsigned long long mask, cudaStream_t st) {
  if (n > 0) mask_keys_kernel<<<(int)((n + 255) / 256), 256, 0, st>>>(keys, n, mask);
  return n > 0;
}

// ------------------------------------------------------------------------------------------------
// Ranking against ALL entities of a side's table (relations with all_negs=True, torchbiggraph/model.py:582-617;
// what RankingEvaluator needs for full-ranking MRR, torchbiggraph/eval.py:43-81).  One chunk holds the whole
// batch, the negatives of a side are every row of its table, and an edge's own true entity is ignored.
//   allnegs_rows_kernel     per edge: the two scored rows (prepared, operator applied where the mode says so)
//                           and the positive score(s)
//   allnegs_slab_kernel     a slab of table rows as candidates: global embedding, operator (standard relations,
//                           rhs side), prepare -> Y[slab][Dp] and the row's |y|^2
//   allnegs_score_kernel    64 x 64 tiles of scores between the batch's scored rows and the slab, never stored:
//                           per (tile, edge) the count of candidates scoring >= the positive and the loss partials
//   allnegs_merge_kernel    folds a slab's tiles into the per-edge running state, in tile order
//   allnegs_finish_kernel   ranks, loss and the evaluator's sums
// ------------------------------------------------------------------------------------------------
struct AllNegs {
  float *Q[2];            // [B][Dp]  Q[0]: scored against lhs candidates (op_rhs(rhs) rows), Q[1]: against rhs candidates
  float *qn[2];           // [B] |q|^2 (l2 family)
  float *pos[2];          // [B] positive score of problem 0 / 1
  float *Y, *yn;          // candidate slab [slab][Dp], |y|^2
  int *pcnt; float *pa, *pb;      // per (tile of the slab, edge): count, loss partials
  int *cnt[2]; float *ra[2], *rb[2];   // running per-edge state of side 0 / 1
  int B, slab;
};

template <int VEC>
__global__ void __launch_bounds__(32 * GATHER_WARPS) allnegs_rows_kernel(WaveDims d, WaveBufs w, AllNegs a, int rel_std) {
  int lane = threadIdx.x & 31;
  int e = blockIdx.x * GATHER_WARPS + (threadIdx.x >> 5);
  if (e >= a.B) return;
  const int D = d.D;
  long long il = w.lhs[e], ir = w.rhs[e], rl = d.dynamic ? 0 : rel_std;
  if (d.dynamic && d.op != PBG_OP_NONE) rl = w.rel[e];
  bool ok = il >= 0 && il < d.n_rows[0] && ir >= 0 && ir < d.n_rows[1] && (d.op == PBG_OP_NONE || (rl >= 0 && rl < d.num_rels));
  float *q0 = a.Q[0] + (size_t)e * d.Dp, *q1 = a.Q[1] + (size_t)e * d.Dp;
  if (!ok) {
    if (lane == 0) { atomicOr(w.errflag, 1); a.pos[0][e] = 0.f; a.pos[1][e] = 0.f; a.qn[0][e] = 0.f; a.qn[1][e] = 0.f; }
    zero_row<VEC>(q0, D, lane); zero_row<VEC>(q1, D, lane);
    return;
  }
  const float *xl = w.W[0] + (size_t)il * D, *xr = w.W[1] + (size_t)ir * D;
  float4 x[VEC], yl[VEC], yr[VEC], z[VEC];
  // lhs row, prepared (no operator)
  load_row<VEC>(x, xl, D, lane);
  const float scl = renorm_row<VEC>(x, d.max_norm);
  add_global<VEC>(x, w.glob[0], D, lane);
#pragma unroll
  for (int c = 0; c < VEC; ++c) yl[c] = x[c];
  float al = prepare_row<VEC>(yl, d.cmp);
  float s1 = 0.f, a1 = al;
  if (d.dynamic) {
    // problem 1 scores op_lhs(lhs) against the rhs candidates
    const float *th1 = (d.op != PBG_OP_NONE && w.theta[1]) ? w.theta[1] + (size_t)rl * D : nullptr;
    apply_operator<VEC>(z, x, xl, th1, d.op, D, lane, nullptr, scl);
    a1 = prepare_row<VEC>(z, d.cmp);
    store_row<VEC>(q1, z, D, lane);
  } else {
    store_row<VEC>(q1, yl, D, lane);
  }
  // rhs row through the rhs operator, prepared
  load_row<VEC>(x, xr, D, lane);
  const float scr = renorm_row<VEC>(x, d.max_norm);
  add_global<VEC>(x, w.glob[1], D, lane);
  const float *th0 = (d.op != PBG_OP_NONE && w.theta[0]) ? w.theta[0] + (size_t)rl * D : nullptr;
  apply_operator<VEC>(yr, x, xr, th0, d.op, D, lane, w.glob[1], scr);
  float a0 = prepare_row<VEC>(yr, d.cmp);
  store_row<VEC>(q0, yr, D, lane);
  float s0 = positive_score<VEC>(yl, yr, d.cmp);          // problem 0: c(lhs, op_rhs(rhs))
  if (d.dynamic) {
    // problem 1: c(prepared rhs without operator, op_lhs(lhs))
#pragma unroll
    for (int c = 0; c < VEC; ++c) yr[c] = x[c];
    prepare_row<VEC>(yr, d.cmp);
    s1 = positive_score<VEC>(yr, z, d.cmp);
  } else {
    s1 = s0;
  }
  if (lane == 0) {
    a.pos[0][e] = s0; a.pos[1][e] = s1;
    a.qn[0][e] = d.cmp >= PBG_CMP_L2 ? a0 : 0.f;
    a.qn[1][e] = d.cmp >= PBG_CMP_L2 ? a1 : 0.f;
  }
}

// candidates: rows [row0, row0 + n) of the table of `side`
template <int VEC>
__global__ void __launch_bounds__(32 * GATHER_WARPS) allnegs_slab_kernel(WaveDims d, WaveBufs w, AllNegs a, int side, long long row0, int n, int rel_std) {
  int lane = threadIdx.x & 31;
  int r = blockIdx.x * GATHER_WARPS + (threadIdx.x >> 5);
  if (r >= n) return;
  const int D = d.D;
  const float *xrow = w.W[side] + (size_t)(row0 + r) * D;
  float4 x[VEC], z[VEC];
  load_row<VEC>(x, xrow, D, lane);
  const float sc = renorm_row<VEC>(x, d.max_norm);
  add_global<VEC>(x, w.glob[side], D, lane);
  // standard relations apply the operator to every rhs row, negatives included; with dynamic relations negatives get none
  const float *th = (side == 1 && !d.dynamic && d.op != PBG_OP_NONE && w.theta[0]) ? w.theta[0] + (size_t)rel_std * D : nullptr;
  apply_operator<VEC>(z, x, xrow, th, d.op, D, lane, w.glob[side], sc);
  float aux = prepare_row<VEC>(z, d.cmp);
  store_row<VEC>(a.Y + (size_t)r * d.Dp, z, D, lane);
  if (lane == 0) a.yn[r] = d.cmp >= PBG_CMP_L2 ? aux : 0.f;
}

#define AN_TILE 64
// grid (edge tiles, candidate tiles of the slab); 256 threads, each a 4 x 4 block of the 64 x 64 score tile
__global__ void __launch_bounds__(256) allnegs_score_kernel(WaveDims d, WaveBufs w, AllNegs a, int side, long long row0, int n) {
  __shared__ float sq[16][AN_TILE + 1], sy[16][AN_TILE + 1];
  __shared__ int scnt[16][AN_TILE];
  __shared__ float sa[16][AN_TILE], sb[16][AN_TILE];
  const int te = blockIdx.x, tc = blockIdx.y, t = threadIdx.x;
  const int ty = t >> 4, tx = t & 15;                        // rows 4 ty .. 4 ty + 3 (edges), cols 4 tx .. (candidates)
  const float *Q = a.Q[side];
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  const int e0 = te * AN_TILE, c0 = tc * AN_TILE;
  for (int k0 = 0; k0 < d.D; k0 += 16) {
    // 64 rows x 16 k of each operand: thread t loads row t / 4, k (t % 4) * 4 .. + 3
    int lr = t >> 2, lk = (t & 3) * 4;
    float4 vq = f4zero(), vy = f4zero();
    if (e0 + lr < a.B && k0 + lk < d.D) vq = ld4(Q + (size_t)(e0 + lr) * d.Dp + k0 + lk);
    if (c0 + lr < n && k0 + lk < d.D) vy = ld4(a.Y + (size_t)(c0 + lr) * d.Dp + k0 + lk);
    __syncthreads();
    sq[lk][lr] = vq.x; sq[lk + 1][lr] = vq.y; sq[lk + 2][lr] = vq.z; sq[lk + 3][lr] = vq.w;
    sy[lk][lr] = vy.x; sy[lk + 1][lr] = vy.y; sy[lk + 2][lr] = vy.z; sy[lk + 3][lr] = vy.w;
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      float qv[4], yv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) { qv[i] = sq[k][ty * 4 + i]; yv[i] = sy[k][tx * 4 + i]; }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(qv[i], yv[j], acc[i][j]);
    }
  }
  // comparator, the ignored true entity, count and loss partials of this thread's 4 candidates per edge
  const long long *truth = side == 0 ? w.lhs : w.rhs;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int e = e0 + ty * 4 + i;
    int cnt = 0;
    float pa = 0.f, pb = d.loss == PBG_LOSS_SOFTMAX ? -INFINITY : 0.f;
    if (e < a.B) {
      const float pos = a.pos[side][e];
      const long long tid = truth[e];
      float sv[4];
      bool live[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int c = c0 + tx * 4 + j;
        live[j] = c < n && row0 + c != tid;
        float s = acc[i][j];
        if (d.cmp >= PBG_CMP_L2) {
          float qv = (a.yn[c < n ? c : 0] - 2.0f * s) + a.qn[side][e];       // model.py:226-246
          s = d.cmp == PBG_CMP_L2 ? -sqrtf(fmaxf(qv, 1e-30f)) : -qv;
        }
        sv[j] = s;
        if (live[j]) {
          cnt += s >= pos;
          if (d.loss == PBG_LOSS_RANKING) pa += fmaxf(0.f, (s - pos) + d.margin);
          else if (d.loss == PBG_LOSS_LOGISTIC) pa += fmaxf(s, 0.f) + log1pf(expf(-fabsf(s)));
          else pb = fmaxf(pb, s);
        }
      }
      if (d.loss == PBG_LOSS_SOFTMAX && pb > -INFINITY)
#pragma unroll
        for (int j = 0; j < 4; ++j) if (live[j]) pa += expf(sv[j] - pb);
    }
    scnt[tx][ty * 4 + i] = cnt; sa[tx][ty * 4 + i] = pa; sb[tx][ty * 4 + i] = pb;
  }
  __syncthreads();
  if (t < AN_TILE) {
    const int e = e0 + t;
    if (e < a.B) {
      int cnt = 0;
      float pa = 0.f, pb = d.loss == PBG_LOSS_SOFTMAX ? -INFINITY : 0.f;
      for (int x = 0; x < 16; ++x) {                       // the 16 column groups in a fixed order
        cnt += scnt[x][t];
        if (d.loss == PBG_LOSS_SOFTMAX) {
          float m2 = sb[x][t];
          if (m2 > -INFINITY) {
            float m = fmaxf(pb, m2);
            pa = (pb > -INFINITY ? pa * expf(pb - m) : 0.f) + sa[x][t] * expf(m2 - m);
            pb = m;
          }
        } else pa += sa[x][t];
      }
      size_t o = (size_t)tc * a.B + e;
      a.pcnt[o] = cnt; a.pa[o] = pa; a.pb[o] = pb;
    }
  }
}

__global__ void allnegs_merge_kernel(WaveDims d, AllNegs a, int side, int ntiles, int first) {
  int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= a.B) return;
  int cnt = first ? 0 : a.cnt[side][e];
  float ra = first ? 0.f : a.ra[side][e];
  float rb = first ? (d.loss == PBG_LOSS_SOFTMAX ? -INFINITY : 0.f) : a.rb[side][e];
  for (int tcl = 0; tcl < ntiles; ++tcl) {
    size_t o = (size_t)tcl * a.B + e;
    cnt += a.pcnt[o];
    if (d.loss == PBG_LOSS_SOFTMAX) {
      float m2 = a.pb[o];
      if (m2 > -INFINITY) {
        float m = fmaxf(rb, m2);
        ra = (rb > -INFINITY ? ra * expf(rb - m) : 0.f) + a.pa[o] * expf(m2 - m);
        rb = m;
      }
    } else ra += a.pa[o];
  }
  a.cnt[side][e] = cnt; a.ra[side][e] = ra; a.rb[side][e] = rb;
}

// out8: loss, pos_rank, mrr, r1, r10, r50 sums over both sides' ranks (as eval_reduce_kernel); AUC slots are filled by allnegs_auc_kernel
__global__ void __launch_bounds__(256) allnegs_finish_kernel(WaveDims d, WaveBufs w, AllNegs a, float wrel, double *out8) {
  __shared__ double sm[6][256];
  int t = threadIdx.x;
  double acc[6] = {0, 0, 0, 0, 0, 0};
  for (int e = t; e < a.B; e += 256) {
    const float wgt = wrel * (w.ew ? w.ew[e] : 1.0f);
    for (int side = 0; side < 2; ++side) {
      if (!d.neg_enabled[side]) continue;
      const float pos = a.pos[side][e];
      const long long n = d.n_rows[side];
      float lossv;
      if (d.loss == PBG_LOSS_RANKING) lossv = a.ra[side][e];
      else if (d.loss == PBG_LOSS_LOGISTIC) lossv = a.ra[side][e] / (float)n + (fmaxf(-pos, 0.f) + log1pf(expf(-fabsf(pos))));   // M counts the ignored column
      else {
        float m = fmaxf(a.rb[side][e], pos);
        float z = (a.rb[side][e] > -INFINITY ? a.ra[side][e] * expf(a.rb[side][e] - m) : 0.f) + expf(pos - m);
        lossv = -pos + m + logf(z);
      }
      acc[0] += (double)(wgt * lossv);
      int rk = a.cnt[side][e] + 1;
      acc[1] += rk; acc[2] += 1.0 / rk; acc[3] += rk <= 1; acc[4] += rk <= 10; acc[5] += rk <= 50;
    }
  }
  for (int k = 0; k < 6; ++k) sm[k][t] = acc[k];
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if (t < o) for (int k = 0; k < 6; ++k) sm[k][t] += sm[k][t + o];
    __syncthreads();
  }
  if (t < 6) out8[t] = sm[t][0];
}

// randomized AUC (torchbiggraph/util.py:415-428): `count` random (positive, (edge, candidate)) pairs per side; one warp per sample
template <int VEC>
__global__ void __launch_bounds__(32 * GATHER_WARPS) allnegs_auc_kernel(WaveDims d, WaveBufs w, AllNegs a, int rel_std, double *out8) {
  int lane = threadIdx.x & 31;
  int smp = blockIdx.x * GATHER_WARPS + (threadIdx.x >> 5);
  int side = blockIdx.y;
  if (smp >= a.B || !d.neg_enabled[side]) return;
  const int D = d.D;
  unsigned long long h = pbg_mix64(w.seed ^ pbg_mix64(0xA11CE5ull + (unsigned long long)side * 0x10001ull + smp));
  int ei = (int)(h % (unsigned long long)a.B);
  h = pbg_mix64(h);
  int er = (int)(h % (unsigned long long)a.B);
  h = pbg_mix64(h);
  long long cand = (long long)(h % (unsigned long long)d.n_rows[side]);
  const long long *truth = side == 0 ? w.lhs : w.rhs;
  float neg;
  if (cand == truth[er]) neg = PBG_MASKED;
  else {
    const float *xrow = w.W[side] + (size_t)cand * D;
    float4 x[VEC], z[VEC], q[VEC];
    load_row<VEC>(x, xrow, D, lane);
    const float sc = renorm_row<VEC>(x, d.max_norm);
    add_global<VEC>(x, w.glob[side], D, lane);
    const float *th = (side == 1 && !d.dynamic && d.op != PBG_OP_NONE && w.theta[0]) ? w.theta[0] + (size_t)rel_std * D : nullptr;
    apply_operator<VEC>(z, x, xrow, th, d.op, D, lane, w.glob[side], sc);
    float yn = prepare_row<VEC>(z, d.cmp);
    load_row<VEC>(q, a.Q[side] + (size_t)er * d.Dp, D, lane);
    float s = 0.f;
#pragma unroll
    for (int c = 0; c < VEC; ++c) s += f4dot(q[c], z[c]);
    s = warp_sum(s);
    if (d.cmp >= PBG_CMP_L2) {
      float qv = (yn - 2.0f * s) + a.qn[side][er];
      s = d.cmp == PBG_CMP_L2 ? -sqrtf(fmaxf(qv, 1e-30f)) : -qv;
    }
    neg = s;
  }
  if (lane == 0 && a.pos[side][ei] > neg) atomicAdd(&out8[6 + side], 1.0);
}

size_t pbg_allnegs_bytes(int B, int Dp, int slab) {
  size_t f = 2ull * B * Dp + 2ull * B + 2ull * B + (size_t)slab * Dp + slab;      // Q, qn, pos, Y, yn
  size_t tiles = (size_t)(slab + AN_TILE - 1) / AN_TILE;
  f += 3ull * tiles * B + 6ull * B;                                               // partials, running state
  return f * 4 + 4096;
}

// Runs the whole evaluation of one batch against all rows of both tables; `mem` holds pbg_allnegs_bytes bytes.
int launch_allnegs_eval(const WaveDims &d, const WaveBufs &w, char *mem, int B, int slab, int rel_std, float wrel,
                        double *out8_dev, cudaStream_t st) {
  AllNegs a;
  float *p = (float *)mem;
  auto take = [&](size_t n) { float *r = p; p += (n + 63) / 64 * 64; return r; };
  a.B = B; a.slab = slab;
  a.Q[0] = take((size_t)B * d.Dp); a.Q[1] = take((size_t)B * d.Dp);
  a.qn[0] = take(B); a.qn[1] = take(B); a.pos[0] = take(B); a.pos[1] = take(B);
  a.Y = take((size_t)slab * d.Dp); a.yn = take(slab);
  const int tiles_slab = (slab + AN_TILE - 1) / AN_TILE;
  a.pcnt = (int *)take((size_t)tiles_slab * B); a.pa = take((size_t)tiles_slab * B); a.pb = take((size_t)tiles_slab * B);
  for (int s = 0; s < 2; ++s) { a.cnt[s] = (int *)take(B); a.ra[s] = take(B); a.rb[s] = take(B); }
  int launches = 0;
  const int vec = (d.D + 127) / 128;
  const int ectas = (B + GATHER_WARPS - 1) / GATHER_WARPS;
  cudaMemsetAsync(out8_dev, 0, 8 * sizeof(double), st);
#define AN_V(K, ...) do { if (vec <= 1) K<1>__VA_ARGS__; else if (vec <= 2) K<2>__VA_ARGS__; else if (vec <= 4) K<4>__VA_ARGS__; else if (vec <= 8) K<8>__VA_ARGS__; else K<16>__VA_ARGS__; } while (0)
  AN_V(allnegs_rows_kernel, <<<ectas, 32 * GATHER_WARPS, 0, st>>>(d, w, a, rel_std));
  ++launches;
  for (int side = 0; side < 2; ++side) {
    if (!d.neg_enabled[side]) continue;
    const long long N = d.n_rows[side];
    bool first = true;
    for (long long row0 = 0; row0 < N; row0 += slab) {
      const int n = (int)(N - row0 < slab ? N - row0 : slab);
      const int sctas = (n + GATHER_WARPS - 1) / GATHER_WARPS;
      AN_V(allnegs_slab_kernel, <<<sctas, 32 * GATHER_WARPS, 0, st>>>(d, w, a, side, row0, n, rel_std));
      const int ntiles = (n + AN_TILE - 1) / AN_TILE;
      dim3 g((B + AN_TILE - 1) / AN_TILE, ntiles);
      allnegs_score_kernel<<<g, 256, 0, st>>>(d, w, a, side, row0, n);
      allnegs_merge_kernel<<<(B + 127) / 128, 128, 0, st>>>(d, a, side, ntiles, first ? 1 : 0);
      first = false;
      launches += 3;
    }
  }
  allnegs_finish_kernel<<<1, 256, 0, st>>>(d, w, a, wrel, out8_dev);
  dim3 ga(ectas, 2);
  AN_V(allnegs_auc_kernel, <<<ga, 32 * GATHER_WARPS, 0, st>>>(d, w, a, rel_std, out8_dev));
#undef AN_V
  pbg_note_launch();
  return launches + 2;
}
