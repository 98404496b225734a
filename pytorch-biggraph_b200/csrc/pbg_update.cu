// Optimizer steps of one wave, one warp per touched table row.
//
// The sorted occurrence list (pbg_sort.cu) puts all gradient slots of a table row next to each
// other, in batch order.  A warp owns a row: it keeps the row in registers, and for every batch of
// the wave that touched it sums the slots' gradients -- each taken back through
// comparator.prepare and the relation operator on the fly -- and applies one optimizer step:
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
#define UPD_RUN 2          // sorted positions whose segment heads one warp looks after

// Everything needed to pull one gradient slot back to the embedding row it came from.
template <int VEC>
struct SlotGrad {
  const float *g, *y;      // gradient row, prepared operand row
  const float *theta;      // operator row or null
  float dotgy, inv, cf;    // cos: <g', y> and 1/|z|; l2 family: coefficient of y
  int op, cmp, D;

  __device__ __forceinline__ void init(const WaveDims &d, const WaveBatches &wb, const WaveBufs &w,
                                       int a, int blk, int r, int b, int lane) {
    D = d.D; op = d.op; cmp = d.cmp;
    size_t xr = (size_t)blk * w.xrows[a] + r, gr = (size_t)blk * w.grows[a] + r;
    y = w.X[a] + xr * d.Dp;
    g = w.GX[a] + gr * d.Dp;
    theta = nullptr;
    if (op != PBG_OP_NONE) {
      if (!d.dynamic) {
        if ((a == ARR_N1 || a == ARR_Q0) && w.theta[0]) theta = w.theta[0] + (size_t)wb.rel[b] * D;
      } else if (a == ARR_Q0 || a == ARR_Q1) {
        BlockInfo bi = block_info(d, wb, blk);
        long long rl = w.rel[bi.e0 + r];
        const float *tab = w.theta[a == ARR_Q0 ? 0 : 1];
        if (tab && rl >= 0 && rl < d.num_rels) theta = tab + (size_t)rl * D;
      }
    }
    cf = 0.f; inv = 1.f; dotgy = 0.f;
    if (cmp >= PBG_CMP_L2) {
      // ga = T.N - rowsum(T) a ;  gb = T^T.Q - colsum(T) b
      const float *cp = (a == ARR_N0) ? w.coef[0] : (a == ARR_N1) ? w.coef[1] : (a == ARR_Q0) ? w.coef[2] : w.coef[3];
      cf = cp[gr];
    } else if (cmp == PBG_CMP_COS) {
      inv = w.aux[a][xr];
      float s = 0.f;
#pragma unroll
      for (int c = 0; c < VEC; ++c) {
        int dd = c * 128 + lane * 4;
        if (dd < D) s += f4dot(ld4(g + dd), ld4(y + dd));
      }
      dotgy = warp_sum(s);
    }
  }
  // gradient w.r.t. the operator output z at elements [dd, dd+4)
  __device__ __forceinline__ float4 gz(int dd) const {
    float4 v = ld4(g + dd);
    if (cmp >= PBG_CMP_L2) v = v - ld4(y + dd) * cf;
    else if (cmp == PBG_CMP_COS) v = (v - ld4(y + dd) * dotgy) * inv;   // (g - y <g,y>) / |z|
    return v;
  }
  // gradient w.r.t. the embedding row at elements [dd, dd+4)
  __device__ __forceinline__ float4 gx(int dd) const {
    float4 v = gz(dd);
    if (theta == nullptr || op == PBG_OP_TRANSLATION) return v;
    float4 t = ld4(theta + dd);
    if (op == PBG_OP_DIAGONAL) return v * t;
    int h = D >> 1;
    int dp = dd < h ? dd + h : dd - h;
    float4 vp = gz(dp), tp = ld4(theta + dp);
    // gx_re = g_re p_re + g_im p_im ;  gx_im = -g_re p_im + g_im p_re
    return dd < h ? v * t + vp * tp : v * tp - vp * t;
  }
};

template <int VEC>
__global__ void __launch_bounds__(32 * UPD_WARPS)
emb_update_kernel(WaveDims d, WaveBatches wb, WaveBufs w, const unsigned long long *__restrict__ keys,
                  const unsigned int *__restrict__ vals, float lr) {
  int lane = threadIdx.x & 31;
  long long wid = (long long)blockIdx.x * UPD_WARPS + (threadIdx.x >> 5);
  long long p0 = wid * UPD_RUN;
  const int D = d.D;
  const float invD = 1.0f / (float)D;
  for (long long pos = p0; pos < p0 + UPD_RUN && pos < d.nocc; ++pos) {
    unsigned long long key = keys[pos];
    if (key >= d.key_rel_base) return;                       // operator rows and empty slots follow
    if (pos > 0 && keys[pos - 1] == key) continue;           // not the head of a segment
    int side = (!d.shared_table && key >= (unsigned long long)d.n_rows[0]) ? 1 : 0;
    long long row = (long long)(side ? key - (unsigned long long)d.n_rows[0] : key);
    float *wrow = w.W[side] + (size_t)row * D;
    float4 wv[VEC], acc[VEC];
#pragma unroll
    for (int c = 0; c < VEC; ++c) {
      int dd = c * 128 + lane * 4;
      wv[c] = dd < D ? ld4(wrow + dd) : f4zero();
      acc[c] = f4zero();
    }
    float G = w.G[side][row];
    int cur_b = -1;
    for (long long q = pos; q <= d.nocc; ++q) {
      bool same = q < d.nocc && keys[q] == key;
      Occ oc;
      if (same) oc = occ_decode(d, (int)vals[q]);
      if (cur_b >= 0 && (!same || oc.b != cur_b)) {          // close the batch: one RowAdagrad step
        float ss = 0.f;
#pragma unroll
        for (int c = 0; c < VEC; ++c) ss += f4dot(acc[c], acc[c]);
        ss = warp_sum(ss);
        G += ss * invD;
        float stepv = lr / (sqrtf(G) + PBG_ADAGRAD_EPS);
#pragma unroll
        for (int c = 0; c < VEC; ++c) { wv[c] = wv[c] - acc[c] * stepv; acc[c] = f4zero(); }
      }
      if (!same) break;
      cur_b = oc.b;
      SlotGrad<VEC> sg;
      sg.init(d, wb, w, oc.a, oc.blk, oc.r, oc.b, lane);
#pragma unroll
      for (int c = 0; c < VEC; ++c) {
        int dd = c * 128 + lane * 4;
        if (dd < D) acc[c] = acc[c] + sg.gx(dd);
      }
    }
#pragma unroll
    for (int c = 0; c < VEC; ++c) {
      int dd = c * 128 + lane * 4;
      if (dd < D) st4(wrow + dd, wv[c]);
    }
    if (lane == 0) w.G[side][row] = G;
  }
}

// d(loss)/d(operator row) contributed by one slot whose operand went through the operator:
// needs the gradient at the operator output (gz) and the raw embedding row x.
template <int VEC>
__device__ __forceinline__ float4 op_param_grad(const SlotGrad<VEC> &sg, const float *x, float xscale, int dd) {
  float4 v = sg.gz(dd);
  if (sg.op == PBG_OP_TRANSLATION) return v;
  float4 xv = ld4(x + dd) * xscale;
  if (sg.op == PBG_OP_DIAGONAL) return v * xv;
  int h = sg.D >> 1;
  int dp = dd < h ? dd + h : dd - h;
  float4 vp = sg.gz(dp), xp = ld4(x + dp) * xscale;
  // d real = g_re a_re + g_im a_im ;  d imag = -g_re a_im + g_im a_re
  return dd < h ? v * xv + vp * xp : v * xp - vp * xv;
}

// Dynamic relations: operator-table rows are sort keys of their own (key >= key_rel_base); the
// raw embedding row of a slot is its operator-free copy in N0 / N1 (times |x| for cos).
template <int VEC>
__global__ void __launch_bounds__(32 * UPD_WARPS)
rel_update_dyn_kernel(WaveDims d, WaveBatches wb, WaveBufs w, const unsigned long long *__restrict__ keys,
                      const unsigned int *__restrict__ vals, float lr) {
  int lane = threadIdx.x & 31;
  long long wid = (long long)blockIdx.x * UPD_WARPS + (threadIdx.x >> 5);
  long long p0 = wid * UPD_RUN;
  const int D = d.D;
  for (long long pos = p0; pos < p0 + UPD_RUN && pos < d.nocc; ++pos) {
    unsigned long long key = keys[pos];
    if (key >= d.key_invalid) return;
    if (key < d.key_rel_base) continue;
    if (pos > 0 && keys[pos - 1] == key) continue;
    unsigned long long rk = key - d.key_rel_base;
    int t = rk >= (unsigned long long)d.num_rels ? 1 : 0;
    long long rl = (long long)(rk - (unsigned long long)t * d.num_rels);
    float *th = w.theta[t] + (size_t)rl * D, *ac = w.acc[t] + (size_t)rl * D;
    float4 tv[VEC], av[VEC], acc[VEC];
#pragma unroll
    for (int c = 0; c < VEC; ++c) {
      int dd = c * 128 + lane * 4;
      tv[c] = dd < D ? ld4(th + dd) : f4zero();
      av[c] = dd < D ? ld4(ac + dd) : f4zero();
      acc[c] = f4zero();
    }
    int cur_b = -1;
    for (long long q = pos; q <= d.nocc; ++q) {
      bool same = q < d.nocc && keys[q] == key;
      Occ oc;
      if (same) oc = occ_decode(d, (int)vals[q]);
      if (cur_b >= 0 && (!same || oc.b != cur_b)) {          // one AsyncAdagrad step
#pragma unroll
        for (int c = 0; c < VEC; ++c) {
          float4 g = acc[c];
          av[c] = av[c] + g * g;
          tv[c].x -= lr * g.x / (sqrtf(av[c].x) + PBG_ADAGRAD_EPS);
          tv[c].y -= lr * g.y / (sqrtf(av[c].y) + PBG_ADAGRAD_EPS);
          tv[c].z -= lr * g.z / (sqrtf(av[c].z) + PBG_ADAGRAD_EPS);
          tv[c].w -= lr * g.w / (sqrtf(av[c].w) + PBG_ADAGRAD_EPS);
          acc[c] = f4zero();
        }
      }
      if (!same) break;
      cur_b = oc.b;
      int qa = oc.a == ARR_R0 ? ARR_Q0 : ARR_Q1;             // slot that carried the operator
      int na = oc.a == ARR_R0 ? ARR_N1 : ARR_N0;             // its operator-free copy
      SlotGrad<VEC> sg;
      sg.init(d, wb, w, qa, oc.blk, oc.r, oc.b, lane);
      size_t nrow = (size_t)oc.blk * w.xrows[na] + oc.r;
      const float *x = w.X[na] + nrow * d.Dp;
      float xscale = d.cmp == PBG_CMP_COS ? 1.0f / w.aux[na][nrow] : 1.0f;
#pragma unroll
      for (int c = 0; c < VEC; ++c) {
        int dd = c * 128 + lane * 4;
        if (dd < D) acc[c] = acc[c] + op_param_grad<VEC>(sg, x, xscale, dd);
      }
    }
#pragma unroll
    for (int c = 0; c < VEC; ++c) {
      int dd = c * 128 + lane * 4;
      if (dd < D) { st4(th + dd, tv[c]); st4(ac + dd, av[c]); }
    }
  }
}

// Standard relations: every rhs row of a batch went through the same operator row.  Stage 1: one
// CTA per chunk sums the parameter gradient of its rows (N1 rows: chunk + uniform; Q0 rows: chunk)
// into relpart[b][c][warp][D]; the raw rows are re-read from the rhs table, which this wave has not
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
  int items = d.Mm + d.Pm;                                   // N1 slots then Q0 slots
  if (bi.n > 0) {
    for (int it = wl; it < items; it += UPD_WARPS) {
      int a = it < d.Mm ? ARR_N1 : ARR_Q0;
      int r = it < d.Mm ? it : it - d.Mm;
      long long row = slot_row(d, wb, w, bi, 1, r);
      if (row < 0 || row >= d.n_rows[1]) continue;
      SlotGrad<VEC> sg;
      sg.init(d, wb, w, a, blk, r, bi.b, lane);
      const float *x = w.W[1] + (size_t)row * D;
#pragma unroll
      for (int c = 0; c < VEC; ++c) {
        int dd = c * 128 + lane * 4;
        if (dd < D) acc[c] = acc[c] + op_param_grad<VEC>(sg, x, 1.0f, dd);
      }
    }
  }
  float *out = w.relpart + ((size_t)blk * UPD_WARPS + wl) * D;     // one partial per warp
#pragma unroll
  for (int c = 0; c < VEC; ++c) {
    int dd = c * 128 + lane * 4;
    if (dd < D) st4(out + dd, acc[c]);
  }
}

__global__ void relupdate_std_kernel(WaveDims d, WaveBatches wb, WaveBufs w, float lr) {
  int dd = blockIdx.x * blockDim.x + threadIdx.x;
  if (dd >= d.D) return;
  for (int b = 0; b < d.k; ++b) {
    if (wb.n[b] <= 0) continue;
    int rl = wb.rel[b];
    if (rl < 0 || rl >= d.num_rels) continue;
    float g = 0.f;
    for (int c = 0; c < d.Cm * UPD_WARPS; ++c) g += w.relpart[((size_t)b * d.Cm * UPD_WARPS + c) * d.D + dd];
    size_t idx = (size_t)rl * d.D + dd;
    float a = w.acc[0][idx] + g * g;
    w.acc[0][idx] = a;
    w.theta[0][idx] -= lr * g / (sqrtf(a) + PBG_ADAGRAD_EPS);
  }
}

template <int VEC>
static int launch_update_vec(const WaveDims &d, const WaveBatches &wb, const WaveBufs &w,
                             const unsigned long long *keys, const unsigned int *vals, float lr, float rel_lr,
                             cudaStream_t st) {
  int launches = 0;
  long long warps = ((long long)d.nocc + UPD_RUN - 1) / UPD_RUN;
  int ctas = (int)((warps + UPD_WARPS - 1) / UPD_WARPS);
  bool has_op = d.op != PBG_OP_NONE && w.theta[0] != nullptr;
  if (has_op && !d.dynamic) {
    relgrad_std_kernel<VEC><<<d.nblk, 32 * UPD_WARPS, 0, st>>>(d, wb, w);
    ++launches;
  }
  emb_update_kernel<VEC><<<ctas, 32 * UPD_WARPS, 0, st>>>(d, wb, w, keys, vals, lr);
  ++launches;
  if (has_op) {
    if (d.dynamic) rel_update_dyn_kernel<VEC><<<ctas, 32 * UPD_WARPS, 0, st>>>(d, wb, w, keys, vals, rel_lr);
    else relupdate_std_kernel<<<(d.D + 127) / 128, 128, 0, st>>>(d, wb, w, rel_lr);
    ++launches;
  }
  return launches;
}

int launch_update(const WaveDims &d, const WaveBatches &wb, const WaveBufs &w, const unsigned long long *keys,
                  const unsigned int *vals, float lr, float rel_lr, cudaStream_t st) {
  int vec = (d.D + 127) / 128;
  if (vec <= 1) return launch_update_vec<1>(d, wb, w, keys, vals, lr, rel_lr, st);
  if (vec <= 2) return launch_update_vec<2>(d, wb, w, keys, vals, lr, rel_lr, st);
  if (vec <= 4) return launch_update_vec<4>(d, wb, w, keys, vals, lr, rel_lr, st);
  if (vec <= 8) return launch_update_vec<8>(d, wb, w, keys, vals, lr, rel_lr, st);
  return launch_update_vec<16>(d, wb, w, keys, vals, lr, rel_lr, st);
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
