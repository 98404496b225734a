// Loss, its gradient, masks and batch statistics, one warp per positive edge and problem.
// Fuses, for a whole wave:
//   the ignore masks (-1e9)             torchbiggraph/model.py:566-580, 836-844
//   logistic / ranking / softmax        torchbiggraph/losses.py:53-161
//   relation weight, sum of both sides  torchbiggraph/batching.py:139-150
//   violator counts                     torchbiggraph/train_cpu.py:98-99
//   d(loss)/d(score)                    (autograd of the above)
// and rewrites the score matrix S_p in place as the coefficient matrix T_p whose two products
// with the operand tiles are the backward pass of the comparator:
//   dot / cos :  T_ij = dS_ij,            T_ii = d(loss)/d(pos score_i)
//   l2        :  T_ij = -dS_ij / S_ij     (= -2 dLoss/d(squared distance)), same on the diagonal
//   squared_l2:  T_ij = 2 dS_ij
// The diagonal of S is always masked, which is what frees it to carry the positive pair.
#include "pbg_common.cuh"

#define LOSS_WARPS 8

__device__ __forceinline__ float softplusf(float x) {           // log(1 + e^x), stable
  return fmaxf(x, 0.f) + log1pf(expf(-fabsf(x)));
}
__device__ __forceinline__ float sigmoidf(float x) { return 1.0f / (1.0f + expf(-x)); }

// column j of the negatives of a chunk: is it ignored, and does it exist at all?
struct ColMask { bool masked; };
__device__ __forceinline__ bool col_masked(const WaveDims &d, const BlockInfo &bi, int enabled, int i, int j) {
  if (!enabled) return true;
  if (j >= d.Pm) return false;                       // uniform negatives are never masked
  if (!d.batch_negs) return true;                    // uniform-only mode: no batch negatives
  return j == i || j >= bi.n;                        // own positive; padding of the last chunk
}

__device__ __forceinline__ float coef_from_dscore(int cmp, float dS, float S) {
  if (cmp == PBG_CMP_L2) return (-S > 1e-15f) ? -dS / S : 0.f;   // clamp at 1e-30 kills the gradient
  if (cmp == PBG_CMP_SQUARED_L2) return 2.0f * dS;
  return dS;
}

__global__ void __launch_bounds__(32 * LOSS_WARPS) loss_kernel(WaveDims d, WaveBatches wb, WaveBufs w) {
  int lane = threadIdx.x & 31;
  long long item = (long long)blockIdx.x * LOSS_WARPS + (threadIdx.x >> 5);
  long long per_prob = (long long)d.nblk * d.Pm;
  if (item >= 2 * per_prob) return;
  int p = (int)(item / per_prob);
  long long rem = item - p * per_prob;
  int lb = (int)(rem / d.Pm), i = (int)(rem - (long long)lb * d.Pm);
  const int blk = d.blk0 + lb;
  BlockInfo bi = block_info(d, wb, blk);
  if (bi.n == 0) return;
  float *S = w.S[p] + ((size_t)blk * d.Pm + i) * d.Ms;
  // bf16-plane tier with dynamic relations: T is an MMA operand, its planes go beside it
  unsigned short *TBr = w.TB[p] ? w.TB[p] + ((size_t)blk * w.npl * d.Pm + i) * w.Kb : nullptr;
  const size_t tplane = (size_t)d.Pm * w.Kb;
  auto put = [&](int j, float t) {
    S[j] = t;
    if (TBr) put_planes1(TBr + j, tplane, t, w.npl);
  };
  size_t prow = (size_t)blk * d.Pm + i;
  const int Mm = d.Mm;
  if (i >= bi.n) {                                   // padded positive: contributes nothing
    for (int j = lane; j < d.Ms; j += 32) put(j, 0.f);
    if (lane == 0) {
      w.lossrow[p][prow] = 0.f; w.violrow[p][prow] = 0;
      if (d.cmp >= PBG_CMP_L2) w.coef[2 + p][prow] = 0.f;
    }
    return;
  }
  const int enabled = d.neg_enabled[p];
  const float s = w.spos[p][prow];
  const float wr = wb.wrel[bi.b] * (w.ew ? w.ew[bi.e0 + i] : 1.0f);   // relation weight x edge weight
  // number of negative columns the reference's score matrix has for this row (masked included)
  const int Mlog = !enabled ? 0 : (d.batch_negs ? bi.Pl + d.U : d.U);
  float lossv = 0.f, ds = 0.f, rowsum = 0.f;
  int viol = 0;

  if (d.loss == PBG_LOSS_SOFTMAX) {
    // -s + log(e^s + sum_j e^S_ij); masked entries are e^-1e9 = 0 (losses.py:143-159)
    float mx = -INFINITY;
    for (int j = lane; j < Mm; j += 32)
      if (!col_masked(d, bi, enabled, i, j)) mx = fmaxf(mx, S[j]);
    mx = warp_max(mx);
    if (Mlog > 0) {
      float m = fmaxf(mx, s);
      if (mx == -INFINITY) m = fmaxf(s, PBG_MASKED);      // every column masked
      float z = 0.f;
      for (int j = lane; j < Mm; j += 32)
        if (!col_masked(d, bi, enabled, i, j)) { z += expf(S[j] - m); viol += S[j] > s; }
      z = warp_sum(z);
      float es = expf(s - m);
      float Z = z + es;
      lossv = -s + m + logf(Z);
      ds = es / Z - 1.0f;
      float invZ = 1.0f / Z;
      for (int j = lane; j < d.Ms; j += 32) {
        float t = 0.f;
        if (j < Mm && !col_masked(d, bi, enabled, i, j)) t = coef_from_dscore(d.cmp, wr * expf(S[j] - m) * invZ, S[j]);
        if (j == i) t = 0.f;                                // filled below
        rowsum += t;
        put(j, t);
      }
    } else {
      for (int j = lane; j < d.Ms; j += 32) put(j, 0.f);    // losses.py:139-140: loss 0, no gradient
    }
  } else if (d.loss == PBG_LOSS_RANKING) {
    // sum_j max(0, margin - s + S_ij) (losses.py:116-122)
    if (Mlog > 0) {
      for (int j = lane; j < d.Ms; j += 32) {
        float t = 0.f;
        if (j < Mm && !col_masked(d, bi, enabled, i, j)) {
          float sj = S[j];
          float v = (sj - s) + d.margin;
          viol += sj > s;
          if (v > 0.f) { lossv += v; ds -= 1.0f; t = coef_from_dscore(d.cmp, wr, sj); }
        }
        rowsum += t;
        put(j, t);
      }
      lossv = warp_sum(lossv);
      ds = warp_sum(ds);
    } else {
      for (int j = lane; j < d.Ms; j += 32) put(j, 0.f);
    }
  } else {
    // softplus(-s) + (1/M) sum_j softplus(S_ij), M counts masked columns (losses.py:61-80)
    float nw = Mlog > 0 ? 1.0f / (float)Mlog : 0.f;
    for (int j = lane; j < d.Ms; j += 32) {
      float t = 0.f;
      if (j < Mm && !col_masked(d, bi, enabled, i, j)) {
        float sj = S[j];
        viol += sj > s;
        lossv += softplusf(sj);
        t = coef_from_dscore(d.cmp, wr * nw * sigmoidf(sj), sj);
      }
      rowsum += t;
      put(j, t);
    }
    lossv = warp_sum(lossv) * nw + softplusf(-s);
    ds = -sigmoidf(-s);
  }
  viol = warp_sum_int(viol);
  rowsum = warp_sum(rowsum);
  // positive pair folded into the diagonal; the positive score of the l2 family is the direct
  // form -sqrt(max(sum (a-b)^2, 1e-30)) (model.py:267-274)
  float tdiag = coef_from_dscore(d.cmp, wr * ds, s);
  __syncwarp();
  if (lane == 0) {
    put(i, tdiag);
    w.lossrow[p][prow] = wr * lossv;
    w.violrow[p][prow] = viol;
    if (d.cmp >= PBG_CMP_L2) w.coef[2 + p][prow] = rowsum + tdiag;
  }
}

// l2 family: column sums of T_p over the chunk's positives (coefficient of the negative row's
// own |b|^2 term).  One thread per column.
__global__ void colsum_kernel(WaveDims d, WaveBatches wb, WaveBufs w) {
  int p = blockIdx.z, blk = d.blk0 + blockIdx.y;
  int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= d.Mm) return;
  BlockInfo bi = block_info(d, wb, blk);
  float s = 0.f;
  const float *T = w.S[p] + (size_t)blk * d.Pm * d.Ms + j;
  for (int i = 0; i < bi.n; ++i) s += T[(size_t)i * d.Ms];
  w.coef[p][(size_t)blk * d.Mm + j] = s;
}

// Standard relations: a chunk row is scored in both problems (as a negative of one, as the
// scored side of the other), and both gradients land on the same prepared row.  One warp per
// (side, block, row m) merges them into the combined coefficient matrix A[side] (see WaveBufs), so
// that the backward pass is ONE product per side with K = Mm, and keeps the row sum of A for the
// l2 family (coefficient of the row's own |y|^2 term).
__global__ void __launch_bounds__(32 * LOSS_WARPS) coef_kernel(WaveDims d, WaveBatches wb, WaveBufs w) {
  int lane = threadIdx.x & 31;
  long long item = (long long)blockIdx.x * LOSS_WARPS + (threadIdx.x >> 5);
  long long per_side = (long long)d.nblk * d.Mm;
  if (item >= 2 * per_side) return;
  int side = (int)(item / per_side);
  long long rem = item - side * per_side;
  int lb = (int)(rem / d.Mm), m = (int)(rem - (long long)lb * d.Mm);
  const int blk = d.blk0 + lb;
  BlockInfo bi = block_info(d, wb, blk);
  if (bi.n == 0) return;
  // side 0 (lhs rows): negatives of problem 0 (columns of T0), scored side of problem 1 (rows of T1)
  const float *Tcol = w.S[side] + (size_t)blk * d.Pm * d.Ms;        // T_side[j][m], j < Pm
  const float *Trow = w.S[1 - side] + ((size_t)blk * d.Pm + m) * d.Ms;   // T_other[m][j], m < Pm
  size_t arow = ((size_t)blk * d.Mm + m) * w.Ma;
  float *A = w.A[side] + arow;
  float rowsum = 0.f;
  // bf16-plane tier: the planes of the row beside it
  unsigned short *ABr = w.AB[side] ? w.AB[side] + ((size_t)blk * w.npl * d.Mm + m) * w.Kb : nullptr;
  for (int j = lane; j < w.Ma; j += 32) {
    float a = 0.f;
    if (j < d.Mm) {
      if (j < bi.n) a += Tcol[(size_t)j * d.Ms + m];
      if (m < bi.n) a += Trow[j];
    }
    rowsum += a;
    A[j] = a;
    if (ABr) put_planes1(ABr + j, (size_t)d.Mm * w.Kb, a, w.npl);
  }
  if (d.cmp >= PBG_CMP_L2) {
    rowsum = warp_sum(rowsum);
    if (lane == 0) w.coef[side][(size_t)blk * d.Mm + m] = rowsum;
  }
}

// Softmax under the dot / cos comparators with at most 32 NV negative columns: the warp keeps the
// row in registers, so the scores are read once, the masks evaluated once and every exponential
// taken once (the general kernel makes three passes).  Same arithmetic, same summation order.
template <int NV>
__global__ void __launch_bounds__(32 * LOSS_WARPS) loss_softmax_kernel(WaveDims d, WaveBatches wb, WaveBufs w) {
  int lane = threadIdx.x & 31;
  long long item = (long long)blockIdx.x * LOSS_WARPS + (threadIdx.x >> 5);
  long long per_prob = (long long)d.nblk * d.Pm;
  if (item >= 2 * per_prob) return;
  int p = (int)(item / per_prob);
  long long rem = item - p * per_prob;
  int lb = (int)(rem / d.Pm), i = (int)(rem - (long long)lb * d.Pm);
  const int blk = d.blk0 + lb;
  BlockInfo bi = block_info(d, wb, blk);
  if (bi.n == 0) return;
  float *S = w.S[p] + ((size_t)blk * d.Pm + i) * d.Ms;
  // bf16-plane tier with dynamic relations: T is an MMA operand, its planes go beside it
  unsigned short *TBr = w.TB[p] ? w.TB[p] + ((size_t)blk * w.npl * d.Pm + i) * w.Kb : nullptr;
  const size_t tplane = (size_t)d.Pm * w.Kb;
  const int npl = w.npl;
  size_t prow = (size_t)blk * d.Pm + i;
  const int Mm = d.Mm;
  const int enabled = d.neg_enabled[p];
  const int Mlog = !enabled ? 0 : (d.batch_negs ? bi.Pl + d.U : d.U);
  if (i >= bi.n || Mlog == 0) {                      // padded positive, or no negatives at all: no loss, no gradient
#pragma unroll
    for (int u = 0; u < NV; ++u) { int j = lane + 32 * u; if (j < d.Ms) S[j] = 0.f; }
    if (TBr)
      for (int j = 2 * lane; j < d.Ms; j += 64) { *(unsigned *)(TBr + j) = 0u; *(unsigned *)(TBr + tplane + j) = 0u; if (npl > 2) *(unsigned *)(TBr + 2 * tplane + j) = 0u; }
    if (lane == 0) { w.lossrow[p][prow] = 0.f; w.violrow[p][prow] = 0; }
    return;
  }
  const float s = w.spos[p][prow];
  const float wr = wb.wrel[bi.b] * (w.ew ? w.ew[bi.e0 + i] : 1.0f);   // relation weight x edge weight
  float sv[NV];
  float mx = -INFINITY;
#pragma unroll
  for (int u = 0; u < NV; ++u) {
    int j = lane + 32 * u;
    bool valid = j < Mm && !col_masked(d, bi, enabled, i, j);
    sv[u] = valid ? S[j] : -INFINITY;
    mx = fmaxf(mx, sv[u]);
  }
  mx = warp_max(mx);
  float m = fmaxf(mx, s);
  if (mx == -INFINITY) m = fmaxf(s, PBG_MASKED);      // every column masked
  float z = 0.f;
  int viol = 0;
#pragma unroll
  for (int u = 0; u < NV; ++u) {
    bool valid = sv[u] != -INFINITY;
    viol += valid && sv[u] > s;
    sv[u] = valid ? expf(sv[u] - m) : 0.f;
    z += sv[u];
  }
  z = warp_sum(z);
  viol = warp_sum_int(viol);
  float es = expf(s - m);
  float Z = z + es;
  float lossv = -s + m + logf(Z);
  float invZ = 1.0f / Z;
  float tdiag = wr * (es / Z - 1.0f);
#pragma unroll
  for (int u = 0; u < NV; ++u) {
    int j = lane + 32 * u;
    if (j < d.Ms) S[j] = j == i ? tdiag : wr * sv[u] * invZ;
  }
  if (TBr) {
    // two column groups at a time: neighbouring lanes swap one group's planes, so that every lane stores
    // two columns of one group (4-byte stores): even lanes (j, j + 1) of group u, odd lanes (j - 1, j) of u + 1
    const bool odd = lane & 1;
#pragma unroll
    for (int u = 0; u < NV; u += 2) {
      const int j0 = lane + 32 * u, j1 = j0 + 32;
      unsigned a[3], b[3], give[3], keep[3];
      bf16_planes(j0 == i ? tdiag : wr * sv[u] * invZ, a[0], a[1], a[2]);
      bf16_planes(j1 == i ? tdiag : wr * sv[u + 1] * invZ, b[0], b[1], b[2]);
#pragma unroll
      for (int q = 0; q < 3; ++q) { give[q] = odd ? a[q] : b[q]; keep[q] = odd ? b[q] : a[q]; }
      unsigned g01 = __shfl_xor_sync(0xffffffffu, give[0] | (give[1] << 16), 1);
      unsigned g2 = __shfl_xor_sync(0xffffffffu, give[2], 1);
      unsigned got[3] = {g01 & 0xffffu, g01 >> 16, g2};
      const int col = (odd ? j1 : j0) & ~1;
      if (col < d.Ms) {
#pragma unroll
        for (int q = 0; q < 3; ++q) {
          unsigned lo = odd ? got[q] : keep[q], hi = odd ? keep[q] : got[q];
          if (q < npl) *(unsigned *)(TBr + q * tplane + col) = lo | (hi << 16);
        }
      }
    }
  }
  if (lane == 0) { w.lossrow[p][prow] = wr * lossv; w.violrow[p][prow] = viol; }
}

// Combined coefficient matrices under the dot / cos comparators, one warp per 32 x 32 tile of
// A[side]: lane l reads 32 consecutive values of row j0 + l of T_side (whole 128-byte lines, eight
// 16-byte loads) and keeps them; value r of every lane is then column j0 + l of output row m0 + r,
// so that both the transposed term and the direct term T_other[m][j] are read and A is written in
// whole lines without a shuffle or shared memory.
template <bool PL>
__global__ void __launch_bounds__(32 * LOSS_WARPS) coef_tile_kernel(WaveDims d, WaveBatches wb, WaveBufs w) {
  int lane = threadIdx.x & 31;
  long long item = (long long)blockIdx.x * LOSS_WARPS + (threadIdx.x >> 5);
  const int tiles = (d.Mm + 31) / 32;
  long long per_side = (long long)d.nblk * tiles * tiles;
  if (item >= 2 * per_side) return;
  int side = (int)(item / per_side);
  long long rem = item - side * per_side;
  int lb = (int)(rem / (tiles * tiles)), tt = (int)(rem - (long long)lb * tiles * tiles);
  int m0 = (tt / tiles) * 32, j0 = (tt % tiles) * 32;
  const int blk = d.blk0 + lb;
  BlockInfo bi = block_info(d, wb, blk);
  if (bi.n == 0) return;
  const int j = j0 + lane;
  float t[32];
  const float *src = w.S[side] + ((size_t)blk * d.Pm + j) * d.Ms + m0;       // T_side[j][m0 ..]
  const bool has = j < bi.n;
#pragma unroll
  for (int q = 0; q < 8; ++q) {
    float4 v = (has && m0 + 4 * q < d.Ms) ? ld4(src + 4 * q) : f4zero();
    t[4 * q] = v.x; t[4 * q + 1] = v.y; t[4 * q + 2] = v.z; t[4 * q + 3] = v.w;
  }
  const float *orow = w.S[1 - side] + (size_t)blk * d.Pm * d.Ms;              // T_other[m][j]
  float *A = w.A[side] + (size_t)blk * d.Mm * w.Ma;
  if (!PL) {
#pragma unroll
    for (int r = 0; r < 32; ++r) {
      int m = m0 + r;
      if (m < d.Mm && j < w.Ma) {
        float a = j < d.Mm ? t[r] : 0.f;
        if (m < bi.n && j < d.Mm) a += orow[(size_t)m * d.Ms + j];
        A[(size_t)m * w.Ma + j] = a;
      }
    }
    return;
  }
  // bf16-plane tier: the three planes instead of the fp32 matrix.  Two rows at a time: neighbouring
  // lanes swap one row's planes, so that every lane stores two columns of one row (4-byte stores):
  // even lanes the columns (j, j + 1) of row m, odd lanes (j - 1, j) of row m + 1.
  unsigned short *AB = w.AB[side] + (size_t)blk * w.npl * d.Mm * w.Kb;
  const size_t aplane = (size_t)d.Mm * w.Kb;
  const int npl = w.npl;
  const bool odd = lane & 1;
#pragma unroll
  for (int r = 0; r < 32; r += 2) {
    unsigned pl[2][3];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      int m = m0 + r + h;
      float a = (m < d.Mm && j < d.Mm) ? t[r + h] : 0.f;
      if (m < bi.n && j < d.Mm) a += orow[(size_t)m * d.Ms + j];
      bf16_planes(a, pl[h][0], pl[h][1], pl[h][2]);
    }
    // what the neighbour stores: its row is m for an even neighbour, m + 1 for an odd one
    unsigned give[3], keep[3];
#pragma unroll
    for (int q = 0; q < 3; ++q) { give[q] = odd ? pl[0][q] : pl[1][q]; keep[q] = odd ? pl[1][q] : pl[0][q]; }
    unsigned g01 = __shfl_xor_sync(0xffffffffu, give[0] | (give[1] << 16), 1);
    unsigned g2 = __shfl_xor_sync(0xffffffffu, give[2], 1);
    unsigned got[3] = {g01 & 0xffffu, g01 >> 16, g2};
    const int m = m0 + r + (odd ? 1 : 0), col = j & ~1;
    if (m < d.Mm && col < w.Kb) {
      unsigned short *dst = AB + (size_t)m * w.Kb + col;
#pragma unroll
      for (int q = 0; q < 3; ++q) {
        unsigned lo = odd ? got[q] : keep[q], hi = odd ? keep[q] : got[q];
        if (q < npl) *(unsigned *)(dst + q * aplane) = lo | (hi << 16);
      }
    }
  }
}

int launch_loss(const WaveDims &d, const WaveBatches &wb, const WaveBufs &w, cudaStream_t st) {
  long long items = 2ll * d.nblk * d.Pm;
  const int loss_ctas = (int)((items + LOSS_WARPS - 1) / LOSS_WARPS);
  const bool dotlike = d.cmp < PBG_CMP_L2;
  if (dotlike && d.loss == PBG_LOSS_SOFTMAX && d.Ms <= 128) loss_softmax_kernel<4><<<loss_ctas, 32 * LOSS_WARPS, 0, st>>>(d, wb, w);
  else if (dotlike && d.loss == PBG_LOSS_SOFTMAX && d.Ms <= 256) loss_softmax_kernel<8><<<loss_ctas, 32 * LOSS_WARPS, 0, st>>>(d, wb, w);
  else if (dotlike && d.loss == PBG_LOSS_SOFTMAX && d.Ms <= 512) loss_softmax_kernel<16><<<loss_ctas, 32 * LOSS_WARPS, 0, st>>>(d, wb, w);
  else if (dotlike && d.loss == PBG_LOSS_SOFTMAX && d.Ms <= 1024) loss_softmax_kernel<32><<<loss_ctas, 32 * LOSS_WARPS, 0, st>>>(d, wb, w);
  else loss_kernel<<<loss_ctas, 32 * LOSS_WARPS, 0, st>>>(d, wb, w);
  if (!d.dynamic) {
    if (dotlike) {
      const int tiles = (d.Mm + 31) / 32;
      long long warps = 2ll * d.nblk * tiles * tiles;
      if (w.AB[0]) coef_tile_kernel<true><<<(int)((warps + LOSS_WARPS - 1) / LOSS_WARPS), 32 * LOSS_WARPS, 0, st>>>(d, wb, w);
      else coef_tile_kernel<false><<<(int)((warps + LOSS_WARPS - 1) / LOSS_WARPS), 32 * LOSS_WARPS, 0, st>>>(d, wb, w);
    } else {
      long long rows = 2ll * d.nblk * d.Mm;
      coef_kernel<<<(int)((rows + LOSS_WARPS - 1) / LOSS_WARPS), 32 * LOSS_WARPS, 0, st>>>(d, wb, w);
    }
    return 2;
  }
  if (d.cmp >= PBG_CMP_L2) {
    dim3 g((d.Mm + 127) / 128, d.nblk, 2);
    colsum_kernel<<<g, 128, 0, st>>>(d, wb, w);
    return 2;
  }
  return 1;
}

// N3 regularizer value (torchbiggraph/regularizers.py:51-97), one warp per positive row of a chunk
// block: coef * sum m^3 over the adjusted rows of the edge -- standard relations: the prepared lhs
// row and the prepared op(rhs) row; dynamic relations: those of both passes (N0, Q0, N1, Q1) -- plus
// the operator parameters: per edge with dynamic relations; once per CHUNK with standard relations
// (sum(params^3) * len(src_pos) where src_pos is the [chunks, P, D] view, regularizers.py:88-92),
// which row 0 of the block carries.  Runs after the gather, on the snapshot the wave reads.
__global__ void __launch_bounds__(32 * LOSS_WARPS) reg_value_kernel(WaveDims d, WaveBatches wb, WaveBufs w) {
  int lane = threadIdx.x & 31;
  long long item = (long long)blockIdx.x * LOSS_WARPS + (threadIdx.x >> 5);
  if (item >= (long long)d.nblk * d.Pm) return;
  int lb = (int)(item / d.Pm), i = (int)(item - (long long)lb * d.Pm);
  const int blk = d.blk0 + lb;
  BlockInfo bi = block_info(d, wb, blk);
  if (bi.n == 0) return;
  size_t prow = (size_t)blk * d.Pm + i;
  float tot = 0.f;
  if (i < bi.n) {
    const bool cplx = d.op == PBG_OP_COMPLEX_DIAGONAL;
    const int D = d.D;
    const float *rows[6];
    int nr = 0;
    rows[nr++] = w.X[ARR_N0] + ((size_t)blk * w.xrows[ARR_N0] + i) * d.Dp;
    rows[nr++] = w.X[ARR_N1] + ((size_t)blk * w.xrows[ARR_N1] + i) * d.Dp;
    if (d.dynamic) {
      rows[nr++] = w.X[ARR_Q0] + ((size_t)blk * w.xrows[ARR_Q0] + i) * d.Dp;
      rows[nr++] = w.X[ARR_Q1] + ((size_t)blk * w.xrows[ARR_Q1] + i) * d.Dp;
    }
    if (d.op != PBG_OP_NONE) {
      if (d.dynamic) {
        long long rl = w.rel[bi.e0 + i];
        if (rl >= 0 && rl < d.num_rels) {
          if (w.theta[0]) rows[nr++] = w.theta[0] + (size_t)rl * D;
          if (w.theta[1]) rows[nr++] = w.theta[1] + (size_t)rl * D;
        }
      } else if (i == 0 && w.theta[0]) {
        rows[nr++] = w.theta[0] + (size_t)wb.rel[bi.b] * D;
      }
    }
    for (int q = 0; q < nr; ++q)
      for (int dd = lane * 4; dd < D; dd += 128) tot += n3_val4(rows[q], dd, D, cplx);
    tot = warp_sum(tot) * d.reg_coef;
  }
  if (lane == 0) w.regrow[prow] = tot;
}

int launch_reg_value(const WaveDims &d, const WaveBatches &wb, const WaveBufs &w, cudaStream_t st) {
  long long items = (long long)d.nblk * d.Pm;
  reg_value_kernel<<<(int)((items + LOSS_WARPS - 1) / LOSS_WARPS), 32 * LOSS_WARPS, 0, st>>>(d, wb, w);
  return 1;
}

// Per-batch Stats (train_cpu.py:95-101): one CTA per batch of the wave sums its rows in a fixed
// order; the running totals of the call live in sum_dev (loss, violators_lhs, violators_rhs, count).
__global__ void __launch_bounds__(256) stats_kernel(WaveDims d, WaveBatches wb, WaveBufs w,
                                                    pbg_batch_stats *per_batch, double *sum) {
  __shared__ double sl[256], sr[256];
  __shared__ long long sv0[256], sv1[256];
  int b = blockIdx.x, t = threadIdx.x;
  double l = 0.0, rg = 0.0;
  long long v0 = 0, v1 = 0;
  int rows = d.Cm * d.Pm;
  for (int r = t; r < rows; r += 256) {
    int c = r / d.Pm, i = r - c * d.Pm;
    int blk = b * d.Cm + c;
    BlockInfo bi = block_info(d, wb, blk);
    if (i >= bi.n) continue;
    size_t prow = (size_t)blk * d.Pm + i;
    l += (double)w.lossrow[0][prow] + (double)w.lossrow[1][prow];
    if (d.reg_coef != 0.f) rg += (double)w.regrow[prow];
    v0 += w.violrow[0][prow];
    v1 += w.violrow[1][prow];
  }
  sl[t] = l; sr[t] = rg; sv0[t] = v0; sv1[t] = v1;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if (t < o) { sl[t] += sl[t + o]; sr[t] += sr[t + o]; sv0[t] += sv0[t + o]; sv1[t] += sv1[t + o]; }
    __syncthreads();
  }
  if (t == 0) {
    pbg_batch_stats s;
    s.loss = (float)sl[0]; s.reg = (float)sr[0]; s.violators_lhs = sv0[0]; s.violators_rhs = sv1[0]; s.count = wb.n[b];
    if (per_batch) per_batch[wb.gidx[b]] = s;
    atomicAdd(&sum[0], sl[0]);
    atomicAdd(&sum[1], (double)sv0[0]);
    atomicAdd(&sum[2], (double)sv1[0]);
    atomicAdd(&sum[3], (double)wb.n[b]);
    atomicAdd(&sum[4], sr[0]);
  }
}

int launch_stats(const WaveDims &d, const WaveBatches &wb, const WaveBufs &w,
                 pbg_batch_stats *per_batch_dev, double *sum_dev, cudaStream_t st) {
  stats_kernel<<<d.k, 256, 0, st>>>(d, wb, w, per_batch_dev, sum_dev);
  return 1;
}

// Scores as the reference returns them (model.py:842-844): [count] positives and
// [count, Pl + U] negatives per side with ignored entries set to -1e9; single batch (wave of 1).
__global__ void export_scores_kernel(WaveDims d, WaveBatches wb, WaveBufs w, float *lhs_pos, float *rhs_pos,
                                     float *lhs_neg, float *rhs_neg) {
  int e = blockIdx.x;                       // edge of the batch
  int p = blockIdx.y;
  BlockInfo b0 = block_info(d, wb, 0);
  int Pl = b0.Pl;
  if (Pl == 0) return;
  int c = e / Pl, i = e - c * Pl;
  BlockInfo bi = block_info(d, wb, c);
  float *pos = p == 0 ? lhs_pos : rhs_pos;
  float *neg = p == 0 ? lhs_neg : rhs_neg;
  size_t prow = (size_t)c * d.Pm + i;
  if (threadIdx.x == 0) pos[e] = w.spos[p][prow];
  if (!d.neg_enabled[p]) return;
  int cols = d.batch_negs ? Pl + d.U : d.U;
  const float *S = w.S[p] + prow * d.Ms;
  for (int j = threadIdx.x; j < cols; j += blockDim.x) {
    int src = d.batch_negs ? (j < Pl ? j : d.Pm + (j - Pl)) : d.Pm + j;
    neg[(size_t)e * cols + j] = col_masked(d, bi, 1, i, src) ? PBG_MASKED : S[src];
  }
}

int launch_export_scores(const WaveDims &d, const WaveBatches &wb, const WaveBufs &w, float *lhs_pos,
                         float *rhs_pos, float *lhs_neg, float *rhs_neg, cudaStream_t st) {
  if (wb.n[0] <= 0) return 0;
  dim3 g(wb.n[0], 2);
  export_scores_kernel<<<g, 128, 0, st>>>(d, wb, w, lhs_pos, rhs_pos, lhs_neg, rhs_neg);
  return 1;
}

// ---- evaluation (RankingEvaluator, torchbiggraph/eval.py:43-81), one batch at a time -------------
// rank of every positive among its negatives, before the loss kernel turns S into coefficients
__global__ void __launch_bounds__(32 * LOSS_WARPS) rank_kernel(WaveDims d, WaveBatches wb, WaveBufs w) {
  int lane = threadIdx.x & 31;
  long long item = (long long)blockIdx.x * LOSS_WARPS + (threadIdx.x >> 5);
  long long per_prob = (long long)d.nblk * d.Pm;
  if (item >= 2 * per_prob) return;
  int p = (int)(item / per_prob);
  long long rem = item - p * per_prob;
  int blk = (int)(rem / d.Pm), i = (int)(rem - (long long)blk * d.Pm);
  BlockInfo bi = block_info(d, wb, blk);
  size_t prow = (size_t)blk * d.Pm + i;
  if (i >= bi.n || !d.neg_enabled[p]) { if (lane == 0) w.rankrow[p][prow] = 0; return; }
  const float *S = w.S[p] + prow * d.Ms;
  const float s = w.spos[p][prow];
  int ge = 0;
  for (int j = lane; j < d.Mm; j += 32) {
    if (j < d.Pm && (!d.batch_negs || j >= bi.Pl)) continue;             // column does not exist in the reference's matrix
    float v = col_masked(d, bi, 1, i, j) ? PBG_MASKED : S[j];
    ge += v >= s;
  }
  ge = warp_sum_int(ge);
  if (lane == 0) w.rankrow[p][prow] = ge + 1;
}

// randomized AUC (torchbiggraph/util.py:415-428): `count` random (positive, negative) pairs per side
__global__ void auc_kernel(WaveDims d, WaveBatches wb, WaveBufs w, double *out8) {
  int p = blockIdx.y;
  int smp = blockIdx.x * blockDim.x + threadIdx.x;
  int count = wb.n[0];
  if (smp >= count || !d.neg_enabled[p]) return;
  BlockInfo b0 = block_info(d, wb, 0);
  int Pl = b0.Pl, cols = d.batch_negs ? Pl + d.U : d.U;
  if (Pl == 0 || cols == 0) return;
  unsigned long long h = pbg_mix64(w.seed ^ pbg_mix64(0xA0C0FFEEull + (unsigned long long)p * 0x10001ull + smp));
  int ei = (int)(h % (unsigned long long)count);
  h = pbg_mix64(h);
  long long flat = (long long)(h % ((unsigned long long)count * cols));
  int er = (int)(flat / cols), j = (int)(flat - (long long)er * cols);
  int src = d.batch_negs ? (j < Pl ? j : d.Pm + (j - Pl)) : d.Pm + j;
  int c = er / Pl, i = er - c * Pl;
  BlockInfo bi = block_info(d, wb, c);
  float neg = col_masked(d, bi, 1, i, src) ? PBG_MASKED : w.S[p][((size_t)c * d.Pm + i) * d.Ms + src];
  float pos = w.spos[p][(size_t)(ei / Pl) * d.Pm + (ei % Pl)];
  if (pos > neg) atomicAdd(&out8[6 + 0], p == 0 ? 1.0 : 0.0), atomicAdd(&out8[7], p == 1 ? 1.0 : 0.0);
}

// out8: loss, pos_rank, mrr, r1, r10, r50 (sums over both sides' ranks), then AUC hit counts per side
__global__ void __launch_bounds__(256) eval_reduce_kernel(WaveDims d, WaveBatches wb, WaveBufs w, double *out8) {
  __shared__ double sm[6][256];
  int t = threadIdx.x;
  double acc[6] = {0, 0, 0, 0, 0, 0};
  int rows = d.Cm * d.Pm;
  for (int r = t; r < rows; r += 256) {
    int c = r / d.Pm, i = r - c * d.Pm;
    BlockInfo bi = block_info(d, wb, c);
    if (i >= bi.n) continue;
    size_t prow = (size_t)c * d.Pm + i;
    acc[0] += (double)w.lossrow[0][prow] + (double)w.lossrow[1][prow];
    for (int p = 0; p < 2; ++p) {
      int rk = w.rankrow[p][prow];
      if (rk <= 0) continue;
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

// call order: gather, score, launch_eval_ranks (this), launch_loss, launch_eval_reduce
int launch_eval(const WaveDims &d, const WaveBatches &wb, const WaveBufs &w, double *out8_dev, cudaStream_t st) {
  long long items = 2ll * d.nblk * d.Pm;
  cudaMemsetAsync(out8_dev, 0, 8 * sizeof(double), st);
  rank_kernel<<<(int)((items + LOSS_WARPS - 1) / LOSS_WARPS), 32 * LOSS_WARPS, 0, st>>>(d, wb, w);
  dim3 g((wb.n[0] + 127) / 128, 2);
  auc_kernel<<<g, 128, 0, st>>>(d, wb, w, out8_dev);
  loss_kernel<<<(int)((items + LOSS_WARPS - 1) / LOSS_WARPS), 32 * LOSS_WARPS, 0, st>>>(d, wb, w);
  eval_reduce_kernel<<<1, 256, 0, st>>>(d, wb, w, out8_dev);
  return 4;
}
