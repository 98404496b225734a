// fp32 contractions on the CUDA cores (precision tier PBG_PREC_FP32): exact-fp32 counterparts of
// the torch.bmm / baddbmm calls of the reference comparators (torchbiggraph/model.py:179-180,
// 226-236) and of the four bmm calls autograd issues for them in the backward pass.
//
//   score  : S_p[blk] (Pm x Mm)  = Q_p[blk] (Pm x D) . N_p[blk]^T            (+ l2 epilogue)
//   grad Q : GQ_p[blk] (Pm x D)  = T_p[blk] (Pm x Mm) . N_p[blk] (Mm x D)
//   grad N : GN_p[blk] (Mm x D)  = T_p[blk]^T (Mm x Pm) . Q_p[blk] (Pm x D)
//
// One generic tile kernel: CTA tile BM x 64 x 16, 256 threads, (BM/16) x 4 outputs per thread,
// operands staged through shared memory as [k][m] / [k][n] so that the inner product reads
// 16-byte vectors without bank conflicts.  Either operand may be stored k-contiguous (transposed
// while staging) or m/n-contiguous (copied as is).
#include <cstring>

#include "pbg_common.cuh"

#define BN 64
#define BK 16

struct GemmTask {
  const float *A; long long a_blk; int lda;   // per-block stride (floats), leading dimension
  const float *B; long long b_blk; int ldb;
  long long b_rel;                            // added to B per block: relation of the block's batch * b_rel (operator tables)
  float *C; long long c_blk; int ldc;
  int M, N, K;
  // score epilogue
  const float *auxA; long long auxa_blk;      // |a|^2 per A row   (l2 family)
  const float *auxB; long long auxb_blk;      // |b|^2 per B row
  int cmp;
};
struct GemmTasks { GemmTask t[2]; };

template <int BM, bool A_KCONTIG, bool B_KCONTIG, bool SCORE>
__global__ void __launch_bounds__(256) gemm_tile_kernel(GemmTasks tasks, WaveDims d, WaveBatches wb) {
  constexpr int TM = BM / 16;
  __shared__ __align__(16) float As[BK][BM + 4];
  __shared__ __align__(16) float Bs[BK][BN + 4];
  int p = blockIdx.z & 1, blk = d.blk0 + (blockIdx.z >> 1);
  {
    BlockInfo bi = block_info(d, wb, blk);
    if (bi.n == 0) return;                          // chunk without edges
    if (SCORE && !d.neg_enabled[p]) return;         // no negatives on this side: nothing to score
  }
  const GemmTask &t = tasks.t[p];
  if (t.M <= 0) return;
  const float *A = t.A + (size_t)blk * t.a_blk, *B = t.B + (size_t)blk * t.b_blk;
  if (t.b_rel) B += (size_t)wb.rel[blk / d.Cm] * t.b_rel;
  float *C = t.C + (size_t)blk * t.c_blk;
  const int M = t.M, N = t.N, K = t.K;
  int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  if (m0 >= M || n0 >= N) return;
  int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  float acc[TM][4];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
    // ---- stage A ----
    if (A_KCONTIG) {   // A[m][k], k contiguous: BM rows x 16 k = BM*4 float4
#pragma unroll
      for (int it = 0; it < (BM * 4) / 256; ++it) {
        int idx = tid + it * 256, row = idx >> 2, kq = (idx & 3) * 4;
        float4 v = f4zero();
        if (m0 + row < M && k0 + kq < K) {
          v = ld4(A + (size_t)(m0 + row) * t.lda + k0 + kq);
          if (k0 + kq + 1 >= K) v.y = 0.f;
          if (k0 + kq + 2 >= K) v.z = 0.f;
          if (k0 + kq + 3 >= K) v.w = 0.f;
        }
        As[kq + 0][row] = v.x; As[kq + 1][row] = v.y; As[kq + 2][row] = v.z; As[kq + 3][row] = v.w;
      }
    } else {           // A[k][m], m contiguous: 16 k rows x BM = BM*4 float4
#pragma unroll
      for (int it = 0; it < (BM * 4) / 256; ++it) {
        int idx = tid + it * 256, kr = idx / (BM / 4), c4 = (idx % (BM / 4)) * 4;
        float4 v = f4zero();
        if (k0 + kr < K && m0 + c4 < M) {
          v = ld4(A + (size_t)(k0 + kr) * t.lda + m0 + c4);
          if (m0 + c4 + 1 >= M) v.y = 0.f;
          if (m0 + c4 + 2 >= M) v.z = 0.f;
          if (m0 + c4 + 3 >= M) v.w = 0.f;
        }
        st4(&As[kr][c4], v);
      }
    }
    // ---- stage B ----
    if (B_KCONTIG) {   // B[n][k]
      int row = tid >> 2, kq = (tid & 3) * 4;
      float4 v = f4zero();
      if (n0 + row < N && k0 + kq < K) {
        v = ld4(B + (size_t)(n0 + row) * t.ldb + k0 + kq);
        if (k0 + kq + 1 >= K) v.y = 0.f;
        if (k0 + kq + 2 >= K) v.z = 0.f;
        if (k0 + kq + 3 >= K) v.w = 0.f;
      }
      Bs[kq + 0][row] = v.x; Bs[kq + 1][row] = v.y; Bs[kq + 2][row] = v.z; Bs[kq + 3][row] = v.w;
    } else {           // B[k][n]
      int kr = tid >> 4, c4 = (tid & 15) * 4;
      float4 v = f4zero();
      if (k0 + kr < K && n0 + c4 < N) {
        v = ld4(B + (size_t)(k0 + kr) * t.ldb + n0 + c4);
        if (n0 + c4 + 1 >= N) v.y = 0.f;
        if (n0 + c4 + 2 >= N) v.z = 0.f;
        if (n0 + c4 + 3 >= N) v.w = 0.f;
      }
      st4(&Bs[kr][c4], v);
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[TM];
#pragma unroll
      for (int i = 0; i < TM; i += 4) {
        float4 v = ld4(&As[kk][ty * TM + i]);
        a[i] = v.x; a[i + 1] = v.y; a[i + 2] = v.z; a[i + 3] = v.w;
      }
      float4 b = ld4(&Bs[kk][tx * 4]);
#pragma unroll
      for (int i = 0; i < TM; ++i) {
        acc[i][0] = fmaf(a[i], b.x, acc[i][0]);
        acc[i][1] = fmaf(a[i], b.y, acc[i][1]);
        acc[i][2] = fmaf(a[i], b.z, acc[i][2]);
        acc[i][3] = fmaf(a[i], b.w, acc[i][3]);
      }
    }
    __syncthreads();
  }
  // ---- epilogue ----
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    int m = m0 + ty * TM + i;
    if (m >= M) continue;
    float an = 0.f;
    if (SCORE && t.cmp >= PBG_CMP_L2) an = t.auxA[(size_t)blk * t.auxa_blk + m];
    float out[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int n = n0 + tx * 4 + j;
      float v = acc[i][j];
      if (SCORE && t.cmp >= PBG_CMP_L2 && n < N) {
        // model.py:226-246: (|b|^2 - 2 a.b) + |a|^2, then clamp/sqrt for l2, negated
        float q = (t.auxB[(size_t)blk * t.auxb_blk + n] - 2.0f * v) + an;
        v = t.cmp == PBG_CMP_L2 ? -sqrtf(fmaxf(q, 1e-30f)) : -q;
      }
      out[j] = v;
    }
    int n = n0 + tx * 4;
    float *c = C + (size_t)m * t.ldc + n;
    if (n + 3 < N) st4(c, make_float4(out[0], out[1], out[2], out[3]));
    else
      for (int j = 0; j < 4 && n + j < N; ++j) c[j] = out[j];
  }
}

template <bool A_KCONTIG, bool B_KCONTIG, bool SCORE>
static void launch_tiles(const GemmTasks &ts, const WaveDims &d, const WaveBatches &wb, cudaStream_t st) {
  int M = ts.t[0].M, N = ts.t[0].N;
  if (M <= 64) {
    dim3 g((N + BN - 1) / BN, (M + 63) / 64, d.nblk * 2);
    gemm_tile_kernel<64, A_KCONTIG, B_KCONTIG, SCORE><<<g, 256, 0, st>>>(ts, d, wb);
  } else {
    dim3 g((N + BN - 1) / BN, (M + 127) / 128, d.nblk * 2);
    gemm_tile_kernel<128, A_KCONTIG, B_KCONTIG, SCORE><<<g, 256, 0, st>>>(ts, d, wb);
  }
}

int launch_score_simt(const WaveDims &d, const WaveBatches &wb, const WaveBufs &w, cudaStream_t st) {
  GemmTasks ts;
  for (int p = 0; p < 2; ++p) {
    GemmTask &t = ts.t[p];
    int q = ARR_Q0 + p, n = ARR_N0 + p;
    t.A = w.X[q]; t.a_blk = (long long)w.xrows[q] * d.Dp; t.lda = d.Dp;
    t.B = w.X[n]; t.b_blk = (long long)w.xrows[n] * d.Dp; t.ldb = d.Dp;
    t.C = w.S[p]; t.c_blk = (long long)d.Pm * d.Ms; t.ldc = d.Ms;
    t.M = d.Pm; t.N = d.Mm; t.K = d.D;
    t.b_rel = 0;
    t.auxA = w.aux[q]; t.auxa_blk = w.xrows[q];
    t.auxB = w.aux[n]; t.auxb_blk = w.xrows[n];
    t.cmp = d.cmp;
  }
  launch_tiles<true, true, true>(ts, d, wb, st);
  return 1;
}

int launch_grad_simt(const WaveDims &d, const WaveBatches &wb, const WaveBufs &w, cudaStream_t st) {
  if (!d.dynamic) {            // GN_side = A[side] . N_(1-side): one product per side, K = Mm
    GemmTasks tm;
    for (int side = 0; side < 2; ++side) {
      GemmTask &t = tm.t[side];
      int o = ARR_N0 + (1 - side);
      t.A = w.A[side]; t.a_blk = (long long)d.Mm * w.Ma; t.lda = w.Ma;
      t.B = w.X[o]; t.b_blk = (long long)w.xrows[o] * d.Dp; t.ldb = d.Dp;
      t.C = w.GX[ARR_N0 + side]; t.c_blk = (long long)d.Mm * d.Dp; t.ldc = d.Dp;
      t.M = d.Mm; t.N = d.D; t.K = d.Mm;
      t.b_rel = 0;
      t.auxA = t.auxB = nullptr; t.auxa_blk = t.auxb_blk = 0; t.cmp = 0;
    }
    launch_tiles<true, false, false>(tm, d, wb, st);
    return 1;
  }
  GemmTasks tq, tn;
  for (int p = 0; p < 2; ++p) {
    int q = ARR_Q0 + p, n = ARR_N0 + p;
    GemmTask &a = tq.t[p];       // GQ_p = T_p . N_p
    a.A = w.S[p]; a.a_blk = (long long)d.Pm * d.Ms; a.lda = d.Ms;
    a.B = w.X[n]; a.b_blk = (long long)w.xrows[n] * d.Dp; a.ldb = d.Dp;
    a.C = w.GX[q]; a.c_blk = (long long)w.grows[q] * d.Dp; a.ldc = d.Dp;
    a.M = d.Pm; a.N = d.D; a.K = d.Mm;
    a.b_rel = 0;
    a.auxA = a.auxB = nullptr; a.auxa_blk = a.auxb_blk = 0; a.cmp = 0;
    GemmTask &b = tn.t[p];       // GN_p = T_p^T . Q_p
    b.A = w.S[p]; b.a_blk = (long long)d.Pm * d.Ms; b.lda = d.Ms;
    b.B = w.X[q]; b.b_blk = (long long)w.xrows[q] * d.Dp; b.ldb = d.Dp;
    b.C = w.GX[n]; b.c_blk = (long long)w.grows[n] * d.Dp; b.ldc = d.Dp;
    b.M = d.Mm; b.N = d.D; b.K = d.Pm;
    b.b_rel = 0;
    b.auxA = b.auxB = nullptr; b.auxa_blk = b.auxb_blk = 0; b.cmp = 0;
  }
  launch_tiles<true, false, false>(tq, d, wb, st);
  launch_tiles<false, false, false>(tn, d, wb, st);
  return 2;
}

// ---- linear / affine operators (standard relations): the operator is a D x D matrix A per relation ----
static void matrix_task(GemmTasks &ts, const float *A, long long a_blk, int lda, const float *B, long long b_blk, int ldb,
                        long long b_rel, float *C, long long c_blk, int ldc, int M, int N, int K) {
  memset(&ts, 0, sizeof ts);
  GemmTask &t = ts.t[0];
  t.A = A; t.a_blk = a_blk; t.lda = lda; t.B = B; t.b_blk = b_blk; t.ldb = ldb; t.b_rel = b_rel;
  t.C = C; t.c_blk = c_blk; t.ldc = ldc; t.M = M; t.N = N; t.K = K;
  ts.t[1] = t;
  ts.t[1].M = 0;                                  // only "problem 0" does work
}

// R2[blk] (Mm x D) = R1[blk] (raw rhs rows) . A^T : z_i = sum_j A[i][j] x_j  (operators.py:88-99)
int launch_matrix_forward(const WaveDims &d, const WaveBatches &wb, const WaveBufs &w, cudaStream_t st) {
  GemmTasks ts;
  long long blk = (long long)d.Mm * d.Dp;
  matrix_task(ts, w.R1, blk, d.Dp, w.theta[0], 0, d.D, d.opw, w.R2, blk, d.Dp, d.Mm, d.D, d.D);
  launch_tiles<true, true, false>(ts, d, wb, st);
  return 1;
}

// GN1 holds d(loss)/dz for every rhs row (after launch_gz_rows):
//   R2[blk] = GN1[blk] . A          gradient w.r.t. the raw rows      (gx_j = sum_i gz_i A[i][j])
//   dA[b]   = GN1[b]^T . R1[b]      gradient of the operator matrix   (dA[i][j] = sum_rows gz_i x_j), one product per batch
int launch_matrix_backward(const WaveDims &d, const WaveBatches &wb, const WaveBufs &w, cudaStream_t st) {
  GemmTasks ts;
  long long blk = (long long)d.Mm * d.Dp;
  matrix_task(ts, w.GX[ARR_N1], blk, d.Dp, w.theta[0], 0, d.D, d.opw, w.R2, blk, d.Dp, d.Mm, d.D, d.D);
  launch_tiles<true, false, false>(ts, d, wb, st);
  // per batch: treat the Cm chunk blocks of a batch as one block of Cm*Mm rows
  WaveDims db = d;
  db.Cm = 1; db.blk0 = d.blk0 / d.Cm; db.nblk = d.nblk / d.Cm;
  long long bstride = (long long)d.Cm * d.Mm * d.Dp;
  matrix_task(ts, w.GX[ARR_N1], bstride, d.Dp, w.R1, bstride, d.Dp, 0, w.dA, d.opw, d.D, d.D, d.D, d.Cm * d.Mm);
  launch_tiles<false, false, false>(ts, db, wb, st);
  return 2;
}
