// Shared declarations of the sm_100a training-step library: wave layout in HBM, decoding of
// row slots, and the small device helpers every kernel uses.
//
// Vocabulary (PyTorch-BigGraph's): a *bucket* is a (lhs partition, rhs partition) pair; a
// *batch* is batch_size edges; a batch is cut into *chunks* of P = num_batch_negs edges which
// serve as each other's negatives, plus U uniformly drawn negative rows per chunk
// (torchbiggraph/model.py:508-622).  A *wave* is the k batches this library keeps in flight.
//
// Layout of one wave in the workspace (all float32, row stride Dp = dim rounded up to 32):
//   block blk = b * Cm + c        (b-th batch of the wave, c-th chunk, Cm chunks per batch)
//   N0[blk][Mm][Dp]  prepared lhs rows: Pm chunk rows then U uniform rows   (Mm = Pm + U)
//   N1[blk][Mm][Dp]  prepared rhs rows: Pm chunk rows then U uniform rows
//   Q0[blk][Pm][Dp]  rows scored against N0 (the "lhs corrupted" problem 0)
//   Q1[blk][Pm][Dp]  rows scored against N1 (the "rhs corrupted" problem 1)
// Standard relations (operator on the rhs only): Q0 is the first Pm rows of N1 and Q1 the first
// Pm rows of N0 (aliases).  Dynamic relations: N0/N1 hold rows WITHOUT operator, Q0 holds
// op_rhs[rel](rhs rows), Q1 holds op_lhs[rel](lhs rows) (model.py:705-758).
//   S_p[blk][Pm][Ms]   scores of problem p, later overwritten by the coefficient matrix T_p
//   dynamic relations:  GN_p[blk][Mm][Dp] = T_p^T . Q_p      GQ_p[blk][Pm][Dp] = T_p . N_p
//   standard relations: GN0 = A[0] . N1,  GN1 = A[1] . N0  with the combined matrices A (WaveBufs)
// T_p holds d(loss)/d(score) with the gradient of the positive score folded into its (masked,
// otherwise unused) diagonal, so the two products above are the whole backward of the
// comparator.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <mutex>
#include <map>
#include <utility>
#include "../../include/pbg_b200.h"

#define PBG_KMAX 32                 // most batches in one wave
#define PBG_MASKED (-1e9f)          // torchbiggraph/model.py:836-839
#define PBG_ADAGRAD_EPS 1e-10f      // row_adagrad.py:94, async_adagrad.py:84

enum { ARR_N0 = 0, ARR_N1 = 1, ARR_Q0 = 2, ARR_Q1 = 3, ARR_R0 = 4, ARR_R1 = 5 };

struct WaveDims {
  int D, Dp;            // dim, workspace row stride (floats)
  int Pm, U, Mm, Ms;    // chunk slots, uniform negatives, Pm+U, score row stride
  int Cm;               // chunks per batch (max)
  int k, nblk;          // batches in this wave; chunk blocks THIS LAUNCH covers (k*Cm for a whole wave)
  int blk0;             // first chunk block of this launch (a wave may be launched in two parts)
  int op, cmp, loss, dynamic;
  int batch_negs;       // 1: batch_uniform mode, 0: uniform-only mode (num_batch_negs == 0)
  int neg_enabled[2];   // problem 0 = lhs negatives, problem 1 = rhs negatives
  int num_batch_negs;
  int spb;              // occurrence slots per batch (see occ_decode)
  int nocc;             // k * spb
  float margin;
  float reg_coef;       // N3 regularizer weight, 0 = off
  float max_norm;       // > 0: looked-up rows longer than this are used (and kept) scaled to it
  long long n_rows[2];  // rows of the lhs / rhs table
  int shared_table;     // lhs and rhs read the same table
  int num_rels;
  int matrix_op;        // operator is linear / affine (standard relations): applied by contractions, not in the gather
  int opw;              // floats per operator-table row: D, or D*D (+ D) for linear (affine)
  unsigned long long key_rel_base;   // first sort key of operator-table rows
  unsigned long long key_invalid;    // sort key of slots that carry no gradient
};

struct WaveBatches {
  long long off[PBG_KMAX];    // first edge of the batch in the edge arrays
  long long gidx[PBG_KMAX];   // index of the batch in the call (uniform-id array, stats, RNG)
  int n[PBG_KMAX];            // edges in the batch
  int rel[PBG_KMAX];          // relation of the batch (standard mode)
  float wrel[PBG_KMAX];       // relation weight of the batch
};

struct WaveBufs {
  float *X[4];       int xrows[4];   // operand arrays N0,N1,Q0,Q1 (rows per block; aliases allowed)
  float *aux[4];                     // per operand row: cos -> 1/|z|, l2 -> |y|^2 (indexed like X)
  float *GX[4];      int grows[4];   // gradient arrays GN0,GN1,GQ0,GQ1
  float *GR[2];                      // dynamic relations with an operator: per edge the gradient of its operator row,
                                     // [0] rhs table (slots ARR_R0), [1] lhs table (ARR_R1), rows like GQ; null: not kept
  float *S[2];                       // scores / coefficient matrices
  // Standard relations: combined coefficient matrices, one per side, [nblk][Mm][Ma]:
  //   A[0][m][j] = (j < Pm ? T0[j][m] : 0) + (m < Pm ? T1[m][j] : 0)   gradient of the lhs rows  = A[0] . N1
  //   A[1][m][j] = (j < Pm ? T1[j][m] : 0) + (m < Pm ? T0[m][j] : 0)   gradient of the rhs rows  = A[1] . N0
  float *A[2];
  int Ma;                            // row stride of A (Mm rounded up to 4)
  // bf16-plane tier: every fp32 operand value as three bf16 planes b0 + b1 + b2 (b0 = bf16(x), b1 =
  // bf16(x - b0), b2 = bf16(x - b0 - b1)); the contractions read these instead of X / A
  //   XB[a]     [nblk][3][xrows[a]][Dpb]   planes of the operand rows N0, N1, Q0, Q1 (aliased like X)
  //   AB[side]  [nblk][3][Mm][Kb]          planes of the merged coefficient matrices (standard relations)
  //   TB[p]     [nblk][3][Pm][Kb]          planes of the coefficient matrices T_p (dynamic relations)
  //                                          (also standard relations with the fused score / loss kernel; AB is then unused)
  unsigned short *XB[4], *AB[2], *TB[2];     // null outside that tier
  int Dpb, Kb;                       // row strides in elements (D and Mm rounded up to 8: 16-byte rows)
  int npl;                           // planes per value: 3 (bf16x6: all six products of order <= 2) or 2 (bf16x3: b0.b0 + b0.b1 + b1.b0)
  float *spos[2];                    // positive scores [nblk][Pm]
  float *coef[4];                    // l2: colsum(T0), colsum(T1), rowsum(T0), rowsum(T1)
  float *lossrow[2];                 // per positive row: weighted loss term
  float *rscale;                     // max_norm: scale applied to the raw row of every N1 slot [blk][Mm] (1 = none)
  float *regrow;                     // per positive row: its share of the N3 regularizer (reg_coef != 0)
  int *violrow[2];                   // per positive row: #(neg > pos)
  int *rankrow[2];                   // evaluation: per positive row, 1 + #(neg >= pos)
  const long long *lhs, *rhs, *rel;  // edge arrays
  const float *ew;                  // per-edge weights parallel to the edge arrays, or null
  const long long *ul, *ur;          // uniform ids [batches][Cm][U] or null
  unsigned long long seed;
  float *W[2], *G[2];                // embedding tables / RowAdagrad state (lhs, rhs)
  float *theta[2], *acc[2];          // operator tables: [0] applied to rhs rows, [1] to lhs rows
  // linear / affine operators: R1 = raw rhs rows, R2 = A.x (forward) then g.A (backward), both laid
  // out like N1; dA = per-batch gradient of the operator row [k][opw]
  float *R1, *R2, *dA;
  float *relpart;                    // standard mode: [k][Cm][D] partial operator gradients
  float *glob[2], *gacc[2];          // global embedding of the lhs / rhs entity type + AsyncAdagrad accumulator, or null
  int glob_shared;                   // both sides are of one entity type: glob[0] == glob[1], one step per batch
  float *globpart;                   // [blk][side][warp][D] partial sums of the row gradients (global-embedding gradient)
  int *errflag;                      // device error word (bit 0: id out of range)
};

struct BlockInfo { int b, c, Pl, n; long long e0; };

// Which batch/chunk a block is, its logical chunk size Pl = min(num_batch_negs or U, batch
// edges) (model.py:648-656) and how many of its Pm slots hold real edges.
__device__ __forceinline__ BlockInfo block_info(const WaveDims &d, const WaveBatches &wb, int blk) {
  BlockInfo bi;
  bi.b = blk / d.Cm;
  bi.c = blk - bi.b * d.Cm;
  int nb = wb.n[bi.b];
  int lim = d.batch_negs ? d.num_batch_negs : d.U;
  bi.Pl = nb < lim ? nb : lim;
  int first = bi.c * bi.Pl;
  int n = nb - first;
  bi.n = bi.Pl > 0 ? (n < 0 ? 0 : (n > bi.Pl ? bi.Pl : n)) : 0;
  bi.e0 = wb.off[bi.b] + first;
  return bi;
}

// Counter-based generator for device-drawn uniform negatives (stands where the reference
// calls torch.randint, model.py:70-75): splitmix64 of (seed, batch, side, chunk, j).
__device__ __forceinline__ unsigned long long pbg_mix64(unsigned long long z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}
__device__ __forceinline__ long long pbg_uniform_id(unsigned long long seed, long long gidx, int side,
                                                    int c, int j, long long nrows) {
  unsigned long long h = pbg_mix64(seed ^ pbg_mix64((unsigned long long)gidx * 2ull + (unsigned)side));
  h = pbg_mix64(h + ((unsigned long long)(unsigned)c << 32) + (unsigned)j);
  return (long long)__umul64hi(h, (unsigned long long)nrows);
}

// Table row behind slot r of block (b, c) on `side` (0 lhs, 1 rhs); -1 when the slot is empty.
__device__ __forceinline__ long long slot_row(const WaveDims &d, const WaveBatches &wb, const WaveBufs &w,
                                              const BlockInfo &bi, int side, int r) {
  if (r < d.Pm) {
    if (r >= bi.n) return -1;
    return side == 0 ? w.lhs[bi.e0 + r] : w.rhs[bi.e0 + r];
  }
  if (bi.n == 0 || !d.neg_enabled[side]) return -1;
  int j = r - d.Pm;
  const long long *u = side == 0 ? w.ul : w.ur;
  if (u) return u[(wb.gidx[bi.b] * d.Cm + bi.c) * (long long)d.U + j];
  return pbg_uniform_id(w.seed, wb.gidx[bi.b], side, bi.c, j, d.n_rows[side]);
}

// Occurrence index o -> (batch b, array a, block, row).  Per batch the slots are enumerated
// [N0: Cm*Mm | N1: Cm*Mm | Q0: Cm*Pm | Q1: Cm*Pm | R0: Cm*Pm | R1: Cm*Pm]; the Q slots and R0/R1
// (operator-table rows touched through Q0/Q1) exist only with dynamic relations -- with standard
// relations a chunk row has ONE gradient slot, in GN0 / GN1.  Enumeration is batch-major so that
// a stable sort by row keeps a row's occurrences in batch order.
struct Occ { int b, a, blk, r; };
__device__ __forceinline__ Occ occ_decode(const WaveDims &d, int o) {
  Occ q;
  q.b = o / d.spb;
  int w = o - q.b * d.spb;
  int nN = d.Cm * d.Mm, nQ = d.dynamic ? d.Cm * d.Pm : 0;   // standard relations: N slots only
  int rows;
  if (w < nN) { q.a = ARR_N0; rows = d.Mm; }
  else if ((w -= nN) < nN) { q.a = ARR_N1; rows = d.Mm; }
  else if ((w -= nN) < nQ) { q.a = ARR_Q0; rows = d.Pm; }
  else if ((w -= nQ) < nQ) { q.a = ARR_Q1; rows = d.Pm; }
  else if ((w -= nQ) < nQ) { q.a = ARR_R0; rows = d.Pm; }
  else { w -= nQ; q.a = ARR_R1; rows = d.Pm; }
  int c = w / rows;
  q.r = w - c * rows;
  q.blk = q.b * d.Cm + c;
  return q;
}

// N3 regularizer pieces at elements [dd, dd + 4) of a row y: the term is sum m^3 with m = |y_d|, or for
// complex_diagonal the modulus of the pair (y_d, y_{d +- D/2}) counted once per pair
// (torchbiggraph/operators.py:42-43, 151-157).  n3_grad4: d(sum m^3)/dy = 3 m y.
__device__ __forceinline__ float4 n3_grad4(const float *y, int dd, int D, bool cplx) {
  float4 v = *reinterpret_cast<const float4 *>(y + dd);
  if (!cplx) return make_float4(3.f * fabsf(v.x) * v.x, 3.f * fabsf(v.y) * v.y, 3.f * fabsf(v.z) * v.z, 3.f * fabsf(v.w) * v.w);
  int h = D >> 1;
  float4 p = *reinterpret_cast<const float4 *>(y + (dd < h ? dd + h : dd - h));
  return make_float4(3.f * sqrtf(v.x * v.x + p.x * p.x) * v.x, 3.f * sqrtf(v.y * v.y + p.y * p.y) * v.y,
                     3.f * sqrtf(v.z * v.z + p.z * p.z) * v.z, 3.f * sqrtf(v.w * v.w + p.w * p.w) * v.w);
}
__device__ __forceinline__ float n3_val4(const float *y, int dd, int D, bool cplx) {
  float4 v = *reinterpret_cast<const float4 *>(y + dd);
  if (!cplx) { float a = fabsf(v.x), b = fabsf(v.y), c = fabsf(v.z), e = fabsf(v.w); return a * a * a + b * b * b + c * c * c + e * e * e; }
  int h = D >> 1;
  if (dd >= h) return 0.f;                                  // the pair is counted at its real part
  float4 p = *reinterpret_cast<const float4 *>(y + dd + h);
  float a = sqrtf(v.x * v.x + p.x * p.x), b = sqrtf(v.y * v.y + p.y * p.y), c = sqrtf(v.z * v.z + p.z * p.z), e = sqrtf(v.w * v.w + p.w * p.w);
  return a * a * a + b * b * b + c * c * c + e * e * e;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ int warp_sum_int(int v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float4 ld4(const float *p) { return *reinterpret_cast<const float4 *>(p); }
__device__ __forceinline__ void st4(float *p, float4 v) { *reinterpret_cast<float4 *>(p) = v; }
__device__ __forceinline__ float4 f4zero() { return make_float4(0.f, 0.f, 0.f, 0.f); }
__device__ __forceinline__ float4 operator+(float4 a, float4 b) { return make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w); }
__device__ __forceinline__ float4 operator-(float4 a, float4 b) { return make_float4(a.x - b.x, a.y - b.y, a.z - b.z, a.w - b.w); }
__device__ __forceinline__ float4 operator*(float4 a, float4 b) { return make_float4(a.x * b.x, a.y * b.y, a.z * b.z, a.w * b.w); }
__device__ __forceinline__ float4 operator*(float4 a, float s) { return make_float4(a.x * s, a.y * s, a.z * s, a.w * s); }
__device__ __forceinline__ float f4dot(float4 a, float4 b) { return a.x * b.x + a.y * b.y + a.z * b.z + a.w * b.w; }
__device__ __forceinline__ float f4sum(float4 a) { return a.x + a.y + a.z + a.w; }
// tf32(x): round to nearest, 10 mantissa bits kept -- the part of x a kind::tf32 MMA sees exactly
__device__ __forceinline__ float tf32_hi(float x) {
  uint32_t u;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(x));
  return __uint_as_float(u);
}
__device__ __forceinline__ float4 tf32_hi4(float4 v) { return make_float4(tf32_hi(v.x), tf32_hi(v.y), tf32_hi(v.z), tf32_hi(v.w)); }
// The same rounding with two integer instructions (add half an ulp of the 10-bit mantissa, clear the
// low 13 bits): cvt runs at a fraction of the ALU rate, which is what bounds a kernel that splits
// whole operand tiles.  Differs from cvt only on NaN payloads and when rounding carries into Inf.
// The three bf16 planes of x (round to nearest each time; the remainders are exact in fp32):
// float(b0) + float(b1) + float(b2) == x to 24 mantissa bits.
__device__ __forceinline__ void bf16_planes(float x, unsigned &b0, unsigned &b1, unsigned &b2) {
  __nv_bfloat16 h0 = __float2bfloat16_rn(x);
  float r = x - __bfloat162float(h0);
  __nv_bfloat16 h1 = __float2bfloat16_rn(r);
  r -= __bfloat162float(h1);
  b0 = __bfloat16_as_ushort(h0); b1 = __bfloat16_as_ushort(h1); b2 = __bfloat16_as_ushort(__float2bfloat16_rn(r));
}
// planes of four consecutive values, packed for one 8-byte store per plane
__device__ __forceinline__ void bf16_planes4(float4 v, uint2 &p0, uint2 &p1, uint2 &p2) {
  unsigned a0, a1, a2, b0, b1, b2, c0, c1, c2, d0, d1, d2;
  bf16_planes(v.x, a0, a1, a2); bf16_planes(v.y, b0, b1, b2); bf16_planes(v.z, c0, c1, c2); bf16_planes(v.w, d0, d1, d2);
  p0 = make_uint2(a0 | (b0 << 16), c0 | (d0 << 16));
  p1 = make_uint2(a1 | (b1 << 16), c1 | (d1 << 16));
  p2 = make_uint2(a2 | (b2 << 16), c2 | (d2 << 16));
}
// one value's planes into a plane array: p0 at dst, the others one / two plane strides further
__device__ __forceinline__ void put_planes1(unsigned short *dst, size_t plane, float v, int npl) {
  unsigned b0, b1, b2;
  bf16_planes(v, b0, b1, b2);
  dst[0] = (unsigned short)b0; dst[plane] = (unsigned short)b1;
  if (npl > 2) dst[2 * plane] = (unsigned short)b2;
}
__device__ __forceinline__ float tf32_round(float x) { return __uint_as_float((__float_as_uint(x) + 0x1000u) & 0xFFFFE000u); }
__device__ __forceinline__ float4 tf32_round4(float4 v) { return make_float4(tf32_round(v.x), tf32_round(v.y), tf32_round(v.z), tf32_round(v.w)); }

// ---- host-side helpers ---------------------------------------------------------------------------
// Opt-in to more than 48 KB of dynamic shared memory.  The attribute belongs to the (kernel, device)
// pair, so a process that drives several GPUs has to set it on each of them: the pairs already done
// are remembered under a mutex, with the device that is current at the call.
// A launch that fails because of its configuration leaves an error that a later successful call can hide
// from a cudaGetLastError made at the end of an entry point: the launchers note it at once in this
// per-thread latch, which the entry points read (and clear) before they report success.
inline cudaError_t &pbg_launch_error() {
  static thread_local cudaError_t e = cudaSuccess;
  return e;
}
inline void pbg_note_launch(cudaError_t e = cudaGetLastError()) {
  if (e != cudaSuccess && pbg_launch_error() == cudaSuccess) pbg_launch_error() = e;
}
inline cudaError_t pbg_take_launch_error() {
  cudaError_t e = pbg_launch_error();
  pbg_launch_error() = cudaSuccess;
  if (e == cudaSuccess) e = cudaGetLastError();
  return e;
}
inline cudaError_t pbg_opt_in_smem(const void *kernel, int bytes) {
  static std::mutex mu;
  static std::map<std::pair<const void *, int>, int> done;       // (kernel, device) -> bytes opted in so far
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) { pbg_note_launch(e); return e; }
  std::lock_guard<std::mutex> lock(mu);
  auto it = done.find({kernel, dev});
  if (it != done.end() && it->second >= bytes) return cudaSuccess;
  e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e == cudaSuccess) done[{kernel, dev}] = bytes;
  else pbg_note_launch(e);
  return e;
}
inline int pbg_sm_count() {
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 1;
  return sms > 0 ? sms : 1;
}

// ---- host-side launchers (one per translation unit) ------------------------------------------
struct SortPlan {
  unsigned long long *keys[2];
  unsigned int *vals[2];
  unsigned int *hist;     // pbg_sort_hist_entries(max_n) counters
  int max_n;              // capacity
  int result;             // which of keys[]/vals[] holds the sorted output after pbg_sort
};
int pbg_sort_warps(int n);
size_t pbg_sort_hist_entries(int n);   // digit counters (unsigned int) a sort of n pairs needs
// Stable LSD radix sort of n (key, value) pairs on `bits` low key bits; returns launches made.
int pbg_sort(SortPlan &sp, int n, int bits, cudaStream_t st);

int launch_build_keys(const WaveDims &d, const WaveBatches &wb, const WaveBufs &w,
                      unsigned long long *keys, unsigned int *vals, cudaStream_t st, unsigned long long tag = 0ull);
int launch_mask_keys(unsigned long long *keys, long long n, unsigned long long mask, cudaStream_t st);
int launch_gather(const WaveDims &d, const WaveBatches &wb, const WaveBufs &w, cudaStream_t st);
void *pbg_tc_plan_create(const WaveDims &d, const WaveBufs &w, int nblk_max, int precision);
void pbg_tc_plan_destroy(void *plan);
// standard relations, plane tiers: score contraction of both problems + loss + coefficient planes in one kernel
bool pbg_pair_eligible(const WaveDims &d, int precision);
void *pbg_pair_plan_create(const WaveDims &d, const WaveBufs &w, int nblk_max);
void pbg_pair_plan_destroy(void *plan);
int launch_pair_score(const WaveDims &d, const WaveBatches &wb, const WaveBufs &w, void *plan, cudaStream_t st);
int launch_grad_dual_tc(const WaveDims &d, const WaveBatches &wb, const WaveBufs &w, void *plan, cudaStream_t st);
int launch_score_tc(const WaveDims &d, const WaveBatches &wb, const WaveBufs &w, void *plan, cudaStream_t st);
int launch_grad_tc(const WaveDims &d, const WaveBatches &wb, const WaveBufs &w, void *plan, cudaStream_t st);
int launch_matrix_forward(const WaveDims &d, const WaveBatches &wb, const WaveBufs &w, cudaStream_t st);
int launch_matrix_backward(const WaveDims &d, const WaveBatches &wb, const WaveBufs &w, cudaStream_t st);
int launch_matrix_update(const WaveDims &d, const WaveBatches &wb, const WaveBufs &w, float lr, cudaStream_t st);
int launch_postop(const WaveDims &d, const WaveBatches &wb, const WaveBufs &w, cudaStream_t st);
int launch_gz_rows(const WaveDims &d, const WaveBatches &wb, const WaveBufs &w, cudaStream_t st);
int launch_score_simt(const WaveDims &d, const WaveBatches &wb, const WaveBufs &w, cudaStream_t st);
int launch_grad_simt(const WaveDims &d, const WaveBatches &wb, const WaveBufs &w, cudaStream_t st);
int launch_loss(const WaveDims &d, const WaveBatches &wb, const WaveBufs &w, cudaStream_t st);
int launch_export_scores(const WaveDims &d, const WaveBatches &wb, const WaveBufs &w,
                         float *lhs_pos, float *rhs_pos, float *lhs_neg, float *rhs_neg, cudaStream_t st);
// side / fork / join: a second stream and two events for the parts of the update that can run beside the embedding
// rows' kernels (null: everything on st)
int launch_update(const WaveDims &d, const WaveBatches &wb, const WaveBufs &w,
                  const unsigned long long *keys, const unsigned int *vals, float lr, float rel_lr,
                  float *psum, long long *hublist, int *hubcnt, long long *bigtab, cudaStream_t st,
                  cudaStream_t side = nullptr, cudaEvent_t fork = nullptr, cudaEvent_t join = nullptr);
// bigtab: (nocc / 256 + 2) rows of PBG_KMAX + 1 entries: where the batches of a row with 256 and more slots start, and its end
inline size_t pbg_bigtab_bytes(long long nocc) { return (size_t)(nocc / 256 + 2) * (PBG_KMAX + 1) * sizeof(long long); }
int launch_eval(const WaveDims &d, const WaveBatches &wb, const WaveBufs &w, double *out8_dev, cudaStream_t st);
size_t pbg_allnegs_bytes(int B, int Dp, int slab);
int launch_allnegs_eval(const WaveDims &d, const WaveBufs &w, char *mem, int B, int slab, int rel_std, float wrel,
                        double *out8_dev, cudaStream_t st);
int launch_reg_value(const WaveDims &d, const WaveBatches &wb, const WaveBufs &w, cudaStream_t st);
int launch_stats(const WaveDims &d, const WaveBatches &wb, const WaveBufs &w,
                 pbg_batch_stats *per_batch_dev, double *sum_dev, cudaStream_t st);
int launch_row_adagrad_sorted(float *emb, float *state, int dim, const unsigned long long *keys,
                              const unsigned int *vals, const float *grads, int n, float lr,
                              unsigned long long key_invalid, cudaStream_t st);
int launch_reverse_permutation(const long long *perm, long long n, long long *out, int *errflag, cudaStream_t st);
int launch_shuffle_rows(const void *in, void *out, long long rows, long long row_bytes, const long long *perm, int *errflag, cudaStream_t st);
int launch_randperm(SortPlan &sp, long long n, unsigned long long seed, long long *out, cudaStream_t st);
int launch_sub_bucket(SortPlan &sp, const long long *lhs, const long long *rhs, const long long *rel, long long n, int R,
                      const long long *tables_dev, int nl, int nr, int dynamic, long long *lhs_out, long long *rhs_out,
                      long long *rel_out, long long *counts_dev, int *errflag, cudaStream_t st);
int launch_iota_keys(const long long *rows, long long num_rows, int n, unsigned long long *keys,
                     unsigned int *vals, int *errflag, cudaStream_t st);
