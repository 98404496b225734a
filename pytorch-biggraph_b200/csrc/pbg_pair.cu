// Standard relations in the bf16-plane tiers: both score problems of a chunk block from ONE set of
// operand stages, with the loss, its gradient, the masks and the per-row statistics in the epilogue.
//
// With the operator on the rhs only (torchbiggraph/model.py:666-703) the rows scored in problem 0 are
// the first Pm rows of N1 and those of problem 1 the first Pm rows of N0 (see pbg_common.cuh):
//     S0 = N1[:Pm] . N0^T          S1 = N0[:Pm] . N1^T
// so a stage of 32 k-values of N0 and N1 (all planes) serves both products: the rows of N0 are the B
// operand of S0 and the A operand of S1, and the other way round for N1.  Every operand row of a chunk
// block crosses L2 -> shared memory once per k-stage instead of 1.5 times, and one CTA ends up with the
// score rows of both problems in tensor memory (two accumulators of up to 256 columns).
//
// Epilogue (sixteen warps, four threads per positive row i, each with two 32-column chunks of the row): what loss_kernel / loss_softmax_kernel do for a
// row, straight from tensor memory -- masks (model.py:566-580, 836-844), logistic / ranking / softmax
// (losses.py:53-161), relation and edge weight (batching.py:139-150), violators (train_cpu.py:98-99) --
// and the coefficient rows T_p[i][:] = d(loss)/d(score) with the positive pair in the diagonal, written
// as bf16 planes TB[p][blk][plane][i][j] = T_p[i][j] (rows i < Pm, columns j < Mm), which the gradient
// contraction reads both ways: K-major (k = j) and MN-major (k = i).
// The score matrix itself never leaves the SM.  dot and cos comparators (the l2 family keeps the
// separate kernels: its coefficients need the row and column sums of T).
//
// Every mbarrier wait is bounded (bit 1 of the error word, PBG_ERR_TIMEOUT); every TMA load is CTA-local.
#include "pbg_tc.cuh"

#define PAIR_THREADS 576          // warp 0 TMA, warp 1 MMA, warps 2-17 epilogue
#define PAIR_SMAX 4
#define PAIR_SMEM_MAX (227 * 1024 - 14 * 1024)   // dynamic shared memory opted in: the 227 KB of a CTA less its static part (reduction slots)

struct PairMaps { CUtensorMap n[2]; };     // planes of N0 / N1: 4-D (k, row, plane, block), K-major boxes {32, rows_pad}

struct PairGeom {
  int BN;               // columns of a score tile: Mm rounded up to 16 (<= 256)
  int rows_pad;         // rows of one operand plane in a stage: max(BN, 128)
  int nst, stage_bytes; // stages in flight, bytes of one
};

__device__ __forceinline__ float pair_softplus(float x) { return fmaxf(x, 0.f) + log1pf(expf(-fabsf(x))); }
__device__ __forceinline__ float pair_sigmoid(float x) { return 1.0f / (1.0f + expf(-x)); }

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
                 "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
                 "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]),
                 "=r"(r[30]), "=r"(r[31]) : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// 32 columns of this thread's tensor-memory lane back (the epilogue keeps per-score intermediates there)
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
               :: "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
                  "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]),
                  "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]),
                  "r"(r[30]), "r"(r[31]) : "memory");
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

template <int NPL>
// (18 warps are allocated as 20: 96 registers per thread is what fits, which is what ptxas settles on)
__global__ void __launch_bounds__(PAIR_THREADS, 1)
pair_score_kernel(const __grid_constant__ PairMaps maps, PairGeom g, WaveDims d, WaveBatches wb, WaveBufs w) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char *smem = (unsigned char *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) unsigned long long bars[2 * PAIR_SMAX + 2];
  __shared__ uint32_t tmem_base_s;
  __shared__ volatile int failed;
  __shared__ volatile int epi_go;
  // partial results of the four epilogue warps that share a row: [quantity][problem][column group][row]
  __shared__ float red_f[2][2][4][128];
  __shared__ int red_i[2][4][128];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t bar0 = smem_u32(&bars[0]);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };                  // TMA landed
  auto empty_bar = [&](int s) { return bar0 + 8u * (PAIR_SMAX + s); };   // MMAs have read the stage
  const uint32_t accf_bar = bar0 + 8u * (2 * PAIR_SMAX);                 // both accumulators complete
  const uint32_t acce_bar = bar0 + 8u * (2 * PAIR_SMAX + 1);             // both accumulators drained
  int *errflag = w.errflag;
  if (threadIdx.x == 0) {
    for (int i = 0; i < 2 * PAIR_SMAX; ++i) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" :: "r"(bar0 + 8u * i));
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" :: "r"(accf_bar));
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 512;" :: "r"(acce_bar));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    failed = 0;
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" :: "r"(smem_u32(&tmem_base_s)) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = tmem_base_s;
  const int STAGES = g.nst;
  const uint32_t plane_bytes = (uint32_t)g.rows_pad * 64u;               // one plane of one operand array: rows of 32 bf16
  const uint32_t arr_bytes = (uint32_t)NPL * plane_bytes;
  const uint32_t stage_tx = 2u * arr_bytes;
  const int nkb = (d.D + 31) / 32;
  // tile t of this launch = chunk block d.blk0 + t; every role walks the same list
  auto tile_live = [&](int t) { return block_info(d, wb, d.blk0 + t).n != 0; };

  if (warp == 0) {
    // ---------------- TMA producer: one box per (operand array, plane), each from its own lane ----------------
    long long git = 0;
    bool stop = false;
    for (int t = blockIdx.x; t < d.nblk && !stop; t += gridDim.x) {
      if (__any_sync(0xffffffffu, failed != 0)) break;
      if (!tile_live(t)) continue;
      const int blk = d.blk0 + t;
      for (int kb = 0; kb < nkb; ++kb, ++git) {
        const int s = (int)(git % STAGES);
        bool okw = true;
        if (git >= STAGES && lane == 0) okw = mbar_wait(empty_bar(s), (uint32_t)((git / STAGES) - 1) & 1, errflag);
        if (!__all_sync(0xffffffffu, okw)) { failed = 1; stop = true; break; }
        const uint32_t fb = full_bar(s);
        if (lane == 0) asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(fb), "r"(stage_tx) : "memory");
        __syncwarp();
        if (lane < 2 * NPL) {
          const int arr = lane / NPL, pl = lane - arr * NPL;
          const uint32_t dst = smem_u32(smem + (size_t)s * g.stage_bytes) + arr * arr_bytes + pl * plane_bytes;
          tma_load_4d(dst, &maps.n[arr], kb * 32, 0, pl, blk, fb);
        }
      }
    }
  } else if (warp == 1 && lane == 0) {
    // ---------------- MMA issuer ----------------
    // instruction descriptor: D fp32, A / B bf16, both K-major, N >> 3, M = 128
    const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(g.BN >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
    // plane pairs (a, b) of order a + b <= 2, the smallest contributions first; two planes: the last three
    const int pa[6] = {2, 0, 1, 1, 0, 0}, pb[6] = {0, 2, 1, 0, 1, 0};
    constexpr int T0 = NPL == 3 ? 0 : 3;
    long long git = 0, j = 0;
    for (int t = blockIdx.x; t < d.nblk && !failed; t += gridDim.x) {
      if (!tile_live(t)) continue;
      if (j >= 1 && !mbar_wait(acce_bar, (uint32_t)(j - 1) & 1, errflag)) { failed = 1; break; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      bool ok = true;
      for (int kb = 0; kb < nkb; ++kb, ++git) {
        const int s = (int)(git % STAGES);
        if (!mbar_wait(full_bar(s), (uint32_t)(git / STAGES) & 1, errflag)) { failed = 1; ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t st = smem_u32(smem + (size_t)s * g.stage_bytes);
        const int kleft = d.D - kb * 32;
#pragma unroll
        for (int k16 = 0; k16 < 2; ++k16) {
          if (k16 * 16 >= kleft) break;                          // the tail of K is zero fill
#pragma unroll
          for (int tt = T0; tt < 6; ++tt) {
            const uint32_t acc = (kb > 0 || k16 > 0 || tt > T0) ? 1u : 0u;
#pragma unroll
            for (int p = 0; p < 2; ++p) {
              if (!d.neg_enabled[p]) continue;
              // problem 0: A = rows of N1 (array 1), B = rows of N0 (array 0); problem 1 the other way round
              const uint32_t aarr = p == 0 ? 1u : 0u, barr = 1u - aarr;
              const uint64_t da = smem_desc(st + aarr * arr_bytes + pa[tt] * plane_bytes + k16 * 32, 0, 512, 4);
              const uint64_t db = smem_desc(st + barr * arr_bytes + pb[tt] * plane_bytes + k16 * 32, 0, 512, 4);
              asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
                           :: "r"(tmem + (uint32_t)p * 256u), "l"(da), "l"(db), "r"(idesc), "r"(acc) : "memory");
            }
          }
        }
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(empty_bar(s)) : "memory");
      }
      if (!ok) break;
      asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(accf_bar) : "memory");
      ++j;
    }
  } else if (warp >= 2) {
    // ---------------- epilogue: loss, statistics and coefficient planes of both problems ----------------
    // Sixteen warps: the four warps that share a tensor-memory lane group (rows i = q * 32 + lane) take two
    // 32-column chunks of the row each and combine their partial maxima / sums through shared memory.  A chunk
    // is read from tensor memory, reduced, and (softmax) its exponentials are written back over the scores, so
    // that every score costs one exponential and no more than 32 values are ever held in registers.
    long long j = 0;
    const int q = warp & 3;                            // the 32 tensor-memory lanes this warp may read
    const int cg = (warp - 2) >> 2;                    // column group: chunks 2 cg and 2 cg + 1
    const int i = q * 32 + lane;                       // positive row of the chunk
    const int Mm = d.Mm, Pm = d.Pm;
    auto epi_sync = [] { asm volatile("bar.sync 1, 512;" ::: "memory"); };     // the sixteen epilogue warps
    for (int t = blockIdx.x; t < d.nblk; t += gridDim.x) {
      if (!tile_live(t)) continue;
      const int blk = d.blk0 + t;
      // One thread waits for the accumulators (a bounded wait) and tells the others through shared memory: all
      // sixteen warps take the same decision, so that none is left alone at the named barrier further down.
      if (warp == 2 && lane == 0) {
        bool go = failed == 0 && mbar_wait(accf_bar, (uint32_t)j & 1, errflag);
        if (!go) failed = 1;
        epi_go = go ? 1 : 0;
      }
      epi_sync();
      if (!epi_go) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const BlockInfo bi = block_info(d, wb, blk);
      const bool row_valid = i < bi.n;
      const size_t prow = (size_t)blk * Pm + (i < Pm ? i : 0);
      const float wr = row_valid ? wb.wrel[bi.b] * (w.ew ? w.ew[bi.e0 + i] : 1.0f) : 0.f;   // relation weight x edge weight
#pragma unroll 1
      for (int p = 0; p < 2; ++p) {
        const int enabled = d.neg_enabled[p];
        const int Mlog = !enabled ? 0 : (d.batch_negs ? bi.Pl + d.U : d.U);   // columns of the reference's score matrix
        const float s = row_valid ? w.spos[p][prow] : 0.f;
        const int col0 = cg * 64;                                // first column of this warp's part of the row
        const uint32_t trow = tmem + (uint32_t)p * 256u + ((uint32_t)(q * 32) << 16) + (uint32_t)col0;
        const int nch = col0 >= w.Kb ? 0 : (col0 + 32 >= w.Kb ? 1 : 2);      // chunks of this warp that hold coefficient columns
        // Which columns of this warp's chunks count for this row (model.py:566-580): bit jj of live[c] is set when
        // column col0 + 32 c + jj exists (< Mm) and is not ignored -- uniform negatives (>= Pm) never are; a batch
        // negative is when the mode has none, when it is the row's own positive, or padding of the last chunk.
        auto below = [](int n) { return n <= 0 ? 0u : (n >= 32 ? 0xffffffffu : ((1u << n) - 1u)); };   // bits [0, n)
        unsigned live[2];
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int lo = col0 + c * 32;
          unsigned m = 0u;
          if (enabled) {
            m = below(Mm - lo) & ~below(Pm - lo);                               // uniform negatives
            if (d.batch_negs) {
              unsigned bn = below((bi.n < Pm ? bi.n : Pm) - lo);                   // real batch negatives
              if (i >= lo && i < lo + 32) bn &= ~(1u << (i - lo));                  // without the row's own positive
              m |= bn;
            }
          }
          live[c] = m;
        }
        auto masked = [&](int c, int jj) { return ((live[c] >> jj) & 1u) == 0u; };
        uint32_t r[32];
        float lossv = 0.f, ds = 0.f, scale = 0.f;
        int viol = 0;
        if (d.loss == PBG_LOSS_SOFTMAX) {
          // -s + log(e^s + sum_j e^S_ij), masked entries are e^-1e9 = 0 (losses.py:143-159)
          float mx = -INFINITY;
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            if (c >= nch) break;
            tmem_ld32(trow + (uint32_t)c * 32u, r);
#pragma unroll
            for (int jj = 0; jj < 32; ++jj) {
              const float sv = __uint_as_float(r[jj]);
              if (!masked(c, jj)) { mx = fmaxf(mx, sv); viol += sv > s; }
            }
          }
          red_f[0][p][cg][i] = mx;
          red_i[p][cg][i] = viol;
          epi_sync();
          mx = fmaxf(fmaxf(red_f[0][p][0][i], red_f[0][p][1][i]), fmaxf(red_f[0][p][2][i], red_f[0][p][3][i]));
          viol = red_i[p][0][i] + red_i[p][1][i] + red_i[p][2][i] + red_i[p][3][i];
          float m = fmaxf(mx, s);
          if (mx == -INFINITY) m = fmaxf(s, PBG_MASKED);         // every column masked
          float z = 0.f;
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            if (c >= nch) break;
            tmem_ld32(trow + (uint32_t)c * 32u, r);
#pragma unroll
            for (int jj = 0; jj < 32; ++jj) {
              const float e = masked(c, jj) ? 0.f : __expf(__uint_as_float(r[jj]) - m);
              r[jj] = __float_as_uint(e);                        // kept in tensor memory: the coefficient is scale * e
              z += e;
            }
            tmem_st32(trow + (uint32_t)c * 32u, r);
          }
          red_f[1][p][cg][i] = z;
          epi_sync();
          z = (red_f[1][p][0][i] + red_f[1][p][1][i]) + (red_f[1][p][2][i] + red_f[1][p][3][i]);
          const float es = expf(s - m), Z = z + es;
          if (Mlog > 0) { lossv = -s + m + logf(Z); ds = es / Z - 1.0f; scale = wr / Z; }
          else viol = 0;                                          // losses.py:139-140: no negatives, loss 0, no gradient
        } else if (d.loss == PBG_LOSS_RANKING) {
          // sum_j max(0, margin - s + S_ij) (losses.py:116-122); the scores are replaced by the 0 / 1 indicator of an active column
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            if (c >= nch) break;
            tmem_ld32(trow + (uint32_t)c * 32u, r);
#pragma unroll
            for (int jj = 0; jj < 32; ++jj) {
              const float sj = __uint_as_float(r[jj]);
              float act = 0.f;
              if (Mlog > 0 && !masked(c, jj)) {
                const float x = (sj - s) + d.margin;
                viol += sj > s;
                if (x > 0.f) { lossv += x; ds -= 1.0f; act = 1.0f; }
              }
              r[jj] = __float_as_uint(act);
            }
            tmem_st32(trow + (uint32_t)c * 32u, r);
          }
          red_f[0][p][cg][i] = lossv; red_f[1][p][cg][i] = ds; red_i[p][cg][i] = viol;
          epi_sync();
          lossv = (red_f[0][p][0][i] + red_f[0][p][1][i]) + (red_f[0][p][2][i] + red_f[0][p][3][i]);
          ds = (red_f[1][p][0][i] + red_f[1][p][1][i]) + (red_f[1][p][2][i] + red_f[1][p][3][i]);
          viol = red_i[p][0][i] + red_i[p][1][i] + red_i[p][2][i] + red_i[p][3][i];
          scale = wr;
        } else {
          // softplus(-s) + (1/M) sum_j softplus(S_ij), M counts masked columns (losses.py:61-80); the scores are replaced by sigmoid(S)
          const float nw = Mlog > 0 ? 1.0f / (float)Mlog : 0.f;
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            if (c >= nch) break;
            tmem_ld32(trow + (uint32_t)c * 32u, r);
#pragma unroll
            for (int jj = 0; jj < 32; ++jj) {
              const float sj = __uint_as_float(r[jj]);
              float sg = 0.f;
              if (!masked(c, jj)) { viol += sj > s; lossv += pair_softplus(sj); sg = pair_sigmoid(sj); }
              r[jj] = __float_as_uint(sg);
            }
            tmem_st32(trow + (uint32_t)c * 32u, r);
          }
          red_f[0][p][cg][i] = lossv; red_i[p][cg][i] = viol;
          epi_sync();
          lossv = ((red_f[0][p][0][i] + red_f[0][p][1][i]) + (red_f[0][p][2][i] + red_f[0][p][3][i])) * nw + pair_softplus(-s);
          viol = red_i[p][0][i] + red_i[p][1][i] + red_i[p][2][i] + red_i[p][3][i];
          ds = -pair_sigmoid(-s);
          scale = wr * nw;
        }
        const float tdiag = wr * ds;                             // the positive pair, folded into the diagonal
        // ---- coefficient row: planes into TB[p][i][:] (16-byte stores) ----
        unsigned short *tb = w.TB[p] + ((size_t)blk * NPL * Pm + (i < Pm ? i : 0)) * w.Kb;
        const size_t tb_plane = (size_t)Pm * w.Kb;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          if (c >= nch) break;
          tmem_ld32(trow + (uint32_t)c * 32u, r);
#pragma unroll
          for (int g8 = 0; g8 < 4; ++g8) {
            unsigned pk[3][4];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
              const int jj = g8 * 8 + u, jc = col0 + c * 32 + jj;
              float tv = row_valid ? scale * __uint_as_float(r[jj]) : 0.f;        // masked columns hold 0
              if (row_valid && jc == i) tv = tdiag;
              unsigned b0, b1, b2;
              bf16_planes(tv, b0, b1, b2);
              if (u & 1) { pk[0][u >> 1] |= b0 << 16; pk[1][u >> 1] |= b1 << 16; pk[2][u >> 1] |= b2 << 16; }
              else { pk[0][u >> 1] = b0; pk[1][u >> 1] = b1; pk[2][u >> 1] = b2; }
            }
            const int j0 = col0 + c * 32 + g8 * 8;
            if (i < Pm && j0 < w.Kb) {
#pragma unroll
              for (int pl = 0; pl < NPL; ++pl)
                *reinterpret_cast<uint4 *>(tb + pl * tb_plane + j0) = make_uint4(pk[pl][0], pk[pl][1], pk[pl][2], pk[pl][3]);
            }
          }
        }
        if (cg == 0 && i < Pm) {
          w.lossrow[p][prow] = row_valid ? wr * lossv : 0.f;
          w.violrow[p][prow] = row_valid ? viol : 0;
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(acce_bar) : "memory");
      ++j;
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    // if a wait ran out, copies / MMAs may still be in flight: a bounded grace period before the tensor memory goes back
    if (failed) for (int it = 0; it < 200000; ++it) __nanosleep(20);
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" :: "r"(tmem) : "memory");
  }
}

// ------------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------------
struct PairPlan {
  PairMaps maps;
  PairGeom geom;
  int npl;
};

bool pbg_pair_eligible(const WaveDims &d, int precision) {
  const bool planes = precision == PBG_PREC_BF16X6 || precision == PBG_PREC_BF16X3;
  return planes && !d.dynamic && !d.matrix_op && d.cmp < PBG_CMP_L2 && d.Pm <= 128 && d.Mm <= 256;
}

void *pbg_pair_plan_create(const WaveDims &d, const WaveBufs &w, int nblk_max) {
  PairPlan *pl = new PairPlan();
  pl->npl = w.npl;
  PairGeom &g = pl->geom;
  g.BN = (d.Mm + 15) / 16 * 16;
  g.rows_pad = g.BN > 128 ? g.BN : 128;
  g.stage_bytes = 2 * w.npl * g.rows_pad * 64;
  const int room = PAIR_SMEM_MAX - 1024;                       // dynamic shared memory left for the stages (1 KB: alignment)
  g.nst = room / g.stage_bytes > PAIR_SMAX ? PAIR_SMAX : room / g.stage_bytes;
  bool ok = g.nst >= 2 && w.TB[0];
  // rows beyond the Mm operand rows of a block are outside the map: the box brings zeros for them
  for (int a = 0; a < 2; ++a)
    ok = ok && encode4_planes(&pl->maps.n[a], w.XB[a], w.npl, d.D, d.Mm, d.Mm, nblk_max, w.Dpb, 32, g.rows_pad);
  if (!ok) { delete pl; return nullptr; }
  return pl;
}

void pbg_pair_plan_destroy(void *plan) { delete (PairPlan *)plan; }

int launch_pair_score(const WaveDims &d, const WaveBatches &wb, const WaveBufs &w, void *plan, cudaStream_t st) {
  PairPlan *pl = (PairPlan *)plan;
  const int sms = pbg_sm_count();
  const dim3 grid((unsigned)(d.nblk < sms ? d.nblk : sms));
  const size_t smem = (size_t)pl->geom.nst * pl->geom.stage_bytes + 1024;
  // the opt-in covers the largest stage ring this kernel is ever launched with (227 KB less its static shared memory)
  if (pl->npl == 3) {
    pbg_opt_in_smem((const void *)pair_score_kernel<3>, PAIR_SMEM_MAX);
    pair_score_kernel<3><<<grid, PAIR_THREADS, smem, st>>>(pl->maps, pl->geom, d, wb, w);
  } else {
    pbg_opt_in_smem((const void *)pair_score_kernel<2>, PAIR_SMEM_MAX);
    pair_score_kernel<2><<<grid, PAIR_THREADS, smem, st>>>(pl->maps, pl->geom, d, wb, w);
  }
  pbg_note_launch();
  return 1;
}
