// Score and gradient contractions on the 5th-generation tensor cores (tcgen05) with fp32
// accumulation in tensor memory -- precision tiers PBG_PREC_TF32X3 and PBG_PREC_TF32.  They take
// the place of torch.bmm / baddbmm in the reference comparators (torchbiggraph/model.py:179-180,
// 226-236) and of the bmm calls autograd issues for their backward.
//
//   score  : S_p[blk] (Pm x Mm) = Q_p[blk] (Pm x D) . N_p[blk]^T      A, B both K-major
//   grad Q : GQ_p[blk] (Pm x D) = T_p[blk] (Pm x Mm) . N_p[blk]        A K-major, B MN-major
//   grad N : GN_p[blk] (Mm x D) = T_p[blk]^T . Q_p[blk]                A, B both MN-major
//
// Persistent CTAs (one per SM) walk the list of 128 x BN output tiles (BN <= 256) of all (chunk,
// problem) pairs; two 256-column accumulators in tensor memory alternate, so the epilogue of one
// tile overlaps the main loop of the next:
//   warp 0      TMA producer: cp.async.bulk.tensor tiles of 32 k-values into a ring of
//               shared-memory stages, completion on an mbarrier per stage
//   warp 1      allocates tensor memory, issues tcgen05.mma.kind::tf32 (one elected lane) and
//               commits to the stage's "empty" barrier / the final "accumulator ready" barrier
//   warps 2-5   epilogue: tcgen05.ld 32 columns at a time (each warp its 32 TMEM lanes = 32
//               rows), comparator epilogue for scores; the 32 x 32 block goes through a private
//               swizzled shared-memory buffer (two per warp) and leaves as one bulk tensor
//               store, which writes whole 128-byte row segments and clips at the matrix edge
//   warps 6-13  TF32X3 only: split every landed stage into hi / lo (see below)
// K-major operands use the 128-byte swizzle; MN-major tf32 operands must use the 128-byte swizzle
// with 32-byte atoms (descriptor layout type 1, TMA swizzle 128B_ATOM_32B), 32 x 32 element boxes.
//
// TF32X3: the fp32 tiles TMA brings in are split in shared memory by eight warps: hi = tf32(x) in place, lo = x - hi into a second buffer of the
// stage; the tile is lo.hi + hi.lo + hi.hi accumulated in fp32, which restores fp32-level
// accuracy while every operand crosses HBM/L2 once, as plain fp32.
//
// Every wait on an mbarrier is bounded; when one runs out the CTA raises bit 1 of the error word,
// stops issuing work, releases its tensor memory and returns.  Every TMA load is CTA-local.
#include "pbg_tc.cuh"

// k-values per pipeline stage: 32 (two stages of 96 KB with their low parts in TF32X3) or 16 (four stages of
// 48 KB; K-major tiles then have 64-byte rows -- TMA 64-byte swizzle, descriptor layout 4, 512 bytes per 8
// rows -- and MN-major boxes are 32 x 16, descriptor LBO 2048).  Both are verified and give the same speed:
// the main loop is bound by shared-memory bandwidth (load 1x, split 3x, MMA operand reads 3x the tile per
// stage), not by the depth of the ring, and a tile takes the same time whether 20 or 148 CTAs run.
#define TC_KB 32
#define TC_THREADS 448          // warp 0 TMA, warp 1 MMA, warps 2-5 epilogue, warps 6-13 split operands (TF32X3)
#define TC_SPLIT_THREADS 256

struct TcMaps { CUtensorMap a[2]; CUtensorMap b[2]; CUtensorMap c[2]; CUtensorMap b2[2]; };   // [problem]; c = output (stores); b2: second B operand (dual mode)

struct TcGeom {
  int M, N, K;          // output rows, columns, contraction length (per block)
  int BN;               // tile columns (multiple of 16, <= 256)
  int ldc;
  long long c_blk;
  float *C[2];
  const float *auxA[2]; long long auxa_blk;   // score epilogue (l2 family): |a|^2, |b|^2
  const float *auxB[2]; long long auxb_blk;
  int cmp, score;
  int nst, stage_bytes;  // bf16-plane tier: stages in flight and bytes of one (three planes of A and of the B tile)
  int tr;                // the output map is that of the transposed matrix: tile element (row, col) goes to C[col][row]
  // Dual mode (standard relations, plane tiers, transposed gradient without a merged coefficient matrix):
  //   GN_side^T (D x Mm) = N_other^T[:, k < K1] . B1   +   N_other^T[:, k < K] . B2   (B2 fills the first BN2 columns)
  // with B1[k = i][n = m] = T_side[i][m] and B2[n = i][k = j] = T_other[i][j]: the two halves of the combined
  // matrix A[side][m][j] = T_side[j][m] + T_other[m][j], both read from the row-major coefficient planes TB --
  // B1 as an MN-major operand (K1 = Pm rows), B2 as a K-major one (BN2 = Pm rounded up to 16 rows, K = Mm).
  // A stage holds the A tile, B1 (for the k-blocks below K1) and B2.
  int dual, K1, BN2;
};

template <bool A_MN, bool B_MN, int NTERMS, bool L2EPI>
__global__ void __launch_bounds__(TC_THREADS, 1)
tc_gemm_kernel(const __grid_constant__ TcMaps maps, TcGeom g, WaveDims d, WaveBatches wb, int *errflag) {
  constexpr bool SPLIT = NTERMS == 3;
  // NTERMS == 6: the operands arrive as three bf16 planes each (x = b0 + b1 + b2, written by the producers);
  // a product is the six plane pairs of order <= 2 as kind::f16 MMAs -- no split in this kernel, and the
  // operand bytes the MMAs read from shared memory are half those of tf32
  // NTERMS == 2: the same on two planes per operand (x ~ b0 + b1) and the three products b1.b0, b0.b1, b0.b0
  constexpr bool PLANES = NTERMS == 6 || NTERMS == 2;
  constexpr int NPL = NTERMS == 6 ? 3 : 2;                               // planes per operand
  static_assert(!PLANES || TC_KB == 32, "bf16 planes: 32 k-values per stage");
  constexpr int KB = TC_KB;
  constexpr int SMAX = PLANES ? 4 : (SPLIT ? 2 : 4) * (32 / KB);      // stages (bf16 planes: as many as fit, at most 4)
  constexpr uint32_t ROW_BYTES = PLANES ? KB * 2 : KB * 4;               // bytes of one K-major row of a stage
  constexpr uint32_t BOX_BYTES = PLANES ? 4096 : KB * 128;               // one MN-major box: 64 x 32 bf16 or 32 x KB fp32
  constexpr uint32_t A_PLANE = 128 * ROW_BYTES, B_PLANE = 256 * ROW_BYTES;
  constexpr uint32_t A_BYTES = PLANES ? NPL * A_PLANE : A_PLANE, B_BYTES = PLANES ? NPL * B_PLANE : B_PLANE;   // one KB-k tile of 128 / 256 rows
  constexpr uint32_t RAW_BYTES = A_BYTES + B_BYTES;
  constexpr uint32_t STAGE_BYTES = SPLIT ? 2 * RAW_BYTES : RAW_BYTES;   // [A hi][B hi] ([A lo][B lo]) or [A planes][B planes]

  extern __shared__ unsigned char smem_raw[];
  unsigned char *smem = (unsigned char *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  // the plane tier sizes its stages by the tile's real width, and takes as many of them as fit
  const int STAGES = PLANES ? g.nst : SMAX;
  const uint32_t stage_bytes = PLANES ? (uint32_t)g.stage_bytes : STAGE_BYTES;
  unsigned char *ostage = smem + (size_t)STAGES * stage_bytes;          // [4 warps][2][32 rows x 128 B], epilogue staging
  __shared__ __align__(8) unsigned long long bars[3 * SMAX + 4];
  __shared__ uint32_t tmem_base_s;
  __shared__ volatile int failed;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t bar0 = smem_u32(&bars[0]);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };                 // TMA landed
  auto empty_bar = [&](int s) { return bar0 + 8u * (SMAX + s); };     // MMAs have read the stage
  auto conv_bar = [&](int s) { return bar0 + 8u * (2 * SMAX + s); };  // hi / lo written (SPLIT)
  auto accf_bar = [&](int a) { return bar0 + 8u * (3 * SMAX + a); };      // accumulator a complete
  auto acce_bar = [&](int a) { return bar0 + 8u * (3 * SMAX + 2 + a); };  // accumulator a drained
  if (threadIdx.x == 0) {
    for (int i = 0; i < 2 * SMAX; ++i) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" :: "r"(bar0 + 8u * i));
    for (int i = 0; i < SMAX; ++i) asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(conv_bar(i)), "r"(TC_SPLIT_THREADS));
    for (int a = 0; a < 2; ++a) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" :: "r"(accf_bar(a)));
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 128;" :: "r"(acce_bar(a)));
    }
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
  const int nkb = (g.K + KB - 1) / KB;
  const int b_atoms = PLANES ? (g.BN + 63) / 64 : (g.BN + 31) / 32;     // MN-major boxes per B tile (per plane)
  const uint32_t b_plane = B_MN ? (uint32_t)b_atoms * BOX_BYTES : (uint32_t)g.BN * ROW_BYTES;   // bytes of one B tile (plane)
  const uint32_t b_used = PLANES ? (uint32_t)NPL * b_plane : b_plane;
  const uint32_t stage_tx = A_BYTES + b_used;
  const bool dual = PLANES && A_MN && B_MN && g.dual != 0;
  const int nkb1 = dual ? (g.K1 + KB - 1) / KB : 0;                    // k-blocks that carry B1
  const uint32_t b2_plane = (uint32_t)g.BN2 * ROW_BYTES;                 // dual: one plane of the B2 tile
  // persistent tile loop: tile t -> (n tile, m tile, chunk block, problem); every role walks the same list
  const int tiles_n = (g.N + g.BN - 1) / g.BN, tiles_m = (g.M + 127) / 128;
  const long long ntiles = (long long)tiles_n * tiles_m * d.nblk * 2;
  auto tile_live = [&](long long t, int &p, int &blk, int &m0, int &n0) {
    int x = (int)(t % tiles_n);
    long long r = t / tiles_n;
    int y = (int)(r % tiles_m);
    int z = (int)(r / tiles_m);
    p = z & 1; blk = d.blk0 + (z >> 1); m0 = y * 128; n0 = x * g.BN;
    BlockInfo bi = block_info(d, wb, blk);
    return bi.n != 0 && !(g.score && !d.neg_enabled[p]);
  };

  if (warp == 0) {
    // ---------------- TMA producer (whole warp: every box of a stage is issued by its own lane) ----------------
    // Issuing one cp.async.bulk.tensor costs the issuing thread a few hundred cycles; an MN-major
    // B tile is up to eight 32 x 32 boxes, which issued from one lane made the producer the
    // longest link of the stage's chain.
    const int a_boxes = PLANES ? (A_MN ? 2 * NPL : NPL) : (A_MN ? 4 : 1), b_boxes = PLANES ? NPL * (B_MN ? b_atoms : 1) : (B_MN ? b_atoms : 1);
    long long git = 0;
    bool stop = false;
    for (long long t = blockIdx.x; t < ntiles && !stop; t += gridDim.x) {
      int p, blk, m0, n0;
      if (__any_sync(0xffffffffu, failed != 0)) break;
      if (!tile_live(t, p, blk, m0, n0)) continue;
      for (int kb = 0; kb < nkb; ++kb, ++git) {
        int s = (int)(git % STAGES);
        bool okw = true;
        if (git >= STAGES && lane == 0) okw = mbar_wait(empty_bar(s), (uint32_t)((git / STAGES) - 1) & 1, errflag);
        if (!__all_sync(0xffffffffu, okw)) { failed = 1; stop = true; break; }
        uint32_t fb = full_bar(s);
        const bool with_b1 = !dual || kb < nkb1;
        const uint32_t tx = dual ? A_BYTES + (with_b1 ? b_used : 0u) + (uint32_t)NPL * b2_plane : stage_tx;
        if (lane == 0) asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(fb), "r"(tx) : "memory");
        __syncwarp();
        unsigned char *st = smem + (size_t)s * stage_bytes;
        int k0 = kb * KB;
        uint32_t dA = smem_u32(st), dB = smem_u32(st + A_BYTES);
        if (PLANES) {
          if (lane < a_boxes) {
            if (!A_MN) tma_load_4d(dA + lane * A_PLANE, &maps.a[p], k0, m0, lane, blk, fb);
            else { int pl = lane >> 1, mb = lane & 1; tma_load_4d(dA + pl * A_PLANE + mb * BOX_BYTES, &maps.a[p], m0 + mb * 64, k0, pl, blk, fb); }
          } else if (lane < a_boxes + b_boxes) {
            int ib = lane - a_boxes;
            if (!B_MN) tma_load_4d(dB + ib * b_plane, &maps.b[p], k0, n0, ib, blk, fb);
            else if (with_b1) { int pl = ib / b_atoms, nb = ib - pl * b_atoms; tma_load_4d(dB + pl * b_plane + nb * BOX_BYTES, &maps.b[p], n0 + nb * 64, k0, pl, blk, fb); }
          } else if (dual && lane < a_boxes + b_boxes + NPL) {
            int ib = lane - a_boxes - b_boxes;
            tma_load_4d(dB + b_used + ib * b2_plane, &maps.b2[p], k0, 0, ib, blk, fb);
          }
        } else if (lane < a_boxes) {
          if (!A_MN) tma_load_3d(dA, &maps.a[p], k0, m0, blk, fb);
          else tma_load_3d(dA + lane * BOX_BYTES, &maps.a[p], m0 + lane * 32, k0, blk, fb);
        } else if (lane < a_boxes + b_boxes) {
          int nb = lane - a_boxes;
          if (!B_MN) tma_load_3d(dB, &maps.b[p], k0, n0, blk, fb);
          else tma_load_3d(dB + nb * BOX_BYTES, &maps.b[p], n0 + nb * 32, k0, blk, fb);
        }
      }
    }
  } else if (warp == 1 && lane == 0) {
    // ---------------- MMA issuer ----------------
    // instruction descriptor: D fp32, A/B tf32, operand majors, N >> 3, M >> 4
    const uint32_t fmt = PLANES ? 1u : 2u;            // operand format: bf16 (kind::f16) or tf32
    const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((A_MN ? 1u : 0u) << 15) | ((B_MN ? 1u : 0u) << 16) |
                           ((uint32_t)(g.BN >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
    const uint32_t idesc2 = (idesc & ~((0x3Fu << 17) | (1u << 16))) | ((uint32_t)(g.BN2 >> 3) << 17);   // dual: the B2 products are K-major, BN2 columns wide
    long long git = 0, j = 0;
    for (long long t = blockIdx.x; t < ntiles && !failed; t += gridDim.x) {
      int p, blk, m0, n0;
      if (!tile_live(t, p, blk, m0, n0)) continue;
      const int ab = (int)(j & 1);
      if (j >= 2 && !mbar_wait(acce_bar(ab), (uint32_t)((j >> 1) - 1) & 1, errflag)) { failed = 1; break; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t tacc = tmem + (uint32_t)ab * 256u;
      bool ok = true;
      for (int kb = 0; kb < nkb; ++kb, ++git) {
        int s = (int)(git % STAGES);
        if (!mbar_wait(SPLIT ? conv_bar(s) : full_bar(s), (uint32_t)(git / STAGES) & 1, errflag)) { failed = 1; ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        unsigned char *st = smem + (size_t)s * stage_bytes;
        uint32_t aH = smem_u32(st), bH = smem_u32(st + A_BYTES);
        uint32_t aL = aH + RAW_BYTES, bL = bH + RAW_BYTES;
        const int kleft = g.K - kb * KB;                        // k-values of this block that exist (the rest is zero fill)
        if (PLANES) {
          // plane pairs (a, b) of order a + b <= 2, the smallest contributions first; K = 16 per MMA:
          // K-major 64-byte rows (64-byte swizzle: layout 4, 512 bytes per 8 rows, 32 bytes per step),
          // MN-major 64 x 32 boxes (128-byte swizzle: layout 2, LBO = box, SBO 1024, 2048 bytes per step)
          // (two planes: the last three pairs of the list)
          const int pa[6] = {2, 0, 1, 1, 0, 0}, pb[6] = {0, 2, 1, 0, 1, 0};
          constexpr int T0 = NPL == 3 ? 0 : 3;
          const int kleft1 = dual ? g.K1 - kb * KB : kleft;    // k-values of this block under B1
#pragma unroll
          for (int k16 = 0; k16 < 2; ++k16) {
            if (k16 * 16 >= kleft) break;                     // the tail of K: those k-values are zero fill
#pragma unroll
            for (int t = T0; t < 6; ++t) {
              uint64_t da = A_MN ? smem_desc(aH + pa[t] * A_PLANE + k16 * 2048, BOX_BYTES, 1024, 2)
                                 : smem_desc(aH + pa[t] * A_PLANE + k16 * 32, 0, 512, 4);
              uint64_t db = B_MN ? smem_desc(bH + pb[t] * b_plane + k16 * 2048, BOX_BYTES, 1024, 2)
                                 : smem_desc(bH + pb[t] * b_plane + k16 * 32, 0, 512, 4);
              uint32_t acc = (kb > 0 || k16 > 0 || t > T0) ? 1u : 0u;
              if (dual && k16 * 16 >= kleft1) continue;       // past K1: no B1 product for these k-values
              asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
                           :: "r"(tacc), "l"(da), "l"(db), "r"(idesc), "r"(acc) : "memory");
            }
            if (dual) {
              // B2 = rows of the other problem's coefficient matrix: every k-block, BN2 columns wide, always
              // accumulating -- the first product of a tile is a B1 product (k-block 0 carries B1 and K1 >= 1),
              // which initialises all BN columns
#pragma unroll
              for (int t = T0; t < 6; ++t) {
                uint64_t da = smem_desc(aH + pa[t] * A_PLANE + k16 * 2048, BOX_BYTES, 1024, 2);
                uint64_t db = smem_desc(bH + b_used + pb[t] * b2_plane + k16 * 32, 0, 512, 4);
                asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
                             :: "r"(tacc), "l"(da), "l"(db), "r"(idesc2), "r"(1u) : "memory");
              }
            }
          }
        } else
#pragma unroll
        for (int k8 = 0; k8 < KB / 8; ++k8) {
          if (k8 * 8 >= kleft) break;                         // the tail of K: those k-values are zero fill
          constexpr uint32_t KSBO = KB == 32 ? 1024 : 512, KLAY = KB == 32 ? 2 : 4;     // K-major: 8 rows of ROW_BYTES; 128- / 64-byte swizzle
          uint32_t ao = A_MN ? k8 * 1024 : k8 * 32, bo = B_MN ? k8 * 1024 : k8 * 32;
          uint64_t dAh = A_MN ? smem_desc(aH + ao, BOX_BYTES, 512, 1) : smem_desc(aH + ao, 0, KSBO, KLAY);
          uint64_t dBh = B_MN ? smem_desc(bH + bo, BOX_BYTES, 512, 1) : smem_desc(bH + bo, 0, KSBO, KLAY);
          uint32_t acc = (kb > 0 || k8 > 0) ? 1u : 0u;
          if (SPLIT) {
            uint64_t dAl = A_MN ? smem_desc(aL + ao, BOX_BYTES, 512, 1) : smem_desc(aL + ao, 0, KSBO, KLAY);
            uint64_t dBl = B_MN ? smem_desc(bL + bo, BOX_BYTES, 512, 1) : smem_desc(bL + bo, 0, KSBO, KLAY);
            asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n}"
                         :: "r"(tacc), "l"(dAl), "l"(dBh), "r"(idesc), "r"(acc) : "memory");
            asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n}"
                         :: "r"(tacc), "l"(dAh), "l"(dBl), "r"(idesc), "r"(1u) : "memory");
            acc = 1u;
          }
          asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n}"
                       :: "r"(tacc), "l"(dAh), "l"(dBh), "r"(idesc), "r"(acc) : "memory");
        }
        // frees the stage for the producer once the MMAs above have read it
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(empty_bar(s)) : "memory");
      }
      if (!ok) break;
      asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(accf_bar(ab)) : "memory");
      ++j;
    }
  } else if (SPLIT && warp >= 6) {
    // ---------------- hi / lo split of every landed stage (warps 6-13) ----------------
    const int ct = threadIdx.x - 192;                             // 0..255
    const uint32_t nchunks = stage_tx / 16;
    long long git = 0;
    bool stop = false;
    for (long long t = blockIdx.x; t < ntiles && !stop; t += gridDim.x) {
      int p, blk, m0, n0;
      if (__any_sync(0xffffffffu, failed != 0)) break;           // warp-uniform exit
      if (!tile_live(t, p, blk, m0, n0)) continue;
      for (int kb = 0; kb < nkb; ++kb, ++git) {
        int s = (int)(git % STAGES);
        // one lane per warp polls the barrier (256 polling threads would take issue slots from the warps
        // that have work); the warp-wide vote that follows orders the other lanes' reads after it
        bool okw = true;
        if (lane == 0) okw = mbar_wait(full_bar(s), (uint32_t)(git / STAGES) & 1, errflag);
        if (!__all_sync(0xffffffffu, okw)) { failed = 1; stop = true; break; }
        unsigned char *st = smem + (size_t)s * stage_bytes;
        for (uint32_t c0 = ct; c0 < nchunks; c0 += 4 * TC_SPLIT_THREADS) {
          float4 v[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            uint32_t c = c0 + u * TC_SPLIT_THREADS;
            if (c < nchunks) v[u] = *reinterpret_cast<const float4 *>(st + (size_t)c * 16);
          }
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            uint32_t c = c0 + u * TC_SPLIT_THREADS;
            if (c < nchunks) {
              float4 h = tf32_round4(v[u]);
              *reinterpret_cast<float4 *>(st + (size_t)c * 16) = h;
              *reinterpret_cast<float4 *>(st + RAW_BYTES + (size_t)c * 16) = v[u] - h;
            }
          }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy writes -> tensor-core reads
        asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(conv_bar(s)) : "memory");
      }
    }
  } else if (warp >= 2 && warp < 6) {
    // ---------------- epilogue: drains accumulator j & 1 while the next tile is being multiplied ----------------
    long long j = 0, nst = 0;
    const int q = warp & 3;                           // the 32 TMEM lanes this warp may read
    for (long long t = blockIdx.x; t < ntiles; t += gridDim.x) {
      int p, blk, m0, n0;
      if (__any_sync(0xffffffffu, failed != 0)) break;           // warp-uniform exit (tcgen05.ld is warp-wide)
      if (!tile_live(t, p, blk, m0, n0)) continue;
      const int ab = (int)(j & 1);
      bool okw = true;
      if (lane == 0) okw = mbar_wait(accf_bar(ab), (uint32_t)(j >> 1) & 1, errflag);
      if (!__all_sync(0xffffffffu, okw)) { failed = 1; break; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int mrow0 = m0 + q * 32;                 // first output row of this warp's block
      const int m = mrow0 + lane;
      float an = 0.f;
      // comparator epilogue of the l2 family: compiled in only where it is used (predicated-off
      // copies of it in the unrolled loop cost more issue slots than the stores themselves)
      constexpr bool l2 = L2EPI;
      if (l2 && m < g.M) an = g.auxA[p][(size_t)blk * g.auxa_blk + m];
      const float *bn = l2 ? g.auxB[p] + (size_t)blk * g.auxb_blk : nullptr;
      for (int c0 = 0; c0 < g.BN; c0 += 32) {
        uint32_t r[32];
        uint32_t taddr = tmem + (uint32_t)ab * 256u + ((uint32_t)(q * 32) << 16) + (uint32_t)c0;
        asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                     : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
                       "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
                       "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]),
                       "=r"(r[30]), "=r"(r[31]) : "r"(taddr));
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        const int ncol0 = n0 + c0;
        if (mrow0 >= g.M || ncol0 >= g.N) continue;    // block entirely outside the matrix (warp-uniform)
        // the buffer used two blocks ago must have been read by its store before it is rewritten
        if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
        __syncwarp();
        unsigned char *buf = ostage + (size_t)(q * 2 + (int)(nst & 1)) * 4096;
        ++nst;
        if (g.tr) {
          // transposed output: column jj of the block is row jj of the store box, this lane's tile row its
          // element `lane` -- 4-byte writes, conflict-free in the same 128-byte swizzle
#pragma unroll
          for (int jj = 0; jj < 32; ++jj)
            *reinterpret_cast<uint32_t *>(buf + jj * 128 + (((lane >> 2) ^ (jj & 7)) << 4) + ((lane & 3) << 2)) = r[jj];
        } else
#pragma unroll
        for (int jj = 0; jj < 32; jj += 4) {
          float v[4];
#pragma unroll
          for (int tt = 0; tt < 4; ++tt) {
            v[tt] = __uint_as_float(r[jj + tt]);
            if (l2) {
              int n = ncol0 + jj + tt;
              float qv = ((n < g.N ? bn[n] : 0.f) - 2.0f * v[tt]) + an;     // model.py:226-246
              v[tt] = g.cmp == PBG_CMP_L2 ? -sqrtf(fmaxf(qv, 1e-30f)) : -qv;
            }
          }
          // row `lane` of the block, 16-byte unit jj / 4, in the 128-byte swizzle the store map expects
          *reinterpret_cast<float4 *>(buf + lane * 128 + (((jj >> 2) ^ (lane & 7)) << 4)) = make_float4(v[0], v[1], v[2], v[3]);
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // generic writes -> bulk store reads
        __syncwarp();
        if (lane == 0) {
          asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%1, %2, %3}], [%4];"
                       :: "l"(&maps.c[p]), "r"(g.tr ? mrow0 : ncol0), "r"(g.tr ? ncol0 : mrow0), "r"(blk), "r"(smem_u32(buf)) : "memory");
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(acce_bar(ab)) : "memory");
      ++j;
    }
    if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // the stores have left shared memory and are performed
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    // If a wait ran out the asynchronous copies / MMAs may still be in flight: give them a
    // bounded grace period before the tensor memory goes back.
    if (failed) for (int i = 0; i < 200000; ++i) __nanosleep(20);
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" :: "r"(tmem) : "memory");
  }
}

// ------------------------------------------------------------------------------------------------
// host side: tensor maps (encoded once per context) and launchers
// ------------------------------------------------------------------------------------------------
struct TcPlan {
  TcMaps score, gradq, gradn, gradm, gradt, gradu;
  bool has_dual;
  int bn2;
  bool dynamic;
  int bn_score, bn_grad;
  int nterms;
};

// Columns per tile: equal tiles of at most 256.  With more than one tile the width is a multiple of
// 32, the width of the epilogue's store blocks (a block must not reach into the next tile); a single
// tile may end on a multiple of 16, what lies beyond it is outside the matrix and clipped.
static int tile_cols(int n) {
  int tiles = (n + 255) / 256;
  int unit = tiles > 1 ? 32 : 16;
  int bn = ((n + tiles - 1) / tiles + unit - 1) / unit * unit;
  return bn > 256 ? 256 : bn;
}

// Builds the tensor maps for the context's workspace.  Returns null when the driver entry point
// is missing or an encode fails.
void *pbg_tc_plan_create(const WaveDims &d, const WaveBufs &w, int nblk_max, int precision) {
  TcPlan *pl = new TcPlan();
  pl->has_dual = false; pl->bn2 = 0;
  pl->dynamic = d.dynamic != 0;
  pl->nterms = precision == PBG_PREC_TF32X3 ? 3 : precision == PBG_PREC_BF16X6 ? 6 : precision == PBG_PREC_BF16X3 ? 2 : 1;
  pl->bn_score = tile_cols(d.Mm);
  pl->bn_grad = tile_cols(d.D);
  bool ok = true;
  if (pl->nterms == 6 || pl->nterms == 2) {
    const int npl = w.npl;
    // bf16-plane tiers: the same products on the plane arrays (K-major boxes {32 k, rows}, MN-major boxes {64, 32 k})
    for (int p = 0; p < 2; ++p) {
      int q = ARR_Q0 + p, n = ARR_N0 + p;
      ok &= encode4_planes(&pl->score.a[p], w.XB[q], npl, d.D, d.Pm, w.xrows[q], nblk_max, w.Dpb, 32, 128);
      ok &= encode4_planes(&pl->score.b[p], w.XB[n], npl, d.D, w.xrows[n], w.xrows[n], nblk_max, w.Dpb, 32, pl->bn_score);
      ok &= encode3(&pl->score.c[p], w.S[p], d.Mm, d.Pm, nblk_max, d.Ms, (long long)d.Pm * d.Ms, 32, 32, false);
      if (pl->dynamic) {
        // grad Q: A = T (K-major, k = Mm), B = N (MN-major); grad N: A = T^T (MN-major: k rows = Pm), B = Q (MN-major)
        ok &= encode4_planes(&pl->gradq.a[p], w.TB[p], npl, d.Mm, d.Pm, d.Pm, nblk_max, w.Kb, 32, 128);
        ok &= encode4_planes(&pl->gradq.b[p], w.XB[n], npl, d.D, w.xrows[n], w.xrows[n], nblk_max, w.Dpb, 64, 32);
        ok &= encode4_planes(&pl->gradn.a[p], w.TB[p], npl, d.Mm, d.Pm, d.Pm, nblk_max, w.Kb, 64, 32);
        ok &= encode4_planes(&pl->gradn.b[p], w.XB[q], npl, d.D, w.xrows[q], w.xrows[q], nblk_max, w.Dpb, 64, 32);
        ok &= encode3(&pl->gradq.c[p], w.GX[q], d.D, d.Pm, nblk_max, d.Dp, (long long)w.grows[q] * d.Dp, 32, 32, false);
        ok &= encode3(&pl->gradn.c[p], w.GX[n], d.D, d.Mm, nblk_max, d.Dp, (long long)w.grows[n] * d.Dp, 32, 32, false);
      } else {
        int o = ARR_N0 + (1 - p);
        ok &= encode4_planes(&pl->gradm.a[p], w.AB[p], npl, d.Mm, d.Mm, d.Mm, nblk_max, w.Kb, 32, 128);
        ok &= encode4_planes(&pl->gradm.b[p], w.XB[o], npl, d.D, w.xrows[o], w.xrows[o], nblk_max, w.Dpb, 64, 32);
        ok &= encode3(&pl->gradm.c[p], w.GX[n], d.D, d.Mm, nblk_max, d.Dp, (long long)d.Mm * d.Dp, 32, 32, false);
        // the same product transposed, GN^T = N_other^T . A^T: tile rows run over D (every 128-row tile full,
        // where Mm = 200 leaves the second one 56 % used), tile columns over the Mm coefficient rows
        pl->gradt.a[p] = pl->gradm.b[p];
        ok &= encode4_planes(&pl->gradt.b[p], w.AB[p], npl, d.Mm, d.Mm, d.Mm, nblk_max, w.Kb, 32, pl->bn_score);
        pl->gradt.c[p] = pl->gradm.c[p];
        if (w.TB[0]) {
          // dual mode: B1 = TB[side] read MN-major (k = i < Pm rows, n = m < Mm), B2 = TB[other side] read K-major (rows
          // i < Pm, k = j < Mm); what lies beyond those extents is outside the maps and arrives as zeros
          pl->has_dual = true;
          pl->bn2 = (d.Pm + 15) / 16 * 16;
          pl->gradu.a[p] = pl->gradm.b[p];
          ok &= encode4_planes(&pl->gradu.b[p], w.TB[p], npl, d.Mm, d.Pm, d.Pm, nblk_max, w.Kb, 64, 32);
          ok &= encode4_planes(&pl->gradu.b2[p], w.TB[1 - p], npl, d.Mm, d.Pm, d.Pm, nblk_max, w.Kb, 32, pl->bn2);
          pl->gradu.c[p] = pl->gradm.c[p];
        }
      }
    }
    if (!ok) { delete pl; return nullptr; }
    return pl;
  }
  for (int p = 0; p < 2; ++p) {
    int q = ARR_Q0 + p, n = ARR_N0 + p;
    const float *Xq = w.X[q], *Xn = w.X[n], *T = w.S[p];
    long long qblk = (long long)w.xrows[q] * d.Dp, nblk_s = (long long)w.xrows[n] * d.Dp, tblk = (long long)d.Pm * d.Ms;
    // score: A = Q (K-major, k = D), B = N (K-major)
    // only the Pm scored rows exist for the map: the rest of the 128-row box is filled with zeros without touching L2
    ok &= encode3(&pl->score.a[p], Xq, d.D, d.Pm, nblk_max, d.Dp, qblk, TC_KB, 128, false);
    ok &= encode3(&pl->score.b[p], Xn, d.D, w.xrows[n], nblk_max, d.Dp, nblk_s, TC_KB, pl->bn_score, false);
    // outputs leave through 32 x 32 bulk stores (128-byte swizzle in shared memory), clipped at the matrix edge
    ok &= encode3(&pl->score.c[p], w.S[p], d.Mm, d.Pm, nblk_max, d.Ms, tblk, 32, 32, false);
    if (pl->dynamic) {
      // grad Q: A = T (K-major, k = Mm), B = N (MN-major: k rows = Mm, contiguous D)
      ok &= encode3(&pl->gradq.a[p], T, d.Mm, d.Pm, nblk_max, d.Ms, tblk, TC_KB, 128, false);
      ok &= encode3(&pl->gradq.b[p], Xn, d.D, w.xrows[n], nblk_max, d.Dp, nblk_s, 32, TC_KB, true);
      // grad N: A = T^T (MN-major: k rows = Pm, contiguous Mm), B = Q (MN-major: k rows = Pm, contiguous D)
      ok &= encode3(&pl->gradn.a[p], T, d.Mm, d.Pm, nblk_max, d.Ms, tblk, 32, TC_KB, true);
      ok &= encode3(&pl->gradn.b[p], Xq, d.D, w.xrows[q], nblk_max, d.Dp, qblk, 32, TC_KB, true);
      ok &= encode3(&pl->gradq.c[p], w.GX[q], d.D, d.Pm, nblk_max, d.Dp, (long long)w.grows[q] * d.Dp, 32, 32, false);
      ok &= encode3(&pl->gradn.c[p], w.GX[n], d.D, d.Mm, nblk_max, d.Dp, (long long)w.grows[n] * d.Dp, 32, 32, false);
    } else {
      // merged: side p: A = A[p] (K-major, k = Mm), B = the other side's operand rows (MN-major)
      int o = ARR_N0 + (1 - p);
      ok &= encode3(&pl->gradm.a[p], w.A[p], d.Mm, d.Mm, nblk_max, w.Ma, (long long)d.Mm * w.Ma, TC_KB, 128, false);
      ok &= encode3(&pl->gradm.b[p], w.X[o], d.D, w.xrows[o], nblk_max, d.Dp, (long long)w.xrows[o] * d.Dp, 32, TC_KB, true);
      ok &= encode3(&pl->gradm.c[p], w.GX[n], d.D, d.Mm, nblk_max, d.Dp, (long long)d.Mm * d.Dp, 32, 32, false);
      // the same product transposed (see the bf16-plane tier above): A = the other side's operand rows (MN-major),
      // B = the coefficient rows (K-major)
      pl->gradt.a[p] = pl->gradm.b[p];
      ok &= encode3(&pl->gradt.b[p], w.A[p], d.Mm, d.Mm, nblk_max, w.Ma, (long long)d.Mm * w.Ma, TC_KB, pl->bn_score, false);
      pl->gradt.c[p] = pl->gradm.c[p];
    }
  }
  if (!ok) { delete pl; return nullptr; }
  return pl;
}

void pbg_tc_plan_destroy(void *plan) { delete (TcPlan *)plan; }

template <bool A_MN, bool B_MN, int NTERMS, bool L2EPI>
static void launch_tc_inst(const TcMaps &maps, const TcGeom &g, const WaveDims &d, const WaveBatches &wb, int *errflag,
                           dim3 grid, size_t smem, cudaStream_t st) {
  TcGeom gg = g;
  constexpr bool planes = NTERMS == 6 || NTERMS == 2;
  if (planes) {
    // two or three planes of 64-byte rows: A 128 rows; B the tile's rows (K-major) or its 64-column boxes (MN-major)
    constexpr int npl = NTERMS == 6 ? 3 : 2;
    const int b_plane = B_MN ? (g.BN + 63) / 64 * 4096 : g.BN * 64;
    gg.stage_bytes = npl * 128 * 64 + npl * b_plane + (g.dual ? npl * g.BN2 * 64 : 0);
    const int room = (int)smem - (4 * 2 * 4096 + 1024);            // what the stages get of the kernel's dynamic shared memory
    gg.nst = room / gg.stage_bytes > 4 ? 4 : room / gg.stage_bytes;
    smem = (size_t)room + 4 * 2 * 4096 + 1024;
  }
  // if the opt-in fails the launch below fails too, and the caller's cudaGetLastError reports it
  pbg_opt_in_smem((const void *)tc_gemm_kernel<A_MN, B_MN, NTERMS, L2EPI>, (int)smem);
  // the plane tier has no split warps: producer, MMA issuer and the four epilogue warps
  tc_gemm_kernel<A_MN, B_MN, NTERMS, L2EPI><<<grid, planes ? 192 : TC_THREADS, smem, st>>>(maps, gg, d, wb, errflag);
  pbg_note_launch();
}

template <bool A_MN, bool B_MN>
static void launch_tc(const TcMaps &maps, const TcGeom &g, int nterms, const WaveDims &d, const WaveBatches &wb, int *errflag,
                      cudaStream_t st) {
  long long tiles = (long long)((g.N + g.BN - 1) / g.BN) * ((g.M + 127) / 128) * d.nblk * 2;
  const int sms = pbg_sm_count();
  dim3 grid((unsigned)(tiles < sms ? tiles : sms));
  size_t smem = 4 * (128 * 128 + 256 * 128) + 4 * 2 * 4096 + 1024;   // 2 stages x (hi, lo) or 4 stages x raw; epilogue staging
  // the comparator epilogue of the l2 family exists only in the score kernels (both operands K-major)
  const bool l2 = !A_MN && !B_MN && g.score && g.cmp >= PBG_CMP_L2;
  if constexpr (!A_MN && !B_MN) {
    if (l2) {
      if (nterms == 6) launch_tc_inst<A_MN, B_MN, 6, true>(maps, g, d, wb, errflag, grid, smem, st);
      else if (nterms == 2) launch_tc_inst<A_MN, B_MN, 2, true>(maps, g, d, wb, errflag, grid, smem, st);
      else if (nterms == 3) launch_tc_inst<A_MN, B_MN, 3, true>(maps, g, d, wb, errflag, grid, smem, st);
      else launch_tc_inst<A_MN, B_MN, 1, true>(maps, g, d, wb, errflag, grid, smem, st);
      return;
    }
  }
  if (nterms == 6) { launch_tc_inst<A_MN, B_MN, 6, false>(maps, g, d, wb, errflag, grid, smem, st); return; }
  if (nterms == 2) { launch_tc_inst<A_MN, B_MN, 2, false>(maps, g, d, wb, errflag, grid, smem, st); return; }
  if (nterms == 3) launch_tc_inst<A_MN, B_MN, 3, false>(maps, g, d, wb, errflag, grid, smem, st);
  else launch_tc_inst<A_MN, B_MN, 1, false>(maps, g, d, wb, errflag, grid, smem, st);
}

int launch_score_tc(const WaveDims &d, const WaveBatches &wb, const WaveBufs &w, void *plan, cudaStream_t st) {
  TcPlan *pl = (TcPlan *)plan;
  TcGeom g;
  memset(&g, 0, sizeof g);
  g.M = d.Pm; g.N = d.Mm; g.K = d.D; g.BN = pl->bn_score; g.ldc = d.Ms; g.c_blk = (long long)d.Pm * d.Ms;
  g.cmp = d.cmp; g.score = 1;
  for (int p = 0; p < 2; ++p) {
    g.C[p] = w.S[p];
    g.auxA[p] = w.aux[ARR_Q0 + p]; g.auxB[p] = w.aux[ARR_N0 + p];
  }
  g.auxa_blk = w.xrows[ARR_Q0]; g.auxb_blk = w.xrows[ARR_N0];
  launch_tc<false, false>(pl->score, g, pl->nterms, d, wb, w.errflag, st);
  return 1;
}

// Standard relations, plane tiers, coefficient planes TB written by the fused score kernel: the transposed
// gradient product with two B operands per stage (see TcGeom).
int launch_grad_dual_tc(const WaveDims &d, const WaveBatches &wb, const WaveBufs &w, void *plan, cudaStream_t st) {
  TcPlan *pl = (TcPlan *)plan;
  TcGeom g;
  memset(&g, 0, sizeof g);
  g.M = d.D; g.N = d.Mm; g.K = d.Mm; g.BN = pl->bn_score; g.ldc = d.Dp; g.tr = 1;
  g.dual = 1; g.K1 = d.Pm; g.BN2 = pl->bn2;
  for (int p = 0; p < 2; ++p) g.C[p] = w.GX[ARR_N0 + p];
  long long tiles = (long long)((g.N + g.BN - 1) / g.BN) * ((g.M + 127) / 128) * d.nblk * 2;
  const int sms = pbg_sm_count();
  const dim3 grid((unsigned)(tiles < sms ? tiles : sms));
  const size_t smem = 4 * (128 * 128 + 256 * 128) + 4 * 2 * 4096 + 1024;
  if (pl->nterms == 6) launch_tc_inst<true, true, 6, false>(pl->gradu, g, d, wb, w.errflag, grid, smem, st);
  else launch_tc_inst<true, true, 2, false>(pl->gradu, g, d, wb, w.errflag, grid, smem, st);
  return 1;
}

int launch_grad_tc(const WaveDims &d, const WaveBatches &wb, const WaveBufs &w, void *plan, cudaStream_t st) {
  TcPlan *pl = (TcPlan *)plan;
  TcGeom g;
  memset(&g, 0, sizeof g);
  g.N = d.D; g.BN = pl->bn_grad; g.ldc = d.Dp;
  if (!pl->dynamic && pl->nterms != 1) {     // standard relations: the transposed product (see pbg_tc_plan_create)
    g.M = d.D; g.N = d.Mm; g.K = d.Mm; g.BN = pl->bn_score; g.tr = 1;
    for (int p = 0; p < 2; ++p) g.C[p] = w.GX[ARR_N0 + p];
    long long tiles = (long long)((g.N + g.BN - 1) / g.BN) * ((g.M + 127) / 128) * d.nblk * 2;
    const int sms = pbg_sm_count();
    const dim3 grid((unsigned)(tiles < sms ? tiles : sms));
    const size_t smem = 4 * (128 * 128 + 256 * 128) + 4 * 2 * 4096 + 1024;
    if (pl->nterms == 6) launch_tc_inst<true, false, 6, false>(pl->gradt, g, d, wb, w.errflag, grid, smem, st);
    else if (pl->nterms == 2) launch_tc_inst<true, false, 2, false>(pl->gradt, g, d, wb, w.errflag, grid, smem, st);
    else launch_tc_inst<true, false, 3, false>(pl->gradt, g, d, wb, w.errflag, grid, smem, st);
    return 1;
  }
  if (!pl->dynamic) {          // GN_side = A[side] . N_(1-side)
    g.M = d.Mm; g.K = d.Mm; g.c_blk = (long long)d.Mm * d.Dp;
    for (int p = 0; p < 2; ++p) g.C[p] = w.GX[ARR_N0 + p];
    launch_tc<false, true>(pl->gradm, g, pl->nterms, d, wb, w.errflag, st);
    return 1;
  }
  // GQ_p = T_p . N_p
  g.M = d.Pm; g.K = d.Mm; g.c_blk = (long long)w.grows[ARR_Q0] * d.Dp;
  for (int p = 0; p < 2; ++p) g.C[p] = w.GX[ARR_Q0 + p];
  launch_tc<false, true>(pl->gradq, g, pl->nterms, d, wb, w.errflag, st);
  // GN_p = T_p^T . Q_p
  g.M = d.Mm; g.K = d.Pm; g.c_blk = (long long)w.grows[ARR_N0] * d.Dp;
  for (int p = 0; p < 2; ++p) g.C[p] = w.GX[ARR_N0 + p];
  launch_tc<true, true>(pl->gradn, g, pl->nterms, d, wb, w.errflag, st);
  return 2;
}
