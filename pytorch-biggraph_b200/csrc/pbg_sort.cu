// Stable LSD radix sort of (row key, occurrence) pairs: groups the gradient slots of one wave by
// the embedding row they belong to, in batch order, so that the update kernel can sum duplicate
// rows before the (non-linear) RowAdagrad step -- the device counterpart of `grad.coalesce()` in
// torchbiggraph/row_adagrad.py:83.
//
// One pass sorts `db` key bits (up to 11, 2048 bins; the passes split the key bits evenly) with
// three launches:
//   radix_hist     every warp owns a run of RUN consecutive pairs and counts its digits into
//                  hist[digit][warp]
//   radix_scan     one CTA per digit: exclusive scan of that digit's row of warp counts, row total
//                  to totals[digit]
//   radix_scatter  every CTA turns totals[] into digit bases (a block scan of <= 2048 values), then
//                  every warp walks its run in order and writes each pair to
//                  base[digit] + scanned[digit][warp] + (earlier pairs of the run with that digit)
// Ranking inside a run uses __match_any_sync, so equal digits keep their input order (stable).
#include "pbg_common.cuh"

#define RUN_ITEMS 8                      // pairs per lane per run
#define RUN (32 * RUN_ITEMS)             // pairs per warp
#define SORT_WARPS_PER_CTA 4
#define MAX_BINS 2048

int pbg_sort_warps(int n) { return (n + RUN - 1) / RUN; }
// counters a sort of n pairs needs: [MAX_BINS][warps] + [MAX_BINS] totals
size_t pbg_sort_hist_entries(int n) { return (size_t)MAX_BINS * pbg_sort_warps(n) + MAX_BINS; }

__global__ void __launch_bounds__(32 * SORT_WARPS_PER_CTA)
radix_hist(const unsigned long long *__restrict__ keys, int n, int shift, int nbins, unsigned int *__restrict__ hist,
           int nwarps) {
  __shared__ unsigned int cnt[SORT_WARPS_PER_CTA][MAX_BINS];
  int wl = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int wg = blockIdx.x * SORT_WARPS_PER_CTA + wl;
  const unsigned long long mask = (unsigned long long)(nbins - 1);
  for (int i = lane; i < nbins; i += 32) cnt[wl][i] = 0;
  __syncwarp();
  if (wg < nwarps) {
    int base = wg * RUN;
    for (int it = 0; it < RUN_ITEMS; ++it) {
      int i = base + it * 32 + lane;
      bool ok = i < n;
      unsigned int dg = ok ? (unsigned int)((keys[i] >> shift) & mask) : 0u;
      unsigned int act = __ballot_sync(0xffffffffu, ok);
      if (ok) {
        unsigned int peers = __match_any_sync(act, dg);
        if ((peers & ((1u << lane) - 1u)) == 0u) cnt[wl][dg] += __popc(peers);   // lowest peer adds
      }
      __syncwarp();
    }
    for (int i = lane; i < nbins; i += 32) hist[(size_t)i * nwarps + wg] = cnt[wl][i];
  }
}

// grid = nbins CTAs of 128 threads: exclusive scan of hist[digit][0..nwarps) in place.
__global__ void __launch_bounds__(128) radix_scan(unsigned int *__restrict__ hist, int nwarps,
                                                  unsigned int *__restrict__ totals) {
  __shared__ unsigned int part[128];
  unsigned int *row = hist + (size_t)blockIdx.x * nwarps;
  int t = threadIdx.x;
  int per = (nwarps + 127) / 128;
  int lo = t * per, hi = lo + per < nwarps ? lo + per : nwarps;
  unsigned int s = 0;
  for (int i = lo; i < hi; ++i) s += row[i];
  part[t] = s;
  __syncthreads();
  for (int off = 1; off < 128; off <<= 1) {
    unsigned int v = t >= off ? part[t - off] : 0u;
    __syncthreads();
    part[t] += v;
    __syncthreads();
  }
  unsigned int run = part[t] - s;
  for (int i = lo; i < hi; ++i) { unsigned int v = row[i]; row[i] = run; run += v; }
  if (t == 127) totals[blockIdx.x] = part[127];
}

__global__ void __launch_bounds__(32 * SORT_WARPS_PER_CTA)
radix_scatter(const unsigned long long *__restrict__ keys, const unsigned int *__restrict__ vals, int n,
              int shift, int nbins, const unsigned int *__restrict__ hist, const unsigned int *__restrict__ totals,
              int nwarps, unsigned long long *__restrict__ keys_out, unsigned int *__restrict__ vals_out) {
  __shared__ unsigned int pos[SORT_WARPS_PER_CTA][MAX_BINS];
  __shared__ unsigned int base[MAX_BINS];
  __shared__ unsigned int wsum[SORT_WARPS_PER_CTA];
  int wl = threadIdx.x >> 5, lane = threadIdx.x & 31, t = threadIdx.x;
  const unsigned long long mask = (unsigned long long)(nbins - 1);
  // digit bases: exclusive scan of totals[0..nbins) by the whole CTA (each thread a contiguous chunk)
  {
    constexpr int T = 32 * SORT_WARPS_PER_CTA;
    int per = (nbins + T - 1) / T;
    int lo = t * per, hi = lo + per < nbins ? lo + per : nbins;
    unsigned int s = 0;
    for (int i = lo; i < hi; ++i) s += totals[i];
    unsigned int incl = s;                                   // inclusive scan inside the warp
    for (int off = 1; off < 32; off <<= 1) {
      unsigned int v = __shfl_up_sync(0xffffffffu, incl, off);
      if (lane >= off) incl += v;
    }
    if (lane == 31) wsum[wl] = incl;
    __syncthreads();
    unsigned int before = 0;
    for (int k = 0; k < wl; ++k) before += wsum[k];
    unsigned int run = before + incl - s;
    for (int i = lo; i < hi; ++i) { base[i] = run; run += totals[i]; }
    __syncthreads();
  }
  int wg = blockIdx.x * SORT_WARPS_PER_CTA + wl;
  if (wg >= nwarps) return;
  for (int i = lane; i < nbins; i += 32) pos[wl][i] = base[i] + hist[(size_t)i * nwarps + wg];
  __syncwarp();
  int b0 = wg * RUN;
  for (int it = 0; it < RUN_ITEMS; ++it) {
    int i = b0 + it * 32 + lane;
    bool ok = i < n;
    unsigned long long key = ok ? keys[i] : 0ull;
    unsigned int dg = (unsigned int)((key >> shift) & mask);
    unsigned int act = __ballot_sync(0xffffffffu, ok);
    unsigned int peers = 0u;
    if (ok) {
      peers = __match_any_sync(act, dg);
      unsigned int before = __popc(peers & ((1u << lane) - 1u));
      unsigned int dst = pos[wl][dg] + before;
      keys_out[dst] = key;
      vals_out[dst] = vals[i];
    }
    __syncwarp();                                          // every peer has read pos[] by now
    if (ok && (peers & ((1u << lane) - 1u)) == 0u) pos[wl][dg] += __popc(peers);
    __syncwarp();
  }
}

int pbg_sort(SortPlan &sp, int n, int bits, cudaStream_t st) {
  int launches = 0;
  int src = 0;
  sp.result = 0;
  if (n <= 0) return 0;
  int nwarps = pbg_sort_warps(n);
  int ctas = (nwarps + SORT_WARPS_PER_CTA - 1) / SORT_WARPS_PER_CTA;
  int passes = (bits + 10) / 11;
  int db = (bits + passes - 1) / passes;                   // digit bits of every pass (<= 11)
  int nbins = 1 << db;
  unsigned int *totals = sp.hist + (size_t)MAX_BINS * nwarps;
  for (int pass = 0, shift = 0; pass < passes; ++pass, shift += db) {
    radix_hist<<<ctas, 32 * SORT_WARPS_PER_CTA, 0, st>>>(sp.keys[src], n, shift, nbins, sp.hist, nwarps);
    radix_scan<<<nbins, 128, 0, st>>>(sp.hist, nwarps, totals);
    radix_scatter<<<ctas, 32 * SORT_WARPS_PER_CTA, 0, st>>>(sp.keys[src], sp.vals[src], n, shift, nbins, sp.hist, totals,
                                                           nwarps, sp.keys[src ^ 1], sp.vals[src ^ 1]);
    launches += 3;
    src ^= 1;
  }
  sp.result = src;
  return launches;
}

// keys[i] = rows[i] (invalid rows flagged and sent to the end), vals[i] = i: the set-up of the
// stand-alone sparse RowAdagrad entry point.
__global__ void iota_keys(const long long *__restrict__ rows, long long num_rows, int n,
                          unsigned long long *__restrict__ keys, unsigned int *__restrict__ vals,
                          int *errflag) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  long long r = rows[i];
  bool bad = r < 0 || r >= num_rows;
  if (bad) atomicOr(errflag, 1);
  keys[i] = bad ? (unsigned long long)num_rows : (unsigned long long)r;
  vals[i] = (unsigned int)i;
}

int launch_iota_keys(const long long *rows, long long num_rows, int n, unsigned long long *keys,
                     unsigned int *vals, int *errflag, cudaStream_t st) {
  iota_keys<<<(n + 255) / 256, 256, 0, st>>>(rows, num_rows, n, keys, vals, errflag);
  return 1;
}
