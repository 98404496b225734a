// Stable LSD radix sort of (row key, occurrence) pairs: groups the gradient slots of one wave by
// the embedding row they belong to, in batch order, so that the update kernel can sum duplicate
// rows before the (non-linear) RowAdagrad step -- the device counterpart of `grad.coalesce()` in
// torchbiggraph/row_adagrad.py:83.
//
// One pass = 8 key bits = three launches:
//   radix_hist    every warp owns a run of RUN consecutive pairs and counts its digits
//   radix_scan    exclusive scan of the [digit][warp] count table (one CTA)
//   radix_scatter every warp walks its run in order and writes each pair to
//                 scanned[digit][warp] + (number of earlier pairs of the run with that digit)
// Ranking inside a run uses __match_any_sync, so equal digits keep their input order.
#include "pbg_common.cuh"

#define RUN_ITEMS 8                      // pairs per lane per run
#define RUN (32 * RUN_ITEMS)             // pairs per warp
#define SORT_WARPS_PER_CTA 8

int pbg_sort_warps(int n) { return (n + RUN - 1) / RUN; }

__global__ void __launch_bounds__(32 * SORT_WARPS_PER_CTA)
radix_hist(const unsigned long long *__restrict__ keys, int n, int shift, unsigned int *__restrict__ hist,
           int nwarps) {
  __shared__ unsigned int cnt[SORT_WARPS_PER_CTA][256];
  int wl = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int wg = blockIdx.x * SORT_WARPS_PER_CTA + wl;
  for (int i = lane; i < 256; i += 32) cnt[wl][i] = 0;
  __syncwarp();
  if (wg < nwarps) {
    int base = wg * RUN;
    for (int it = 0; it < RUN_ITEMS; ++it) {
      int i = base + it * 32 + lane;
      bool ok = i < n;
      unsigned int dg = ok ? (unsigned int)((keys[i] >> shift) & 255ull) : 0u;
      unsigned int act = __ballot_sync(0xffffffffu, ok);
      if (ok) {
        unsigned int peers = __match_any_sync(act, dg);
        if ((peers & ((1u << lane) - 1u)) == 0u) cnt[wl][dg] += __popc(peers);   // lowest peer adds
      }
      __syncwarp();
    }
    for (int i = lane; i < 256; i += 32) hist[(size_t)i * nwarps + wg] = cnt[wl][i];
  }
}

// Exclusive scan of `total` counters in place, one CTA of 1024 threads.
__global__ void __launch_bounds__(1024) radix_scan(unsigned int *__restrict__ hist, int total) {
  __shared__ unsigned int part[1024];
  int t = threadIdx.x;
  int per = (total + 1023) / 1024;
  int lo = t * per, hi = lo + per < total ? lo + per : total;
  unsigned int s = 0;
  for (int i = lo; i < hi; ++i) s += hist[i];
  part[t] = s;
  __syncthreads();
  for (int off = 1; off < 1024; off <<= 1) {          // Hillis-Steele inclusive scan
    unsigned int v = t >= off ? part[t - off] : 0u;
    __syncthreads();
    part[t] += v;
    __syncthreads();
  }
  unsigned int run = part[t] - s;                      // exclusive prefix of this thread's range
  for (int i = lo; i < hi; ++i) { unsigned int v = hist[i]; hist[i] = run; run += v; }
}

__global__ void __launch_bounds__(32 * SORT_WARPS_PER_CTA)
radix_scatter(const unsigned long long *__restrict__ keys, const unsigned int *__restrict__ vals, int n,
              int shift, const unsigned int *__restrict__ hist, int nwarps,
              unsigned long long *__restrict__ keys_out, unsigned int *__restrict__ vals_out) {
  __shared__ unsigned int pos[SORT_WARPS_PER_CTA][256];
  int wl = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int wg = blockIdx.x * SORT_WARPS_PER_CTA + wl;
  if (wg >= nwarps) return;
  for (int i = lane; i < 256; i += 32) pos[wl][i] = hist[(size_t)i * nwarps + wg];
  __syncwarp();
  int base = wg * RUN;
  for (int it = 0; it < RUN_ITEMS; ++it) {
    int i = base + it * 32 + lane;
    bool ok = i < n;
    unsigned long long key = ok ? keys[i] : 0ull;
    unsigned int dg = (unsigned int)((key >> shift) & 255ull);
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
  for (int shift = 0; shift < bits; shift += 8) {
    radix_hist<<<ctas, 32 * SORT_WARPS_PER_CTA, 0, st>>>(sp.keys[src], n, shift, sp.hist, nwarps);
    radix_scan<<<1, 1024, 0, st>>>(sp.hist, 256 * nwarps);
    radix_scatter<<<ctas, 32 * SORT_WARPS_PER_CTA, 0, st>>>(sp.keys[src], sp.vals[src], n, shift, sp.hist,
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
