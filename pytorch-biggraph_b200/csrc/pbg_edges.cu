// The edge-list utilities either side of the training step, on the device: what the reference's native
// module torchbiggraph._C does on host threads (torchbiggraph/util.cpp) --
//   reverse_permutation   util.cpp:103-125   out[perm[i]] = i
//   shuffle               util.cpp:127-220   row i of a table moves to row perm[i]
//   sub_bucket            util.cpp:260-423   stable split of a bucket's edges into N x M sub-buckets
//   randperm              util.cpp:14-101    a seeded random permutation (also stands where the trainers call
//                                            torch.randperm for the per-bucket edge shuffle, train_cpu.py:857-859,
//                                            train_gpu.py:245)
// All of it is integer / byte work bound by HBM: coalesced 8- and 16-byte accesses, one stable LSD radix sort
// (pbg_sort.cu) where an order is needed.  Range violations are reported through the context's error word and the
// offending elements skipped; nothing faults.
#include "pbg_common.cuh"

// res[perm[i]] = i
__global__ void reverse_permutation_kernel(const long long *__restrict__ perm, long long n, long long *__restrict__ out, int *errflag) {
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  long long p = perm[i];
  if (p < 0 || p >= n) { atomicOr(errflag, 1); return; }
  out[p] = i;
}

// out row perm[r] = in row r, rows of `units` elements of type T
template <class T>
__global__ void shuffle_rows_kernel(const T *__restrict__ in, T *__restrict__ out, long long rows, long long units,
                                    const long long *__restrict__ perm, int *errflag) {
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= rows * units) return;
  long long r = idx / units, u = idx - r * units;
  long long p = perm[r];
  if (p < 0 || p >= rows) { if (u == 0) atomicOr(errflag, 1); return; }
  out[p * units + u] = in[idx];
}

// keys of a random permutation: 44 hashed bits per index (ties, vanishingly rare, keep index order: still a permutation)
__global__ void randperm_keys_kernel(long long n, unsigned long long seed, unsigned long long *keys, unsigned int *vals) {
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  keys[i] = pbg_mix64(seed ^ pbg_mix64((unsigned long long)i + 0x51ED270B0F1ull)) >> 20;
  vals[i] = (unsigned int)i;
}
__global__ void widen_kernel(const unsigned int *__restrict__ vals, long long n, long long *__restrict__ out) {
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = (long long)vals[i];
}

// Per-relation tables of a sub_bucket call, in device memory: [R] lhs permutation pointers, [R] rhs permutation
// pointers, [R] lhs entity counts, [R] rhs entity counts, [R] lhs sub-partition sizes, [R] rhs sub-partition sizes.
struct SubBucketArgs {
  const long long *lhs, *rhs, *rel;
  long long n;
  const long long *const *lperm, *const *rperm;
  const long long *lcount, *rcount, *lsize, *rsize;
  int R, nl, nr, dynamic;
};

// permuted offsets of edge e; false (and the error word set) when an id is outside its table
__device__ __forceinline__ bool sub_bucket_offsets(const SubBucketArgs &a, long long e, long long &lo, long long &ro, long long &relid, int *errflag) {
  relid = a.dynamic ? 0 : a.rel[e];
  if (relid < 0 || relid >= a.R) { atomicOr(errflag, 4); return false; }          // "rel > numRelations" (util.cpp:320-322)
  long long l = a.lhs[e], r = a.rhs[e];
  if (l < 0 || l >= a.lcount[relid] || r < 0 || r >= a.rcount[relid]) { atomicOr(errflag, 1); return false; }
  lo = a.lperm[relid][l];
  ro = a.rperm[relid][r];
  if (lo < 0 || lo >= a.lcount[relid] || ro < 0 || ro >= a.rcount[relid]) { atomicOr(errflag, 1); return false; }
  return true;
}

__global__ void sub_bucket_keys_kernel(SubBucketArgs a, unsigned long long *keys, unsigned int *vals, int *errflag) {
  long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= a.n) return;
  long long lo, ro, relid;
  unsigned long long key = (unsigned long long)a.nl * a.nr;            // edges that cannot be placed sort to the end
  if (sub_bucket_offsets(a, e, lo, ro, relid, errflag))
    key = (unsigned long long)(lo / a.lsize[relid]) * a.nr + (unsigned long long)(ro / a.rsize[relid]);
  keys[e] = key;
  vals[e] = (unsigned int)e;
}

__global__ void sub_bucket_emit_kernel(SubBucketArgs a, const unsigned long long *__restrict__ keys, const unsigned int *__restrict__ vals,
                                       long long *lhs_out, long long *rhs_out, long long *rel_out, int *errflag) {
  long long q = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (q >= a.n) return;
  if (keys[q] >= (unsigned long long)a.nl * a.nr) return;
  long long e = vals[q], lo, ro, relid;
  if (!sub_bucket_offsets(a, e, lo, ro, relid, errflag)) return;
  lhs_out[q] = lo % a.lsize[relid];
  rhs_out[q] = ro % a.rsize[relid];
  rel_out[q] = a.rel[e];
}

// counts[b] = number of sorted keys equal to b (one thread per sub-bucket, two binary searches)
__global__ void sub_bucket_counts_kernel(const unsigned long long *__restrict__ keys, long long n, int nb, long long *counts) {
  int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= nb) return;
  auto lower = [&](unsigned long long v) {
    long long lo = 0, hi = n;
    while (lo < hi) { long long mid = (lo + hi) >> 1; if (keys[mid] < v) lo = mid + 1; else hi = mid; }
    return lo;
  };
  counts[b] = lower((unsigned long long)b + 1) - lower((unsigned long long)b);
}

static inline int grid_for(long long n, int threads) { return (int)((n + threads - 1) / threads); }

int launch_reverse_permutation(const long long *perm, long long n, long long *out, int *errflag, cudaStream_t st) {
  if (n > 0) reverse_permutation_kernel<<<grid_for(n, 256), 256, 0, st>>>(perm, n, out, errflag);
  return n > 0;
}

int launch_shuffle_rows(const void *in, void *out, long long rows, long long row_bytes, const long long *perm, int *errflag, cudaStream_t st) {
  if (rows <= 0 || row_bytes <= 0) return 0;
  const uintptr_t al = (uintptr_t)in | (uintptr_t)out | (uintptr_t)row_bytes;
  if (al % 16 == 0) {
    long long u = row_bytes / 16;
    shuffle_rows_kernel<uint4><<<grid_for(rows * u, 256), 256, 0, st>>>((const uint4 *)in, (uint4 *)out, rows, u, perm, errflag);
  } else if (al % 8 == 0) {
    long long u = row_bytes / 8;
    shuffle_rows_kernel<unsigned long long><<<grid_for(rows * u, 256), 256, 0, st>>>((const unsigned long long *)in, (unsigned long long *)out, rows, u, perm, errflag);
  } else if (al % 4 == 0) {
    long long u = row_bytes / 4;
    shuffle_rows_kernel<unsigned int><<<grid_for(rows * u, 256), 256, 0, st>>>((const unsigned int *)in, (unsigned int *)out, rows, u, perm, errflag);
  } else {
    shuffle_rows_kernel<unsigned char><<<grid_for(rows * row_bytes, 256), 256, 0, st>>>((const unsigned char *)in, (unsigned char *)out, rows, row_bytes, perm, errflag);
  }
  return 1;
}

int launch_randperm(SortPlan &sp, long long n, unsigned long long seed, long long *out, cudaStream_t st) {
  if (n <= 0) return 0;
  randperm_keys_kernel<<<grid_for(n, 256), 256, 0, st>>>(n, seed, sp.keys[0], sp.vals[0]);
  int launches = 1 + pbg_sort(sp, (int)n, 44, st);
  widen_kernel<<<grid_for(n, 256), 256, 0, st>>>(sp.vals[sp.result], n, out);
  return launches + 1;
}

int launch_sub_bucket(SortPlan &sp, const long long *lhs, const long long *rhs, const long long *rel, long long n, int R,
                      const long long *tables_dev, int nl, int nr, int dynamic, long long *lhs_out, long long *rhs_out,
                      long long *rel_out, long long *counts_dev, int *errflag, cudaStream_t st) {
  SubBucketArgs a;
  a.lhs = lhs; a.rhs = rhs; a.rel = rel; a.n = n; a.R = R; a.nl = nl; a.nr = nr; a.dynamic = dynamic;
  a.lperm = (const long long *const *)tables_dev;
  a.rperm = (const long long *const *)(tables_dev + R);
  a.lcount = tables_dev + 2 * R; a.rcount = tables_dev + 3 * R; a.lsize = tables_dev + 4 * R; a.rsize = tables_dev + 5 * R;
  const int nb = nl * nr;
  if (n <= 0) { cudaMemsetAsync(counts_dev, 0, (size_t)nb * sizeof(long long), st); return 0; }
  sub_bucket_keys_kernel<<<grid_for(n, 256), 256, 0, st>>>(a, sp.keys[0], sp.vals[0], errflag);
  int bits = 1;
  while ((1ll << bits) <= nb) ++bits;                                   // keys run up to nb (the "cannot be placed" key)
  int launches = 1 + pbg_sort(sp, (int)n, bits, st);
  sub_bucket_emit_kernel<<<grid_for(n, 256), 256, 0, st>>>(a, sp.keys[sp.result], sp.vals[sp.result], lhs_out, rhs_out, rel_out, errflag);
  sub_bucket_counts_kernel<<<grid_for(nb, 128), 128, 0, st>>>(sp.keys[sp.result], n, nb, counts_dev);
  return launches + 2;
}
