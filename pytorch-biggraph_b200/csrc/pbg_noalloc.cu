// pbg_row_adagrad_static: the sparse RowAdagrad step for callers that must not allocate.
//
// A trainer process that has handed every byte of HBM to its partitions (or runs under an
// allocator that owns the whole device, or sits on a path where the implicit synchronisation of
// cudaMalloc / cudaFree is not acceptable) cannot create a pbg_context, because creating one
// allocates its workspace.  This entry point needs no context: the scratch the step uses (sort
// keys and values, digit counters, an error word) lives in the file-scope device array below,
// which every GPU that loads the library holds until the process exits.
#include <mutex>

#include "pbg_common.cuh"

#define NOALLOC_MAX_ROWS 16384          // most gradient rows per call
#define NOALLOC_MAX_DEVICES 64

// scratch layout (bytes): 2 x keys | 2 x values | digit counters | error word
#define NA_KEYS_BYTES (NOALLOC_MAX_ROWS * 8)
#define NA_VALS_BYTES (NOALLOC_MAX_ROWS * 4)
#define NA_HIST_BYTES ((2048 * ((NOALLOC_MAX_ROWS + 255) / 256) + 2048) * 4)   // pbg_sort_hist_entries(16384) counters
#define NA_TOTAL_BYTES (2 * NA_KEYS_BYTES + 2 * NA_VALS_BYTES + NA_HIST_BYTES + 256)

static __device__ __align__(256) unsigned char pbg_noalloc_scratch[NA_TOTAL_BYTES];

// In host code `pbg_noalloc_scratch` is only a handle: its device address is looked up once per
// device, with that device current, and that address is what the kernels get.
static unsigned char *scratch_addr[NOALLOC_MAX_DEVICES];
static std::mutex scratch_mutex;

static int scratch_for_current_device(unsigned char **out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess) return PBG_ERR_NO_DEVICE;
  if (dev < 0 || dev >= NOALLOC_MAX_DEVICES) return PBG_ERR_TOO_LARGE;
  std::lock_guard<std::mutex> lock(scratch_mutex);
  if (!scratch_addr[dev]) {
    void *p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, pbg_noalloc_scratch);
    if (e != cudaSuccess || !p) return PBG_ERR_CUDA;
    scratch_addr[dev] = (unsigned char *)p;
  }
  *out = scratch_addr[dev];
  return PBG_OK;
}

static int bit_len(unsigned long long v) { int b = 0; while (v) { ++b; v >>= 1; } return b < 1 ? 1 : b; }

extern "C" int pbg_row_adagrad_static(float *emb, float *state, int64_t num_rows, int32_t dim,
                                      const int64_t *rows_dev, const float *grads_dev, int32_t n, float lr,
                                      void *stream) {
  if (n == 0) return PBG_OK;
  if (!emb || !state || !rows_dev || !grads_dev || n < 0 || num_rows <= 0) return PBG_ERR_BAD_ARGUMENT;
  if (dim <= 0 || dim % 4 != 0 || dim > 2048) return PBG_ERR_UNSUPPORTED;
  if (n > NOALLOC_MAX_ROWS) return PBG_ERR_TOO_LARGE;      // the fixed scratch holds 16384 rows
  unsigned char *base = nullptr;
  int rc = scratch_for_current_device(&base);
  if (rc != PBG_OK) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  SortPlan sp;
  sp.keys[0] = (unsigned long long *)base;
  sp.keys[1] = (unsigned long long *)(base + NA_KEYS_BYTES);
  sp.vals[0] = (unsigned int *)(base + 2 * NA_KEYS_BYTES);
  sp.vals[1] = (unsigned int *)(base + 2 * NA_KEYS_BYTES + NA_VALS_BYTES);
  sp.hist = (unsigned int *)(base + 2 * NA_KEYS_BYTES + 2 * NA_VALS_BYTES);
  sp.max_n = NOALLOC_MAX_ROWS;
  sp.result = 0;
  int *errflag = (int *)(base + 2 * NA_KEYS_BYTES + 2 * NA_VALS_BYTES + NA_HIST_BYTES);
  // the array keeps whatever the previous call left: the error word has to start at zero
  if (cudaMemsetAsync(errflag, 0, sizeof(int), st) != cudaSuccess) return PBG_ERR_CUDA;
  launch_iota_keys((const long long *)rows_dev, num_rows, n, sp.keys[0], sp.vals[0], errflag, st);
  pbg_sort(sp, n, bit_len((unsigned long long)num_rows), st);
  launch_row_adagrad_sorted(emb, state, dim, sp.keys[sp.result], sp.vals[sp.result], grads_dev, n, lr,
                            (unsigned long long)num_rows, st);
  if (cudaGetLastError() != cudaSuccess) return PBG_ERR_CUDA;
  int flag = 0;
  if (cudaMemcpyAsync(&flag, errflag, sizeof flag, cudaMemcpyDeviceToHost, st) != cudaSuccess) return PBG_ERR_CUDA;
  if (cudaStreamSynchronize(st) != cudaSuccess) return PBG_ERR_CUDA;
  return flag ? PBG_ERR_INDEX_RANGE : PBG_OK;
}
