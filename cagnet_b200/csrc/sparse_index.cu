// Integer index work on the sparse operand: COO row indices -> CSR row offsets, and validation.
// Pure integer arithmetic, bit-exact by construction.
#include <limits.h>

#include "common.cuh"

namespace cagnet {

static thread_local char g_last_error[256] = "";
char* last_error_buf() { return g_last_error; }

// rowptr[i] = first e with rows[e] >= i  (= number of entries whose row index is < i).
// One thread per output; used when rows are few compared with nonzeros (log2(nnz) probes each,
// the top of the search tree stays in L1/L2).
__global__ void coo2csr_search_kernel(const int* __restrict__ rows, int nnz, int n, int* __restrict__ rowptr) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i > n) return;
  int lo = 0, hi = nnz;
  while (lo < hi) {
    const int mid = lo + ((hi - lo) >> 1);
    if (__ldg(rows + mid) < i) lo = mid + 1; else hi = mid;
  }
  rowptr[i] = lo;
}

// Same result by boundary detection: entry e closes every row in (rows[e-1], rows[e]].
// One coalesced pass over the row indices; used when n is comparable with nnz.
__global__ void coo2csr_boundary_kernel(const int* __restrict__ rows, int nnz, int n, int* __restrict__ rowptr) {
  const int64_t e = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (e > nnz) return;
  const int prev = (e == 0) ? -1 : max(-1, __ldg(rows + e - 1));
  const int cur = (e == nnz) ? n : min(n, __ldg(rows + e));   // clamped: malformed input cannot write out of range
  for (int r = prev + 1; r <= cur; ++r) rowptr[r] = static_cast<int>(e);
}

__global__ void check_csr_kernel(const int* __restrict__ rowptr, const int* __restrict__ col,
                                 const int* __restrict__ rows, int n, int m, int nnz, int* status) {
  const int64_t t = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (rows && t < nnz) {
    const int r = rows[t];
    if (r < 0 || r >= n) atomicMax(status, 5);
    else if (t > 0 && rows[t - 1] > r) atomicMax(status, 3);
  }
  if (t == 0) {
    if (rowptr[0] != 0) atomicMax(status, 1);
    if (rowptr[n] != nnz) atomicMax(status, 2);
  }
  if (t < n && rowptr[t] > rowptr[t + 1]) atomicMax(status, 3);
  if (t < nnz) {
    const int c = col[t];
    if (c < 0 || c >= m) atomicMax(status, 4);
  }
}

}  // namespace cagnet

using namespace cagnet;

extern "C" int cagnet_version(void) { return 100; }

extern "C" const char* cagnet_last_error_string(void) { return last_error_buf(); }

extern "C" int cagnet_coo2csr_i32(const int32_t* rows, int64_t nnz, int32_t n, int32_t* rowptr, void* stream) {
  if (n < 0 || nnz < 0 || !rowptr || (nnz > 0 && !rows)) return fail(CAGNET_E_ARG, "cagnet_coo2csr_i32: bad argument");
  if (nnz > INT_MAX) return fail(CAGNET_E_OVERFLOW, "cagnet_coo2csr_i32: nnz %s%lld exceeds int32", "", nnz);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int innz = static_cast<int>(nnz);
  if (nnz > 16 * static_cast<int64_t>(n)) {
    coo2csr_search_kernel<<<(n + 1 + 255) / 256, 256, 0, s>>>(rows, innz, n, rowptr);
  } else {
    coo2csr_boundary_kernel<<<static_cast<unsigned>((nnz + 1 + 255) / 256), 256, 0, s>>>(rows, innz, n, rowptr);
  }
  return check_launch("cagnet_coo2csr_i32");
}

extern "C" int cagnet_check_csr_i32(const int32_t* rowptr, const int32_t* col, const int32_t* rows, int32_t n, int32_t m,
                                    int64_t nnz, int32_t* status_dev, void* stream) {
  if (n < 0 || m < 0 || nnz < 0 || !rowptr || !status_dev || (nnz > 0 && !col))
    return fail(CAGNET_E_ARG, "cagnet_check_csr_i32: bad argument");
  if (nnz > INT_MAX) return fail(CAGNET_E_OVERFLOW, "cagnet_check_csr_i32: nnz %s%lld exceeds int32", "", nnz);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaMemsetAsync(status_dev, 0, sizeof(int), s);
  const int64_t work = (nnz > n ? nnz : n) + 1;
  check_csr_kernel<<<static_cast<unsigned>((work + 255) / 256), 256, 0, s>>>(rowptr, col, rows, n, m,
                                                                            static_cast<int>(nnz), status_dev);
  return check_launch("cagnet_check_csr_i32");
}
